"""Tekosun design in the layer-stack engine against the plain restatement in tests/tekosun_oracle.py: every mechanism
alone (the attention preparation, window edges and far keys with crafted scores, the linear-recurrence scan in both of its
forms with carried state, softmax-routed experts, each mixer as a one-layer model), whole prompts, decoding through caches
and states, prompts cut into portions down to one and two tokens, unequal batches, slots given back and used again, long
decoding past the window, other sizes and layer orders, the constants shown to matter, greedy generation through the
engine's own entry points."""
import copy
import math

import pytest
import torch

import tekosun_oracle as so
from tinygpt_b200 import engine, models, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
# fp32 engines are held to summation-order noise on EVERY row.  bf16 engines round activations to 8 bits of mantissa; a
# token whose router scores nearly tie may then take another expert than in the fp32 restatement, and the recurrent states
# carry that on: against the restatement they are held to the median row and to most rows, and to each other across paths.
TOL = {torch.float32: 3e-4, torch.bfloat16: 9e-2}


def row_err(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: rms of the difference (mean removed) over rms of the wanted row (mean removed)."""
    got, want = got.float().cpu(), want.float().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp_min(1e-6)


def assert_close(got, want, dtype, what=""):
    e = row_err(got, want)
    if dtype == torch.float32:
        assert float(e.max()) < TOL[dtype], f"{what}: worst row {float(e.max()):.2e} at {int(e.argmax())}"
    else:
        assert bool(torch.isfinite(got.float()).all()), what
        assert float(e.median()) < TOL[dtype] and float((e < TOL[dtype]).float().mean()) >= 0.6, \
            f"{what}: {int((e >= TOL[dtype]).sum())} of {len(e)} rows off, median {float(e.median()):.2e}"


ROT = {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "high": 4.0, "low": 1.0, "original": 32}}


def attn(heads=4, kv_heads=2, dim=12, vdim=20, window=9, rot=ROT, v_mix=True, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim)}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = copy.deepcopy(rot)
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def delta(heads=3, dim=16):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def mamba(heads=3, vdim=8, state=16, groups=1, conv=4, norm_groups=1):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def moe(experts=6, top=2, ff=24, shared=40, scale=1.5):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def config(layers, width=64, vocab=96, embed_scale=3.0, eps=1e-5):
    return {"architecture": "Tekosun", "embedding": {"scale": embed_scale},
            "layers": [dict(copy.deepcopy(mix), mlp=copy.deepcopy(mlp)) for mix, mlp in layers], "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def base_config():
    return config([(delta(), moe()), (attn(), moe(experts=5, top=3, ff=16, shared=0)), (mamba(heads=4, groups=2, norm_groups=2), moe()),
                   (delta(heads=2, dim=24), None), (attn(heads=2, kv_heads=2, dim=16, vdim=20, window=5), moe(top=1))])


def make(cfg, dtype, seed=0, max_ctx=160, max_slots=4, rank=6):
    for lc in cfg["layers"]:                       # the decay bottleneck's rank travels in the tensors, not in config.json
        if lc["type"] == "general_delta":
            lc["mixer"].setdefault("rank", rank)
    spec = models.tekosun_from_config(cfg).with_ctx(max_ctx, max_slots)
    w = models.synth_tekosun_weights(spec, seed=seed)
    eng = engine.DecodeEngine(spec, models.pack_weights(spec, w, device=DEV, dtype=dtype))
    return eng, {k: v.float() for k, v in w.items()}


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rot", [ROT, {"base": 500.0, "dims": 12}, {"base": 100.0, "dims": 2}, None])
def test_attention_preparation_op(dtype, rot):
    """q | k | v rows through the preparation alone: whole-projection norms, rotation of the first dims of every head,
    unit-rms values; then a second 'layer' that mixes the first one's values in."""
    H, G, dk, dv, n, eps = 4, 2, 12, 20, 23, 1e-5
    g = torch.Generator().manual_seed(1)
    proj = (torch.randn(n, H * dk + G * dk + G * dv, generator=g) * 2).to(dtype)
    qn, kn = 1 + 0.2 * torch.randn(H * dk, generator=g), 1 + 0.2 * torch.randn(G * dk, generator=g)
    pos = torch.arange(40, 40 + n)
    p = proj.float()
    q = so.rms_norm(p[:, :H * dk], qn, eps).view(n, H, dk)
    k = so.rms_norm(p[:, H * dk:(H + G) * dk], kn, eps).view(n, G, dk)
    v = so.unit_rms(p[:, (H + G) * dk:].view(n, G, dv), eps)
    if rot:
        q, k = so.rotate_half(q, pos, rot), so.rotate_half(k, pos, rot)
    tab = None
    if rot:
        sc = rot.get("scaling") or {}
        tab = models.HalfRotarySpec(rot["dims"], rot["base"], sc.get("factor", 0.0), sc.get("low", 0.0), sc.get("high", 0.0),
                                    sc.get("original", 0)).table(128).to(DEV)
    keep = torch.zeros(n, G * dv, dtype=dtype, device=DEV)
    kw = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, eps=eps, q_norm=qn.to(DEV), k_norm=kn.to(DEV), rot_table=tab, v_norm=True)
    got = ops.stack_attn_prep(proj.clone().to(DEV), 0, H * dk, (H + G) * dk, i32(pos.tolist()), v_mix=1, vkeep=keep, **kw)
    want = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1)
    tol = 2e-6 if dtype == torch.float32 else 1.2e-2
    assert (got.float().cpu() - want).abs().max() < tol * want.abs().max()
    assert torch.equal(keep.float().cpu(), got.float().cpu()[:, (H + G) * dk:])
    lam = torch.tensor([0.3])
    got2 = ops.stack_attn_prep(proj.clone().to(DEV), 0, H * dk, (H + G) * dk, i32(pos.tolist()), v_mix=2, vkeep=keep,
                               mix_lambda=lam.to(DEV), **kw)
    want_v = 0.7 * v.reshape(n, -1) + 0.3 * keep.float().cpu()
    assert (got2.float().cpu()[:, (H + G) * dk:] - want_v).abs().max() < tol * 2


def _selector_attention(dtype, m, n, seed):
    """An attention case whose input rows ARE the projections: the weights pick columns of h, the output weight is the
    identity, the norm weights are one."""
    g = torch.Generator().manual_seed(seed)
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    nq, nk, nv = H * dk, G * dk, G * dv
    eye = torch.eye(nq + nk + nv)
    w = {"q": eye[:nq], "k": eye[nq:nq + nk], "v": eye[nq + nk:], "q.norm": torch.ones(nq), "k.norm": torch.ones(nk),
         "o": torch.eye(H * dv), "vmix": torch.tensor(0.0)}
    h = torch.randn(n, nq + nk + nv, generator=g).to(dtype).float()
    return h, w


def _run_attention_op(h, m, dtype, steps, max_ctx, slot=1, eps=1e-5):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    nq, nk = H * dk, G * dk
    kc = torch.zeros(3, max_ctx, nk, dtype=dtype, device=DEV)
    vc = torch.zeros(3, max_ctx, G * dv, dtype=dtype, device=DEV)
    rot = m.get("rot")
    tab = models.HalfRotarySpec(rot["dims"], rot["base"]).table(max_ctx).to(DEV) if rot else None
    out, at = [], 0
    for c in steps:
        rows = h[at:at + c].to(dtype).to(DEV).contiguous()
        pos, sl = i32(list(range(at, at + c))), i32([slot] * c)
        ops.stack_attn_prep(rows, 0, nq, nq + nk, pos, heads=H, kv_heads=G, dim=dk, vdim=dv, eps=eps,
                            q_norm=torch.ones(nq, device=DEV), k_norm=torch.ones(nk, device=DEV), rot_table=tab, v_norm=True)
        ops.stack_kv_store(kc, vc, rows, nq, nq + nk, sl, pos, heads=H, kv_heads=G, dim=dk, vdim=dv)
        out.append(ops.stack_attention(rows, 0, 0, kc, vc, sl, pos, heads=H, kv_heads=G, dim=dk, vdim=dv, scale=m["scale"],
                                       window=(m.get("mask") or {}).get("size", 0)))
        at += c
    return torch.cat(out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("case", ["last_inside", "first_outside", "far"])
def test_attention_crafted_scores_at_the_window_edge_and_far_away(dtype, decode, case):
    """300 positions.  The last query (head 3, key/value head 1) is aimed at ONE earlier key through the entries the
    rotation leaves alone, so that this score would dominate: the key just inside the window must own the output, the
    key just outside must not be seen at all, and without a window a key 296 positions back must be found."""
    n, window = 300, 64
    m = attn(heads=4, kv_heads=2, dim=16, vdim=12, window=0 if case == "far" else window, rot={"base": 100.0, "dims": 4},
             v_mix=False, scale=6.0)["mixer"]
    target = {"last_inside": n - window, "first_outside": n - 1 - window, "far": 3}[case]
    h, w = _selector_attention(dtype, m, n, seed=2)
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    nq = H * dk
    aim = torch.zeros(dk)
    aim[4:] = torch.randn(dk - 4, generator=torch.Generator().manual_seed(3))
    h[target, nq + dk:nq + 2 * dk] = (aim * 3).to(dtype).float()          # key of kv head 1 at the target position
    h[n - 1, 3 * dk:4 * dk] = (aim * 3).to(dtype).float()                  # query of head 3 (→ kv head 1) at the last one
    want, _ = so.attention(h, m, w, "", 1e-5, None)
    # what the last row would be if the target were (not) visible tells the cases apart by a wide margin
    seen, _ = so.attention(h, dict(m, mask={"size": 0}), w, "", 1e-5, None)
    if case == "first_outside":
        assert float(row_err(seen[-1:], want[-1:]).max()) > 0.3
    got = _run_attention_op(h, m, dtype, [n - 1, 1] if decode else [n], max_ctx=320)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    assert float(row_err(got[-1:], want[-1:]).max()) < tol
    # the other rows' scores are large and random (scale 6): bf16 rounding of q and k moves their softmax more
    assert float(row_err(got, want).max()) < (tol if dtype == torch.float32 else 0.15)


def _scan_ref(d, b, r, v, p=None, q=None, vscale=None, share=1, H=1, dk=1, dv=1):
    n = v.shape[0]
    S = torch.zeros(H, dk, dv, dtype=torch.float64)
    out = torch.zeros(n, H, dv, dtype=torch.float64)
    for t in range(n):
        for hd in range(H):
            dd = d[t].view(H, -1)[hd].double()
            bb, rr = b[t].view(H // share, dk)[hd // share].double(), r[t].view(H // share, dk)[hd // share].double()
            vv = v[t].view(H, dv)[hd].double() * (float(vscale[t, hd]) if vscale is not None else 1.0)
            new = dd[:, None] * S[hd] if dd.numel() == dk else float(dd) * S[hd]
            if p is not None:
                new = new - p[t].view(H, dk)[hd].double()[:, None] * (q[t].view(H, dk)[hd].double() @ S[hd])[None, :]
            S[hd] = new + bb[:, None] * vv[None, :]
            out[t, hd] = S[hd].T @ rr
    return out.reshape(n, H * dv).float()


def _scan_case(form, H, dk, dv, n, seed):
    g = torch.Generator().manual_seed(seed)
    if form == "delta":
        k = torch.randn(n, H * dk, generator=g)
        u = (k.view(n, H, dk) / k.view(n, H, dk).norm(dim=-1, keepdim=True)).reshape(n, H * dk)
        cols = dict(d=torch.exp(-0.6 * torch.rand(n, H * dk, generator=g)), p=torch.rand(n, H * dk, generator=g) * u, q=u, b=k,
                    r=torch.randn(n, H * dk, generator=g), v=torch.randn(n, H * dv, generator=g))
        kw = dict(share=1)
    else:
        share = 2 if H % 2 == 0 else 1
        cols = dict(d=torch.exp(-torch.rand(n, H, generator=g)), b=torch.randn(n, H // share * dk, generator=g),
                    r=torch.randn(n, H // share * dk, generator=g), v=torch.randn(n, H * dv, generator=g),
                    vscale=torch.rand(n, H, generator=g) + 0.1)
        kw = dict(share=share)
    return cols, kw


def _scan_run(cols, kw, H, dk, dv, steps, slot, state):
    names = list(cols)
    big = torch.cat([cols[k] for k in names], 1).to(DEV)
    off, views = 0, {}
    for k in names:
        views[k] = big[:, off:off + cols[k].shape[1]]
        off += cols[k].shape[1]
    out, at = [], 0
    for c in steps:
        sl = {k: t[at:at + c] for k, t in views.items()}
        out.append(ops.stack_lin_scan(sl["d"], sl["b"], sl["r"], sl["v"], state, i32([0]), i32([c]), i32([slot] * c),
                                      i32(list(range(at, at + c))), heads=H, dk=dk, dv=dv, p=sl.get("p"), q=sl.get("q"),
                                      vscale=sl.get("vscale"), **kw))
        at += c
    return torch.cat(out).cpu()


@pytest.mark.parametrize("form", ["delta", "ssm"])
@pytest.mark.parametrize("sizes", [(3, 16, 24), (1, 40, 7), (2, 33, 64), (4, 8, 9), (2, 130, 5), (1, 200, 40), (1, 300, 33)])
def test_linear_recurrence_scan_op_and_carried_state(form, sizes):
    H, dk, dv = sizes
    n = 70
    cols, kw = _scan_case(form, H, dk, dv, n, seed=5)
    want = _scan_ref(H=H, dk=dk, dv=dv, **cols, **kw)
    for steps in ([n], [n - 9] + [1] * 9, [2, 30, 38]):
        state = torch.full((3, H * dk * dv), 7.0, device=DEV)   # whatever an earlier sequence left: position 0 starts from zero
        got = _scan_run(cols, kw, H, dk, dv, steps, 2, state)
        assert float((got - want).abs().max() / want.abs().max()) < 2e-5, steps


@pytest.mark.parametrize("form", ["delta", "ssm"])
def test_scan_sequences_side_by_side(form):
    """Three sequences of unequal length in one launch, in scrambled slots, against each alone."""
    H, dk, dv, lens = 2, 16, 20, [5, 1, 17]
    cases = [_scan_case(form, H, dk, dv, n, seed=10 + i) for i, n in enumerate(lens)]
    kw = cases[0][1]
    cols = {k: torch.cat([c[0][k] for c in cases]) for k in cases[0][0]}
    big = torch.cat([cols[k] for k in cols], 1).to(DEV)
    off, views = 0, {}
    for k in cols:
        views[k] = big[:, off:off + cols[k].shape[1]]
        off += cols[k].shape[1]
    slots = [2, 0, 1]
    state = torch.zeros(3, H * dk * dv, device=DEV)
    got = ops.stack_lin_scan(views["d"], views["b"], views["r"], views["v"], state, i32([0, 5, 6]), i32(lens),
                             i32(sum(([s] * n for s, n in zip(slots, lens)), [])), i32(sum((list(range(n)) for n in lens), [])),
                             heads=H, dk=dk, dv=dv, p=views.get("p"), q=views.get("q"), vscale=views.get("vscale"), **kw).cpu()
    want = torch.cat([_scan_ref(H=H, dk=dk, dv=dv, **c[0], **c[1]) for c in cases])
    assert float((got - want).abs().max() / want.abs().max()) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(6, 2, 24), (5, 1, 16), (9, 9, 8), (33, 4, 40)])
def test_softmax_routed_experts_op(dtype, shape):
    E, top, ff = shape
    W, n = 48, 37
    g = torch.Generator().manual_seed(6)
    w = {"router": torch.randn(E, W, generator=g) * 0.5}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = torch.randn(ff, W, generator=g) * 0.3, torch.randn(W, ff, generator=g) * 0.3
    w = {k: v.to(dtype).float() for k, v in w.items()}
    h = torch.randn(n, W, generator=g).to(dtype).float()
    mlp = {"router": {"experts": E, "top": top, "scale": 2.5}, "expert": {"ff": ff}}
    want = so.moe(h, mlp, w, "")
    idx, val = so.route(h, mlp, w["router"])
    t = lambda v: v.to(dtype).to(DEV)
    y, chosen, weights = ops.stack_moe(t(h), t(w["router"]), t(torch.stack([w[f"e{e}.up"] for e in range(E)])),
                                       t(torch.stack([w[f"e{e}.down"] for e in range(E)])), top, softmax=True,
                                       weight_output=True, act="relu2", route_scale=2.5)
    assert torch.equal(chosen.cpu().long().sort(-1).values, idx.sort(-1).values)
    assert (weights.cpu().sort(-1).values - val.sort(-1).values).abs().max() < 1e-5
    assert abs(float(weights.sum(-1).mean()) - 2.5) < 1e-4            # renormalised, then scaled
    assert float(row_err(y, want).max()) < (2e-5 if dtype == torch.float32 else 3e-2)


ONE_LAYER = {
    "delta": delta(heads=3, dim=16), "delta_wide": delta(heads=2, dim=40), "mamba": mamba(), "mamba_taps2": mamba(conv=2),
    "mamba_groups": mamba(heads=4, vdim=12, state=8, groups=2, conv=3, norm_groups=4), "mamba_tap1": mamba(conv=1),
    "attention": attn(), "attention_full": attn(window=0, rot={"base": 50.0, "dims": 12}, v_mix=False),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_mixer_alone_whole_decoded_and_in_portions(dtype, name):
    """A model of ONE layer without a feed-forward: the mixer's own path from the stream to the stream — in one go, with a
    decoded tail (state and the convolution's last inputs carried token by token), in portions of two and one."""
    cfg = config([(ONE_LAYER[name], None)])
    eng, w = make(cfg, dtype)
    toks = tokens(41, cfg["vocab"], 7)
    want = so.forward(cfg, w, toks)
    assert_close(eng.step([(0, toks, list(range(41)))]), want, dtype, "whole")
    rows = [eng.step([(1, toks[:30], list(range(30)))])] + [eng.step([(1, [t], [0])]) for t in toks[30:]]
    assert_close(torch.cat(rows), want, dtype, "decoded tail")
    rows, at = [], 0
    for c in [2, 1, 2, 2, 1, 1, 30, 2]:
        rows.append(eng.step([(3, toks[at:at + c], list(range(c)))]))
        at += c
    assert_close(torch.cat(rows), want, dtype, "portions")


# ------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompt(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(50, cfg["vocab"], 7)
    got = eng.step([(0, toks, list(range(50)))])
    want = so.forward(cfg, w, toks)
    assert_close(got, want, dtype, "whole prompt")
    assert_close(got[:3], want[:3], dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token_and_long_decode(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(120, cfg["vocab"], 8)
    want = so.forward(cfg, w, toks)
    rows = [eng.step([(2, toks[:30], list(range(30)))])]
    for t in range(30, 120):
        rows.append(eng.step([(2, [toks[t]], [0])]))
    assert_close(torch.cat(rows), want, dtype, "prefill + 90 decode steps")
    assert eng.slot_position(2) == 120


@pytest.mark.parametrize("dtype", DTYPES)
def test_from_the_first_token_one_by_one(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(20, cfg["vocab"], 9)
    rows = [eng.step([(1, [t], [0])]) for t in toks]
    assert_close(torch.cat(rows), so.forward(cfg, w, toks), dtype, "one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 44], [33, 2, 15], [1, 48, 1], [17, 16, 17]])
def test_prompt_in_portions(dtype, cuts):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    toks = tokens(sum(cuts), cfg["vocab"], 10)
    rows, at = [], 0
    for c in cuts:
        rows.append(eng.step([(0, toks[at:at + c], list(range(c)))]))
        at += c
    assert_close(torch.cat(rows), so.forward(cfg, w, toks), dtype, f"portions {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_against_each_alone_then_decoded_together(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    lens, new = [1, 37, 9], 12
    seqs = [tokens(n + new, cfg["vocab"], 20 + i) for i, n in enumerate(lens)]
    want = [so.forward(cfg, w, s) for s in seqs]
    slots = [3, 0, 2]
    got = eng.step([(sl, s[:n], list(range(n))) for sl, s, n in zip(slots, seqs, lens)])
    at = 0
    for i, n in enumerate(lens):
        assert_close(got[at:at + n], want[i][:n], dtype, f"batched prompt {i}")
        at += n
    live = [0, 1, 2]
    for t in range(new):
        if t == 5:                       # the middle request ends early; its slot goes back
            eng.release(slots[1])
            live = [0, 2]
        got = eng.step([(slots[i], [seqs[i][lens[i] + t]], [0]) for i in live])
        for r, i in enumerate(live):
            assert_close(got[r:r + 1], want[i][lens[i] + t:lens[i] + t + 1], dtype, f"decoded together {i} step {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_slot_given_back_and_used_again(dtype):
    """A finished request's slot is taken by a new one at position 0: nothing of the old caches, states or convolution
    inputs may show, whether the new request starts with a prompt or with a single token."""
    cfg = base_config()
    eng, w = make(cfg, dtype)
    old = tokens(60, cfg["vocab"], 30)
    eng.step([(1, old, [])])
    for start in (9, 1):
        eng.release(1)
        new = tokens(25, cfg["vocab"], 31 + start)
        rows = [eng.step([(1, new[:start], list(range(start)))])] + [eng.step([(1, [t], [0])]) for t in new[start:]]
        assert_close(torch.cat(rows), so.forward(cfg, w, new), dtype, f"reused slot, start {start}")


OTHER = {
    "attention_first": [(attn(v_mix=False), moe()), (delta(), None)],
    "one_mix_layer_only": [(attn(window=0), None), (mamba(), moe(shared=0))],
    "three_mix_layers": [(attn(), None), (attn(heads=2, kv_heads=2, dim=8, vdim=20, window=3), moe()), (delta(), None),
                         (attn(heads=6, kv_heads=2, dim=10, vdim=20, window=0, rot=None), None)],
    "plain_rotary_all_dims": [(attn(rot={"base": 30.0, "dims": 12}), moe(top=6))],
    "window_of_one": [(attn(window=1), moe(experts=2, top=1, ff=8, shared=8))],
    "one_head_each": [(delta(heads=1, dim=8), None), (mamba(heads=1, vdim=16, state=8, conv=2), None),
                      (attn(heads=1, kv_heads=1, dim=8, vdim=8, rot={"base": 10.0, "dims": 2}), moe(experts=3, top=3, shared=0))],
    "mamba_only": [(mamba(heads=2, vdim=40, state=40, conv=8), moe()), (mamba(heads=6, vdim=4, state=4, groups=3, norm_groups=3), None)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(OTHER))
@pytest.mark.parametrize("width,vocab", [(64, 96), (50, 77)])
def test_other_layer_orders_and_sizes(dtype, name, width, vocab):
    cfg = config(OTHER[name], width=width, vocab=vocab, embed_scale=1.0 if name == "one_head_each" else 2.5, eps=1e-6)
    eng, w = make(cfg, dtype, seed=3, rank=5)
    toks = tokens(36, vocab, 11)
    want = so.forward(cfg, w, toks)
    assert_close(eng.step([(0, toks, list(range(36)))]), want, dtype, name)
    rows = [eng.step([(2, toks[:7], list(range(7)))])] + [eng.step([(2, toks[t:t + 2], [0, 1][:len(toks[t:t + 2])])])
                                                         for t in range(7, 36, 2)]
    assert_close(torch.cat(rows), want, dtype, name + " in portions of two")


@pytest.mark.parametrize("what", ["embed_scale", "route_scale", "eps", "window", "rot_base", "rot_factor", "rot_dims", "scale",
                                  "v_mix", "top", "norm_groups"])
def test_constants_matter(what):
    """Each constant of the config changes the logits (a reader that dropped one would go unnoticed otherwise), and the
    engine follows the restatement under the change."""
    cfg = base_config()
    eng, w = make(cfg, torch.float32)
    toks = tokens(40, cfg["vocab"], 12)
    base = eng.step([(0, toks, list(range(40)))])
    eng.close()
    c2 = copy.deepcopy(cfg)
    a1 = c2["layers"][1]["mixer"]
    if what == "embed_scale":
        c2["embedding"]["scale"] = 1.0
    elif what == "route_scale":
        c2["layers"][0]["mlp"]["router"]["scale"] = 0.5
    elif what == "eps":
        c2["norm"]["eps"] = 0.3
    elif what == "window":
        a1["mask"]["size"] += 1
    elif what == "rot_base":
        a1["rot"]["base"] = 300.0
    elif what == "rot_factor":
        a1["rot"]["scaling"]["factor"] = 2.0
    elif what == "rot_dims":
        a1["rot"]["dims"] = 4
    elif what == "scale":
        a1["scale"] *= 1.7
    elif what == "v_mix":
        del c2["layers"][4]["mixer"]["v_mix"]
    elif what == "top":
        c2["layers"][1]["mlp"]["router"]["top"] = 2
    elif what == "norm_groups":
        c2["layers"][2]["mixer"]["norm_groups"] = 1
    spec = models.tekosun_from_config(c2).with_ctx(160, 4)
    eng2 = engine.DecodeEngine(spec, models.pack_weights(spec, {k: v for k, v in w.items() if k in models.tekosun_tensor_shapes(spec)},
                                                         device=DEV, dtype=torch.float32))
    got = eng2.step([(0, toks, list(range(40)))])
    assert float(row_err(got, base).max()) > 1e-3, what
    assert_close(got, so.forward(c2, w, toks), torch.float32, what)


def fast_config():
    """Sizes that reach the bf16 engines' fast paths: tcgen05 products (widths on multiples of 8, 64 and up), the tensor-core
    prompt attention (key size = value size = 64), per-expert tensor-core products, split-key decode."""
    return config([(delta(heads=4, dim=32), moe(experts=8, top=2, ff=64, shared=64)),
                   (attn(heads=4, kv_heads=2, dim=64, vdim=64, window=48, rot={"base": 10000.0, "dims": 32}), moe(experts=4, top=2, ff=64, shared=0)),
                   (mamba(heads=4, vdim=32, state=32, groups=2, conv=4, norm_groups=2), None),
                   (attn(heads=4, kv_heads=2, dim=64, vdim=64, window=0, rot=ROT), moe(experts=8, top=3, ff=64))],
                  width=128, vocab=256)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fast_path_sizes_whole_portions_and_decoded_beside_another(dtype):
    cfg = fast_config()
    eng, w = make(cfg, dtype, max_ctx=320, rank=64)
    toks, other = tokens(200, cfg["vocab"], 13), tokens(110, cfg["vocab"], 14)
    want = so.forward(cfg, w, toks)
    whole = eng.step([(0, toks, list(range(200)))])
    assert_close(whole, want, dtype, "whole")
    rows = [eng.step([(1, toks[:64], list(range(64))), (2, other[:50], [])]), eng.step([(1, toks[64:150], list(range(86)))])]
    for t in range(150, 200):
        rows.append(eng.step([(2, [other[50 + t - 150]], []), (1, [toks[t]], [0])]))
    cut = torch.cat(rows)
    assert_close(cut, want, dtype, "portions + decoded beside another request")
    if dtype == torch.bfloat16:       # the bf16 paths agree with each other far better than with the fp32 restatement
        e = row_err(cut, whole.float().cpu())
        assert float(e.median()) < 3e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_engine(dtype):
    cfg = base_config()
    eng, w = make(cfg, dtype)
    prompt, new = tokens(17, cfg["vocab"], 15), 12
    got = eng.generate_sync(prompt, new).tolist()
    seq = list(prompt)
    for i in range(new):              # the restatement's own greedy continuation; a near-tie may part the two in bf16
        lg = so.forward(cfg, w, seq)[-1]
        top2 = lg.topk(2).values
        if got[i] != int(lg.argmax()):
            assert dtype == torch.bfloat16 and float(top2[0] - top2[1]) < 0.05 * float(lg.std()), (i, got[i], int(lg.argmax()))
            break
        seq.append(got[i])
    prompts = [tokens(n, cfg["vocab"], 16 + n) for n in (3, 21, 8)]
    batch = eng.generate_sync_batch(prompts, 6).tolist()
    for p, g in zip(prompts, batch):
        eng2_first = int(so.forward(cfg, w, p)[-1].argmax())
        if dtype == torch.float32:
            assert g[0] == eng2_first
            assert g == eng.generate_sync(p, 6).tolist()


def test_prompt_longer_than_one_pass_of_the_engine():
    """A step of more rows than the engine takes through its layers at once goes in several passes: the states, the
    convolution's last inputs and the caches carry over the seam, also for a batch whose second sequence straddles it."""
    cfg = config([(delta(heads=2, dim=16), None), (mamba(heads=2, vdim=8, state=8, conv=4), None),
                  (attn(heads=2, kv_heads=1, dim=8, vdim=8, window=40), moe(experts=4, top=2, ff=16, shared=16))], width=32, vocab=64)
    n = 4096 + 300
    eng, w = make(cfg, torch.float32, max_ctx=n + 8, max_slots=2)
    toks = tokens(n, 64, 3)
    want = so.forward(cfg, w, toks)
    idx = list(range(0, n, 211)) + list(range(4090, 4104)) + [n - 1]
    assert_close(eng.step([(0, toks, idx)]), want[idx], torch.float32, "whole")
    eng.release(0)
    got = eng.step([(1, toks[:2500], [2499]), (0, toks[:3000], [0, 2999])])
    assert_close(got, torch.stack([want[2499], want[0], want[2999]]), torch.float32, "batch over the seam")


def test_seek_and_overflow_refused():
    cfg = base_config()
    eng, _ = make(cfg, torch.float32, max_ctx=32)
    toks = tokens(20, cfg["vocab"], 17)
    eng.step([(0, toks, [])], greedy=True)
    with pytest.raises(Exception):
        eng.seek(5)                   # the recurrent states hold the whole prefix and nothing of its past
    with pytest.raises(Exception):
        eng.step([(0, toks, [])])     # 20 + 20 > 32
    assert eng.slot_position(0) == 20
