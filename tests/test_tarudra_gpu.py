"""Tarudra design in the layer-stack engine against the plain restatement in tests/tarudra_oracle.py: every mixer alone as a
one-layer model (whole, decoded, in portions), crafted scores at every window's edge, far away and under the sink, whole
prompts, decoding through caches and states, prompts cut into portions down to one and two tokens, unequal batches, slots
given back and used again, long decoding past the windows, other sizes and layer orders, the constants shown to matter,
sizes that reach the tensor-core paths, greedy generation through the engine's own entry points."""
import copy
import math

import pytest
import torch

import tarudra_oracle as so
from tinygpt_b200 import engine, models

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
# fp32 engines are held to summation-order noise on EVERY row; bf16 engines round matrices' operands to 8 bits of mantissa
# and are held to the median row and to most rows against the fp32 restatement.
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


YARN = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "fast": 8.0, "original": 24, "slow": 1.0}}


def attn(heads=4, kv_heads=2, dim=12, vdim=20, window=9, rot=YARN, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim)}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = copy.deepcopy(rot)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=8, rot_dim=4, vdim=10, kv_rank=12, q_rank=10, window=7, base=100.0, scale=None, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale or 1.0 / math.sqrt(dim + rot_dim)}
    if window:
        m["mask"] = {"size": window}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            m["rot"]["scaling"] = copy.deepcopy(scaling)
    return {"type": "latent_attention", "mixer": m}


def delta(heads=4, kv_heads=2, dim=16, vdim=8, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def ff(n=48):
    return {"kind": "dense", "ff": n}


def config(layers, width=64, vocab=96, eps=1e-5, cap=12.0):
    return {"architecture": "Tarudra", "layers": [dict(copy.deepcopy(mix), mlp=copy.deepcopy(mlp)) for mix, mlp in layers],
            "logit_softcap": cap, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def base_config():
    return config([(attn(), ff()), (delta(), ff(40)), (latent(), ff()), (attn(window=5, kv_from=0), None),
                   (latent(heads=2, dim=6, rot_dim=6, vdim=7, kv_rank=9, q_rank=5, window=0, base=50.0), ff(24)),
                   (delta(heads=2, kv_heads=2, dim=24, vdim=24, conv=4), ff())])


def make(cfg, dtype, seed=0, max_ctx=160, max_slots=4, weights=None):
    spec = models.tarudra_from_config(cfg).with_ctx(max_ctx, max_slots)
    w = weights if weights is not None else models.synth_tarudra_weights(spec, seed=seed)
    eng = engine.DecodeEngine(spec, models.pack_weights(spec, w, device=DEV, dtype=dtype))
    return eng, {k: v.float() for k, v in w.items()}


def tokens(n, vocab, seed, low=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(low, vocab, (n,), generator=g).tolist()


def run_ways(eng, toks, head):
    """The same tokens whole, with a decoded tail, and in small portions → three [n, vocab] results."""
    n = len(toks)
    whole = eng.step([(0, toks, list(range(n)))])
    tail = torch.cat([eng.step([(1, toks[:head], list(range(head)))])] + [eng.step([(1, [t], [0])]) for t in toks[head:]])
    rows, at, cuts = [], 0, [2, 1, 2, 2, 1, 1]
    cuts = cuts + [n - sum(cuts) - 2, 2]
    for c in cuts:
        rows.append(eng.step([(3, toks[at:at + c], list(range(c)))]))
        at += c
    return whole, tail, torch.cat(rows)


# ------------------------------------------------------------------------------------------- each mechanism alone
ONE_LAYER = {
    "attention": attn(), "attention_full_rotation": attn(window=0, rot={"base": 50.0, "dims": 12}),
    "attention_no_rotation_no_groups": attn(heads=3, kv_heads=3, dim=10, vdim=6, window=4, rot=None),
    "attention_one_kv_head": attn(heads=6, kv_heads=1, dim=8, vdim=40, window=13, rot={"base": 10.0, "dims": 2}),
    "latent": latent(), "latent_no_window_yarn": latent(window=0, rot_dim=8, scaling={"factor": 3.0, "fast": 4.0, "original": 16, "slow": 1.0}),
    "latent_no_rotated_part": latent(rot_dim=0, kv_rank=20, q_rank=3), "latent_one_head": latent(heads=1, dim=4, rot_dim=2, vdim=33, kv_rank=5, q_rank=17, window=2),
    "delta": delta(), "delta_equal_heads": delta(heads=3, kv_heads=3, dim=20, vdim=33, conv=2),
    "delta_one_tap": delta(heads=2, kv_heads=1, dim=40, vdim=8, conv=1), "delta_wide_key": delta(heads=2, kv_heads=1, dim=130, vdim=5, conv=4),
    "delta_six_taps": delta(heads=6, kv_heads=2, dim=8, vdim=16, conv=6),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_mixer_alone_whole_decoded_and_in_portions(dtype, name):
    """A model of ONE layer without a feed-forward: the mixer's own path from the stream to the stream — in one go, with a
    decoded tail (caches, state and the convolutions' last inputs carried token by token), in portions of two and one."""
    cfg = config([(ONE_LAYER[name], None)])
    eng, w = make(cfg, dtype)
    toks = tokens(41, cfg["vocab"], 7)
    want = so.forward(cfg, w, toks)
    for what, got in zip(("whole", "decoded tail", "portions"), run_ways(eng, toks, 30)):
        assert_close(got, want, dtype, what)


def _aimed(cfg, seed, n, target, dtype):
    """A one-layer model and n tokens in which the LAST token's query is aimed at the key of position `target`: token 0 stands
    only at the target, token 1 only at the end; in every head the rows of the key projection that feed one entry are set along
    token 0's normed embedding and the query's along token 1's, ten times larger than anything random."""
    spec = models.tarudra_from_config(cfg)
    w = models.synth_tarudra_weights(spec, seed=seed)
    toks = tokens(n, cfg["vocab"], seed + 1, low=2)
    toks[target], toks[-1] = 0, 1
    f = {k: v.float() for k, v in w.items()}
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    hk, hq = so.layer_norm(f["embed"][0], f["l0.norm1"], eps), so.layer_norm(f["embed"][1], f["l0.norm1"], eps)
    c = 10.0
    if cfg["layers"][0]["type"] == "attention":
        dk, last = m["dim"], m["dim"] - 1           # the head's last entry: behind the rotated ones
        assert (m.get("rot") or {"dims": 0})["dims"] < dk
        for g in range(m["kv_heads"]):
            f["l0.mix.k"][g * dk + last] = c * hk / hk.pow(2).sum()
            f["l0.mix.k.b"][g * dk + last] = 0.0
        for h in range(m["heads"]):
            f["l0.mix.q"][h * dk + last] = c * hq / hq.pow(2).sum()
            f["l0.mix.q.b"][h * dk + last] = 0.0
    else:
        r, dr, hd = m["kv_rank"], m["rot_dim"], m["dim"] + m["rot_dim"]
        i = dr // 2 - 1                              # the slowest pair of the shared rotated key part (rotate-half layout)
        f["l0.mix.dkv"][r + i] = c * hk / hk.pow(2).sum()
        f["l0.mix.dkv"][r + i + dr // 2] = 0.0
        cq = so.rms_norm(f["l0.mix.dq"] @ hq, f["l0.mix.dq.norm"], eps)
        for h in range(m["heads"]):
            row = h * hd + m["dim"]
            f["l0.mix.uq"][row + i] = c * cq / cq.pow(2).sum()
            f["l0.mix.uq"][row + i + dr // 2] = 0.0
    w = {k: v.to(torch.bfloat16) for k, v in f.items()}
    return w, toks


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("case", ["last_inside", "first_outside", "far"])
@pytest.mark.parametrize("kind", ["attention", "latent_attention", "attention_tensor_core_sizes", "latent_attention_tensor_core_sizes"])
def test_crafted_scores_at_the_window_edge_and_far_away(dtype, decode, case, kind):
    """300 positions.  The last query is aimed at ONE earlier key so that its score would dominate: the key just inside the
    window must own the output, the key just outside must not be seen at all, and without a window a key 296 positions back
    must be found — in a prompt and when the last token is decoded alone; also at head sizes that send the bf16 engine's
    prompts to the tensor-core attention kernel and its decode steps to the split-key kernels."""
    n, window = 300, 64
    win = 0 if case == "far" else window
    mix = {"attention": attn(window=win, rot={"base": 100.0, "dims": 4}, scale=1.0),
           "latent_attention": latent(heads=2, window=win, rot_dim=8, base=1e6, scale=1.0),
           "attention_tensor_core_sizes": attn(heads=4, kv_heads=2, dim=64, vdim=64, window=win, rot={"base": 100.0, "dims": 32}, scale=1.0),
           "latent_attention_tensor_core_sizes": latent(heads=2, dim=32, rot_dim=32, vdim=64, kv_rank=64, q_rank=64, window=win, base=1e7,
                                                        scale=1.0)}[kind]
    cfg = config([(mix, None)])
    target = {"last_inside": n - window, "first_outside": n - 1 - window, "far": 3}[case]
    w, toks = _aimed(cfg, 2, n, target, dtype)
    eng, wf = make(cfg, dtype, max_ctx=320, weights=w)
    want = so.forward(cfg, wf, toks)
    # what the last row would be with a window one key wider (or narrower) tells the cases apart by a wide margin
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["mask"] = {"size": {"last_inside": window - 1, "first_outside": window + 1, "far": 200}[case]}
    assert float(row_err(so.forward(other, wf, toks)[-1:], want[-1:]).max()) > 0.2
    if decode:
        eng.step([(1, toks[:-1], [])])
        got = eng.step([(1, toks[-1:], [0])])
    else:
        got = eng.step([(1, toks, [n - 1])])
    assert float(row_err(got, want[-1:]).max()) < (1e-4 if dtype == torch.float32 else 6e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_sink_takes_the_weight_when_every_score_is_low(dtype, decode):
    """Every key carries a large bias along one entry and the query the opposite sign there: all scores are far below zero,
    so the sink owns the softmax and the heads' outputs vanish; an ordinary softmax would average the values instead."""
    cfg = config([(attn(window=0, rot={"base": 100.0, "dims": 4}, scale=1.0), None)])
    spec = models.tarudra_from_config(cfg)
    w = models.synth_tarudra_weights(spec, seed=4)
    dk = cfg["layers"][0]["mixer"]["dim"]
    for g in range(2):
        w["l0.mix.k.b"][g * dk + dk - 1] = 6.0
    for h in range(4):
        w["l0.mix.q.b"][h * dk + dk - 1] = -6.0
    eng, wf = make(cfg, dtype, weights=w)
    toks = tokens(70, cfg["vocab"], 5)
    want = so.forward(cfg, wf, toks)
    assert float(row_err(so.forward(cfg, wf, toks, sink=False), want).min()) > 0.2
    got = torch.cat([eng.step([(0, toks[:40], list(range(40)))])] + [eng.step([(0, [t], [0])]) for t in toks[40:]]) if decode \
        else eng.step([(0, toks, list(range(70)))])
    assert_close(got, want, dtype, "sink")


def test_sink_matters_with_ordinary_scores():
    cfg = base_config()
    eng, w = make(cfg, torch.float32)
    toks = tokens(30, cfg["vocab"], 6)
    got = eng.step([(0, toks, list(range(30)))])
    assert float(row_err(so.forward(cfg, w, toks, sink=False), got).max()) > 1e-2
    assert_close(got, so.forward(cfg, w, toks), torch.float32, "with the sink")


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_keeps_a_value_written_long_ago(dtype):
    """Decays close to one: what the first tokens wrote still shows 200 tokens later (a state that was lost or reset on
    the way would not), whole and with the tail decoded one token at a time."""
    cfg = config([(delta(heads=2, kv_heads=1, dim=16, vdim=12, conv=2), None)])
    spec = models.tarudra_from_config(cfg)
    w = models.synth_tarudra_weights(spec, seed=8)
    w["l0.mix.A_log"][:] = -6.0
    eng, wf = make(cfg, dtype, max_ctx=256, weights=w)
    toks = tokens(220, cfg["vocab"], 9)
    want = so.forward(cfg, wf, toks)
    changed = list(toks)
    changed[2] = (toks[2] + 1) % cfg["vocab"]
    assert float(row_err(so.forward(cfg, wf, changed)[-1:], want[-1:]).max()) > 1e-2
    got = torch.cat([eng.step([(2, toks[:150], list(range(150)))])] + [eng.step([(2, [t], [0])]) for t in toks[150:]])
    assert_close(got, want, dtype, "long memory")
    assert_close(eng.step([(1, toks, [219])]), want[-1:], dtype, "whole")


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
@pytest.mark.parametrize("cuts", [[2, 2, 2, 44], [33, 2, 15], [1, 48, 1], [17, 16, 17], [5, 4, 9, 8, 7, 10, 7]])
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
    "delta_first_no_feed_forward_anywhere": [(delta(), None), (attn(), None), (latent(), None)],
    "shared_keys_twice": [(attn(window=0), ff()), (attn(window=3, kv_from=0), ff(8)), (latent(), None), (attn(window=20, kv_from=0), ff())],
    "two_sources": [(attn(), None), (attn(heads=2, kv_heads=1, dim=8, vdim=8, window=6, rot=None), ff()), (attn(heads=2, kv_heads=1, dim=8, vdim=8, window=2, rot=None, kv_from=1), ff()),
                    (attn(kv_from=0, window=0), None)],
    "window_of_one": [(attn(window=1), ff()), (latent(window=1), ff())],
    "one_head_each": [(delta(heads=1, kv_heads=1, dim=8, vdim=8, conv=2), None), (latent(heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=8, q_rank=8), None),
                      (attn(heads=1, kv_heads=1, dim=8, vdim=8, rot={"base": 10.0, "dims": 8}), ff(16))],
    "latent_only": [(latent(heads=5, dim=3, rot_dim=6, vdim=4, kv_rank=40, q_rank=33, window=11), ff()), (latent(window=0), None)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(OTHER))
@pytest.mark.parametrize("width,vocab,cap", [(64, 96, 9.0), (50, 77, 0.0)])
def test_other_layer_orders_and_sizes(dtype, name, width, vocab, cap):
    cfg = config(OTHER[name], width=width, vocab=vocab, eps=1e-6, cap=cap)
    eng, w = make(cfg, dtype, seed=3)
    toks = tokens(36, vocab, 11)
    want = so.forward(cfg, w, toks)
    assert_close(eng.step([(0, toks, list(range(36)))]), want, dtype, name)
    rows = [eng.step([(2, toks[:7], list(range(7)))])] + [eng.step([(2, toks[t:t + 2], [0, 1][:len(toks[t:t + 2])])])
                                                         for t in range(7, 36, 2)]
    assert_close(torch.cat(rows), want, dtype, name + " in portions of two")


@pytest.mark.parametrize("what", ["eps", "window", "latent_window", "rot_base", "rot_factor", "rot_slow", "rot_dims", "scale", "latent_scale",
                                  "latent_base", "kv_from", "softcap", "conv_state"])
def test_constants_matter(what):
    """Each constant of the config changes the logits (a reader that dropped one would go unnoticed otherwise), and the
    engine follows the restatement under the change."""
    cfg = base_config()
    eng, w = make(cfg, torch.float32)
    toks = tokens(40, cfg["vocab"], 12)
    base = eng.step([(0, toks, list(range(40)))])
    eng.close()
    c2 = copy.deepcopy(cfg)
    a0, l2 = c2["layers"][0]["mixer"], c2["layers"][2]["mixer"]
    if what == "eps":
        c2["norm"]["eps"] = 0.3
    elif what == "window":
        a0["mask"]["size"] += 1
    elif what == "latent_window":
        l2["mask"]["size"] -= 1
    elif what == "rot_base":
        a0["rot"]["base"] = 300.0
    elif what == "rot_factor":
        a0["rot"]["scaling"]["factor"] = 2.0
    elif what == "rot_slow":
        a0["rot"]["scaling"]["slow"] = 0.05
    elif what == "rot_dims":
        a0["rot"]["dims"] = 4
    elif what == "scale":
        a0["scale"] *= 1.7
    elif what == "latent_scale":
        l2["scale"] *= 1.7
    elif what == "latent_base":
        l2["rot"]["base"] = 3.0
    elif what == "kv_from":          # keys and values of its own instead of layer 0's: the tensors must exist
        c2["layers"] = c2["layers"][:3] + [dict(attn(window=5), mlp=None)] + c2["layers"][4:]
    elif what == "softcap":
        c2["logit_softcap"] = 3.0
    if what == "kv_from":
        spec = models.tarudra_from_config(c2)
        w2 = models.synth_tarudra_weights(spec, seed=0)
        w2 = {k: (w[k].to(torch.bfloat16) if k in w else v) for k, v in w2.items()}
    else:
        w2 = {k: v.to(torch.bfloat16) for k, v in w.items()}
    if what == "conv_state":         # the third tap back reads another token: the convolution reaches over the portion's edge
        toks2 = list(toks)
        toks2[17] = (toks[17] + 1) % cfg["vocab"]
        eng2, wf = make(c2, torch.float32, weights=w2)
        got = torch.cat([eng2.step([(0, toks2[:18], list(range(18)))]), eng2.step([(0, toks2[18:], list(range(22)))])])
        assert float(row_err(got[18:20], base[18:20]).max()) > 1e-3
        assert_close(got, so.forward(c2, wf, toks2), torch.float32, what)
        return
    eng2, wf = make(c2, torch.float32, weights=w2)
    got = eng2.step([(0, toks, list(range(40)))])
    assert float(row_err(got, base).max()) > 1e-3, what
    assert_close(got, so.forward(c2, wf, toks), torch.float32, what)


def fast_config():
    """Sizes that reach the bf16 engines' fast paths: tcgen05 products (widths on multiples of 8, 64 and up), the tensor-core
    prompt attention for both attentions (key size = value size = 64), split-key decode."""
    return config([(attn(heads=4, kv_heads=2, dim=64, vdim=64, window=48, rot={"base": 10000.0, "dims": 32}), ff(256)),
                   (latent(heads=4, dim=32, rot_dim=32, vdim=64, kv_rank=64, q_rank=64, window=40, base=10000.0), ff(256)),
                   (delta(heads=4, kv_heads=2, dim=32, vdim=32, conv=4), ff(256)),
                   (attn(heads=4, kv_heads=2, dim=64, vdim=64, window=0, rot=YARN, kv_from=0), None),
                   (latent(heads=2, dim=64, rot_dim=64, vdim=128, kv_rank=128, q_rank=96, window=0, base=10000.0), ff(128))],
                  width=128, vocab=256)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fast_path_sizes_whole_portions_and_decoded_beside_another(dtype):
    cfg = fast_config()
    eng, w = make(cfg, dtype, max_ctx=320)
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
    if dtype == torch.float32:
        assert got == so.greedy(cfg, w, prompt, new)
    prompts = [tokens(n, cfg["vocab"], 16 + n) for n in (3, 21, 8)]
    batch = eng.generate_sync_batch(prompts, 6).tolist()
    for p, g in zip(prompts, batch):
        if dtype == torch.float32:
            assert g[0] == int(so.forward(cfg, w, p)[-1].argmax())
            assert g == eng.generate_sync(p, 6).tolist()


def test_prompt_longer_than_one_pass_of_the_engine():
    """A step of more rows than the engine takes through its layers at once goes in several passes: the states, the
    convolutions' last inputs and the caches (also the shared ones) carry over the seam, also for a batch whose second
    sequence straddles it."""
    cfg = config([(delta(heads=2, kv_heads=1, dim=16, vdim=8), None), (attn(heads=2, kv_heads=1, dim=8, vdim=8, window=40), ff(16)),
                  (latent(heads=2, window=30), None), (attn(heads=2, kv_heads=1, dim=8, vdim=8, window=25, kv_from=1), None)],
                 width=32, vocab=64)
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
