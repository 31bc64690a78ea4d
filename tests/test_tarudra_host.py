"""Host side of the Tarudra design (no GPU): config reader and registry, merged layouts, the folded layer scale, rotary
frequencies and tables against the restatement, checkpoint round trip through the loader, and the restatement's own sanity
(causality, the sink, the windows, closed forms of the gated delta rule and of the short convolution)."""
import copy
import math

import pytest
import torch

import tarudra_oracle as so
from tinygpt_b200 import loader, models

YARN = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "fast": 8.0, "original": 24, "slow": 1.0}}


def cfg_small():
    return {"architecture": "Tarudra", "width": 40, "vocab": 50, "norm": {"eps": 1e-4}, "logit_softcap": 7.0,
            "layers": [
                {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 6, "scale": 0.3, "rot": copy.deepcopy(YARN),
                                                "mask": {"size": 7}}, "mlp": {"kind": "dense", "ff": 24}},
                {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 3}, "mlp": None},
                {"type": "latent_attention", "mixer": {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 7, "kv_rank": 9, "q_rank": 11,
                                                       "scale": 0.25, "rot": {"base": 100.0, "dims": 4}, "mask": {"size": 5}},
                 "mlp": {"kind": "dense", "ff": 16}},
                {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 6, "scale": 0.2, "rot": copy.deepcopy(YARN),
                                                "kv_from": 0}, "mlp": None}]}


def test_registry_reads_the_config_and_writes_it_back():
    cfg = cfg_small()
    spec = models.ARCHITECTURES["Tarudra"](cfg)
    assert spec.architecture == "Tarudra" and spec.block == "sandwich" and spec.norm_kind == "layer" and spec.layer_scale
    assert spec.logit_softcap == 7.0 and spec.norm_eps == 1e-4 and [r[0] for r in spec.runs()] == [0, 1, 2, 3]
    a = spec.layers[0]
    assert a.attn.window == 7 and a.attn.sink and a.attn.bias and a.attn.out_bias and not a.attn.out_gate and a.kv_from is None
    assert a.prep.rot_interleaved and a.prep.rot.factor == 4.0 and not a.prep.qk_norm and a.ff_act == "relu2" and a.ff == 24
    d = spec.layers[1].gdelta
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv, d.unit_eps) == (4, 2, 6, 5, 3, 1e-6) and spec.layers[1].ff == 0
    q = spec.layers[2].latent
    assert q.rot_layout == "half" and q.q_rank == 11 and q.window == 5 and q.out_gate and q.rot.factor == 0.0
    assert spec.layers[3].kv_from == 0 and spec.layers[3].attn.window == 0
    assert models.tarudra_from_config(models.tarudra_config(spec)) == spec and models.tarudra_config(spec) == cfg
    for i, bad in ((1, {"type": "mlstm"}), (0, {"mlp": {"kind": "moe"}})):
        c = cfg_small()
        c["layers"][i].update(bad)
        with pytest.raises(ValueError):
            models.tarudra_from_config(c)
    for path, val in ((("layers", 0, "mixer", "rot", "dims"), 12), (("layers", 3, "mixer", "kv_from"), 2), (("layers", 3, "mixer", "kv_from"), 3),
                      (("layers", 3, "mixer", "vdim"), 8), (("layers", 1, "mixer", "kv_heads"), 3)):
        c = cfg_small()
        node = c
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = val
        with pytest.raises(ValueError):
            models.tarudra_from_config(c)


@pytest.mark.parametrize("rot", [YARN, {"base": 100.0, "dims": 4}, {"base": 500000.0, "dims": 32, "scaling": {
    "factor": 16.0, "fast": 32.0, "original": 512, "slow": 2.0}}])
def test_rotary_frequencies_and_table_match_the_restatement(rot):
    sc = rot.get("scaling") or {}
    spec = models.RotarySpec(rot["dims"], rot["base"], sc.get("factor", 0.0), sc.get("original", 0), sc.get("fast", 0.0), sc.get("slow", 0.0))
    f0, mag0 = so.rotary_frequencies(rot)
    f, mag = spec.frequencies()
    assert torch.allclose(torch.from_numpy(f), f0, rtol=1e-12, atol=0) and abs(mag - mag0) < 1e-15
    tab = spec.table(77)
    pos = torch.arange(77)
    for layout in ("interleaved", "half"):
        v = torch.randn(77, 2, rot["dims"] + 3, dtype=torch.float64)
        want = so.rotate(v, pos, rot, layout)
        h = rot["dims"] // 2
        a, b = (v[..., 0:2 * h:2], v[..., 1:2 * h:2]) if layout == "interleaved" else (v[..., :h], v[..., h:2 * h])
        c, s = tab[:, None, :, 0].double(), tab[:, None, :, 1].double()
        got = v.clone()
        if layout == "interleaved":
            got[..., 0:2 * h:2], got[..., 1:2 * h:2] = a * c - b * s, b * c + a * s
        else:
            got[..., :h], got[..., h:2 * h] = a * c - b * s, b * c + a * s
        assert (got - want).abs().max() < 1e-6 and torch.equal(got[..., 2 * h:], v[..., 2 * h:])


def test_layouts_and_packed_weights():
    spec = models.tarudra_from_config(cfg_small())
    w = models.synth_tarudra_weights(spec, seed=1)
    assert set(w) == set(models.tarudra_tensor_shapes(spec)) and "l3.mix.k" not in w and "l1.mlp.up" not in w
    pk = models.pack_weights(spec, w, device="cpu", dtype=torch.float32)
    la = spec.mix_layout(0)
    assert (la.off_q, la.off_k, la.off_v, la.n_in, la.k_out) == (0, 40, 64, 80, 24)
    assert torch.equal(pk["l0.w_in"][la.off_k:la.off_k + 20], w["l0.mix.k"].float()) and float(pk["l0.w_in"][60:64].abs().max()) == 0
    assert torch.equal(pk["l0.b_in"][la.off_v:la.off_v + 12], w["l0.mix.v.b"].float()) and torch.equal(pk["l0.b_out"], w["l0.mix.o.b"].float())
    ld = spec.mix_layout(1)
    assert (ld.off_q, ld.off_k, ld.off_v, ld.off_g, ld.off_gate, ld.off_up, ld.n_in) == (0, 16, 32, 56, 80, 88, 96)
    assert torch.equal(pk["l1.w_in"][ld.off_gate:ld.off_gate + 4], w["l1.mix.b"].float()) and torch.equal(pk["l1.w_in"][ld.off_up:ld.off_up + 4], w["l1.mix.a"].float())
    assert pk["l1.conv_w"].shape == ((12 + 12 + 20) * 3,) and torch.equal(pk["l1.conv_w"].view(44, 3)[12:24], w["l1.mix.k.conv"].float())
    ll = spec.mix_layout(2)
    assert (ll.off_q, ll.off_k, ll.off_g, ll.n_in, ll.k_out) == (0, 16, 32, 56, 21)
    assert pk["l2.uq"].shape == (30, 16) and float(pk["l2.uq"][:, 11:].abs().max()) == 0 and pk["l2.uk_t"].shape == (3, 9, 6)
    assert spec.mix_layout(3).n_in == 40 and "l3.b_out" in pk
    # the layer scale rides on the post-norm's weight, exactly
    assert torch.equal(pk["l2.ff_post_norm"], w["l2.norm2b"].float() * w["l2.ls2"].float())
    assert torch.equal(pk["l1.post_norm"], w["l1.norm1b"].float() * w["l1.ls1"].float()) and "l1.ff_post_norm" not in pk
    assert spec.weight_params() > 0


def test_checkpoint_round_trip_through_the_loader(tmp_path):
    spec = models.tarudra_from_config(cfg_small())
    w = models.synth_tarudra_weights(spec, seed=2)
    models.save_stack_checkpoint(spec, w, str(tmp_path))
    assert loader.is_stack_model(tmp_path)
    spec2, pk = loader.load_model(tmp_path, device="cpu", dtype=torch.float32, max_ctx=99, max_slots=3)
    assert spec2 == spec.with_ctx(99, 3)
    want = models.pack_weights(spec, w, device="cpu", dtype=torch.float32)
    assert set(pk) == set(want) and all(torch.equal(pk[k], want[k]) for k in want)
    (tmp_path / "config.json").write_text((tmp_path / "config.json").read_text().replace('"conv": 3', '"conv": 4'))
    with pytest.raises(loader.LoaderError):
        loader.load_model(tmp_path, device="cpu", dtype=torch.float32)


def test_restatement_is_causal_and_its_mechanisms_are_what_the_equations_say():
    cfg = cfg_small()
    spec = models.tarudra_from_config(cfg)
    w = {k: v.double() for k, v in models.synth_tarudra_weights(spec, seed=3).items()}
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=g).tolist()
    full = so.forward(cfg, w, toks)
    assert (so.forward(cfg, w, toks[:11]) - full[:11]).abs().max() < 1e-9
    seq = so.Sequence(cfg)                                                  # in portions, through the carried memory
    parts = torch.cat([so.forward(cfg, w, toks[a:b], seq) for a, b in ((0, 1), (1, 3), (3, 12), (12, 19))])
    assert (parts - full).abs().max() < 1e-9 and float(full.abs().max()) < 7.0
    # windows: position i sees itself and the size − 1 positions before it
    vis = so.window_mask(torch.arange(6), torch.arange(6), 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True, False, False, False, False]
    assert bool(so.window_mask(torch.arange(4), torch.arange(4), 0)[3].all())
    # the sink: one key of score s gets e^s / (1 + e^s) of its value
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0}
    ww = {"mix.q": torch.zeros(2, 3, dtype=torch.float64), "mix.q.b": torch.tensor([1.0, 0.0], dtype=torch.float64),
          "mix.o": torch.ones(1, 1, dtype=torch.float64), "mix.o.b": torch.zeros(1, dtype=torch.float64)}
    out = so.attention(torch.zeros(1, 3, dtype=torch.float64), torch.arange(1), m, ww, "", torch.tensor([[[0.7, 5.0]]], dtype=torch.float64),
                       torch.tensor([[[3.0]]], dtype=torch.float64), torch.arange(1))
    assert abs(float(out) - 3.0 * math.exp(0.7) / (1.0 + math.exp(0.7))) < 1e-12
    # the short convolution: the last column meets the current token, zeros stand before the sequence, the state carries on
    taps = torch.tensor([[1.0, 10.0, 100.0]], dtype=torch.float64)
    x = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=torch.float64)
    y, last = so.short_conv(x, taps, None)
    assert y[:, 0].tolist() == [100.0, 210.0, 321.0, 432.0] and last[:, 0].tolist() == [3.0, 4.0]
    y2, _ = so.short_conv(x[2:], taps, so.short_conv(x[:2], taps, None)[1])
    assert torch.equal(y2, y[2:])
    # gated delta rule, ONE token into a fresh state: S = k (beta v)ᵀ, so o = (k·q) beta v, whatever the decay is
    md = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "conv": 1}
    W = 6
    wd = {"mix.q": torch.randn(4, W, dtype=torch.float64), "mix.k": torch.randn(4, W, dtype=torch.float64), "mix.v": torch.randn(3, W, dtype=torch.float64),
          "mix.q.conv": torch.ones(4, 1, dtype=torch.float64), "mix.k.conv": torch.ones(4, 1, dtype=torch.float64),
          "mix.v.conv": torch.ones(3, 1, dtype=torch.float64), "mix.b": torch.randn(1, W, dtype=torch.float64),
          "mix.a": torch.randn(1, W, dtype=torch.float64), "mix.A_log": torch.zeros(1, dtype=torch.float64),
          "mix.dt_bias": torch.zeros(1, dtype=torch.float64), "mix.norm": torch.ones(3, dtype=torch.float64),
          "mix.g": torch.randn(3, W, dtype=torch.float64), "mix.o": torch.eye(3, dtype=torch.float64)}
    h = torch.randn(1, W, dtype=torch.float64)
    out, st = so.delta_mixer(h, md, wd, "", 1e-5, None)
    silu = torch.nn.functional.silu
    q, k, v = silu(wd["mix.q"] @ h[0]), silu(wd["mix.k"] @ h[0]), silu(wd["mix.v"] @ h[0])
    q, k = q / torch.sqrt(q @ q + 1e-6) / 2.0, k / torch.sqrt(k @ k + 1e-6)
    beta = torch.sigmoid(wd["mix.b"] @ h[0])
    o = float(k @ q) * beta * v
    want = o / torch.sqrt((o * o).mean() + 1e-5) * silu(wd["mix.g"] @ h[0])
    assert (out[0] - want).abs().max() < 1e-12 and (st["S"][0] - torch.outer(k, beta * v)).abs().max() < 1e-12
    # a second, equal token: the state first decays, then gives up what it holds along k before the new value goes in —
    # with a unit key the state along k is replaced by a blend: S k-row = (1 − beta) g S + beta v
    out2, st2 = so.delta_mixer(torch.cat([h, h]), md, wd, "", 1e-5, None)
    gdec = math.exp(-math.exp(0.0) * float(torch.nn.functional.softplus(wd["mix.a"] @ h[0])))
    kk = float(k @ k)
    want_S = gdec * st["S"][0] - torch.outer(k, float(beta) * (gdec * st["S"][0].T @ k)) + torch.outer(k, beta * v)
    assert (st2["S"][0] - want_S).abs().max() < 1e-12 and abs(kk - 1.0) < 1e-5
