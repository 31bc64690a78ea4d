"""Host side of the Tekosun design (no GPU): config reader and registry, merged layouts, rotary frequencies against the
restatement, checkpoint round trip through the loader (the decay bottleneck's rank read from the tensors), and the
restatement's own sanity (causality and closed forms of the recurrences)."""
import copy
import math

import pytest
import torch

import tekosun_oracle as so
from tinygpt_b200 import loader, models

ROT = {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "high": 4.0, "low": 1.0, "original": 32}}


def cfg_small():
    moe = {"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 4, "top": 2, "scale": 1.5}, "shared": {"ff": 11}}
    return {"architecture": "Tekosun", "width": 40, "vocab": 50, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-4},
            "layers": [
                {"type": "general_delta", "mixer": {"heads": 2, "dim": 6}, "mlp": None},
                {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 6, "scale": 0.3, "rot": copy.deepcopy(ROT),
                                                "mask": {"size": 7}, "v_mix": True}, "mlp": moe},
                {"type": "mamba2", "mixer": {"heads": 4, "vdim": 6, "state": 5, "groups": 2, "conv": 3, "norm_groups": 2},
                 "mlp": {"kind": "moe", "expert": {"ff": 5}, "router": {"experts": 3, "top": 1, "scale": 1.0}}},
                {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.5,
                                                "rot": {"base": 100.0, "dims": 2}, "v_mix": True}, "mlp": None}]}


def test_registry_reads_the_config_and_writes_it_back():
    cfg = cfg_small()
    spec = models.ARCHITECTURES["Tekosun"](cfg, {"l0.mix.w1": (3, 40)})
    assert spec.architecture == "Tekosun" and spec.block == "postnorm" and spec.norm_kind == "rms" and spec.embed_scale == 2.0
    assert [r[0] for r in spec.runs()] == [0, 1, 2, 3]
    assert spec.layers[0].delta.rank == 3                                   # from the tensor's shape
    assert abs(spec.layers[0].delta.decay_scale - math.exp(-0.5)) < 1e-15 and spec.layers[0].delta.unit_eps == 1e-6
    a = spec.layers[1]
    assert a.attn.window == 7 and a.attn.keep_first == 0 and not a.attn.out_gate and a.prep.qk_norm and a.prep.v_norm and a.prep.v_mix
    assert a.prep.rot.factor == 8.0 and spec.layers[3].prep.rot.factor == 0.0 and spec.layers[3].attn.window == 0
    assert a.moe.router == "softmax" and a.moe.weight_output and a.moe.act == "relu2" and a.moe.shared_plain and a.moe.route_scale == 1.5
    assert spec.layers[2].moe.shared_ff == 0 and spec.layers[0].ff == 0 and spec.layers[0].ff_kind == "dense"
    assert models.tekosun_from_config(models.tekosun_config(spec), shapes={"l0.mix.w1": (3, 40)}) == spec
    for bad in ({"type": "mlstm"}, {"mlp": {"kind": "dense", "ff": 8}}):
        c = cfg_small()
        c["layers"][1].update(bad)
        with pytest.raises(ValueError):
            models.tekosun_from_config(c)
    c = cfg_small()
    c["layers"][1]["mixer"]["rot"]["dims"] = 12                             # more than the head has
    with pytest.raises(ValueError):
        models.tekosun_from_config(c)


@pytest.mark.parametrize("rot", [ROT, {"base": 100.0, "dims": 4}, {"base": 500000.0, "dims": 32, "scaling": {
    "factor": 16.0, "high": 8.0, "low": 0.5, "original": 512}}])
def test_rotary_frequencies_and_table_match_the_restatement(rot):
    sc = rot.get("scaling") or {}
    spec = models.HalfRotarySpec(rot["dims"], rot["base"], sc.get("factor", 0.0), sc.get("low", 0.0), sc.get("high", 0.0),
                                 sc.get("original", 0))
    f0 = so.rotary_frequencies(rot)
    assert torch.allclose(torch.from_numpy(spec.frequencies()), f0, rtol=1e-12, atol=0)
    if sc:   # all three regimes occur: kept, divided, blended
        plain = float(rot["base"]) ** (-2.0 * torch.arange(rot["dims"] // 2, dtype=torch.float64) / rot["dims"])
        ratio = f0 / plain
        assert float(ratio.max()) == 1.0 and abs(float(ratio.min()) - 1.0 / sc["factor"]) < 1e-12
    tab = spec.table(70)
    half = rot["dims"] // 2
    v = torch.randn(70, 1, rot["dims"] + 3, dtype=torch.float64)
    want = so.rotate_half(v, torch.arange(70), rot)[:, 0]
    a, b = v[:, 0, :half], v[:, 0, half:rot["dims"]]
    c, s = tab[..., 0].double(), tab[..., 1].double()
    assert (a * c - b * s - want[:, :half]).abs().max() < 1e-5
    assert (b * c + a * s - want[:, half:rot["dims"]]).abs().max() < 1e-5
    assert torch.equal(want[:, rot["dims"]:], v[:, 0, rot["dims"]:])        # the rest passes unchanged


def test_merged_layouts_and_packed_weights():
    spec = models.tekosun_from_config(cfg_small(), shapes={"l0.mix.w1": (3, 40)})
    w = models.synth_tekosun_weights(spec, seed=1)
    assert set(w) == set(models.tekosun_tensor_shapes(spec))
    assert w["l1.mix.vmix"].shape == () and "l1.norm2" in w and "l0.norm2" not in w
    pk = models.pack_weights(spec, w, device="cpu", dtype=torch.float32)
    lay, d = spec.mix_layout(0), spec.layers[0].delta                       # [r | k | v | g | a | bottleneck]
    n = d.heads * d.dim
    assert lay.off_k % 8 == 0 and lay.off_up % 8 == 0 and lay.n_in % 8 == 0 and lay.k_out == n
    assert torch.equal(pk["l0.w_in"][lay.off_gate:lay.off_gate + n], w["l0.mix.a"].float())
    assert torch.equal(pk["l0.b_in"][lay.off_gate:lay.off_gate + n], w["l0.mix.a.b"].float())
    assert float(pk["l0.b_in"][:lay.off_gate].abs().sum()) == 0.0
    assert torch.equal(pk["l0.w_in"][lay.off_up:lay.off_up + 3], w["l0.mix.w1"].float())
    assert pk["l0.w2"].shape == (n, 8) and torch.equal(pk["l0.w2"][:, :3], w["l0.mix.w2"].float()) and float(pk["l0.w2"][:, 3:].abs().sum()) == 0.0
    lay, m = spec.mix_layout(2), spec.layers[2].mamba                       # [z | x | B | C | dt]
    t = w["l2.mix.in"].float()
    assert lay.off_g == 0 and lay.off_k == lay.off_v + m.inner and lay.off_q == lay.off_k + m.groups * m.state
    assert torch.equal(pk["l2.w_in"][:m.inner], t[:m.inner])
    assert torch.equal(pk["l2.w_in"][lay.off_v:lay.off_v + m.channels], t[m.inner:m.inner + m.channels])
    assert torch.equal(pk["l2.w_in"][lay.off_gate:lay.off_gate + m.heads], t[m.inner + m.channels:])
    assert pk["l2.conv_w"].shape == (m.channels * m.conv,)
    lay, a = spec.mix_layout(1), spec.layers[1].attn
    assert torch.equal(pk["l1.w_in"][lay.off_v:lay.off_v + a.kv_heads * a.vdim], w["l1.mix.v"].float())
    mo = spec.layers[1].moe
    assert pk["l1.w_exp_in"].shape == (mo.experts, mo.expert_ff, spec.width)
    assert torch.equal(pk["l1.w_exp_out"][2], w["l1.mlp.e2.down"].float())
    assert pk["l1.w_ff_in"].shape == (16, spec.width) and "l2.w_ff_in" not in pk and "l0.ff_post_norm" not in pk
    assert spec.weight_params() > 0


def test_checkpoint_round_trip_through_the_loader(tmp_path):
    spec = models.tekosun_from_config(cfg_small(), shapes={"l0.mix.w1": (5, 40)})
    w = models.synth_tekosun_weights(spec, seed=2)
    models.save_stack_checkpoint(spec, w, str(tmp_path))
    assert loader.is_stack_model(tmp_path)
    spec2, pk = loader.load_model(tmp_path, device="cpu", dtype=torch.float32, max_ctx=99, max_slots=3)
    assert spec2 == spec.with_ctx(99, 3) and spec2.layers[0].delta.rank == 5
    want = models.pack_weights(spec, w, device="cpu", dtype=torch.float32)
    assert set(pk) == set(want) and all(torch.equal(pk[k], want[k]) for k in want)
    (tmp_path / "config.json").write_text((tmp_path / "config.json").read_text().replace('"state": 5', '"state": 6'))
    with pytest.raises(loader.LoaderError):
        loader.load_model(tmp_path, device="cpu", dtype=torch.float32)


def test_restatement_is_causal_and_its_states_are_what_the_equations_say():
    cfg = cfg_small()
    spec = models.tekosun_from_config(cfg)
    w = {k: v.double() for k, v in models.synth_tekosun_weights(spec, seed=3).items()}
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=g).tolist()
    full = so.forward(cfg, w, toks)
    assert (so.forward(cfg, w, toks[:11]) - full[:11]).abs().max() < 1e-9
    # delta rule: removal rate 1 and no decay make the state forget what it held along the unit key before the new pair
    # goes in — after ONE token of a fresh state, o = (k·r) v whatever the rates are
    m = {"heads": 1, "dim": 4}
    W = 6
    ww = {n: torch.randn(4, W, dtype=torch.float64) for n in ("r", "k", "v", "g", "a")}
    ww.update({"a.b": torch.zeros(4, dtype=torch.float64), "w1": torch.randn(2, W, dtype=torch.float64),
               "w2": torch.randn(4, 2, dtype=torch.float64), "w0": torch.zeros(4, dtype=torch.float64),
               "norm": torch.ones(4, dtype=torch.float64), "o": torch.eye(4, dtype=torch.float64)})
    h = torch.randn(1, W, dtype=torch.float64)
    out = so.general_delta(h, m, ww, "", 1e-5)[0]
    r, k, v = ww["r"] @ h[0], ww["k"] @ h[0], ww["v"] @ h[0]
    o = float(k @ r) * v
    want = o / torch.sqrt((o * o).mean() + 1e-5) * torch.sigmoid(ww["g"] @ h[0])
    assert (out - want).abs().max() < 1e-12
    # the decay lies between exp(-exp(-1/2)) and 1
    assert 0.545 < math.exp(-math.exp(-0.5)) < 0.546
    # Mamba-2 with one tap is a plain per-token SiLU in front of the recurrence; a zero step size leaves the state alone
    mm = {"heads": 1, "vdim": 2, "state": 3, "groups": 1, "conv": 1, "norm_groups": 1}
    wm = {"in": torch.randn(2 + 2 + 3 + 3 + 1, W, dtype=torch.float64), "conv": torch.ones(8, 1, dtype=torch.float64),
          "conv.b": torch.zeros(8, dtype=torch.float64), "dt_bias": torch.tensor([-80.0], dtype=torch.float64),
          "A_log": torch.zeros(1, dtype=torch.float64), "D": torch.tensor([2.0], dtype=torch.float64),
          "norm": torch.ones(2, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64)}
    h = torch.randn(5, W, dtype=torch.float64)
    out = so.mamba2(h, mm, wm, "", 1e-5)
    zz = h @ wm["in"].T
    y = 2.0 * torch.nn.functional.silu(zz[:, 2:4]) * torch.nn.functional.silu(zz[:, :2])   # D·x alone: softplus(−80 + ·) ≈ 0
    assert (out - so.unit_rms(y, 1e-5)).abs().max() < 1e-9
    # routing: the chosen weights sum to the scale, and the weight multiplies the expert's OUTPUT
    hh = torch.randn(3, cfg["width"], dtype=torch.float64)
    idx, val = so.route(hh, cfg["layers"][2]["mlp"], w["l2.mlp.router"])
    assert (val.sum(-1) - 1.0).abs().max() < 1e-12
    idx2, val2 = so.route(hh, cfg["layers"][1]["mlp"], w["l1.mlp.router"])
    assert (val2.sum(-1) - 1.5).abs().max() < 1e-12
    one = so.expert(hh[:1], w[f"l2.mlp.e{int(idx[0, 0])}.up"], w[f"l2.mlp.e{int(idx[0, 0])}.down"])
    assert (so.moe(hh, cfg["layers"][2]["mlp"], w, "l2.mlp.")[0] - one[0]).abs().max() < 1e-12
