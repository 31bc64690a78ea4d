"""Prefill and decode throughput of a layer-stack design (Kozusun) beside the closest Llama-family model of equal size.

`python bench.py --stack-compare` prints ONE JSON line: per size, tokens/s of a prompt pass and of greedy decoding (one
sequence and eight), for both engines, with random weights of the real shapes.  "Equal size": same width, head counts,
head size, feed-forward width and vocabulary, and as many Llama layers as the stack model has layer runs, so both read
the same matrices per token (the stack model adds its gate rows, the token table and the loop's mix-in product).

Timing: CUDA events on the launching stream, synchronised on both sides, warm-up first; a buffer larger than L2 is
written between timed iterations.
"""
from __future__ import annotations

import json
from typing import Dict, List

import torch

from . import engine, models

SIZES = {
    # name: width, heads, kv_heads, head size, ff, vocab, layers, (loop start, stop, times), window, kept first, side columns
    "w2048": dict(width=2048, heads=16, kv_heads=8, dim=128, ff=6144, vocab=65536, layers=6, loop=(0, 2, 2),
                  window=1024, keep_first=4, side_dim=64),
    "w3072": dict(width=3072, heads=24, kv_heads=8, dim=128, ff=8192, vocab=65536, layers=6, loop=(0, 2, 2),
                  window=1024, keep_first=4, side_dim=64),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, vocab=32768, layers=3, loop=(0, 1, 2),
                  window=1024, keep_first=4, side_dim=64),
}


def stack_spec(name: str, max_ctx: int, max_slots: int = 8) -> models.StackSpec:
    z = SIZES[name]
    attn = models.AttnSpec(z["heads"], z["kv_heads"], z["dim"], z["dim"], z["dim"] ** -0.5, z["window"], z["keep_first"])
    lo, hi, times = z["loop"]
    return models.StackSpec(name="kozusun-" + name, architecture="Kozusun", width=z["width"], vocab=z["vocab"],
                            layers=tuple(models.StackLayerSpec(attn, z["ff"]) for _ in range(z["layers"])),
                            loop_start=lo, loop_stop=hi, loop_times=times, embed_scale=8.0, residual_mult=0.3,
                            norm_eps=1e-5, norm_offset=1.0, side_dim=z["side_dim"], max_ctx=max_ctx, max_slots=max_slots)


def llama_spec(name: str, n_layers: int, max_ctx: int) -> models.ModelSpec:
    z = SIZES[name]
    return models.ModelSpec("llama-" + name, "llama", z["width"], n_layers, z["heads"], z["kv_heads"], z["dim"], z["ff"],
                            z["vocab"], 5e5, 1e-5, tie=False, max_ctx=max_ctx)


def device_stack_weights(spec: models.StackSpec, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random weights straight in the engine's layout on the device (no host copy of a multi-GB checkpoint)."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(o, i):
        return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * (i ** -0.5)).to(torch.bfloat16)

    def vec(n, centre=0.0):
        return centre + torch.randn(n, generator=g, device=device, dtype=torch.float32) * 0.05

    w = {"embed": mat(spec.vocab, W), "head": mat(spec.vocab, W), "final_norm": vec(W)}
    if spec.loop_times > 0:
        w["mix_in"] = mat(W, 2 * W)
    if spec.side_dim > 0:
        w["side_table"] = mat(spec.vocab, spec.side_dim * len(spec.layers))
    for i, L in enumerate(spec.layers):
        lay, p = spec.layout(i), f"l{i}."
        w[p + "norm"] = vec(W)
        w[p + "w_in"], w[p + "b_in"] = mat(lay.n_in, W), vec(lay.n_in)
        w[p + "w_out"] = mat(W, lay.k_out)
        if spec.side_dim > 0:
            w[p + "side_gate"], w[p + "side_proj"], w[p + "side_norm"] = mat(spec.side_dim, W), mat(W, spec.side_dim), vec(W, 1.0)
    return w


# Silatar sizes: four layers [mLSTM + dense, latent attention + experts, latent attention + dense, mLSTM + experts], the
# middle two run twice (six runs).  The Kozusun model beside it has the same width, vocabulary and number of runs, full
# causal attention of 128-wide heads, and a gated feed-forward of two thirds the dense width (equal parameters).
SILATAR_SIZES = {
    "s2048": dict(width=2048, vocab=65536, heads=16, dim=64, rot_dim=64, vdim=128, kv_rank=512, rec_heads=8, rec_dim=128,
                  rec_vdim=256, ff=8192, experts=32, top=4, expert_ff=1024, shared_ff=1024, koz_heads=16, koz_kv=8, koz_ff=5464),
    "s3072": dict(width=3072, vocab=65536, heads=24, dim=64, rot_dim=64, vdim=128, kv_rank=512, rec_heads=8, rec_dim=192,
                  rec_vdim=384, ff=12288, experts=32, top=4, expert_ff=1536, shared_ff=1536, koz_heads=24, koz_kv=8, koz_ff=8192),
}


def silatar_spec(name: str, max_ctx: int, max_slots: int = 8) -> models.StackSpec:
    z = SILATAR_SIZES[name]
    rot = models.RotarySpec(dims=z["rot_dim"], base=5e5, factor=4.0, original=2048, fast=32.0, slow=1.0)
    lat = models.LatentSpec(z["heads"], z["dim"], z["rot_dim"], z["vdim"], z["kv_rank"], (z["dim"] + z["rot_dim"]) ** -0.5, rot)
    rec = models.MlstmSpec(z["rec_heads"], z["rec_dim"], z["rec_vdim"], 15.0)
    moe = models.MoeSpec(z["experts"], z["top"], z["expert_ff"], 7.0, z["shared_ff"], 7.0)
    L = models.StackLayerSpec
    layers = (L(mixer="mlstm", mlstm=rec, ff_kind="dense", ff=z["ff"], ff_act="gelu_erf"),
              L(mixer="latent_attention", latent=lat, ff_kind="moe", moe=moe),
              L(mixer="latent_attention", latent=lat, ff_kind="dense", ff=z["ff"], ff_act="gelu_erf"),
              L(mixer="mlstm", mlstm=rec, ff_kind="moe", moe=moe))
    return models.StackSpec(name="silatar-" + name, architecture="Silatar", width=z["width"], vocab=z["vocab"], layers=layers,
                            loop_start=1, loop_stop=3, loop_times=2, norm_eps=1e-5, block="sandwich", norm_kind="layer",
                            loop_mix=False, logit_softcap=30.0, max_ctx=max_ctx, max_slots=max_slots)


def kozusun_beside(name: str, n_runs: int, max_ctx: int, max_slots: int = 8) -> models.StackSpec:
    z = SILATAR_SIZES[name]
    attn = models.AttnSpec(z["koz_heads"], z["koz_kv"], 128, 128, 128 ** -0.5, 0, 0)
    return models.StackSpec(name="kozusun-" + name, architecture="Kozusun", width=z["width"], vocab=z["vocab"],
                            layers=tuple(models.StackLayerSpec(attn, z["koz_ff"]) for _ in range(n_runs)), embed_scale=8.0,
                            residual_mult=0.3, norm_eps=1e-5, norm_offset=1.0, side_dim=0, max_ctx=max_ctx, max_slots=max_slots)


def device_silatar_weights(spec: models.StackSpec, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random Silatar weights straight in the engine's layout on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(*shape):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * (shape[-1] ** -0.5)).to(torch.bfloat16)

    def vec(n, centre=1.0):
        return centre + torch.randn(n, generator=g, device=device, dtype=torch.float32) * 0.05

    w = {"embed": mat(spec.vocab, W), "head": mat(spec.vocab, W), "final_norm": vec(W)}
    for i, L in enumerate(spec.layers):
        lay, p = spec.mix_layout(i), f"l{i}."
        w[p + "norm"], w[p + "post_norm"], w[p + "ff_norm"], w[p + "ff_post_norm"] = vec(W), vec(W), vec(W), vec(W)
        w[p + "w_in"], w[p + "b_in"], w[p + "w_out"] = mat(lay.n_in, W), vec(lay.n_in, 0.0), mat(W, lay.k_out)
        if L.mixer == "latent_attention":
            a = L.latent
            w[p + "c_norm"], w[p + "uv"] = vec(a.kv_rank), mat(a.heads * a.vdim, a.kv_rank)
            w[p + "uk"] = mat(a.heads * a.dim, a.kv_rank)
            w[p + "uk_t"] = w[p + "uk"].view(a.heads, a.dim, a.kv_rank).transpose(1, 2).contiguous()
        else:
            w[p + "head_norm"] = vec(L.mlstm.heads * L.mlstm.vdim)
            w[p + "b_in"][lay.off_gate + L.mlstm.heads:lay.off_gate + 2 * L.mlstm.heads] += 3.0   # a memory that keeps
        if L.ff_kind == "moe":
            m = L.moe
            w[p + "router"] = mat(m.experts, W)
            w[p + "w_exp_in"], w[p + "w_exp_out"] = mat(m.experts, 2 * m.expert_ff, W), mat(m.experts, W, m.expert_ff)
            if m.shared_ff > 0:
                w[p + "w_ff_in"], w[p + "w_ff_out"] = mat((2 * m.shared_ff + 1 + 7) // 8 * 8, W), mat(W, m.shared_ff)
        else:
            w[p + "w_ff_in"], w[p + "w_ff_out"] = mat(L.ff, W), mat(W, L.ff)
    return w


def compare_silatar(sizes: List[str], steps: int = 5, warmup: int = 3, prompt_len: int = 2048, n_decode: int = 32) -> dict:
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    timer = _Timer(dev)
    max_ctx = prompt_len + n_decode + 8
    rows = {}
    for name in sizes:
        sspec = silatar_spec(name, max_ctx)
        eng = engine.DecodeEngine(sspec, device_silatar_weights(sspec, dev))
        k = _measure(eng, True, prompt_len, n_decode, timer, steps, warmup, sspec.vocab)
        k["bytes_per_decode_token"] = eng.bytes_per_token(prompt_len)
        k["launches_per_decode_token"] = eng.launches_per_token
        eng.close()
        del eng
        torch.cuda.empty_cache()
        kspec = kozusun_beside(name, len(sspec.runs()), max_ctx)
        eng = engine.DecodeEngine(kspec, device_stack_weights(kspec, dev))
        l = _measure(eng, True, prompt_len, n_decode, timer, steps, warmup, kspec.vocab)
        l["bytes_per_decode_token"] = eng.bytes_per_token(prompt_len)
        l["launches_per_decode_token"] = eng.launches_per_token
        eng.close()
        del eng
        torch.cuda.empty_cache()
        rows[name] = {"silatar": k, "kozusun": l, "ratio": {m: round(k[m] / l[m], 3) for m in k if m.endswith("tok_s")}}
    return {"metric": "silatar_compare", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
            "decode_steps": n_decode, "steps": steps, "warmup": warmup, "l2": "flushed between timed iterations",
            "sizes": rows}


def main_silatar(sizes: str, steps: int, warmup: int) -> None:
    names = [s for s in sizes.split(",") if s] if sizes and sizes != "all" else list(SILATAR_SIZES)
    print(json.dumps(compare_silatar(names, steps=steps, warmup=warmup)), flush=True)


# Tekosun sizes: six layers [delta rule, attention, Mamba-2, delta rule, attention, Mamba-2], every one with routed experts
# (32 experts of the Silatar size, top 4, a shared expert).  The model beside it is the Silatar model of the same width,
# vocabulary and number of layer runs (six): the framework's other design with recurrent mixers, an attention over cached
# rows and routed experts.
TEKOSUN_SIZES = {
    "t2048": dict(width=2048, vocab=65536, heads=16, kv_heads=8, dim=128, window=1024, rot_dims=64, d_heads=16, d_dim=128, rank=64,
                  m_heads=32, m_vdim=64, m_state=128, m_groups=1, conv=4, experts=32, top=4, expert_ff=1024, shared_ff=1024,
                  beside="s2048"),
    "t3072": dict(width=3072, vocab=65536, heads=24, kv_heads=8, dim=128, window=1024, rot_dims=64, d_heads=24, d_dim=128, rank=96,
                  m_heads=48, m_vdim=64, m_state=128, m_groups=1, conv=4, experts=32, top=4, expert_ff=1536, shared_ff=1536,
                  beside="s3072"),
}


def tekosun_spec(name: str, max_ctx: int, max_slots: int = 8) -> models.StackSpec:
    z = TEKOSUN_SIZES[name]
    rot = models.HalfRotarySpec(dims=z["rot_dims"], base=5e5, factor=8.0, low=1.0, high=4.0, original=2048)
    attn = models.AttnSpec(z["heads"], z["kv_heads"], z["dim"], z["dim"], z["dim"] ** -0.5, z["window"], 0, out_gate=False, bias=False)
    prep = models.AttnPrepSpec(qk_norm=True, rot=rot, v_norm=True, v_mix=True)
    moe = models.MoeSpec(z["experts"], z["top"], z["expert_ff"], shared_ff=z["shared_ff"], router="softmax", weight_output=True,
                         route_scale=2.0, act="relu2", shared_plain=True)
    L = models.StackLayerSpec
    kw = dict(ff_kind="moe", moe=moe, ff_act="relu2")
    d = L(mixer="general_delta", delta=models.DeltaSpec(z["d_heads"], z["d_dim"], z["rank"]), **kw)
    a = L(mixer="attention", attn=attn, prep=prep, **kw)
    m = L(mixer="mamba2", mamba=models.Mamba2Spec(z["m_heads"], z["m_vdim"], z["m_state"], z["m_groups"], z["conv"], 1), **kw)
    return models.StackSpec(name="tekosun-" + name, architecture="Tekosun", width=z["width"], vocab=z["vocab"],
                            layers=(d, a, m, d, a, m), embed_scale=8.0, norm_eps=1e-5, block="postnorm", norm_kind="rms",
                            loop_mix=False, max_ctx=max_ctx, max_slots=max_slots)


def device_tekosun_weights(spec: models.StackSpec, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random Tekosun weights straight in the engine's layout on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(*shape):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * (shape[-1] ** -0.5)).to(torch.bfloat16)

    def vec(n, centre=1.0, spread=0.05):
        return centre + torch.randn(n, generator=g, device=device, dtype=torch.float32) * spread

    w = {"embed": mat(spec.vocab, W), "head": mat(spec.vocab, W), "final_norm": vec(W)}
    for i, L in enumerate(spec.layers):
        lay, p = spec.mix_layout(i), f"l{i}."
        w[p + "post_norm"], w[p + "ff_post_norm"] = vec(W), vec(W)
        w[p + "w_in"], w[p + "b_in"], w[p + "w_out"] = mat(lay.n_in, W), vec(lay.n_in, 0.0), mat(W, lay.k_out)
        if L.mixer == "attention":
            a = L.attn
            w[p + "q_norm"], w[p + "k_norm"], w[p + "vmix"] = vec(a.heads * a.dim), vec(a.kv_heads * a.dim), vec(1, 0.4)
        elif L.mixer == "general_delta":
            a = L.delta
            w[p + "w2"], w[p + "w0"] = mat(a.heads * a.dim, (a.rank + 7) // 8 * 8), vec(a.heads * a.dim, 0.0, 1.0)
            w[p + "head_norm"] = vec(a.heads * a.dim)
        else:
            a = L.mamba
            w[p + "conv_w"], w[p + "conv_b"] = vec(a.channels * a.conv, 0.0, 0.4), vec(a.channels, 0.0, 0.2)
            w[p + "dt_bias"], w[p + "A_log"], w[p + "D"] = vec(a.heads, -1.0, 0.5), vec(a.heads, 0.0, 0.5), vec(a.heads)
            w[p + "mix_norm"] = vec(a.inner)
        m = L.moe
        w[p + "router"] = mat(m.experts, W)
        w[p + "w_exp_in"], w[p + "w_exp_out"] = mat(m.experts, m.expert_ff, W), mat(m.experts, W, m.expert_ff)
        w[p + "w_ff_in"], w[p + "w_ff_out"] = mat((m.shared_ff + 7) // 8 * 8, W), mat(W, m.shared_ff)
    return w


def compare_tekosun(sizes: List[str], steps: int = 5, warmup: int = 3, prompt_len: int = 2048, n_decode: int = 32) -> dict:
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    timer = _Timer(dev)
    max_ctx = prompt_len + n_decode + 8
    rows = {}
    for name in sizes:
        def one(spec, weights):
            eng = engine.DecodeEngine(spec, weights)
            k = _measure(eng, True, prompt_len, n_decode, timer, steps, warmup, spec.vocab)
            k["bytes_per_decode_token"] = eng.bytes_per_token(prompt_len)
            k["launches_per_decode_token"] = eng.launches_per_token
            k["matrix_params_per_token"] = spec.weight_params()
            eng.close()
            del eng
            torch.cuda.empty_cache()
            return k
        tspec = tekosun_spec(name, max_ctx)
        k = one(tspec, device_tekosun_weights(tspec, dev))
        sspec = silatar_spec(TEKOSUN_SIZES[name]["beside"], max_ctx)
        l = one(sspec, device_silatar_weights(sspec, dev))
        rows[name] = {"tekosun": k, "silatar": l, "ratio": {m: round(k[m] / l[m], 3) for m in k if m.endswith("tok_s")}}
    return {"metric": "tekosun_compare", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
            "decode_steps": n_decode, "steps": steps, "warmup": warmup, "l2": "flushed between timed iterations",
            "sizes": rows}


def main_tekosun(sizes: str, steps: int, warmup: int) -> None:
    names = [s for s in sizes.split(",") if s] if sizes and sizes != "all" else list(TEKOSUN_SIZES)
    print(json.dumps(compare_tekosun(names, steps=steps, warmup=warmup)), flush=True)


# Tarudra sizes: eight layers [latent, latent, gated delta rule, attention, latent, latent, gated delta rule, attention reading
# the first attention layer's keys and values], every one with a dense squared-ReLU feed-forward.  The model beside it is
# the Silatar design — the framework's other sandwich-block design with layer norms, a latent attention, a recurrent mixer and
# capped logits — with dense feed-forwards of the same width, the same latent sizes in every attention place and its mLSTM (a
# matrix memory of the same number of floats as the delta rule's) in the recurrent places.
TARUDRA_SIZES = {
    "r2048": dict(width=2048, vocab=65536, heads=16, kv_heads=8, dim=128, window=1024, rot_dims=64, l_heads=16, l_dim=64, l_rot=64,
                  l_vdim=128, kv_rank=512, q_rank=768, d_heads=16, d_kv=8, d_dim=128, d_vdim=128, conv=4, ff=8192,
                  rec_heads=8, rec_dim=128, rec_vdim=256),
    "r3072": dict(width=3072, vocab=65536, heads=24, kv_heads=8, dim=128, window=1024, rot_dims=64, l_heads=24, l_dim=64, l_rot=64,
                  l_vdim=128, kv_rank=512, q_rank=1536, d_heads=24, d_kv=8, d_dim=128, d_vdim=128, conv=4, ff=12288,
                  rec_heads=8, rec_dim=192, rec_vdim=384),
}


def tarudra_spec(name: str, max_ctx: int, max_slots: int = 8) -> models.StackSpec:
    z = TARUDRA_SIZES[name]
    yarn = models.RotarySpec(dims=z["rot_dims"], base=1e4, factor=2.0, original=1024, fast=32.0, slow=1.0)
    attn = models.AttnSpec(z["heads"], z["kv_heads"], z["dim"], z["dim"], z["dim"] ** -0.5, z["window"], 0, out_gate=False, bias=True,
                           sink=True, out_bias=True)
    prep = models.AttnPrepSpec(rot=yarn, rot_interleaved=True)
    lat = models.LatentSpec(z["l_heads"], z["l_dim"], z["l_rot"], z["l_vdim"], z["kv_rank"], (z["l_dim"] + z["l_rot"]) ** -0.5,
                            models.RotarySpec(dims=z["l_rot"], base=5e5), rot_layout="half", q_rank=z["q_rank"], window=z["window"],
                            out_gate=True)
    gd = models.GatedDeltaSpec(z["d_heads"], z["d_kv"], z["d_dim"], z["d_vdim"], z["conv"])
    L = models.StackLayerSpec
    kw = dict(ff_kind="dense", ff=z["ff"], ff_act="relu2")
    l, d = L(mixer="latent_attention", latent=lat, **kw), L(mixer="gated_delta", gdelta=gd, **kw)
    a, a2 = L(mixer="attention", attn=attn, prep=prep, **kw), L(mixer="attention", attn=attn, prep=prep, kv_from=3, **kw)
    return models.StackSpec(name="tarudra-" + name, architecture="Tarudra", width=z["width"], vocab=z["vocab"],
                            layers=(l, l, d, a, l, l, d, a2), norm_eps=1e-6, block="sandwich", norm_kind="layer", loop_mix=False,
                            logit_softcap=15.0, layer_scale=True, max_ctx=max_ctx, max_slots=max_slots)


def silatar_dense_beside(name: str, max_ctx: int, max_slots: int = 8) -> models.StackSpec:
    z = TARUDRA_SIZES[name]
    rot = models.RotarySpec(dims=z["l_rot"], base=5e5, factor=4.0, original=2048, fast=32.0, slow=1.0)
    lat = models.LatentSpec(z["l_heads"], z["l_dim"], z["l_rot"], z["l_vdim"], z["kv_rank"], (z["l_dim"] + z["l_rot"]) ** -0.5, rot)
    rec = models.MlstmSpec(z["rec_heads"], z["rec_dim"], z["rec_vdim"], 15.0)
    L = models.StackLayerSpec
    kw = dict(ff_kind="dense", ff=z["ff"], ff_act="gelu_erf")
    l, r = L(mixer="latent_attention", latent=lat, **kw), L(mixer="mlstm", mlstm=rec, **kw)
    return models.StackSpec(name="silatar-dense-" + name, architecture="Silatar", width=z["width"], vocab=z["vocab"],
                            layers=(l, l, r, l, l, l, r, l), norm_eps=1e-5, block="sandwich", norm_kind="layer", loop_mix=False,
                            logit_softcap=30.0, max_ctx=max_ctx, max_slots=max_slots)


def device_tarudra_weights(spec: models.StackSpec, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random Tarudra weights straight in the engine's layout on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(*shape):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * (shape[-1] ** -0.5)).to(torch.bfloat16)

    def vec(n, centre=1.0, spread=0.05):
        return centre + torch.randn(n, generator=g, device=device, dtype=torch.float32) * spread

    w = {"embed": mat(spec.vocab, W), "head": mat(spec.vocab, W), "final_norm": vec(W)}
    for i, L in enumerate(spec.layers):
        lay, p = spec.mix_layout(i), f"l{i}."
        w[p + "norm"], w[p + "post_norm"], w[p + "ff_norm"], w[p + "ff_post_norm"] = vec(W), vec(W, 0.6), vec(W), vec(W, 0.6)
        w[p + "w_in"], w[p + "w_out"] = mat(lay.n_in, W), mat(W, lay.k_out)
        if L.mixer == "attention":
            w[p + "b_in"], w[p + "b_out"] = vec(lay.n_in, 0.0, 0.2), vec(W, 0.0, 0.2)
        elif L.mixer == "latent_attention":
            a = L.latent
            w[p + "c_norm"], w[p + "q_norm"] = vec(a.kv_rank), vec(a.q_rank)
            w[p + "uq"] = mat(a.heads * (a.dim + a.rot_dim), (a.q_rank + 7) // 8 * 8)
            w[p + "uk"], w[p + "uv"] = mat(a.heads * a.dim, a.kv_rank), mat(a.heads * a.vdim, a.kv_rank)
            w[p + "uk_t"] = w[p + "uk"].view(a.heads, a.dim, a.kv_rank).transpose(1, 2).contiguous()
        else:
            a = L.gdelta
            w[p + "conv_w"] = vec(a.channels * a.conv, 0.0, 0.4)
            w[p + "A_log"], w[p + "dt_bias"], w[p + "head_norm"] = vec(a.heads, 0.0, 0.5), vec(a.heads, -1.0, 0.5), vec(a.vdim)
        w[p + "w_ff_in"], w[p + "w_ff_out"] = mat(L.ff, W), mat(W, L.ff)
    return w


def compare_tarudra(sizes: List[str], steps: int = 5, warmup: int = 3, prompt_len: int = 2048, n_decode: int = 32) -> dict:
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    timer = _Timer(dev)
    max_ctx = prompt_len + n_decode + 8
    rows = {}
    for name in sizes:
        def one(spec, weights):
            eng = engine.DecodeEngine(spec, weights)
            k = _measure(eng, True, prompt_len, n_decode, timer, steps, warmup, spec.vocab)
            k["bytes_per_decode_token"] = eng.bytes_per_token(prompt_len)
            k["launches_per_decode_token"] = eng.launches_per_token
            k["matrix_params_per_token"] = spec.weight_params()
            eng.close()
            del eng
            torch.cuda.empty_cache()
            return k
        tspec = tarudra_spec(name, max_ctx)
        k = one(tspec, device_tarudra_weights(tspec, dev))
        sspec = silatar_dense_beside(name, max_ctx)
        l = one(sspec, device_silatar_weights(sspec, dev))
        rows[name] = {"tarudra": k, "silatar_dense": l, "ratio": {m: round(k[m] / l[m], 3) for m in k if m.endswith("tok_s")}}
    return {"metric": "tarudra_compare", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
            "decode_steps": n_decode, "steps": steps, "warmup": warmup, "l2": "flushed between timed iterations",
            "sizes": rows}


def main_tarudra(sizes: str, steps: int, warmup: int) -> None:
    names = [s for s in sizes.split(",") if s] if sizes and sizes != "all" else list(TARUDRA_SIZES)
    print(json.dumps(compare_tarudra(names, steps=steps, warmup=warmup)), flush=True)


class _Timer:
    def __init__(self, device):
        self.device = device
        self.flush = torch.empty(160 << 20, dtype=torch.uint8, device=device)   # larger than the 126 MB L2

    def run(self, fn, prepare, steps: int, warmup: int) -> float:
        """Median milliseconds of fn() over `steps` runs after `warmup` runs; prepare() and an L2 flush before each."""
        times = []
        for i in range(warmup + steps):
            prepare()
            self.flush.fill_(i & 0xff)
            torch.cuda.synchronize(self.device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(self.device)
            if i >= warmup:
                times.append(a.elapsed_time(b))
        times.sort()
        return times[len(times) // 2]


def _measure(eng, is_stack: bool, prompt_len: int, n_decode: int, timer: _Timer, steps: int, warmup: int, vocab: int) -> dict:
    dev = eng.device
    g = torch.Generator().manual_seed(1)
    out = {}
    for B in (1, 8):
        ids = torch.randint(0, vocab, (B, prompt_len), generator=g).to(dev)

        def prefill():
            eng.gen_next_token(ids)

        ms = timer.run(prefill, eng.reset_cache, steps, warmup)
        out[f"prefill_b{B}_tok_s"] = round(B * prompt_len / ms * 1e3, 1)
        out[f"prefill_b{B}_ms"] = round(ms, 3)

        def prep():
            eng.reset_cache()
            eng.gen_next_token(ids)

        ms = timer.run(lambda: eng.decode(n_decode), prep, steps, warmup)
        out[f"decode_b{B}_tok_s"] = round(B * n_decode / ms * 1e3, 1)
        out[f"decode_b{B}_us_per_step"] = round(ms / n_decode * 1e3, 1)
    return out


def compare(sizes: List[str], steps: int = 5, warmup: int = 3, prompt_len: int = 2048, n_decode: int = 32) -> dict:
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    timer = _Timer(dev)
    max_ctx = prompt_len + n_decode + 8
    rows = {}
    for name in sizes:
        sspec = stack_spec(name, max_ctx)
        eng = engine.DecodeEngine(sspec, device_stack_weights(sspec, dev))
        k = _measure(eng, True, prompt_len, n_decode, timer, steps, warmup, sspec.vocab)
        k["bytes_per_decode_token"] = eng.bytes_per_token(prompt_len)
        eng.close()
        del eng
        torch.cuda.empty_cache()
        lspec = llama_spec(name, len(sspec.runs()), max_ctx)
        eng = engine.DecodeEngine(lspec, models.synth_weights(lspec, seed=0, device=str(dev), device_generator=True))
        l = _measure(eng, False, prompt_len, n_decode, timer, steps, warmup, lspec.vocab)
        l["bytes_per_decode_token"] = eng.bytes_per_token(prompt_len)
        eng.close()
        del eng
        torch.cuda.empty_cache()
        rows[name] = {"kozusun": k, "llama_family": l,
                      "ratio": {m: round(k[m] / l[m], 3) for m in k if m.endswith("tok_s")}}
    return {"metric": "stack_compare", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
            "decode_steps": n_decode, "steps": steps, "warmup": warmup, "l2": "flushed between timed iterations",
            "sizes": rows}


def main(sizes: str, steps: int, warmup: int) -> None:
    names = [s for s in sizes.split(",") if s] if sizes and sizes != "all" else list(SIZES)
    print(json.dumps(compare(names, steps=steps, warmup=warmup)), flush=True)
