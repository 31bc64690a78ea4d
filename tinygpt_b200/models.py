"""Model constants and synthetic checkpoints for the decode path.

Mirrors what the reference derives from config.json (src/huggingface/ModelConfig.cpp:73-122) and the weight-name /
merged-weight layout of its model classes (src/model/GPTModel.h:43-48, src/layer/Attention.h:61-68,
src/layer/GatedMLP.h:44-50, src/layer/Linear.h:64-79).  No weights are available offline, so checkpoints are seeded
synthetic tensors of the real shapes.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch


@dataclass(frozen=True)
class RopeScaling:
    factor: float
    high_freq_factor: float
    low_freq_factor: float
    original_context_length: int


@dataclass(frozen=True)
class ModelSpec:
    name: str
    model_type: str          # llama | qwen2 | qwen3 | mistral  (src/huggingface/ModelLoader.cpp:50-68)
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float
    rms_eps: float
    tie: bool = True
    qkv_bias: bool = False   # Qwen2 (src/model/ModelQwen2.h:26-31)
    qk_norm: bool = False    # Qwen3 (src/model/ModelQwen3.h:28-31)
    max_ctx: int = 4096      # rows of the RoPE table / KV-cache capacity used here
    rope_scaling: Optional[RopeScaling] = None

    @property
    def q_dim(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def per_layer_params(self) -> int:
        return (self.q_dim + 2 * self.kv_dim) * self.hidden + self.q_dim * self.hidden + 3 * self.intermediate * self.hidden

    @property
    def weight_params(self) -> int:
        """Matrix parameters one decode step reads (tied lm_head counted once) — SURVEY.md §8a table."""
        return self.layers * self.per_layer_params + self.vocab * self.hidden

    def bytes_per_token(self, ctx: int = 0) -> int:
        """Algorithmic HBM bytes per decoded token: weights once + K/V rows read + new K/V row written."""
        return 2 * self.weight_params + 4 * self.layers * self.kv_dim * ctx + 4 * self.layers * self.kv_dim

    def with_ctx(self, max_ctx: int) -> "ModelSpec":
        return replace(self, max_ctx=max_ctx)


# The BASELINE.json configurations (standard HF configs; table in SURVEY.md §8).
QWEN25_05B = ModelSpec("Qwen2.5-0.5B", "qwen2", 896, 24, 14, 2, 64, 4864, 151936, 1e6, 1e-6, tie=True, qkv_bias=True)
LLAMA32_3B = ModelSpec("Llama-3.2-3B", "llama", 3072, 28, 24, 8, 128, 8192, 128256, 5e5, 1e-5, tie=True,
                       rope_scaling=RopeScaling(32.0, 4.0, 1.0, 8192))
QWEN3_17B = ModelSpec("Qwen3-1.7B", "qwen3", 2048, 28, 16, 8, 128, 6144, 151936, 1e6, 1e-6, tie=True, qk_norm=True)
MISTRAL_7B = ModelSpec("Mistral-7B-v0.3", "mistral", 4096, 32, 32, 8, 128, 14336, 32768, 1e6, 1e-5, tie=False)

# Small shapes for CPU-oracle parity (same code paths: bias / qk-norm / llama3 scaling / GQA group sizes 7,3,2,4).
# Llama, Qwen2 and Mistral derive head_dim = hidden / heads in the reference (src/model/ModelQwen2.h:20,
# ModelLlama.h:37), so hidden = q_heads * head_dim there; Qwen3 carries an explicit head_dim.
TINY_QWEN2 = ModelSpec("tiny-qwen2", "qwen2", 896, 2, 14, 2, 64, 256, 512, 1e6, 1e-6, tie=True, qkv_bias=True,
                       max_ctx=256)
TINY_LLAMA = ModelSpec("tiny-llama", "llama", 768, 2, 6, 2, 128, 512, 640, 5e5, 1e-5, tie=True, max_ctx=256,
                       rope_scaling=RopeScaling(32.0, 4.0, 1.0, 64))
TINY_QWEN3 = ModelSpec("tiny-qwen3", "qwen3", 192, 2, 4, 2, 128, 320, 384, 1e6, 1e-6, tie=True, qk_norm=True,
                       max_ctx=256)
TINY_MISTRAL = ModelSpec("tiny-mistral", "mistral", 1024, 2, 8, 2, 128, 448, 512, 1e6, 1e-5, tie=False, max_ctx=256)

# 8 KV heads: attention heads shard over 2, 4 and 8 tensor-parallel ranks (the other tiny shapes have 2 KV heads)
TINY_TP8 = ModelSpec("tiny-tp8", "mistral", 1024, 2, 8, 8, 128, 512, 1024, 1e6, 1e-5, tie=False, max_ctx=256)

SPECS: Dict[str, ModelSpec] = {s.name: s for s in
                               (QWEN25_05B, LLAMA32_3B, QWEN3_17B, MISTRAL_7B, TINY_QWEN2, TINY_LLAMA, TINY_QWEN3,
                                TINY_MISTRAL, TINY_TP8)}


def synth_weights(spec: ModelSpec, seed: int = 0, device: str = "cpu", std: float = 0.02,
                  device_generator: bool = False) -> Dict[str, torch.Tensor]:
    """Seeded synthetic checkpoint in bf16 with the reference's state names.

    Matrices N(0, std); norm weights 1 + N(0, std) (so the fp32 weight multiply inside RMSNorm is exercised); qkv bias
    N(0, std).  q/k/v and gate/up are stored MERGED ("…qkv_proj.weight", "…gate_up_proj.weight": rows [q|k|v],
    [gate|up]) exactly as the reference's MergedLinear holds them; `split_views()` exposes the HF-named slices.
    Generation is per tensor from a CPU generator so that the same seed gives the same checkpoint on every machine
    (what the oracle-parity tests need).  `device_generator=True` draws on `device` instead (Philox, seconds instead of
    minutes for 7B parameters; identical on every GPU of the same type, which is what tensor-parallel ranks need).
    """
    gen_dev = device if device_generator else "cpu"
    g = torch.Generator(device=gen_dev).manual_seed(seed)

    def mat(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32, device=gen_dev) * std).to(torch.bfloat16).to(device)

    def norm(n):
        return (1.0 + torch.randn(n, generator=g, dtype=torch.float32, device=gen_dev) * std).to(torch.bfloat16).to(device)

    w: Dict[str, torch.Tensor] = {}
    w["model.embed_tokens.weight"] = mat(spec.vocab, spec.hidden)
    for l in range(spec.layers):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = norm(spec.hidden)
        w[p + "self_attn.qkv_proj.weight"] = mat(spec.q_dim + 2 * spec.kv_dim, spec.hidden)
        if spec.qkv_bias:
            w[p + "self_attn.qkv_proj.bias"] = mat(spec.q_dim + 2 * spec.kv_dim)
        if spec.qk_norm:
            w[p + "self_attn.q_norm.weight"] = norm(spec.head_dim)
            w[p + "self_attn.k_norm.weight"] = norm(spec.head_dim)
        w[p + "self_attn.o_proj.weight"] = mat(spec.hidden, spec.q_dim)
        w[p + "post_attention_layernorm.weight"] = norm(spec.hidden)
        w[p + "mlp.gate_up_proj.weight"] = mat(2 * spec.intermediate, spec.hidden)
        w[p + "mlp.down_proj.weight"] = mat(spec.hidden, spec.intermediate)
    w["model.norm.weight"] = norm(spec.hidden)
    if not spec.tie:
        w["lm_head.weight"] = mat(spec.vocab, spec.hidden)
    return w


def split_views(spec: ModelSpec, w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """HF-named state dict (q_proj/k_proj/v_proj, gate_proj/up_proj as dim-0 views of the merged tensors)."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in w.items():
        if k.endswith("self_attn.qkv_proj.weight") or k.endswith("self_attn.qkv_proj.bias"):
            base, kind = k.rsplit("qkv_proj.", 1)
            q, kk, vv = v.split([spec.q_dim, spec.kv_dim, spec.kv_dim], dim=0)
            out[base + "q_proj." + kind], out[base + "k_proj." + kind], out[base + "v_proj." + kind] = q, kk, vv
        elif k.endswith("mlp.gate_up_proj.weight"):
            base = k[: -len("gate_up_proj.weight")]
            gt, up = v.split([spec.intermediate, spec.intermediate], dim=0)
            out[base + "gate_proj.weight"], out[base + "up_proj.weight"] = gt, up
        else:
            out[k] = v
    return out


def rope_table(spec: ModelSpec) -> torch.Tensor:
    """fp32 cos/sin table [max_ctx, head_dim, 2] computed on the host exactly like the reference's ropeInit formulae
    (TT/Operation/OpNNLayerCuda.cuh:359-410): invFreq = 1/powf(θ, 2i/hd) (+ llama3 scaling), angle = pos·invFreq,
    (cosf, sinf) duplicated for both halves.  In a TinyGPT integration the engine is handed the reference's own table
    (RoPE::cache(), TT/Module/Basic.cpp:111) instead."""
    hd, half = spec.head_dim, spec.head_dim // 2
    i = np.arange(half, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(spec.rope_theta), (i * np.float32(2.0)) / np.float32(hd),
                                      dtype=np.float32)).astype(np.float32)
    sc = spec.rope_scaling
    if sc is not None:
        orig = np.float32(sc.original_context_length)
        low_wave, high_wave = orig / np.float32(sc.low_freq_factor), orig / np.float32(sc.high_freq_factor)
        wave = np.float32(2.0) * np.float32(np.pi) / inv
        smooth = (orig / wave - np.float32(sc.low_freq_factor)) / (np.float32(sc.high_freq_factor) -
                                                                   np.float32(sc.low_freq_factor))
        scaled = inv / np.float32(sc.factor)
        mid = ((np.float32(1.0) - smooth) * scaled + smooth * inv).astype(np.float32)
        inv = np.where(wave > low_wave, scaled, np.where(wave < high_wave, inv, mid)).astype(np.float32)
    ang = (np.arange(spec.max_ctx, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    c, s = np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)
    tab = np.empty((spec.max_ctx, hd, 2), dtype=np.float32)
    tab[:, :half, 0], tab[:, :half, 1], tab[:, half:, 0], tab[:, half:, 1] = c, s, c, s
    return torch.from_numpy(tab)


# ------------------------------------------------------------------------------------------------ layer-stack models
# Models whose wiring is data: a list of layers (attention mixer + optional gated feed-forward + optional token-table
# side input), optionally with a looped span.  The engine runs them through b200_engine_create_stack; what follows is
# the host-side description, the registry that picks a description from config.json, and the weight layout.
@dataclass(frozen=True)
class AttnSpec:
    heads: int
    kv_heads: int
    dim: int                 # per-head query/key size
    vdim: int                # per-head value size
    scale: float             # score = (q·k)·scale
    window: int = 0          # key j visible from i when j <= i and i - j < window; 0 = every earlier key
    keep_first: int = 0      # keys j < keep_first stay visible whatever the window
    out_gate: bool = True    # head output × sigmoid(gate logit)
    bias: bool = True        # q/k/v projections carry a bias
    sink: bool = False       # the softmax's denominator gains 1 (a sink of score 0 that has no value)
    out_bias: bool = False   # the out-projection carries a bias (sandwich blocks)

    def visible(self, i: int, j: int) -> bool:
        return j <= i and (self.window <= 0 or i - j < self.window or j < self.keep_first)


@dataclass(frozen=True)
class RotarySpec:
    """Rotary positions on the first `dims` entries of a vector, pair (2i, 2i+1) turned by p·f_i at position p
    (interleaved layout), f_i = base^(-2i/dims).  factor > 0: YaRN stretching — pairs that turn fewer than `slow` times
    over `original` positions have their frequency divided by `factor`, pairs that turn more than `fast` times keep it,
    a linear ramp over the pair index in between; cos and sin are scaled by 0.1·ln(factor) + 1."""
    dims: int
    base: float
    factor: float = 0.0
    original: int = 0
    fast: float = 0.0
    slow: float = 0.0

    def frequencies(self) -> Tuple[np.ndarray, float]:
        """→ (angular frequency per pair [dims/2] in float64, magnitude of cos / sin)."""
        i = np.arange(self.dims // 2, dtype=np.float64)
        f = np.power(float(self.base), -2.0 * i / max(self.dims, 1))
        if self.factor <= 0:
            return f, 1.0

        def pair_of(turns: float) -> float:   # the (fractional) pair index that makes `turns` turns over `original` positions
            return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo = max(math.floor(pair_of(self.fast)), 0)
        hi = min(math.ceil(pair_of(self.slow)), self.dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp), 0.1 * math.log(self.factor) + 1.0

    def table(self, max_ctx: int) -> torch.Tensor:
        """fp32 [max_ctx, dims/2, 2]: {cos, sin}(p·f_i)·magnitude, angles taken in float64."""
        f, mag = self.frequencies()
        ang = np.arange(max_ctx, dtype=np.float64)[:, None] * f[None, :]
        return torch.from_numpy(np.stack([np.cos(ang) * mag, np.sin(ang) * mag], axis=-1).astype(np.float32))


@dataclass(frozen=True)
class LatentSpec:
    """Latent attention: per head `dim` plain + `rot_dim` rotated query/key entries and `vdim` value entries; keys and
    values are expanded from a cached latent of `kv_rank` entries, one rotated key part is shared by all heads."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotarySpec
    rot_layout: str = "interleaved"   # interleaved: pairs (2i, 2i+1) | half: pairs (i, i + dims/2)
    q_rank: int = 0          # > 0: queries go through an RMS-normed latent of this size (down- and up-projection)
    window: int = 0          # key j visible from i when j <= i and i - j < window; 0 = every earlier key
    out_gate: bool = False   # concatenated head outputs × sigmoid(gate projection of the layer input)


@dataclass(frozen=True)
class MlstmSpec:
    """mLSTM matrix memory: per head keys / queries of `dim`, values of `vdim`; gate logits capped at ±gate_cap."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class MoeSpec:
    """Routed experts: `top` of `experts` per token.  router "sigmoid": the weight is the chosen expert's sigmoid score;
    "softmax": scores are a softmax over all experts and the chosen ones are divided by their sum (+ 1e-20) and multiplied by
    route_scale.  The weight multiplies the expert's input, or (weight_output) its output.  act "glu_clamp": clamped gated
    experts of width expert_ff (clamp `limit`); "relu2": down·relu(up·h)², no gate rows.  shared_ff > 0: a shared expert of
    that width (clamp shared_limit) behind a per-token sigmoid gate, or (shared_plain) added as it is."""
    experts: int
    top: int
    expert_ff: int
    limit: float = 0.0
    shared_ff: int = 0
    shared_limit: float = 0.0
    router: str = "sigmoid"
    weight_output: bool = False
    route_scale: float = 1.0
    act: str = "glu_clamp"
    shared_plain: bool = False


@dataclass(frozen=True)
class HalfRotarySpec:
    """Rotary positions on the first `dims` entries of every head, entry i paired with entry i + dims/2 (rotate-half
    layout), pair i turned by p·f_i at position p, f_i = base^(-2i/dims).  factor > 0: Llama-3.1 frequency scaling — with
    the wavelength l = 2π/f, f is kept where l < original/high, divided by factor where l > original/low, and blended
    linearly in original/l between the two."""
    dims: int
    base: float
    factor: float = 0.0
    low: float = 0.0
    high: float = 0.0
    original: int = 0

    def frequencies(self) -> np.ndarray:
        i = np.arange(self.dims // 2, dtype=np.float64)
        f = np.power(float(self.base), -2.0 * i / max(self.dims, 1))
        if self.factor <= 0:
            return f
        wave = 2.0 * np.pi / f
        blend = (self.original / wave - self.low) / (self.high - self.low)
        mid = (1.0 - blend) * f / self.factor + blend * f
        return np.where(wave < self.original / self.high, f, np.where(wave > self.original / self.low, f / self.factor, mid))

    def table(self, max_ctx: int) -> torch.Tensor:
        """fp32 [max_ctx, dims/2, 2]: {cos, sin}(p·f_i), angles taken in float64."""
        ang = np.arange(max_ctx, dtype=np.float64)[:, None] * self.frequencies()[None, :]
        return torch.from_numpy(np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32))


@dataclass(frozen=True)
class AttnPrepSpec:
    """What happens to q | k | v between the in-projection and the cache: an RMS norm with a weight over the WHOLE query
    and key projections, rotary positions, every value head divided by its root mean square, and the value mix-in (the
    first such layer of the model keeps its values, the later ones blend theirs with them by a learned weight)."""
    qk_norm: bool = False
    rot: Optional[object] = None   # HalfRotarySpec (pairs i, i + dims/2), or a RotarySpec with rot_interleaved
    v_norm: bool = False
    v_mix: bool = False
    rot_interleaved: bool = False  # pairs (2i, 2i+1)


@dataclass(frozen=True)
class DeltaSpec:
    """Generalized delta rule: per head a dim × dim state, per-channel decay exp(−decay_scale·sigmoid(·)) from a low-rank
    (`rank`) tanh bottleneck, per-channel removal rate along the unit key k / sqrt(Σk² + unit_eps)."""
    heads: int
    dim: int
    rank: int
    decay_scale: float = math.exp(-0.5)
    unit_eps: float = 1e-6


@dataclass(frozen=True)
class Mamba2Spec:
    """Mamba-2: `heads` heads of `vdim` channels, a state of `state` entries per channel, B and C shared by heads/groups
    heads, a causal convolution of `conv` taps over x | B | C, the gated output RMS-normed in `norm_groups` equal parts."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int = 1

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule: `heads` value heads of `vdim`, `kv_heads` query / key heads of `dim` (value head h reads query / key
    head h // (heads // kv_heads)); q, k, v pass causal convolutions of `conv` taps and SiLU; one decay and one write strength
    per head; the state is a dim × vdim matrix per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    unit_eps: float = 1e-6

    @property
    def channels(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim


@dataclass(frozen=True)
class StackLayerSpec:
    attn: Optional[AttnSpec] = None  # mixer "attention"
    ff: int = 0                      # feed-forward width (gated / dense), 0 = none
    ff_act: str = "gelu_tanh"        # gelu_tanh | silu | gelu_erf
    mixer: str = "attention"         # attention | latent_attention | mlstm | general_delta | mamba2 | gated_delta
    latent: Optional[LatentSpec] = None
    mlstm: Optional[MlstmSpec] = None
    ff_kind: str = "gated"           # gated | dense | moe
    moe: Optional[MoeSpec] = None
    prep: Optional[AttnPrepSpec] = None   # attention mixers of sandwich / post-norm blocks
    delta: Optional[DeltaSpec] = None
    mamba: Optional[Mamba2Spec] = None
    gdelta: Optional[GatedDeltaSpec] = None
    kv_from: Optional[int] = None    # attention mixers: read the keys and values layer kv_from cached (no projections of its own)


@dataclass(frozen=True)
class MixLayout:
    """Rows of the merged in-projection of a sandwich or post-norm block's mixer (segments on multiples of 8, zero padding).
    latent attention: [q | down];  mLSTM: [q | k | v | out-gate logits | input-gate, forget-gate logits];  attention:
    [q | k | v];  generalized delta rule: [r | k | v | out-gate logits | removal logits | decay bottleneck] (the last at
    off_up);  Mamba-2: [z | x | B | C | dt] with z at off_g, x at off_v, B at off_k, C at off_q (x | B | C contiguous), dt at
    off_gate."""
    off_q: int = 0
    off_k: int = 0
    off_v: int = 0
    off_g: int = 0
    off_gate: int = 0
    n_in: int = 0
    k_out: int = 0
    off_up: int = 0


@dataclass(frozen=True)
class StackLayout:
    """Rows of the merged in-projection and columns of the merged out-projection of one layer (segments start on
    multiples of 8 so that vector loads and the tensor-core paths see aligned pieces; padding rows / columns are zero)."""
    off_q: int
    off_k: int
    off_v: int
    off_g: int
    off_gate: int
    off_up: int
    n_in: int
    off_act: int
    k_out: int


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass(frozen=True)
class StackSpec:
    name: str
    architecture: str
    width: int
    vocab: int
    layers: Tuple[StackLayerSpec, ...]
    loop_start: int = 0              # layers loop_start … loop_stop-1 run loop_times times in a row (own cache per pass),
    loop_stop: int = 0               # every pass starting with x <- mix_in·[x; x0]; loop_times == 0: no loop
    loop_times: int = 0
    embed_scale: float = 1.0
    residual_mult: float = 1.0
    norm_eps: float = 1e-5
    norm_offset: float = 0.0         # block / final norms multiply by (norm_offset + w)
    side_dim: int = 0                # columns of the per-layer token table, 0 = none
    max_ctx: int = 4096              # cache rows per slot
    max_slots: int = 8               # sequences the engine holds at a time
    block: str = "parallel"          # parallel: x += m·(mixer(h) + ff(h)), one norm | sandwich: a norm before and after
    norm_kind: str = "rms"           # each sublayer | postnorm: a norm behind each sublayer only.  rms | layer (weight-only)
    loop_mix: bool = True            # every pass of the loop starts with x <- mix_in·[x; x0]
    logit_softcap: float = 0.0       # > 0: logits <- cap·tanh(logits / cap)
    layer_scale: bool = False        # every sublayer's normed output is multiplied by a per-channel vector (the packer folds
                                     # it into the post-norm's weight: both are element-wise factors of the same product)

    def runs(self) -> List[Tuple[int, bool]]:
        """(layer, mix the embedding in first) for every layer run, in execution order."""
        n = len(self.layers)
        if self.loop_times <= 0:
            return [(i, False) for i in range(n)]
        out = [(i, False) for i in range(self.loop_start)]
        for _ in range(self.loop_times):
            out += [(i, self.loop_mix and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, False) for i in range(self.loop_stop, n)]

    def layout(self, i: int) -> StackLayout:
        L, a = self.layers[i], self.layers[i].attn
        off_q = 0
        off_k = off_q + _up8(a.heads * a.dim)
        off_v = off_k + _up8(a.kv_heads * a.dim)
        off_g = off_v + _up8(a.kv_heads * a.vdim)
        off_gate = off_g + (_up8(a.heads) if a.out_gate else 0)
        off_up = off_gate + _up8(L.ff)
        n_in = off_up + _up8(L.ff)
        off_act = _up8(a.heads * a.vdim)
        return StackLayout(off_q, off_k, off_v, off_g, off_gate, off_up, n_in, off_act, off_act + _up8(L.ff))

    def mix_layout(self, i: int) -> MixLayout:
        L = self.layers[i]
        if L.mixer == "latent_attention":
            a = L.latent
            off_k = _up8(a.q_rank if a.q_rank > 0 else a.heads * (a.dim + a.rot_dim))
            off_g = off_k + _up8(a.kv_rank + a.rot_dim)
            return MixLayout(off_q=0, off_k=off_k, off_g=off_g, n_in=off_g + (_up8(a.heads * a.vdim) if a.out_gate else 0),
                             k_out=a.heads * a.vdim)
        if L.mixer == "gated_delta":
            a = L.gdelta
            off_k = _up8(a.kv_heads * a.dim)
            off_v = off_k + _up8(a.kv_heads * a.dim)
            off_g = off_v + _up8(a.heads * a.vdim)
            off_gate = off_g + _up8(a.heads * a.vdim)
            off_up = off_gate + _up8(a.heads)
            return MixLayout(off_q=0, off_k=off_k, off_v=off_v, off_g=off_g, off_gate=off_gate, off_up=off_up,
                             n_in=off_up + _up8(a.heads), k_out=a.heads * a.vdim)
        if L.mixer == "mlstm":
            a = L.mlstm
            off_k = _up8(a.heads * a.dim)
            off_v = off_k + _up8(a.heads * a.dim)
            off_g = off_v + _up8(a.heads * a.vdim)
            off_gate = off_g + _up8(a.heads * a.vdim)
            return MixLayout(0, off_k, off_v, off_g, off_gate, off_gate + _up8(2 * a.heads), a.heads * a.vdim)
        if L.mixer == "attention" and L.kv_from is not None:   # queries only
            a = L.attn
            return MixLayout(off_q=0, n_in=_up8(a.heads * a.dim), k_out=a.heads * a.vdim)
        if L.mixer == "attention":
            a = L.attn
            off_k = _up8(a.heads * a.dim)
            off_v = off_k + _up8(a.kv_heads * a.dim)
            return MixLayout(off_q=0, off_k=off_k, off_v=off_v, n_in=off_v + _up8(a.kv_heads * a.vdim), k_out=a.heads * a.vdim)
        if L.mixer == "general_delta":
            a = L.delta
            seg = _up8(a.heads * a.dim)
            return MixLayout(off_q=0, off_k=seg, off_v=2 * seg, off_g=3 * seg, off_gate=4 * seg, off_up=5 * seg,
                             n_in=5 * seg + _up8(a.rank), k_out=a.heads * a.dim)
        if L.mixer == "mamba2":
            a = L.mamba
            off_v = _up8(a.inner)
            off_k = off_v + a.inner
            off_q = off_k + a.groups * a.state
            off_gate = _up8(off_q + a.groups * a.state)
            return MixLayout(off_q=off_q, off_k=off_k, off_v=off_v, off_g=0, off_gate=off_gate, n_in=off_gate + _up8(a.heads),
                             k_out=a.inner)
        raise ValueError(f"mix_layout: layer {i} has mixer {L.mixer!r}")

    def with_ctx(self, max_ctx: int, max_slots: Optional[int] = None) -> "StackSpec":
        return replace(self, max_ctx=int(max_ctx), max_slots=int(max_slots if max_slots is not None else self.max_slots))

    def weight_params(self) -> int:
        """Matrix parameters one decode step reads (every run of a looped layer reads its layer again)."""
        n = self.vocab * self.width
        for i, mix in self.runs():
            L, a = self.layers[i], self.layers[i].attn
            if L.mixer == "latent_attention":
                q = L.latent
                hq = q.heads * (q.dim + q.rot_dim)
                n += self.width * ((q.q_rank if q.q_rank > 0 else hq) + q.kv_rank + q.rot_dim + q.heads * q.vdim)
                n += q.heads * (q.dim + q.vdim) * q.kv_rank + hq * q.q_rank
                n += self.width * q.heads * q.vdim if q.out_gate else 0
            elif L.mixer == "gated_delta":
                q = L.gdelta
                n += self.width * (2 * q.kv_heads * q.dim + 3 * q.heads * q.vdim + 2 * q.heads)
            elif L.mixer == "mlstm":
                q = L.mlstm
                n += self.width * (2 * q.heads * q.dim + 3 * q.heads * q.vdim + 2 * q.heads)
            elif L.mixer == "general_delta":
                q = L.delta
                n += self.width * (6 * q.heads * q.dim + q.rank) + q.heads * q.dim * q.rank
            elif L.mixer == "mamba2":
                q = L.mamba
                n += self.width * (2 * q.inner + 2 * q.groups * q.state + q.heads + q.inner)
            elif self.block != "parallel":
                n += self.width * (a.heads * a.dim + (a.kv_heads * (a.dim + a.vdim) if L.kv_from is None else 0) + a.heads * a.vdim)
            if self.block != "parallel":
                if L.ff_kind == "dense":
                    n += 2 * L.ff * self.width
                elif L.ff_kind == "moe" and L.moe.act == "glu_clamp":   # the router, the chosen experts, the shared expert and its gate
                    n += self.width * (L.moe.experts + 3 * L.moe.top * L.moe.expert_ff + 3 * L.moe.shared_ff + 1)
                elif L.ff_kind == "moe":
                    n += self.width * (L.moe.experts + 2 * L.moe.top * L.moe.expert_ff + 2 * L.moe.shared_ff)
                continue
            n += self.width * (a.heads * a.dim + a.kv_heads * (a.dim + a.vdim) + (a.heads if a.out_gate else 0) + 2 * L.ff)
            n += self.width * (a.heads * a.vdim + L.ff) + 2 * self.side_dim * self.width
            n += 2 * self.width * self.width if mix else 0
        return n


def kozusun_from_config(doc: dict, name: str = "Kozusun") -> StackSpec:
    """config.json of the Kozusun design → StackSpec.  Kozusun: parallel blocks (one zero-centred RMS norm feeds a gated
    sliding-window attention with kept first tokens and a tanh-GELU gated feed-forward), a looped span of layers that
    re-reads [x; x0] at the start of every pass, a gated per-layer token table added through a weighted RMS norm, scaled
    embedding and residual."""
    layers = []
    for i, lc in enumerate(doc["layers"]):
        if lc.get("type") != "attention":
            raise ValueError(f"Kozusun: layer {i}: mixer type {lc.get('type')!r} is not part of the design")
        m = lc["mixer"]
        mask = m.get("mask") or {}
        attn = AttnSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                        scale=float(m["scale"]), window=int(mask.get("size", 0)), keep_first=int(mask.get("keep_first", 0)),
                        out_gate=True, bias=True)
        mlp = lc.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise ValueError(f"Kozusun: layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of the design")
        layers.append(StackLayerSpec(attn=attn, ff=int(mlp["ff"]) if mlp is not None else 0, ff_act="gelu_tanh"))
    loop = doc.get("loop") or {}
    side = doc.get("token_side") or {}
    spec = StackSpec(name=name, architecture="Kozusun", width=int(doc["width"]), vocab=int(doc["vocab"]),
                     layers=tuple(layers), loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                     loop_times=int(loop.get("times", 0)), embed_scale=float(doc["embedding"]["scale"]),
                     residual_mult=float(doc["residual_mult"]), norm_eps=float(doc["norm"]["eps"]), norm_offset=1.0,
                     side_dim=int(side.get("dim", 0)))
    if spec.loop_times > 0 and not 0 <= spec.loop_start < spec.loop_stop <= len(layers):
        raise ValueError(f"Kozusun: loop {spec.loop_start}..{spec.loop_stop} does not fit {len(layers)} layers")
    return spec


# ---------------------------------------------------------------------------------------------------------- Silatar
def _rotary_from_config(rot: dict) -> RotarySpec:
    sc = rot.get("scaling") or {}
    return RotarySpec(dims=int(rot["dims"]), base=float(rot["base"]), factor=float(sc.get("factor", 0.0)),
                      original=int(sc.get("original", 0)), fast=float(sc.get("fast", 0.0)), slow=float(sc.get("slow", 0.0)))


def silatar_from_config(doc: dict, name: str = "Silatar") -> StackSpec:
    """config.json of the Silatar design → StackSpec.  Silatar: sandwich blocks with weight-only layer norms; mixers are a
    latent attention (YaRN-stretched interleaved rotary part) or an mLSTM matrix memory; feed-forwards are a dense
    erf-GELU layer or sigmoid-routed clamped experts with a gated shared expert; a looped span of layers (own cache or
    state per pass, nothing between passes); tanh-capped logits."""
    layers = []
    for i, lc in enumerate(doc["layers"]):
        kind, m = lc.get("type"), lc["mixer"]
        kw = {}
        if kind == "latent_attention":
            rot = _rotary_from_config(m["rot"]) if m.get("rot") else RotarySpec(dims=0, base=10000.0)
            if rot.dims % 2 or rot.dims > int(m["rot_dim"]):
                raise ValueError(f"Silatar: layer {i}: rot.dims {rot.dims} must be even and at most rot_dim")
            kw = dict(mixer=kind, latent=LatentSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
                                                    vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                                                    rot=rot))
        elif kind == "mlstm":
            kw = dict(mixer=kind, mlstm=MlstmSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                                  gate_cap=float(m["gate_cap"])))
        else:
            raise ValueError(f"Silatar: layer {i}: mixer type {kind!r} is not part of the design")
        mlp = lc.get("mlp")
        if mlp is None:
            kw.update(ff_kind="dense", ff=0, ff_act="gelu_erf")
        elif mlp.get("kind") == "dense":
            kw.update(ff_kind="dense", ff=int(mlp["ff"]), ff_act="gelu_erf")
        elif mlp.get("kind") == "moe":
            sh = mlp.get("shared") or {}
            kw.update(ff_kind="moe", moe=MoeSpec(experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                                                 expert_ff=int(mlp["expert"]["ff"]), limit=float(mlp["expert"]["limit"]),
                                                 shared_ff=int(sh.get("ff", 0)), shared_limit=float(sh.get("limit", 0.0))))
            if not 1 <= kw["moe"].top <= kw["moe"].experts:
                raise ValueError(f"Silatar: layer {i}: top {kw['moe'].top} of {kw['moe'].experts} experts")
        else:
            raise ValueError(f"Silatar: layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of the design")
        layers.append(StackLayerSpec(**kw))
    loop = doc.get("loop") or {}
    spec = StackSpec(name=name, architecture="Silatar", width=int(doc["width"]), vocab=int(doc["vocab"]),
                     layers=tuple(layers), loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                     loop_times=int(loop.get("times", 0)), norm_eps=float(doc["norm"]["eps"]), norm_offset=0.0,
                     block="sandwich", norm_kind="layer", loop_mix=False,
                     logit_softcap=float(doc.get("logit_softcap") or 0.0))
    if spec.loop_times > 0 and not 0 <= spec.loop_start <= spec.loop_stop <= len(layers):
        raise ValueError(f"Silatar: loop {spec.loop_start}..{spec.loop_stop} does not fit {len(layers)} layers")
    return spec


def silatar_config(spec: StackSpec) -> dict:
    """The config.json a Silatar StackSpec is read from (inverse of silatar_from_config)."""
    doc = {"architecture": "Silatar", "layers": [], "logit_softcap": spec.logit_softcap, "norm": {"eps": spec.norm_eps},
           "vocab": spec.vocab, "width": spec.width}
    for L in spec.layers:
        if L.mixer == "latent_attention":
            a, r = L.latent, L.latent.rot
            rot = {"base": r.base, "dims": r.dims}
            if r.factor > 0:
                rot["scaling"] = {"factor": r.factor, "fast": r.fast, "original": r.original, "slow": r.slow}
            mixer = {"dim": a.dim, "heads": a.heads, "kv_rank": a.kv_rank, "rot": rot, "rot_dim": a.rot_dim,
                     "scale": a.scale, "vdim": a.vdim}
        else:
            a = L.mlstm
            mixer = {"dim": a.dim, "gate_cap": a.gate_cap, "heads": a.heads, "vdim": a.vdim}
        if L.ff_kind == "moe":
            mlp = {"expert": {"ff": L.moe.expert_ff, "limit": L.moe.limit}, "kind": "moe",
                   "router": {"experts": L.moe.experts, "top": L.moe.top}}
            if L.moe.shared_ff > 0:
                mlp["shared"] = {"ff": L.moe.shared_ff, "limit": L.moe.shared_limit}
        else:
            mlp = {"ff": L.ff, "kind": "dense"} if L.ff > 0 else None
        doc["layers"].append({"mixer": mixer, "mlp": mlp, "type": L.mixer})
    if spec.loop_times > 0:
        doc["loop"] = {"start": spec.loop_start, "stop": spec.loop_stop, "times": spec.loop_times}
    return doc


def silatar_tensor_shapes(spec: StackSpec) -> Dict[str, Tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a Silatar model (Linear weights are [out, in])."""
    W, out = spec.width, {}
    out["embed"] = (spec.vocab, W)
    for i, L in enumerate(spec.layers):
        p = f"l{i}."
        out[p + "norm1"], out[p + "norm1b"] = (W,), (W,)
        if L.mixer == "latent_attention":
            a = L.latent
            out[p + "mix.q"] = (a.heads * (a.dim + a.rot_dim), W)
            out[p + "mix.dkv"] = (a.kv_rank + a.rot_dim, W)
            out[p + "mix.dkv.norm"] = (a.kv_rank,)
            out[p + "mix.uk"] = (a.heads * a.dim, a.kv_rank)
            out[p + "mix.uv"] = (a.heads * a.vdim, a.kv_rank)
            out[p + "mix.o"] = (W, a.heads * a.vdim)
        else:
            a = L.mlstm
            out[p + "mix.q"], out[p + "mix.k"] = (a.heads * a.dim, W), (a.heads * a.dim, W)
            out[p + "mix.v"], out[p + "mix.g"] = (a.heads * a.vdim, W), (a.heads * a.vdim, W)
            out[p + "mix.o"] = (W, a.heads * a.vdim)
            out[p + "mix.norm"] = (a.heads * a.vdim,)
            for nm in ("i", "f"):
                out[p + "mix." + nm], out[p + "mix." + nm + ".b"] = (a.heads, W), (a.heads,)
        if L.ff_kind == "moe":
            out[p + "norm2"], out[p + "norm2b"] = (W,), (W,)
            for e in range(L.moe.experts):
                q = f"{p}mlp.e{e}."
                out[q + "gate"], out[q + "up"], out[q + "down"] = (L.moe.expert_ff, W), (L.moe.expert_ff, W), (W, L.moe.expert_ff)
            out[p + "mlp.router"] = (L.moe.experts, W)
            if L.moe.shared_ff > 0:
                q = p + "mlp.shared."
                out[q + "gate"], out[q + "up"], out[q + "down"] = (L.moe.shared_ff, W), (L.moe.shared_ff, W), (W, L.moe.shared_ff)
                out[q + "sg"] = (1, W)
        elif L.ff > 0:
            out[p + "norm2"], out[p + "norm2b"] = (W,), (W,)
            out[p + "mlp.up"], out[p + "mlp.down"] = (L.ff, W), (W, L.ff)
    out["final.norm"] = (W,)
    out["head"] = (spec.vocab, W)
    return out


def synth_silatar_weights(spec: StackSpec, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Seeded synthetic Silatar checkpoint (bf16, checkpoint names): matrices N(0, std·√(64/in)), norm weights 1 + N(0, 0.1),
    biases N(0, 1) (the forget gate's shifted up so that the memory keeps something)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in silatar_tensor_shapes(spec).items():
        if len(shape) == 1:
            t = torch.randn(shape, generator=g)
            t = t + 2.0 if name.endswith("f.b") else t if name.endswith(".b") else 1.0 + 0.1 * t
        else:
            t = torch.randn(shape, generator=g) * (std * (64.0 / shape[1]) ** 0.5)
            if name.endswith("router"):
                t = t * 4.0   # spread the scores so that the choice does not hang on the last bit
        w[name] = t.to(torch.bfloat16)
    return w


def pack_silatar_weights(spec: StackSpec, named: Dict[str, torch.Tensor], device="cuda",
                         dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (Silatar names) → the engine's layout on `device`.  Per layer: w_in = the mixer's in-projections
    merged by rows (StackSpec.mix_layout), b_in fp32 (the mLSTM gates' biases), w_out = mix.o; latent attention: uk both
    as stored and transposed per head [heads, kv_rank, dim], uv as stored; dense feed-forward: up / down; experts: gate|up of all experts
    as one [experts, 2·ff, width] block and down as [experts, width, ff]; shared expert: [gate | up | shared-gate row]
    (padded to 8 rows) and down.  Vectors in fp32, matrices in `dtype`."""
    W = spec.width
    out: Dict[str, torch.Tensor] = {}

    def mat(t):
        return t.to(dtype).contiguous().to(device)

    def vec(t):
        return t.to(torch.float32).contiguous().to(device)

    out["embed"], out["head"], out["final_norm"] = mat(named["embed"]), mat(named["head"]), vec(named["final.norm"])
    for i, L in enumerate(spec.layers):
        lay, p = spec.mix_layout(i), f"l{i}."
        w_in = torch.zeros(lay.n_in, W, dtype=dtype)
        b_in = torch.zeros(lay.n_in, dtype=torch.float32)

        def put(off, name, bias=None):
            t = named[p + name]
            w_in[off:off + t.shape[0]] = t.to(dtype)
            if bias is not None:
                b_in[off:off + t.shape[0]] = named[p + bias].to(torch.float32)

        if L.mixer == "latent_attention":
            a = L.latent
            put(lay.off_q, "mix.q")
            put(lay.off_k, "mix.dkv")
            out[p + "c_norm"] = vec(named[p + "mix.dkv.norm"])
            out[p + "uk_t"] = mat(named[p + "mix.uk"].view(a.heads, a.dim, a.kv_rank).transpose(1, 2))
            out[p + "uk"] = mat(named[p + "mix.uk"])
            out[p + "uv"] = mat(named[p + "mix.uv"])
        else:
            a = L.mlstm
            put(lay.off_q, "mix.q"), put(lay.off_k, "mix.k"), put(lay.off_v, "mix.v"), put(lay.off_g, "mix.g")
            put(lay.off_gate, "mix.i", "mix.i.b")
            put(lay.off_gate + a.heads, "mix.f", "mix.f.b")
            out[p + "head_norm"] = vec(named[p + "mix.norm"])
        out[p + "w_in"], out[p + "b_in"], out[p + "w_out"] = w_in.to(device), b_in.to(device), mat(named[p + "mix.o"])
        out[p + "norm"], out[p + "post_norm"] = vec(named[p + "norm1"]), vec(named[p + "norm1b"])
        if L.ff_kind == "moe" or L.ff > 0:
            out[p + "ff_norm"], out[p + "ff_post_norm"] = vec(named[p + "norm2"]), vec(named[p + "norm2b"])
        if L.ff_kind == "moe":
            m, q = L.moe, p + "mlp."
            out[p + "router"] = mat(named[q + "router"])
            out[p + "w_exp_in"] = mat(torch.stack([torch.cat([named[f"{q}e{e}.gate"], named[f"{q}e{e}.up"]], 0)
                                                   for e in range(m.experts)]))
            out[p + "w_exp_out"] = mat(torch.stack([named[f"{q}e{e}.down"] for e in range(m.experts)]))
            if m.shared_ff > 0:
                sh = torch.zeros(_up8(2 * m.shared_ff + 1), W, dtype=dtype)
                sh[:m.shared_ff] = named[q + "shared.gate"].to(dtype)
                sh[m.shared_ff:2 * m.shared_ff] = named[q + "shared.up"].to(dtype)
                sh[2 * m.shared_ff] = named[q + "shared.sg"].to(dtype)[0]
                out[p + "w_ff_in"], out[p + "w_ff_out"] = sh.to(device), mat(named[q + "shared.down"])
        elif L.ff > 0:
            out[p + "w_ff_in"], out[p + "w_ff_out"] = mat(named[p + "mlp.up"]), mat(named[p + "mlp.down"])
    return out


# ---------------------------------------------------------------------------------------------------------- Tekosun
def tekosun_from_config(doc: dict, name: str = "Tekosun", shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> StackSpec:
    """config.json of the Tekosun design → StackSpec.  Tekosun: post-norm blocks (x += rms(mixer(x))·w, x += rms(ff(x))·w) with
    three mixers — a generalized delta rule, Mamba-2, and a sliding-window attention with whole-projection query / key norms,
    rotate-half rotary positions under Llama-3.1 frequency scaling, unit-rms values and a mix-in of the first such layer's
    values — and softmax-routed squared-ReLU experts with a plain shared expert; scaled embedding.  `shapes` (tensor name →
    shape, from the checkpoint's header) gives the one size config.json leaves to the tensors: the rank of the delta rule's
    decay bottleneck (without it a default stands in, for synthetic checkpoints)."""
    layers, mix_size = [], None
    for i, lc in enumerate(doc["layers"]):
        kind, m = lc.get("type"), lc["mixer"]
        kw = {}
        if kind == "attention":
            if m.get("v_mix"):   # the mixed values are those of the same token in another layer: the sizes must agree
                if mix_size not in (None, int(m["kv_heads"]) * int(m["vdim"])):
                    raise ValueError(f"Tekosun: layer {i}: v_mix layers need as many value entries per token as the first one")
                mix_size = int(m["kv_heads"]) * int(m["vdim"])
            rot = None
            if m.get("rot"):
                sc = m["rot"].get("scaling") or {}
                rot = HalfRotarySpec(dims=int(m["rot"]["dims"]), base=float(m["rot"]["base"]), factor=float(sc.get("factor", 0.0)),
                                     low=float(sc.get("low", 0.0)), high=float(sc.get("high", 0.0)),
                                     original=int(sc.get("original", 0)))
                if rot.dims % 2 or rot.dims > int(m["dim"]):
                    raise ValueError(f"Tekosun: layer {i}: rot.dims {rot.dims} must be even and at most dim")
                if rot.dims == 0:
                    rot = None
            heads, kv = int(m["heads"]), int(m["kv_heads"])
            if heads % kv:
                raise ValueError(f"Tekosun: layer {i}: {heads} heads over {kv} kv_heads")
            kw = dict(mixer="attention",
                      attn=AttnSpec(heads=heads, kv_heads=kv, dim=int(m["dim"]), vdim=int(m["vdim"]), scale=float(m["scale"]),
                                    window=int((m.get("mask") or {}).get("size", 0)), keep_first=0, out_gate=False, bias=False),
                      prep=AttnPrepSpec(qk_norm=True, rot=rot, v_norm=True, v_mix=bool(m.get("v_mix", False))))
        elif kind == "general_delta":
            rank = int(shapes[f"l{i}.mix.w1"][0]) if shapes and f"l{i}.mix.w1" in shapes else int(m.get("rank", 16))
            kw = dict(mixer=kind, delta=DeltaSpec(heads=int(m["heads"]), dim=int(m["dim"]), rank=rank))
        elif kind == "mamba2":
            kw = dict(mixer=kind, mamba=Mamba2Spec(heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]),
                                                    groups=int(m["groups"]), conv=int(m["conv"]),
                                                    norm_groups=int(m.get("norm_groups", 1))))
            q = kw["mamba"]
            if q.heads % q.groups or q.inner % q.norm_groups or q.conv < 1:
                raise ValueError(f"Tekosun: layer {i}: Mamba-2 sizes do not divide")
        else:
            raise ValueError(f"Tekosun: layer {i}: mixer type {kind!r} is not part of the design")
        mlp = lc.get("mlp")
        if mlp is None:
            kw.update(ff_kind="dense", ff=0, ff_act="relu2")
        elif mlp.get("kind") == "moe":
            sh = mlp.get("shared") or {}
            kw.update(ff_kind="moe", ff_act="relu2",
                      moe=MoeSpec(experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                                  expert_ff=int(mlp["expert"]["ff"]), shared_ff=int(sh.get("ff", 0)), router="softmax",
                                  weight_output=True, route_scale=float(mlp["router"].get("scale", 1.0)), act="relu2",
                                  shared_plain=True))
            if not 1 <= kw["moe"].top <= kw["moe"].experts:
                raise ValueError(f"Tekosun: layer {i}: top {kw['moe'].top} of {kw['moe'].experts} experts")
        else:
            raise ValueError(f"Tekosun: layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of the design")
        layers.append(StackLayerSpec(**kw))
    return StackSpec(name=name, architecture="Tekosun", width=int(doc["width"]), vocab=int(doc["vocab"]), layers=tuple(layers),
                     embed_scale=float((doc.get("embedding") or {}).get("scale", 1.0)), norm_eps=float(doc["norm"]["eps"]),
                     norm_offset=0.0, block="postnorm", norm_kind="rms", loop_mix=False)


def tekosun_config(spec: StackSpec) -> dict:
    """The config.json a Tekosun StackSpec is read from (inverse of tekosun_from_config; the decay bottleneck's rank
    travels in the tensors' shapes)."""
    doc = {"architecture": "Tekosun", "embedding": {"scale": spec.embed_scale}, "layers": [], "norm": {"eps": spec.norm_eps},
           "vocab": spec.vocab, "width": spec.width}
    for L in spec.layers:
        if L.mixer == "attention":
            a, q = L.attn, L.prep
            mixer = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
            if a.window > 0:
                mixer["mask"] = {"size": a.window}
            if q.rot is not None:
                mixer["rot"] = {"base": q.rot.base, "dims": q.rot.dims}
                if q.rot.factor > 0:
                    mixer["rot"]["scaling"] = {"factor": q.rot.factor, "high": q.rot.high, "low": q.rot.low,
                                               "original": q.rot.original}
            if q.v_mix:
                mixer["v_mix"] = True
        elif L.mixer == "general_delta":
            mixer = {"dim": L.delta.dim, "heads": L.delta.heads}
        else:
            a = L.mamba
            mixer = {"conv": a.conv, "groups": a.groups, "heads": a.heads, "norm_groups": a.norm_groups, "state": a.state,
                     "vdim": a.vdim}
        mlp = None
        if L.ff_kind == "moe":
            mlp = {"expert": {"ff": L.moe.expert_ff}, "kind": "moe",
                   "router": {"experts": L.moe.experts, "scale": L.moe.route_scale, "top": L.moe.top}}
            if L.moe.shared_ff > 0:
                mlp["shared"] = {"ff": L.moe.shared_ff}
        doc["layers"].append({"mixer": mixer, "mlp": mlp, "type": L.mixer})
    return doc


def tekosun_tensor_shapes(spec: StackSpec) -> Dict[str, Tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a Tekosun model (Linear weights are [out, in])."""
    W, out = spec.width, {}
    out["embed"] = (spec.vocab, W)
    for i, L in enumerate(spec.layers):
        p = f"l{i}."
        out[p + "norm1"] = (W,)
        if L.mixer == "attention":
            a = L.attn
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = (a.heads * a.dim, W), (a.kv_heads * a.dim, W), (a.kv_heads * a.vdim, W)
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = (a.heads * a.dim,), (a.kv_heads * a.dim,)
            if L.prep.v_mix:
                out[p + "mix.vmix"] = ()
            out[p + "mix.o"] = (W, a.heads * a.vdim)
        elif L.mixer == "general_delta":
            a = L.delta
            n = a.heads * a.dim
            for nm in ("r", "k", "v", "g", "a"):
                out[p + "mix." + nm] = (n, W)
            out[p + "mix.a.b"], out[p + "mix.w0"], out[p + "mix.norm"] = (n,), (n,), (n,)
            out[p + "mix.w1"], out[p + "mix.w2"] = (a.rank, W), (n, a.rank)
            out[p + "mix.o"] = (W, n)
        else:
            a = L.mamba
            out[p + "mix.in"] = (2 * a.inner + 2 * a.groups * a.state + a.heads, W)
            out[p + "mix.conv"], out[p + "mix.conv.b"] = (a.channels, a.conv), (a.channels,)
            out[p + "mix.dt_bias"], out[p + "mix.A_log"], out[p + "mix.D"] = (a.heads,), (a.heads,), (a.heads,)
            out[p + "mix.norm"], out[p + "mix.o"] = (a.inner,), (W, a.inner)
        if L.ff_kind == "moe":
            out[p + "norm2"] = (W,)
            for e in range(L.moe.experts):
                out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = (L.moe.expert_ff, W), (W, L.moe.expert_ff)
            out[p + "mlp.router"] = (L.moe.experts, W)
            if L.moe.shared_ff > 0:
                out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = (L.moe.shared_ff, W), (W, L.moe.shared_ff)
    out["final.norm"] = (W,)
    out["head"] = (spec.vocab, W)
    return out


def synth_tekosun_weights(spec: StackSpec, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Seeded synthetic Tekosun checkpoint (bf16, checkpoint names): matrices N(0, std·√(64/in)) (routers four times wider,
    so that the choice does not hang on the last bit), norm weights 1 + N(0, 0.1), biases N(0, 1), the value mix-in weight
    in (0.2, 0.6), decays and step sizes in the range where the state both keeps and forgets."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tekosun_tensor_shapes(spec).items():
        t = torch.randn(shape, generator=g) if len(shape) else torch.randn((), generator=g)
        if name.endswith("vmix"):
            t = 0.4 + 0.2 * torch.tanh(t)
        elif name.endswith("A_log"):
            t = 0.5 * t
        elif name.endswith("dt_bias"):
            t = t - 1.0
        elif name.endswith("mix.D") or name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.1 * t
        elif name.endswith("mix.conv"):
            t = t * 0.5
        elif len(shape) == 2:
            t = t * (std * (64.0 / shape[1]) ** 0.5)
            if name.endswith("router"):
                t = t * 4.0
        w[name] = t.to(torch.bfloat16)
    return w


def pack_tekosun_weights(spec: StackSpec, named: Dict[str, torch.Tensor], device="cuda",
                         dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (Tekosun names) → the engine's layout on `device`.  Per layer: w_in = the mixer's in-projections
    merged by rows (StackSpec.mix_layout), b_in fp32 (the delta rule's removal bias), w_out = mix.o; the delta rule's second
    decay stage with its columns padded to 8; Mamba-2's convolution and per-head vectors in fp32; experts as one
    [experts, ff, width] and one [experts, width, ff] block; the shared expert's up rows padded to 8.  Vectors in fp32,
    matrices in `dtype`."""
    W = spec.width
    out: Dict[str, torch.Tensor] = {}

    def mat(t):
        return t.to(dtype).contiguous().to(device)

    def vec(t):
        return t.to(torch.float32).reshape(-1).contiguous().to(device)

    out["embed"], out["head"], out["final_norm"] = mat(named["embed"]), mat(named["head"]), vec(named["final.norm"])
    for i, L in enumerate(spec.layers):
        lay, p = spec.mix_layout(i), f"l{i}."
        w_in = torch.zeros(lay.n_in, W, dtype=dtype)
        b_in = torch.zeros(lay.n_in, dtype=torch.float32)

        def put(off, name, bias=None):
            t = named[p + name]
            w_in[off:off + t.shape[0]] = t.to(dtype)
            if bias is not None:
                b_in[off:off + t.shape[0]] = named[p + bias].to(torch.float32)

        if L.mixer == "attention":
            put(lay.off_q, "mix.q"), put(lay.off_k, "mix.k"), put(lay.off_v, "mix.v")
            out[p + "q_norm"], out[p + "k_norm"] = vec(named[p + "mix.q.norm"]), vec(named[p + "mix.k.norm"])
            if L.prep.v_mix:
                out[p + "vmix"] = vec(named[p + "mix.vmix"])
        elif L.mixer == "general_delta":
            a = L.delta
            put(lay.off_q, "mix.r"), put(lay.off_k, "mix.k"), put(lay.off_v, "mix.v"), put(lay.off_g, "mix.g")
            put(lay.off_gate, "mix.a", "mix.a.b"), put(lay.off_up, "mix.w1")
            w2 = torch.zeros(a.heads * a.dim, _up8(a.rank), dtype=dtype)
            w2[:, :a.rank] = named[p + "mix.w2"].to(dtype)
            out[p + "w2"], out[p + "w0"], out[p + "head_norm"] = w2.to(device), vec(named[p + "mix.w0"]), vec(named[p + "mix.norm"])
        else:
            a = L.mamba
            t = named[p + "mix.in"]
            w_in[lay.off_g:lay.off_g + a.inner] = t[:a.inner].to(dtype)
            w_in[lay.off_v:lay.off_v + a.channels] = t[a.inner:a.inner + a.channels].to(dtype)
            w_in[lay.off_gate:lay.off_gate + a.heads] = t[a.inner + a.channels:].to(dtype)
            out[p + "conv_w"], out[p + "conv_b"] = vec(named[p + "mix.conv"]), vec(named[p + "mix.conv.b"])
            out[p + "dt_bias"], out[p + "A_log"], out[p + "D"] = vec(named[p + "mix.dt_bias"]), vec(named[p + "mix.A_log"]), vec(named[p + "mix.D"])
            out[p + "mix_norm"] = vec(named[p + "mix.norm"])
        out[p + "w_in"], out[p + "b_in"], out[p + "w_out"] = w_in.to(device), b_in.to(device), mat(named[p + "mix.o"])
        out[p + "post_norm"] = vec(named[p + "norm1"])
        if L.ff_kind == "moe":
            m, q = L.moe, p + "mlp."
            out[p + "ff_post_norm"] = vec(named[p + "norm2"])
            out[p + "router"] = mat(named[q + "router"])
            out[p + "w_exp_in"] = mat(torch.stack([named[f"{q}e{e}.up"] for e in range(m.experts)]))
            out[p + "w_exp_out"] = mat(torch.stack([named[f"{q}e{e}.down"] for e in range(m.experts)]))
            if m.shared_ff > 0:
                sh = torch.zeros(_up8(m.shared_ff), W, dtype=dtype)
                sh[:m.shared_ff] = named[q + "shared.up"].to(dtype)
                out[p + "w_ff_in"], out[p + "w_ff_out"] = sh.to(device), mat(named[q + "shared.down"])
    return out


# ---------------------------------------------------------------------------------------------------------- Tarudra
def tarudra_from_config(doc: dict, name: str = "Tarudra") -> StackSpec:
    """config.json of the Tarudra design → StackSpec.  Tarudra: sandwich blocks with weight-only layer norms and a per-channel
    layer scale on every sublayer's normed output; mixers are a sliding-window attention (grouped heads, biases on q / k / v / o,
    interleaved rotary pairs under YaRN stretching, a sink in the softmax's denominator; a layer may read the keys and
    values an earlier layer cached), a latent attention (query latent, rotate-half rotary part, sliding window, element-wise
    sigmoid output gate) or the gated delta rule behind short convolutions; dense squared-ReLU feed-forwards; tanh-capped logits."""
    layers = []
    for i, lc in enumerate(doc["layers"]):
        kind, m = lc.get("type"), lc["mixer"]
        window = int((m.get("mask") or {}).get("size", 0))
        if kind == "attention":
            heads, kv = int(m["heads"]), int(m["kv_heads"])
            if kv < 1 or heads % kv:
                raise ValueError(f"Tarudra: layer {i}: {heads} heads over {kv} kv_heads")
            rot = _rotary_from_config(m["rot"]) if m.get("rot") else None
            if rot is not None and (rot.dims % 2 or rot.dims > int(m["dim"])):
                raise ValueError(f"Tarudra: layer {i}: rot.dims {rot.dims} must be even and at most dim")
            if rot is not None and rot.dims == 0:
                rot = None
            attn = AttnSpec(heads=heads, kv_heads=kv, dim=int(m["dim"]), vdim=int(m["vdim"]), scale=float(m["scale"]),
                            window=window, keep_first=0, out_gate=False, bias=True, sink=True, out_bias=True)
            src = m.get("kv_from")
            if src is not None:
                src = int(src)
                S = layers[src] if 0 <= src < i else None
                if S is None or S.mixer != "attention" or S.kv_from is not None:
                    raise ValueError(f"Tarudra: layer {i}: kv_from {src} is not an earlier attention layer with keys and values of its own")
                if (S.attn.kv_heads, S.attn.dim, S.attn.vdim) != (kv, attn.dim, attn.vdim):
                    raise ValueError(f"Tarudra: layer {i}: the keys and values of layer {src} have other sizes")
            kw = dict(mixer="attention", attn=attn, kv_from=src,
                      prep=AttnPrepSpec(qk_norm=False, rot=rot, v_norm=False, v_mix=False, rot_interleaved=True))
        elif kind == "latent_attention":
            rot = _rotary_from_config(m["rot"]) if m.get("rot") and int(m["rot_dim"]) > 0 else RotarySpec(dims=0, base=10000.0)
            if rot.dims % 2 or rot.dims > int(m["rot_dim"]):
                raise ValueError(f"Tarudra: layer {i}: rot.dims {rot.dims} must be even and at most rot_dim")
            kw = dict(mixer=kind, latent=LatentSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
                                                    vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                                                    rot=rot, rot_layout="half", q_rank=int(m["q_rank"]), window=window,
                                                    out_gate=True))
            if kw["latent"].q_rank < 1:
                raise ValueError(f"Tarudra: layer {i}: q_rank {kw['latent'].q_rank}")
        elif kind == "delta":
            heads, kv = int(m["heads"]), int(m["kv_heads"])
            if kv < 1 or heads % kv or int(m["conv"]) < 1:
                raise ValueError(f"Tarudra: layer {i}: {heads} heads over {kv} kv_heads, {m['conv']} taps")
            kw = dict(mixer="gated_delta", gdelta=GatedDeltaSpec(heads=heads, kv_heads=kv, dim=int(m["dim"]), vdim=int(m["vdim"]),
                                                                 conv=int(m["conv"])))
        else:
            raise ValueError(f"Tarudra: layer {i}: mixer type {kind!r} is not part of the design")
        mlp = lc.get("mlp")
        if mlp is None:
            kw.update(ff_kind="dense", ff=0, ff_act="relu2")
        elif mlp.get("kind") == "dense":
            kw.update(ff_kind="dense", ff=int(mlp["ff"]), ff_act="relu2")
        else:
            raise ValueError(f"Tarudra: layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of the design")
        layers.append(StackLayerSpec(**kw))
    return StackSpec(name=name, architecture="Tarudra", width=int(doc["width"]), vocab=int(doc["vocab"]), layers=tuple(layers),
                     norm_eps=float(doc["norm"]["eps"]), norm_offset=0.0, block="sandwich", norm_kind="layer", loop_mix=False,
                     logit_softcap=float(doc.get("logit_softcap") or 0.0), layer_scale=True)


def _rotary_config(r: RotarySpec) -> dict:
    rot = {"base": r.base, "dims": r.dims}
    if r.factor > 0:
        rot["scaling"] = {"factor": r.factor, "fast": r.fast, "original": r.original, "slow": r.slow}
    return rot


def tarudra_config(spec: StackSpec) -> dict:
    """The config.json a Tarudra StackSpec is read from (inverse of tarudra_from_config)."""
    doc = {"architecture": "Tarudra", "layers": [], "logit_softcap": spec.logit_softcap, "norm": {"eps": spec.norm_eps},
           "vocab": spec.vocab, "width": spec.width}
    kinds = {"attention": "attention", "latent_attention": "latent_attention", "gated_delta": "delta"}
    for L in spec.layers:
        if L.mixer == "attention":
            a = L.attn
            mixer = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
            if a.window > 0:
                mixer["mask"] = {"size": a.window}
            if L.prep.rot is not None:
                mixer["rot"] = _rotary_config(L.prep.rot)
            if L.kv_from is not None:
                mixer["kv_from"] = L.kv_from
        elif L.mixer == "latent_attention":
            a = L.latent
            mixer = {"dim": a.dim, "heads": a.heads, "kv_rank": a.kv_rank, "q_rank": a.q_rank, "rot_dim": a.rot_dim,
                     "scale": a.scale, "vdim": a.vdim}
            if a.window > 0:
                mixer["mask"] = {"size": a.window}
            if a.rot_dim > 0:
                mixer["rot"] = _rotary_config(a.rot)
        else:
            a = L.gdelta
            mixer = {"conv": a.conv, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "vdim": a.vdim}
        doc["layers"].append({"mixer": mixer, "mlp": {"ff": L.ff, "kind": "dense"} if L.ff > 0 else None, "type": kinds[L.mixer]})
    return doc


def tarudra_tensor_shapes(spec: StackSpec) -> Dict[str, Tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a Tarudra model (Linear weights are [out, in])."""
    W, out = spec.width, {}
    out["embed"] = (spec.vocab, W)
    for i, L in enumerate(spec.layers):
        p = f"l{i}."
        out[p + "norm1"], out[p + "norm1b"], out[p + "ls1"] = (W,), (W,), (W,)
        if L.mixer == "attention":
            a = L.attn
            segs = [("q", a.heads * a.dim)] + ([("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)] if L.kv_from is None else [])
            for nm, rows in segs:
                out[p + "mix." + nm], out[p + "mix." + nm + ".b"] = (rows, W), (rows,)
            out[p + "mix.o"], out[p + "mix.o.b"] = (W, a.heads * a.vdim), (W,)
        elif L.mixer == "latent_attention":
            a = L.latent
            out[p + "mix.dq"], out[p + "mix.dq.norm"] = (a.q_rank, W), (a.q_rank,)
            out[p + "mix.uq"] = (a.heads * (a.dim + a.rot_dim), a.q_rank)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = (a.kv_rank + a.rot_dim, W), (a.kv_rank,)
            out[p + "mix.uk"], out[p + "mix.uv"] = (a.heads * a.dim, a.kv_rank), (a.heads * a.vdim, a.kv_rank)
            out[p + "mix.g"], out[p + "mix.o"] = (a.heads * a.vdim, W), (W, a.heads * a.vdim)
        else:
            a = L.gdelta
            for nm, rows in (("q", a.kv_heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.heads * a.vdim)):
                out[p + "mix." + nm], out[p + "mix." + nm + ".conv"] = (rows, W), (rows, a.conv)
            out[p + "mix.b"], out[p + "mix.a"] = (a.heads, W), (a.heads, W)
            out[p + "mix.A_log"], out[p + "mix.dt_bias"], out[p + "mix.norm"] = (a.heads,), (a.heads,), (a.vdim,)
            out[p + "mix.g"], out[p + "mix.o"] = (a.heads * a.vdim, W), (W, a.heads * a.vdim)
        if L.ff > 0:
            out[p + "norm2"], out[p + "norm2b"], out[p + "ls2"] = (W,), (W,), (W,)
            out[p + "mlp.up"], out[p + "mlp.down"] = (L.ff, W), (W, L.ff)
    out["final.norm"] = (W,)
    out["head"] = (spec.vocab, W)
    return out


def synth_tarudra_weights(spec: StackSpec, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Seeded synthetic Tarudra checkpoint (bf16, checkpoint names): matrices N(0, std·√(64/in)), norm weights 1 + N(0, 0.1),
    layer scales in (0.3, 1.0), biases N(0, 0.5), convolution taps N(0, 0.5), decays and write strengths in the range where
    the state both keeps and forgets."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tarudra_tensor_shapes(spec).items():
        t = torch.randn(shape, generator=g)
        if name.endswith("ls1") or name.endswith("ls2"):
            t = 0.65 + 0.35 * torch.tanh(t)
        elif name.endswith("A_log"):
            t = 0.5 * t
        elif name.endswith("dt_bias"):
            t = t - 1.0
        elif name.endswith(".conv") or name.endswith(".b") and len(shape) == 1:
            t = t * 0.5
        elif len(shape) == 1:
            t = 1.0 + 0.1 * t
        else:
            t = t * (std * (64.0 / shape[1]) ** 0.5)
        w[name] = t.to(torch.bfloat16)
    return w


def pack_tarudra_weights(spec: StackSpec, named: Dict[str, torch.Tensor], device="cuda",
                         dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (Tarudra names) → the engine's layout on `device`.  Per layer: w_in = the mixer's in-projections merged
    by rows (StackSpec.mix_layout) with their biases in the fp32 b_in, w_out = mix.o (+ b_out); the layer scale is folded into the
    post-norm's weight (the product of two bf16 values is exact in fp32); latent attention: the query's up-projection with its
    columns padded to 8, uk both as stored and transposed per head; gated delta rule: the three convolutions' taps as one fp32
    [channels, taps] block in q | k | v order.  Vectors in fp32, matrices in `dtype`."""
    W = spec.width
    out: Dict[str, torch.Tensor] = {}

    def mat(t):
        return t.to(dtype).contiguous().to(device)

    def vec(t):
        return t.to(torch.float32).reshape(-1).contiguous().to(device)

    out["embed"], out["head"], out["final_norm"] = mat(named["embed"]), mat(named["head"]), vec(named["final.norm"])
    for i, L in enumerate(spec.layers):
        lay, p = spec.mix_layout(i), f"l{i}."
        w_in = torch.zeros(lay.n_in, W, dtype=dtype)
        b_in = torch.zeros(lay.n_in, dtype=torch.float32)

        def put(off, name, bias=None):
            t = named[p + name]
            w_in[off:off + t.shape[0]] = t.to(dtype)
            if bias is not None:
                b_in[off:off + t.shape[0]] = named[p + bias].to(torch.float32)

        if L.mixer == "attention":
            put(lay.off_q, "mix.q", "mix.q.b")
            if L.kv_from is None:
                put(lay.off_k, "mix.k", "mix.k.b"), put(lay.off_v, "mix.v", "mix.v.b")
            out[p + "b_in"], out[p + "b_out"] = b_in.to(device), vec(named[p + "mix.o.b"])
        elif L.mixer == "latent_attention":
            a = L.latent
            put(lay.off_q, "mix.dq"), put(lay.off_k, "mix.dkv"), put(lay.off_g, "mix.g")
            uq = torch.zeros(a.heads * (a.dim + a.rot_dim), _up8(a.q_rank), dtype=dtype)
            uq[:, :a.q_rank] = named[p + "mix.uq"].to(dtype)
            out[p + "uq"], out[p + "q_norm"] = uq.to(device), vec(named[p + "mix.dq.norm"])
            out[p + "c_norm"] = vec(named[p + "mix.dkv.norm"])
            out[p + "uk_t"] = mat(named[p + "mix.uk"].view(a.heads, a.dim, a.kv_rank).transpose(1, 2))
            out[p + "uk"], out[p + "uv"] = mat(named[p + "mix.uk"]), mat(named[p + "mix.uv"])
        else:
            put(lay.off_q, "mix.q"), put(lay.off_k, "mix.k"), put(lay.off_v, "mix.v"), put(lay.off_g, "mix.g")
            put(lay.off_gate, "mix.b"), put(lay.off_up, "mix.a")
            out[p + "conv_w"] = vec(torch.cat([named[p + "mix.q.conv"], named[p + "mix.k.conv"], named[p + "mix.v.conv"]], 0))
            out[p + "A_log"], out[p + "dt_bias"] = vec(named[p + "mix.A_log"]), vec(named[p + "mix.dt_bias"])
            out[p + "head_norm"] = vec(named[p + "mix.norm"])
        out[p + "w_in"], out[p + "w_out"] = w_in.to(device), mat(named[p + "mix.o"])
        out[p + "norm"] = vec(named[p + "norm1"])
        out[p + "post_norm"] = vec(named[p + "norm1b"].to(torch.float32) * named[p + "ls1"].to(torch.float32))
        if L.ff > 0:
            out[p + "ff_norm"] = vec(named[p + "norm2"])
            out[p + "ff_post_norm"] = vec(named[p + "norm2b"].to(torch.float32) * named[p + "ls2"].to(torch.float32))
            out[p + "w_ff_in"], out[p + "w_ff_out"] = mat(named[p + "mlp.up"]), mat(named[p + "mlp.down"])
    return out


@dataclass(frozen=True)
class Architecture:
    """One design of the layer-stack registry: its config reader and writer, checkpoint tensor list, synthetic checkpoint
    and the packer into the engine's layout.  with_shapes: the config reader also takes the checkpoint's tensor shapes
    (name → shape) for sizes config.json leaves to the tensors."""
    from_config: Callable[..., StackSpec]
    to_config: Callable[[StackSpec], dict]
    tensor_shapes: Callable[[StackSpec], Dict[str, Tuple[int, ...]]]
    synth_weights: Callable[..., Dict[str, torch.Tensor]]
    pack: Callable[..., Dict[str, torch.Tensor]]
    with_shapes: bool = False

    def __call__(self, doc: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> StackSpec:
        return self.from_config(doc, shapes=shapes) if self.with_shapes else self.from_config(doc)


# config.json "architecture" → design.  (The Llama-family checkpoints are told apart by "model_type": loader.py.)
ARCHITECTURES: Dict[str, Architecture] = {}


def kozusun_config(spec: StackSpec) -> dict:
    """The config.json a Kozusun StackSpec is read from (inverse of kozusun_from_config)."""
    doc = {"architecture": "Kozusun", "embedding": {"scale": spec.embed_scale}, "layers": [],
           "norm": {"eps": spec.norm_eps}, "residual_mult": spec.residual_mult, "vocab": spec.vocab, "width": spec.width}
    for L in spec.layers:
        a = L.attn
        doc["layers"].append({"type": "attention",
                              "mixer": {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "vdim": a.vdim,
                                        "scale": a.scale, "mask": {"keep_first": a.keep_first, "size": a.window}},
                              "mlp": {"ff": L.ff, "kind": "dense"} if L.ff > 0 else None})
    if spec.loop_times > 0:
        doc["loop"] = {"start": spec.loop_start, "stop": spec.loop_stop, "times": spec.loop_times}
    if spec.side_dim > 0:
        doc["token_side"] = {"dim": spec.side_dim}
    return doc


def kozusun_tensor_shapes(spec: StackSpec) -> Dict[str, Tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a Kozusun model (Linear weights are [out, in])."""
    W, out = spec.width, {}
    out["embed"] = (spec.vocab, W)
    if spec.loop_times > 0:
        out["loop.in"] = (W, 2 * W)
    if spec.side_dim > 0:
        out["side.embed"] = (spec.vocab, spec.side_dim * len(spec.layers))
    for i, L in enumerate(spec.layers):
        a, p = L.attn, f"l{i}."
        out[p + "norm1"] = (W,)
        for nm, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
            out[p + "mix." + nm] = (rows, W)
            out[p + "mix." + nm + ".b"] = (rows,)
        out[p + "mix.g"] = (a.heads, W)
        out[p + "mix.o"] = (W, a.heads * a.vdim)
        if L.ff > 0:
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (L.ff, W), (L.ff, W), (W, L.ff)
        if spec.side_dim > 0:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = (spec.side_dim, W), (W, spec.side_dim), (W,)
    out["final.norm"] = (W,)
    out["head"] = (spec.vocab, W)
    return out


def synth_kozusun_weights(spec: StackSpec, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Seeded synthetic Kozusun checkpoint (bf16, checkpoint names): matrices N(0, std·√(64/in)), vectors N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in kozusun_tensor_shapes(spec).items():
        if len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.1
            if name.endswith("side.norm"):
                t = t + 1.0
        else:
            t = torch.randn(shape, generator=g) * (std * (64.0 / shape[1]) ** 0.5)
        w[name] = t.to(torch.bfloat16)
    return w


def pack_stack_weights(spec: StackSpec, named: Dict[str, torch.Tensor], device="cuda",
                       dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (Kozusun names) → the engine's layout on `device`: per layer w_in = [q | k | v | g | gate | up]
    (rows, segments on multiples of 8, zero padding), b_in (fp32, zero where a segment has no bias), w_out = [o | down]
    (columns), vectors in fp32; matrices in `dtype` (bf16 values are exact in fp32)."""
    W = spec.width
    out: Dict[str, torch.Tensor] = {}

    def mat(t):
        return t.to(dtype).contiguous().to(device)

    def vec(t):
        return t.to(torch.float32).contiguous().to(device)

    out["embed"] = mat(named["embed"])
    out["head"] = mat(named["head"])
    out["final_norm"] = vec(named["final.norm"])
    if spec.loop_times > 0:
        out["mix_in"] = mat(named["loop.in"])
    if spec.side_dim > 0:
        out["side_table"] = mat(named["side.embed"])
    for i, L in enumerate(spec.layers):
        a, lay, p = L.attn, spec.layout(i), f"l{i}."
        w_in = torch.zeros(lay.n_in, W, dtype=dtype)
        b_in = torch.zeros(lay.n_in, dtype=torch.float32)
        segs = [("q", lay.off_q), ("k", lay.off_k), ("v", lay.off_v)]
        for nm, off in segs:
            t = named[p + "mix." + nm]
            w_in[off:off + t.shape[0]] = t.to(dtype)
            if a.bias:
                b_in[off:off + t.shape[0]] = named[p + "mix." + nm + ".b"].to(torch.float32)
        if a.out_gate:
            w_in[lay.off_g:lay.off_g + a.heads] = named[p + "mix.g"].to(dtype)
        w_out = torch.zeros(W, lay.k_out, dtype=dtype)
        w_out[:, :a.heads * a.vdim] = named[p + "mix.o"].to(dtype)
        if L.ff > 0:
            w_in[lay.off_gate:lay.off_gate + L.ff] = named[p + "mlp.gate"].to(dtype)
            w_in[lay.off_up:lay.off_up + L.ff] = named[p + "mlp.up"].to(dtype)
            w_out[:, lay.off_act:lay.off_act + L.ff] = named[p + "mlp.down"].to(dtype)
        out[p + "norm"] = vec(named[p + "norm1"])
        out[p + "w_in"], out[p + "b_in"], out[p + "w_out"] = w_in.to(device), b_in.to(device), w_out.to(device)
        if spec.side_dim > 0:
            out[p + "side_gate"] = mat(named[p + "side.gate"])
            out[p + "side_proj"] = mat(named[p + "side.proj"])
            out[p + "side_norm"] = vec(named[p + "side.norm"])
    return out


def pack_weights(spec: StackSpec, named: Dict[str, torch.Tensor], device="cuda",
                 dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors of any registered design → the engine's layout."""
    return ARCHITECTURES[spec.architecture].pack(spec, named, device=device, dtype=dtype)


def save_stack_checkpoint(spec: StackSpec, named: Dict[str, torch.Tensor], out_dir: str) -> None:
    """config.json + model.safetensors (bf16) of a layer-stack model, as loader.load_model reads them."""
    d = Path(out_dir)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps(ARCHITECTURES[spec.architecture].to_config(spec), indent=1))
    header, off, blobs = {}, 0, []
    for name in sorted(named):
        raw = named[name].detach().to("cpu").to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(named[name].shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(d / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


ARCHITECTURES["Kozusun"] = Architecture(kozusun_from_config, kozusun_config, kozusun_tensor_shapes, synth_kozusun_weights,
                                        pack_stack_weights)
ARCHITECTURES["Silatar"] = Architecture(silatar_from_config, silatar_config, silatar_tensor_shapes, synth_silatar_weights,
                                        pack_silatar_weights)
ARCHITECTURES["Tekosun"] = Architecture(tekosun_from_config, tekosun_config, tekosun_tensor_shapes, synth_tekosun_weights,
                                        pack_tekosun_weights, with_shapes=True)
ARCHITECTURES["Tarudra"] = Architecture(tarudra_from_config, tarudra_config, tarudra_tensor_shapes, synth_tarudra_weights,
                                        pack_tarudra_weights)


# ------------------------------------------------------------------------------------------- checkpoint writer
def save_checkpoint(spec: ModelSpec, w: Dict[str, torch.Tensor], out_dir: str) -> None:
    """Write config.json + generation_config.json + model.safetensors in the layout the reference's loader accepts
    (src/huggingface/ModelLoader.cpp:25-87, src/util/SafeTensors.cpp:141-229), so the same synthetic checkpoint can be
    fed to an unmodified TinyGPT build.  Tokenizer files are not written (copy them from the reference's
    assets/tokenizer/<family>)."""
    d = Path(out_dir)
    d.mkdir(parents=True, exist_ok=True)
    cfg = {
        "model_type": spec.model_type, "hidden_size": spec.hidden, "num_hidden_layers": spec.layers,
        "num_attention_heads": spec.q_heads, "num_key_value_heads": spec.kv_heads, "head_dim": spec.head_dim,
        "intermediate_size": spec.intermediate, "vocab_size": spec.vocab, "rope_theta": spec.rope_theta,
        "rms_norm_eps": spec.rms_eps, "tie_word_embeddings": spec.tie, "max_position_embeddings": spec.max_ctx,
        "torch_dtype": "bfloat16", "hidden_act": "silu",
    }
    if spec.rope_scaling is not None:
        sc = spec.rope_scaling
        cfg["rope_scaling"] = {"factor": sc.factor, "high_freq_factor": sc.high_freq_factor,
                               "low_freq_factor": sc.low_freq_factor,
                               "original_max_position_embeddings": sc.original_context_length, "rope_type": "llama3"}
    (d / "config.json").write_text(json.dumps(cfg, indent=1))
    (d / "generation_config.json").write_text(json.dumps({"do_sample": False, "temperature": 0.0, "top_p": 1.0}))
    state = split_views(spec, w)
    header, off, blobs = {}, 0, []
    for name in sorted(state):
        t = state[name].detach().to("cpu").contiguous()
        assert t.dtype == torch.bfloat16
        raw = t.view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(d / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
