"""Host-side mirror of the TinyTorch functions on the decode path, over torch CUDA tensors → C ABI → sm_100a kernels.

Names and argument meaning follow tinytorch::function::* / op::* (third_party/TinyTorch/src/Function/FuncNNLayer.h,
FuncFused.h, FuncElemWise.h, FuncReduce.h); torch is used only for device memory and the current stream.
Every function raises B200Error when the CUDA library or an sm_100 device is missing — no fallback.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import B200Error, check, lib

BSHD, BHSD = 1, 0  # b200_qkv_layout


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: torch.Tensor, name: str, dtype=torch.bfloat16) -> torch.Tensor:
    if not t.is_cuda:
        raise B200Error(f"{name}: tensor must live on a CUDA device (there is no CPU path)")
    if t.dtype != dtype:
        raise B200Error(f"{name}: expected dtype {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """function::linear(x, W, b) = op::matmul(x, W, false, true, b)  [ref: TT/Function/FuncNNLayer.h:14-18].
    x [..., k] bf16, W [n, k] bf16 → [..., n] bf16."""
    x, weight = _chk(x, "linear.x"), _chk(weight, "linear.weight")
    if bias is not None:
        bias = _chk(bias, "linear.bias")
    n, k = weight.shape
    if x.shape[-1] != k:
        raise B200Error(f"linear: x[..., {x.shape[-1]}] does not match W[{n}, {k}]")
    m = x.numel() // k
    y = torch.empty(*x.shape[:-1], n, dtype=torch.bfloat16, device=x.device)
    check(lib().b200_gemv_bf16(y.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(bias), m, n, k, _stream()),
          "b200_gemv_bf16")
    return y


def gemm(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Batched Linear without bias on the tcgen05 tensor cores: a [..., k] · W[n, k]ᵀ → [..., n] (prefill, m > 1)."""
    a, weight = _chk(a, "gemm.a"), _chk(weight, "gemm.weight")
    n, k = weight.shape
    if a.shape[-1] != k:
        raise B200Error(f"gemm: a[..., {a.shape[-1]}] does not match W[{n}, {k}]")
    m = a.numel() // k
    c = torch.empty(*a.shape[:-1], n, dtype=torch.bfloat16, device=a.device)
    check(lib().b200_gemm_bf16(c.data_ptr(), a.data_ptr(), weight.data_ptr(), m, n, k, _stream()), "b200_gemm_bf16")
    return c


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """function::rmsNorm(x, {dim}, w, eps)  [ref: TT/Function/FuncNNLayer.h:220-227]."""
    x = _chk(x, "rms_norm.x")
    if weight is not None:
        weight = _chk(weight, "rms_norm.weight")
    dim = x.shape[-1]
    y = torch.empty_like(x)
    check(lib().b200_rmsnorm_bf16(y.data_ptr(), x.data_ptr(), _ptr(weight), x.numel() // dim, dim, float(eps),
                                  _stream()), "b200_rmsnorm_bf16")
    return y


def rope_apply(x: torch.Tensor, table: torch.Tensor, offset: int, layout: int = BSHD) -> torch.Tensor:
    """function::ropeApply(x, rope, offset, layout)  [ref: TT/Function/FuncNNLayer.h:279-286]. x is 4-D."""
    x, table = _chk(x, "rope_apply.x"), _chk(table, "rope_apply.table", torch.float32)
    if x.dim() != 4:
        raise B200Error("rope_apply: input must be 4-D")
    if layout == BSHD:
        B, S, N, D = x.shape
    else:
        B, N, S, D = x.shape
    if table.shape[-2] != D or offset + S > table.shape[0]:
        raise B200Error("rope_apply: table does not cover the requested positions / head_dim")
    y = torch.empty_like(x)
    check(lib().b200_rope_bf16(y.data_ptr(), x.data_ptr(), table.data_ptr(), B, S, N, D, int(offset), layout,
                               _stream()), "b200_rope_bf16")
    return y


def rope_init(head_dim: int, ctx: int, theta: float, scaling=None, device="cuda") -> torch.Tensor:
    """op::ropeInit  [ref: TT/Operation/OpNNLayerCuda.cuh:621-656] → fp32 [ctx, head_dim, 2] built on the device."""
    t = torch.empty(ctx, head_dim, 2, dtype=torch.float32, device=device)
    f, hi, lo, orig = (0.0, 0.0, 0.0, 0) if scaling is None else (
        scaling.factor, scaling.high_freq_factor, scaling.low_freq_factor, scaling.original_context_length)
    check(lib().b200_rope_init_f32(t.data_ptr(), head_dim, ctx, float(theta), float(f), float(hi), float(lo),
                                   int(orig), _stream()), "b200_rope_init_f32")
    return t


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False) -> torch.Tensor:
    """function::flashAttention(q, k, v, isCausal), BSHD  [ref: TT/Function/FuncNNLayer.h:270-277]."""
    q, k, v = _chk(q, "flash_attention.q"), _chk(k, "flash_attention.k"), _chk(v, "flash_attention.v")
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    o = torch.empty_like(q)
    check(lib().b200_attn_bf16(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, Sq, Skv, Hq, Hkv, D,
                               int(bool(is_causal)), _stream()), "b200_attn_bf16")
    return o


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    """function::siluMul(x): last dim = [gate | up]  [ref: TT/Function/FuncFused.h:14-21]."""
    x = _chk(x, "silu_mul.x")
    I = x.shape[-1] // 2
    if x.shape[-1] % 2:
        raise B200Error("silu_mul: last dimension must be even")
    y = torch.empty(*x.shape[:-1], I, dtype=torch.bfloat16, device=x.device)
    check(lib().b200_silu_mul_bf16(y.data_ptr(), x.data_ptr(), x.numel() // (2 * I), I, _stream()),
          "b200_silu_mul_bf16")
    return y


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """function::add(a, b) with alpha = 1, same shapes  [ref: TT/Function/FuncElemWise.h:74]."""
    a, b = _chk(a, "add.a"), _chk(b, "add.b")
    if a.shape != b.shape:
        raise B200Error("add: the decode path only adds same-shape tensors")
    y = torch.empty_like(a)
    check(lib().b200_add_bf16(y.data_ptr(), a.data_ptr(), b.data_ptr(), a.numel(), _stream()), "b200_add_bf16")
    return y


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """function::embedding(ids, table) → op::indexAdvance  [ref: TT/Function/FuncNNLayer.h:202-207]; ids Int64."""
    table, ids = _chk(table, "embedding.table"), _chk(ids, "embedding.ids", torch.int64)
    V, H = table.shape
    y = torch.empty(*ids.shape, H, dtype=torch.bfloat16, device=table.device)
    if ids.numel():
        check(lib().b200_embedding_bf16(y.data_ptr(), table.data_ptr(), ids.data_ptr(), ids.numel(), V, H, _stream()),
              "b200_embedding_bf16")
    return y


def argmax(logits: torch.Tensor, keepdim: bool = True) -> torch.Tensor:
    """function::argmax(logits, -1, keepdim): fp32 compare, HIGHEST index wins ties (reference CUDA rule)
    [ref: src/engine/Sampler.cpp:23-29; TT/Operation/OpReduceCuda.cuh:145-156]."""
    logits = _chk(logits, "argmax.logits")
    V = logits.shape[-1]
    rows = logits.numel() // V
    ws = torch.zeros(lib().b200_argmax_workspace_bytes(rows, V), dtype=torch.uint8, device=logits.device)
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    check(lib().b200_argmax_bf16(out.data_ptr(), logits.data_ptr(), rows, V, ws.data_ptr(), _stream()),
          "b200_argmax_bf16")
    shape = list(logits.shape[:-1]) + ([1] if keepdim else [])
    return out.view(shape)


# ---- fused building blocks (the kernels the engine actually runs)
def gemv_fused(x, weight, *, norm_weight=None, eps=0.0, bias=None, residual=None, silu_mul=False) -> torch.Tensor:
    """[RMSNorm] → GEMV → {bias | residual | SiLU·mul over merged gate|up} in ONE launch (m = 1)."""
    x, weight = _chk(x, "gemv_fused.x"), _chk(weight, "gemv_fused.weight")
    rows, k = weight.shape
    nseg = 2 if silu_mul else 1
    n = rows // nseg
    y = torch.empty(n, dtype=torch.bfloat16, device=x.device)
    check(lib().b200_gemv_fused_bf16(y.data_ptr(), x.data_ptr(), weight.data_ptr(), n, k, nseg, _ptr(norm_weight),
                                     float(eps), _ptr(bias), _ptr(residual), int(silu_mul), _stream()),
          "b200_gemv_fused_bf16")
    return y


def attn_decode(qkv, kcache, vcache, *, q_heads, kv_heads, head_dim, pos=None, fixed_len=0, rope_table=None,
                q_norm=None, k_norm=None, eps=0.0) -> torch.Tensor:
    """Fused decode attention of one layer (see include/b200_decode.h b200_attn_decode_bf16)."""
    qkv, kcache, vcache = _chk(qkv, "attn_decode.qkv"), _chk(kcache, "attn_decode.kcache"), _chk(vcache, "attn_decode.vcache")
    max_ctx = kcache.shape[0]
    ws = torch.zeros(lib().b200_attn_decode_workspace_bytes(q_heads, kv_heads, head_dim, max_ctx), dtype=torch.uint8,
                     device=qkv.device)
    out = torch.empty(q_heads * head_dim, dtype=torch.bfloat16, device=qkv.device)
    check(lib().b200_attn_decode_bf16(out.data_ptr(), qkv.data_ptr(), _ptr(q_norm), _ptr(k_norm), float(eps),
                                      _ptr(rope_table), _ptr(pos), int(fixed_len), kcache.data_ptr(),
                                      vcache.data_ptr(), q_heads, kv_heads, head_dim, max_ctx, ws.data_ptr(),
                                      _stream()), "b200_attn_decode_bf16")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
           u: float = 0.5) -> torch.Tensor:
    """Sampler::sample for one row of bf16 logits [V] with the uniform number u supplied by the caller
    [ref: src/engine/Sampler.cpp:31-78].  Returns an int64 device tensor [1]."""
    logits = _chk(logits, "sample.logits").view(-1)
    ws = torch.empty(lib().b200_sample_workspace_bytes(), dtype=torch.uint8, device=logits.device)
    out = torch.empty(1, dtype=torch.int64, device=logits.device)
    check(lib().b200_sample_bf16(out.data_ptr(), logits.data_ptr(), logits.numel(), float(temperature), int(top_k),
                                 float(top_p), float(min_p), float(u), ws.data_ptr(), _stream()), "b200_sample_bf16")
    return out


# ------------------------------------------------------------------------------- mechanisms of the layer-stack engine
# T = bf16 or fp32 storage (taken from the tensors); norms, softmax, gates and accumulation are fp32 in both.
def _sdt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise B200Error(f"stack op: dtype {t.dtype} (bf16 or fp32)")


def _tdt(code_or_dtype) -> torch.dtype:
    return code_or_dtype if isinstance(code_or_dtype, torch.dtype) else (torch.float32 if code_or_dtype else torch.bfloat16)


def stack_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float = 0.0,
                  out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out_dtype( x·rsqrt(mean(x²) + eps)·(offset + w) ) for fp32 x [rows, dim] and fp32 w [dim]."""
    x, w = _chk(x, "stack_rmsnorm x", torch.float32), _chk(w, "stack_rmsnorm w", torch.float32)
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(lib().b200_stack_rmsnorm(y.data_ptr(), x.data_ptr(), w.data_ptr(), x.numel() // x.shape[-1], x.shape[-1],
                                   float(eps), float(offset), _sdt(y), _stream()), "b200_stack_rmsnorm")
    return y


def stack_linear(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] · weight [N, K]ᵀ (+ fp32 bias [N]) with fp32 accumulation, any sizes; a, weight and the result share T."""
    a, weight = _chk(a, "stack_linear a", a.dtype), _chk(weight, "stack_linear weight", a.dtype)
    if bias is not None:
        bias = _chk(bias, "stack_linear bias", torch.float32)
    M, K = a.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise B200Error("stack_linear: inner sizes differ")
    c = torch.empty(M, N, dtype=a.dtype, device=a.device)
    check(lib().b200_stack_linear(c.data_ptr(), a.data_ptr(), weight.data_ptr(), _ptr(bias), M, N, K, _sdt(a), _stream()),
          "b200_stack_linear")
    return c


_ACTS = {"gelu_tanh": 0, "silu": 1, "gelu_erf": 2, "relu2": 3, "tanh": 4}


def _attn_desc(heads, kv_heads, dim, vdim, scale, window, keep_first, out_gate):
    from ._lib import AttnDesc
    return AttnDesc(int(heads), int(kv_heads), int(dim), int(vdim), float(scale), int(window), int(keep_first),
                    int(bool(out_gate)))


def stack_kv_store(kcache: torch.Tensor, vcache: torch.Tensor, proj: torch.Tensor, off_k: int, off_v: int,
                   slot: torch.Tensor, pos: torch.Tensor, *, heads, kv_heads, dim, vdim) -> None:
    """Rows pos[t] of slot[t]'s cache ← the k / v segments of proj[t].  kcache [slots, ctx, kv_heads·dim], vcache
    [slots, ctx, kv_heads·vdim]; slot, pos int32 [n_tok]."""
    import ctypes as C
    d = _attn_desc(heads, kv_heads, dim, vdim, 1.0, 0, 0, 0)
    check(lib().b200_stack_kv_store(kcache.data_ptr(), vcache.data_ptr(), kcache.stride(0), vcache.stride(0),
                                    proj.data_ptr(), proj.stride(0), off_k, off_v, slot.data_ptr(), pos.data_ptr(),
                                    proj.shape[0], C.byref(d), _sdt(proj), _stream()), "b200_stack_kv_store")


def stack_attention(proj: torch.Tensor, off_q: int, off_g: int, kcache: torch.Tensor, vcache: torch.Tensor,
                    slot: torch.Tensor, pos: torch.Tensor, *, heads, kv_heads, dim, vdim, scale, window=0, keep_first=0,
                    out_gate=False) -> torch.Tensor:
    """Windowed attention of n_tok query rows (q at columns off_q of proj, gate logits at off_g) over the slots' caches →
    [n_tok, heads·vdim]."""
    import ctypes as C
    d = _attn_desc(heads, kv_heads, dim, vdim, scale, window, keep_first, out_gate)
    out = torch.empty(proj.shape[0], heads * vdim, dtype=proj.dtype, device=proj.device)
    check(lib().b200_stack_attention(out.data_ptr(), out.stride(0), proj.data_ptr(), proj.stride(0), off_q, off_g,
                                     kcache.data_ptr(), vcache.data_ptr(), kcache.stride(0), vcache.stride(0),
                                     slot.data_ptr(), pos.data_ptr(), proj.shape[0], C.byref(d), _sdt(proj), _stream()),
          "b200_stack_attention")
    return out


def stack_act_mul(g: torch.Tensor, u: torch.Tensor, act: str = "gelu_tanh") -> torch.Tensor:
    """T( act(g)·u ) elementwise over [rows, n] (row strides may differ from n: column slices of one projection)."""
    if g.shape != u.shape or g.stride(0) != u.stride(0) or g.stride(1) != 1 or u.stride(1) != 1 or g.dtype != u.dtype:
        raise B200Error("stack_act_mul: g and u must be equally shaped column slices of one row-major matrix")
    y = torch.empty(g.shape, dtype=g.dtype, device=g.device)
    check(lib().b200_stack_act_mul(y.data_ptr(), y.stride(0), g.data_ptr(), u.data_ptr(), g.stride(0), g.shape[0],
                                   g.shape[1], _ACTS[act], _sdt(g), _stream()), "b200_stack_act_mul")
    return y


def stack_act(g: torch.Tensor, act: str = "gelu_erf") -> torch.Tensor:
    """T( act(g) ) elementwise over a row-major [rows, n]."""
    y = torch.empty(g.shape, dtype=g.dtype, device=g.device)
    check(lib().b200_stack_act_mul(y.data_ptr(), y.stride(0), g.data_ptr(), None, g.stride(0), g.shape[0], g.shape[1],
                                   _ACTS[act], _sdt(g), _stream()), "b200_stack_act_mul")
    return y


def stack_rms_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, mult: float) -> torch.Tensor:
    """x += mult · y·rsqrt(mean(y²) + eps)·w, in place on fp32 x [rows, dim]; returns x."""
    x, y, w = (_chk(t, "stack_rms_add", torch.float32) for t in (x, y, w))
    check(lib().b200_stack_rms_add(x.data_ptr(), y.data_ptr(), w.data_ptr(), x.numel() // x.shape[-1], x.shape[-1],
                                   float(eps), float(mult), _stream()), "b200_stack_rms_add")
    return x


# ---- mechanisms of sandwich blocks (csrc/stack_mix.cu)
_NORM_KINDS = {"rms": 0, "layer": 1}


def stack_norm(x: torch.Tensor, w: torch.Tensor, eps: float, kind: str = "layer",
               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out_dtype( norm(x)·w ) for fp32 x [rows, dim]: kind "layer" = (x − mean)·rsqrt(var + eps), "rms" = x·rsqrt(mean(x²) + eps)."""
    x, w = _chk(x, "stack_norm x", torch.float32), _chk(w, "stack_norm w", torch.float32)
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(lib().b200_stack_norm(y.data_ptr(), None, x.data_ptr(), w.data_ptr(), x.numel() // x.shape[-1], x.shape[-1],
                                float(eps), _NORM_KINDS[kind], 0, _sdt(y), _stream()), "b200_stack_norm")
    return y


def stack_norm_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, kind: str = "layer") -> torch.Tensor:
    """x += norm(y)·w in place on fp32 x [rows, dim]; returns x."""
    x, y, w = (_chk(t, "stack_norm_add", torch.float32) for t in (x, y, w))
    check(lib().b200_stack_norm(None, x.data_ptr(), y.data_ptr(), w.data_ptr(), x.numel() // x.shape[-1], x.shape[-1],
                                float(eps), _NORM_KINDS[kind], 1, 1, _stream()), "b200_stack_norm")
    return x


def stack_glu_clamp(gu: torch.Tensor, limit: float) -> torch.Tensor:
    """gu [rows, 2n] = [g | u] → T( min(g, limit)·sigmoid(1.702·min(g, limit))·(clamp(u, ±limit) + 1) ) [rows, n]."""
    gu = _chk(gu, "stack_glu_clamp", gu.dtype)
    n = gu.shape[1] // 2
    y = torch.empty(gu.shape[0], n, dtype=gu.dtype, device=gu.device)
    check(lib().b200_stack_glu_clamp(y.data_ptr(), gu.data_ptr(), gu.shape[0], n, float(limit), _sdt(gu), _stream()),
          "b200_stack_glu_clamp")
    return y


def stack_latent_attention(proj: torch.Tensor, off_down: int, cache: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor, *,
                           heads, dim, rot_dim, vdim, kv_rank, scale, rot_dims, c_norm: torch.Tensor, uk_t: torch.Tensor,
                           uv: torch.Tensor, rot_table: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """Latent attention of n_tok rows of proj = [q | down] over the slots' caches [slots, ctx, kv_rank + rot_dim] (the new
    rows are written first) → [n_tok, heads·vdim].  uk_t [heads, kv_rank, dim], uv [heads·vdim, kv_rank] of proj's dtype."""
    import ctypes as C
    from ._lib import LatentDesc
    a = _attn_desc(heads, 1, dim, vdim, scale, 0, 0, 0)
    l = LatentDesc(int(kv_rank), int(rot_dim), int(rot_dims), c_norm.data_ptr(), uk_t.data_ptr(), None, uv.data_ptr(),
                   _ptr(rot_table))
    out = torch.empty(proj.shape[0], heads * vdim, dtype=proj.dtype, device=proj.device)
    check(lib().b200_stack_latent_attention(out.data_ptr(), out.stride(0), proj.data_ptr(), proj.stride(0), int(off_down),
                                            cache.data_ptr(), cache.stride(0), slot.data_ptr(), pos.data_ptr(), proj.shape[0],
                                            C.byref(a), C.byref(l), float(eps), _sdt(proj), _stream()),
          "b200_stack_latent_attention")
    return out


def stack_mlstm_state(slots: int, heads: int, dim: int, vdim: int, device) -> torch.Tensor:
    """Zeroed fp32 state [slots, floats per slot] of one mLSTM run."""
    return torch.zeros(slots, int(lib().b200_stack_mlstm_state_floats(heads, dim, vdim)), dtype=torch.float32, device=device)


def stack_mlstm(proj: torch.Tensor, off_q: int, off_k: int, off_v: int, gates: torch.Tensor, state: torch.Tensor,
                row0: torch.Tensor, count: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor, *, heads, dim, vdim,
                gate_cap) -> torch.Tensor:
    """mLSTM recurrence over the sequences {row0, count} of proj's rows (slot / pos per row), continuing `state` →
    fp32 [rows, heads, vdim + 2]: numerators, n·q, m."""
    import ctypes as C
    a = _attn_desc(heads, heads, dim, vdim, 1.0, 0, 0, 0)
    gates = _chk(gates, "stack_mlstm gates", torch.float32)
    out = torch.zeros(proj.shape[0], heads, vdim + 2, dtype=torch.float32, device=proj.device)
    check(lib().b200_stack_mlstm(out.data_ptr(), proj.data_ptr(), proj.stride(0), off_q, off_k, off_v, gates.data_ptr(),
                                 state.data_ptr(), state.stride(0), row0.data_ptr(), count.data_ptr(), slot.data_ptr(),
                                 pos.data_ptr(), row0.shape[0], proj.shape[0], C.byref(a), float(gate_cap), _sdt(proj),
                                 _stream()), "b200_stack_mlstm")
    return out


def stack_moe(h: torch.Tensor, router: torch.Tensor, w_exp_in: torch.Tensor, w_exp_out: torch.Tensor, top: int, limit: float = 0.0,
              *, softmax: bool = False, weight_output: bool = False, act: str = "glu_clamp", route_scale: float = 1.0):
    """Routed experts on h [rows, width]: router [E, width], w_exp_in [E, 2·ff, width] (gate | up; [E, ff, width] under a plain
    activation), w_exp_out [E, width, ff] → (y fp32 [rows, width], chosen int32 [rows, top], weights fp32 [rows, top]).
    softmax: softmax scores with the chosen ones renormalised and scaled (else sigmoid scores); weight_output: the weight
    multiplies the expert's output (else its input)."""
    import ctypes as C
    from ._lib import MoeDesc
    h = _chk(h, "stack_moe h", h.dtype)
    E, ff2, W = w_exp_in.shape
    plain = act != "glu_clamp"
    m = MoeDesc(E, int(top), ff2 if plain else ff2 // 2, 0, float(limit), 0.0, router.data_ptr(), w_exp_in.data_ptr(),
                w_exp_out.data_ptr(), int(softmax), int(weight_output), _ACTS[act] if plain else 0, 1, float(route_scale))
    y = torch.empty(h.shape[0], W, dtype=torch.float32, device=h.device)
    chosen = torch.empty(h.shape[0], top, dtype=torch.int32, device=h.device)
    scores = torch.empty(h.shape[0], top, dtype=torch.float32, device=h.device)
    check(lib().b200_stack_moe(y.data_ptr(), h.data_ptr(), h.shape[0], W, C.byref(m), chosen.data_ptr(), scores.data_ptr(),
                               _sdt(h), _stream()), "b200_stack_moe")
    return y, chosen, scores


# ---- mechanisms of post-norm blocks (csrc/stack_rec.cu)
def stack_attn_prep(proj: torch.Tensor, off_q: int, off_k: int, off_v: int, pos: torch.Tensor, *, heads, kv_heads, dim, vdim,
                    eps: float, q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None,
                    rot_table: Optional[torch.Tensor] = None, v_norm: bool = False, v_mix: int = 0,
                    vkeep: Optional[torch.Tensor] = None, mix_lambda: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The preparation of an attention mixer's q | k | v rows, IN PLACE in proj [n_tok, ·] (returned): whole-projection RMS
    norms with weights (q_norm / k_norm given), rotate-half rotary positions on the first 2·rot_table.shape[1] entries of
    every head (rot_table fp32 [ctx, dims/2, 2]), unit-rms values, value mix-in (v_mix 1 fills vkeep, 2 blends with it)."""
    import ctypes as C
    from ._lib import AttnPrepDesc
    a = _attn_desc(heads, kv_heads, dim, vdim, 1.0, 0, 0, 0)
    d = AttnPrepDesc(int(q_norm is not None), 2 * rot_table.shape[1] if rot_table is not None else 0, int(v_norm), int(v_mix),
                     _ptr(q_norm), _ptr(k_norm), _ptr(rot_table), _ptr(mix_lambda))
    check(lib().b200_stack_attn_prep(proj.data_ptr(), proj.stride(0), off_q, off_k, off_v, pos.data_ptr(), proj.shape[0],
                                     C.byref(a), C.byref(d), _ptr(vkeep), vkeep.stride(0) if vkeep is not None else 0, float(eps),
                                     _sdt(proj), _stream()), "b200_stack_attn_prep")
    return proj


def stack_lin_scan(d: torch.Tensor, b: torch.Tensor, r: torch.Tensor, v: torch.Tensor, state: torch.Tensor, row0: torch.Tensor,
                   count: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor, *, heads, dk, dv, p: Optional[torch.Tensor] = None,
                   q: Optional[torch.Tensor] = None, vscale: Optional[torch.Tensor] = None, share: int = 1) -> torch.Tensor:
    """The linear recurrence S ← diag(d) S − p (qᵀS) + b (v·vscale)ᵀ, o = Sᵀr over the sequences {row0, count} of the operands'
    rows (all fp32 [rows, ·] with ONE common row stride: column slices of one matrix; slot / pos per row), continuing `state`
    [slots, heads·dk·dv] → fp32 [rows, heads·dv].  d [rows, heads·dk], or [rows, heads] (one decay per head)."""
    rows = v.shape[0]
    ld = v.stride(0)
    for t in (d, b, r, p, q, vscale):
        if t is not None and (t.dtype != torch.float32 or t.stride(0) != ld or t.stride(1) != 1):
            raise B200Error("stack_lin_scan: operands must be fp32 column slices of one row-major matrix")
    out = torch.zeros(rows, heads * dv, dtype=torch.float32, device=v.device)
    check(lib().b200_stack_lin_scan(out.data_ptr(), d.data_ptr(), _ptr(p), _ptr(q), b.data_ptr(), r.data_ptr(), v.data_ptr(),
                                    _ptr(vscale), ld, heads, dk, dv, share, int(d.shape[1] == heads and dk != 1), state.data_ptr(),
                                    state.stride(0), row0.data_ptr(), count.data_ptr(), slot.data_ptr(), pos.data_ptr(),
                                    row0.shape[0], rows, _stream()), "b200_stack_lin_scan")
    return out
