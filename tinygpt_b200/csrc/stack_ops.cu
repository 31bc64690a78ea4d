// stack_ops.cu — the layer-stack engine's mechanisms as plain kernels: any shape, storage type T = bf16 or fp32, fp32
// arithmetic for norms, softmax, gates and everything that touches the residual stream.  These are the kernels every
// shape can fall back on; the tensor-core GEMM (gemm.cu) and the weight-streaming GEMV (gemv.cu) take over the matrix
// products whose shapes they accept (engine_stack.cu decides per product).
#include "stack.cuh"

namespace b200 {

// Every kernel of this file starts with griddepcontrol.launch_dependents + griddepcontrol.wait, so it may be launched
// ahead of the end of its predecessor (programmatic dependent launch): the launch latency hides behind the predecessor's
// tail and nothing is read or written before the predecessor's results are complete.  B200_NO_PDL=1 turns it off.
bool stack_pdl() {
  static const bool on = !env_flag("B200_NO_PDL", false);
  return on;
}

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ T cvt(float v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
// the value a T-typed operand carries when its source is fp32
template <typename T> __device__ __forceinline__ float as_operand(float v);
template <> __device__ __forceinline__ float as_operand<float>(float v) { return v; }
template <> __device__ __forceinline__ float as_operand<__nv_bfloat16>(float v) { return round_bf16(v); }

__device__ __forceinline__ float gelu_tanh(float z) {
  const float c = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * z * (1.f + tanhf(c * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  __syncthreads();
  return tot;
}

// ------------------------------------------------------------------------------------------------------- general GEMM
// 64 × 64 output tile per CTA, 16-wide k slices through shared memory (as fp32), 4 × 4 outputs per thread, fp32 FMA.
// bf16 × bf16 products are exact in fp32, so T = bf16 gives "bf16 operands, fp32 accumulation"; T = fp32 is a true fp32
// product (no reduced-precision matrix mode).
constexpr int kBM = 64, kBN = 64, kBK = 16;

template <typename T>
__global__ void __launch_bounds__(256) stack_gemm_kernel(const StackGemm g) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[kBK][kBM + 4];
  __shared__ float Ws[kBK][kBN + 4];
  // which rows and which operands this CTA serves: a plain tile, a tile of batch item blockIdx.z (operands moved by
  // sa / sw / sc elements per item), or tile blockIdx.y of a grouped product (rows of group e meet matrix e)
  int m0 = blockIdx.y * kBM, m_end = g.M;
  int64_t za = 0, zw = 0, zc = 0;
  if (g.tile_group != nullptr) {
    const int e = g.tile_group[blockIdx.y];
    if (e < 0) return;
    m0 = g.tile_row0[blockIdx.y];
    m_end = min(m0 + kBM, g.group_end[e]);
    zw = (int64_t)e * g.sw;
  } else {
    za = (int64_t)blockIdx.z * g.sa;
    zw = (int64_t)blockIdx.z * g.sw;
    zc = (int64_t)blockIdx.z * g.sc;
  }
  const int n0 = blockIdx.x * kBN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const T* W = static_cast<const T*>(g.w) + zw;
  for (int k0 = 0; k0 < g.K; k0 += kBK) {
    for (int e = threadIdx.x; e < kBM * kBK; e += 256) {
      const int r = e / kBK, c = e % kBK;
      const int m = m0 + r, k = k0 + c;
      float v = 0.f;
      if (m < m_end && k < g.K) {
        const bool first = k < g.k1;
        const void* src = first ? g.a : g.a2;
        const int64_t idx = first ? (int64_t)m * g.lda + k + za : (int64_t)m * g.lda2 + (k - g.k1);
        v = g.a_f32 ? as_operand<T>(static_cast<const float*>(src)[idx]) : ldf<T>(static_cast<const T*>(src) + idx);
      }
      As[c][r] = v;
      const int n = n0 + r;
      Ws[c][r] = (n < g.N && k < g.K) ? ldf<T>(W + (int64_t)n * g.K + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kBK; ++c) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.bias != nullptr) v += g.bias[n];
      const int64_t o = (int64_t)m * g.ldc + n + zc;
      switch (g.epi) {
        case SEPI_STORE: static_cast<T*>(g.c)[o] = cvt<T>(v); break;
        case SEPI_STORE_F32: static_cast<float*>(g.c)[o] = v; break;
        case SEPI_RESIDUAL: static_cast<float*>(g.c)[o] += g.mult * v; break;
        case SEPI_ACT_TABLE: {
          const float e = ldf<T>(static_cast<const T*>(g.table) + (int64_t)g.tok[m] * g.table_ld + g.table_col + n);
          static_cast<T*>(g.c)[o] = cvt<T>(gelu_tanh(v) * e);
          break;
        }
        default:
          if (g.softcap > 0.f) v = g.softcap * tanhf(v / g.softcap);
          static_cast<float*>(g.c)[o] = v;
          if (g.c2 != nullptr) g.c2[o] = __float2bfloat16_rn(v);
      }
    }
  }
}

// --------------------------------------------------------------------------------------------------------------- norms
template <typename T>
__global__ void __launch_bounds__(256) stack_rmsnorm_kernel(T* __restrict__ y, const float* __restrict__ x,
                                                            const float* __restrict__ w, const int32_t* __restrict__ rows,
                                                            int dim, float eps, float offset) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int64_t src = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) ss += xr[i] * xr[i];
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)dim + eps);
  T* yr = y + (int64_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) yr[i] = cvt<T>(xr[i] * inv * (offset + w[i]));
}

template <typename YT>
__global__ void __launch_bounds__(256) stack_rms_add_kernel(float* __restrict__ x, const YT* __restrict__ y,
                                                            const float* __restrict__ w, int dim, float eps, float mult) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const YT* yr = y + (int64_t)blockIdx.x * dim;
  float* xr = x + (int64_t)blockIdx.x * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) ss += ldf<YT>(yr + i) * ldf<YT>(yr + i);
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) xr[i] += mult * (ldf<YT>(yr + i) * inv * w[i]);
}

// The same for a few rows that fit the CTA's registers (decode steps, where latency counts): y, w and x are requested
// together — one memory round trip before the reduction instead of three.  dim <= 16 · 256.
template <typename YT>
__global__ void __launch_bounds__(256) stack_rms_add_small_kernel(float* __restrict__ x, const YT* __restrict__ y,
                                                                  const float* __restrict__ w, int dim, float eps,
                                                                  float mult) {
  __shared__ float red[8];
  pdl_trigger();
  pdl_wait();
  const YT* yr = y + (int64_t)blockIdx.x * dim;
  float* xr = x + (int64_t)blockIdx.x * dim;
  float yv[16], wv[16], xv[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const int i = threadIdx.x + k * 256;
    yv[k] = i < dim ? ldf<YT>(yr + i) : 0.f;
    wv[k] = i < dim ? w[i] : 0.f;
    xv[k] = i < dim ? xr[i] : 0.f;
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 16; ++k) ss += yv[k] * yv[k];
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < dim) xr[i] = xv[k] + mult * (yv[k] * inv * wv[k]);
  }
}

__global__ void __launch_bounds__(256) stack_cast_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ x,
                                                         int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x)
    y[e] = __float2bfloat16_rn(x[e]);
}
// y[r, j] = bf16( gelu_tanh(g[r, j]) · table[tok[r]·table_ld + col + j] )
__global__ void __launch_bounds__(256) stack_act_table_kernel(__nv_bfloat16* __restrict__ y,
                                                              const __nv_bfloat16* __restrict__ g,
                                                              const __nv_bfloat16* __restrict__ table,
                                                              const int32_t* __restrict__ tok, int64_t table_ld, int col,
                                                              int n, int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / n;
    const int j = (int)(e % n);
    y[e] = __float2bfloat16_rn(gelu_tanh(__bfloat162float(g[e])) * __bfloat162float(table[(int64_t)tok[r] * table_ld + col + j]));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) stack_act_mul_kernel(T* __restrict__ y, int64_t ld_y, const T* __restrict__ g,
                                                            const T* __restrict__ u, int64_t ld_gu, int n, int act,
                                                            int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / n;
    const int j = (int)(e % n);
    const float gv = ldf<T>(g + r * ld_gu + j);
    const float av = act == B200_ACT_SILU ? silu(gv)
                     : act == B200_ACT_GELU_ERF ? 0.5f * gv * (1.f + erff(gv * 0.70710678118654752f))
                     : act == B200_ACT_RELU2 ? fmaxf(gv, 0.f) * fmaxf(gv, 0.f)
                     : act == B200_ACT_TANH ? tanhf(gv) : gelu_tanh(gv);
    if (u == nullptr) {   // the activation alone
      y[r * ld_y + j] = cvt<T>(av);
      continue;
    }
    // the activation is a value of type T before it meets the other factor
    y[r * ld_y + j] = cvt<T>(as_operand<T>(av) * ldf<T>(u + r * ld_gu + j));
  }
}

template <typename T>
__global__ void __launch_bounds__(128) stack_embed_kernel(float* __restrict__ x, float* __restrict__ x0,
                                                          const T* __restrict__ embed, const int32_t* __restrict__ tok,
                                                          int vocab, int width, float scale) {
  pdl_trigger();
  pdl_wait();
  int id = tok[blockIdx.x];
  if (id < 0 || id >= vocab) id = 0;
  const T* row = embed + (int64_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = ldf<T>(row + i) * scale;
    x[(int64_t)blockIdx.x * width + i] = v;
    x0[(int64_t)blockIdx.x * width + i] = v;
  }
}

// ----------------------------------------------------------------------------------------------------------- attention
template <typename T>
__global__ void __launch_bounds__(128) stack_kv_store_kernel(const StackAttn p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int nk = p.a.kv_heads * p.a.dim, nv = p.a.kv_heads * p.a.vdim;
  const T* row = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj;
  T* kd = static_cast<T*>(p.kcache) + (int64_t)p.slot[t] * p.k_slot_stride + (int64_t)p.pos[t] * nk;
  T* vd = static_cast<T*>(p.vcache) + (int64_t)p.slot[t] * p.v_slot_stride + (int64_t)p.pos[t] * nv;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) kd[i] = row[p.off_k + i];
  for (int i = threadIdx.x; i < nv; i += blockDim.x) vd[i] = row[p.off_v + i];
}

// One warp merges the key splits' partial softmaxes {max, sum, weighted values} of a (token, head) pair, applies the
// gate and stores the head's output.  Run by the CTA that finishes a pair last (ticket), so it reads through L2.
template <typename T>
__device__ __forceinline__ void stack_attn_merge_pair(const StackAttn& p, int64_t pair, int t, int h, int lane) {
  const int vdim = p.a.vdim;
  const float* base = p.split_ws + (size_t)pair * p.nsplit * (2 + vdim);
  // lanes over splits (nsplit <= 64: two per lane) for the maxima and the sums …
  const int s0 = lane, s1 = lane + 32;
  const float m0 = s0 < p.nsplit ? __ldcg(base + (size_t)s0 * (2 + vdim)) : -INFINITY;
  const float m1 = s1 < p.nsplit ? __ldcg(base + (size_t)s1 * (2 + vdim)) : -INFINITY;
  const float l0 = s0 < p.nsplit ? __ldcg(base + (size_t)s0 * (2 + vdim) + 1) : 0.f;
  const float l1 = s1 < p.nsplit ? __ldcg(base + (size_t)s1 * (2 + vdim) + 1) : 0.f;
  const float mt = warp_max(fmaxf(m0, m1));
  const float f0 = m0 == -INFINITY ? 0.f : expf(m0 - mt), f1 = m1 == -INFINITY ? 0.f : expf(m1 - mt);
  float l = warp_sum(l0 * f0 + l1 * f1);
  if (p.a.sink) l += expf(-mt);   // the sink: a key of score 0 that has no value
  const T* prow = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj;
  float gate = 1.f;
  if (p.a.out_gate) gate = 1.f / (1.f + expf(-ldf<T>(prow + p.off_g + h)));
  const float fin = gate / l;
  T* orow = static_cast<T*>(p.out) + (int64_t)t * p.ld_out + (int64_t)h * vdim;
  // … then lanes over value columns, the splits' weights handed round by shuffle (independent loads per split)
  for (int d0 = 0; d0 < vdim; d0 += 32) {
    const int d = d0 + lane;
    float a = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const float f = __shfl_sync(0xffffffffu, s < 32 ? f0 : f1, s & 31);
      // (an empty split holds zeros: no guard, so the loads do not wait for the weights)
      if (d < vdim) a = fmaf(__ldcg(base + (size_t)s * (2 + vdim) + 2 + d), f, a);
    }
    if (d < vdim) orow[d] = cvt<T>(a * fin);
  }
}

// NW warps per (token, query head); NW = 1: four pairs per CTA (prompts: pairs abound), NW = 4: one pair per CTA, its keys
// dealt to the warps 32 at a time and the partial softmaxes merged through shared memory (decode steps: few pairs, long
// key lists).  The visible keys of a query at position i are the kept first rows [0, min(keep_first, lo)) followed by
// the window [lo, i], lo = max(0, i − window + 1) (window 0: lo = 0).  A warp walks its share of that list 32 keys at a
// time: lane j scores key j (fp32 dot, times scale), the chunk joins an online softmax, then the lanes turn to the value
// columns and add the chunk's weighted rows: column lane + 32·r of one row at a time, or — VEC: bf16, key size a multiple
// of 8, value size 8 … 256 and a power of two — 16-byte loads throughout, vdim/8 lanes per value row and 256/vdim rows
// per pass (the groups' sums meet in a butterfly after the walk).
template <typename T, int VR, int NW, bool VEC>
__global__ void __launch_bounds__(128) stack_attn_kernel(const StackAttn p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem_f[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wi = warp % NW;
  const int64_t pair = (int64_t)blockIdx.x * (4 / NW) + warp / NW;
  const int t = (int)(pair / p.a.heads), h = (int)(pair % p.a.heads);
  if (t >= p.n_tok) return;   // NW = 4: the whole CTA leaves together
  const int dim = p.a.dim, vdim = p.a.vdim;
  float* qs = smem_f + warp * dim;
  const T* prow = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj;
  for (int d = lane; d < dim; d += 32) qs[d] = ldf<T>(prow + p.off_q + h * dim + d);
  __syncwarp();
  const int slot = p.slot[t], i = p.pos[t];
  const int kvh = h / (p.a.heads / p.a.kv_heads);
  const int64_t krs = (int64_t)p.a.kv_heads * dim, vrs = (int64_t)p.a.kv_heads * vdim;
  const T* kb = static_cast<const T*>(p.kcache) + (int64_t)slot * p.k_slot_stride + kvh * dim;
  const T* vb = static_cast<const T*>(p.vcache) + (int64_t)slot * p.v_slot_stride + kvh * vdim;
  const int lo = p.a.window > 0 ? max(0, i - p.a.window + 1) : 0;
  const int na = min(p.a.keep_first, lo);
  const int total = na + (i - lo + 1);
  // this CTA's share of the visible list (all of it unless the keys are split over blockIdx.y)
  const bool split = NW > 1 && p.split_ws != nullptr;
  // the row's own key / value: from proj when the launch also appends them (own_from_proj), else already in the cache
  const T* own_k = prow + p.off_k + kvh * dim;
  const T* own_v = prow + p.off_v + kvh * vdim;
  if (p.own_from_proj && wi == 0 && blockIdx.y == 0 && h % (p.a.heads / p.a.kv_heads) == 0) {
    T* kd = static_cast<T*>(p.kcache) + (int64_t)slot * p.k_slot_stride + (int64_t)i * krs + kvh * dim;
    T* vd = static_cast<T*>(p.vcache) + (int64_t)slot * p.v_slot_stride + (int64_t)i * vrs + kvh * vdim;
    for (int d = lane; d < dim; d += 32) kd[d] = own_k[d];
    for (int d = lane; d < vdim; d += 32) vd[d] = own_v[d];
  }
  const int begin = split ? (int)blockIdx.y * p.keys_per_split : 0;
  const int end = split ? min(total, begin + p.keys_per_split) : total;
  constexpr int NA = VEC ? 8 : VR;
  float m = -INFINITY, l = 0.f, acc[NA];
#pragma unroll
  for (int r = 0; r < NA; ++r) acc[r] = 0.f;
  // the value columns a lane owns once the walk is over, as fn(column, accumulator)
  auto cols = [&](auto&& fn) {
    if constexpr (VEC) {
      if (lane < (vdim >> 3)) {
#pragma unroll
        for (int e = 0; e < 8; ++e) fn(lane * 8 + e, acc[e]);
      }
    } else {
#pragma unroll
      for (int r = 0; r < VR; ++r) {
        const int d = lane + 32 * r;
        if (d < vdim) fn(d, acc[r]);
      }
    }
  };
  for (int c0 = begin + wi * 32; c0 < end; c0 += NW * 32) {
    const int idx = c0 + lane;
    const bool valid = idx < end;
    const int j = idx < na ? idx : lo + (idx - na);
    float s = -INFINITY;
    if (valid) {
      const T* kr = (p.own_from_proj && j == i) ? own_k : kb + (int64_t)j * krs;
      float dot = 0.f;
      if constexpr (VEC) {
        // eight 16-byte pieces of the key row are requested together, then consumed: the row costs dim/64 memory
        // round trips instead of dim/8
        const uint4* k4 = reinterpret_cast<const uint4*>(kr);
        const int nd8 = dim >> 3;
        for (int d0 = 0; d0 < nd8; d0 += 8) {
          uint4 kq[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) kq[u] = d0 + u < nd8 ? k4[d0 + u] : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (d0 + u < nd8) {
              float kf[8];
              unpack8(kq[u], kf);
#pragma unroll
              for (int e = 0; e < 8; ++e) dot = fmaf(qs[(d0 + u) * 8 + e], kf[e], dot);
            }
          }
        }
      } else {
        for (int d = 0; d < dim; ++d) dot = fmaf(qs[d], ldf<T>(kr + d), dot);
      }
      s = dot * p.a.scale;
    }
    const float mn = fmaxf(m, warp_max(s));
    const float corr = m == -INFINITY ? 0.f : expf(m - mn);
    const float pj = valid ? expf(s - mn) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int r = 0; r < NA; ++r) acc[r] *= corr;
    const int cn = min(32, end - c0);
    if constexpr (VEC) {
      const int G = vdim >> 3, KP = 32 / G;   // lanes per value row, rows per pass
      const int grp = lane / G, gl = lane % G;
      // eight passes' value pieces are requested together, then consumed (as for the key rows)
      for (int jj0 = 0; jj0 < cn; jj0 += 8 * KP) {
        uint4 vq[8];
        float pw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int src = jj0 + u * KP + grp;   // key of this lane's row group in pass u
          pw[u] = __shfl_sync(0xffffffffu, pj, src & 31);
          const int jr = __shfl_sync(0xffffffffu, j, src & 31);
          vq[u] = make_uint4(0, 0, 0, 0);
          if (src < cn) {
            const T* vr = (p.own_from_proj && jr == i) ? own_v : vb + (int64_t)jr * vrs;
            vq[u] = *reinterpret_cast<const uint4*>(vr + gl * 8);
          } else {
            pw[u] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float vf[8];
          unpack8(vq[u], vf);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(pw[u], vf[e], acc[e]);
        }
      }
    } else {
      for (int jj = 0; jj < cn; ++jj) {
        const float pw = __shfl_sync(0xffffffffu, pj, jj);
        const int jr = __shfl_sync(0xffffffffu, j, jj);
        const T* vr = (p.own_from_proj && jr == i) ? own_v : vb + (int64_t)jr * vrs;
#pragma unroll
        for (int r = 0; r < VR; ++r) {
          const int d = lane + 32 * r;
          if (d < vdim) acc[r] = fmaf(pw, ldf<T>(vr + d), acc[r]);
        }
      }
    }
    m = mn;
  }
  if constexpr (VEC) {   // the row groups' partial sums of a column meet
    for (int off = vdim >> 3; off < 32; off <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
    }
  }
  if constexpr (NW > 1) {
    // merge the warps' partial softmaxes: scratch [NW][2 + vdim] behind the four query vectors
    float* sc = smem_f + 4 * dim;
    float* mine = sc + wi * (2 + vdim);
    if (lane == 0) {
      mine[0] = m;
      mine[1] = l;
    }
    cols([&](int d, float& a) { mine[2 + d] = a; });
    __syncthreads();
    if (wi != 0) return;
    float mt = -INFINITY;
    for (int w = 0; w < NW; ++w) mt = fmaxf(mt, sc[w * (2 + vdim)]);
    m = mt;
    l = 0.f;
#pragma unroll
    for (int r = 0; r < NA; ++r) acc[r] = 0.f;
    for (int w = 0; w < NW; ++w) {
      const float* o = sc + w * (2 + vdim);
      const float f = o[0] == -INFINITY ? 0.f : expf(o[0] - mt);
      l += o[1] * f;
      cols([&](int d, float& a) { a += o[2 + d] * f; });
    }
    if (split) {   // partial of this split: {max, sum, weighted values}; stack_attn_merge_kernel finishes the pair
      float* o = p.split_ws + ((size_t)pair * p.nsplit + blockIdx.y) * (2 + vdim);
      if (lane == 0) {
        o[0] = mt;
        o[1] = l;
      }
      cols([&](int d, float& a) { o[2 + d] = a; });
      // the CTA that hands in a pair's last partial merges them (tickets start at zero and reset themselves)
      __threadfence();
      __syncwarp();
      unsigned int tk = 0;
      if (lane == 0) tk = atomicAdd(p.split_tickets + pair, 1u);
      tk = __shfl_sync(0xffffffffu, tk, 0);
      if (tk != (unsigned int)p.nsplit - 1u) return;
      if (lane == 0) p.split_tickets[pair] = 0;
      __threadfence();
      stack_attn_merge_pair<T>(p, pair, t, h, lane);
      return;
    }
  }
  float gate = 1.f;
  if (p.a.out_gate) gate = 1.f / (1.f + expf(-ldf<T>(prow + p.off_g + h)));
  T* orow = static_cast<T*>(p.out) + (int64_t)t * p.ld_out + (int64_t)h * vdim;
  if (p.a.sink) l += expf(-m);   // the sink: a key of score 0 that has no value
  const float fin = gate / l;
  cols([&](int d, float& a) { orow[d] = cvt<T>(a * fin); });
}

// Decode-shaped steps (every row its sequence's only new row) of bf16 engines with key size <= 128 and value size 64 or
// 128: one CTA per (row, head, split of 128 visible keys), warp w takes keys 32w … of the split, ONE key per lane.
// The cached rows a lane needs — its key's 16-byte pieces and its row group's value pieces — are requested BEFORE the
// programmatic-dependency wait: they were written by earlier steps, and the row's slot and position by the step's
// first kernel, so all of it is stable while the projection that produces q still runs.  After the wait: q, the row's
// own key / value from proj (appended to the cache by one CTA per KV head), scores, one softmax per warp, values, the
// four warps merged through shared memory, the splits by ticket (stack_attn_merge_pair).
__global__ void __launch_bounds__(128) stack_attn_decode_kernel(const StackAttn p) {
  using T = __nv_bfloat16;
  extern __shared__ float smem_f[];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t pair = blockIdx.x;
  const int t = (int)(pair / p.a.heads), h = (int)(pair % p.a.heads);
  const int dim = p.a.dim, vdim = p.a.vdim, nd8 = dim >> 3;
  const int G = vdim >> 3, KP = 32 / G;       // lanes per value row, value rows per pass; G passes cover 32 keys
  const int grp = lane / G, gl = lane % G;
  const int slot = p.slot[t], i = p.pos[t];
  const int kvh = h / (p.a.heads / p.a.kv_heads);
  const int64_t krs = (int64_t)p.a.kv_heads * dim, vrs = (int64_t)p.a.kv_heads * vdim;
  const T* kb = static_cast<const T*>(p.kcache) + (int64_t)slot * p.k_slot_stride + kvh * dim;
  const T* vb = static_cast<const T*>(p.vcache) + (int64_t)slot * p.v_slot_stride + kvh * vdim;
  const int lo = p.a.window > 0 ? max(0, i - p.a.window + 1) : 0;
  const int na = min(p.a.keep_first, lo);
  const int total = na + (i - lo + 1);
  const int begin = (int)blockIdx.y * p.keys_per_split;
  const int end = min(total, begin + p.keys_per_split);
  const int c0 = begin + warp * 32;            // keys_per_split <= 128: one chunk per warp
  const int idx = c0 + lane;
  const bool valid = idx < end;
  const int j = idx < na ? idx : lo + (idx - na);
  const int cn = max(0, min(32, end - c0));
  // ---- cached rows, ahead of the wait
  uint4 kq[16], vq[16];
  int vj[16];
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    kq[u] = make_uint4(0, 0, 0, 0);
    if (valid && j != i && u < nd8) kq[u] = reinterpret_cast<const uint4*>(kb + (int64_t)j * krs)[u];
  }
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int src = u * KP + grp;              // key (within the chunk) of this lane's row group in pass u
    vj[u] = __shfl_sync(0xffffffffu, j, src & 31);
    vq[u] = make_uint4(0, 0, 0, 0);
    if (u < G && src < cn && vj[u] != i) vq[u] = *reinterpret_cast<const uint4*>(vb + (int64_t)vj[u] * vrs + gl * 8);
  }
  pdl_wait();
  // ---- what this step produced: q, the gate logit, the row's own key and value
  float* qs = smem_f;                          // [dim], shared by the four warps
  const T* prow = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj;
  for (int d = threadIdx.x; d < dim; d += 128) qs[d] = __bfloat162float(prow[p.off_q + h * dim + d]);
  const T* own_k = prow + p.off_k + kvh * dim;
  const T* own_v = prow + p.off_v + kvh * vdim;
  if (valid && j == i) {
#pragma unroll
    for (int u = 0; u < 16; ++u)
      if (u < nd8) kq[u] = reinterpret_cast<const uint4*>(own_k)[u];
  }
#pragma unroll
  for (int u = 0; u < 16; ++u)
    if (u < G && u * KP + grp < cn && vj[u] == i) vq[u] = *reinterpret_cast<const uint4*>(own_v + gl * 8);
  if (warp == 0 && blockIdx.y == 0 && h % (p.a.heads / p.a.kv_heads) == 0) {
    T* kd = static_cast<T*>(p.kcache) + (int64_t)slot * p.k_slot_stride + (int64_t)i * krs + kvh * dim;
    T* vd = static_cast<T*>(p.vcache) + (int64_t)slot * p.v_slot_stride + (int64_t)i * vrs + kvh * vdim;
    for (int d = lane; d < dim; d += 32) kd[d] = own_k[d];
    for (int d = lane; d < vdim; d += 32) vd[d] = own_v[d];
  }
  __syncthreads();
  // ---- scores and the warp's softmax
  float dot = 0.f;
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    if (u < nd8) {
      float kf[8];
      unpack8(kq[u], kf);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot = fmaf(qs[u * 8 + e], kf[e], dot);
    }
  }
  const float sc_ = valid ? dot * p.a.scale : -INFINITY;
  const float m = warp_max(sc_);
  const float pj = valid ? expf(sc_ - m) : 0.f;
  const float l = warp_sum(pj);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int src = u * KP + grp;
    const float pw = __shfl_sync(0xffffffffu, pj, src & 31);
    if (u < G && src < cn) {
      float vf[8];
      unpack8(vq[u], vf);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(pw, vf[e], acc[e]);
    }
  }
  for (int off = G; off < 32; off <<= 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
  }
  // ---- the four warps, then the splits
  float* sc = smem_f + dim;                    // [4][2 + vdim]
  float* mine = sc + warp * (2 + vdim);
  if (lane == 0) {
    mine[0] = m;
    mine[1] = l;
  }
  if (lane < G) {
#pragma unroll
    for (int e = 0; e < 8; ++e) mine[2 + lane * 8 + e] = acc[e];
  }
  __syncthreads();
  if (warp != 0) return;
  float mt = -INFINITY;
  for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sc[w * (2 + vdim)]);
  float lt = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int w = 0; w < 4; ++w) {
    const float* o = sc + w * (2 + vdim);
    const float f = o[0] == -INFINITY ? 0.f : expf(o[0] - mt);
    lt += o[1] * f;
    if (lane < G) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += o[2 + lane * 8 + e] * f;
    }
  }
  float* o = p.split_ws + ((size_t)pair * p.nsplit + blockIdx.y) * (2 + vdim);
  if (lane == 0) {
    o[0] = mt;
    o[1] = lt;
  }
  if (lane < G) {
#pragma unroll
    for (int e = 0; e < 8; ++e) o[2 + lane * 8 + e] = acc[e];
  }
  __threadfence();
  __syncwarp();
  unsigned int tk = 0;
  if (lane == 0) tk = atomicAdd(p.split_tickets + pair, 1u);
  tk = __shfl_sync(0xffffffffu, tk, 0);
  if (tk != (unsigned int)p.nsplit - 1u) return;
  if (lane == 0) p.split_tickets[pair] = 0;
  __threadfence();
  stack_attn_merge_pair<T>(p, pair, t, h, lane);
}

__global__ void __launch_bounds__(256) stack_bias_add_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ b,
                                                             int n, int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x)
    y[e] = __float2bfloat16_rn(__bfloat162float(y[e]) + b[e % n]);
}
__global__ void __launch_bounds__(256) stack_axpy_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ t,
                                                         float mult, int add, int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x)
    x[e] = (add ? x[e] : 0.f) + mult * __bfloat162float(t[e]);
}
__global__ void __launch_bounds__(256) stack_cat_cast_kernel(__nv_bfloat16* __restrict__ cat, const float* __restrict__ a,
                                                             const float* __restrict__ b, float* __restrict__ zero,
                                                             int width, int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / width;
    const int j = (int)(e % width);
    cat[r * 2 * width + j] = __float2bfloat16_rn(a[e]);
    cat[r * 2 * width + width + j] = __float2bfloat16_rn(b[e]);
    if (zero != nullptr) zero[e] = 0.f;
  }
}

inline int grid_cap(int64_t n, int block) {
  int64_t g = (n + block - 1) / block;
  return (int)std::max<int64_t>(1, std::min<int64_t>(g, 148 * 16));
}

}  // namespace

#define STACK_DTYPE_CHECK(dtype) \
  B200_CHECK_ARG((dtype) == B200_BF16 || (dtype) == B200_F32, "stack op: unknown dtype %d", (int)(dtype))

int launch_stack_gemm(const StackGemm& g, int dtype, cudaStream_t st) {
  STACK_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(g.a && g.w && g.c && g.M > 0 && g.N > 0 && g.K > 0, "stack gemm: bad arguments M=%d N=%d K=%d", g.M, g.N,
                 g.K);
  B200_CHECK_ARG(g.k1 == g.K || g.a2 != nullptr, "stack gemm: second operand source missing");
  B200_CHECK_ARG(g.epi != SEPI_ACT_TABLE || (g.table && g.tok), "stack gemm: table epilogue without a table");
  B200_CHECK_ARG(g.batch >= 1 && (g.batch == 1 || g.a2 == nullptr), "stack gemm: bad batch");
  B200_CHECK_ARG(g.tile_group == nullptr || (g.tile_row0 && g.group_end && g.n_tiles > 0 && g.batch == 1),
                 "stack gemm: incomplete grouping");
  const dim3 grid((g.N + kBN - 1) / kBN, g.tile_group ? g.n_tiles : (g.M + kBM - 1) / kBM, g.batch);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(stack_gemm_kernel<float>, grid, dim3(256), 0, st, stack_pdl(), g));
  else B200_CUDA(launch_pdl(stack_gemm_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, stack_pdl(), g));
  return B200_OK;
}

int launch_stack_rmsnorm(void* y, const float* x, const float* w, const int32_t* rows, int64_t n_rows, int dim, float eps,
                         float offset, int dtype, cudaStream_t st) {
  STACK_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(y && x && w && n_rows > 0 && dim > 0, "stack rmsnorm: bad arguments");
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_rmsnorm_kernel<float>, dim3((unsigned)n_rows), dim3(256), 0, st, stack_pdl(), (float*)y, x, w, rows,
                         dim, eps, offset));
  else
    B200_CUDA(launch_pdl(stack_rmsnorm_kernel<__nv_bfloat16>, dim3((unsigned)n_rows), dim3(256), 0, st, stack_pdl(),
                         (__nv_bfloat16*)y, x, w, rows, dim, eps, offset));
  return B200_OK;
}

int launch_stack_rms_add(float* x, const float* y, const float* w, int64_t rows, int dim, float eps, float mult,
                         cudaStream_t st) {
  B200_CHECK_ARG(x && y && w && rows > 0 && dim > 0, "stack rms_add: bad arguments");
  if (rows <= 64 && dim <= 16 * 256)
    B200_CUDA(launch_pdl(stack_rms_add_small_kernel<float>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x, y, w, dim,
                         eps, mult));
  else
    B200_CUDA(launch_pdl(stack_rms_add_kernel<float>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x, y, w, dim, eps,
                         mult));
  return B200_OK;
}

int launch_stack_rms_add_bf16(float* x, const __nv_bfloat16* y, const float* w, int64_t rows, int dim, float eps, float mult,
                              cudaStream_t st) {
  B200_CHECK_ARG(x && y && w && rows > 0 && dim > 0, "stack rms_add: bad arguments");
  B200_CUDA(launch_pdl(stack_rms_add_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x, y, w, dim, eps,
                       mult));
  return B200_OK;
}

int launch_stack_cast(__nv_bfloat16* y, const float* x, int64_t total, cudaStream_t st) {
  B200_CHECK_ARG(y && x && total > 0, "stack cast: bad arguments");
  B200_CUDA(launch_pdl(stack_cast_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), y, x, total));
  return B200_OK;
}

int launch_stack_act_table(__nv_bfloat16* y, const __nv_bfloat16* g, const void* table, const int32_t* tok, int64_t table_ld,
                           int col, int64_t rows, int n, cudaStream_t st) {
  B200_CHECK_ARG(y && g && table && tok && rows > 0 && n > 0, "stack act_table: bad arguments");
  const int64_t total = rows * n;
  B200_CUDA(launch_pdl(stack_act_table_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), y, g,
                       (const __nv_bfloat16*)table, tok, table_ld, col, n, total));
  return B200_OK;
}

int launch_stack_act_mul(void* y, int64_t ld_y, const void* g, const void* u, int64_t ld_gu, int64_t rows, int n, int act,
                         int dtype, cudaStream_t st) {
  STACK_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(y && g && rows > 0 && n > 0, "stack act_mul: bad arguments");
  B200_CHECK_ARG(act >= B200_ACT_GELU_TANH && act <= B200_ACT_TANH, "stack act_mul: unknown activation %d", act);
  const int64_t total = rows * n;
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_act_mul_kernel<float>, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), (float*)y, ld_y,
                         (const float*)g, (const float*)u, ld_gu, n, act, total));
  else
    B200_CUDA(launch_pdl(stack_act_mul_kernel<__nv_bfloat16>, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(),
                         (__nv_bfloat16*)y, ld_y, (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, ld_gu, n, act, total));
  return B200_OK;
}

int launch_stack_embed(float* x, float* x0, const void* embed, const int32_t* tok, int64_t n_tok, int vocab, int width,
                       float scale, int dtype, cudaStream_t st) {
  STACK_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(x && x0 && embed && tok && n_tok > 0, "stack embed: bad arguments");
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_embed_kernel<float>, dim3((unsigned)n_tok), dim3(128), 0, st, stack_pdl(), x, x0,
                         (const float*)embed, tok, vocab, width, scale));
  else
    B200_CUDA(launch_pdl(stack_embed_kernel<__nv_bfloat16>, dim3((unsigned)n_tok), dim3(128), 0, st, stack_pdl(), x, x0,
                         (const __nv_bfloat16*)embed, tok, vocab, width, scale));
  return B200_OK;
}

int launch_stack_bias_add(__nv_bfloat16* y, const float* b, int64_t rows, int n, cudaStream_t st) {
  B200_CHECK_ARG(y && b && rows > 0 && n > 0, "stack bias_add: bad arguments");
  const int64_t total = rows * n;
  B200_CUDA(launch_pdl(stack_bias_add_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), y, b, n, total));
  return B200_OK;
}

int launch_stack_axpy(float* x, const __nv_bfloat16* t, float mult, bool add, int64_t total, cudaStream_t st) {
  B200_CHECK_ARG(x && t && total > 0, "stack axpy: bad arguments");
  B200_CUDA(launch_pdl(stack_axpy_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), x, t, mult, add ? 1 : 0, total));
  return B200_OK;
}

int launch_stack_cat_cast(__nv_bfloat16* cat, const float* a, const float* b, float* zero, int64_t rows, int width,
                          cudaStream_t st) {
  B200_CHECK_ARG(cat && a && b && rows > 0 && width > 0, "stack cat_cast: bad arguments");
  const int64_t total = rows * width;
  B200_CUDA(launch_pdl(stack_cat_cast_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), cat, a, b, zero, width,
                       total));
  return B200_OK;
}

static int check_attn(const StackAttn& p) {
  const b200_attn_desc& a = p.a;
  B200_CHECK_ARG(a.heads > 0 && a.kv_heads > 0 && a.heads % a.kv_heads == 0 && a.dim > 0 && a.vdim > 0,
                 "stack attention: bad head counts / sizes (heads %d, kv_heads %d, dim %d, vdim %d)", a.heads, a.kv_heads,
                 a.dim, a.vdim);
  B200_CHECK_ARG(a.window >= 0 && a.keep_first >= 0, "stack attention: negative window");
  B200_CHECK_ARG(a.vdim <= 256 && a.dim <= 1024, "stack attention: head sizes above 1024 / 256 are not built");
  B200_CHECK_ARG(p.proj && p.kcache && p.vcache && p.slot && p.pos && p.n_tok > 0, "stack attention: null argument");
  return B200_OK;
}

int launch_stack_kv_store(const StackAttn& p, int dtype, cudaStream_t st) {
  STACK_DTYPE_CHECK(dtype);
  int rc = check_attn(p);
  if (rc != B200_OK) return rc;
  if (dtype == B200_F32) B200_CUDA(launch_pdl(stack_kv_store_kernel<float>, dim3(p.n_tok), dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(stack_kv_store_kernel<__nv_bfloat16>, dim3(p.n_tok), dim3(128), 0, st, stack_pdl(), p));
  return B200_OK;
}

template <typename T, int NW, bool VEC>
static cudaError_t launch_attn_t(const StackAttn& p, cudaStream_t st) {
  const int64_t pairs = (int64_t)p.n_tok * p.a.heads;
  const int ppb = 4 / NW;
  const dim3 grid((unsigned)((pairs + ppb - 1) / ppb), (unsigned)((NW > 1 && p.split_ws != nullptr) ? p.nsplit : 1));
  const size_t smem = ((size_t)4 * p.a.dim + (NW > 1 ? (size_t)NW * (2 + p.a.vdim) : 0)) * sizeof(float);
  const int vr = (p.a.vdim + 31) / 32;
  if (vr <= 1) return launch_pdl(stack_attn_kernel<T, 1, NW, VEC>, grid, dim3(128), smem, st, stack_pdl(), p);
  if (vr <= 2) return launch_pdl(stack_attn_kernel<T, 2, NW, VEC>, grid, dim3(128), smem, st, stack_pdl(), p);
  if (vr <= 4) return launch_pdl(stack_attn_kernel<T, 4, NW, VEC>, grid, dim3(128), smem, st, stack_pdl(), p);
  return launch_pdl(stack_attn_kernel<T, 8, NW, VEC>, grid, dim3(128), smem, st, stack_pdl(), p);
}

int launch_stack_attention(const StackAttn& p, int dtype, cudaStream_t st) {
  STACK_DTYPE_CHECK(dtype);
  int rc = check_attn(p);
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(p.out != nullptr, "stack attention: null output");
  B200_CHECK_ARG(p.split_ws == nullptr || (p.split_tickets != nullptr && p.nsplit >= 1 && p.nsplit <= kStackMaxSplits &&
                                           p.keys_per_split > 0 && p.n_tok <= kStackSplitRows),
                 "stack attention: bad key split");
  // few (token, head) pairs: four warps share one pair's keys
  const bool wide = p.split_ws != nullptr || (int64_t)p.n_tok * p.a.heads < 4 * 148 * 4;
  const int vd = p.a.vdim;
  const bool vec = dtype == B200_BF16 && p.a.dim % 8 == 0 && vd >= 8 && vd <= 256 && (vd & (vd - 1)) == 0 &&
                   p.k_slot_stride % 8 == 0 && p.v_slot_stride % 8 == 0 &&
                   (!p.own_from_proj || (p.off_k % 8 == 0 && p.off_v % 8 == 0 && p.ld_proj % 8 == 0 &&
                                         (reinterpret_cast<uintptr_t>(p.proj) & 15) == 0)) &&
                   ((reinterpret_cast<uintptr_t>(p.kcache) | reinterpret_cast<uintptr_t>(p.vcache)) & 15) == 0;
  if (vec && p.split_ws != nullptr && p.own_from_proj && p.a.dim <= 128 && (vd == 64 || vd == 128) &&
      p.keys_per_split <= 128 && (int64_t)p.n_tok * p.a.heads * p.nsplit <= 2 * 148) {
    // the decode shape, and few enough CTAs to be resident together (the prefetch costs 242 registers per thread: two
    // CTAs per SM): cached rows requested ahead of the dependency wait
    const dim3 grid((unsigned)((int64_t)p.n_tok * p.a.heads), (unsigned)p.nsplit);
    const size_t smem = ((size_t)p.a.dim + 4 * (2 + (size_t)vd)) * sizeof(float);
    B200_CUDA(launch_pdl(stack_attn_decode_kernel, grid, dim3(128), smem, st, stack_pdl(), p));
    return B200_OK;
  }
  if (dtype == B200_F32) {
    if (wide) B200_CUDA((launch_attn_t<float, 4, false>(p, st)));
    else B200_CUDA((launch_attn_t<float, 1, false>(p, st)));
  } else if (vec) {
    if (wide) B200_CUDA((launch_attn_t<__nv_bfloat16, 4, true>(p, st)));
    else B200_CUDA((launch_attn_t<__nv_bfloat16, 1, true>(p, st)));
  } else {
    if (wide) B200_CUDA((launch_attn_t<__nv_bfloat16, 4, false>(p, st)));
    else B200_CUDA((launch_attn_t<__nv_bfloat16, 1, false>(p, st)));
  }

  return B200_OK;
}

}  // namespace b200
