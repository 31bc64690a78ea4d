// stack_mix.cu — mixers and feed-forwards of sandwich blocks as plain kernels: any shape, storage type T = bf16 or fp32.
// fp32 throughout for norms, the softmax, routing scores, the gates of the recurrence, the recurrence and its state.
// Every kernel starts with griddepcontrol.launch_dependents + griddepcontrol.wait (programmatic dependent launch).
#include "stack_mix.cuh"

#include <algorithm>
#include <vector>

#include "ops.cuh"

namespace b200 {

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ T cvt(float v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  __syncthreads();
  return tot;
}

inline int grid_cap(int64_t n, int block) {
  int64_t g = (n + block - 1) / block;
  return (int)std::max<int64_t>(1, std::min<int64_t>(g, 148 * 16));
}

// --------------------------------------------------------------------------------------------------------- layer norm
// One CTA per row.  mean, then the mean of squared deviations (two passes over the row, which stays in L1), then
// (x − mean)·rsqrt(var + eps)·(offset + w): written as T, or added (× mult) into an fp32 stream.
template <typename XT, typename YT, bool ADD>
__global__ void __launch_bounds__(256) stack_layernorm_kernel(YT* __restrict__ y, float* __restrict__ xadd,
                                                              const XT* __restrict__ x, const float* __restrict__ w,
                                                              const int32_t* __restrict__ rows, int dim, float eps,
                                                              float offset, float mult) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int64_t src = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  const XT* xr = x + src * dim;
  float s = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) s += ldf<XT>(xr + i);
  const float mean = block_sum(s, red) / (float)dim;
  float q = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float d = ldf<XT>(xr + i) - mean;
    q += d * d;
  }
  const float inv = rsqrtf(block_sum(q, red) / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = (ldf<XT>(xr + i) - mean) * inv * (offset + w[i]);
    if constexpr (ADD) xadd[(int64_t)blockIdx.x * dim + i] += mult * v;
    else y[(int64_t)blockIdx.x * dim + i] = cvt<YT>(v);
  }
}

// A sublayer's post-norm, the residual sum and the next sublayer's pre-norm in one pass over the row:
//   x ← x + mult·LN(y)·w_post (fp32, stored),   h ← T(LN(x)·(offset + w_next))
// One CTA per row; the new x stays in registers between the two norms (dim <= 256·kLn2Regs).
constexpr int kLn2Regs = 32;
template <typename YT, typename HT>
__global__ void __launch_bounds__(256) stack_layernorm2_kernel(float* __restrict__ x, const YT* __restrict__ y,
                                                               const float* __restrict__ w_post, HT* __restrict__ h,
                                                               const float* __restrict__ w_next, int dim, float eps,
                                                               float offset, float mult) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int64_t base = (int64_t)blockIdx.x * dim;
  float v[kLn2Regs];
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < kLn2Regs; ++u) {
    const int i = threadIdx.x + 256 * u;
    v[u] = i < dim ? ldf<YT>(y + base + i) : 0.f;
    s += v[u];
  }
  float mean = block_sum(s, red) / (float)dim, q = 0.f;
#pragma unroll
  for (int u = 0; u < kLn2Regs; ++u) {
    const int i = threadIdx.x + 256 * u;
    const float d = i < dim ? v[u] - mean : 0.f;
    q += d * d;
  }
  float inv = rsqrtf(block_sum(q, red) / (float)dim + eps);
  s = 0.f;
#pragma unroll
  for (int u = 0; u < kLn2Regs; ++u) {
    const int i = threadIdx.x + 256 * u;
    if (i < dim) {
      v[u] = x[base + i] + mult * (v[u] - mean) * inv * w_post[i];
      x[base + i] = v[u];
      s += v[u];
    } else {
      v[u] = 0.f;
    }
  }
  mean = block_sum(s, red) / (float)dim;
  q = 0.f;
#pragma unroll
  for (int u = 0; u < kLn2Regs; ++u) {
    const int i = threadIdx.x + 256 * u;
    const float d = i < dim ? v[u] - mean : 0.f;
    q += d * d;
  }
  inv = rsqrtf(block_sum(q, red) / (float)dim + eps);
#pragma unroll
  for (int u = 0; u < kLn2Regs; ++u) {
    const int i = threadIdx.x + 256 * u;
    if (i < dim) h[base + i] = cvt<HT>((v[u] - mean) * inv * (offset + w_next[i]));
  }
}

// ------------------------------------------------------------------------------------------------------- elementwise
template <typename T>
__global__ void __launch_bounds__(256) stack_glu_clamp_kernel(T* __restrict__ y, int64_t ld_y, const T* __restrict__ gu,
                                                              int64_t ld_gu, int n, float limit, int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / n;
    const int j = (int)(e % n);
    const float g = fminf(ldf<T>(gu + r * ld_gu + j), limit);
    const float u = fminf(fmaxf(ldf<T>(gu + r * ld_gu + n + j), -limit), limit);
    y[r * ld_y + j] = cvt<T>(g / (1.f + expf(-1.702f * g)) * (u + 1.f));
  }
}

__global__ void __launch_bounds__(256) stack_softcap_kernel(float* __restrict__ lg, __nv_bfloat16* __restrict__ lb,
                                                            int64_t total, float cap) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const float v = cap * tanhf(lg[e] / cap);
    lg[e] = v;
    if (lb != nullptr) lb[e] = __float2bfloat16_rn(v);
  }
}

// y[r, :dim] = T(rms(x[r, :dim])·w), y[r, dim:dim_pad] = 0 over row-strided T-typed rows (a latent's norm between two products)
template <typename T>
__global__ void __launch_bounds__(128) stack_rmsnorm_rows_kernel(T* __restrict__ y, int64_t ld_y, const T* __restrict__ x,
                                                                 int64_t ld_x, const float* __restrict__ w, int dim, int dim_pad,
                                                                 float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[4];
  const T* xr = x + (int64_t)blockIdx.x * ld_x;
  T* yr = y + (int64_t)blockIdx.x * ld_y;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = ldf<T>(xr + i);
    ss += v * v;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) yr[i] = cvt<T>(ldf<T>(xr + i) * inv * w[i]);
  for (int i = dim + threadIdx.x; i < dim_pad; i += blockDim.x) yr[i] = cvt<T>(0.f);
}

// y[r, j] = T(y[r, j]·sigmoid(g[r, j])) over row-strided operands (an element-wise output gate)
template <typename T>
__global__ void __launch_bounds__(256) stack_sigmoid_gate_kernel(T* __restrict__ y, int64_t ld_y, const T* __restrict__ g,
                                                                 int64_t ld_g, int n, int64_t total) {
  pdl_trigger();
  pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / n;
    const int j = (int)(e % n);
    T* dst = y + r * ld_y + j;
    *dst = cvt<T>(ldf<T>(dst) / (1.f + expf(-ldf<T>(g + r * ld_g + j))));
  }
}

// --------------------------------------------------------------------------------------------------- latent attention
// One CTA per new token: the latent c = rms(down[:r])·c_norm and the rotated shared key part go into the slot's cache
// row of the token's position; the rotated part of every head's query goes behind that head's folded query in qa.  Pair i of
// the first rot_dims entries is (2i, 2i+1), or — rot_half — (i, i + rot_dims/2); the entries behind them pass unchanged.
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const LatentRun p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[4];
  const int t = blockIdx.x;
  const int r = p.l.kv_rank, dr = p.l.rot_dim, kd = r + dr, dn = p.a.dim, half = p.l.rot_dims / 2;
  const T* row = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj;
  const T* qrow = static_cast<const T*>(p.q) + (int64_t)t * p.ld_q;
  const T* down = row + p.off_down;
  const int pos = p.pos[t];
  T* crow = static_cast<T*>(p.cache) + (int64_t)p.slot[t] * p.slot_stride + (int64_t)pos * kd;
  float ss = 0.f;
  for (int i = threadIdx.x; i < r; i += blockDim.x) {
    const float v = ldf<T>(down + i);
    ss += v * v;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)r + p.eps);
  for (int i = threadIdx.x; i < r; i += blockDim.x) crow[i] = cvt<T>(ldf<T>(down + i) * inv * p.l.c_norm[i]);
  const float* cs = p.l.rot_table + (int64_t)pos * half * 2;
  // rotated vectors: index 0 the shared key part, 1 … heads the queries' rotated parts; per vector `half` pairs, then the
  // dr − 2·half entries that do not turn
  const int per = half + (dr - 2 * half);
  for (int e = threadIdx.x; e < (p.a.heads + 1) * per; e += blockDim.x) {
    const int which = e / per, i = e % per;
    const T* src = which == 0 ? down + r : qrow + (int64_t)(which - 1) * (dn + dr) + dn;
    T* dst = which == 0 ? crow + r : static_cast<T*>(p.qa) + (int64_t)t * p.a.heads * kd + (int64_t)(which - 1) * kd + r;
    if (i >= half) {
      const int c = 2 * half + (i - half);
      dst[c] = cvt<T>(ldf<T>(src + c));
      continue;
    }
    const int ia = p.l.rot_half ? i : 2 * i, ib = p.l.rot_half ? i + half : 2 * i + 1;
    const float u = ldf<T>(src + ia), v = ldf<T>(src + ib);
    const float c = cs[2 * i], sn = cs[2 * i + 1];
    dst[ia] = cvt<T>(u * c - v * sn);
    dst[ib] = cvt<T>(v * c + u * sn);
  }
}

// One CTA of four warps per (token, head).  The query is [folded query (kv_rank) | rotated part]; key j is the cache row
// [c_j | rotated key part], value j is c_j — the same row.  A warp walks keys 32 at a time: every key's dot product is
// taken by the whole warp over the row's columns, lane l keeps the score of key l, the chunk joins an online softmax and
// the rows are read once more as values.  The warps' partial softmaxes meet in shared memory.
constexpr int kLatVR = 16;   // latents up to 512 entries in the split-key kernel and the common case of this one
template <typename T, int VR>
__global__ void __launch_bounds__(128) latent_attn_kernel(const LatentRun p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float sm[];
  const int t = blockIdx.x, hd = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = p.l.kv_rank, kd = r + p.l.rot_dim;
  float* q = sm;                 // [kd]
  float* part = sm + kd;         // [4][2 + r]
  const T* qrow = static_cast<const T*>(p.qa) + ((int64_t)t * p.a.heads + hd) * kd;
  for (int i = threadIdx.x; i < kd; i += blockDim.x) q[i] = ldf<T>(qrow + i) * p.a.scale;
  __syncthreads();
  const int n_keys = p.pos[t] + 1;
  const int k_first = p.a.window > 0 ? max(0, n_keys - p.a.window) : 0;   // the window's first key
  const T* K = static_cast<const T*>(p.cache) + (int64_t)p.slot[t] * p.slot_stride;
  float m = -INFINITY, sum = 0.f, acc[VR];
#pragma unroll
  for (int i = 0; i < VR; ++i) acc[i] = 0.f;
  for (int j0 = k_first + warp * 32; j0 < n_keys; j0 += 128) {
    const int cnt = min(32, n_keys - j0);
    float s_mine = -INFINITY;
    for (int jj = 0; jj < cnt; ++jj) {
      const T* kr = K + (int64_t)(j0 + jj) * kd;
      float d = 0.f;
      for (int i = lane; i < kd; i += 32) d = fmaf(q[i], ldf<T>(kr + i), d);
      d = warp_sum(d);
      if (lane == jj) s_mine = d;
    }
    const float m_new = fmaxf(m, warp_max(s_mine));
    const float pr = lane < cnt ? expf(s_mine - m_new) : 0.f;
    const float corr = expf(m - m_new);   // m = −inf on the first chunk: 0
    sum = sum * corr + warp_sum(pr);
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[i] *= corr;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pr, jj);
      const T* kr = K + (int64_t)(j0 + jj) * kd;
#pragma unroll
      for (int i = 0; i < VR; ++i)
        if (lane + 32 * i < r) acc[i] = fmaf(pj, ldf<T>(kr + lane + 32 * i), acc[i]);
    }
    m = m_new;
  }
  float* mine = part + warp * (2 + r);
  if (lane == 0) {
    mine[0] = m;
    mine[1] = sum;
  }
#pragma unroll
  for (int i = 0; i < VR; ++i)
    if (lane + 32 * i < r) mine[2 + lane + 32 * i] = acc[i];
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < 4; ++w) M = fmaxf(M, part[w * (2 + r)]);
  float f[4], tot = 0.f;
  for (int w = 0; w < 4; ++w) {
    const float mw = part[w * (2 + r)];
    f[w] = mw == -INFINITY ? 0.f : expf(mw - M);
    tot += f[w] * part[w * (2 + r) + 1];
  }
  T* orow = static_cast<T*>(p.ol) + ((int64_t)t * p.a.heads + hd) * r;
  for (int c = threadIdx.x; c < r; c += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < 4; ++w) v += f[w] * part[w * (2 + r) + 2 + c];
    orow[c] = cvt<T>(v / tot);
  }
}

// Per-head key and query rows for the tensor-core prompt attention (see LatentPack): one CTA per key row, then per query row.
__global__ void __launch_bounds__(128) latent_pack_kernel(const LatentPack p) {
  pdl_trigger();
  pdl_wait();
  const int H = p.a.heads, dn = p.a.dim, dr = p.l.rot_dim, r = p.l.kv_rank, hd = dn + dr, kd = r + dr;
  const int row = blockIdx.x;
  if (row < p.ctx) {
    const __nv_bfloat16* kp = p.kp + (int64_t)row * H * dn;
    const __nv_bfloat16* rot = p.cache_rows + (int64_t)row * kd + r;
    __nv_bfloat16* dst = p.kbuf + (int64_t)row * H * hd;
    for (int i = threadIdx.x; i < H * hd; i += blockDim.x) {
      const int h = i / hd, e = i % hd;
      dst[i] = e < dn ? kp[h * dn + e] : rot[e - dn];
    }
  } else {
    const int t = row - p.ctx;
    const __nv_bfloat16* q = p.proj + (int64_t)t * p.ld_proj + p.off_q;   // the caller points proj / ld_proj / off_q at the query rows
    const __nv_bfloat16* qa = p.qa + (int64_t)t * H * kd;
    __nv_bfloat16* dst = p.qbuf + (int64_t)t * H * hd;
    for (int i = threadIdx.x; i < H * hd; i += blockDim.x) {
      const int h = i / hd, e = i % hd;
      dst[i] = e < dn ? q[h * hd + e] : qa[h * kd + r + (e - dn)];
    }
  }
}

// ------------------------------------------------------------------------------------------------- small products
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  unpack8(*reinterpret_cast<const uint4*>(p), v);
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// One warp per output row n of item blockIdx.y.  VEC: 16-byte (bf16) / 32-byte (fp32) pieces of the matrix row and of
// the M activation rows, lane l takes pieces l, l + 32, …; otherwise element by element.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) small_gemv_kernel(const SmallGemv g) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31, z = blockIdx.y;
  if (n >= g.N) return;
  const int64_t mat = g.item_mat != nullptr ? g.item_mat[z] : z;
  const T* wr = static_cast<const T*>(g.w) + mat * g.sw + (int64_t)n * g.K;
  const T* a = static_cast<const T*>(g.a) + (int64_t)(z / g.item_div) * g.sa;
  const int M = g.m_total > 0 ? min(g.M, g.m_total - z * g.M) : g.M;
  float acc[kSmallRows];
#pragma unroll
  for (int m = 0; m < kSmallRows; ++m) acc[m] = 0.f;
  if constexpr (VEC) {
    for (int k = lane * 8; k < g.K; k += 256) {
      float wv[8];
      load8<T>(wr + k, wv);
#pragma unroll
      for (int m = 0; m < kSmallRows; ++m) {
        if (m < M) {
          float av[8];
          load8<T>(a + (int64_t)m * g.lda + k, av);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[m] = fmaf(wv[i], av[i], acc[m]);
        }
      }
    }
  } else {
    for (int k = lane; k < g.K; k += 32) {
      const float wv = ldf<T>(wr + k);
#pragma unroll
      for (int m = 0; m < kSmallRows; ++m)
        if (m < M) acc[m] = fmaf(wv, ldf<T>(a + (int64_t)m * g.lda + k), acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < kSmallRows; ++m) {
    if (m >= M) break;
    float v = warp_sum(acc[m]);
    if (lane == 0) {
      if (g.bias != nullptr) v += g.bias[n];
      if (g.bias_m != nullptr) v += g.bias_m[z * g.M + m];
      if (g.act == B200_ACT_RELU2) v = fmaxf(v, 0.f) * fmaxf(v, 0.f);
      else if (g.act == B200_ACT_TANH) v = tanhf(v);
      else if (g.act == B200_ACT_SILU) v = v / (1.f + expf(-v));
      const int64_t o = (int64_t)m * g.ldc + (int64_t)z * g.sc + (int64_t)n * g.nc;
      if (g.c_f32) static_cast<float*>(g.c)[o] = v;
      else static_cast<T*>(g.c)[o] = cvt<T>(v);
    }
  }
}

// ------------------------------------------------------------------------------------- latent attention, decode-shaped
// One CTA of eight warps per (row, split of the key list).  The split's key rows [c | rotated key part] are staged in
// shared memory 32 at a time and serve ALL heads (warp w takes heads w, w + 8, …): the rows are read from memory once per
// row of the step instead of once per head.  Scores: warp w keeps keys 4w … 4w+3 of the chunk in registers, every head's
// query streams past them from shared memory and the four dot products are summed over the warp side by side; the
// chunk's scores [head][key] go through shared memory to the heads' warps.  Then per head: the online softmax and the
// weighted latents.  Partials go to split_ws; latent_merge_kernel joins the splits.
constexpr int kLatHeadsPerWarp = 4;   // heads <= 32
constexpr int kLatKeyRegs = 20;       // cache row (kv_rank + rot_dim) <= 640
template <typename T>
__global__ void __launch_bounds__(256) latent_attn_split_kernel(const LatentRun p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float sm[];
  __shared__ float sc[8 * kLatHeadsPerWarp * 32];   // the chunk's scores [head][key]
  const int t = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = p.l.kv_rank, kd = r + p.l.rot_dim, H = p.a.heads;
  float* q = sm;                          // [H][kd], scaled
  float* kc = sm + (size_t)H * kd;        // [32][kd] staged key rows
  const T* qrow = static_cast<const T*>(p.qa) + (int64_t)t * H * kd;
  const int n_keys = p.pos[t] + 1;
  const int k_first = p.a.window > 0 ? max(0, n_keys - p.a.window) : 0;   // the window's first key: split 0 starts there
  const int k_lo = k_first + split * p.keys_per_split, k_hi = min(n_keys, k_lo + p.keys_per_split);
  if (k_lo >= n_keys) return;   // the merge reads the splits that saw a key, and only those
  if (p.stage_vec) {
    for (int i = threadIdx.x * 8; i < H * kd; i += blockDim.x * 8) {
      float v[8];
      load8<T>(qrow + i, v);
#pragma unroll
      for (int u = 0; u < 8; ++u) q[i + u] = v[u] * p.a.scale;
    }
  } else {
    for (int i = threadIdx.x; i < H * kd; i += blockDim.x) q[i] = ldf<T>(qrow + i) * p.a.scale;
  }
  const T* K = static_cast<const T*>(p.cache) + (int64_t)p.slot[t] * p.slot_stride;
  float m[kLatHeadsPerWarp], sum[kLatHeadsPerWarp], acc[kLatHeadsPerWarp][kLatVR];
#pragma unroll
  for (int u = 0; u < kLatHeadsPerWarp; ++u) {
    m[u] = -INFINITY;
    sum[u] = 0.f;
#pragma unroll
    for (int i = 0; i < kLatVR; ++i) acc[u][i] = 0.f;
  }
  for (int j0 = k_lo; j0 < k_hi; j0 += 32) {
    const int cnt = min(32, k_hi - j0);
    __syncthreads();
    {   // rows j0 … j0+cnt-1 are contiguous in the cache: one flat copy, eight elements a piece where alignment allows
      const T* src = K + (int64_t)j0 * kd;
      const int total = cnt * kd;
      if (p.stage_vec) {
        for (int i = threadIdx.x * 8; i < total; i += blockDim.x * 8) {
          float v[8];
          load8<T>(src + i, v);
#pragma unroll
          for (int u = 0; u < 8; ++u) kc[i + u] = v[u];
        }
      } else {
        for (int i = threadIdx.x; i < total; i += blockDim.x) kc[i] = ldf<T>(src + i);
      }
    }
    __syncthreads();
    {   // scores: warp w holds keys 4w … 4w+3 of the chunk in registers and lets every head's query stream past them
      float kreg[4][kLatKeyRegs];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int ii = 0; ii < kLatKeyRegs; ++ii) {
          const int c = lane + 32 * ii;
          kreg[u][ii] = (4 * warp + u < cnt && c < kd) ? kc[(size_t)(4 * warp + u) * kd + c] : 0.f;
        }
      for (int hd = 0; hd < H; ++hd) {
        const float* qh = q + (size_t)hd * kd;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ii = 0; ii < kLatKeyRegs; ++ii) {
          const int c = lane + 32 * ii;
          const float qv = c < kd ? qh[c] : 0.f;
#pragma unroll
          for (int u = 0; u < 4; ++u) d[u] = fmaf(qv, kreg[u][ii], d[u]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int u = 0; u < 4; ++u) d[u] += __shfl_xor_sync(0xffffffffu, d[u], o);
        if (lane < 4) sc[hd * 32 + 4 * warp + lane] = lane == 0 ? d[0] : lane == 1 ? d[1] : lane == 2 ? d[2] : d[3];
      }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kLatHeadsPerWarp; ++u) {
      const int hd = warp + 8 * u;
      if (hd >= H) break;
      const float s_mine = lane < cnt ? sc[hd * 32 + lane] : -INFINITY;
      const float m_new = fmaxf(m[u], warp_max(s_mine));
      const float pr = lane < cnt ? expf(s_mine - m_new) : 0.f;
      const float corr = expf(m[u] - m_new);
      sum[u] = sum[u] * corr + warp_sum(pr);
#pragma unroll
      for (int i = 0; i < kLatVR; ++i) acc[u][i] *= corr;
      for (int jj = 0; jj < cnt; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
        const float* kr = kc + (size_t)jj * kd;
#pragma unroll
        for (int i = 0; i < kLatVR; ++i)
          if (lane + 32 * i < r) acc[u][i] = fmaf(pj, kr[lane + 32 * i], acc[u][i]);
      }
      m[u] = m_new;
    }
  }
  // partials of this split
#pragma unroll
  for (int u = 0; u < kLatHeadsPerWarp; ++u) {
    const int hd = warp + 8 * u;
    if (hd >= H) break;
    float* dst = p.split_ws + (((int64_t)t * H + hd) * p.nsplit + split) * (2 + r);
    if (lane == 0) {
      dst[0] = m[u];
      dst[1] = sum[u];
    }
#pragma unroll
    for (int i = 0; i < kLatVR; ++i)
      if (lane + 32 * i < r) dst[2 + lane + 32 * i] = acc[u][i];
  }
}

// One CTA per (row, head): the splits' partial softmaxes {max, sum, weighted latents} become the head's weighted latent.
// The splits' maxima and sums are fetched side by side and turned into one weight per split in shared memory; then
// every thread sums its columns over the splits (independent loads).
template <typename T>
__global__ void __launch_bounds__(256) latent_merge_kernel(const LatentRun p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float wgt[kLatentMaxSplits];
  __shared__ float s_tot;
  const int t = blockIdx.x, hd = blockIdx.y, H = p.a.heads, r = p.l.kv_rank;
  const float* src = p.split_ws + ((int64_t)t * H + hd) * p.nsplit * (2 + r);
  const int visible = p.a.window > 0 ? min(p.pos[t] + 1, p.a.window) : p.pos[t] + 1;
  const int used = min(p.nsplit, (visible + p.keys_per_split - 1) / p.keys_per_split);   // splits that saw a key
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mx[kLatentMaxSplits / 32], sm_[kLatentMaxSplits / 32], M = -INFINITY;
#pragma unroll
    for (int u = 0; u < kLatentMaxSplits / 32; ++u) {
      const int sp = lane + 32 * u;
      mx[u] = sp < used ? src[(int64_t)sp * (2 + r)] : -INFINITY;
      sm_[u] = sp < used ? src[(int64_t)sp * (2 + r) + 1] : 0.f;
      M = fmaxf(M, mx[u]);
    }
    M = warp_max(M);
    float tot = 0.f;
#pragma unroll
    for (int u = 0; u < kLatentMaxSplits / 32; ++u) {
      const int sp = lane + 32 * u;
      const float w = sp < used ? expf(mx[u] - M) : 0.f;
      if (sp < kLatentMaxSplits) wgt[sp] = w;
      tot += w * sm_[u];
    }
    tot = warp_sum(tot);
    if (lane == 0) s_tot = tot;
  }
  __syncthreads();
  const float inv = 1.f / s_tot;
  T* orow = static_cast<T*>(p.ol) + ((int64_t)t * H + hd) * r;
  for (int c = threadIdx.x; c < r; c += blockDim.x) {
    float v = 0.f;
#pragma unroll 8
    for (int sp = 0; sp < used; ++sp) v = fmaf(wgt[sp], src[(int64_t)sp * (2 + r) + 2 + c], v);
    orow[c] = cvt<T>(v * inv);
  }
}

// --------------------------------------------------------------------------------------------------------------- mLSTM
// One warp per (sequence, head, state column): lane l holds rows l, l + 32, … of its column of S; column vdim is the
// normaliser n (the column whose "value" is 1).  Every warp carries its own copy of the running maximum m, so columns
// never read what another column's warp wrote.  Per token: the capped gates, m_t = max(f + m, i), the column's decay and
// update, then the column's dot with q (a numerator of the output, or n·q).  The next token's operands are requested
// while the current one is summed.  Eight columns per CTA.
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// One warp per (sequence, head): the gates of every token — i = cap·tanh(z_i/cap), f = logsigmoid(cap·tanh(z_f/cap)) — the
// running maximum m_t = max(f + m_(t-1), i) along the sequence (32 tokens' gates are computed side by side, the maximum
// walks through them), and from it the decay a_t = e^(f + m_(t-1) − m_t) and the input weight b_t = e^(i − m_t).
// gab[row][head] = {a, b, m}: the column warps of the scan below no longer repeat any of this.
__global__ void __launch_bounds__(32) mlstm_gates_kernel(const MlstmRun p) {
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.x, hd = blockIdx.y, lane = threadIdx.x;
  const int dk = p.a.dim, dv = p.a.vdim, H = p.a.heads;
  const int r0 = p.seg_row0 != nullptr ? p.seg_row0[seg] : seg;
  const int cnt = p.seg_count != nullptr ? p.seg_count[seg] : 1;
  const float* st_m = p.state + (int64_t)p.slot[r0] * p.slot_stride + (int64_t)hd * ((int64_t)dk * (dv + 1) + dv + 1) +
                      (int64_t)dk * (dv + 1);
  float m_prev = p.pos[r0] > 0 ? st_m[0] : 0.f;
  const float cap = p.gate_cap;
  for (int t0 = 0; t0 < cnt; t0 += 32) {
    const int t = t0 + lane;
    float gi = 0.f, gf = 0.f;
    if (t < cnt) {
      gi = cap * tanhf(p.gates[(int64_t)(r0 + t) * p.ld_gates + hd] / cap);
      gf = log_sigmoid(cap * tanhf(p.gates[(int64_t)(r0 + t) * p.ld_gates + H + hd] / cap));
    }
    float before = 0.f, after = 0.f;
    const int n = min(32, cnt - t0);
#pragma unroll
    for (int u = 0; u < 32; ++u) {   // fixed length: the 64 shuffles do not wait for the walk
      const float fu = __shfl_sync(0xffffffffu, gf, u), iu = __shfl_sync(0xffffffffu, gi, u);
      const float m_new = u < n ? fmaxf(fu + m_prev, iu) : m_prev;
      if (lane == u) {
        before = m_prev;
        after = m_new;
      }
      m_prev = m_new;
    }
    if (t < cnt) {
      float* o = p.gab + ((int64_t)(r0 + t) * H + hd) * 3;
      o[0] = expf(gf + before - after);
      o[1] = expf(gi - after);
      o[2] = after;
    }
  }
}

// DR = rows of S per lane (key size <= 32·DR).  One warp per (sequence, head, state column): lane l holds rows l, l + 32, …
// of its column of S; column vdim is the normaliser n (the column whose "value" is 1); eight columns per CTA.  The CTA
// walks its sequence CH tokens at a time: the chunk's q (scaled), k, the eight columns' v and the gate factors sit in
// shared memory as fp32, converted once for all eight warps, while the next chunk's values are already on their way
// into registers — the walk waits for memory once per sequence, and a token costs a warp a handful of shared-memory
// reads, 2·DR multiply-adds and one warp sum.
template <typename T, int DR>
__global__ void __launch_bounds__(256) mlstm_scan_kernel(const MlstmRun p) {
  pdl_trigger();
  pdl_wait();
  constexpr int CH = DR >= 16 ? 8 : 16;          // tokens per chunk
  constexpr int DK = 32 * DR;                    // padded key size
  constexpr int NQK = CH * 2 * DK / 256;         // q / k elements a thread stages per chunk
  __shared__ float s_qk[CH][2][DK];
  __shared__ float s_ab[CH][3];
  __shared__ float s_v[CH][8];
  const int seg = blockIdx.x, hd = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int dk = p.a.dim, dv = p.a.vdim, H = p.a.heads;
  const int j0 = blockIdx.z * 8, j = j0 + warp;
  const bool live = j <= dv;                     // warps past the last column only help with the staging
  const int r0 = p.seg_row0 != nullptr ? p.seg_row0[seg] : seg;
  const int cnt = p.seg_count != nullptr ? p.seg_count[seg] : 1;
  const int pos0 = p.pos[r0];
  float* st = p.state + (int64_t)p.slot[r0] * p.slot_stride + (int64_t)hd * ((int64_t)dk * (dv + 1) + dv + 1);
  float* st_m = st + (int64_t)dk * (dv + 1);
  float S[DR], m = 0.f;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = lane + 32 * i;
    S[i] = (live && pos0 > 0 && d < dk) ? st[(int64_t)d * (dv + 1) + j] : 0.f;
  }
  const float qs = rsqrtf((float)dk);
  const T* P = static_cast<const T*>(p.proj);
  float r_qk[NQK], r_x = 0.f;   // staged values of the next chunk; r_x: a gate factor (threads 0 … 3·CH) or a v (next 8·CH)
  auto fetch = [&](int c0) {
#pragma unroll
    for (int i = 0; i < NQK; ++i) {
      const int e = tid + 256 * i, t = e / (2 * DK), w = (e / DK) & 1, d = e % DK;
      r_qk[i] = (c0 + t < cnt && d < dk) ? ldf<T>(P + (int64_t)(r0 + c0 + t) * p.ld_proj + (w ? p.off_k : p.off_q) + hd * dk + d)
                                         : 0.f;
    }
    if (tid < 3 * CH) {
      const int t = tid / 3;
      r_x = c0 + t < cnt ? p.gab[((int64_t)(r0 + c0 + t) * H + hd) * 3 + tid % 3] : 0.f;
    } else if (tid < 11 * CH) {
      const int t = (tid - 3 * CH) / 8, c = j0 + (tid - 3 * CH) % 8;
      r_x = (c0 + t < cnt && c < dv) ? ldf<T>(P + (int64_t)(r0 + c0 + t) * p.ld_proj + p.off_v + hd * dv + c) : 1.f;
    }
  };
  fetch(0);
  for (int c0 = 0; c0 < cnt; c0 += CH) {
    __syncthreads();   // the previous chunk has been read
#pragma unroll
    for (int i = 0; i < NQK; ++i) {
      const int e = tid + 256 * i, w = (e / DK) & 1;
      (&s_qk[0][0][0])[e] = w ? r_qk[i] : r_qk[i] * qs;
    }
    if (tid < 3 * CH) (&s_ab[0][0])[tid] = r_x;
    else if (tid < 11 * CH) (&s_v[0][0])[tid - 3 * CH] = r_x;
    __syncthreads();
    if (c0 + CH < cnt) fetch(c0 + CH);
    if (!live) continue;
    const int n = min(CH, cnt - c0);
    for (int t4 = 0; t4 < n; t4 += 4) {   // four tokens' dots are summed over the warp side by side
      float dot[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int t = t4 + u;             // t < CH always (CH is a multiple of 4); rows past n hold zeros with a = b = 0
        const bool on = t < n;
        const float a = on ? s_ab[t][0] : 1.f, b = on ? s_ab[t][1] * s_v[t][warp] : 0.f;
        dot[u] = 0.f;
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          S[i] = fmaf(a, S[i], b * s_qk[t][1][lane + 32 * i]);
          dot[u] = fmaf(S[i], s_qk[t][0][lane + 32 * i], dot[u]);
        }
        if (on) m = s_ab[t][2];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
      }
      if (lane < 4 && t4 + lane < n) {
        float* orow = p.o + ((int64_t)(r0 + c0 + t4 + lane) * H + hd) * (dv + 2);
        const float mine = lane == 0 ? dot[0] : lane == 1 ? dot[1] : lane == 2 ? dot[2] : dot[3];
        orow[j] = mine;
        if (j == dv) orow[dv + 1] = s_ab[t4 + lane][2];
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = lane + 32 * i;
    if (d < dk) st[(int64_t)d * (dv + 1) + j] = S[i];
  }
  if (lane == 0) st_m[j] = m;
}

// One warp per (token, head): o = numerators / (max(|n·q|, e^(−m)) + 1e-6), o / rms(o), · head_norm · sigmoid(out gate).
template <typename T>
__global__ void __launch_bounds__(128) mlstm_out_kernel(const MlstmRun p) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int H = p.a.heads, dv = p.a.vdim;
  if (pair >= p.n_tok * H) return;
  const int t = pair / H, hd = pair % H;
  const float* orow = p.o + (int64_t)pair * (dv + 2);
  const float den = fmaxf(fabsf(orow[dv]), expf(-orow[dv + 1])) + 1e-6f;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    const float v = orow[c] / den;
    ss += v * v;
  }
  const float inv = rsqrtf(warp_sum(ss) / (float)dv + p.eps);
  const T* g = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj + p.off_g + hd * dv;
  T* y = static_cast<T*>(p.mid) + (int64_t)t * p.ld_mid + hd * dv;
  for (int c = lane; c < dv; c += 32) {
    const float gate = 1.f / (1.f + expf(-ldf<T>(g + c)));
    y[c] = cvt<T>(orow[c] / den * inv * p.head_norm[hd * dv + c] * gate);
  }
}

// ------------------------------------------------------------------------------------------------------ routed experts
// One warp per token: the `top` largest router logits (the sigmoid is monotonic, so the order is that of the scores; ties
// go to the lower index), their sigmoids as weights, and a count per expert.
__global__ void __launch_bounds__(128) moe_route_kernel(const MoeRun p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= p.n_tok) return;
  const int E = p.m.experts, top = p.m.top;
  const float* z = p.z + (int64_t)t * E;
  // softmax routing: the scores' common denominator (the order of the scores is that of the logits)
  float zmax = -INFINITY, zsum = 0.f, picked = 0.f;
  if (p.m.router_kind == 1) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
    for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    for (int e = lane; e < E; e += 32) zsum += expf(z[e] - zmax);
    zsum = warp_sum(zsum);
  }
  float last_v = INFINITY;
  int last_i = -1;
  for (int k = 0; k < top; ++k) {
    // the best entry that comes after (last_v, last_i) in the order (value descending, index ascending)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      const bool after = v < last_v || (v == last_v && e > last_i);
      if (after && (v > bv || (v == bv && e < bi))) {
        bv = v;
        bi = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = 0;   // fewer finite logits than choices: cannot happen with top <= experts
    if (lane == 0) {
      p.sel_e[(int64_t)t * top + k] = bi;
      const float score = p.m.router_kind == 1 ? expf(bv - zmax) / zsum : 1.f / (1.f + expf(-bv));
      p.sel_w[(int64_t)t * top + k] = score;
      picked += score;
      if (p.small) p.pair_slot[(int64_t)t * top + k] = t * top + k;   // no sorting: a pair stays where it is
      else atomicAdd(p.plan + bi, 1);
    }
    last_v = bv;
    last_i = bi;
  }
  if (p.m.router_kind == 1 && lane == 0)   // the chosen scores over their sum, times the design's scale
    for (int k = 0; k < top; ++k) p.sel_w[(int64_t)t * top + k] = p.sel_w[(int64_t)t * top + k] / (picked + 1e-20f) * p.m.route_scale;
}

// One CTA: counts → group ends, the row tiles of every group, and a sorted position for every pair.
__global__ void __launch_bounds__(256) moe_plan_kernel(const MoeRun p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ int sh[];   // cursor [E]
  const int E = p.m.experts, P = p.n_tok * p.m.top, n_tiles = moe_tiles(P, E);
  const int S = p.plan_stride > 0 ? p.plan_stride : E;
  int32_t* counts = p.plan;
  int32_t* group_end = p.plan + S;
  int32_t* tile_group = p.plan + 2 * S;
  int32_t* tile_row0 = tile_group + n_tiles;
  if (threadIdx.x == 0) {
    int row = 0, tile = 0;
    for (int e = 0; e < E; ++e) {
      sh[e] = row;
      const int end = row + counts[e];
      for (int r0 = row; r0 < end; r0 += 64) {
        tile_group[tile] = e;
        tile_row0[tile] = r0;
        ++tile;
      }
      row = end;
      group_end[e] = end;
    }
    for (; tile < n_tiles; ++tile) tile_group[tile] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < P; i += blockDim.x) p.pair_slot[i] = atomicAdd(&sh[p.sel_e[i]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;   // ready for the next routing
}

// a_perm[slot of pair, :] = T(score · h[token, :])   (h itself when the weight multiplies the expert's output)
template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(const MoeRun p) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x, t = pair / p.m.top;
  const float w = p.m.weight_output ? 1.f : p.sel_w[pair];
  const T* src = static_cast<const T*>(p.h) + (int64_t)t * p.width;
  T* dst = static_cast<T*>(p.a_perm) + (int64_t)p.pair_slot[pair] * p.width;
  for (int i = threadIdx.x; i < p.width; i += blockDim.x) dst[i] = cvt<T>(w * ldf<T>(src + i));
}

// y[t, :] = Σ_k [weight_k ·] outp[slot of (t, k), :] + [sigmoid(sg[t]) ·] shared[t, :]   — one thread per (token, column); the
// choices are summed in the order they were made, whatever else is in the step
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeRun p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, top = p.m.top, i = blockIdx.y * 256 + threadIdx.x;
  if (i >= p.width) return;
  const int32_t* slots = p.pair_slot + (int64_t)t * top;
  float v = 0.f;
  for (int k = 0; k < top; ++k) {
    const int64_t o = (int64_t)slots[k] * p.width + i;
    const float ov = p.tc ? __bfloat162float(p.outp_bf[o]) : p.outp[o];
    v = p.m.weight_output ? fmaf(p.sel_w[(int64_t)t * top + k], ov, v) : v + ov;
  }
  if (p.shared != nullptr) {
    const float gate = p.m.shared_plain ? 1.f : 1.f / (1.f + expf(-ldf<T>(static_cast<const T*>(p.sg) + (int64_t)t * p.ld_sg)));
    const int64_t o = (int64_t)t * p.width + i;
    v += gate * (p.shared_f32 ? static_cast<const float*>(p.shared)[o] : ldf<T>(static_cast<const T*>(p.shared) + o));
  }
  p.y[(int64_t)t * p.width + i] = v;
}

}  // namespace

#define MIX_DTYPE_CHECK(dtype) \
  B200_CHECK_ARG((dtype) == B200_BF16 || (dtype) == B200_F32, "stack op: unknown dtype %d", (int)(dtype))

int launch_stack_norm(void* y, const float* x, const float* w, const int32_t* rows, int64_t n_rows, int dim, float eps,
                      float offset, int kind, int dtype, cudaStream_t st) {
  if (kind == B200_NORM_RMS) return launch_stack_rmsnorm(y, x, w, rows, n_rows, dim, eps, offset, dtype, st);
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(kind == B200_NORM_LAYER, "stack norm: unknown kind %d", kind);
  B200_CHECK_ARG(y && x && w && n_rows > 0 && dim > 0, "stack norm: bad arguments");
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_layernorm_kernel<float, float, false>, dim3((unsigned)n_rows), dim3(256), 0, st, stack_pdl(),
                         (float*)y, (float*)nullptr, x, w, rows, dim, eps, offset, 1.f));
  else
    B200_CUDA(launch_pdl(stack_layernorm_kernel<float, __nv_bfloat16, false>, dim3((unsigned)n_rows), dim3(256), 0, st,
                         stack_pdl(), (__nv_bfloat16*)y, (float*)nullptr, x, w, rows, dim, eps, offset, 1.f));
  return B200_OK;
}

int launch_stack_norm_add(float* x, const void* y, bool y_bf16, const float* w, int64_t rows, int dim, float eps, float mult,
                          int kind, cudaStream_t st) {
  if (kind == B200_NORM_RMS)
    return y_bf16 ? launch_stack_rms_add_bf16(x, (const __nv_bfloat16*)y, w, rows, dim, eps, mult, st)
                  : launch_stack_rms_add(x, (const float*)y, w, rows, dim, eps, mult, st);
  B200_CHECK_ARG(kind == B200_NORM_LAYER, "stack norm_add: unknown kind %d", kind);
  B200_CHECK_ARG(x && y && w && rows > 0 && dim > 0, "stack norm_add: bad arguments");
  if (y_bf16)
    B200_CUDA(launch_pdl(stack_layernorm_kernel<__nv_bfloat16, float, true>, dim3((unsigned)rows), dim3(256), 0, st,
                         stack_pdl(), (float*)nullptr, x, (const __nv_bfloat16*)y, w, (const int32_t*)nullptr, dim, eps, 0.f,
                         mult));
  else
    B200_CUDA(launch_pdl(stack_layernorm_kernel<float, float, true>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(),
                         (float*)nullptr, x, (const float*)y, w, (const int32_t*)nullptr, dim, eps, 0.f, mult));
  return B200_OK;
}

int launch_stack_norm_add_norm(float* x, const void* y, bool y_bf16, const float* w_post, void* h, const float* w_next,
                               int64_t rows, int dim, float eps, float offset, float mult, int kind, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(x && y && w_post && h && w_next && rows > 0 && dim > 0, "stack norm_add_norm: bad arguments");
  if (kind != B200_NORM_LAYER || dim > 256 * kLn2Regs) {   // two launches do the same
    int rc = launch_stack_norm_add(x, y, y_bf16, w_post, rows, dim, eps, mult, kind, st);
    if (rc != B200_OK) return rc;
    return launch_stack_norm(h, x, w_next, nullptr, rows, dim, eps, offset, kind, dtype, st);
  }
  const dim3 grid((unsigned)rows);
#define B200_LN2(YT, HT)                                                                                                     \
  B200_CUDA(launch_pdl(stack_layernorm2_kernel<YT, HT>, grid, dim3(256), 0, st, stack_pdl(), x, (const YT*)y, w_post, (HT*)h, \
                       w_next, dim, eps, offset, mult))
  if (y_bf16 && dtype == B200_F32) B200_LN2(__nv_bfloat16, float);
  else if (y_bf16) B200_LN2(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == B200_F32) B200_LN2(float, float);
  else B200_LN2(float, __nv_bfloat16);
#undef B200_LN2
  return B200_OK;
}

int launch_stack_glu_clamp(void* y, int64_t ld_y, const void* gu, int64_t ld_gu, int64_t rows, int n, float limit, int dtype,
                           cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(y && gu && rows > 0 && n > 0, "stack glu_clamp: bad arguments");
  const int64_t total = rows * n;
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_glu_clamp_kernel<float>, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(), (float*)y,
                         ld_y, (const float*)gu, ld_gu, n, limit, total));
  else
    B200_CUDA(launch_pdl(stack_glu_clamp_kernel<__nv_bfloat16>, dim3(grid_cap(total, 256)), dim3(256), 0, st, stack_pdl(),
                         (__nv_bfloat16*)y, ld_y, (const __nv_bfloat16*)gu, ld_gu, n, limit, total));
  return B200_OK;
}

int launch_stack_softcap(float* logits, __nv_bfloat16* logits_bf, int64_t total, float cap, cudaStream_t st) {
  B200_CHECK_ARG(logits && total > 0 && cap > 0.f, "stack softcap: bad arguments");
  // copies and the argmax follow: a full dependency
  B200_CUDA(launch_pdl(stack_softcap_kernel, dim3(grid_cap(total, 256)), dim3(256), 0, st, false, logits, logits_bf, total, cap));
  return B200_OK;
}

int launch_small_gemv(const SmallGemv& g, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(g.a && g.w && g.c && g.M >= 1 && g.M <= kSmallRows && g.N > 0 && g.K > 0 && g.items > 0 && g.items <= 65535 && g.item_div >= 1,
                 "small gemv: bad arguments M=%d N=%d K=%d items=%d", g.M, g.N, g.K, g.items);
  const size_t esz = dtype == B200_F32 ? 4 : 2;
  const size_t al = dtype == B200_F32 ? 32 : 16;   // bytes of one 8-element piece
  const bool vec = g.K % 8 == 0 && (reinterpret_cast<uintptr_t>(g.a) % al) == 0 && (reinterpret_cast<uintptr_t>(g.w) % al) == 0 &&
                   (g.lda * esz) % al == 0 && (g.sa * esz) % al == 0 && (g.sw * esz) % al == 0;
  const dim3 grid((g.N + 7) / 8, g.items);
  if (dtype == B200_F32) {
    if (vec) B200_CUDA(launch_pdl(small_gemv_kernel<float, true>, grid, dim3(256), 0, st, stack_pdl(), g));
    else B200_CUDA(launch_pdl(small_gemv_kernel<float, false>, grid, dim3(256), 0, st, stack_pdl(), g));
  } else {
    if (vec) B200_CUDA(launch_pdl(small_gemv_kernel<__nv_bfloat16, true>, grid, dim3(256), 0, st, stack_pdl(), g));
    else B200_CUDA(launch_pdl(small_gemv_kernel<__nv_bfloat16, false>, grid, dim3(256), 0, st, stack_pdl(), g));
  }
  return B200_OK;
}

int launch_skinny_f32(float* C, const void* A, const void* W, const float* bias, int rows, int n, int K, int dtype,
                      cudaStream_t st) {
  SmallGemv g;
  g.a = W; g.lda = K; g.sa = (int64_t)kSmallRows * K;
  g.w = A; g.sw = 0;
  g.c = C; g.ldc = 1; g.sc = kSmallRows; g.nc = n; g.c_f32 = true;
  g.M = kSmallRows; g.m_total = n; g.N = rows; g.K = K; g.items = (n + kSmallRows - 1) / kSmallRows;
  g.bias_m = bias;
  return launch_small_gemv(g, dtype, st);
}

int launch_latent_pack(const LatentPack& p, cudaStream_t st) {
  B200_CHECK_ARG(p.kp && p.cache_rows && p.proj && p.qa && p.kbuf && p.qbuf && p.ctx > 0 && p.count > 0, "latent pack: null argument");
  B200_CUDA(launch_pdl(latent_pack_kernel, dim3(p.ctx + p.count), dim3(128), 0, st, false, p));
  return B200_OK;
}

int launch_stack_rmsnorm_rows(void* y, int64_t ld_y, const void* x, int64_t ld_x, const float* w, int64_t rows, int dim, int dim_pad,
                              float eps, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(y && x && w && rows > 0 && dim > 0 && ld_y >= std::max(dim, dim_pad) && ld_x >= dim, "stack rmsnorm rows: bad arguments");
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_rmsnorm_rows_kernel<float>, dim3((unsigned)rows), dim3(128), 0, st, stack_pdl(), (float*)y, ld_y,
                         (const float*)x, ld_x, w, dim, dim_pad, eps));
  else
    B200_CUDA(launch_pdl(stack_rmsnorm_rows_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(128), 0, st, stack_pdl(),
                         (__nv_bfloat16*)y, ld_y, (const __nv_bfloat16*)x, ld_x, w, dim, dim_pad, eps));
  return B200_OK;
}

int launch_stack_sigmoid_gate(void* y, int64_t ld_y, const void* g, int64_t ld_g, int64_t rows, int n, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(y && g && rows > 0 && n > 0 && ld_y >= n && ld_g >= n, "stack sigmoid gate: bad arguments");
  const int64_t total = rows * n;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 4 * 148);
  if (dtype == B200_F32)
    B200_CUDA(launch_pdl(stack_sigmoid_gate_kernel<float>, dim3(grid), dim3(256), 0, st, stack_pdl(), (float*)y, ld_y,
                         (const float*)g, ld_g, n, total));
  else
    B200_CUDA(launch_pdl(stack_sigmoid_gate_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, stack_pdl(), (__nv_bfloat16*)y,
                         ld_y, (const __nv_bfloat16*)g, ld_g, n, total));
  return B200_OK;
}

// the per-head query rows: the caller's, or the q segment of the merged projection
static LatentRun latent_with_q(const LatentRun& p, int dtype) {
  LatentRun q = p;
  if (q.q == nullptr) {
    q.q = (const uint8_t*)p.proj + (size_t)p.off_q * (dtype == B200_F32 ? 4 : 2);
    q.ld_q = p.ld_proj;
  }
  return q;
}

int launch_latent_prep(const LatentRun& p0, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  const LatentRun p = latent_with_q(p0, dtype);
  B200_CHECK_ARG(p.proj && p.cache && p.slot && p.pos && p.qa && p.n_tok > 0, "latent prep: null argument");
  if (dtype == B200_F32) B200_CUDA(launch_pdl(latent_prep_kernel<float>, dim3(p.n_tok), dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(latent_prep_kernel<__nv_bfloat16>, dim3(p.n_tok), dim3(128), 0, st, stack_pdl(), p));
  return B200_OK;
}

int run_latent_attention(const LatentRun& p0, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  const LatentRun p = latent_with_q(p0, dtype);
  const int r = p.l.kv_rank, dr = p.l.rot_dim, H = p.a.heads, dn = p.a.dim, kd = r + dr;
  B200_CHECK_ARG(p.proj && p.cache && p.slot && p.pos && p.qa && p.ol && p.out && p.n_tok > 0, "latent attention: null argument");
  B200_CHECK_ARG(H > 0 && dn > 0 && p.a.vdim > 0 && r > 0 && dr >= 0 && p.l.rot_dims >= 0 && p.l.rot_dims <= dr &&
                     p.l.rot_dims % 2 == 0,
                 "latent attention: bad sizes");
  B200_CHECK_ARG(r <= kLatentMaxRank, "latent attention: kv_rank above %d not built", kLatentMaxRank);
  B200_CHECK_ARG(p.l.c_norm && p.l.uk_t && p.l.uv && (p.l.rot_dims == 0 || p.l.rot_table), "latent attention: null weight");
  int rc;
  if (dtype == B200_F32) B200_CUDA(launch_pdl(latent_prep_kernel<float>, dim3(p.n_tok), dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(latent_prep_kernel<__nv_bfloat16>, dim3(p.n_tok), dim3(128), 0, st, stack_pdl(), p));
  const size_t esz = dtype == B200_F32 ? 4 : 2;
  const bool small = p.n_tok <= kSmallRows;
  // folded query of head h = uk_hᵀ · q_plain of head h
  if (small) {
    SmallGemv g;
    g.a = p.q; g.lda = p.ld_q; g.sa = dn + dr;
    g.w = p.l.uk_t; g.sw = (int64_t)r * dn;
    g.c = p.qa; g.ldc = (int64_t)H * kd; g.sc = kd;
    g.M = p.n_tok; g.N = r; g.K = dn; g.items = H;
    if ((rc = launch_small_gemv(g, dtype, st)) != B200_OK) return rc;
  } else {
    StackGemm g;
    g.a = p.q; g.lda = p.ld_q; g.k1 = dn; g.sa = dn + dr;
    g.w = p.l.uk_t; g.sw = (int64_t)r * dn;
    g.M = p.n_tok; g.N = r; g.K = dn; g.batch = H;
    g.epi = SEPI_STORE; g.c = p.qa; g.ldc = (int64_t)H * kd; g.sc = kd;
    if ((rc = launch_stack_gemm(g, dtype, st)) != B200_OK) return rc;
  }
  const size_t split_smem = (size_t)(H + 32) * kd * 4;
  if (small && p.split_ws != nullptr && p.nsplit >= 1 && H <= 8 * kLatHeadsPerWarp && kd <= 32 * kLatKeyRegs && r <= 32 * kLatVR &&
      split_smem <= 200 * 1024) {
    static bool attr_done = false;
    if (!attr_done) {
      B200_CUDA(cudaFuncSetAttribute(latent_attn_split_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      B200_CUDA(cudaFuncSetAttribute(latent_attn_split_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_done = true;
    }
    const dim3 grid(p.n_tok, p.nsplit);
    LatentRun q = p;
    const size_t al = dtype == B200_F32 ? 32 : 16;
    q.stage_vec = ((size_t)kd * esz) % al == 0 && (reinterpret_cast<uintptr_t>(p.cache) % al) == 0 &&
                  ((size_t)p.slot_stride * esz) % al == 0 && (reinterpret_cast<uintptr_t>(p.qa) % al) == 0;
    if (dtype == B200_F32) {
      B200_CUDA(launch_pdl(latent_attn_split_kernel<float>, grid, dim3(256), split_smem, st, stack_pdl(), q));
      B200_CUDA(launch_pdl(latent_merge_kernel<float>, dim3(p.n_tok, H), dim3(256), 0, st, stack_pdl(), q));
    } else {
      B200_CUDA(launch_pdl(latent_attn_split_kernel<__nv_bfloat16>, grid, dim3(256), split_smem, st, stack_pdl(), q));
      B200_CUDA(launch_pdl(latent_merge_kernel<__nv_bfloat16>, dim3(p.n_tok, H), dim3(256), 0, st, stack_pdl(), q));
    }
  } else {
    const size_t smem = (size_t)(kd + 4 * (2 + r)) * 4;
    const dim3 grid(p.n_tok, H);
    if (r <= 32 * kLatVR) {
      if (dtype == B200_F32) B200_CUDA(launch_pdl(latent_attn_kernel<float, kLatVR>, grid, dim3(128), smem, st, stack_pdl(), p));
      else B200_CUDA(launch_pdl(latent_attn_kernel<__nv_bfloat16, kLatVR>, grid, dim3(128), smem, st, stack_pdl(), p));
    } else {
      constexpr int kWide = kLatentMaxRank / 32;
      if (dtype == B200_F32) B200_CUDA(launch_pdl(latent_attn_kernel<float, kWide>, grid, dim3(128), smem, st, stack_pdl(), p));
      else B200_CUDA(launch_pdl(latent_attn_kernel<__nv_bfloat16, kWide>, grid, dim3(128), smem, st, stack_pdl(), p));
    }
  }
  // head h's output = uv_h · (softmax-weighted latent of head h)
  if (small) {
    SmallGemv v;
    v.a = p.ol; v.lda = (int64_t)H * r; v.sa = r;
    v.w = p.l.uv; v.sw = (int64_t)p.a.vdim * r;
    v.c = p.out; v.ldc = p.ld_out; v.sc = p.a.vdim;
    v.M = p.n_tok; v.N = p.a.vdim; v.K = r; v.items = H;
    return launch_small_gemv(v, dtype, st);
  }
  StackGemm v;
  v.a = p.ol; v.lda = (int64_t)H * r; v.k1 = r; v.sa = r;
  v.w = p.l.uv; v.sw = (int64_t)p.a.vdim * r;
  v.M = p.n_tok; v.N = p.a.vdim; v.K = r; v.batch = H;
  v.epi = SEPI_STORE; v.c = p.out; v.ldc = p.ld_out; v.sc = p.a.vdim;
  return launch_stack_gemm(v, dtype, st);
}

int run_mlstm(const MlstmRun& p, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(p.proj && p.gates && p.state && p.slot && p.pos && p.o && p.n_seg > 0 && p.n_tok > 0, "mlstm: null argument");
  B200_CHECK_ARG(p.a.heads > 0 && p.a.dim > 0 && p.a.vdim > 0 && p.gate_cap > 0.f, "mlstm: bad sizes");
  B200_CHECK_ARG(p.a.dim <= kMlstmMaxDim, "mlstm: key size above %d not built", kMlstmMaxDim);
  B200_CHECK_ARG(p.gab != nullptr, "mlstm: null gate workspace");
  B200_CUDA(launch_pdl(mlstm_gates_kernel, dim3(p.n_seg, p.a.heads), dim3(32), 0, st, stack_pdl(), p));
  const dim3 grid(p.n_seg, p.a.heads, (p.a.vdim + 1 + 7) / 8);
#define B200_SCAN(DR)                                                                                              \
  do {                                                                                                             \
    if (dtype == B200_F32) B200_CUDA(launch_pdl(mlstm_scan_kernel<float, DR>, grid, dim3(256), 0, st, stack_pdl(), p)); \
    else B200_CUDA(launch_pdl(mlstm_scan_kernel<__nv_bfloat16, DR>, grid, dim3(256), 0, st, stack_pdl(), p));     \
  } while (0)
  if (p.a.dim <= 32) B200_SCAN(1);
  else if (p.a.dim <= 64) B200_SCAN(2);
  else if (p.a.dim <= 128) B200_SCAN(4);
  else if (p.a.dim <= 256) B200_SCAN(8);
  else B200_SCAN(16);
#undef B200_SCAN
  if (p.mid == nullptr) return B200_OK;
  B200_CHECK_ARG(p.head_norm != nullptr, "mlstm: null head norm");
  const dim3 og((p.n_tok * p.a.heads + 3) / 4);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(mlstm_out_kernel<float>, og, dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(mlstm_out_kernel<__nv_bfloat16>, og, dim3(128), 0, st, stack_pdl(), p));
  return B200_OK;
}

int run_moe(const MoeRun& p, int dtype, cudaStream_t st) {
  MIX_DTYPE_CHECK(dtype);
  const b200_moe_desc& m = p.m;
  B200_CHECK_ARG(p.h && p.z && p.sel_e && p.sel_w && p.plan && p.pair_slot && p.a_perm && p.gu && p.act && p.outp && p.y &&
                     p.n_tok > 0 && p.width > 0,
                 "moe: null argument");
  B200_CHECK_ARG(m.experts > 0 && m.top > 0 && m.top <= m.experts && m.expert_ff > 0 && m.router && m.w_exp_in && m.w_exp_out,
                 "moe: bad description");
  B200_CHECK_ARG(m.experts <= 8192, "moe: more than 8192 experts not built");
  const int P = p.n_tok * m.top, n_tiles = moe_tiles(P, m.experts), E = m.experts, S = p.plan_stride > 0 ? p.plan_stride : E;
  B200_CHECK_ARG(S >= E, "moe: plan stride below the expert count");
  B200_CHECK_ARG(m.router_kind == 0 || m.router_kind == 1, "moe: router kind %d", m.router_kind);
  int rc;
  // rows of an expert's in-projection: gate | up of the clamped gated unit, or up alone under a plain activation
  const int n_up = m.expert_act != 0 ? m.expert_ff : 2 * m.expert_ff;
  auto hidden = [&]() -> int {
    if (m.expert_act != 0) return launch_stack_act_mul(p.act, m.expert_ff, p.gu, nullptr, n_up, P, m.expert_ff, m.expert_act, dtype, st);
    return launch_stack_glu_clamp(p.act, m.expert_ff, p.gu, n_up, P, m.expert_ff, m.limit, dtype, st);
  };
  if (p.small) {   // a few tokens: router, then every (token, choice) pair is an item of a small product with its expert
    B200_CHECK_ARG(p.n_tok <= kSmallRows, "moe: the small path takes up to %d tokens", kSmallRows);
    SmallGemv rz;
    rz.a = p.h; rz.lda = p.width; rz.w = m.router; rz.c = p.z; rz.ldc = E; rz.c_f32 = true;
    rz.M = p.n_tok; rz.N = E; rz.K = p.width; rz.items = 1;
    if ((rc = launch_small_gemv(rz, dtype, st)) != B200_OK) return rc;
    B200_CUDA(launch_pdl(moe_route_kernel, dim3((p.n_tok + 3) / 4), dim3(128), 0, st, stack_pdl(), p));
    SmallGemv g;
    if (m.weight_output) {   // the experts read the token's row itself: no weighted copies to make
      g.a = p.h; g.sa = p.width; g.item_div = m.top;
    } else {
      if (dtype == B200_F32) B200_CUDA(launch_pdl(moe_gather_kernel<float>, dim3(P), dim3(128), 0, st, stack_pdl(), p));
      else B200_CUDA(launch_pdl(moe_gather_kernel<__nv_bfloat16>, dim3(P), dim3(128), 0, st, stack_pdl(), p));
      g.a = p.a_perm; g.sa = p.width;
    }
    g.w = m.w_exp_in; g.sw = (int64_t)n_up * p.width; g.item_mat = p.sel_e;
    g.M = 1; g.N = n_up; g.K = p.width; g.items = P;
    const bool act_in_product = m.expert_act == B200_ACT_RELU2 || m.expert_act == B200_ACT_TANH || m.expert_act == B200_ACT_SILU;
    if (act_in_product) {   // a plain activation rides on the product's store: the hidden rows leave in one launch
      g.c = p.act; g.sc = m.expert_ff; g.act = m.expert_act;
      if ((rc = launch_small_gemv(g, dtype, st)) != B200_OK) return rc;
    } else {
      g.c = p.gu; g.sc = n_up;
      if ((rc = launch_small_gemv(g, dtype, st)) != B200_OK) return rc;
      if ((rc = hidden()) != B200_OK) return rc;
    }
    SmallGemv d;
    d.a = p.act; d.sa = m.expert_ff; d.w = m.w_exp_out; d.sw = (int64_t)p.width * m.expert_ff; d.item_mat = p.sel_e;
    d.c = p.outp; d.sc = p.width; d.c_f32 = true; d.M = 1; d.N = p.width; d.K = m.expert_ff; d.items = P;
    if ((rc = launch_small_gemv(d, dtype, st)) != B200_OK) return rc;
  } else {
  // router logits in fp32
  if ((rc = launch_skinny_f32(p.z, p.h, m.router, nullptr, p.n_tok, E, p.width, dtype, st)) != B200_OK) return rc;
  B200_CUDA(launch_pdl(moe_route_kernel, dim3((p.n_tok + 3) / 4), dim3(128), 0, st, stack_pdl(), p));
  B200_CUDA(launch_pdl(moe_plan_kernel, dim3(1), dim3(256), (size_t)E * 4, st, stack_pdl(), p));
  if (dtype == B200_F32) B200_CUDA(launch_pdl(moe_gather_kernel<float>, dim3(P), dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(moe_gather_kernel<__nv_bfloat16>, dim3(P), dim3(128), 0, st, stack_pdl(), p));
  if (p.tc) {
    B200_CHECK_ARG(dtype == B200_BF16 && p.outp_bf != nullptr, "moe: the tensor-core path is bf16");
    std::vector<int32_t> ends(E);
    B200_CUDA(cudaMemcpyAsync(ends.data(), p.plan + S, (size_t)E * 4, cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    const __nv_bfloat16* A = (const __nv_bfloat16*)p.a_perm;
    __nv_bfloat16 *GU = (__nv_bfloat16*)p.gu, *ACT = (__nv_bfloat16*)p.act;
    const int64_t f2 = n_up;
    // one expert's rows rarely fill the GPU: the experts' products go round eight side streams that fork from and join
    // back into the step's stream
    constexpr int kSide = 8;
    static cudaStream_t side[kSide];
    static cudaEvent_t fork_ev, join_ev[kSide];
    static bool side_ok = false;
    if (!side_ok) {
      for (int i = 0; i < kSide; ++i) {
        B200_CUDA(cudaStreamCreateWithFlags(&side[i], cudaStreamNonBlocking));
        B200_CUDA(cudaEventCreateWithFlags(&join_ev[i], cudaEventDisableTiming));
      }
      B200_CUDA(cudaEventCreateWithFlags(&fork_ev, cudaEventDisableTiming));
      side_ok = true;
    }
    auto fork = [&]() -> int {
      B200_CUDA(cudaEventRecord(fork_ev, st));
      for (int i = 0; i < kSide; ++i) B200_CUDA(cudaStreamWaitEvent(side[i], fork_ev, 0));
      return B200_OK;
    };
    auto join = [&]() -> int {
      for (int i = 0; i < kSide; ++i) {
        B200_CUDA(cudaEventRecord(join_ev[i], side[i]));
        B200_CUDA(cudaStreamWaitEvent(st, join_ev[i], 0));
      }
      return B200_OK;
    };
    if ((rc = fork()) != B200_OK) return rc;
    for (int e = 0, row = 0, n = 0; e < E; row = ends[e], ++e)
      if (ends[e] > row && (rc = launch_gemm_bf16(GU + (int64_t)row * f2, A + (int64_t)row * p.width,
                                                  (const __nv_bfloat16*)m.w_exp_in + (int64_t)e * f2 * p.width, ends[e] - row, f2,
                                                  p.width, side[n++ % kSide])) != B200_OK)
        return rc;
    if ((rc = join()) != B200_OK) return rc;
    if ((rc = hidden()) != B200_OK) return rc;
    if ((rc = fork()) != B200_OK) return rc;
    for (int e = 0, row = 0, n = 0; e < E; row = ends[e], ++e)
      if (ends[e] > row && (rc = launch_gemm_bf16(p.outp_bf + (int64_t)row * p.width, ACT + (int64_t)row * m.expert_ff,
                                                  (const __nv_bfloat16*)m.w_exp_out + (int64_t)e * p.width * m.expert_ff,
                                                  ends[e] - row, p.width, m.expert_ff, side[n++ % kSide])) != B200_OK)
        return rc;
    if ((rc = join()) != B200_OK) return rc;
  } else {
  StackGemm g;
  g.a = p.a_perm; g.lda = p.width; g.k1 = p.width;
  g.w = m.w_exp_in; g.sw = (int64_t)n_up * p.width;
  g.M = P; g.N = n_up; g.K = p.width;
  g.epi = SEPI_STORE; g.c = p.gu; g.ldc = n_up;
  g.tile_group = p.plan + 2 * S; g.tile_row0 = p.plan + 2 * S + n_tiles; g.group_end = p.plan + S; g.n_tiles = n_tiles;
  if ((rc = launch_stack_gemm(g, dtype, st)) != B200_OK) return rc;
  if ((rc = hidden()) != B200_OK) return rc;
  StackGemm d;
  d.a = p.act; d.lda = m.expert_ff; d.k1 = m.expert_ff;
  d.w = m.w_exp_out; d.sw = (int64_t)p.width * m.expert_ff;
  d.M = P; d.N = p.width; d.K = m.expert_ff;
  d.epi = SEPI_STORE_F32; d.c = p.outp; d.ldc = p.width;
  d.tile_group = g.tile_group; d.tile_row0 = g.tile_row0; d.group_end = g.group_end; d.n_tiles = n_tiles;
  if ((rc = launch_stack_gemm(d, dtype, st)) != B200_OK) return rc;
  }
  }
  const dim3 cg(p.n_tok, (p.width + 255) / 256);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(moe_combine_kernel<float>, cg, dim3(256), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(moe_combine_kernel<__nv_bfloat16>, cg, dim3(256), 0, st, stack_pdl(), p));
  return B200_OK;
}

}  // namespace b200
