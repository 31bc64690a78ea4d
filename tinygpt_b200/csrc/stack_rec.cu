// stack_rec.cu — mixers of post-norm blocks as plain kernels: the preparation of an attention mixer's projection rows, one
// scan for linear recurrences with a per-channel or per-head decay and an optional rank-one removal, the passes of the
// generalized delta rule and of Mamba-2 around it, and the post-norm that also leaves the next sublayer's operand copy.
// fp32 for norms, angles, gates, decays, step sizes, the recurrence and its state; storage type T = bf16 or fp32.
// Every kernel starts with griddepcontrol.launch_dependents + griddepcontrol.wait (programmatic dependent launch).
#include "stack_rec.cuh"

#include <algorithm>

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
__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float siluf(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------------------------------------ attention preparation
// One CTA per token.  q and k: the sum of squares over the WHOLE projection (all heads), the weight of that entry, then the
// rotation of the first rot_dims entries of every head (entry i with entry i + rot_dims/2).  v: every head by its own root
// mean square, then the mix with the kept values.  All in fp32 from the T-typed projection, written back as T once.
template <typename T>
__global__ void __launch_bounds__(256) attn_prep_kernel(const AttnPrep p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = p.a.heads, G = p.a.kv_heads, dk = p.a.dim, dv = p.a.vdim;
  const int half = p.d.rot_dims / 2, items = dk - half;   // per head: `half` pairs, then the entries from rot_dims on
  T* row = static_cast<T*>(p.proj) + (int64_t)t * p.ld_proj;
  const float* tab = half > 0 ? p.d.rot_table + (int64_t)p.pos[t] * half * 2 : nullptr;
  for (int which = 0; which < 2; ++which) {
    T* x = row + (which ? p.off_k : p.off_q);
    const int n = (which ? G : H) * dk, nh = which ? G : H;
    const float* w = which ? p.d.k_norm : p.d.q_norm;
    float inv = 1.f;
    if (p.d.qk_norm) {
      float ss = 0.f;
      for (int i = tid; i < n; i += 256) {
        const float v = ldf<T>(x + i);
        ss += v * v;
      }
      inv = 1.f / sqrtf(block_sum(ss, red) / (float)n + p.eps);
    }
    if (!p.d.qk_norm && half == 0) continue;
    for (int e = tid; e < nh * items; e += 256) {
      const int hd = e / items, j = e % items;
      if (j < half) {
        const int i0 = hd * dk + j, i1 = i0 + half;
        float a = ldf<T>(x + i0) * inv, b = ldf<T>(x + i1) * inv;
        if (p.d.qk_norm) {
          a *= w[i0];
          b *= w[i1];
        }
        const float c = tab[2 * j], s = tab[2 * j + 1];
        x[i0] = cvt<T>(a * c - b * s);
        x[i1] = cvt<T>(b * c + a * s);
      } else if (p.d.qk_norm) {
        const int i = hd * dk + j + half;
        x[i] = cvt<T>(ldf<T>(x + i) * inv * w[i]);
      }
    }
  }
  if (!p.d.v_norm && p.d.v_mix == 0) return;
  T* v = row + p.off_v;
  T* keep = p.vkeep != nullptr ? static_cast<T*>(p.vkeep) + (int64_t)t * p.ld_keep : nullptr;
  const float lam = p.d.v_mix == 2 ? p.d.mix_lambda[0] : 0.f;
  const int warp = tid >> 5, lane = tid & 31;
  for (int g = warp; g < G; g += 8) {
    float inv = 1.f;
    if (p.d.v_norm) {
      float ss = 0.f;
      for (int i = lane; i < dv; i += 32) {
        const float a = ldf<T>(v + g * dv + i);
        ss += a * a;
      }
      inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + p.eps);
    }
    for (int i = lane; i < dv; i += 32) {
      float a = ldf<T>(v + g * dv + i) * inv;
      if (p.d.v_mix == 2) a = (1.f - lam) * a + lam * ldf<T>(keep + g * dv + i);
      v[g * dv + i] = cvt<T>(a);
      if (p.d.v_mix == 1) keep[g * dv + i] = cvt<T>(a);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------ the scan
// One warp per (sequence, head, value column): lane l holds rows l, l + 32, … of its column of S (DR rows per lane); eight
// columns per CTA.  The CTA walks its sequence CH tokens at a time: the chunk's decay, removal, unit key, key and query
// rows (fp32, zero past dk) and the eight columns' values sit in shared memory, staged once for all eight warps.  A token
// costs a warp the removal's dot with the OLD column (one warp sum the update waits for), DR multiply-adds per operand and
// the output's dot with the NEW column.  Columns never read each other, so the logits of a sequence do not depend on what
// else is in the step; the order of the sums inside a column is fixed by dk alone.
template <int DR, bool REMOVE>
__global__ void __launch_bounds__(256) lin_scan_kernel(const LinScan p) {
  pdl_trigger();
  pdl_wait();
  constexpr int DK = 32 * DR;
  constexpr int CH = 2048 / DK >= 32 ? 32 : 2048 / DK;   // tokens per chunk
  constexpr int NV = REMOVE ? 5 : 3;                      // staged vectors per token: d, b, r (, p, q)
  __shared__ float s_x[CH][NV][DK];
  __shared__ float s_v[CH][8];
  const int seg = blockIdx.x, hd = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int dk = p.dk, dv = p.dv;
  const int j0 = blockIdx.z * 8, j = j0 + warp;
  const bool live = j < dv;
  const int r0 = p.seg_row0 != nullptr ? p.seg_row0[seg] : seg;
  const int cnt = p.seg_count != nullptr ? p.seg_count[seg] : 1;
  float* st = p.state + (int64_t)p.slot[r0] * p.slot_stride + (int64_t)hd * dk * dv;
  const bool fresh = p.pos[r0] == 0;
  float S[DR];
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = lane + 32 * i;
    S[i] = (live && !fresh && d < dk) ? st[(int64_t)d * dv + j] : 0.f;
  }
  const int hs = hd / p.share;   // the head whose b / r vectors this head reads
  for (int c0 = 0; c0 < cnt; c0 += CH) {
    const int n = min(CH, cnt - c0);
    __syncthreads();   // the previous chunk has been read
    for (int e = tid; e < n * NV * DK; e += 256) {
      const int t = e / (NV * DK), w = (e / DK) % NV, d = e % DK;
      const float* row;
      float val = 0.f;
      if (d < dk) {
        const int64_t base = (int64_t)(r0 + c0 + t) * p.ld;
        switch (w) {
          case 0: val = p.d_scalar ? p.d[base + hd] : p.d[base + (int64_t)hd * dk + d]; break;
          case 1: row = p.b + base + (int64_t)hs * dk; val = row[d]; break;
          case 2: row = p.r + base + (int64_t)hs * dk; val = row[d]; break;
          case 3: val = p.p[base + (int64_t)hd * dk + d]; break;
          default: val = p.q[base + (int64_t)hd * dk + d]; break;
        }
      }
      s_x[t][w][d] = val;
    }
    for (int e = tid; e < n * 8; e += 256) {
      const int t = e / 8, c = j0 + e % 8;
      const int64_t base = (int64_t)(r0 + c0 + t) * p.ld;
      float val = c < dv ? p.v[base + (int64_t)hd * dv + c] : 0.f;
      if (p.vscale != nullptr) val *= p.vscale[base + hd];
      s_v[t][e % 8] = val;
    }
    __syncthreads();
    if (!live) continue;
    for (int t = 0; t < n; ++t) {
      const float vj = s_v[t][warp];
      float rem = 0.f;
      if constexpr (REMOVE) {
#pragma unroll
        for (int i = 0; i < DR; ++i) rem = fmaf(s_x[t][4][lane + 32 * i], S[i], rem);
        rem = warp_sum(rem);
      }
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < DR; ++i) {
        const int d = lane + 32 * i;
        float sn = s_x[t][0][d] * S[i];
        if constexpr (REMOVE) sn = fmaf(-s_x[t][3][d], rem, sn);
        sn = fmaf(s_x[t][1][d], vj, sn);
        S[i] = sn;
        dot = fmaf(sn, s_x[t][2][d], dot);
      }
      dot = warp_sum(dot);
      if (lane == 0) p.o[(int64_t)(r0 + c0 + t) * p.ld_o + (int64_t)hd * dv + j] = dot;
    }
  }
  if (!live) return;
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int d = lane + 32 * i;
    if (d < dk) st[(int64_t)d * dv + j] = S[i];
  }
}

// ------------------------------------------------------------------------------------------- generalized delta rule
// One warp per (token, head): decay w = exp(−c·sigmoid(wl)), removal a = sigmoid(logit), unit key u = k / sqrt(Σk² + ε); the
// scan's rows [decay | a∘u | u | k | r | v] in fp32.
template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(const DeltaRun p) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int H = p.a.heads, dk = p.a.dim, dv = p.a.vdim;
  if (pair >= p.scan.n_tok * H) return;
  const int t = pair / H, hd = pair % H;
  const T* row = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj;
  const T* k = row + p.off_k + hd * dk;
  float ss = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float v = ldf<T>(k + i);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) + p.d.unit_eps);
  float* f = p.f + (int64_t)t * p.scan.ld;
  const int64_t n = (int64_t)H * dk;
  for (int i = lane; i < dk; i += 32) {
    const int c = hd * dk + i;
    const float kv = ldf<T>(k + i), u = kv * inv;
    f[c] = expf(-p.d.decay_scale * sigmoidf(p.wl[(int64_t)t * n + c]));
    f[n + c] = sigmoidf(ldf<T>(row + p.off_a + c)) * u;
    f[2 * n + c] = u;
    f[3 * n + c] = kv;
    f[4 * n + c] = ldf<T>(row + p.off_r + c);
  }
  for (int i = lane; i < dv; i += 32) f[5 * n + hd * dv + i] = ldf<T>(row + p.off_v + hd * dv + i);
}

// One warp per (token, head): o / rms(o) · head_norm · sigmoid(out gate)
template <typename T>
__global__ void __launch_bounds__(128) delta_out_kernel(const DeltaRun p) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int H = p.a.heads, dv = p.a.vdim;
  if (pair >= p.scan.n_tok * H) return;
  const int t = pair / H, hd = pair % H;
  const float* o = p.scan.o + (int64_t)t * p.scan.ld_o + hd * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += o[c] * o[c];
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + p.eps);
  const T* g = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj + p.off_g + hd * dv;
  T* y = static_cast<T*>(p.mid) + (int64_t)t * p.ld_mid + hd * dv;
  for (int c = lane; c < dv; c += 32) y[c] = cvt<T>(o[c] * inv * p.d.head_norm[hd * dv + c] * sigmoidf(ldf<T>(g + c)));
}

// -------------------------------------------------------------------------------------------------------------- Mamba-2
// One thread per (sequence, channel) walks the sequence's rows in order with the last taps − 1 inputs in registers (from
// the slot's state, or zeros at position 0): convolution + bias + SiLU into the fp32 workspace, and at the end the slot's
// new last inputs — the thread is the only reader and writer of its channel's state.  The threads past the channels serve
// one head each: dt = softplus(logit + bias) and the decay exp(−exp(A_log)·dt) of every row.
template <typename T>
__global__ void __launch_bounds__(128) mamba_conv_kernel(const MambaRun p) {
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
  const int H = p.a.heads, inner = H * p.a.vdim, ch = inner + 2 * p.m.groups * p.m.state, taps = p.m.taps;
  const int r0 = p.scan.seg_row0 != nullptr ? p.scan.seg_row0[seg] : seg;
  const int cnt = p.scan.seg_count != nullptr ? p.scan.seg_count[seg] : 1;
  if (c >= ch + H) return;
  if (c >= ch) {
    const int hd = c - ch;
    const float bias = p.m.dt_bias[hd], rate = expf(p.m.A_log[hd]);
    for (int t = 0; t < cnt; ++t) {
      float* f = p.f + (int64_t)(r0 + t) * p.scan.ld;
      const float dt = softplusf(p.dt[(int64_t)(r0 + t) * p.ld_dt + hd] + bias);
      f[ch + hd] = expf(-rate * dt);
      f[ch + H + hd] = dt;
    }
    return;
  }
  float* cs = p.conv_state + (int64_t)p.scan.slot[r0] * p.scan.slot_stride;
  const bool fresh = p.scan.pos[r0] == 0;
  float win[kMambaMaxTaps], w[kMambaMaxTaps];   // win[taps − 1] is the current input
#pragma unroll
  for (int j = 0; j < kMambaMaxTaps; ++j) {
    w[j] = j < taps ? p.m.conv_w[(int64_t)c * taps + j] : 0.f;
    win[j] = (j < taps - 1 && !fresh) ? cs[(int64_t)j * ch + c] : 0.f;
  }
  const float bias = p.m.conv_b[c];
  const T* x = static_cast<const T*>(p.proj) + p.off_x + c;
  for (int t = 0; t < cnt; ++t) {
    const float cur = ldf<T>(x + (int64_t)(r0 + t) * p.ld_proj);
    float acc = bias;
#pragma unroll
    for (int j = 0; j < kMambaMaxTaps; ++j) {
      if (j == taps - 1) win[j] = cur;
      if (j < taps) acc = fmaf(w[j], win[j], acc);
    }
    p.f[(int64_t)(r0 + t) * p.scan.ld + c] = siluf(acc);
#pragma unroll
    for (int j = 0; j + 1 < kMambaMaxTaps; ++j) win[j] = win[j + 1];
  }
#pragma unroll
  for (int j = 0; j < kMambaMaxTaps; ++j)
    if (j < taps - 1) cs[(int64_t)j * ch + c] = win[j];
}

// One CTA per token: y = o + D·x, · silu(z), an RMS norm in norm_groups equal parts, · norm
template <typename T>
__global__ void __launch_bounds__(256) mamba_out_kernel(const MambaRun p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = p.a.heads, dv = p.a.vdim, inner = H * dv, part = inner / p.m.norm_groups;
  const float* o = p.scan.o + (int64_t)t * p.scan.ld_o;
  const float* x = p.f + (int64_t)t * p.scan.ld;
  const T* z = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj + p.off_z;
  T* y = static_cast<T*>(p.mid) + (int64_t)t * p.ld_mid;
  for (int g = 0; g < p.m.norm_groups; ++g) {
    float ss = 0.f;
    for (int i = g * part + tid; i < (g + 1) * part; i += 256) {
      const float v = (o[i] + p.m.D[i / dv] * x[i]) * siluf(ldf<T>(z + i));
      ss += v * v;
    }
    const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)part + p.eps);
    for (int i = g * part + tid; i < (g + 1) * part; i += 256) {
      const float v = (o[i] + p.m.D[i / dv] * x[i]) * siluf(ldf<T>(z + i));
      y[i] = cvt<T>(v * inv * p.m.norm[i]);
    }
  }
}

// --------------------------------------------------------------------------------- post-norm + residual + operand copy
template <typename YT>
__global__ void __launch_bounds__(256) stack_rms_add_cast_kernel(float* __restrict__ x, const YT* __restrict__ y,
                                                                 const float* __restrict__ w, __nv_bfloat16* __restrict__ h,
                                                                 int dim, float eps, float mult) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const YT* yr = y + (int64_t)blockIdx.x * dim;
  float* xr = x + (int64_t)blockIdx.x * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) ss += ldf<YT>(yr + i) * ldf<YT>(yr + i);
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = xr[i] + mult * (ldf<YT>(yr + i) * inv * w[i]);
    xr[i] = v;
    if (h != nullptr) h[(int64_t)blockIdx.x * dim + i] = __float2bfloat16_rn(v);
  }
}

}  // namespace

#define REC_DTYPE_CHECK(dtype) \
  B200_CHECK_ARG((dtype) == B200_BF16 || (dtype) == B200_F32, "stack op: unknown dtype %d", (int)(dtype))

int launch_attn_prep(const AttnPrep& p, int dtype, cudaStream_t st) {
  REC_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(p.proj && p.pos && p.n_tok > 0, "attention prep: null argument");
  B200_CHECK_ARG(p.d.rot_dims >= 0 && p.d.rot_dims % 2 == 0 && p.d.rot_dims <= p.a.dim && (p.d.rot_dims == 0 || p.d.rot_table),
                 "attention prep: rot_dims %d must be even, at most the head size %d, with a table", p.d.rot_dims, p.a.dim);
  B200_CHECK_ARG(!p.d.qk_norm || (p.d.q_norm && p.d.k_norm), "attention prep: null norm weight");
  B200_CHECK_ARG(p.d.v_mix >= 0 && p.d.v_mix <= 2 && (p.d.v_mix == 0 || p.vkeep) && (p.d.v_mix != 2 || p.d.mix_lambda),
                 "attention prep: value mix-in without its buffer or weight");
  if (dtype == B200_F32) B200_CUDA(launch_pdl(attn_prep_kernel<float>, dim3(p.n_tok), dim3(256), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(attn_prep_kernel<__nv_bfloat16>, dim3(p.n_tok), dim3(256), 0, st, stack_pdl(), p));
  return B200_OK;
}

int launch_lin_scan(const LinScan& p, cudaStream_t st) {
  B200_CHECK_ARG(p.d && p.b && p.r && p.v && p.state && p.slot && p.pos && p.o && p.n_seg > 0 && p.n_tok > 0,
                 "linear scan: null argument");
  B200_CHECK_ARG((p.p == nullptr) == (p.q == nullptr), "linear scan: the removal needs both of its vectors");
  B200_CHECK_ARG(p.heads > 0 && p.dk > 0 && p.dv > 0 && p.share > 0 && p.heads % p.share == 0, "linear scan: bad sizes");
  B200_CHECK_ARG(p.dk <= kScanMaxDim, "linear scan: more than %d key channels not built", kScanMaxDim);
  const dim3 grid(p.n_seg, p.heads, (p.dv + 7) / 8);
#define B200_SCAN(DR)                                                                                    \
  do {                                                                                                   \
    if (p.p != nullptr) B200_CUDA(launch_pdl(lin_scan_kernel<DR, true>, grid, dim3(256), 0, st, stack_pdl(), p));  \
    else B200_CUDA(launch_pdl(lin_scan_kernel<DR, false>, grid, dim3(256), 0, st, stack_pdl(), p));     \
  } while (0)
  if (p.dk <= 32) B200_SCAN(1);
  else if (p.dk <= 64) B200_SCAN(2);
  else if (p.dk <= 128) B200_SCAN(4);
  else if (p.dk <= 256) B200_SCAN(8);
  else B200_SCAN(16);
#undef B200_SCAN
  return B200_OK;
}

int run_delta(const DeltaRun& p, int dtype, cudaStream_t st) {
  REC_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(p.proj && p.wl && p.f && p.scan.n_tok > 0, "delta rule: null argument");
  const int H = p.a.heads, dk = p.a.dim, dv = p.a.vdim;
  const dim3 grid((p.scan.n_tok * H + 3) / 4);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(delta_prep_kernel<float>, grid, dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(delta_prep_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, stack_pdl(), p));
  LinScan s = p.scan;
  const int64_t n = (int64_t)H * dk;
  s.heads = H; s.dk = dk; s.dv = dv; s.share = 1; s.d_scalar = 0;
  s.d = p.f; s.p = p.f + n; s.q = p.f + 2 * n; s.b = p.f + 3 * n; s.r = p.f + 4 * n; s.v = p.f + 5 * n; s.vscale = nullptr;
  int rc = launch_lin_scan(s, st);
  if (rc != B200_OK || p.mid == nullptr) return rc;
  B200_CHECK_ARG(p.d.head_norm != nullptr, "delta rule: null head norm");
  if (dtype == B200_F32) B200_CUDA(launch_pdl(delta_out_kernel<float>, grid, dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(delta_out_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, stack_pdl(), p));
  return B200_OK;
}

int run_mamba(const MambaRun& p, int dtype, cudaStream_t st) {
  REC_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(p.proj && p.dt && p.conv_state && p.f && p.mid && p.scan.n_tok > 0 && p.scan.n_seg > 0, "mamba2: null argument");
  const b200_mamba_desc& m = p.m;
  const int H = p.a.heads, dv = p.a.vdim, N = m.state, inner = H * dv, ch = inner + 2 * m.groups * N;
  B200_CHECK_ARG(m.taps >= 1 && m.taps <= kMambaMaxTaps, "mamba2: 1 … %d convolution taps", kMambaMaxTaps);
  B200_CHECK_ARG(m.groups > 0 && H % m.groups == 0 && m.norm_groups > 0 && inner % m.norm_groups == 0 && N > 0,
                 "mamba2: heads %d, groups %d, norm_groups %d do not divide", H, m.groups, m.norm_groups);
  B200_CHECK_ARG(m.conv_w && m.conv_b && m.dt_bias && m.A_log && m.D && m.norm, "mamba2: null weight");
  const dim3 cg(p.scan.n_seg, (ch + H + 127) / 128);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(mamba_conv_kernel<float>, cg, dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(mamba_conv_kernel<__nv_bfloat16>, cg, dim3(128), 0, st, stack_pdl(), p));
  LinScan s = p.scan;
  s.heads = H; s.dk = N; s.dv = dv; s.share = H / m.groups; s.d_scalar = 1;
  s.v = p.f; s.b = p.f + inner; s.r = p.f + inner + (int64_t)m.groups * N; s.d = p.f + ch; s.vscale = p.f + ch + H;
  s.p = s.q = nullptr;
  int rc = launch_lin_scan(s, st);
  if (rc != B200_OK) return rc;
  if (dtype == B200_F32) B200_CUDA(launch_pdl(mamba_out_kernel<float>, dim3(p.scan.n_tok), dim3(256), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(mamba_out_kernel<__nv_bfloat16>, dim3(p.scan.n_tok), dim3(256), 0, st, stack_pdl(), p));
  return B200_OK;
}

int launch_stack_rms_add_cast(float* x, const void* y, bool y_bf16, const float* w, __nv_bfloat16* h, int64_t rows, int dim,
                              float eps, float mult, cudaStream_t st) {
  B200_CHECK_ARG(x && y && w && rows > 0 && dim > 0, "stack rms_add_cast: bad arguments");
  if (y_bf16)
    B200_CUDA(launch_pdl(stack_rms_add_cast_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x,
                         (const __nv_bfloat16*)y, w, h, dim, eps, mult));
  else
    B200_CUDA(launch_pdl(stack_rms_add_cast_kernel<float>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x,
                         (const float*)y, w, h, dim, eps, mult));
  return B200_OK;
}

}  // namespace b200
