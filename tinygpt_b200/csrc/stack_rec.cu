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
// rotation of the first rot_dims entries of every head (entry i with entry i + rot_dims/2, or — rot_interleaved — entry 2i
// with entry 2i + 1).  v: every head by its own root
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
  for (int which = 0; which < (p.q_only ? 1 : 2); ++which) {
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
        const int i0 = hd * dk + (p.d.rot_interleaved ? 2 * j : j), i1 = i0 + (p.d.rot_interleaved ? 1 : half);
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
  if ((!p.d.v_norm && p.d.v_mix == 0) || p.q_only) return;
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
// One warp per (sequence, head, NC value columns): lane l holds rows l, l + 32, … of its columns of S (DR rows per lane and
// column); 8·NC columns per CTA.  The CTA walks its sequence CH tokens at a time: the chunk's decay, key, query (and removal,
// unit key) rows (fp32, zero past dk) and the CTA's columns of v sit in shared memory, staged once for all eight warps,
// while the next chunk's values are already on their way into registers — the walk waits for memory once per sequence.  A
// token costs a warp the removal's dot with the OLD columns (warp sums the update waits for, NC side by side), DR
// multiply-adds per operand and column, and the output's dot with the NEW columns.  Columns never read each other, so
// the result of a sequence does not depend on what else is in the step; the order of the sums inside a column is fixed by
// dk alone (lane l sums rows l, l + 32, …, then the butterfly), whatever NC is.
template <int DR, bool REMOVE, int NC>
__global__ void __launch_bounds__(256, 2) lin_scan_kernel(const LinScan p) {
  pdl_trigger();
  pdl_wait();
  constexpr int DK = 32 * DR;
  // tokens per chunk: what 8 KB (with the removal's two extra rows: 4 KB) of one operand hold, 4 … 32 — the next chunk waits
  // in registers, and two CTAs share an SM
  constexpr int CH0 = (REMOVE ? 1024 : 2048) / DK;
  constexpr int CH = CH0 > 32 ? 32 : CH0 < 4 ? 4 : CH0;
  constexpr int NV = REMOVE ? 5 : 3;                      // staged vectors per token: d, b, r (, p, q)
  constexpr int NQ = CH * NV * DK / 256;                  // staged vector elements per thread and chunk
  constexpr int COLS = 8 * NC;
  constexpr int NVR = (CH * COLS + 255) / 256;            // staged values per thread and chunk
  __shared__ float s_x[CH][NV][DK];
  __shared__ float s_v[CH][COLS];
  const int seg = blockIdx.x, hd = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int dk = p.dk, dv = p.dv;
  const int j0 = blockIdx.z * COLS, jw = j0 + warp * NC;
  const int r0 = p.seg_row0 != nullptr ? p.seg_row0[seg] : seg;
  const int cnt = p.seg_count != nullptr ? p.seg_count[seg] : 1;
  float* st = p.state + (int64_t)p.slot[r0] * p.slot_stride + (int64_t)hd * dk * dv;
  const bool fresh = p.pos[r0] == 0;
  float S[NC][DR];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
#pragma unroll
    for (int i = 0; i < DR; ++i) {
      const int d = lane + 32 * i;
      S[c][i] = (jw + c < dv && !fresh && d < dk) ? st[(int64_t)d * dv + jw + c] : 0.f;
    }
  }
  const int hs = hd / p.share;   // the head whose b / r vectors this head reads
  const float* src_d = p.d_scalar ? p.d + hd : p.d + (int64_t)hd * dk;
  const float* src_b = p.b + (int64_t)hs * dk;
  const float* src_r = p.r + (int64_t)hs * dk;
  const float* src_p = REMOVE ? p.p + (int64_t)hd * dk : nullptr;
  const float* src_q = REMOVE ? p.q + (int64_t)(p.q_shared ? hs : hd) * dk : nullptr;
  float r_x[NQ], r_v[NVR];
  auto fetch = [&](int c0) {
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      const int e = tid + 256 * i, t = e / (NV * DK), w = (e / DK) % NV, d = e % DK;
      float val = 0.f;
      if (c0 + t < cnt && d < dk) {
        const int64_t base = (int64_t)(r0 + c0 + t) * p.ld;
        const float* src = w == 0 ? src_d : w == 1 ? src_b : w == 2 ? src_r : w == 3 ? src_p : src_q;
        val = src[base + ((w == 0 && p.d_scalar) ? 0 : d)];
      }
      r_x[i] = val;
    }
#pragma unroll
    for (int i = 0; i < NVR; ++i) {
      const int e = tid + 256 * i, t = e / COLS, c = j0 + e % COLS;
      float val = 0.f;
      if (e < CH * COLS && c0 + t < cnt && c < dv) {
        const int64_t base = (int64_t)(r0 + c0 + t) * p.ld;
        val = p.v[base + (int64_t)hd * dv + c];
        if (p.vscale != nullptr) val *= p.vscale[base + hd];
      }
      r_v[i] = val;
    }
  };
  fetch(0);
  for (int c0 = 0; c0 < cnt; c0 += CH) {
    const int n = min(CH, cnt - c0);
    __syncthreads();   // the previous chunk has been read
#pragma unroll
    for (int i = 0; i < NQ; ++i) (&s_x[0][0][0])[tid + 256 * i] = r_x[i];
#pragma unroll
    for (int i = 0; i < NVR; ++i)
      if (tid + 256 * i < CH * COLS) (&s_v[0][0])[tid + 256 * i] = r_v[i];
    __syncthreads();
    if (c0 + CH < cnt) fetch(c0 + CH);
    if (jw >= dv) continue;   // warps past the last column only help with the staging
    for (int t4 = 0; t4 < n; t4 += 4) {   // the outputs' warp sums of four tokens run side by side, off the state's chain
      float dot[4][NC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int t = t4 + u;             // t < CH always (CH is a multiple of 4)
#pragma unroll
        for (int c = 0; c < NC; ++c) dot[u][c] = 0.f;
        if (t >= n) continue;             // rows past the chunk's end hold zeros: they must not touch the state
        float rem[NC], vj[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          rem[c] = 0.f;
          vj[c] = s_v[t][warp * NC + c];
        }
        if constexpr (REMOVE) {
#pragma unroll
          for (int i = 0; i < DR; ++i) {
            const float qq = s_x[t][4][lane + 32 * i];
#pragma unroll
            for (int c = 0; c < NC; ++c) rem[c] = fmaf(qq, S[c][i], rem[c]);
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int c = 0; c < NC; ++c) rem[c] += __shfl_xor_sync(0xffffffffu, rem[c], o);
          }
        }
#pragma unroll
        for (int i = 0; i < DR; ++i) {
          const int d = lane + 32 * i;
          const float dd = s_x[t][0][d], bb = s_x[t][1][d], rr = s_x[t][2][d];
          float pp = 0.f;
          if constexpr (REMOVE) pp = s_x[t][3][d];
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            float sn = dd * S[c][i];
            if constexpr (REMOVE) sn = fmaf(-pp, rem[c], sn);
            sn = fmaf(bb, vj[c], sn);
            S[c][i] = sn;
            dot[u][c] = fmaf(sn, rr, dot[u][c]);
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int c = 0; c < NC; ++c) dot[u][c] += __shfl_xor_sync(0xffffffffu, dot[u][c], o);
        }
      }
      if (lane < 4 * NC) {                // lane u·NC + c hands out token t4 + u, column jw + c
        const int u = lane / NC, c = lane % NC;
        float mine = 0.f;
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) mine = (uu == u && cc == c) ? dot[uu][cc] : mine;
        }
        if (t4 + u < n && jw + c < dv) p.o[(int64_t)(r0 + c0 + t4 + u) * p.ld_o + (int64_t)hd * dv + jw + c] = mine;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    if (jw + c >= dv) continue;
#pragma unroll
    for (int i = 0; i < DR; ++i) {
      const int d = lane + 32 * i;
      if (d < dk) st[(int64_t)d * dv + jw + c] = S[c][i];
    }
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
// The rows of a sequence lie side by side in the step, in order: row t − j is position pos[t] − j of the same sequence
// exactly when it has the same slot and that position.  Inputs from before the step's first row come from the slot's
// state, which holds the last taps − 1 inputs, oldest first (zeros before position 0).
__device__ __forceinline__ bool same_seq(const int32_t* slot, const int32_t* pos, int t, int j) {
  return t - j >= 0 && slot[t - j] == slot[t] && pos[t - j] == pos[t] - j;
}

// One thread per (row, channel): convolution over the row's own input and the taps − 1 before it + bias + SiLU into the
// fp32 workspace.  The state is only READ here (mamba_out_kernel, a later launch, moves it on).  The threads past the
// channels serve one head each: dt = softplus(logit + bias) and the decay exp(−exp(A_log)·dt).
template <typename T>
__global__ void __launch_bounds__(128) mamba_conv_kernel(const MambaRun p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
  const int H = p.a.heads, inner = H * p.a.vdim, ch = inner + 2 * p.m.groups * p.m.state, taps = p.m.taps;
  if (c >= ch + H) return;
  float* f = p.f + (int64_t)t * p.scan.ld;
  if (c >= ch) {
    const int hd = c - ch;
    const float dt = softplusf(p.dt[(int64_t)t * p.ld_dt + hd] + p.m.dt_bias[hd]);
    f[ch + hd] = expf(-expf(p.m.A_log[hd]) * dt);
    f[ch + H + hd] = dt;
    return;
  }
  const int32_t *slot = p.scan.slot, *pos = p.scan.pos;
  const T* x = static_cast<const T*>(p.proj) + p.off_x + c;
  const float* cs = p.conv_state + (int64_t)slot[t] * p.scan.slot_stride;
  float acc = p.m.conv_b[c];
  int in_step = 0;   // rows of this sequence in front of row t, counted up to taps − 1
  while (in_step < taps - 1 && same_seq(slot, pos, t, in_step + 1)) ++in_step;
  for (int j = 0; j < taps; ++j) {   // j positions back; weight column taps − 1 − j
    float v = 0.f;
    if (j <= in_step) v = ldf<T>(x + (int64_t)(t - j) * p.ld_proj);
    else if (pos[t] - j >= 0) v = cs[(int64_t)(taps - 1 - (j - in_step)) * ch + c];   // j − in_step inputs before the step's first row
    acc = fmaf(p.m.conv_w[(int64_t)c * taps + taps - 1 - j], v, acc);
  }
  f[c] = siluf(acc);
}

// First CTA of a token: y = o + D·x, · silu(z), an RMS norm in norm_groups equal parts, · norm.  The other CTAs of a sequence's
// LAST row in the step move the slot's convolution state on: the last taps − 1 inputs, from the step's rows where it has that
// many, else from the old state shifted in place.
template <typename T>
__global__ void __launch_bounds__(256) mamba_out_kernel(const MambaRun p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = p.a.heads, dv = p.a.vdim, inner = H * dv, part = inner / p.m.norm_groups;
  if (blockIdx.y > 0) {   // the CTAs behind the first move the state on, 256 channels each
    const int32_t *slot = p.scan.slot, *pos = p.scan.pos;
    const int taps = p.m.taps, ch = inner + 2 * p.m.groups * p.m.state;
    const bool last = t + 1 >= p.scan.n_tok || slot[t + 1] != slot[t] || pos[t + 1] != pos[t] + 1;
    if (last && taps > 1) {
      int in_step = 0;
      while (in_step < taps - 1 && same_seq(slot, pos, t, in_step + 1)) ++in_step;
      float* cs = p.conv_state + (int64_t)slot[t] * p.scan.slot_stride;
      const T* x = static_cast<const T*>(p.proj) + p.off_x;
      for (int c = (blockIdx.y - 1) * 256 + tid; c < ch; c += 256 * (gridDim.y - 1)) {
        // new entry i = the input taps − 2 − i positions back from row t: a step row, or the old entry i + 1 + in_step — always
        // further along than anything written so far, so the shift runs in place
        for (int i = 0; i < taps - 1; ++i) {
          const int j = taps - 2 - i;
          float v = 0.f;
          if (j <= in_step) v = ldf<T>(x + (int64_t)(t - j) * p.ld_proj + c);
          else if (pos[t] - j >= 0) v = cs[(int64_t)(i + 1 + in_step) * ch + c];
          cs[(int64_t)i * ch + c] = v;
        }
      }
    }
    return;
  }
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

// ------------------------------------------------------------------------------------------------- gated delta rule
// Channel c of the convolved q | k | v → its column in the projection rows
__device__ __forceinline__ int gdelta_col(const GatedDeltaRun& p, int c, int nqk) {
  return c < nqk ? p.off_q + c : c < 2 * nqk ? p.off_k + (c - nqk) : p.off_v + (c - 2 * nqk);
}

// One CTA per (token, query / key head g): the channels of q head g, k head g and the value heads that read them.  First the
// short causal convolution of every such channel over the row's own input and the taps − 1 before it (rows of the same
// sequence in this step, else the slot's state; zeros before position 0), then SiLU, into shared memory.  Then q and k
// become unit vectors (q also times dim^(−1/2)), and one warp per value head: its write strength beta = sigmoid(·), its decay
// g = exp(−exp(A_log)·softplus(· + dt_bias)).  The scan's fp32 rows:
//   [g: H | beta·g·k (the removal's weight vector): H·dk | k: G·dk | q: G·dk | v: H·dv | beta: H]
// The state is only READ here (gdelta_out_kernel, a later launch, moves it on).
template <typename T>
__global__ void __launch_bounds__(256) gdelta_prep_kernel(const GatedDeltaRun p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float sm[];   // [dk: q | dk: k | per·dv: v] convolved channels of this group
  const int t = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.a.heads, G = p.a.kv_heads, dk = p.a.dim, dv = p.a.vdim, taps = p.d.taps, per = H / G;
  const int nqk = G * dk, ch = 2 * nqk + H * dv, mine = 2 * dk + per * dv;
  const int32_t *slot = p.scan.slot, *pos = p.scan.pos;
  const T* proj = static_cast<const T*>(p.proj);
  const float* cs = p.conv_state + (int64_t)slot[t] * p.scan.slot_stride;
  int in_step = 0;   // rows of this sequence in front of row t, counted up to taps − 1
  while (in_step < taps - 1 && same_seq(slot, pos, t, in_step + 1)) ++in_step;
  for (int e = tid; e < mine; e += 256) {
    // the group's e-th channel → its place c among the q | k | v channels
    const int c = e < dk ? g * dk + e : e < 2 * dk ? nqk + g * dk + (e - dk) : 2 * nqk + g * per * dv + (e - 2 * dk);
    const int col = gdelta_col(p, c, nqk);
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {   // j positions back; weight column taps − 1 − j
      float v = 0.f;
      if (j <= in_step) v = ldf<T>(proj + (int64_t)(t - j) * p.ld_proj + col);
      else if (pos[t] - j >= 0) v = cs[(int64_t)(taps - 1 - (j - in_step)) * ch + c];
      acc = fmaf(p.d.conv_w[(int64_t)c * taps + taps - 1 - j], v, acc);
    }
    sm[e] = siluf(acc);
  }
  __syncthreads();
  float* f = p.f + (int64_t)t * p.scan.ld;
  float* f_g = f;
  float* f_p = f + H;
  float* f_k = f_p + (int64_t)H * dk;
  float* f_q = f_k + nqk;
  float* f_v = f_q + nqk;
  float* f_beta = f_v + (int64_t)H * dv;
  if (warp < 2) {   // warp 0: the unit query, warp 1: the unit key (kept in shared memory for the value heads)
    float* x = sm + warp * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += x[i] * x[i];
    float inv = 1.f / sqrtf(warp_sum(ss) + p.d.unit_eps);
    if (warp == 0) inv *= rsqrtf((float)dk);
    float* dst = (warp == 0 ? f_q : f_k) + (int64_t)g * dk;
    for (int i = lane; i < dk; i += 32) {
      const float u = x[i] * inv;
      x[i] = u;
      dst[i] = u;
    }
  }
  __syncthreads();
  const T* row = proj + (int64_t)t * p.ld_proj;
  const float* k = sm + dk;
  for (int u = warp; u < per; u += 8) {
    const int hd = g * per + u;
    const float beta = sigmoidf(ldf<T>(row + p.off_b + hd));
    const float dec = expf(-expf(p.d.A_log[hd]) * softplusf(ldf<T>(row + p.off_a + hd) + p.d.dt_bias[hd]));
    if (lane == 0) {
      f_g[hd] = dec;
      f_beta[hd] = beta;
    }
    for (int i = lane; i < dk; i += 32) f_p[(int64_t)hd * dk + i] = beta * dec * k[i];
    for (int i = lane; i < dv; i += 32) f_v[(int64_t)hd * dv + i] = sm[2 * dk + u * dv + i];
  }
}

// First CTA of a token: one warp per head, o / rms(o) · head_norm (shared by the heads) · silu(out gate).  The other CTAs of a
// sequence's LAST row in the step move the slot's convolution state on: the last taps − 1 inputs, from the step's rows where
// it has that many, else from the old state shifted in place.
template <typename T>
__global__ void __launch_bounds__(256) gdelta_out_kernel(const GatedDeltaRun p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.a.heads, G = p.a.kv_heads, dk = p.a.dim, dv = p.a.vdim;
  if (blockIdx.y > 0) {
    const int32_t *slot = p.scan.slot, *pos = p.scan.pos;
    const int taps = p.d.taps, nqk = G * dk, ch = 2 * nqk + H * dv;
    const bool last = t + 1 >= p.scan.n_tok || slot[t + 1] != slot[t] || pos[t + 1] != pos[t] + 1;
    if (last && taps > 1) {
      int in_step = 0;
      while (in_step < taps - 1 && same_seq(slot, pos, t, in_step + 1)) ++in_step;
      float* cs = p.conv_state + (int64_t)slot[t] * p.scan.slot_stride;
      const T* proj = static_cast<const T*>(p.proj);
      for (int c = (blockIdx.y - 1) * 256 + tid; c < ch; c += 256 * (gridDim.y - 1)) {
        const int col = gdelta_col(p, c, nqk);
        // new entry i = the input taps − 2 − i positions back from row t: a step row, or the old entry i + 1 + in_step — always
        // further along than anything written so far, so the shift runs in place
        for (int i = 0; i < taps - 1; ++i) {
          const int j = taps - 2 - i;
          float v = 0.f;
          if (j <= in_step) v = ldf<T>(proj + (int64_t)(t - j) * p.ld_proj + col);
          else if (pos[t] - j >= 0) v = cs[(int64_t)(i + 1 + in_step) * ch + c];
          cs[(int64_t)i * ch + c] = v;
        }
      }
    }
    return;
  }
  const T* g = static_cast<const T*>(p.proj) + (int64_t)t * p.ld_proj + p.off_g;
  T* y = static_cast<T*>(p.mid) + (int64_t)t * p.ld_mid;
  for (int hd = warp; hd < H; hd += 8) {
    const float* o = p.scan.o + (int64_t)t * p.scan.ld_o + hd * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss += o[c] * o[c];
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + p.eps);
    for (int c = lane; c < dv; c += 32) y[hd * dv + c] = cvt<T>(o[c] * inv * p.d.head_norm[c] * siluf(ldf<T>(g + hd * dv + c)));
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

// The same for a few rows that fit the CTA's registers (decode steps, where latency counts): y, w and x are requested
// together — one memory round trip before the reduction instead of three.  dim <= 16 · 256.
template <typename YT>
__global__ void __launch_bounds__(256) stack_rms_add_cast_small_kernel(float* __restrict__ x, const YT* __restrict__ y,
                                                                       const float* __restrict__ w, __nv_bfloat16* __restrict__ h,
                                                                       int dim, float eps, float mult) {
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
    if (i < dim) {
      const float v = xv[k] + mult * (yv[k] * inv * wv[k]);
      xr[i] = v;
      if (h != nullptr) h[(int64_t)blockIdx.x * dim + i] = __float2bfloat16_rn(v);
    }
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
  // two columns per warp where the value size fills them and the registers hold them: half the CTAs stage the same rows
  const int nc = (p.dv >= 32 && p.dk <= 256) ? 2 : 1;
  const dim3 grid(p.n_seg, p.heads, (p.dv + 8 * nc - 1) / (8 * nc));
#define B200_SCAN_NC(DR, NC)                                                                                       \
  do {                                                                                                             \
    if (p.p != nullptr) B200_CUDA(launch_pdl(lin_scan_kernel<DR, true, NC>, grid, dim3(256), 0, st, stack_pdl(), p));  \
    else B200_CUDA(launch_pdl(lin_scan_kernel<DR, false, NC>, grid, dim3(256), 0, st, stack_pdl(), p));           \
  } while (0)
#define B200_SCAN(DR)              \
  do {                             \
    if (nc == 2) B200_SCAN_NC(DR, 2); \
    else B200_SCAN_NC(DR, 1);      \
  } while (0)
  if (p.dk <= 32) B200_SCAN(1);
  else if (p.dk <= 64) B200_SCAN(2);
  else if (p.dk <= 128) B200_SCAN(4);
  else if (p.dk <= 256) B200_SCAN(8);
  else B200_SCAN(16);
#undef B200_SCAN
#undef B200_SCAN_NC
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

int run_gdelta(const GatedDeltaRun& p, int dtype, cudaStream_t st) {
  REC_DTYPE_CHECK(dtype);
  B200_CHECK_ARG(p.proj && p.conv_state && p.f && p.mid && p.scan.n_tok > 0 && p.scan.n_seg > 0, "gated delta rule: null argument");
  const int H = p.a.heads, G = p.a.kv_heads, dk = p.a.dim, dv = p.a.vdim;
  B200_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, "gated delta rule: heads %d over %d query / key heads", H, G);
  B200_CHECK_ARG(p.d.taps >= 1 && p.d.taps <= kMambaMaxTaps, "gated delta rule: 1 … %d convolution taps", kMambaMaxTaps);
  B200_CHECK_ARG(p.d.conv_w && p.d.A_log && p.d.dt_bias && p.d.head_norm && p.d.unit_eps >= 0.f, "gated delta rule: null weight");
  const int nqk = G * dk, ch = 2 * nqk + H * dv;
  const size_t smem = (size_t)(2 * dk + (H / G) * dv) * 4;
  B200_CHECK_ARG(smem <= 200 * 1024, "gated delta rule: the channels of one query / key head and its value heads exceed one CTA's shared memory");
  if (smem > 48 * 1024) {
    static bool attr_done = false;
    if (!attr_done) {
      B200_CUDA(cudaFuncSetAttribute(gdelta_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      B200_CUDA(cudaFuncSetAttribute(gdelta_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_done = true;
    }
  }
  const dim3 pg(p.scan.n_tok, G);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(gdelta_prep_kernel<float>, pg, dim3(256), smem, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(gdelta_prep_kernel<__nv_bfloat16>, pg, dim3(256), smem, st, stack_pdl(), p));
  LinScan s = p.scan;
  s.heads = H; s.dk = dk; s.dv = dv; s.share = H / G; s.d_scalar = 1; s.q_shared = 1;
  s.d = p.f; s.p = p.f + H; s.q = s.p + (int64_t)H * dk; s.b = s.q; s.r = s.q + nqk; s.v = s.r + nqk;
  s.vscale = s.v + (int64_t)H * dv;
  int rc = launch_lin_scan(s, st);
  if (rc != B200_OK) return rc;
  const dim3 og(p.scan.n_tok, p.d.taps > 1 ? 1 + std::min((ch + 255) / 256, 16) : 1);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(gdelta_out_kernel<float>, og, dim3(256), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(gdelta_out_kernel<__nv_bfloat16>, og, dim3(256), 0, st, stack_pdl(), p));
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
  const dim3 cg(p.scan.n_tok, (ch + H + 127) / 128);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(mamba_conv_kernel<float>, cg, dim3(128), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(mamba_conv_kernel<__nv_bfloat16>, cg, dim3(128), 0, st, stack_pdl(), p));
  LinScan s = p.scan;
  s.heads = H; s.dk = N; s.dv = dv; s.share = H / m.groups; s.d_scalar = 1;
  s.v = p.f; s.b = p.f + inner; s.r = p.f + inner + (int64_t)m.groups * N; s.d = p.f + ch; s.vscale = p.f + ch + H;
  s.p = s.q = nullptr;
  int rc = launch_lin_scan(s, st);
  if (rc != B200_OK) return rc;
  const dim3 og(p.scan.n_tok, m.taps > 1 ? 1 + std::min((ch + 255) / 256, 16) : 1);
  if (dtype == B200_F32) B200_CUDA(launch_pdl(mamba_out_kernel<float>, og, dim3(256), 0, st, stack_pdl(), p));
  else B200_CUDA(launch_pdl(mamba_out_kernel<__nv_bfloat16>, og, dim3(256), 0, st, stack_pdl(), p));
  return B200_OK;
}

int launch_stack_rms_add_cast(float* x, const void* y, bool y_bf16, const float* w, __nv_bfloat16* h, int64_t rows, int dim,
                              float eps, float mult, cudaStream_t st) {
  B200_CHECK_ARG(x && y && w && rows > 0 && dim > 0, "stack rms_add_cast: bad arguments");
  if (rows <= 64 && dim <= 16 * 256) {
    if (y_bf16)
      B200_CUDA(launch_pdl(stack_rms_add_cast_small_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x,
                           (const __nv_bfloat16*)y, w, h, dim, eps, mult));
    else
      B200_CUDA(launch_pdl(stack_rms_add_cast_small_kernel<float>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x,
                           (const float*)y, w, h, dim, eps, mult));
    return B200_OK;
  }
  if (y_bf16)
    B200_CUDA(launch_pdl(stack_rms_add_cast_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x,
                         (const __nv_bfloat16*)y, w, h, dim, eps, mult));
  else
    B200_CUDA(launch_pdl(stack_rms_add_cast_kernel<float>, dim3((unsigned)rows), dim3(256), 0, st, stack_pdl(), x,
                         (const float*)y, w, h, dim, eps, mult));
  return B200_OK;
}

}  // namespace b200
