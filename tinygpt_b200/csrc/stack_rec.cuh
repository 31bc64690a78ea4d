// stack_rec.cuh — mixers of post-norm blocks (stack_rec.cu): the per-token preparation of an attention mixer (query / key
// norms over the whole projection, rotate-half rotary positions, unit-rms values, value mix-in), and the linear
// recurrences — ONE scan kernel for every recurrence of the form  S ← diag(d) S − p (qᵀS) + b vᵀ,  o = Sᵀr  (generalized
// delta rule: all terms; Mamba-2: a scalar d per head, no removal, b and r shared by a group of heads), with the
// design-specific passes before it (gates, decays, unit keys, the short convolution) and behind it (head norms, gates).
// Storage type T = bf16 or fp32; everything that enters a recurrence, its state and every norm are fp32.
#pragma once
#include "stack.cuh"

namespace b200 {

// ---- attention preparation, in place in the projection rows
struct AttnPrep {
  b200_attn_desc a{};
  b200_attn_prep_desc d{};
  float eps = 1e-5f;
  void* proj = nullptr;          // [n_tok, ld_proj] T: q | k | v at off_q / off_k / off_v
  int64_t ld_proj = 0;
  int off_q = 0, off_k = 0, off_v = 0;
  const int32_t* pos = nullptr;
  int n_tok = 0;
  void* vkeep = nullptr;         // [n_tok, ld_keep] T: the values a v_mix 1 layer keeps and a v_mix 2 layer reads
  int64_t ld_keep = 0;
  int q_only = 0;                // 1: the rows hold queries only (a layer that reads another layer's cached keys and values)
};
int launch_attn_prep(const AttnPrep& p, int dtype, cudaStream_t st);

// ---- the scan.  Per sequence (rows [row0, row0 + count) of the step, in order), head h and value column j:
//   s ← d ∘ s − p·(q·s) + b·(v_j·vscale),   o_j = s·r          s: the dk entries of column j of S
// All operands are fp32 rows of stride `ld`.  d: [heads·dk] per row, or (d_scalar) [heads]; p, q: [heads·dk] or null (no
// removal); b, r: [heads / share][dk] — `share` consecutive heads read the same vector; v: [heads·dv]; vscale: [heads] per
// row or null.  State of a slot: [heads][dk][dv] fp32 at state + slot·slot_stride; a sequence whose first row has
// position 0 starts from zero.
constexpr int kScanMaxDim = 512;
struct LinScan {
  int heads = 0, dk = 0, dv = 0, share = 1, d_scalar = 0;
  int q_shared = 0;   // 1: q is [heads / share][dk] like b and r (the removal reads along a shared key)
  const float *d = nullptr, *p = nullptr, *q = nullptr, *b = nullptr, *r = nullptr, *v = nullptr, *vscale = nullptr;
  int64_t ld = 0;
  float* state = nullptr;
  int64_t slot_stride = 0;
  const int32_t* seg_row0 = nullptr;   // [n_seg] first row / row count of every sequence; null: every row is a sequence
  const int32_t* seg_count = nullptr;
  const int32_t* slot = nullptr;       // per row
  const int32_t* pos = nullptr;        // per row
  int n_seg = 0, n_tok = 0;
  float* o = nullptr;                  // [n_tok, ld_o]: head h at columns h·dv
  int64_t ld_o = 0;
};
int launch_lin_scan(const LinScan& p, cudaStream_t st);

// ---- generalized delta rule around the scan
struct DeltaRun {
  b200_attn_desc a{};            // heads, dim (key channels), vdim
  b200_delta_desc d{};
  float eps = 1e-5f;
  const void* proj = nullptr;    // [n_tok, ld_proj] T: r | k | v | out-gate logits | removal logits at off_r / off_k / off_v / off_g / off_a
  int64_t ld_proj = 0;
  int off_r = 0, off_k = 0, off_v = 0, off_g = 0, off_a = 0;
  const float* wl = nullptr;     // [n_tok, heads·dim] fp32: w2·tanh(bottleneck) + w0
  float* f = nullptr;            // [n_tok, delta_row_floats] fp32 workspace: decay | removal | unit key | key | query | value
  LinScan scan{};                // state, slots, positions, sequences, o
  void* mid = nullptr;           // [n_tok, ld_mid] T
  int64_t ld_mid = 0;
};
inline int64_t delta_row_floats(int heads, int dim, int vdim) { return (int64_t)heads * (5 * dim + vdim); }
int run_delta(const DeltaRun& p, int dtype, cudaStream_t st);

// ---- Mamba-2 around the scan
constexpr int kMambaMaxTaps = 16;
struct MambaRun {
  b200_attn_desc a{};            // heads, vdim; dim = state
  b200_mamba_desc m{};
  float eps = 1e-5f;
  const void* proj = nullptr;    // [n_tok, ld_proj] T: z at off_z, x | B | C (contiguous) at off_x
  int64_t ld_proj = 0;
  int off_z = 0, off_x = 0;
  const float* dt = nullptr;     // [n_tok, ld_dt] fp32: raw step-size logits per head
  int64_t ld_dt = 0;
  float* conv_state = nullptr;   // this run's [taps − 1][channels] fp32 of slot 0 (the slot stride is the scan's)
  float* f = nullptr;            // [n_tok, mamba_row_floats] fp32 workspace: x | B | C (after convolution and SiLU) | decay | dt
  LinScan scan{};
  void* mid = nullptr;
  int64_t ld_mid = 0;
};
inline int64_t mamba_row_floats(int heads, int vdim, int state, int groups) {
  return (int64_t)heads * vdim + 2ll * groups * state + 2 * heads;
}
// floats of state per slot: S [heads][state][vdim], then the convolution's last taps − 1 inputs [taps − 1][channels]
inline int64_t mamba_state_floats(int heads, int vdim, int state, int groups, int taps) {
  return (int64_t)heads * state * vdim + (int64_t)(taps - 1) * ((int64_t)heads * vdim + 2ll * groups * state);
}
int run_mamba(const MambaRun& p, int dtype, cudaStream_t st);

// ---- gated delta rule around the scan: S ← g S − (beta·g·k)(kᵀS) + k (beta·v)ᵀ — the decayed state loses what it held
// along the unit key and gains the new value there, both weighted by the write strength beta
struct GatedDeltaRun {
  b200_attn_desc a{};            // heads (value heads), kv_heads (query / key heads), dim, vdim
  b200_gdelta_desc d{};
  float eps = 1e-5f;
  const void* proj = nullptr;    // [n_tok, ld_proj] T: q | k | v | out-gate logits | write strengths | decay logits
  int64_t ld_proj = 0;
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_b = 0, off_a = 0;
  float* conv_state = nullptr;   // this run's [taps − 1][channels] fp32 of slot 0 (the slot stride is the scan's)
  float* f = nullptr;            // [n_tok, gdelta_row_floats] fp32 workspace
  LinScan scan{};
  void* mid = nullptr;
  int64_t ld_mid = 0;
};
inline int64_t gdelta_row_floats(int heads, int kv_heads, int dim, int vdim) {
  return 2ll * heads + (int64_t)heads * dim + 2ll * kv_heads * dim + (int64_t)heads * vdim;
}
// floats of state per slot: S [heads][dim][vdim], then the convolutions' last taps − 1 inputs [taps − 1][channels]
inline int64_t gdelta_state_floats(int heads, int kv_heads, int dim, int vdim, int taps) {
  return (int64_t)heads * dim * vdim + (int64_t)(taps - 1) * (2ll * kv_heads * dim + (int64_t)heads * vdim);
}
int run_gdelta(const GatedDeltaRun& p, int dtype, cudaStream_t st);

// x[r, :] += mult · rmsnorm(y[r, :]) · w  (fp32 stream), and h[r, :] = bf16(x[r, :]) — a sublayer's post-norm, the
// residual sum and the next sublayer's operand copy in one pass; h may be null
int launch_stack_rms_add_cast(float* x, const void* y, bool y_bf16, const float* w, __nv_bfloat16* h, int64_t rows, int dim,
                              float eps, float mult, cudaStream_t st);

}  // namespace b200
