// stack_mix.cuh — mixers and feed-forwards of sandwich blocks (stack_mix.cu): layer norm, latent attention, the mLSTM
// matrix memory, routed experts, soft-capped logits.  Storage type T = bf16 or fp32; fp32 arithmetic for norms, softmax,
// routing, gates, the recurrence and its state.
#pragma once
#include "stack.cuh"

namespace b200 {

// y[r, :] = T(norm(x[rows ? rows[r] : r, :]) · (offset + w)), norm of b200_norm_kind `kind`
int launch_stack_norm(void* y, const float* x, const float* w, const int32_t* rows_or_null, int64_t n_rows, int dim,
                      float eps, float offset, int kind, int dtype, cudaStream_t st);
// x[r, :] += mult · norm(y[r, :]) · w, y fp32 or bf16
int launch_stack_norm_add(float* x, const void* y, bool y_bf16, const float* w, int64_t rows, int dim, float eps, float mult,
                          int kind, cudaStream_t st);
// x[r, :] += mult · norm(y[r, :]) · w_post, then h[r, :] = T(norm(x[r, :]) · (offset + w_next)): a sublayer's post-norm, the
// residual sum and the next sublayer's pre-norm in one pass (layer norms of rows up to 8192 wide; else two launches)
int launch_stack_norm_add_norm(float* x, const void* y, bool y_bf16, const float* w_post, void* h, const float* w_next,
                               int64_t rows, int dim, float eps, float offset, float mult, int kind, int dtype, cudaStream_t st);
// y[r, j] = T(min(g, limit)·sigmoid(1.702·min(g, limit))·(clamp(u, ±limit) + 1)), g = gu[r, j], u = gu[r, n + j]
int launch_stack_glu_clamp(void* y, int64_t ld_y, const void* gu, int64_t ld_gu, int64_t rows, int n, float limit, int dtype,
                           cudaStream_t st);
// logits (fp32) and their bf16 copy <- cap·tanh(logits / cap)
int launch_stack_softcap(float* logits, __nv_bfloat16* logits_bf, int64_t total, float cap, cudaStream_t st);

// y[r, :dim] = T(rms(x[r, :dim])·w), y[r, dim:dim_pad] = 0 over row-strided T-typed rows
int launch_stack_rmsnorm_rows(void* y, int64_t ld_y, const void* x, int64_t ld_x, const float* w, int64_t rows, int dim, int dim_pad,
                              float eps, int dtype, cudaStream_t st);
// y[r, j] = T(y[r, j]·sigmoid(g[r, j])) over row-strided T-typed operands
int launch_stack_sigmoid_gate(void* y, int64_t ld_y, const void* g, int64_t ld_g, int64_t rows, int n, int dtype, cudaStream_t st);

// ---- small products of decode-shaped steps: `items` independent products of up to 8 rows each, one warp per output row.
// Item z multiplies rows a + m·lda + (z / item_div)·sa (m < M) with matrix w + (item_mat ? item_mat[z] : z)·sw ([N, K] row-major) into
// c + m·ldc + z·sc (T, or fp32 when c_f32).  Serves the per-head folds of latent attention, router and gate logits, and
// the chosen experts of a few tokens (item = (token, choice) pair, matrix = that pair's expert).
constexpr int kSmallRows = 8;
struct SmallGemv {
  const void* a = nullptr;
  int64_t lda = 0, sa = 0;
  int item_div = 1;              // item z reads rows a + (z / item_div)·sa: item_div consecutive items share their rows
  const void* w = nullptr;
  int64_t sw = 0;
  const int32_t* item_mat = nullptr;
  const float* bias = nullptr;   // [N], shared by the items
  void* c = nullptr;
  int64_t ldc = 0, sc = 0;
  bool c_f32 = false;
  int M = 1, N = 0, K = 0, items = 1;
  int64_t nc = 1;                // stride of the output row index n inside c
  int m_total = 0;               // > 0: item z has min(M, m_total − z·M) rows (the last item may be short)
  const float* bias_m = nullptr; // [m_total]: bias of row z·M + m
  int act = -1;                  // B200_ACT_RELU2 / _TANH / _SILU: applied to the fp32 sum (+ bias) before it is stored
};
int launch_small_gemv(const SmallGemv& g, int dtype, cudaStream_t st);
// C[rows, n] (fp32) = A[rows, K]·W[n, K]ᵀ + bias[n] for a FEW output columns n and any number of rows (router and gate
// logits of a prompt): the small product with the roles swapped — W's rows, eight at a time, are the "activations", A's
// rows the matrix.
int launch_skinny_f32(float* C, const void* A, const void* W, const float* bias_or_null, int rows, int n, int K, int dtype,
                      cudaStream_t st);

// ---- latent attention: everything between the in-projection and the out-projection
constexpr int kLatentMaxRank = 1024;
struct LatentRun {
  b200_attn_desc a{};
  b200_latent_desc l{};
  float eps = 1e-5f;
  const void* proj = nullptr;    // [n_tok, ld_proj] T: q at off_q (heads·(dim + rot_dim)), down at off_down (kv_rank + rot_dim)
  int64_t ld_proj = 0;
  int off_q = 0, off_down = 0;
  const void* q = nullptr;       // [n_tok, ld_q] T: the per-head queries when they are not the q segment of proj (queries that
  int64_t ld_q = 0;              // went through a latent of their own); null: proj + off_q
  void* cache = nullptr;         // this run's rows of slot 0: [max_ctx][kv_rank + rot_dim] T; slot s is s·slot_stride further
  int64_t slot_stride = 0;
  const int32_t* slot = nullptr;
  const int32_t* pos = nullptr;
  int n_tok = 0;
  void* qa = nullptr;            // [n_tok, heads·(kv_rank + rot_dim)] T: the query folded through uk, and its rotated part
  void* ol = nullptr;            // [n_tok, heads·kv_rank] T: softmax-weighted latents
  void* out = nullptr;           // [n_tok, ld_out] T: head h at columns h·vdim
  int64_t ld_out = 0;
  // decode-shaped steps (up to kSmallRows rows, long key lists): one CTA per (row, split of the key list) serves ALL heads
  // from key rows staged once in shared memory; the partial softmaxes [row][head][split][2 + kv_rank] in split_ws are
  // joined by a second small launch
  float* split_ws = nullptr;
  int nsplit = 0, keys_per_split = 0;
  bool stage_vec = false;        // set by the launcher: the staged rows can be copied in 16-byte pieces
};
constexpr int kLatentMaxSplits = 128;
constexpr int kLatentSplitKeys = 32;
int run_latent_attention(const LatentRun& p, int dtype, cudaStream_t st);
// the first step alone: cache rows and rotated query parts of the new tokens
int launch_latent_prep(const LatentRun& p, int dtype, cudaStream_t st);
// Prompt-shaped steps of bf16 engines whose heads suit the tensor-core attention kernel (dim + rot_dim == vdim): the keys
// and values of ONE sequence are expanded from its cache rows and laid out per head.
//   kbuf[j, h, :] = [kp[j, h·dim …] | rotated key part of cache row j]        j < ctx      (kp = latents · ukᵀ)
//   qbuf[t, h, :] = [q_plain of row row0 + t, head h | its rotated part from qa]            t < count
struct LatentPack {
  b200_attn_desc a{};
  b200_latent_desc l{};
  const __nv_bfloat16* kp = nullptr;       // [ctx, heads·dim]
  const __nv_bfloat16* cache_rows = nullptr;   // the sequence's cache rows [ctx][kv_rank + rot_dim]
  const __nv_bfloat16* proj = nullptr;     // the sequence's first row of the merged projection
  int64_t ld_proj = 0;
  int off_q = 0;
  const __nv_bfloat16* qa = nullptr;       // the sequence's first row of qa
  __nv_bfloat16* kbuf = nullptr;           // [ctx, heads·(dim + rot_dim)]
  __nv_bfloat16* qbuf = nullptr;           // [count, heads·(dim + rot_dim)]
  int ctx = 0, count = 0;
};
int launch_latent_pack(const LatentPack& p, cudaStream_t st);

// ---- mLSTM: recurrence + head norm + output gate
constexpr int kMlstmMaxDim = 512;
struct MlstmRun {
  b200_attn_desc a{};            // heads, dim (key size), vdim
  float gate_cap = 15.f, eps = 1e-5f;
  const void* proj = nullptr;    // [n_tok, ld_proj] T: q | k | v | out-gate logits at off_q / off_k / off_v / off_g
  int64_t ld_proj = 0;
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0;
  const float* gates = nullptr;  // [n_tok, ld_gates]: 2·heads raw input- and forget-gate logits per row
  int64_t ld_gates = 0;
  float* state = nullptr;        // this run's state of slot 0; slot s is s·slot_stride floats further
  int64_t slot_stride = 0;
  const int32_t* seg_row0 = nullptr;   // [n_seg] first row / row count of every sequence; null: every row is a sequence
  const int32_t* seg_count = nullptr;
  const int32_t* slot = nullptr;       // per row
  const int32_t* pos = nullptr;        // per row
  int n_seg = 0, n_tok = 0;
  float* gab = nullptr;          // [n_tok, heads, 3] fp32 workspace: decay, input weight, running maximum of every token
  float* o = nullptr;            // [n_tok, heads·(vdim + 2)] fp32: numerators | n·q | m
  const float* head_norm = nullptr;
  void* mid = nullptr;           // [n_tok, ld_mid] T: normed, gated head outputs
  int64_t ld_mid = 0;
};
// floats of state per head: S [dim][vdim + 1] (column vdim is the normaliser n) and the running maximum per column
inline int64_t mlstm_state_floats(int heads, int dim, int vdim) { return (int64_t)heads * ((int64_t)dim * (vdim + 1) + vdim + 1); }
int run_mlstm(const MlstmRun& p, int dtype, cudaStream_t st);

// ---- routed experts
struct MoeRun {
  b200_moe_desc m{};
  int width = 0, n_tok = 0;
  const void* h = nullptr;       // [n_tok, width] T
  float* z = nullptr;            // [n_tok, experts] router logits
  int32_t* sel_e = nullptr;      // [n_tok·top] chosen expert of every (token, choice) pair
  float* sel_w = nullptr;        // [n_tok·top] its score
  int32_t* plan = nullptr;       // counts [S] | group_end [S] | tile_group [n_tiles] | tile_row0 [n_tiles], S = plan_stride
  int plan_stride = 0;           // >= experts; 0: experts.  Layers of unequal expert counts share one plan: the counts (kept
                                 // zero between uses) of one must not lie under the other arrays of another
  int32_t* pair_slot = nullptr;  // [n_tok·top] sorted position of a pair
  void* a_perm = nullptr;        // [P, width] T: score·h of every pair, sorted by expert
  void* gu = nullptr;            // [P, 2·expert_ff] T
  void* act = nullptr;           // [P, expert_ff] T
  float* outp = nullptr;         // [P, width] fp32
  float* y = nullptr;            // [n_tok, width] fp32 result
  const void* shared = nullptr;  // [n_tok, width] T or fp32 (shared_f32): shared expert's output, or null
  bool shared_f32 = false;
  const void* sg = nullptr;      // T: the shared gate's logit of token t at sg[t·ld_sg]
  int64_t ld_sg = 0;
  // steps of up to kSmallRows tokens: no sorting — every (token, choice) pair is an item of a small product with its
  // expert's matrices
  bool small = false;
  // bf16 steps of many rows: the group sizes are read back to the host (one small copy and a wait per feed-forward) and
  // every expert's rows go through the tcgen05 GEMM; the down-projections leave bf16 rows in outp_bf
  bool tc = false;
  __nv_bfloat16* outp_bf = nullptr;   // [P, width]
};
__host__ __device__ inline int moe_tiles(int pairs, int experts) { return (pairs + 63) / 64 + experts; }
inline int64_t moe_plan_ints(int pairs, int experts) { return 2 * (int64_t)experts + 2 * moe_tiles(pairs, experts); }   // experts = the stride
int run_moe(const MoeRun& p, int dtype, cudaStream_t st);

}  // namespace b200
