// engine_stack.cu — layer-stack models behind the engine handle: a model given as data (runs of layers, each an
// attention mixer + optional gated feed-forward + optional token-table side input), sequence slots with their own KV
// caches and positions, and ONE step function for every kind of step: the new tokens of all sequences of a step are
// laid side by side as rows {token id, slot, position}; every kernel works on that row list, so a prompt, a part of a
// prompt, a batch of unequal prompts and a batch of single decode tokens are the same code with a different list.
//
// Per run of a layer (parallel block, fp32 residual stream x):
//   [x ← mix_in·[x; x0]]                       general GEMM over two operand sources, fp32 out (first run of a loop pass)
//   h    = rmsnorm(x)·(offset + w)             fp32 → T
//   proj = h·w_inᵀ + b_in                      ONE product for q | k | v | gate logits | ff gate | ff up
//   K/V rows → this run's cache of the slot    (every pass of a looped layer is a run with a cache of its own)
//   mid[:, 0 … heads·vdim)  = gated windowed attention(proj, cache)
//   mid[:, off_act …)       = act(ff gate)·ff up
//   x   += m · mid·w_outᵀ                      ONE product for o | ff down, summed in fp32 straight into the stream
//   x   += m · rmsnorm(side_proj·(gelu(side_gate·x) ∘ table[token]))·w_side
// then the final norm of the wanted rows only and the head product (fp32 logits + the bf16 copy argmax / sampler read).
//
// Per run of a layer (sandwich block: a norm before and after each sublayer; norms of either kind):
//   h    = norm(x)·w                            fp32 → T
//   proj = h·w_inᵀ + b_in                       the mixer's in-projections in one product
//   mid  = latent attention(proj, cache)        cache row of a position = [latent | rotated shared key part]
//        | mLSTM(proj, fp32 gate logits, state) state of a run = fp32 matrix memory per head, carried in the slot
//   x   += norm(mid·w_outᵀ)·post_norm
//   h    = norm(x)·ff_norm
//   y    = w_ff_out·act(w_ff_in·h)              dense, or
//        | Σ_chosen expert(score·h) + sigmoid(sg·h)·shared(h)    routed experts: rows sorted by expert, grouped products
//   x   += norm(y)·ff_post_norm
// and the logits may be soft-capped.
//
// Post-norm blocks are the same run without the norms in front: the sublayers read the stream itself (its T-typed copy),
//   x += norm(mixer(x))·post_norm,   x += norm(ff(x))·ff_post_norm
// with three more mixers: the windowed attention behind a per-token preparation of q | k | v (norms, rotary positions,
// value mix-in), the generalized delta rule and Mamba-2 — two recurrences that share one scan kernel and keep their fp32
// state (and the convolution's last inputs) in the slot, beside the caches of the attention runs.
//
// Sandwich blocks also take the prepared attention (biases, either rotary layout, a sink in the softmax; a layer may read the
// keys and values an earlier layer cached instead of projecting its own), the latent attention with a query latent, a
// sliding window and an element-wise output gate, and the gated delta rule behind short convolutions.
#include <algorithm>
#include <cstring>
#include <map>
#include <new>
#include <vector>

#include "engine.cuh"
#include "stack_mix.cuh"
#include "stack_rec.cuh"

namespace b200 {

constexpr int kStackChunk = 4096;   // most rows one pass through the runs takes; longer steps go in several passes

struct StackEngine {
  b200_stack_desc d{};
  std::vector<b200_stack_layer> layers;
  std::vector<int> run_layer, run_mix;
  int dtype = B200_BF16;
  size_t esz = 2;
  int gen_cap = 1 << 14;
  // caches: [slot][run][max_ctx][kv_heads·dim] and [slot][run][max_ctx][kv_heads·vdim]
  uint8_t* cache = nullptr;
  uint8_t *kbase = nullptr, *vbase = nullptr;
  std::vector<size_t> run_k_off, run_v_off;   // elements from the start of a slot (a run that shares another run's keys and
                                              // values carries that run's offsets)
  std::vector<char> run_kv_shared;            // the run reads another run's cache and writes none
  size_t k_slot = 0, v_slot = 0;              // elements per slot
  // per-slot device state
  uint8_t* state = nullptr;
  int* pos_dev = nullptr;
  int64_t* cur_tok = nullptr;
  int64_t* gen_log = nullptr;
  unsigned long long* gen_count = nullptr;
  int* row_slot = nullptr;
  void* argmax_ws = nullptr;
  int64_t* amax_out = nullptr;
  void* sample_ws = nullptr;
  std::vector<int64_t> h_pos, h_gen;
  std::vector<int> active;                    // slots of the batch decode / last_token follow, in row order
  // workspace of a pass (grows)
  uint8_t* ws = nullptr;
  int ws_tok = 0, ws_rows = 0;
  float *x = nullptr, *x_alt = nullptr, *x0 = nullptr, *y = nullptr, *logits = nullptr;
  void *h = nullptr, *proj = nullptr, *mid = nullptr, *sg = nullptr, *hn = nullptr;
  __nv_bfloat16* logits_bf = nullptr;
  int32_t *m_tok = nullptr, *m_slot = nullptr, *m_pos = nullptr, *m_want = nullptr, *m_upd = nullptr;
  int n_in_max = 0, k_out_max = 0;
  // bf16 engines: the big products leave the general kernel where their shapes allow — the weight-streaming GEMV
  // (gemv.cu / gemv_batch.cu) for steps of up to kMaxBatch rows, the tcgen05 GEMM (gemm.cu) for steps of kGemmRows and
  // more rows; B200_STACK_PLAIN=1 keeps everything on the general kernels
  bool fast = false;
  // the GEMV kernels wait for their producer themselves (griddepcontrol.wait) after they have filled their weight ring,
  // so they may be launched ahead of the end of whatever kernel precedes them; B200_NO_PDL=1 turns that off
  bool pdl = true;
  int num_sms = 148;
  struct Plans {
    GemvPlan in{}, out{}, side_gate{}, side_proj{};
    bool ok_in = false, ok_out = false, ok_side = false;
  };
  // the step's sequences as row ranges of the row list (host mirror; empty for decode steps): the tensor-core prompt
  // attention runs per sequence
  struct Seg {
    int row0, count, slot, pos0;
  };
  std::vector<Seg> segs;
  float* attn_ws = nullptr;       // split-key partials of decode steps
  unsigned int* attn_tickets = nullptr;
  int max_heads = 1, max_vdim = 1;
  std::vector<Plans> plans;
  GemvPlan p_mix{}, p_head{}, p_head_f{};   // p_head_f: final norm fused (rows in stream order)
  bool ok_mix = false, ok_head = false;
  __nv_bfloat16* cat = nullptr;   // bf16 [x | x0] rows for the mix-in product
  // greedy decode steps as CUDA graphs, one per number of rows (row → slot goes through row_slot on the device, so a
  // graph outlives changes of the active set); dropped when the workspace moves
  std::map<int, cudaGraphExec_t> g_dec;
  std::map<int, int> g_launches_of;
  // ---- sandwich blocks
  // recurrent state (mLSTM runs): fp32 [slot][run's share]; a sequence at position 0 starts from zero, so a slot that is
  // given back needs no clearing
  float* rstate = nullptr;
  std::vector<size_t> run_s_off;   // floats from the start of a slot
  size_t s_slot = 0;               // floats per slot
  bool recurrent = false;          // some run carries state that cannot be rewound
  void *qa = nullptr, *ol = nullptr, *lin_tmp = nullptr;
  float *projf = nullptr, *rec_o = nullptr, *rec_ab = nullptr, *y2 = nullptr;
  int32_t *m_seg_row0 = nullptr, *m_seg_count = nullptr;
  MoeRun moe_ws{};                 // the routing workspace's pointers
  float* lat_ws = nullptr;         // split-key partials of decode-shaped latent attention
  int lat_heads_max = 0, lat_rank_max = 0, lat_hd_max = 0, lat_hv_max = 0;
  __nv_bfloat16 *lat_c = nullptr, *lat_kp = nullptr, *lat_k = nullptr, *lat_v = nullptr, *lat_q = nullptr;   // one sequence's expanded keys / values
  int qa_max = 0, ol_max = 0, rec_o_max = 0, moe_e_max = 0, moe_top_max = 0, moe_ff_max = 0, lin_max = 0;
  bool any_rec = false, any_moe = false;
  bool h_ready = false;            // the previous sublayer's fused post-norm already left this run's normed input in h
  // ---- post-norm blocks: the scan's fp32 operand rows, the decay projection's two stages, the kept values of a pass
  float *rec_f = nullptr, *rec_wl = nullptr;
  void *rec_lr = nullptr, *vkeep = nullptr;
  int rec_f_max = 0, rec_wl_max = 0, rec_lr_max = 0, vkeep_max = 0;
  void* latq = nullptr;            // [tok, heads·(dim + rot_dim)] T: queries that came through a latent of their own
  int latq_max = 0;
  struct SPlans {
    GemvPlan in{}, out{}, ff_in{}, ff_out{}, lora{}, uq{};
    bool ok_in = false, ok_out = false, ok_ff_in = false, ok_ff_out = false, ok_lora = false, ok_uq = false;
  };
  std::vector<SPlans> splans;
};
static inline int up8i(int n) { return (n + 7) / 8 * 8; }
constexpr int kGemmRows = 32;

namespace {

// rows of a [B, S] id matrix (columns s0 … s0+cs) → the step's row list; positions continue each slot's cache
__global__ void stack_meta_from_ids_kernel(const int64_t* __restrict__ ids, int B, int S, int s0, int cs,
                                           const int* __restrict__ pos_dev, int32_t* tok, int32_t* slot, int32_t* pos) {
  const int n = B * cs;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n; e += gridDim.x * blockDim.x) {
    const int b = e / cs, t = e % cs;
    tok[e] = (int32_t)ids[(int64_t)b * S + s0 + t];
    slot[e] = b;
    pos[e] = pos_dev[b] + s0 + t;
  }
}
// one decode token per active row: the slot's current token at the slot's position, which then advances
__global__ void stack_meta_decode_kernel(const int* __restrict__ row_slot, int rows, int* pos_dev,
                                         const int64_t* __restrict__ cur_tok, int32_t* tok, int32_t* slot, int32_t* pos,
                                         int32_t* want) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int s = row_slot[r];
  const int p = pos_dev[s];
  tok[r] = (int32_t)cur_tok[s];
  slot[r] = s;
  pos[r] = p;
  want[r] = r;
  pos_dev[s] = p + 1;
}
// {slot, new position} pairs decided on the host
__global__ void stack_set_pos_kernel(const int32_t* __restrict__ upd, int n, int* pos_dev) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) pos_dev[upd[2 * i]] = upd[2 * i + 1];
}
__global__ void stack_iota_last_kernel(int32_t* want, int B, int cs) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) want[b] = b * cs + cs - 1;
}
__global__ void stack_iota_kernel(int32_t* want, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) want[i] = i;
}

}  // namespace

static int stack_workspace(StackEngine* s, int tok, int rows) {
  if (s->ws != nullptr && s->ws_tok >= tok && s->ws_rows >= rows) return B200_OK;
  tok = std::max(tok, s->ws_tok);
  rows = std::max(rows, s->ws_rows);
  if (s->ws) {
    B200_CUDA(cudaDeviceSynchronize());
    cudaFree(s->ws);
    s->ws = nullptr;
    for (auto& kv : s->g_dec) cudaGraphExecDestroy(kv.second);
    s->g_dec.clear();
  }
  const b200_stack_desc& d = s->d;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  const size_t W = d.width, T = tok;
  const size_t o_x = take(T * W * 4), o_xa = take(T * W * 4), o_x0 = take(T * W * 4), o_y = take(T * W * 4);
  const size_t o_h = take(T * W * s->esz), o_proj = take(T * s->n_in_max * s->esz);
  const size_t o_mid = take(T * s->k_out_max * s->esz), o_sg = take(T * std::max(1, d.side_dim) * s->esz);
  const size_t o_hn = take((size_t)rows * W * s->esz), o_lg = take((size_t)rows * d.vocab * 4);
  const size_t o_lb = take((size_t)rows * d.vocab * 2);
  const size_t o_meta = take((5 * T + rows + 2 * (size_t)d.max_slots) * 4);
  const size_t o_cat = take(d.mix_in != nullptr && s->dtype == B200_BF16 ? T * 2 * W * 2 : 0);
  const size_t o_aws = take((size_t)kStackSplitRows * s->max_heads * kStackMaxSplits * (2 + s->max_vdim) * 4);
  const size_t o_tick = take((size_t)kStackSplitRows * s->max_heads * 4);
  // sandwich blocks
  const bool sw = d.block != B200_BLOCK_PARALLEL;
  const size_t o_qa = take(sw ? T * s->qa_max * s->esz : 0), o_ol = take(sw ? T * s->ol_max * s->esz : 0);
  const size_t o_lt = take(sw ? T * s->lin_max * 2 : 0);
  const size_t o_pf = take(s->any_rec ? (size_t)kMaxBatch * s->n_in_max * 4 + T * 2 * s->max_heads * 4 : 0);
  const size_t o_ro = take(s->any_rec ? T * s->rec_o_max * 4 : 0), o_y2 = take(sw ? T * W * 4 : 0);
  const size_t o_rab = take(s->any_rec ? T * 3 * s->max_heads * 4 : 0);
  const size_t P = T * std::max(1, s->moe_top_max);
  const size_t o_mz = take(s->any_moe ? T * s->moe_e_max * 4 : 0), o_me = take(s->any_moe ? P * 4 : 0);
  const size_t o_mw = take(s->any_moe ? P * 4 : 0), o_mp = take(s->any_moe ? (size_t)moe_plan_ints((int)P, s->moe_e_max) * 4 : 0);
  const size_t o_ms = take(s->any_moe ? P * 4 : 0), o_ma = take(s->any_moe ? P * W * s->esz : 0);
  const size_t o_mg = take(s->any_moe ? P * 2 * s->moe_ff_max * s->esz : 0), o_mc = take(s->any_moe ? P * s->moe_ff_max * s->esz : 0);
  const size_t o_mo = take(s->any_moe ? P * W * 4 : 0), o_mb = take(s->any_moe && s->fast ? P * W * 2 : 0);
  const size_t o_lw = take(s->lat_rank_max > 0 ? (size_t)kSmallRows * s->lat_heads_max * kLatentMaxSplits * (2 + std::min(s->lat_rank_max, 512)) * 4 : 0);
  const bool lx = s->fast && s->lat_rank_max > 0;
  const size_t C = d.max_ctx;
  const size_t o_lc = take(lx ? C * s->lat_rank_max * 2 : 0), o_lkp = take(lx ? C * s->lat_hd_max * 2 : 0);
  const size_t o_lk = take(lx ? C * s->lat_hd_max * 2 : 0), o_lv = take(lx ? C * s->lat_hv_max * 2 : 0);
  const size_t o_lq = take(lx ? T * s->lat_hd_max * 2 : 0);
  const size_t o_rf = take(T * s->rec_f_max * 4), o_rw = take(T * s->rec_wl_max * 4);
  const size_t o_rl = take(T * s->rec_lr_max * s->esz), o_vk = take(T * s->vkeep_max * s->esz);
  const size_t o_lqq = take(T * s->latq_max * s->esz);
  B200_CUDA(cudaMalloc((void**)&s->ws, off));
  B200_CUDA(cudaMemset(s->ws, 0, off));
  s->lat_c = lx ? (__nv_bfloat16*)(s->ws + o_lc) : nullptr;
  s->lat_kp = (__nv_bfloat16*)(s->ws + o_lkp);
  s->lat_k = lx ? (__nv_bfloat16*)(s->ws + o_lk) : nullptr;
  s->lat_v = (__nv_bfloat16*)(s->ws + o_lv);
  s->lat_q = (__nv_bfloat16*)(s->ws + o_lq);
  s->rec_f = (float*)(s->ws + o_rf);
  s->rec_wl = (float*)(s->ws + o_rw);
  s->rec_lr = s->ws + o_rl;
  s->vkeep = s->ws + o_vk;
  s->latq = s->ws + o_lqq;
  s->ws_tok = tok;
  s->ws_rows = rows;
  s->x = (float*)(s->ws + o_x);
  s->x_alt = (float*)(s->ws + o_xa);
  s->x0 = (float*)(s->ws + o_x0);
  s->y = (float*)(s->ws + o_y);
  s->h = s->ws + o_h;
  s->proj = s->ws + o_proj;
  s->mid = s->ws + o_mid;
  s->sg = s->ws + o_sg;
  s->hn = s->ws + o_hn;
  s->logits = (float*)(s->ws + o_lg);
  s->logits_bf = (__nv_bfloat16*)(s->ws + o_lb);
  s->m_tok = (int32_t*)(s->ws + o_meta);
  s->m_slot = s->m_tok + T;
  s->m_pos = s->m_slot + T;
  s->m_want = s->m_pos + T;
  s->m_upd = s->m_want + rows;
  s->m_seg_row0 = s->m_upd + 2 * (size_t)d.max_slots;
  s->m_seg_count = s->m_seg_row0 + T;
  s->qa = s->ws + o_qa;
  s->ol = s->ws + o_ol;
  s->lin_tmp = s->ws + o_lt;
  s->projf = (float*)(s->ws + o_pf);
  s->rec_o = (float*)(s->ws + o_ro);
  s->rec_ab = (float*)(s->ws + o_rab);
  s->y2 = (float*)(s->ws + o_y2);
  s->moe_ws.z = (float*)(s->ws + o_mz);
  s->moe_ws.sel_e = (int32_t*)(s->ws + o_me);
  s->moe_ws.sel_w = (float*)(s->ws + o_mw);
  s->moe_ws.plan = (int32_t*)(s->ws + o_mp);
  s->moe_ws.pair_slot = (int32_t*)(s->ws + o_ms);
  s->moe_ws.a_perm = s->ws + o_ma;
  s->moe_ws.gu = s->ws + o_mg;
  s->moe_ws.act = s->ws + o_mc;
  s->moe_ws.outp = (float*)(s->ws + o_mo);
  s->moe_ws.outp_bf = (__nv_bfloat16*)(s->ws + o_mb);
  s->lat_ws = s->lat_rank_max > 0 ? (float*)(s->ws + o_lw) : nullptr;
  s->cat = (__nv_bfloat16*)(s->ws + o_cat);
  s->attn_ws = (float*)(s->ws + o_aws);
  s->attn_tickets = (unsigned int*)(s->ws + o_tick);
  return B200_OK;
}

static inline bool gemm_shape_ok(int64_t N, int64_t K) { return N % 8 == 0 && K % 8 == 0 && K >= 64; }

// proj = rmsnorm(x)·(offset + w) · w_inᵀ + b_in
static int stack_product_in(StackEngine* s, int li, const float* x, int n_tok, cudaStream_t st) {
  const b200_stack_layer& L = s->layers[li];
  const b200_stack_desc& d = s->d;
  const int W = d.width;
  int rc;
  if (s->fast && n_tok <= kMaxBatch && s->plans[li].ok_in) {   // the norm is the GEMV's prologue
    GemvPlan pl = s->plans[li].in;
    pl.p.xf = x;
    pl.p.fnorm_w = L.norm;
    pl.p.norm_offset = d.norm_offset;
    pl.p.eps = d.norm_eps;
    pl.p.y = (__nv_bfloat16*)s->proj;
    pl.p.fbias = L.b_in;
    if ((rc = gemv_plan_set_batch(&pl, n_tok)) != B200_OK) return rc;
    return gemv_launch(pl, st, s->pdl);
  }
  if ((rc = launch_stack_rmsnorm(s->h, x, L.norm, nullptr, n_tok, W, d.norm_eps, d.norm_offset, s->dtype, st)) != B200_OK)
    return rc;
  if (s->fast && n_tok >= kGemmRows && gemm_shape_ok(L.n_in, W)) {
    if ((rc = launch_gemm_bf16(s->proj, s->h, L.w_in, n_tok, L.n_in, W, st)) != B200_OK) return rc;
    return L.b_in ? launch_stack_bias_add((__nv_bfloat16*)s->proj, L.b_in, n_tok, L.n_in, st) : B200_OK;
  }
  StackGemm g;
  g.a = s->h; g.lda = W; g.k1 = W;
  g.w = L.w_in; g.bias = L.b_in; g.M = n_tok; g.N = L.n_in; g.K = W;
  g.epi = SEPI_STORE; g.c = s->proj; g.ldc = L.n_in;
  return launch_stack_gemm(g, s->dtype, st);
}

// x += m · mid·w_outᵀ
static int stack_product_out(StackEngine* s, int li, float* x, int n_tok, cudaStream_t st) {
  const b200_stack_layer& L = s->layers[li];
  const int W = s->d.width;
  int rc;
  if (s->fast && n_tok <= kMaxBatch && s->plans[li].ok_out) {
    GemvPlan pl = s->plans[li].out;
    pl.p.x = (const __nv_bfloat16*)s->mid;
    pl.p.yf = x;
    pl.p.mult = s->d.residual_mult;
    if ((rc = gemv_plan_set_batch(&pl, n_tok)) != B200_OK) return rc;
    return gemv_launch(pl, st, s->pdl);
  }
  if (s->fast && n_tok >= kGemmRows && gemm_shape_ok(W, L.k_out)) {   // h is free again: it holds the bf16 product
    if ((rc = launch_gemm_bf16(s->h, s->mid, L.w_out, n_tok, W, L.k_out, st)) != B200_OK) return rc;
    return launch_stack_axpy(x, (const __nv_bfloat16*)s->h, s->d.residual_mult, true, (int64_t)n_tok * W, st);
  }
  StackGemm g;
  g.a = s->mid; g.lda = L.k_out; g.k1 = L.k_out;
  g.w = L.w_out; g.M = n_tok; g.N = W; g.K = L.k_out;
  g.epi = SEPI_RESIDUAL; g.c = x; g.ldc = W; g.mult = s->d.residual_mult;
  return launch_stack_gemm(g, s->dtype, st);
}

// other = mix_in·[cur; x0]
static int stack_product_mix(StackEngine* s, const float* cur, float* other, int n_tok, cudaStream_t st) {
  const int W = s->d.width;
  int rc;
  const bool gemv = s->fast && n_tok <= kMaxBatch && s->ok_mix;
  const bool gemm = s->fast && n_tok >= kGemmRows && gemm_shape_ok(W, 2 * W);
  if (gemv || gemm) {
    if ((rc = launch_stack_cat_cast(s->cat, cur, s->x0, gemv ? other : nullptr, n_tok, W, st)) != B200_OK) return rc;
    if (gemv) {
      GemvPlan pl = s->p_mix;
      pl.p.x = s->cat;
      pl.p.yf = other;
      pl.p.mult = 1.f;
      if ((rc = gemv_plan_set_batch(&pl, n_tok)) != B200_OK) return rc;
      return gemv_launch(pl, st, s->pdl);
    }
    if ((rc = launch_gemm_bf16(s->h, s->cat, s->d.mix_in, n_tok, W, 2 * W, st)) != B200_OK) return rc;
    return launch_stack_axpy(other, (const __nv_bfloat16*)s->h, 1.f, false, (int64_t)n_tok * W, st);
  }
  StackGemm g;
  g.a = cur; g.a2 = s->x0; g.lda = g.lda2 = W; g.k1 = W; g.a_f32 = true;
  g.w = s->d.mix_in; g.M = n_tok; g.N = W; g.K = 2 * W;
  g.epi = SEPI_STORE_F32; g.c = other; g.ldc = W;
  return launch_stack_gemm(g, s->dtype, st);
}

// logits (fp32) and logits_bf (bf16) = rmsnorm(x[rows])·(offset + w) · headᵀ; rows == null: the stream's rows in order
static int stack_product_head(StackEngine* s, const float* x, const int32_t* rows, int n_rows, cudaStream_t st) {
  const b200_stack_desc& d = s->d;
  int rc;
  const int64_t n_lg = (int64_t)n_rows * d.vocab;
  if (s->fast && n_rows <= kMaxBatch && s->ok_head && rows == nullptr && d.norm_kind == B200_NORM_RMS) {   // the final norm is the GEMV's prologue
    GemvPlan pl = s->p_head_f;
    pl.p.xf = x;
    pl.p.fnorm_w = d.final_norm;
    pl.p.norm_offset = d.norm_offset;
    pl.p.eps = d.norm_eps;
    pl.p.y = s->logits_bf;
    pl.p.yf = s->logits;
    if ((rc = gemv_plan_set_batch(&pl, n_rows)) != B200_OK) return rc;
    if ((rc = gemv_launch(pl, st, false)) != B200_OK) return rc;   // copies and the argmax follow: a full dependency
    return d.logit_softcap > 0.f ? launch_stack_softcap(s->logits, s->logits_bf, n_lg, d.logit_softcap, st) : B200_OK;
  }
  if ((rc = launch_stack_norm(s->hn, x, d.final_norm, rows, n_rows, d.width, d.norm_eps, d.norm_offset, d.norm_kind, s->dtype,
                              st)) != B200_OK)
    return rc;
  if (s->fast && n_rows <= kMaxBatch && s->ok_head) {
    GemvPlan pl = s->p_head;
    pl.p.x = (const __nv_bfloat16*)s->hn;
    pl.p.y = s->logits_bf;
    pl.p.yf = s->logits;
    if ((rc = gemv_plan_set_batch(&pl, n_rows)) != B200_OK) return rc;
    if ((rc = gemv_launch(pl, st, false)) != B200_OK) return rc;   // copies and the argmax follow: a full dependency
    return d.logit_softcap > 0.f ? launch_stack_softcap(s->logits, s->logits_bf, n_lg, d.logit_softcap, st) : B200_OK;
  }
  StackGemm g;
  g.a = s->hn; g.lda = d.width; g.k1 = d.width;
  g.w = d.head; g.M = n_rows; g.N = d.vocab; g.K = d.width;
  g.epi = SEPI_LOGITS; g.c = s->logits; g.ldc = d.vocab; g.c2 = s->logits_bf; g.softcap = d.logit_softcap;
  return launch_stack_gemm(g, s->dtype, st);
}

// Attention of a run over the step's rows.  bf16 engines with equal key / value head sizes of 64 or 128 send every
// sequence that brings kTcRows rows or more to the tensor-core kernel (prefill_attn.cu), one launch per sequence; what is
// left (short parts, decode tokens, other head sizes, fp32) goes to the general kernel, with the keys split over CTAs when
// the step is a handful of rows over a long key list.
constexpr int kTcRows = 16;
static int stack_attention(StackEngine* s, const StackAttn& a, const b200_stack_layer& L, cudaStream_t st) {
  const b200_attn_desc& d = L.attn;
  const int dt = s->dtype;
  int rc;
  auto general = [&](int row0, int count) {
    StackAttn q = a;
    q.proj = (const uint8_t*)a.proj + (size_t)row0 * a.ld_proj * s->esz;
    q.out = (uint8_t*)a.out + (size_t)row0 * a.ld_out * s->esz;
    q.slot = a.slot + row0;
    q.pos = a.pos + row0;
    q.n_tok = count;
    const int kmax = d.window > 0 ? std::min(d.window + d.keep_first, s->d.max_ctx) : s->d.max_ctx;
    const int nsplit = std::min(kStackMaxSplits, (kmax + kStackSplitKeys - 1) / kStackSplitKeys);
    if (count <= kStackSplitRows && nsplit > 1) {
      q.split_ws = s->attn_ws;
      q.split_tickets = s->attn_tickets;
      q.nsplit = nsplit;
      q.keys_per_split = ((kmax + nsplit - 1) / nsplit + 31) / 32 * 32;
    }
    return launch_stack_attention(q, dt, st);
  };
  const bool tc = s->fast && d.dim == d.vdim && (d.dim == 64 || d.dim == 128);
  bool any = false;
  for (const StackEngine::Seg& g : s->segs) any = any || g.count >= kTcRows;
  if (!tc || !any) return general(0, a.n_tok);
  for (const StackEngine::Seg& g : s->segs) {
    if (g.count < kTcRows) {
      if ((rc = general(g.row0, g.count)) != B200_OK) return rc;
      continue;
    }
    const __nv_bfloat16* prow = (const __nv_bfloat16*)a.proj + (size_t)g.row0 * a.ld_proj;
    if ((rc = launch_attn_prefill_window((__nv_bfloat16*)a.out + (size_t)g.row0 * a.ld_out, a.ld_out, prow + a.off_q,
                                         d.out_gate ? prow + a.off_g : nullptr, a.ld_proj,
                                         (const __nv_bfloat16*)a.kcache + (size_t)g.slot * a.k_slot_stride,
                                         (const __nv_bfloat16*)a.vcache + (size_t)g.slot * a.v_slot_stride, g.count, d.heads,
                                         d.kv_heads, d.dim, g.pos0, d.scale, d.window, d.keep_first, st, d.sink)) != B200_OK)
      return rc;
  }
  return B200_OK;
}

// x += m · rmsnorm(side_proj·(gelu(side_gate·x) ∘ table[token]))·w_side
static int stack_side(StackEngine* s, int li, float* cur, int n_tok, cudaStream_t st) {
  const b200_stack_desc& d = s->d;
  const b200_stack_layer& L = s->layers[li];
  const int W = d.width, sd = d.side_dim;
  int rc;
  const bool gemv = s->fast && n_tok <= kMaxBatch && s->plans[li].ok_side;
  const bool gemm = s->fast && n_tok >= kGemmRows && gemm_shape_ok(sd, W) && gemm_shape_ok(W, sd);
  if (gemv || gemm) {
    // bf16 operand of the stream in h, the gate product in proj (both are free here), the gated table row in sg
    __nv_bfloat16 *xb = (__nv_bfloat16*)s->h, *raw = (__nv_bfloat16*)s->proj, *sg = (__nv_bfloat16*)s->sg;
    if (gemv) {   // one launch: fp32 stream in, gelu(·)·table row out
      GemvPlan pl = s->plans[li].side_gate;
      pl.p.xf = cur;
      pl.p.y = sg;
      pl.p.table = (const __nv_bfloat16*)d.side_table;
      pl.p.tok = s->m_tok;
      pl.p.table_ld = d.side_stride;
      pl.p.table_col = L.side_col;
      if ((rc = gemv_plan_set_batch(&pl, n_tok)) != B200_OK || (rc = gemv_launch(pl, st, s->pdl)) != B200_OK) return rc;
    } else {
      if ((rc = launch_stack_cast(xb, cur, (int64_t)n_tok * W, st)) != B200_OK) return rc;
      if ((rc = launch_gemm_bf16(raw, xb, L.side_gate, n_tok, sd, W, st)) != B200_OK) return rc;
      if ((rc = launch_stack_act_table(sg, raw, d.side_table, s->m_tok, d.side_stride, L.side_col, n_tok, sd, st)) != B200_OK)
        return rc;
    }
    if (gemv) {
      GemvPlan pl = s->plans[li].side_proj;
      pl.p.x = sg;
      pl.p.y = xb;          // the rounded copy is not used
      pl.p.yf = s->y;
      if ((rc = gemv_plan_set_batch(&pl, n_tok)) != B200_OK || (rc = gemv_launch(pl, st, s->pdl)) != B200_OK) return rc;
      return launch_stack_rms_add(cur, s->y, L.side_norm, n_tok, W, d.norm_eps, d.residual_mult, st);
    }
    if ((rc = launch_gemm_bf16(xb, sg, L.side_proj, n_tok, W, sd, st)) != B200_OK) return rc;
    return launch_stack_rms_add_bf16(cur, xb, L.side_norm, n_tok, W, d.norm_eps, d.residual_mult, st);
  }
  StackGemm g;
  g.a = cur; g.lda = W; g.k1 = W; g.a_f32 = true;
  g.w = L.side_gate; g.M = n_tok; g.N = sd; g.K = W;
  g.epi = SEPI_ACT_TABLE; g.c = s->sg; g.ldc = sd;
  g.table = d.side_table; g.tok = s->m_tok; g.table_ld = d.side_stride; g.table_col = L.side_col;
  if ((rc = launch_stack_gemm(g, s->dtype, st)) != B200_OK) return rc;
  StackGemm p;
  p.a = s->sg; p.lda = sd; p.k1 = sd;
  p.w = L.side_proj; p.M = n_tok; p.N = W; p.K = sd;
  p.epi = SEPI_STORE_F32; p.c = s->y; p.ldc = W;
  if ((rc = launch_stack_gemm(p, s->dtype, st)) != B200_OK) return rc;
  return launch_stack_rms_add(cur, s->y, L.side_norm, n_tok, W, d.norm_eps, d.residual_mult, st);
}


// ---------------------------------------------------------------------------------------------------- sandwich blocks
// C = A·Wᵀ + bias for dense T-typed rows A [M, K]: out_t (T [M, N]) and / or out_f (fp32 [M, N]).  bf16 engines stream W
// once for steps of up to kMaxBatch rows (GEMV; both outputs from the same fp32 sums), use the tcgen05 GEMM from kGemmRows
// rows on (bf16 out, widened when fp32 is asked for), and the general kernel otherwise.
static int stack_lin(StackEngine* s, const void* A, const void* Wt, const float* bias, int M, int N, int K, const GemvPlan* plan,
                     void* out_t, float* out_f, cudaStream_t st) {
  int rc;
  if (s->fast && M <= kMaxBatch && plan != nullptr) {
    GemvPlan pl = *plan;
    pl.p.x = (const __nv_bfloat16*)A;
    pl.p.y = (__nv_bfloat16*)(out_t ? out_t : s->lin_tmp);
    pl.p.yf = out_f;
    pl.p.fbias = bias;
    if ((rc = gemv_plan_set_batch(&pl, M)) != B200_OK) return rc;
    return gemv_launch(pl, st, s->pdl);
  }
  if (s->fast && M >= kGemmRows && gemm_shape_ok(N, K)) {
    __nv_bfloat16* o = (__nv_bfloat16*)(out_t ? out_t : s->lin_tmp);
    if ((rc = launch_gemm_bf16(o, A, Wt, M, N, K, st)) != B200_OK) return rc;
    if (bias && (rc = launch_stack_bias_add(o, bias, M, N, st)) != B200_OK) return rc;
    return out_f ? launch_stack_axpy(out_f, o, 1.f, false, (int64_t)M * N, st) : B200_OK;
  }
  StackGemm g;
  g.a = A; g.lda = K; g.k1 = K;
  g.w = Wt; g.bias = bias; g.M = M; g.N = N; g.K = K;
  if (out_t) {
    g.epi = SEPI_STORE; g.c = out_t; g.ldc = N;
    if ((rc = launch_stack_gemm(g, s->dtype, st)) != B200_OK) return rc;
  }
  if (out_f) {
    g.epi = SEPI_STORE_F32; g.c = out_f; g.ldc = N;
    if ((rc = launch_stack_gemm(g, s->dtype, st)) != B200_OK) return rc;
  }
  return B200_OK;
}

// x += norm(A·Wᵀ)·w  — a sublayer's out-projection, its post-norm and the residual sum (fp32)
// x += norm(y)·w, and — when the next sublayer's pre-norm weight is given — h = norm(x)·next_w in the same pass
static int stack_norm_add_next(StackEngine* s, float* x, const void* y, bool y_bf16, const float* norm_w, const float* next_w,
                               int M, cudaStream_t st) {
  const b200_stack_desc& d = s->d;
  if (d.block == B200_BLOCK_POSTNORM)   // the next sublayer reads the stream itself: fp32 engines in place, bf16 engines the
    return launch_stack_rms_add_cast(x, y, y_bf16, norm_w,   // copy this pass leaves in h (next_w only says there is one)
                                     next_w != nullptr && s->dtype == B200_BF16 ? (__nv_bfloat16*)s->h : nullptr, M, d.width,
                                     d.norm_eps, d.residual_mult, st);
  if (next_w != nullptr)
    return launch_stack_norm_add_norm(x, y, y_bf16, norm_w, s->h, next_w, M, d.width, d.norm_eps, d.norm_offset, d.residual_mult,
                                      d.norm_kind, s->dtype, st);
  return launch_stack_norm_add(x, y, y_bf16, norm_w, M, d.width, d.norm_eps, d.residual_mult, d.norm_kind, st);
}

static int stack_lin_norm_add(StackEngine* s, const void* A, const void* Wt, int M, int K, const GemvPlan* plan,
                              const float* norm_w, float* x, const float* next_w, cudaStream_t st, const float* bias = nullptr) {
  const int W = s->d.width;
  int rc;
  if (s->fast && !(M <= kMaxBatch && plan != nullptr) && M >= kGemmRows && gemm_shape_ok(W, K)) {
    if ((rc = launch_gemm_bf16(s->lin_tmp, A, Wt, M, W, K, st)) != B200_OK) return rc;
    if (bias && (rc = launch_stack_bias_add((__nv_bfloat16*)s->lin_tmp, bias, M, W, st)) != B200_OK) return rc;
    return stack_norm_add_next(s, x, s->lin_tmp, true, norm_w, next_w, M, st);
  }
  if ((rc = stack_lin(s, A, Wt, bias, M, W, K, plan, nullptr, s->y, st)) != B200_OK) return rc;
  return stack_norm_add_next(s, x, s->y, false, norm_w, next_w, M, st);
}

static int stack_run_sandwich(StackEngine* s, int r, float* x, int n_tok, cudaStream_t st) {
  const b200_stack_desc& d = s->d;
  const int li = s->run_layer[r];
  const b200_stack_layer& L = s->layers[li];
  const StackEngine::SPlans& pl = s->splans[li];
  const int W = d.width, dt = s->dtype;
  const size_t esz = s->esz;
  int rc;
  // every sublayer's post-norm hands the next sublayer its normed input in the same pass; only the first run norms alone
  const bool has_ff = !(L.ff_kind == B200_FF_DENSE && L.ff <= 0);
  // sandwich blocks norm the stream in front of every sublayer; post-norm blocks hand the sublayer the stream itself —
  // fp32 engines read it in place, bf16 engines its rounded copy in h (left there by the previous post-norm pass)
  const bool pre = d.block == B200_BLOCK_SANDWICH;
  const float* next_run_w = r + 1 < d.n_runs ? (pre ? s->layers[s->run_layer[r + 1]].norm : L.post_norm) : nullptr;
  const void* hin = !pre && dt == B200_F32 ? (const void*)x : (const void*)s->h;
  // ---- mixer
  if (pre) {
    if (!s->h_ready &&
        (rc = launch_stack_norm(s->h, x, L.norm, nullptr, n_tok, W, d.norm_eps, d.norm_offset, d.norm_kind, dt, st)) != B200_OK)
      return rc;
  } else if (dt == B200_BF16 && !s->h_ready) {
    if ((rc = launch_stack_cast((__nv_bfloat16*)s->h, x, (int64_t)n_tok * W, st)) != B200_OK) return rc;
  }
  s->h_ready = false;
  // rows whose logits stay fp32 (an mLSTM's gates, Mamba-2's step sizes): the GEMV hands out its unrounded sums, the other
  // paths run those rows again
  const int n_f32 = L.mixer == B200_MIX_MLSTM ? 2 * L.attn.heads : L.mixer == B200_MIX_MAMBA2 ? L.attn.heads : 0;
  const bool gemv_in = s->fast && n_tok <= kMaxBatch && pl.ok_in;
  if ((rc = stack_lin(s, hin, L.w_in, L.b_in, n_tok, L.n_in, W, pl.ok_in ? &pl.in : nullptr, s->proj,
                      n_f32 > 0 && gemv_in ? s->projf : nullptr, st)) != B200_OK)
    return rc;
  const float* f32_rows = nullptr;   // [n_tok, ld_f32]: the fp32 logits of the n_f32 rows from off_gate on
  int64_t ld_f32 = 0;
  if (n_f32 > 0 && gemv_in) {
    f32_rows = s->projf + L.off_gate; ld_f32 = L.n_in;
  } else if (n_f32 > 0) {
    float* gates = s->projf + (size_t)kMaxBatch * s->n_in_max;
    const void* wg = (const uint8_t*)L.w_in + (size_t)L.off_gate * W * esz;
    const float* bg = L.b_in ? L.b_in + L.off_gate : nullptr;
    if (n_tok <= kSmallRows) {
      SmallGemv g;
      g.a = hin; g.lda = W; g.w = wg; g.bias = bg;
      g.c = gates; g.ldc = n_f32; g.c_f32 = true; g.M = n_tok; g.N = n_f32; g.K = W; g.items = 1;
      if ((rc = launch_small_gemv(g, dt, st)) != B200_OK) return rc;
    } else if ((rc = launch_skinny_f32(gates, hin, wg, bg, n_tok, n_f32, W, dt, st)) != B200_OK) {
      return rc;
    }
    f32_rows = gates; ld_f32 = n_f32;
  }
  // the step's sequences for the recurrences (decode steps: every row is a sequence)
  LinScan seq;
  seq.slot = s->m_slot; seq.pos = s->m_pos; seq.n_tok = n_tok; seq.n_seg = n_tok;
  if (!s->segs.empty()) {
    seq.n_seg = (int)s->segs.size(); seq.seg_row0 = s->m_seg_row0; seq.seg_count = s->m_seg_count;
  }
  if (L.mixer == B200_MIX_ATTENTION) {
    const bool shared_kv = s->run_kv_shared[r] != 0;   // the keys and values of these positions are in another run's cache already
    if (L.prep.qk_norm || L.prep.rot_dims > 0 || L.prep.v_norm || L.prep.v_mix) {
      AttnPrep ap;
      ap.a = L.attn; ap.d = L.prep; ap.eps = d.norm_eps;
      ap.proj = s->proj; ap.ld_proj = L.n_in; ap.off_q = L.off_q; ap.off_k = L.off_k; ap.off_v = L.off_v;
      ap.pos = s->m_pos; ap.n_tok = n_tok; ap.vkeep = s->vkeep; ap.ld_keep = s->vkeep_max;
      ap.q_only = shared_kv ? 1 : 0;
      if ((rc = launch_attn_prep(ap, dt, st)) != B200_OK) return rc;
    }
    StackAttn a;
    a.a = L.attn;
    a.proj = s->proj; a.ld_proj = L.n_in;
    a.off_q = L.off_q; a.off_k = L.off_k; a.off_v = L.off_v; a.off_g = L.off_g;
    a.kcache = s->kbase + s->run_k_off[r] * esz;
    a.vcache = s->vbase + s->run_v_off[r] * esz;
    a.k_slot_stride = (int64_t)s->k_slot; a.v_slot_stride = (int64_t)s->v_slot;
    a.slot = s->m_slot; a.pos = s->m_pos; a.n_tok = n_tok;
    a.out = s->mid; a.ld_out = L.k_out;
    bool single = true;   // decode steps append K/V inside the attention launch
    for (const StackEngine::Seg& g : s->segs) single = single && g.count == 1;
    a.own_from_proj = single && !shared_kv ? 1 : 0;
    if (!a.own_from_proj && !shared_kv && (rc = launch_stack_kv_store(a, dt, st)) != B200_OK) return rc;
    if ((rc = stack_attention(s, a, L, st)) != B200_OK) return rc;
  } else if (L.mixer == B200_MIX_GATED_DELTA) {
    const int H = L.attn.heads, G = L.attn.kv_heads;
    GatedDeltaRun m;
    m.a = L.attn; m.d = L.gdelta; m.eps = d.norm_eps;
    m.proj = s->proj; m.ld_proj = L.n_in;
    m.off_q = L.off_q; m.off_k = L.off_k; m.off_v = L.off_v; m.off_g = L.off_g; m.off_b = L.off_gate; m.off_a = L.off_up;
    m.f = s->rec_f;
    m.scan = seq;
    m.scan.ld = gdelta_row_floats(H, G, L.attn.dim, L.attn.vdim);
    m.scan.state = s->rstate + s->run_s_off[r]; m.scan.slot_stride = (int64_t)s->s_slot;
    m.conv_state = m.scan.state + (size_t)H * L.attn.dim * L.attn.vdim;
    m.scan.o = s->rec_o; m.scan.ld_o = (int64_t)H * L.attn.vdim;
    m.mid = s->mid; m.ld_mid = L.k_out;
    if ((rc = run_gdelta(m, dt, st)) != B200_OK) return rc;
  } else if (L.mixer == B200_MIX_DELTA) {
    const int H = L.attn.heads, hd = H * L.attn.dim, rk = up8i(L.delta.rank);
    // decay logits: tanh of the bottleneck rows (T), then w2·(…) + w0 in fp32
    if ((rc = launch_stack_act_mul(s->rec_lr, rk, (const uint8_t*)s->proj + (size_t)L.off_up * esz, nullptr, L.n_in, n_tok, rk,
                                   B200_ACT_TANH, dt, st)) != B200_OK)
      return rc;
    if ((rc = stack_lin(s, s->rec_lr, L.delta.w2, L.delta.w0, n_tok, hd, rk, pl.ok_lora ? &pl.lora : nullptr, nullptr, s->rec_wl,
                        st)) != B200_OK)
      return rc;
    DeltaRun m;
    m.a = L.attn; m.d = L.delta; m.eps = d.norm_eps;
    m.proj = s->proj; m.ld_proj = L.n_in;
    m.off_r = L.off_q; m.off_k = L.off_k; m.off_v = L.off_v; m.off_g = L.off_g; m.off_a = L.off_gate;
    m.wl = s->rec_wl; m.f = s->rec_f;
    m.scan = seq;
    m.scan.ld = delta_row_floats(H, L.attn.dim, L.attn.vdim);
    m.scan.state = s->rstate + s->run_s_off[r]; m.scan.slot_stride = (int64_t)s->s_slot;
    m.scan.o = s->rec_o; m.scan.ld_o = (int64_t)H * L.attn.vdim;
    m.mid = s->mid; m.ld_mid = L.k_out;
    if ((rc = run_delta(m, dt, st)) != B200_OK) return rc;
  } else if (L.mixer == B200_MIX_MAMBA2) {
    const int H = L.attn.heads;
    MambaRun m;
    m.a = L.attn; m.m = L.mamba; m.eps = d.norm_eps;
    m.proj = s->proj; m.ld_proj = L.n_in; m.off_z = L.off_g; m.off_x = L.off_v;
    m.dt = f32_rows; m.ld_dt = ld_f32;
    m.f = s->rec_f;
    m.scan = seq;
    m.scan.ld = mamba_row_floats(H, L.attn.vdim, L.mamba.state, L.mamba.groups);
    m.scan.state = s->rstate + s->run_s_off[r]; m.scan.slot_stride = (int64_t)s->s_slot;
    m.conv_state = m.scan.state + (size_t)H * L.mamba.state * L.attn.vdim;
    m.scan.o = s->rec_o; m.scan.ld_o = (int64_t)H * L.attn.vdim;
    m.mid = s->mid; m.ld_mid = L.k_out;
    if ((rc = run_mamba(m, dt, st)) != B200_OK) return rc;
  } else if (L.mixer == B200_MIX_LATENT) {
    LatentRun a;
    a.a = L.attn; a.l = L.lat; a.eps = d.norm_eps;
    a.proj = s->proj; a.ld_proj = L.n_in; a.off_q = L.off_q; a.off_down = L.off_k;
    a.cache = s->kbase + s->run_k_off[r] * esz; a.slot_stride = (int64_t)s->k_slot;
    a.slot = s->m_slot; a.pos = s->m_pos; a.n_tok = n_tok;
    a.qa = s->qa; a.ol = s->ol; a.out = s->mid; a.ld_out = L.k_out;
    const int hq = L.attn.heads * (L.attn.dim + L.lat.rot_dim);
    if (L.lat.q_rank > 0) {   // queries through a latent of their own: q = uq·(rms(down-projected rows)·q_norm)
      const int qr = L.lat.q_rank, qr8 = up8i(qr);
      if ((rc = launch_stack_rmsnorm_rows(s->rec_lr, qr8, (const uint8_t*)s->proj + (size_t)L.off_q * esz, L.n_in, L.lat.q_norm, n_tok,
                                          qr, qr8, d.norm_eps, dt, st)) != B200_OK)
        return rc;
      if ((rc = stack_lin(s, s->rec_lr, L.lat.uq, nullptr, n_tok, hq, qr8, pl.ok_uq ? &pl.uq : nullptr, s->latq, nullptr, st)) != B200_OK)
        return rc;
      a.q = s->latq; a.ld_q = hq;
    }
    if (n_tok <= kSmallRows && s->lat_ws != nullptr) {   // splits follow the context the engine was built for (or the window),
      a.split_ws = s->lat_ws;                             // not the positions of the moment: a captured step stays valid
      const int kmax = L.attn.window > 0 ? std::min(L.attn.window, d.max_ctx) : d.max_ctx;
      a.nsplit = std::min(kLatentMaxSplits, (kmax + kLatentSplitKeys - 1) / kLatentSplitKeys);
      a.keys_per_split = ((kmax + a.nsplit - 1) / a.nsplit + 31) / 32 * 32;
    }
    // prompts of bf16 engines whose heads suit the tensor-core attention kernel: per sequence, keys and values are expanded
    // from the cache rows by two tcgen05 products and laid out per head; what is left takes the general kernels
    const int hd = L.attn.dim + L.lat.rot_dim, Hh = L.attn.heads, rk = L.lat.kv_rank;
    bool tc = s->fast && s->lat_k != nullptr && L.lat.uk != nullptr && hd == L.attn.vdim && (hd == 64 || hd == 128) &&
              gemm_shape_ok(Hh * L.attn.dim, rk) && gemm_shape_ok(Hh * hd, rk) && L.k_out % 8 == 0 && L.n_in % 8 == 0;
    bool any = false;
    for (const StackEngine::Seg& g : s->segs) any = any || g.count >= kTcRows;
    if (!tc || !any) {
      if ((rc = run_latent_attention(a, dt, st)) != B200_OK) return rc;
    } else {
      if ((rc = launch_latent_prep(a, dt, st)) != B200_OK) return rc;
      const __nv_bfloat16* P0 = (const __nv_bfloat16*)s->proj;
      const bool own_q = a.q != nullptr;   // the per-head queries: their own rows, or the q segment of the projection
      const __nv_bfloat16* Q0 = own_q ? (const __nv_bfloat16*)a.q : P0;
      const int64_t ldq = own_q ? a.ld_q : L.n_in;
      for (const StackEngine::Seg& g : s->segs) {
        if (g.count < kTcRows) {   // a short part: the general kernels on its rows (the cache rows are written again, equal)
          LatentRun b = a;
          b.proj = P0 + (size_t)g.row0 * L.n_in;
          if (own_q) b.q = Q0 + (size_t)g.row0 * ldq;
          b.slot = a.slot + g.row0; b.pos = a.pos + g.row0; b.n_tok = g.count;
          b.qa = (__nv_bfloat16*)s->qa + (size_t)g.row0 * Hh * (rk + L.lat.rot_dim);
          b.ol = (__nv_bfloat16*)s->ol + (size_t)g.row0 * Hh * rk;
          b.out = (__nv_bfloat16*)s->mid + (size_t)g.row0 * L.k_out;
          b.split_ws = nullptr;
          if ((rc = run_latent_attention(b, dt, st)) != B200_OK) return rc;
          continue;
        }
        const int ctx = g.pos0 + g.count, kd = rk + L.lat.rot_dim;
        const __nv_bfloat16* rows = (const __nv_bfloat16*)a.cache + (size_t)g.slot * a.slot_stride;
        B200_CUDA(cudaMemcpy2DAsync(s->lat_c, (size_t)rk * 2, rows, (size_t)kd * 2, (size_t)rk * 2, (size_t)ctx,
                                    cudaMemcpyDeviceToDevice, st));
        if ((rc = launch_gemm_bf16(s->lat_kp, s->lat_c, L.lat.uk, ctx, Hh * L.attn.dim, rk, st)) != B200_OK) return rc;
        if ((rc = launch_gemm_bf16(s->lat_v, s->lat_c, L.lat.uv, ctx, Hh * L.attn.vdim, rk, st)) != B200_OK) return rc;
        LatentPack k;
        k.a = L.attn; k.l = L.lat; k.kp = s->lat_kp; k.cache_rows = rows;
        k.proj = Q0 + (size_t)g.row0 * ldq; k.ld_proj = ldq; k.off_q = own_q ? 0 : L.off_q;
        k.qa = (const __nv_bfloat16*)s->qa + (size_t)g.row0 * Hh * kd;
        k.kbuf = s->lat_k; k.qbuf = s->lat_q; k.ctx = ctx; k.count = g.count;
        if ((rc = launch_latent_pack(k, st)) != B200_OK) return rc;
        if ((rc = launch_attn_prefill_window((__nv_bfloat16*)s->mid + (size_t)g.row0 * L.k_out, L.k_out, s->lat_q, nullptr,
                                             (int64_t)Hh * hd, s->lat_k, s->lat_v, g.count, Hh, Hh, hd, g.pos0, L.attn.scale,
                                             L.attn.window, 0, st)) != B200_OK)
          return rc;
      }
    }
    if (L.lat.out_gate &&
        (rc = launch_stack_sigmoid_gate(s->mid, L.k_out, (const uint8_t*)s->proj + (size_t)L.off_g * esz, L.n_in, n_tok,
                                        L.attn.heads * L.attn.vdim, dt, st)) != B200_OK)
      return rc;
  } else {
    MlstmRun m;
    m.a = L.attn; m.gate_cap = L.rec.gate_cap; m.eps = d.norm_eps;
    m.proj = s->proj; m.ld_proj = L.n_in; m.off_q = L.off_q; m.off_k = L.off_k; m.off_v = L.off_v; m.off_g = L.off_g;
    m.gates = f32_rows; m.ld_gates = ld_f32;
    m.state = s->rstate + s->run_s_off[r]; m.slot_stride = (int64_t)s->s_slot;
    m.slot = s->m_slot; m.pos = s->m_pos; m.n_tok = n_tok;
    if (s->segs.empty()) {
      m.n_seg = n_tok;
    } else {
      m.n_seg = (int)s->segs.size(); m.seg_row0 = s->m_seg_row0; m.seg_count = s->m_seg_count;
    }
    m.gab = s->rec_ab; m.o = s->rec_o; m.head_norm = L.rec.head_norm; m.mid = s->mid; m.ld_mid = L.k_out;
    if ((rc = run_mlstm(m, dt, st)) != B200_OK) return rc;
  }
  if ((rc = stack_lin_norm_add(s, s->mid, L.w_out, n_tok, L.k_out, pl.ok_out ? &pl.out : nullptr, L.post_norm, x,
                               has_ff ? (pre ? L.ff_norm : L.post_norm) : next_run_w, st, L.b_out)) != B200_OK)
    return rc;
  // ---- feed-forward
  if (!has_ff) {
    s->h_ready = next_run_w != nullptr;
    return B200_OK;
  }
  s->h_ready = next_run_w != nullptr;
  if (L.ff_kind == B200_FF_DENSE) {
    if ((rc = stack_lin(s, hin, L.w_ff_in, nullptr, n_tok, L.ff, W, pl.ok_ff_in ? &pl.ff_in : nullptr, s->proj, nullptr, st)) != B200_OK)
      return rc;
    if ((rc = launch_stack_act_mul(s->mid, L.ff, s->proj, nullptr, L.ff, n_tok, L.ff, L.ff_act, dt, st)) != B200_OK) return rc;
    return stack_lin_norm_add(s, s->mid, L.w_ff_out, n_tok, L.ff, pl.ok_ff_out ? &pl.ff_out : nullptr, L.ff_post_norm, x,
                              next_run_w, st);
  }
  MoeRun m = s->moe_ws;
  m.m = L.moe; m.width = W; m.n_tok = n_tok; m.h = hin; m.y = s->y;
  m.small = n_tok <= kSmallRows;
  m.plan_stride = s->moe_e_max;
  m.tc = s->fast && n_tok >= kGemmRows && gemm_shape_ok((L.moe.expert_act != 0 ? 1 : 2) * L.moe.expert_ff, W) &&
         gemm_shape_ok(W, L.moe.expert_ff);
  if (m.tc) {   // that path reads the group sizes back: not inside a stream capture
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    B200_CUDA(cudaStreamIsCapturing(st, &cs));
    m.tc = cs == cudaStreamCaptureStatusNone;
  }
  if (L.moe.shared_ff > 0) {
    const bool plain = L.moe.expert_act != 0;   // up alone behind a plain activation, no gate row
    const int fs = L.moe.shared_ff, n_sh = plain ? up8i(fs) : up8i(2 * fs + 1);
    if ((rc = stack_lin(s, hin, L.w_ff_in, nullptr, n_tok, n_sh, W, pl.ok_ff_in ? &pl.ff_in : nullptr, s->proj, nullptr, st)) != B200_OK)
      return rc;
    if (plain) rc = launch_stack_act_mul(s->mid, fs, s->proj, nullptr, n_sh, n_tok, fs, L.moe.expert_act, dt, st);
    else rc = launch_stack_glu_clamp(s->mid, fs, s->proj, n_sh, n_tok, fs, L.moe.shared_limit, dt, st);
    if (rc != B200_OK) return rc;
    if ((rc = stack_lin(s, s->mid, L.w_ff_out, nullptr, n_tok, W, fs, pl.ok_ff_out ? &pl.ff_out : nullptr, nullptr, s->y2, st)) != B200_OK)
      return rc;
    m.shared = s->y2; m.shared_f32 = true;
    if (!L.moe.shared_plain) {
      m.sg = (const uint8_t*)s->proj + (size_t)2 * fs * esz; m.ld_sg = n_sh;
    }
  }
  if ((rc = run_moe(m, dt, st)) != B200_OK) return rc;
  return stack_norm_add_next(s, x, s->y, false, L.ff_post_norm, next_run_w, n_tok, st);
}

// One pass: n_tok rows {m_tok, m_slot, m_pos} through every run, then the head for the n_rows rows listed in m_want.
// rows_in_order: m_want is 0 … n_rows-1 (decode steps), so the head may read the stream directly.
static int stack_pass(b200_engine* e, int n_tok, int n_rows, cudaStream_t st, bool rows_in_order = false) {
  StackEngine* s = e->stack;
  const b200_stack_desc& d = s->d;
  const int W = d.width, dt = s->dtype;
  int rc;
  if ((rc = launch_stack_embed(s->x, s->x0, d.embed, s->m_tok, n_tok, d.vocab, W, d.embed_scale, dt, st)) != B200_OK)
    return rc;
  float *cur = s->x, *other = s->x_alt;
  s->h_ready = false;
  if (s->any_rec && !s->segs.empty()) {   // the recurrences walk every sequence's rows in order
    std::vector<int32_t> sr(2 * s->segs.size());
    for (size_t i = 0; i < s->segs.size(); ++i) {
      sr[i] = s->segs[i].row0;
      sr[s->segs.size() + i] = s->segs[i].count;
    }
    B200_CUDA(cudaMemcpyAsync(s->m_seg_row0, sr.data(), s->segs.size() * 4, cudaMemcpyHostToDevice, st));
    B200_CUDA(cudaMemcpyAsync(s->m_seg_count, sr.data() + s->segs.size(), s->segs.size() * 4, cudaMemcpyHostToDevice, st));
  }
  for (int r = 0; r < d.n_runs; ++r) {
    const b200_stack_layer& L = s->layers[s->run_layer[r]];
    if (d.block != B200_BLOCK_PARALLEL) {
      if ((rc = stack_run_sandwich(s, r, cur, n_tok, st)) != B200_OK) return rc;
      continue;
    }
    if (s->run_mix[r]) {
      if ((rc = stack_product_mix(s, cur, other, n_tok, st)) != B200_OK) return rc;
      std::swap(cur, other);
    }
    if ((rc = stack_product_in(s, s->run_layer[r], cur, n_tok, st)) != B200_OK) return rc;
    StackAttn a;
    a.a = L.attn;
    a.proj = s->proj; a.ld_proj = L.n_in;
    a.off_q = L.off_q; a.off_k = L.off_k; a.off_v = L.off_v; a.off_g = L.off_g;
    a.kcache = s->kbase + s->run_k_off[r] * s->esz;
    a.vcache = s->vbase + s->run_v_off[r] * s->esz;
    a.k_slot_stride = (int64_t)s->k_slot; a.v_slot_stride = (int64_t)s->v_slot;
    a.slot = s->m_slot; a.pos = s->m_pos; a.n_tok = n_tok;
    a.out = s->mid; a.ld_out = L.k_out;
    const int hv = L.attn.heads * L.attn.vdim;
    if (hv != L.off_act || L.off_act + L.ff != L.k_out)   // padding columns meet zero weights: keep them finite
      B200_CUDA(cudaMemsetAsync(s->mid, 0, (size_t)n_tok * L.k_out * s->esz, st));
    // steps in which every row is its sequence's only new row (decode) append K/V inside the attention launch
    bool single = true;
    for (const StackEngine::Seg& g : s->segs) single = single && g.count == 1;
    a.own_from_proj = single ? 1 : 0;
    if (!a.own_from_proj && (rc = launch_stack_kv_store(a, dt, st)) != B200_OK) return rc;
    if ((rc = stack_attention(s, a, L, st)) != B200_OK) return rc;
    if (L.ff > 0) {
      const uint8_t* p = (const uint8_t*)s->proj;
      if ((rc = launch_stack_act_mul((uint8_t*)s->mid + (size_t)L.off_act * s->esz, L.k_out, p + (size_t)L.off_gate * s->esz,
                                     p + (size_t)L.off_up * s->esz, L.n_in, n_tok, L.ff, L.ff_act, dt, st)) != B200_OK)
        return rc;
    }
    if ((rc = stack_product_out(s, s->run_layer[r], cur, n_tok, st)) != B200_OK) return rc;
    if (L.side_gate != nullptr && (rc = stack_side(s, s->run_layer[r], cur, n_tok, st)) != B200_OK) return rc;
  }
  if (n_rows > 0 && (rc = stack_product_head(s, cur, rows_in_order ? nullptr : s->m_want, n_rows, st)) != B200_OK) return rc;
  return B200_OK;
}

// greedy / sampled token of logits rows [row0, row0 + n) → the slots in `slots` (row order)
static int stack_publish(b200_engine* e, int row0, const std::vector<int>& slots, cudaStream_t st) {
  StackEngine* s = e->stack;
  const int n = (int)slots.size();
  const __nv_bfloat16* lg = s->logits_bf + (size_t)row0 * s->d.vocab;
  int rc;
  if (e->sampler_on) {
    for (int r = 0; r < n; ++r) {
      ArgmaxPublish pub;
      const int sl = slots[r];
      pub.cur_tok = s->cur_tok + sl;
      pub.gen_log = s->gen_log + (size_t)sl * s->gen_cap;
      pub.gen_count = s->gen_count + sl;
      pub.gen_cap = s->gen_cap;
      if ((rc = launch_sample(nullptr, lg + (size_t)r * s->d.vocab, s->d.vocab, e->s_temperature, e->s_top_k, e->s_top_p,
                              e->s_min_p, 0.f, s->sample_ws, st, &pub, e->s_seed, true)) != B200_OK)
        return rc;
    }
  } else {
    ArgmaxPublish pub;
    pub.cur_tok = s->cur_tok;
    pub.gen_log = s->gen_log;
    pub.gen_count = s->gen_count;
    pub.gen_cap = s->gen_cap;
    pub.row_slot = s->row_slot;
    if ((rc = launch_argmax(s->amax_out, lg, n, s->d.vocab, s->argmax_ws, st, false, &pub)) != B200_OK) return rc;
  }
  return B200_OK;
}
static void stack_count_generated(StackEngine* s, const std::vector<int>& slots, int64_t n) {
  for (int sl : slots) s->h_gen[sl] += n;
}

static int stack_set_active(StackEngine* s, const std::vector<int>& slots, cudaStream_t st) {
  if (slots != s->active) {
    s->active = slots;
    B200_CUDA(cudaMemcpyAsync(s->row_slot, slots.data(), slots.size() * 4, cudaMemcpyHostToDevice, st));
  }
  return B200_OK;
}

void stack_destroy(b200_engine* e) {
  StackEngine* s = e->stack;
  if (!s) return;
  for (auto& kv : s->g_dec) cudaGraphExecDestroy(kv.second);
  if (s->cache) cudaFree(s->cache);
  if (s->state) cudaFree(s->state);
  if (s->rstate) cudaFree(s->rstate);
  if (s->ws) cudaFree(s->ws);
  delete s;
  e->stack = nullptr;
}

int stack_reset(b200_engine* e, cudaStream_t st) {
  StackEngine* s = e->stack;
  B200_CUDA(cudaMemsetAsync(s->pos_dev, 0, (size_t)s->d.max_slots * 4, st));
  std::fill(s->h_pos.begin(), s->h_pos.end(), 0);
  e->h_pos = 0;
  return B200_OK;
}

static int stack_push_positions(StackEngine* s, const std::vector<int32_t>& upd, cudaStream_t st) {
  const int n = (int)upd.size() / 2;
  if (n == 0) return B200_OK;
  B200_CUDA(cudaMemcpyAsync(s->m_upd, upd.data(), upd.size() * 4, cudaMemcpyHostToDevice, st));
  B200_CUDA(launch_pdl(stack_set_pos_kernel, dim3((n + 63) / 64), dim3(64), 0, st, false, (const int32_t*)s->m_upd, n,
                       s->pos_dev));
  return B200_OK;
}

int stack_seek(b200_engine* e, int64_t position, cudaStream_t st) {
  StackEngine* s = e->stack;
  // every slot of the active batch is rewound (they advance together under forward / decode)
  std::vector<int> slots = s->active.empty() ? std::vector<int>{0} : s->active;
  if (s->recurrent)   // a recurrent state holds the whole prefix and nothing of its past
    for (int sl : slots)
      if (position != s->h_pos[sl] && position != 0) {
        set_error("engine_seek: this model carries recurrent state; slot %d can only be rewound to position 0", sl);
        return B200_ERR_UNSUPPORTED;
      }
  for (int sl : slots)
    if (position < 0 || position > s->h_pos[sl]) {
      set_error("engine_seek: position %lld is not inside the cached prefix [0, %lld] of slot %d", (long long)position,
                (long long)s->h_pos[sl], sl);
      return B200_ERR_STATE;
    }
  int rc = stack_workspace(s, 1, 1);
  if (rc != B200_OK) return rc;
  std::vector<int32_t> upd;
  for (int sl : slots) {
    upd.push_back(sl);
    upd.push_back((int32_t)position);
    s->h_pos[sl] = position;
  }
  e->h_pos = position;
  return stack_push_positions(s, upd, st);
}

int stack_forward(b200_engine* e, const int64_t* ids, int64_t B, int64_t S, void* logits_out, int logits_mode,
                  cudaStream_t st) {
  StackEngine* s = e->stack;
  const b200_stack_desc& d = s->d;
  B200_CHECK_ARG(B >= 1 && B <= d.max_slots, "engine_forward: batch %lld exceeds the engine's %d slots", (long long)B,
                 d.max_slots);
  B200_CHECK_ARG(S >= 1, "engine_forward: empty sequence");
  B200_CHECK_ARG(logits_mode == 0 || logits_mode == 1, "engine_forward: logits_mode must be 0 or 1");
  for (int b = 0; b < B; ++b)
    if (s->h_pos[b] + S > d.max_ctx) {
      set_error("engine_forward: slot %d: position %lld + %lld tokens exceeds max_ctx %d", b, (long long)s->h_pos[b],
                (long long)S, d.max_ctx);
      return B200_ERR_STATE;
    }
  const bool all = logits_mode == 1 && logits_out != nullptr;
  const int cs_max = std::max<int>(1, kStackChunk / (int)B);
  int rc;
  std::vector<int> slots((size_t)B);
  for (int b = 0; b < B; ++b) slots[b] = b;
  const int ws_tok = (int)std::min<int64_t>(S, cs_max) * (int)B;
  if ((rc = stack_workspace(s, ws_tok, (all ? ws_tok : 0) + (int)B)) != B200_OK) return rc;
  if ((rc = stack_set_active(s, slots, st)) != B200_OK) return rc;
  const size_t vb = (size_t)d.vocab * 2;
  int head_row0 = 0;   // first of the B rows that hold the sequences' last positions
  for (int64_t s0 = 0; s0 < S; s0 += cs_max) {
    const int cs = (int)std::min<int64_t>(cs_max, S - s0);
    const int n_tok = cs * (int)B;
    const bool last = s0 + cs == S;
    B200_CUDA(launch_pdl(stack_meta_from_ids_kernel, dim3((n_tok + 255) / 256), dim3(256), 0, st, false, ids, (int)B, (int)S,
                         (int)s0, cs, (const int*)s->pos_dev, s->m_tok, s->m_slot, s->m_pos));
    // rows: every token of the chunk when all positions are asked for, then (last chunk) the B last positions
    int n_rows = 0;
    if (all) {
      n_rows = n_tok;
      B200_CUDA(launch_pdl(stack_iota_kernel, dim3((n_tok + 255) / 256), dim3(256), 0, st, false, s->m_want, n_tok));
    }
    if (last) {
      head_row0 = n_rows;
      B200_CUDA(launch_pdl(stack_iota_last_kernel, dim3(((int)B + 63) / 64), dim3(64), 0, st, false, s->m_want + n_rows,
                           (int)B, cs));
      n_rows += (int)B;
    }
    s->segs.clear();
    for (int b = 0; b < B; ++b) s->segs.push_back({b * cs, cs, b, (int)s->h_pos[b] + (int)s0});
    if ((rc = stack_pass(e, n_tok, n_rows, st)) != B200_OK) return rc;
    if (all)   // rows are [b][t of this chunk] → logits_out [B][S][V]
      B200_CUDA(cudaMemcpy2DAsync((uint8_t*)logits_out + (size_t)s0 * vb, (size_t)S * vb, s->logits_bf, (size_t)cs * vb,
                                  (size_t)cs * vb, (size_t)B, cudaMemcpyDeviceToDevice, st));
  }
  if (!all && logits_out != nullptr)
    B200_CUDA(cudaMemcpyAsync(logits_out, s->logits_bf, (size_t)B * vb, cudaMemcpyDeviceToDevice, st));
  // the meta kernels read pos_dev + the column offset: advance only now that the whole matrix went through
  std::vector<int32_t> upd;
  for (int b = 0; b < B; ++b) {
    s->h_pos[b] += S;
    upd.push_back(b);
    upd.push_back((int32_t)s->h_pos[b]);
  }
  if ((rc = stack_push_positions(s, upd, st)) != B200_OK) return rc;
  e->h_pos = s->h_pos[0];
  e->batch = (int)B;
  // the greedy token of every sequence's last position becomes its slot's current token
  stack_count_generated(s, slots, 1);
  return stack_publish(e, head_row0, slots, st);
}

// one greedy decode step of the active batch: row list from the slots' device state, the pass, the publication
static int stack_decode_step(b200_engine* e, int B, cudaStream_t st) {
  StackEngine* s = e->stack;
  int rc;
  B200_CUDA(launch_pdl(stack_meta_decode_kernel, dim3((B + 63) / 64), dim3(64), 0, st, false, (const int*)s->row_slot, B,
                       s->pos_dev, (const int64_t*)s->cur_tok, s->m_tok, s->m_slot, s->m_pos, s->m_want));
  s->segs.clear();
  if ((rc = stack_pass(e, B, B, st, true)) != B200_OK) return rc;
  return stack_publish(e, 0, s->active, st);
}

static int stack_capture_decode(b200_engine* e, int B) {
  StackEngine* s = e->stack;
  cudaStream_t st;
  B200_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  cudaGraph_t g = nullptr;
  cudaError_t err = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
  if (err != cudaSuccess) {
    cudaStreamDestroy(st);
    set_error("cudaStreamBeginCapture failed: %s", cudaGetErrorString(err));
    return B200_ERR_CUDA;
  }
  const int64_t before = g_launches.load();
  int rc = stack_decode_step(e, B, st);
  const int64_t n = g_launches.load() - before;
  g_launches.fetch_sub(n);   // capture does not execute anything
  err = cudaStreamEndCapture(st, &g);
  cudaGraphExec_t ex = nullptr;
  if (rc == B200_OK && err == cudaSuccess) err = cudaGraphInstantiate(&ex, g, 0);
  if (g) cudaGraphDestroy(g);
  cudaStreamDestroy(st);
  if (rc != B200_OK) return rc;
  if (err != cudaSuccess) {
    set_error("stack decode graph: %s", cudaGetErrorString(err));
    return B200_ERR_CUDA;
  }
  s->g_dec[B] = ex;
  s->g_launches_of[B] = (int)n;
  e->launches_per_token = (int)n;
  return B200_OK;
}


int stack_decode(b200_engine* e, int64_t n_steps, int64_t* tokens_out, cudaStream_t st) {
  StackEngine* s = e->stack;
  B200_CHECK_ARG(!s->active.empty(), "engine_decode: no active batch (run a forward or a greedy step first)");
  B200_CHECK_ARG(n_steps <= s->gen_cap, "engine_decode: at most %d steps per call", s->gen_cap);
  const int B = (int)s->active.size();
  for (int sl : s->active)
    if (s->h_pos[sl] + n_steps > s->d.max_ctx) {
      set_error("engine_decode: slot %d: position %lld + %lld steps exceeds max_ctx %d", sl, (long long)s->h_pos[sl],
                (long long)n_steps, s->d.max_ctx);
      return B200_ERR_STATE;
    }
  int rc = stack_workspace(s, B, B);
  if (rc != B200_OK) return rc;
  std::vector<int64_t> first(B);
  for (int r = 0; r < B; ++r) first[r] = s->h_gen[s->active[r]];
  const bool graph = e->use_graph && !e->sampler_on;   // the sampler's publication is bound to slots on the host
  if (graph && n_steps > 0 && s->g_dec.find(B) == s->g_dec.end() && (rc = stack_capture_decode(e, B)) != B200_OK) return rc;
  for (int64_t i = 0; i < n_steps; ++i) {
    if (graph) {
      B200_CUDA(cudaGraphLaunch(s->g_dec[B], st));
      g_launches.fetch_add(s->g_launches_of[B]);
    } else if ((rc = stack_decode_step(e, B, st)) != B200_OK) {
      return rc;
    }
  }
  stack_count_generated(s, s->active, n_steps);
  for (int sl : s->active) s->h_pos[sl] += n_steps;
  e->h_pos = s->h_pos[s->active[0]];
  if (tokens_out != nullptr && n_steps > 0) {   // [n_steps][B] from the slots' own logs
    for (int r = 0; r < B; ++r) {
      const int64_t a = first[r] % s->gen_cap;
      const int64_t n1 = std::min<int64_t>(n_steps, s->gen_cap - a);
      const int64_t* log = s->gen_log + (size_t)s->active[r] * s->gen_cap;
      B200_CUDA(cudaMemcpy2DAsync(tokens_out + r, (size_t)B * 8, log + a, 8, 8, (size_t)n1, cudaMemcpyDeviceToDevice, st));
      if (n1 < n_steps)
        B200_CUDA(cudaMemcpy2DAsync(tokens_out + n1 * B + r, (size_t)B * 8, log, 8, 8, (size_t)(n_steps - n1),
                                    cudaMemcpyDeviceToDevice, st));
    }
  }
  return B200_OK;
}

int stack_last_token(b200_engine* e, int64_t* token_out, cudaStream_t st) {
  StackEngine* s = e->stack;
  B200_CHECK_ARG(!s->active.empty(), "engine_last_token: no active batch");
  for (size_t r = 0; r < s->active.size(); ++r)
    B200_CUDA(cudaMemcpyAsync(token_out + r, s->cur_tok + s->active[r], 8, cudaMemcpyDeviceToDevice, st));
  return B200_OK;
}

int stack_set_sampler(b200_engine* e, cudaStream_t st) {
  (void)e;
  (void)st;   // nothing is captured: the next publication reads the engine's sampler fields
  return B200_OK;
}

int64_t stack_bytes_per_token(const b200_engine* e, int64_t ctx) {
  const StackEngine* s = e->stack;
  const b200_stack_desc& d = s->d;
  int64_t bytes = (int64_t)d.vocab * d.width * s->esz;
  for (int r = 0; r < d.n_runs; ++r) {
    const b200_stack_layer& L = s->layers[s->run_layer[r]];
    bytes += ((int64_t)L.n_in * d.width + (int64_t)d.width * L.k_out) * s->esz;
    if (d.block == B200_BLOCK_SANDWICH) {
      const b200_attn_desc& a = L.attn;
      if (L.mixer == B200_MIX_ATTENTION) {
        int64_t keys = ctx + 1;
        if (a.window > 0) keys = std::min<int64_t>(keys, (int64_t)a.window + a.keep_first);
        bytes += (keys + 1) * a.kv_heads * (a.dim + a.vdim) * s->esz;
      } else if (L.mixer == B200_MIX_GATED_DELTA) {   // the state and the convolutions' inputs read and written
        bytes += 2 * gdelta_state_floats(a.heads, a.kv_heads, a.dim, a.vdim, L.gdelta.taps) * 4;
      } else if (L.mixer == B200_MIX_DELTA) {   // the decay's second stage; the state read and written
        bytes += (int64_t)a.heads * a.dim * L.delta.rank * s->esz + 2ll * a.heads * a.dim * a.vdim * 4;
      } else if (L.mixer == B200_MIX_MAMBA2) {
        bytes += 2 * mamba_state_floats(a.heads, a.vdim, L.mamba.state, L.mamba.groups, L.mamba.taps) * 4;
      } else if (L.mixer == B200_MIX_LATENT) {   // uk, uv (uq), the visible cache rows read once and one written
        int64_t keys = ctx + 1;
        if (a.window > 0) keys = std::min<int64_t>(keys, a.window);
        bytes += ((int64_t)a.heads * (a.dim + a.vdim) * L.lat.kv_rank + (keys + 1) * (L.lat.kv_rank + L.lat.rot_dim) +
                  (int64_t)a.heads * (a.dim + L.lat.rot_dim) * L.lat.q_rank) * s->esz;
      }
      else                              // the state read and written
        bytes += 2 * mlstm_state_floats(a.heads, a.dim, a.vdim) * 4;
      if (L.ff_kind == B200_FF_DENSE) bytes += 2ll * L.ff * d.width * s->esz;
      else if (L.moe.expert_act != 0) bytes += ((int64_t)L.moe.experts + 2ll * L.moe.top * L.moe.expert_ff + 2ll * L.moe.shared_ff) * d.width * s->esz;
      else bytes += ((int64_t)L.moe.experts + 3ll * L.moe.top * L.moe.expert_ff + 3ll * L.moe.shared_ff + 1) * d.width * s->esz;
      continue;
    }
    if (s->run_mix[r]) bytes += 2ll * d.width * d.width * s->esz;
    if (L.side_gate) bytes += 2ll * d.side_dim * d.width * s->esz;
    int64_t keys = ctx + 1;
    if (L.attn.window > 0) keys = std::min<int64_t>(keys, (int64_t)L.attn.window + L.attn.keep_first);
    bytes += (keys + 1) * L.attn.kv_heads * (L.attn.dim + L.attn.vdim) * s->esz;
  }
  return bytes;
}

static int stack_build(const b200_stack_desc* desc, b200_engine** out) {
  B200_CHECK_ARG(desc && out, "engine_create_stack: null argument");
  *out = nullptr;
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  const b200_stack_desc& d = *desc;
  B200_CHECK_ARG(d.dtype == B200_BF16 || d.dtype == B200_F32, "engine_create_stack: unknown dtype %d", d.dtype);
  B200_CHECK_ARG(d.block == B200_BLOCK_PARALLEL || d.block == B200_BLOCK_SANDWICH || d.block == B200_BLOCK_POSTNORM,
                 "engine_create_stack: block kind %d not built", d.block);
  B200_CHECK_ARG(d.block != B200_BLOCK_POSTNORM || d.norm_kind == B200_NORM_RMS,
                 "engine_create_stack: post-norm blocks are built with RMS norms");
  B200_CHECK_ARG(d.norm_kind == B200_NORM_RMS || d.norm_kind == B200_NORM_LAYER, "engine_create_stack: norm kind %d not built",
                 d.norm_kind);
  B200_CHECK_ARG(d.block != B200_BLOCK_PARALLEL || d.norm_kind == B200_NORM_RMS,
                 "engine_create_stack: parallel blocks are built with RMS norms");
  B200_CHECK_ARG(d.logit_softcap >= 0.f, "engine_create_stack: negative logit_softcap");
  B200_CHECK_ARG(d.width > 0 && d.vocab > 0 && d.n_layers > 0 && d.n_runs > 0 && d.max_ctx > 0 && d.max_slots > 0,
                 "engine_create_stack: non-positive size");
  B200_CHECK_ARG(d.run_layer_host && d.run_mix_host && d.layers_host && d.embed && d.final_norm && d.head,
                 "engine_create_stack: null pointer");
  b200_engine* e = new (std::nothrow) b200_engine();
  StackEngine* s = new (std::nothrow) StackEngine();
  if (!e || !s) {
    delete e;
    delete s;
    set_error("engine_create_stack: out of host memory");
    return B200_ERR_INVALID;
  }
  e->stack = s;
  struct Guard {
    b200_engine* e;
    ~Guard() {
      if (e) b200_engine_destroy(e);
    }
  } guard{e};
  s->d = d;
  s->dtype = d.dtype;
  s->esz = d.dtype == B200_F32 ? 4 : 2;
  s->layers.assign(d.layers_host, d.layers_host + d.n_layers);
  s->run_layer.assign(d.run_layer_host, d.run_layer_host + d.n_runs);
  s->run_mix.assign(d.run_mix_host, d.run_mix_host + d.n_runs);
  s->d.layers_host = nullptr;
  s->d.run_layer_host = s->d.run_mix_host = nullptr;
  const bool sandwich = d.block != B200_BLOCK_PARALLEL;   // a norm per sublayer: in front and behind, or behind only
  for (int l = 0; sandwich && l < d.n_layers; ++l) {
    const b200_stack_layer& L = s->layers[l];
    const b200_attn_desc& a = L.attn;
    const int W = d.width;
    B200_CHECK_ARG(L.mixer >= B200_MIX_ATTENTION && L.mixer <= B200_MIX_GATED_DELTA, "engine_create_stack: layer %d: mixer kind %d is not built", l, L.mixer);
    B200_CHECK_ARG(a.heads > 0 && a.dim > 0 && a.vdim > 0, "engine_create_stack: layer %d: bad mixer sizes", l);
    B200_CHECK_ARG((L.norm || d.block == B200_BLOCK_POSTNORM) && L.post_norm && L.w_in && L.w_out && L.n_in > 0 &&
                       L.k_out == a.heads * a.vdim,
                   "engine_create_stack: layer %d: null weight or k_out != heads·vdim", l);
    if (L.mixer == B200_MIX_ATTENTION) {
      const b200_attn_prep_desc& q = L.prep;
      B200_CHECK_ARG(a.kv_heads > 0 && a.heads % a.kv_heads == 0 && a.window >= 0 && a.keep_first >= 0 && a.vdim <= 256 && a.dim <= 1024,
                     "engine_create_stack: layer %d: bad attention sizes", l);
      B200_CHECK_ARG(L.off_q >= 0 && L.off_q + a.heads * a.dim <= L.n_in &&
                         (L.kv_share > 0 || (L.off_k + a.kv_heads * a.dim <= L.n_in && L.off_v + a.kv_heads * a.vdim <= L.n_in)) &&
                         (!a.out_gate || L.off_g + a.heads <= L.n_in),
                     "engine_create_stack: layer %d: segment offsets do not fit", l);
      if (L.kv_share > 0) {   // the source: an earlier attention layer with projections of its own and the same cache rows
        B200_CHECK_ARG(L.kv_share - 1 < l, "engine_create_stack: layer %d reads the keys and values of layer %d, which is not an earlier layer", l, L.kv_share - 1);
        const b200_stack_layer& S = s->layers[L.kv_share - 1];
        B200_CHECK_ARG(S.mixer == B200_MIX_ATTENTION && S.kv_share == 0 && S.attn.kv_heads == a.kv_heads && S.attn.dim == a.dim &&
                           S.attn.vdim == a.vdim,
                       "engine_create_stack: layer %d: layer %d is not an attention layer with keys and values of its own and equal sizes", l, L.kv_share - 1);
        B200_CHECK_ARG(!q.v_norm && !q.v_mix, "engine_create_stack: layer %d: a layer without values of its own cannot norm or mix them", l);
      }
      B200_CHECK_ARG(q.rot_dims >= 0 && q.rot_dims % 2 == 0 && q.rot_dims <= a.dim && (q.rot_dims == 0 || q.rot_table) &&
                         (!q.qk_norm || (q.q_norm && q.k_norm)) && q.v_mix >= 0 && q.v_mix <= 2 && (q.v_mix != 2 || q.mix_lambda),
                     "engine_create_stack: layer %d: attention preparation", l);
      if (q.v_mix) {
        B200_CHECK_ARG(s->vkeep_max == 0 || s->vkeep_max == a.kv_heads * a.vdim,
                       "engine_create_stack: layer %d: layers that mix values need equal value sizes", l);
        B200_CHECK_ARG((q.v_mix == 1) == (s->vkeep_max == 0), "engine_create_stack: layer %d: the first value-mixing layer keeps, the later ones mix", l);
        s->vkeep_max = a.kv_heads * a.vdim;
      }
      s->max_vdim = std::max(s->max_vdim, a.vdim);
    } else if (L.mixer == B200_MIX_GATED_DELTA) {
      const b200_gdelta_desc& q = L.gdelta;
      B200_CHECK_ARG(a.dim <= kScanMaxDim && a.kv_heads > 0 && a.heads % a.kv_heads == 0 && q.taps >= 1 && q.taps <= kMambaMaxTaps &&
                         q.conv_w && q.A_log && q.dt_bias && q.head_norm && q.unit_eps >= 0.f,
                     "engine_create_stack: layer %d: gated delta rule description (key size up to %d, 1 … %d taps)", l, kScanMaxDim,
                     kMambaMaxTaps);
      B200_CHECK_ARG(L.off_q >= 0 && L.off_q + a.kv_heads * a.dim <= L.n_in && L.off_k + a.kv_heads * a.dim <= L.n_in &&
                         L.off_v + a.heads * a.vdim <= L.n_in && L.off_g + a.heads * a.vdim <= L.n_in &&
                         L.off_gate + a.heads <= L.n_in && L.off_up + a.heads <= L.n_in,
                     "engine_create_stack: layer %d: segment offsets do not fit", l);
      s->rec_o_max = std::max(s->rec_o_max, a.heads * a.vdim);
      s->rec_f_max = std::max(s->rec_f_max, (int)gdelta_row_floats(a.heads, a.kv_heads, a.dim, a.vdim));
      s->any_rec = s->recurrent = true;
    } else if (L.mixer == B200_MIX_DELTA) {
      const b200_delta_desc& q = L.delta;
      B200_CHECK_ARG(a.dim <= kScanMaxDim && q.rank > 0 && q.w2 && q.w0 && q.head_norm && q.unit_eps >= 0.f,
                     "engine_create_stack: layer %d: delta-rule description", l);
      B200_CHECK_ARG(L.off_q >= 0 && L.off_q + a.heads * a.dim <= L.n_in && L.off_k + a.heads * a.dim <= L.n_in &&
                         L.off_v + a.heads * a.vdim <= L.n_in && L.off_g + a.heads * a.vdim <= L.n_in &&
                         L.off_gate + a.heads * a.dim <= L.n_in && L.off_up + up8i(q.rank) <= L.n_in,
                     "engine_create_stack: layer %d: segment offsets do not fit", l);
      s->rec_o_max = std::max(s->rec_o_max, a.heads * a.vdim);
      s->rec_f_max = std::max(s->rec_f_max, (int)delta_row_floats(a.heads, a.dim, a.vdim));
      s->rec_wl_max = std::max(s->rec_wl_max, a.heads * a.dim);
      s->rec_lr_max = std::max(s->rec_lr_max, up8i(q.rank));
      s->lin_max = std::max(s->lin_max, a.heads * a.dim);
      s->any_rec = s->recurrent = true;
    } else if (L.mixer == B200_MIX_MAMBA2) {
      const b200_mamba_desc& q = L.mamba;
      B200_CHECK_ARG(q.state > 0 && q.state <= kScanMaxDim && q.groups > 0 && a.heads % q.groups == 0 && q.taps >= 1 &&
                         q.taps <= kMambaMaxTaps && q.norm_groups > 0 && (a.heads * a.vdim) % q.norm_groups == 0 && a.dim == q.state,
                     "engine_create_stack: layer %d: Mamba-2 sizes (state 1 … %d, 1 … %d taps, groups dividing the heads)", l,
                     kScanMaxDim, kMambaMaxTaps);
      B200_CHECK_ARG(q.conv_w && q.conv_b && q.dt_bias && q.A_log && q.D && q.norm, "engine_create_stack: layer %d: null Mamba-2 weight", l);
      B200_CHECK_ARG(L.off_g >= 0 && L.off_g + a.heads * a.vdim <= L.n_in &&
                         L.off_v + a.heads * a.vdim + 2 * q.groups * q.state <= L.n_in && L.off_gate + a.heads <= L.n_in,
                     "engine_create_stack: layer %d: segment offsets do not fit", l);
      s->rec_o_max = std::max(s->rec_o_max, a.heads * a.vdim);
      s->rec_f_max = std::max(s->rec_f_max, (int)mamba_row_floats(a.heads, a.vdim, q.state, q.groups));
      s->any_rec = s->recurrent = true;
    } else if (L.mixer == B200_MIX_LATENT) {
      const b200_latent_desc& q = L.lat;
      B200_CHECK_ARG(q.kv_rank > 0 && q.kv_rank <= kLatentMaxRank && q.rot_dim >= 0 && q.rot_dims >= 0 && q.rot_dims <= q.rot_dim &&
                         q.rot_dims % 2 == 0,
                     "engine_create_stack: layer %d: latent sizes (kv_rank 1 … %d, even rot_dims <= rot_dim)", l, kLatentMaxRank);
      B200_CHECK_ARG(q.c_norm && q.uk_t && q.uv && (q.rot_dims == 0 || q.rot_table), "engine_create_stack: layer %d: null latent weight", l);
      B200_CHECK_ARG(L.off_q >= 0 && L.off_q + (q.q_rank > 0 ? q.q_rank : a.heads * (a.dim + q.rot_dim)) <= L.n_in && L.off_k >= 0 &&
                         L.off_k + q.kv_rank + q.rot_dim <= L.n_in && (!q.out_gate || L.off_g + a.heads * a.vdim <= L.n_in),
                     "engine_create_stack: layer %d: segment offsets do not fit", l);
      B200_CHECK_ARG(q.q_rank >= 0 && (q.q_rank == 0 || (q.q_norm && q.uq)) && a.window >= 0,
                     "engine_create_stack: layer %d: query latent without its norm or up-projection", l);
      if (q.q_rank > 0) {
        s->rec_lr_max = std::max(s->rec_lr_max, up8i(q.q_rank));
        s->latq_max = std::max(s->latq_max, a.heads * (a.dim + q.rot_dim));
      }
      s->qa_max = std::max(s->qa_max, a.heads * (q.kv_rank + q.rot_dim));
      s->ol_max = std::max(s->ol_max, a.heads * q.kv_rank);
      s->lat_heads_max = std::max(s->lat_heads_max, a.heads);
      s->lat_rank_max = std::max(s->lat_rank_max, q.kv_rank);
      s->lat_hd_max = std::max(s->lat_hd_max, a.heads * (a.dim + q.rot_dim));
      s->lat_hv_max = std::max(s->lat_hv_max, a.heads * a.vdim);
    } else {
      B200_CHECK_ARG(L.mixer == B200_MIX_MLSTM, "engine_create_stack: layer %d: mixer kind %d", l, L.mixer);
      B200_CHECK_ARG(a.dim <= kMlstmMaxDim && L.rec.gate_cap > 0.f && L.rec.head_norm, "engine_create_stack: layer %d: mLSTM description", l);
      B200_CHECK_ARG(L.off_q >= 0 && L.off_q + a.heads * a.dim <= L.n_in && L.off_k + a.heads * a.dim <= L.n_in &&
                         L.off_v + a.heads * a.vdim <= L.n_in && L.off_g + a.heads * a.vdim <= L.n_in &&
                         L.off_gate + 2 * a.heads <= L.n_in,
                     "engine_create_stack: layer %d: segment offsets do not fit", l);
      s->rec_o_max = std::max(s->rec_o_max, a.heads * (a.vdim + 2));
      s->any_rec = s->recurrent = true;
    }
    int ff_rows = 0, ff_mid = 0;
    if (L.ff_kind == B200_FF_DENSE) {
      B200_CHECK_ARG(L.ff >= 0 && (L.ff == 0 || ((L.ff_norm || d.block == B200_BLOCK_POSTNORM) && L.ff_post_norm && L.w_ff_in && L.w_ff_out)),
                     "engine_create_stack: layer %d: dense feed-forward", l);
      B200_CHECK_ARG(L.ff_act >= B200_ACT_GELU_TANH && L.ff_act <= B200_ACT_TANH, "engine_create_stack: layer %d: activation %d", l,
                     L.ff_act);
      ff_rows = ff_mid = L.ff;
    } else {
      const b200_moe_desc& m = L.moe;
      B200_CHECK_ARG(L.ff_kind == B200_FF_MOE, "engine_create_stack: layer %d: feed-forward kind %d is not built for sandwich blocks", l, L.ff_kind);
      B200_CHECK_ARG(m.experts > 0 && m.top > 0 && m.top <= m.experts && m.expert_ff > 0 && m.shared_ff >= 0 && m.router &&
                         m.w_exp_in && m.w_exp_out && (L.ff_norm || d.block == B200_BLOCK_POSTNORM) && L.ff_post_norm &&
                         (m.shared_ff == 0 || (L.w_ff_in && L.w_ff_out)),
                     "engine_create_stack: layer %d: mixture-of-experts description", l);
      B200_CHECK_ARG((m.router_kind == 0 || m.router_kind == 1) && m.expert_act >= 0 && m.expert_act <= B200_ACT_TANH &&
                         (m.expert_act == 0 || m.shared_ff == 0 || m.shared_plain),
                     "engine_create_stack: layer %d: router kind %d / expert activation %d (a plain activation takes a plain shared expert)",
                     l, m.router_kind, m.expert_act);
      s->any_moe = true;
      s->moe_e_max = std::max(s->moe_e_max, m.experts);
      s->moe_top_max = std::max(s->moe_top_max, m.top);
      s->moe_ff_max = std::max(s->moe_ff_max, m.expert_ff);
      ff_rows = m.shared_ff > 0 ? (m.expert_act != 0 ? up8i(m.shared_ff) : up8i(2 * m.shared_ff + 1)) : 0;
      ff_mid = m.shared_ff;
    }
    s->max_heads = std::max(s->max_heads, a.heads);
    s->n_in_max = std::max(s->n_in_max, std::max(L.n_in, ff_rows));
    s->k_out_max = std::max(s->k_out_max, std::max(L.k_out, ff_mid));
    s->lin_max = std::max(s->lin_max, std::max(W, std::max(L.n_in, ff_rows)));
  }
  for (int l = 0; !sandwich && l < d.n_layers; ++l) {
    const b200_stack_layer& L = s->layers[l];
    const b200_attn_desc& a = L.attn;
    B200_CHECK_ARG(L.mixer == B200_MIX_ATTENTION && L.ff_kind == B200_FF_GATED,
                   "engine_create_stack: layer %d: parallel blocks are built for attention mixers and gated feed-forwards", l);
    B200_CHECK_ARG(a.heads > 0 && a.kv_heads > 0 && a.heads % a.kv_heads == 0 && a.dim > 0 && a.vdim > 0 && a.window >= 0 &&
                       a.keep_first >= 0,
                   "engine_create_stack: layer %d: bad attention sizes", l);
    B200_CHECK_ARG(a.vdim <= 256 && a.dim <= 1024, "engine_create_stack: layer %d: head sizes above 1024 / 256 not built", l);
    B200_CHECK_ARG(L.norm && L.w_in && L.w_out && L.n_in > 0 && L.k_out > 0 && L.ff >= 0, "engine_create_stack: layer %d: null weight", l);
    B200_CHECK_ARG(L.off_q >= 0 && L.off_q + a.heads * a.dim <= L.n_in && L.off_k + a.kv_heads * a.dim <= L.n_in &&
                       L.off_v + a.kv_heads * a.vdim <= L.n_in && (!a.out_gate || L.off_g + a.heads <= L.n_in) &&
                       (L.ff == 0 || (L.off_gate + L.ff <= L.n_in && L.off_up + L.ff <= L.n_in)) &&
                       a.heads * a.vdim <= L.off_act && L.off_act + L.ff <= L.k_out,
                   "engine_create_stack: layer %d: segment offsets do not fit", l);
    B200_CHECK_ARG(L.side_gate == nullptr || (L.side_proj && L.side_norm && d.side_table && d.side_dim > 0 &&
                                              L.side_col + d.side_dim <= d.side_stride),
                   "engine_create_stack: layer %d: incomplete side input", l);
    s->max_heads = std::max(s->max_heads, a.heads);
    s->max_vdim = std::max(s->max_vdim, a.vdim);
    s->n_in_max = std::max(s->n_in_max, std::max(L.n_in, d.side_dim));
    s->k_out_max = std::max(s->k_out_max, L.k_out);
  }
  s->run_k_off.resize(d.n_runs);
  s->run_v_off.resize(d.n_runs);
  s->run_s_off.resize(d.n_runs);
  s->run_kv_shared.assign(d.n_runs, 0);
  for (int r = 0; r < d.n_runs; ++r) {
    B200_CHECK_ARG(s->run_layer[r] >= 0 && s->run_layer[r] < d.n_layers, "engine_create_stack: run %d names layer %d", r,
                   s->run_layer[r]);
    B200_CHECK_ARG(!s->run_mix[r] || d.mix_in, "engine_create_stack: run %d mixes the embedding in but mix_in is null", r);
    const b200_stack_layer& RL = s->layers[s->run_layer[r]];
    const b200_attn_desc& a = RL.attn;
    s->run_k_off[r] = s->k_slot;
    s->run_v_off[r] = s->v_slot;
    s->run_s_off[r] = s->s_slot;
    if (RL.mixer == B200_MIX_ATTENTION && sandwich && RL.kv_share > 0) {
      // the cache of the latest earlier run of the source layer (the pass of a loop this run belongs to, or the last one)
      int src = -1;
      for (int q = 0; q < r; ++q)
        if (s->run_layer[q] == RL.kv_share - 1) src = q;
      B200_CHECK_ARG(src >= 0, "engine_create_stack: run %d reads the keys and values of layer %d, which has not run before it", r,
                     RL.kv_share - 1);
      s->run_k_off[r] = s->run_k_off[src];
      s->run_v_off[r] = s->run_v_off[src];
      s->run_kv_shared[r] = 1;
    } else if (RL.mixer == B200_MIX_ATTENTION) {
      s->k_slot += (size_t)d.max_ctx * a.kv_heads * a.dim;
      s->v_slot += (size_t)d.max_ctx * a.kv_heads * a.vdim;
    } else if (RL.mixer == B200_MIX_GATED_DELTA) {   // a fixed-size state and the convolutions' last inputs
      s->s_slot += (size_t)gdelta_state_floats(a.heads, a.kv_heads, a.dim, a.vdim, RL.gdelta.taps);
    } else if (RL.mixer == B200_MIX_LATENT) {   // one row per position: [latent | rotated shared key part]
      s->k_slot += (size_t)d.max_ctx * (RL.lat.kv_rank + RL.lat.rot_dim);
    } else if (RL.mixer == B200_MIX_DELTA) {    // no rows per position: a fixed-size state
      s->s_slot += (size_t)a.heads * a.dim * a.vdim;
    } else if (RL.mixer == B200_MIX_MAMBA2) {
      s->s_slot += (size_t)mamba_state_floats(a.heads, a.vdim, RL.mamba.state, RL.mamba.groups, RL.mamba.taps);
    } else {
      s->s_slot += (size_t)mlstm_state_floats(a.heads, a.dim, a.vdim);
    }
  }
  B200_CUDA(cudaDeviceSynchronize());   // weights may still be in flight on the loader's stream
  {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_CUDA(cudaDeviceGetAttribute(&s->num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  s->plans.resize(d.n_layers);
  s->splans.resize(d.n_layers);
  s->fast = d.dtype == B200_BF16 && !env_flag("B200_STACK_PLAIN", false);
  if (s->fast) {
    if ((rc = gemv_setup_attributes()) != B200_OK || (rc = gemv_batch_setup_attributes()) != B200_OK) return rc;
    // a plan that cannot be made (k not a multiple of 8, an unaligned matrix) leaves that product on the general kernel
    auto plan = [&](GemvPlan* pl, const void* w, int64_t n, int64_t k, int epi, int pro = PRO_PLAIN) {
      if (k % 8 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return false;
      return gemv_make_plan(pl, w, n, n, k, 1, pro, epi, s->num_sms) == B200_OK;
    };
    for (int l = 0; !sandwich && l < d.n_layers; ++l) {
      const b200_stack_layer& L = s->layers[l];
      s->plans[l].ok_in = plan(&s->plans[l].in, L.w_in, L.n_in, d.width, EPI_BIAS_F32, PRO_F32);
      s->plans[l].ok_out = plan(&s->plans[l].out, L.w_out, d.width, L.k_out, EPI_RESID_F32);
      s->plans[l].ok_side = L.side_gate != nullptr &&
                            plan(&s->plans[l].side_gate, L.side_gate, d.side_dim, d.width, EPI_ACT_TABLE, PRO_F32) &&
                            plan(&s->plans[l].side_proj, L.side_proj, d.width, d.side_dim, EPI_BIAS_F32);
    }
    for (int l = 0; sandwich && l < d.n_layers; ++l) {
      const b200_stack_layer& L = s->layers[l];
      StackEngine::SPlans& sp = s->splans[l];
      s->plans[l].ok_in = s->plans[l].ok_out = s->plans[l].ok_side = false;
      sp.ok_in = plan(&sp.in, L.w_in, L.n_in, d.width, EPI_BIAS_F32);
      sp.ok_out = plan(&sp.out, L.w_out, d.width, L.k_out, EPI_BIAS_F32);
      if (L.mixer == B200_MIX_DELTA)
        sp.ok_lora = plan(&sp.lora, L.delta.w2, (int64_t)L.attn.heads * L.attn.dim, up8i(L.delta.rank), EPI_BIAS_F32);
      if (L.mixer == B200_MIX_LATENT && L.lat.q_rank > 0)
        sp.ok_uq = plan(&sp.uq, L.lat.uq, (int64_t)L.attn.heads * (L.attn.dim + L.lat.rot_dim), up8i(L.lat.q_rank), EPI_BIAS_F32);
      if (L.ff_kind == B200_FF_DENSE && L.ff > 0) {
        sp.ok_ff_in = plan(&sp.ff_in, L.w_ff_in, L.ff, d.width, EPI_BIAS_F32);
        sp.ok_ff_out = plan(&sp.ff_out, L.w_ff_out, d.width, L.ff, EPI_BIAS_F32);
      } else if (L.ff_kind == B200_FF_MOE && L.moe.shared_ff > 0) {
        sp.ok_ff_in = plan(&sp.ff_in, L.w_ff_in, L.moe.expert_act != 0 ? up8i(L.moe.shared_ff) : up8i(2 * L.moe.shared_ff + 1),
                           d.width, EPI_BIAS_F32);
        sp.ok_ff_out = plan(&sp.ff_out, L.w_ff_out, d.width, L.moe.shared_ff, EPI_BIAS_F32);
      }
    }
    if (d.mix_in) s->ok_mix = plan(&s->p_mix, d.mix_in, d.width, 2 * (int64_t)d.width, EPI_RESID_F32);
    s->ok_head = plan(&s->p_head, d.head, d.vocab, d.width, EPI_BIAS_F32) &&
                 plan(&s->p_head_f, d.head, d.vocab, d.width, EPI_BIAS_F32, PRO_F32);
  }
  const size_t kb = align_up(s->k_slot * d.max_slots * s->esz, 256), vb = align_up(s->v_slot * d.max_slots * s->esz, 256);
  B200_CUDA(cudaMalloc((void**)&s->cache, std::max<size_t>(kb + vb, 256)));
  s->kbase = s->cache;
  s->vbase = s->cache + kb;
  if (s->s_slot > 0) {
    B200_CUDA(cudaMalloc((void**)&s->rstate, s->s_slot * d.max_slots * 4));
    B200_CUDA(cudaMemset(s->rstate, 0, s->s_slot * d.max_slots * 4));
  }
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  const size_t n = d.max_slots;
  const size_t o_pos = take(n * 4), o_tok = take(n * 8), o_log = take(n * s->gen_cap * 8), o_cnt = take(n * 8);
  const size_t o_rs = take(n * 4), o_amax = take((size_t)argmax_workspace_bytes((int64_t)n, d.vocab) + n * 8 + 16);
  const size_t o_smp = take((size_t)sample_workspace_bytes());
  B200_CUDA(cudaMalloc((void**)&s->state, off));
  B200_CUDA(cudaMemset(s->state, 0, off));
  s->pos_dev = (int*)(s->state + o_pos);
  s->cur_tok = (int64_t*)(s->state + o_tok);
  s->gen_log = (int64_t*)(s->state + o_log);
  s->gen_count = (unsigned long long*)(s->state + o_cnt);
  s->row_slot = (int*)(s->state + o_rs);
  s->argmax_ws = s->state + o_amax;
  s->amax_out = (int64_t*)((uint8_t*)s->argmax_ws + argmax_workspace_bytes((int64_t)n, d.vocab));
  s->sample_ws = s->state + o_smp;
  s->h_pos.assign(n, 0);
  s->h_gen.assign(n, 0);
  e->d.vocab = d.vocab;
  e->d.hidden = d.width;
  e->d.max_ctx = d.max_ctx;
  e->d.layers = d.n_layers;
  e->V_l = d.vocab;
  e->use_graph = !env_flag("B200_NO_GRAPH", false);
  s->pdl = !env_flag("B200_NO_PDL", false);
  e->use_pdl = s->pdl;
  guard.e = nullptr;
  *out = e;
  return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_engine_create_stack(const b200_stack_desc* desc, b200_engine** out) { return b200::stack_build(desc, out); }

int b200_engine_step(b200_engine* e, int64_t n_seq, const int32_t* slots, const int32_t* counts, const int64_t* ids,
                     int64_t n_want, const int32_t* want, float* logits_out, int greedy, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(e && slots && counts && ids && n_seq >= 1, "engine_step: null argument");
  if (!e->stack) {
    set_error("engine_step: ragged steps over sequence slots are built for stack engines; Llama-family engines take "
              "b200_engine_forward");
    return B200_ERR_UNSUPPORTED;
  }
  B200_CHECK_ARG(n_want == 0 || (want && logits_out), "engine_step: wanted rows without an output buffer");
  StackEngine* s = e->stack;
  const b200_stack_desc& d = s->d;
  cudaStream_t st = (cudaStream_t)stream;
  int64_t total = 0;
  std::vector<char> seen(d.max_slots, 0);
  for (int64_t i = 0; i < n_seq; ++i) {
    B200_CHECK_ARG(slots[i] >= 0 && slots[i] < d.max_slots && !seen[slots[i]], "engine_step: bad or repeated slot %d", slots[i]);
    seen[slots[i]] = 1;
    B200_CHECK_ARG(counts[i] >= 1, "engine_step: sequence %lld brings no token", (long long)i);
    if (s->h_pos[slots[i]] + counts[i] > d.max_ctx) {
      set_error("engine_step: slot %d: position %lld + %d tokens exceeds max_ctx %d", slots[i], (long long)s->h_pos[slots[i]],
                counts[i], d.max_ctx);
      return B200_ERR_STATE;
    }
    total += counts[i];
  }
  for (int64_t i = 0; i < n_want; ++i)
    B200_CHECK_ARG(want[i] >= 0 && want[i] < total, "engine_step: wanted row %d outside the step's %lld tokens", want[i],
                   (long long)total);
  // the row list on the host: token, slot, position
  std::vector<int32_t> tok(total), slot(total), pos(total), last(n_seq);
  {
    int64_t t = 0;
    for (int64_t i = 0; i < n_seq; ++i) {
      for (int c = 0; c < counts[i]; ++c, ++t) {
        tok[t] = (int32_t)ids[t];
        slot[t] = slots[i];
        pos[t] = (int32_t)s->h_pos[slots[i]] + c;
      }
      last[i] = (int32_t)t - 1;
    }
  }
  const int chunk = kStackChunk;
  int rc;
  const int ws_tok = (int)std::min<int64_t>(total, chunk);
  if ((rc = stack_workspace(s, ws_tok, (int)std::min<int64_t>(n_want + (greedy ? n_seq : 0), (int64_t)ws_tok + n_seq) + 1)) != B200_OK)
    return rc;
  std::vector<int> act_slots(slots, slots + n_seq);
  if (greedy && (rc = stack_set_active(s, act_slots, st)) != B200_OK) return rc;
  const size_t vb4 = (size_t)d.vocab * 4;
  std::vector<int32_t> meta;
  for (int64_t c0 = 0; c0 < total; c0 += chunk) {
    const int n_tok = (int)std::min<int64_t>(chunk, total - c0);
    // wanted rows of this chunk (in the caller's order), then — on the last chunk of a greedy step — the last rows
    std::vector<int32_t> rows;
    std::vector<int64_t> dest;
    for (int64_t i = 0; i < n_want; ++i)
      if (want[i] >= c0 && want[i] < c0 + n_tok) {
        rows.push_back((int32_t)(want[i] - c0));
        dest.push_back(i);
      }
    const int n_user = (int)rows.size();
    const bool tail = c0 + n_tok == total;
    if (greedy && tail) {
      // a sequence whose last token fell into an earlier chunk cannot happen: chunks follow the row order and the
      // last rows of all sequences but the final one may lie before c0 — those are recomputed from the cache
      for (int64_t i = 0; i < n_seq; ++i) B200_CHECK_ARG(last[i] >= c0, "engine_step: greedy steps take at most %d tokens", chunk);
      for (int64_t i = 0; i < n_seq; ++i) rows.push_back((int32_t)(last[i] - c0));
    }
    const int n_rows = (int)rows.size();
    if ((rc = stack_workspace(s, n_tok, std::max(1, n_rows))) != B200_OK) return rc;
    meta.assign(tok.begin() + c0, tok.begin() + c0 + n_tok);
    B200_CUDA(cudaMemcpyAsync(s->m_tok, meta.data(), (size_t)n_tok * 4, cudaMemcpyHostToDevice, st));
    B200_CUDA(cudaMemcpyAsync(s->m_slot, slot.data() + c0, (size_t)n_tok * 4, cudaMemcpyHostToDevice, st));
    B200_CUDA(cudaMemcpyAsync(s->m_pos, pos.data() + c0, (size_t)n_tok * 4, cudaMemcpyHostToDevice, st));
    if (n_rows > 0) B200_CUDA(cudaMemcpyAsync(s->m_want, rows.data(), (size_t)n_rows * 4, cudaMemcpyHostToDevice, st));
    s->segs.clear();
    for (int t = 0; t < n_tok; ++t) {
      const int64_t gi = c0 + t;
      if (t == 0 || slot[gi] != slot[gi - 1]) s->segs.push_back({t, 1, slot[gi], pos[gi]});
      else s->segs.back().count += 1;
    }
    if ((rc = stack_pass(e, n_tok, n_rows, st)) != B200_OK) return rc;
    for (int r = 0; r < n_user;) {   // runs of consecutive destination rows leave in one copy
      int r1 = r + 1;
      while (r1 < n_user && dest[r1] == dest[r1 - 1] + 1) ++r1;
      B200_CUDA(cudaMemcpyAsync((uint8_t*)logits_out + (size_t)dest[r] * vb4, (uint8_t*)s->logits + (size_t)r * vb4,
                                (size_t)(r1 - r) * vb4, cudaMemcpyDeviceToDevice, st));
      r = r1;
    }
    if (greedy && tail) {
      stack_count_generated(s, act_slots, 1);
      if ((rc = stack_publish(e, n_user, act_slots, st)) != B200_OK) return rc;
    }
  }
  std::vector<int32_t> upd;
  for (int64_t i = 0; i < n_seq; ++i) {
    s->h_pos[slots[i]] += counts[i];
    upd.push_back(slots[i]);
    upd.push_back((int32_t)s->h_pos[slots[i]]);
  }
  e->h_pos = s->h_pos[slots[0]];
  if (greedy) e->batch = (int)n_seq;
  return stack_push_positions(s, upd, st);
}

int b200_engine_slot_reset(b200_engine* e, int64_t slot, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(e && e->stack, "engine_slot_reset: not a stack engine");
  StackEngine* s = e->stack;
  B200_CHECK_ARG(slot >= 0 && slot < s->d.max_slots, "engine_slot_reset: slot %lld of %d", (long long)slot, s->d.max_slots);
  int rc = stack_workspace(s, 1, 1);
  if (rc != B200_OK) return rc;
  s->h_pos[slot] = 0;
  auto it = std::find(s->active.begin(), s->active.end(), (int)slot);
  if (it != s->active.end()) {   // the sequence leaves the active batch; the others go on
    std::vector<int> rest = s->active;
    rest.erase(rest.begin() + (it - s->active.begin()));
    s->active.clear();
    if (!rest.empty() && (rc = stack_set_active(s, rest, (cudaStream_t)stream)) != B200_OK) return rc;
  }
  return stack_push_positions(s, {(int32_t)slot, 0}, (cudaStream_t)stream);
}

int64_t b200_engine_slot_position(const b200_engine* e, int64_t slot) {
  if (!e || !e->stack || slot < 0 || slot >= e->stack->d.max_slots) return -1;
  return e->stack->h_pos[slot];
}

int64_t b200_engine_max_slots(const b200_engine* e) {
  if (!e) return -1;
  return e->stack ? e->stack->d.max_slots : b200::kMaxBatch;
}

}  // extern "C"
