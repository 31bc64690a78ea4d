// api.cu — C-ABI entry points for the GEMV and the fused building blocks (declared in include/b200_decode.h).
#include "gemv.cuh"
#include "stack_mix.cuh"
#include "stack_rec.cuh"
#include <vector>
#include "ops.cuh"
#include "stack.cuh"

namespace b200 {

static int num_sms_cached() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) !=
                                                  cudaSuccess) {
      (void)cudaGetLastError();
      sms = 0;
      return 148;
    }
  }
  return sms;
}

}  // namespace b200

extern "C" {

int b200_gemv_bf16(void* y, const void* x, const void* W, const void* bias, int64_t m, int64_t n, int64_t k,
                   void* stream) {
  using namespace b200;
  B200_CHECK_ARG(y && x && W, "gemv: null pointer");
  B200_CHECK_ARG(m >= 1 && m <= 4096, "gemv: m=%lld out of range (this entry point is the decode GEMV)", (long long)m);
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  if ((rc = gemv_setup_attributes()) != B200_OK) return rc;
  GemvPlan plan;
  if ((rc = gemv_make_plan(&plan, W, n, n, k, 1, PRO_PLAIN, EPI_PLAIN, num_sms_cached())) != B200_OK) return rc;
  plan.p.bias = (const __nv_bfloat16*)bias;
  for (int64_t r = 0; r < m; ++r) {  // W is re-streamed per row of x; the batched path is the prefill GEMM
    plan.p.x = (const __nv_bfloat16*)x + r * k;
    plan.p.y = (__nv_bfloat16*)y + r * n;
    if ((rc = gemv_launch(plan, (cudaStream_t)stream, false)) != B200_OK) return rc;
  }
  return B200_OK;
}

int b200_gemv_fused_bf16(void* y, const void* x, const void* W, int64_t n, int64_t k, int nseg, const void* norm_w,
                         float eps, const void* bias, const void* residual, int silu_mul, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(y && x && W, "gemv_fused: null pointer");
  B200_CHECK_ARG(!(silu_mul && (bias || residual)), "gemv_fused: silu_mul excludes bias/residual");
  B200_CHECK_ARG(!(bias && residual), "gemv_fused: bias and residual are exclusive");
  B200_CHECK_ARG((nseg == 2) == (silu_mul != 0), "gemv_fused: nseg == 2 exactly when silu_mul");
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  if ((rc = gemv_setup_attributes()) != B200_OK) return rc;
  GemvPlan plan;
  const int pro = norm_w ? PRO_RMSNORM : PRO_PLAIN;
  const int epi = silu_mul ? EPI_SILU_MUL : (residual ? EPI_RESIDUAL : EPI_PLAIN);
  if (pro == PRO_RMSNORM && epi == EPI_RESIDUAL) {
    set_error("gemv_fused: RMSNorm prologue with residual epilogue is not a combination of the decode path");
    return B200_ERR_UNSUPPORTED;
  }
  if ((rc = gemv_make_plan(&plan, W, n * nseg, n, k, nseg, pro, epi, num_sms_cached())) != B200_OK) return rc;
  plan.p.x = (const __nv_bfloat16*)x;
  plan.p.norm_w = (const __nv_bfloat16*)norm_w;
  plan.p.eps = eps;
  plan.p.bias = (const __nv_bfloat16*)bias;
  plan.p.residual = (const __nv_bfloat16*)residual;
  plan.p.y = (__nv_bfloat16*)y;
  return gemv_launch(plan, (cudaStream_t)stream, false);
}

int64_t b200_attn_decode_workspace_bytes(int64_t Hq, int64_t Hkv, int64_t hd, int64_t max_ctx) {
  if (Hkv <= 0 || Hq % Hkv != 0 || (hd != 64 && hd != 128) || max_ctx < 1) return -1;
  const int nsplit = b200::attn_decode_nsplit((int)hd, (int)max_ctx);
  return b200::attn_decode_ws_floats((int)Hq, (int)Hkv, (int)hd, nsplit) * 4 + ((Hq * 4 + 15) / 16) * 16;
}

int b200_attn_decode_bf16(void* out, const void* qkv, const void* q_norm, const void* k_norm, float eps,
                          const float* rope_table, const int32_t* pos, int64_t fixed_len, void* kcache, void* vcache,
                          int64_t Hq, int64_t Hkv, int64_t hd, int64_t max_ctx, void* workspace, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(out && qkv && kcache && vcache && workspace, "attn_decode: null pointer");
  B200_CHECK_ARG(pos != nullptr || (fixed_len >= 1 && fixed_len <= max_ctx), "attn_decode: fixed_len out of range");
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  if ((rc = attn_setup_attributes()) != B200_OK) return rc;
  AttnDecodeParams a{};
  a.qkv = (const __nv_bfloat16*)qkv;
  a.q_norm = (const __nv_bfloat16*)q_norm;
  a.k_norm = (const __nv_bfloat16*)k_norm;
  a.eps = eps;
  a.rope = rope_table;
  a.pos = pos;
  a.fixed_len = (int)fixed_len;
  a.kcache = (__nv_bfloat16*)kcache;
  a.vcache = (__nv_bfloat16*)vcache;
  a.out = (__nv_bfloat16*)out;
  a.tickets = (unsigned int*)workspace;
  a.ws = (float*)((uint8_t*)workspace + ((Hq * 4 + 15) / 16) * 16);
  a.Hq = (int)Hq;
  a.Hkv = (int)Hkv;
  a.nsplit = attn_decode_nsplit((int)hd, (int)max_ctx);
  a.max_ctx = (int)max_ctx;
  return launch_attn_decode(a, (int)hd, (cudaStream_t)stream, false);
}

}  // extern "C"

// ---- the stack engine's mechanisms as stand-alone ops
extern "C" {

int b200_stack_rmsnorm(void* y, const float* x, const float* w, int64_t rows, int64_t dim, float eps, float offset,
                       int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(dim > 0 && dim < (1ll << 31) && rows < (1ll << 31), "stack_rmsnorm: size out of range");
  return b200::launch_stack_rmsnorm(y, x, w, nullptr, rows, (int)dim, eps, offset, dtype, (cudaStream_t)stream);
}

int b200_stack_linear(void* C, const void* A, const void* W, const float* bias, int64_t M, int64_t N, int64_t K, int dtype,
                      void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(M > 0 && N > 0 && K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
                 "stack_linear: size out of range");
  b200::StackGemm g;
  g.a = A; g.lda = K; g.k1 = (int)K;
  g.w = W; g.bias = bias; g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.epi = b200::SEPI_STORE; g.c = C; g.ldc = N;
  return b200::launch_stack_gemm(g, dtype, (cudaStream_t)stream);
}

static b200::StackAttn stack_attn_args(const void* proj, int64_t ld_proj, const void* kcache, const void* vcache,
                                       int64_t k_slot_stride, int64_t v_slot_stride, const int32_t* slot,
                                       const int32_t* pos, int64_t n_tok, const b200_attn_desc* attn) {
  b200::StackAttn p;
  if (attn) p.a = *attn;
  p.proj = proj; p.ld_proj = ld_proj;
  p.kcache = const_cast<void*>(kcache); p.vcache = const_cast<void*>(vcache);
  p.k_slot_stride = k_slot_stride; p.v_slot_stride = v_slot_stride;
  p.slot = slot; p.pos = pos; p.n_tok = (int)n_tok;
  return p;
}

int b200_stack_attention(void* out, int64_t ld_out, const void* proj, int64_t ld_proj, int64_t off_q, int64_t off_g,
                         const void* kcache, const void* vcache, int64_t k_slot_stride, int64_t v_slot_stride,
                         const int32_t* slot, const int32_t* pos, int64_t n_tok, const b200_attn_desc* attn, int dtype,
                         void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(attn && n_tok > 0 && n_tok < (1ll << 31), "stack_attention: bad arguments");
  b200::StackAttn p = stack_attn_args(proj, ld_proj, kcache, vcache, k_slot_stride, v_slot_stride, slot, pos, n_tok, attn);
  p.off_q = (int)off_q; p.off_g = (int)off_g;
  p.out = out; p.ld_out = ld_out;
  return b200::launch_stack_attention(p, dtype, (cudaStream_t)stream);
}

int b200_stack_kv_store(void* kcache, void* vcache, int64_t k_slot_stride, int64_t v_slot_stride, const void* proj,
                        int64_t ld_proj, int64_t off_k, int64_t off_v, const int32_t* slot, const int32_t* pos,
                        int64_t n_tok, const b200_attn_desc* attn, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(attn && n_tok > 0 && n_tok < (1ll << 31), "stack_kv_store: bad arguments");
  b200::StackAttn p = stack_attn_args(proj, ld_proj, kcache, vcache, k_slot_stride, v_slot_stride, slot, pos, n_tok, attn);
  p.off_k = (int)off_k; p.off_v = (int)off_v;
  return b200::launch_stack_kv_store(p, dtype, (cudaStream_t)stream);
}

int b200_stack_act_mul(void* y, int64_t ld_y, const void* g, const void* u, int64_t ld_gu, int64_t rows, int64_t n, int act,
                       int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(n > 0 && n < (1ll << 31), "stack_act_mul: size out of range");
  return b200::launch_stack_act_mul(y, ld_y, g, u, ld_gu, rows, (int)n, act, dtype, (cudaStream_t)stream);
}

int b200_stack_rms_add(float* x, const float* y, const float* w, int64_t rows, int64_t dim, float eps, float mult,
                       void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(dim > 0 && dim < (1ll << 31) && rows < (1ll << 31), "stack_rms_add: size out of range");
  return b200::launch_stack_rms_add(x, y, w, rows, (int)dim, eps, mult, (cudaStream_t)stream);
}

// ---- mechanisms of sandwich blocks (stack_mix.cu).  The ops that need scratch allocate it, run and synchronise.
namespace {
struct Scratch {
  std::vector<void*> ptrs;
  void* take(size_t bytes) {
    void* p = nullptr;
    if (cudaMalloc(&p, bytes > 0 ? bytes : 1) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, bytes > 0 ? bytes : 1);
    ptrs.push_back(p);
    return p;
  }
  ~Scratch() {
    cudaDeviceSynchronize();
    for (void* p : ptrs) cudaFree(p);
  }
};
}  // namespace

int b200_stack_norm(void* y, float* xadd, const float* x, const float* w, int64_t rows, int64_t dim, float eps, int kind,
                    int add, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(dim > 0 && dim < (1ll << 31) && rows > 0 && rows < (1ll << 31), "stack_norm: size out of range");
  if (add) return b200::launch_stack_norm_add(xadd, x, false, w, rows, (int)dim, eps, 1.f, kind, (cudaStream_t)stream);
  return b200::launch_stack_norm(y, x, w, nullptr, rows, (int)dim, eps, 0.f, kind, dtype, (cudaStream_t)stream);
}

int b200_stack_latent_attention(void* out, int64_t ld_out, const void* proj, int64_t ld_proj, int64_t off_down, void* cache,
                                int64_t slot_stride, const int32_t* slot, const int32_t* pos, int64_t n_tok,
                                const b200_attn_desc* attn, const b200_latent_desc* lat, float eps, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(attn && lat && n_tok > 0 && n_tok < (1 << 24), "stack_latent_attention: bad arguments");
  B200_CHECK_ARG(dtype == B200_BF16 || dtype == B200_F32, "stack_latent_attention: unknown dtype");
  const size_t esz = dtype == B200_F32 ? 4 : 2;
  Scratch sc;
  b200::LatentRun p;
  p.a = *attn; p.l = *lat; p.eps = eps;
  p.proj = proj; p.ld_proj = ld_proj; p.off_q = 0; p.off_down = (int)off_down;
  p.cache = cache; p.slot_stride = slot_stride; p.slot = slot; p.pos = pos; p.n_tok = (int)n_tok;
  p.qa = sc.take((size_t)n_tok * attn->heads * (lat->kv_rank + lat->rot_dim) * esz);
  p.ol = sc.take((size_t)n_tok * attn->heads * lat->kv_rank * esz);
  B200_CHECK_ARG(p.qa && p.ol, "stack_latent_attention: out of device memory");
  p.out = out; p.ld_out = ld_out;
  return b200::run_latent_attention(p, dtype, (cudaStream_t)stream);
}

int b200_stack_mlstm(float* out, const void* proj, int64_t ld_proj, int64_t off_q, int64_t off_k, int64_t off_v,
                     const float* gates, float* state, int64_t slot_stride, const int32_t* row0, const int32_t* count,
                     const int32_t* slot, const int32_t* pos, int64_t n_seq, int64_t n_rows, const b200_attn_desc* sizes,
                     float gate_cap, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(sizes && n_seq > 0 && n_rows >= n_seq && n_rows < (1 << 24), "stack_mlstm: bad arguments");
  b200::MlstmRun p;
  p.a = *sizes; p.gate_cap = gate_cap;
  p.proj = proj; p.ld_proj = ld_proj; p.off_q = (int)off_q; p.off_k = (int)off_k; p.off_v = (int)off_v;
  p.gates = gates; p.ld_gates = 2 * sizes->heads;
  p.state = state; p.slot_stride = slot_stride;
  p.seg_row0 = row0; p.seg_count = count; p.slot = slot; p.pos = pos; p.n_seg = (int)n_seq; p.n_tok = (int)n_rows;
  p.o = out;
  Scratch sc;
  p.gab = (float*)sc.take((size_t)n_rows * sizes->heads * 3 * 4);
  B200_CHECK_ARG(p.gab, "stack_mlstm: out of device memory");
  return b200::run_mlstm(p, dtype, (cudaStream_t)stream);
}

int64_t b200_stack_mlstm_state_floats(int64_t heads, int64_t dim, int64_t vdim) {
  return b200::mlstm_state_floats((int)heads, (int)dim, (int)vdim);
}

int b200_stack_moe(float* y, const void* h, int64_t rows, int64_t width, const b200_moe_desc* moe, int32_t* chosen,
                   float* scores, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(moe && rows > 0 && rows < (1 << 22) && width > 0 && width < (1 << 24) && moe->top > 0 && moe->experts > 0,
                 "stack_moe: bad arguments");
  B200_CHECK_ARG(dtype == B200_BF16 || dtype == B200_F32, "stack_moe: unknown dtype");
  const size_t esz = dtype == B200_F32 ? 4 : 2, P = (size_t)rows * moe->top;
  Scratch sc;
  b200::MoeRun p;
  p.m = *moe; p.width = (int)width; p.n_tok = (int)rows; p.h = h; p.y = y;
  p.z = (float*)sc.take((size_t)rows * moe->experts * 4);
  p.sel_e = (int32_t*)sc.take(P * 4);
  p.sel_w = (float*)sc.take(P * 4);
  p.plan = (int32_t*)sc.take((size_t)b200::moe_plan_ints((int)P, moe->experts) * 4);
  p.pair_slot = (int32_t*)sc.take(P * 4);
  p.a_perm = sc.take(P * width * esz);
  p.gu = sc.take(P * 2 * moe->expert_ff * esz);
  p.act = sc.take(P * moe->expert_ff * esz);
  p.outp = (float*)sc.take(P * width * 4);
  B200_CHECK_ARG(p.z && p.sel_e && p.sel_w && p.plan && p.pair_slot && p.a_perm && p.gu && p.act && p.outp,
                 "stack_moe: out of device memory");
  if ((rc = b200::run_moe(p, dtype, (cudaStream_t)stream)) != B200_OK) return rc;
  if (chosen) B200_CUDA(cudaMemcpyAsync(chosen, p.sel_e, P * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  if (scores) B200_CUDA(cudaMemcpyAsync(scores, p.sel_w, P * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return B200_OK;
}

int b200_stack_lin_scan(float* out, const float* d, const float* p, const float* q, const float* b, const float* r, const float* v,
                        const float* vscale, int64_t ld, int64_t heads, int64_t dk, int64_t dv, int64_t share, int64_t d_scalar,
                        float* state, int64_t slot_stride, const int32_t* row0, const int32_t* count, const int32_t* slot,
                        const int32_t* pos, int64_t n_seq, int64_t n_rows, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(n_seq > 0 && n_rows >= n_seq && n_rows < (1 << 24) && heads > 0 && heads < (1 << 16) && dk > 0 && dv > 0 &&
                     dv < (1 << 20),
                 "stack_lin_scan: bad arguments");
  b200::LinScan s;
  s.heads = (int)heads; s.dk = (int)dk; s.dv = (int)dv; s.share = (int)share; s.d_scalar = (int)d_scalar;
  s.d = d; s.p = p; s.q = q; s.b = b; s.r = r; s.v = v; s.vscale = vscale; s.ld = ld;
  s.state = state; s.slot_stride = slot_stride;
  s.seg_row0 = row0; s.seg_count = count; s.slot = slot; s.pos = pos; s.n_seg = (int)n_seq; s.n_tok = (int)n_rows;
  s.o = out; s.ld_o = heads * dv;
  return b200::launch_lin_scan(s, (cudaStream_t)stream);
}

int b200_stack_attn_prep(void* proj, int64_t ld_proj, int64_t off_q, int64_t off_k, int64_t off_v, const int32_t* pos,
                         int64_t n_tok, const b200_attn_desc* attn, const b200_attn_prep_desc* prep, void* vkeep,
                         int64_t ld_keep, float eps, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(attn && prep && n_tok > 0 && n_tok < (1 << 24), "stack_attn_prep: bad arguments");
  b200::AttnPrep a;
  a.a = *attn; a.d = *prep; a.eps = eps;
  a.proj = proj; a.ld_proj = ld_proj; a.off_q = (int)off_q; a.off_k = (int)off_k; a.off_v = (int)off_v;
  a.pos = pos; a.n_tok = (int)n_tok; a.vkeep = vkeep; a.ld_keep = ld_keep;
  return b200::launch_attn_prep(a, dtype, (cudaStream_t)stream);
}

int b200_stack_glu_clamp(void* y, const void* gu, int64_t rows, int64_t n, float limit, int dtype, void* stream) {
  int rc = b200_device_check();
  if (rc != B200_OK) return rc;
  B200_CHECK_ARG(n > 0 && n < (1ll << 30) && rows > 0, "stack_glu_clamp: size out of range");
  return b200::launch_stack_glu_clamp(y, n, gu, 2 * n, rows, (int)n, limit, dtype, (cudaStream_t)stream);
}

}  // extern "C"
