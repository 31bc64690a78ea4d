/*
 * b200_decode.h — C ABI of the B200-native decode engine that sits behind TinyGPT's
 * GPTEngine::generate*() loop and TinyTorch's operator registry.
 *
 * Conventions (see INTEGRATION.md for the TinyTorch-side adapter):
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - bf16 is raw 16-bit storage (same bits as tinytorch::BFloat16 / __nv_bfloat16), row-major contiguous;
 *   - the caller passes its own cudaStream_t (TinyTorch: cuda::getCurrentCUDAStream(dev).stream(),
 *     third_party/TinyTorch/src/Utils/CUDAUtils.cpp:123-135) as an opaque void*;
 *   - every function returns 0 on success and a negative b200_status on failure, never throws,
 *     never synchronises the device, and (op level) never allocates; the message of the last failure on the calling
 *     thread is available from b200_last_error().  The reference's own convention is LOGE + ASSERT
 *     (third_party/TinyTorch/src/Utils/Macros.h:34-40); the adapter maps non-zero to that.
 *   - there is NO CPU fallback: on a machine without an sm_100 device every compute entry point fails with
 *     B200_ERR_NO_DEVICE.
 *
 * Reference interface each entry point replaces is cited as  [ref: file:line]  with paths relative to the
 * keith2018/TinyGPT checkout (TT/ = third_party/TinyTorch/src/).
 */
#ifndef B200_DECODE_H_
#define B200_DECODE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with -fvisibility=hidden; these are its only exports */
#endif

/* 2: + b200_engine_set_mailbox, b200_engine_generated;  3: + b200_sample_bf16, b200_sample_workspace_bytes,
 * b200_engine_set_sampler, b200_engine_options;  4: + layer-stack models (b200_stack_desc, b200_engine_create_stack),
 * sequence slots and the ragged step (b200_engine_step, b200_engine_slot_*), the per-mechanism stack ops;  5: + sandwich
 * blocks, latent attention, mLSTM, routed experts;  6: + post-norm blocks, the prepared attention (b200_attn_prep_desc), the
 * generalized delta rule, Mamba-2, softmax-routed experts (fields appended to b200_moe_desc and b200_stack_layer),
 * b200_stack_lin_scan, b200_stack_attn_prep.  All additive: callers of an older version keep working. */
#define B200_ABI_VERSION 7

typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_INVALID = -1,     /* bad argument (shape, alignment, null pointer) */
  B200_ERR_UNSUPPORTED = -2, /* valid in the reference, not built here (message says what) */
  B200_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed */
  B200_ERR_NO_DEVICE = -4,   /* no sm_100 device visible */
  B200_ERR_STATE = -5,       /* engine used out of order (e.g. context overflow) */
  B200_ERR_NCCL = -6
} b200_status;

/* QKV layout selector of ropeApply. [ref: TT/Operation/OpNNLayer.h:13-26 enum QKVLayout] */
typedef enum b200_qkv_layout { B200_LAYOUT_BHSD = 0, B200_LAYOUT_BSHD = 1 } b200_qkv_layout;

int b200_abi_version(void);
const char* b200_last_error(void);
/* Number of kernels this library has launched on this process since load (bench.py's gpu_launches claim). */
int64_t b200_launch_count(void);
/* 0 when a compute-capability 10.x device is current, else B200_ERR_NO_DEVICE. */
int b200_device_check(void);

/* ------------------------------------------------------------------------------------------------------------------
 * Boundary B — one entry point per TinyTorch op on the path.
 * ---------------------------------------------------------------------------------------------------------------- */

/* y[m,n] = bf16( x[m,k] · W[n,k]^T ) (fp32 accumulate, one rounding); if bias != NULL:
 * y = bf16( float(y) + float(bias[n]) )  — the reference's second rounding for 3-D Linear inputs.
 * [ref: TT/Operation/OpLinalg.cpp:244-277 matmul + addInplace; TT/Operation/OpLinalgCuda.cuh:276-293
 *  gemmStridedBatchedCudaBF16Impl; caller TT/Function/FuncNNLayer.h:14-18 FuncLinear]
 * Requirements: k % 8 == 0, W 16-byte aligned.  m is small (decode: 1); W is streamed once per 8 rows of x. */
int b200_gemv_bf16(void* y, const void* x, const void* W, const void* bias_or_null, int64_t m, int64_t n, int64_t k,
                   void* stream);

/* Batched (prefill) GEMM on the tcgen05 tensor cores: C[M,N] = bf16( A[M,K] · B[N,K]^T ), fp32 accumulation in TMEM,
 * one rounding.  The m > 1 side of op::matmul for Linear layers (bias / residual are separate ops, as in the reference).
 * [ref: TT/Operation/OpLinalg.cpp:244-277; TT/Operation/OpLinalgCuda.cuh:193-216,276-293]
 * Requirements: K % 8 == 0, N % 8 == 0, 16-byte aligned operands. */
int b200_gemm_bf16(void* C, const void* A, const void* B, int64_t M, int64_t N, int64_t K, void* stream);

/* y[r,:] = bf16( float(x[r,:]) * rsqrtf(mean(x[r,:]^2) + eps) * float(w[:]) )  (single rounding, fp32 weight multiply)
 * [ref: TT/Operation/OpNNLayerCuda.cuh:252-357 kNormSmall/kNormLarge<RMSNorm>, host :569-619] */
int b200_rmsnorm_bf16(void* y, const void* x, const void* w_or_null, int64_t rows, int64_t dim, float eps,
                      void* stream);

/* rotate-half RoPE with the reference's fp32 table [ctx, hd, 2] (cos,sin interleaved):
 * y[i] = bf16(x1*c - x2*s), y[i+hd/2] = bf16(x2*c + x1*s), position = pos_offset + t.
 * [ref: TT/Operation/OpNNLayerCuda.cuh:412-440 kRopeApply, host :658-708] */
int b200_rope_bf16(void* y, const void* x, const float* table_f32, int64_t B, int64_t S, int64_t heads, int64_t hd,
                   int64_t pos_offset, int layout /* b200_qkv_layout */, void* stream);

/* Build the fp32 cos/sin table the way the reference does (device kernels, fp32 powf/cosf/sinf).
 * scaling_factor == 0 disables llama3 scaling.  table_f32 has ctx*hd*2 floats.  Init-time only: uses a stream-ordered
 * temporary (cudaMallocAsync).
 * [ref: TT/Operation/OpNNLayerCuda.cuh:359-410 kRopeComputeInvFreq/kRopeApplyScaling/kRopePrecomputeCosSin,
 *  host :621-656 ropeInitOpCudaImpl] */
int b200_rope_init_f32(float* table_f32, int64_t hd, int64_t ctx, float theta, float scaling_factor,
                       float high_freq_factor, float low_freq_factor, int64_t original_ctx, void* stream);

/* o[B,Sq,Hq,hd] = softmax(q k^T / sqrt(hd)) v, BSHD, GQA (kv head = h / (Hq/Hkv)), causal mask top-left aligned
 * (col > row masked) exactly as TinyFA.  hd in {64, 128}.
 * [ref: TT/Operation/OpNNLayerCuda.cu:12-44 flashAttentionOpCudaImpl → TFA/flash_api.cuh:43-50 tfa::flashAttn →
 *  TFA/mma/kernel.cuh:18-203] */
int b200_attn_bf16(void* o, const void* q, const void* k, const void* v, int64_t B, int64_t Sq, int64_t Skv,
                   int64_t Hq, int64_t Hkv, int64_t hd, int causal, void* stream);

/* y[r,j] = bf16( bf16(silu(g[r,j])) * u[r,j] ), gate_up rows are [gate(I) | up(I)].
 * [ref: TT/Operation/OpFusedCuda.cuh:15-48 kSiluMul; OpElemWiseCuda.cuh:124-131 OpCudaSilu] */
int b200_silu_mul_bf16(void* y, const void* gate_up, int64_t rows, int64_t I, void* stream);

/* y = bf16(a + b) elementwise (alpha = 1). [ref: TT/Operation/OpElemWiseCuda.cuh:133-144,371-381] */
int b200_add_bf16(void* y, const void* a, const void* b, int64_t n, void* stream);

/* y[t,:] = table[ids[t],:] ; ids int64. [ref: TT/Operation/OpTransformCuda.cuh:108-120 kIndex, host :491-526] */
int b200_embedding_bf16(void* y, const void* table, const int64_t* ids, int64_t n_ids, int64_t V, int64_t H,
                        void* stream);

/* idx[r] = argmax_j logits[r,j], compared in fp32, ties resolved to the HIGHEST index (reference CUDA rule).
 * [ref: TT/Operation/OpReduceCuda.cuh:145-156 cudaWarpReduceIdx, :188-224 kReduceIdxMerge, :459-493, :581-636]
 * `workspace` must hold b200_argmax_workspace_bytes(rows, V) bytes, ZERO-INITIALISED once by the caller. */
int64_t b200_argmax_workspace_bytes(int64_t rows, int64_t V);
int b200_argmax_bf16(int64_t* idx, const void* logits, int64_t rows, int64_t V, void* workspace, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Fused building blocks of the engine, exported so that parity tests can drive the exact kernels the engine runs.
 * ---------------------------------------------------------------------------------------------------------------- */

/* One launch = [optional RMSNorm(x, norm_w, eps)] → GEMV → one of
 *   bias      y = bf16(bf16(acc) + bias)                    [ref: TT/Operation/OpLinalg.cpp:273-275]
 *   residual  y = bf16(residual + bf16(acc))                [ref: src/layer/DecoderLayer.h:40-41]
 *   silu_mul  W rows are [gate(n) | up(n)] (nseg = 2):  y = bf16(bf16(silu(bf16(acc_g))) * bf16(acc_u))
 *                                                           [ref: src/layer/GatedMLP.h:37-41]
 * m = 1.  y may alias residual. */
int b200_gemv_fused_bf16(void* y, const void* x, const void* W, int64_t n, int64_t k, int nseg,
                         const void* norm_w_or_null, float eps, const void* bias_or_null,
                         const void* residual_or_null, int silu_mul, void* stream);

/* Decode attention of one layer for one new token (B = 1, Sq = 1), one launch:
 *   q|k|v = qkv  →  [q_norm/k_norm per head]  →  RoPE(q), RoPE(k) at position *pos  →  K/V row *pos written in place
 *   into kcache/vcache [max_ctx, Hkv, hd]  →  split-KV softmax(q kᵀ/√hd) v over rows 0…*pos  →  out [Hq*hd].
 * The context is cut into splits of 256 (hd 64) / 128 (hd 128) keys, one CTA per (KV head, split).
 * *pos must have been written before the kernel that produced `qkv` was launched (the kernel reads it, and the cached
 * rows below it, ahead of its programmatic-dependency wait).
 * pos == NULL: plain attention over `fixed_len` cached rows, nothing appended, no rotation (rope_table may be NULL).
 * workspace: b200_attn_decode_workspace_bytes() bytes, ZERO-INITIALISED once by the caller (tickets self-reset).
 * [ref: src/layer/Attention.h:71-112,156-163; src/engine/CacheManager.h:24-42; TFA/mma/kernel.cuh:18-203] */
int64_t b200_attn_decode_workspace_bytes(int64_t Hq, int64_t Hkv, int64_t hd, int64_t max_ctx);
int b200_attn_decode_bf16(void* out, const void* qkv, const void* q_norm_or_null, const void* k_norm_or_null,
                          float eps, const float* rope_table, const int32_t* pos_or_null, int64_t fixed_len,
                          void* kcache, void* vcache, int64_t Hq, int64_t Hkv, int64_t hd, int64_t max_ctx,
                          void* workspace, void* stream);

/* Sampler::sample for one row of bf16 logits [V] on the device (temperature → top-k → top-p → min-p → softmax →
 * inverse-CDF draw with the caller's uniform number u in (0, 1]), without sorting the vocabulary (sampling.cu).
 * [ref: src/engine/Sampler.cpp:31-78; third_party/TinyTorch/src/Operation/OpSamplingCuda.cu:30-62,97-170,261-330]
 * Greedy decoding (temperature 0, top_k 0, top_p 1, min_p 0) is b200_argmax_bf16.  `workspace`: 256-byte aligned,
 * b200_sample_workspace_bytes() bytes. */
int64_t b200_sample_workspace_bytes(void);
int b200_sample_bf16(int64_t* token_out, const void* logits, int64_t V, float temperature, int64_t top_k, float top_p,
                     float min_p, float u, void* workspace, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Boundary A — the whole per-token forward behind GPTModel::forward / GPTEngine::genNextToken.
 * [ref: src/model/GPTModel.h:51-58 CausalLM::forward, :80-106 GPTModel; src/layer/DecoderLayer.h:38-43;
 *  src/layer/Attention.h:71-112,156-163; src/layer/GatedMLP.h:37-41; src/engine/CacheManager.h:13-55;
 *  src/engine/GPTEngine.cpp:94-99,154-174; src/engine/Sampler.cpp:23-29 greedy branch]
 * ---------------------------------------------------------------------------------------------------------------- */

typedef struct b200_model_desc {
  int32_t hidden;         /* H */
  int32_t layers;         /* L */
  int32_t q_heads;        /* Hq  (global, before tensor-parallel sharding) */
  int32_t kv_heads;       /* Hkv (global) */
  int32_t head_dim;       /* hd: 64 or 128 */
  int32_t intermediate;   /* I   (global) */
  int32_t vocab;          /* V */
  int32_t max_ctx;        /* KV-cache capacity in tokens; also the number of rows of rope_table */
  float rms_eps;
  int32_t qkv_bias;       /* Qwen2: 1 [ref: src/model/ModelQwen2.h:26-31] */
  int32_t qk_norm;        /* Qwen3: per-head RMSNorm on q and k before RoPE [ref: src/layer/Attention.h:156-163] */
  int32_t tp_rank;        /* tensor-parallel rank / world; world == 1 ⇒ single GPU */
  int32_t tp_world;
  int32_t tp_shard_attn;  /* 1: heads sharded over ranks; 0: attention replicated (Hkv % world != 0) */
} b200_model_desc;

/* Per-layer weights, all bf16, exactly the reference's state layout:
 *   qkv_w rows = [q(qDim) | k(kvDim) | v(kvDim)] × H   [ref: src/layer/Linear.h:64-79 MergedLinear views]
 *   gate_up_w rows = [gate(I) | up(I)] × H               [ref: src/layer/GatedMLP.h:19-21]
 * For tensor-parallel engines the pointers are this rank's shard (see tinygpt_b200/tp.py for the slicing rule). */
typedef struct b200_layer_weights {
  const void* input_norm; /* [H] */
  const void* qkv_w;      /* [qDim + 2 kvDim, H] */
  const void* qkv_b;      /* [qDim + 2 kvDim] or NULL */
  const void* q_norm;     /* [hd] or NULL */
  const void* k_norm;     /* [hd] or NULL */
  const void* o_w;        /* [H, qDim] */
  const void* post_norm;  /* [H] */
  const void* gate_up_w;  /* [2 I, H] */
  const void* down_w;     /* [H, I] */
} b200_layer_weights;

typedef struct b200_weight_table {
  const void* embed;        /* [V, H] */
  const void* final_norm;   /* [H] */
  const void* lm_head;      /* [V, H] (== embed when tie_word_embeddings) */
  const float* rope_table;  /* [max_ctx, hd, 2] fp32, the reference's RoPE::cache() tensor */
  const b200_layer_weights* layers_host; /* HOST array of `layers` entries holding device pointers */
} b200_weight_table;

typedef struct b200_engine b200_engine;

/* Borrow the weights (no copy), allocate the in-place KV cache [L][2][max_ctx][Hkv][hd] + workspace once,
 * encode the TMA descriptors, capture the per-token CUDA graphs.  Synchronises the device once (weights may still
 * be in flight on the loader thread's stream, see SURVEY.md §8b "Threading"). */
int b200_engine_create(const b200_model_desc* desc, const b200_weight_table* weights, b200_engine** out);
void b200_engine_destroy(b200_engine* eng);

/* New sequence: position ← 0 (the KV cache is overwritten in place). [ref: GPTModel::resetCache, GPTModel.h:91-94] */
int b200_engine_reset(b200_engine* eng, void* stream);

/* Rewind to `position` (0 <= position <= current): the cached K/V rows below it stay valid, later rows are
 * overwritten as decoding continues.  Used to re-decode from a shared prefix (and by bench.py between timed steps). */
int b200_engine_seek(b200_engine* eng, int64_t position, void* stream);

/* model()(ids): run S tokens of B sequences (ids [B, S] row-major, 1 ≤ B ≤ 8, all at the engine's current position — the
 * reference's left-padded batch, src/engine/GPTEngine.cpp:101-174) and return logits.
 *   logits_mode 0: logits_out is [B, V]      — last position only
 *   logits_mode 1: logits_out is [B, S, V]   — every position, like the reference's lm_head over all S
 * B > 1 (single-GPU, greedy engines): every sequence has its own KV cache; a decode step streams the weights ONCE for the
 * whole batch (gemv_batch.cu: tensor cores, the B activation vectors as the n = 8 MMA operand) and agrees with B independent
 * batch-1 steps to summation-order noise, like the reference's own m = B GEMM against its m = 1 path.  The first call with a new B builds
 * the batch's buffers and graphs.  b200_engine_decode / b200_engine_last_token follow the batch of the latest forward.
 * After the call the engine's "current token" is the greedy argmax of the last position (reference tie rule), so
 * b200_engine_decode can continue without a host round trip.  logits_out may be NULL. */
int b200_engine_forward(b200_engine* eng, const int64_t* ids, int64_t B, int64_t S, void* logits_out,
                        int logits_mode, void* stream);

/* The generateSync hot loop on device: n_steps × { forward(current token) → greedy argmax → becomes current }.
 * tokens_out[i] (int64) receives the token produced by step i ([n_steps][B] after a batched forward).  No host
 * synchronisation. */
int b200_engine_decode(b200_engine* eng, int64_t n_steps, int64_t* tokens_out, void* stream);

/* Greedy token(s) chosen after the most recent forward/decode step (int64 [B], device → device copy on `stream`). */
int b200_engine_last_token(b200_engine* eng, int64_t* token_out, void* stream);

/* Async token pipeline [ref: src/engine/GPTEngine.cpp:17-35 AsyncTokenPipeline / DefaultTokenPipeline::fetchTokenId —
 * a blocking Tensor::item() per token — and :180-232 generateAsync].  Here the kernel that picks the greedy token also
 * posts it into a ring in PINNED, device-mapped HOST memory, as ONE 8-byte word
 *     ((n & 0xffffffff) << 32) | (uint32)token        n = 1-based count of tokens this engine has generated
 * at ring[(n - 1) % capacity], so the host reads tokens by polling memory: no stream synchronisation, no memcpy, and
 * the engine can run several steps ahead of the consumer (EOS / abort: stop launching, b200_engine_seek back).
 * `ring_host_mapped` must be 8-byte aligned pinned memory that the device can address (cudaHostAlloc /
 * cudaHostRegister; with unified addressing the host pointer itself), zero-initialised, alive until the mailbox is
 * cleared with ring = NULL or the engine destroyed.  Re-captures the per-token graphs; single-GPU engines only. */
int b200_engine_set_mailbox(b200_engine* eng, uint64_t* ring_host_mapped, int64_t capacity, void* stream);
/* SamplerConfig of the generate loop [ref: src/engine/Sampler.h:13-22, Sampler.cpp:14-21]: with any knob set
 * (temperature > 0, top_k > 0, top_p < 1, min_p > 0) the engine picks every token with the device sampler
 * (b200_sample_bf16's kernels, uniform number = Philox4x32-10(seed, tokens generated so far)); all knobs off = greedy
 * argmax again.  Re-captures the per-token graph; single-GPU engines only. */
int b200_engine_set_sampler(b200_engine* eng, float temperature, int64_t top_k, float top_p, float min_p, uint64_t seed,
                            void* stream);
/* Host-side mirror: how many tokens this engine has generated (= n of the most recently enqueued token). */
int64_t b200_engine_generated(const b200_engine* eng);

/* Debug (engine created with B200_TRACE=1 in the environment): copies [launch][8] %globaltimer stamps (entry, after
 * the PDL wait, exit, x ready, first stage landed, first row block summed, first row block stored, unused) of the GEMV / attention launches of the most recent token into out_host; synchronises.
 * Returns the number of launches copied (0 when tracing is off). */
int64_t b200_engine_debug_trace(b200_engine* eng, uint64_t* out_host, int64_t max_entries);

/* Host-side mirrors (no device access): tokens consumed so far, and kernels per decoded token (of the batched graph
 * while the engine holds a batch: the same nodes, plus one per layer when the down projection runs in two groups). */
int64_t b200_engine_position(const b200_engine* eng);
int64_t b200_engine_launches_per_token(const b200_engine* eng);
/* Which code paths this engine was built with (environment / defaults at create time): bit 0 CUDA graph, bit 1
 * programmatic dependent launch, bit 3 batched GEMM prefill (bit 2 and bits 8-15 belonged to variants that were measured
 * and removed: profiles/experiments/). */
int64_t b200_engine_options(const b200_engine* eng);
/* Algorithmic HBM bytes one decode step reads on THIS rank at context length ctx (weights once + KV + logits). */
int64_t b200_engine_bytes_per_token(const b200_engine* eng, int64_t ctx);

/* ------------------------------------------------------------------------------------------------------------------
 * Layer-stack models: a model described as DATA — a list of layer runs, each with a mixer, an optional gated
 * feed-forward and an optional per-token side input — instead of the fixed Llama-family wiring above.  The same engine
 * handle, entry points (forward / decode / reset / seek / last_token / set_sampler), argmax and sampler kernels serve
 * it.  What a stack engine adds to the engine:
 *   - the residual stream, every norm, the softmax and the gates are fp32; matrix products take bf16 operands with
 *     fp32 accumulation (B200_BF16) or are true fp32 FMA chains (B200_F32: weights, caches and activations in fp32);
 *   - sequence SLOTS: `max_slots` independent KV caches of `max_ctx` rows with their own positions, and a RAGGED step
 *     (b200_engine_step) that runs any number of new tokens for any subset of the slots in one pass;
 *   - attention with arbitrary head sizes (key size ≠ value size), an explicit score scale, a sliding window with kept
 *     first keys, and a per-head sigmoid output gate; gated feed-forward with tanh-GELU; a parallel block
 *     (x += m·(mixer(h) + ff(h)), one norm); a looped span of layers (own cache per pass) whose passes start with a
 *     projection of [x; x0]; a gated per-layer token table added through a weighted RMS norm.
 * Weight layout (built by tinygpt_b200/loader.py): the projections that read the block norm are merged by rows into
 * w_in = [q | k | v | gate logits | ff gate | ff up] (segments padded to 8 rows), the projections that feed the
 * residual are merged by columns into w_out = [o | ff down]; vectors (norm weights, biases) are fp32.
 * ---------------------------------------------------------------------------------------------------------------- */
typedef enum b200_dtype { B200_BF16 = 0, B200_F32 = 1 } b200_dtype;
/* PARALLEL: x += m·(mixer(h) + ff(h)), h = norm(x), one norm.  SANDWICH: x += post_norm(mixer(norm(x))), then
 * x += ff_post_norm(ff(ff_norm(x))) — a norm before and after every sublayer.  POSTNORM: x += post_norm(mixer(x)), then
 * x += ff_post_norm(ff(x)) — the sublayers read the stream itself, the norm sits on their output only. */
typedef enum b200_block_kind { B200_BLOCK_PARALLEL = 0, B200_BLOCK_SANDWICH = 1, B200_BLOCK_POSTNORM = 2 } b200_block_kind;
/* RELU2: max(z, 0)²; TANH: tanh(z) (the bottleneck of a low-rank decay projection). */
typedef enum b200_ff_act {
  B200_ACT_GELU_TANH = 0, B200_ACT_SILU = 1, B200_ACT_GELU_ERF = 2, B200_ACT_RELU2 = 3, B200_ACT_TANH = 4
} b200_ff_act;
/* RMS: x·rsqrt(mean(x²) + eps)·(offset + w).  LAYER: (x − mean)·rsqrt(var + eps)·(offset + w), no bias. */
typedef enum b200_norm_kind { B200_NORM_RMS = 0, B200_NORM_LAYER = 1 } b200_norm_kind;
/* ATTENTION: the gated windowed attention of b200_attn_desc.  LATENT: keys and values expanded from a cached low-rank
 * latent + one rotated key part shared by the heads (b200_latent_desc).  MLSTM: a matrix memory per head carried from
 * token to token (b200_mlstm_desc); its state lives in fp32 beside the slot's caches.  DELTA: a key × value matrix per
 * head with a per-channel decay and a rank-one removal along the unit key (b200_delta_desc).  MAMBA2: a short causal
 * convolution and a scalar-decay state-space recurrence per head (b200_mamba_desc); the convolution's last inputs are part
 * of the state.  In sandwich and post-norm blocks ATTENTION is the windowed attention of b200_attn_desc behind the
 * per-token preparation of b200_attn_prep_desc (query / key norms, rotary positions, value norm, value mix-in).
 * GATED_DELTA: the gated delta rule — a key × value matrix per head with one decay per head and a removal along the unit
 * key weighted by a per-head write strength, behind short causal convolutions (b200_gdelta_desc). */
typedef enum b200_mixer_kind {
  B200_MIX_ATTENTION = 0, B200_MIX_LATENT = 1, B200_MIX_MLSTM = 2, B200_MIX_DELTA = 3, B200_MIX_MAMBA2 = 4,
  B200_MIX_GATED_DELTA = 5
} b200_mixer_kind;
/* GATED: act(gate)·up → down (merged into w_in / w_out).  DENSE: act(up) → down.  MOE: routed clamped gated experts
 * (+ optional gated shared expert), b200_moe_desc. */
typedef enum b200_ff_kind { B200_FF_GATED = 0, B200_FF_DENSE = 1, B200_FF_MOE = 2 } b200_ff_kind;

typedef struct b200_attn_desc {
  int32_t heads;       /* query heads */
  int32_t kv_heads;    /* key/value heads; query head h reads kv head h / (heads / kv_heads) */
  int32_t dim;         /* per-head query/key size */
  int32_t vdim;        /* per-head value size */
  float scale;         /* score = (q·k)·scale */
  int32_t window;      /* key j visible from query i when j <= i and i - j < window; 0 = every earlier key */
  int32_t keep_first;  /* keys j < keep_first stay visible whatever the window */
  int32_t out_gate;    /* 1: head output × sigmoid(gate logit of that head) */
  int32_t sink;        /* 1: the softmax's denominator gains 1 — a sink of score 0 that has no value */
} b200_attn_desc;

/* Latent attention (sizes heads / dim / vdim / scale / window in b200_attn_desc; kv_heads = 1, no per-head gate).  Per head the
 * query is [dim plain | rot_dim rotated]; w_in rows are [q: heads·(dim + rot_dim) | down: kv_rank + rot_dim] (the down
 * segment starts at off_k).  c = rms(down[:kv_rank])·c_norm is the latent, down[kv_rank:] rotated is the key part all
 * heads share; the slot's cache row of a position is [c | rotated key part].  score = (q_plain·(uk_h c) + q_rot·k_rot)·scale,
 * value = uv_h c; the engine folds uk_h into the query and uv_h behind the softmax, so only cache rows are read.
 * Rotation: pair (2i, 2i+1) of the first rot_dims entries turns by the angle of rot_table[pos][i] = {cos, sin}·magnitude. */
typedef struct b200_latent_desc {
  int32_t kv_rank, rot_dim, rot_dims;
  const float* c_norm;      /* [kv_rank] */
  const void* uk_t;         /* [heads][kv_rank][dim]: uk of head h transposed */
  const void* uk;           /* [heads·dim][kv_rank] as stored, or NULL (then prompts take the general kernels) */
  const void* uv;           /* [heads·vdim][kv_rank] */
  const float* rot_table;   /* [max_ctx][rot_dims/2][2] fp32 */
  /* variants (all 0 / NULL: the form above) */
  int32_t rot_half;         /* 1: entry i of the rotated part is paired with entry i + rot_dims/2 instead of (2i, 2i+1) */
  int32_t q_rank;           /* > 0: queries go through a latent — w_in's q segment holds q_rank rows (the down-projection),
                             * q = uq·(rms(those rows)·q_norm) */
  const float* q_norm;      /* [q_rank] */
  const void* uq;           /* [heads·(dim + rot_dim)][q_rank] */
  int32_t out_gate;         /* 1: the concatenated head outputs × sigmoid(gate logits), heads·vdim rows of w_in at off_g */
} b200_latent_desc;

/* mLSTM (sizes heads / dim / vdim in b200_attn_desc).  w_in rows [q | k | v | out gate: heads·vdim | gates: 2·heads] at
 * off_q / off_k / off_v / off_g / off_gate; the gate rows (input-gate rows, then forget-gate rows, biases in b_in) give raw
 * logits that are kept in fp32 and capped as cap·tanh(z/cap); i = capped, f = logsigmoid(capped); m_t = max(f + m, i),
 * S_t = e^(f+m−m_t) S + e^(i−m_t) k vᵀ, n likewise, o = Sᵀq' / (max(|n·q'|, e^(−m_t)) + 1e-6) with q' = q·dim^(−1/2);
 * then o/rms(o) per head · head_norm · sigmoid(out gate). */
typedef struct b200_mlstm_desc {
  float gate_cap;
  const float* head_norm;   /* [heads·vdim] */
} b200_mlstm_desc;

/* Mixture of experts: scores = sigmoid(router·h) (fp32), the `top` largest are chosen, the chosen expert runs on score·h
 * (the weight multiplies the expert's INPUT), outputs are summed.  Expert: g = min(gate·h, limit), u = clamp(up·h, ±limit),
 * down·(g·sigmoid(1.702 g)·(u + 1)).  Shared expert (shared_ff > 0): the same form on h itself, times sigmoid(sg·h). */
typedef struct b200_moe_desc {
  int32_t experts, top, expert_ff, shared_ff;
  float limit, shared_limit;
  const void* router;       /* [experts, width] */
  const void* w_exp_in;     /* [experts][2·expert_ff, width]: gate rows, then up rows (expert_act != 0: [experts][expert_ff, width]) */
  const void* w_exp_out;    /* [experts][width, expert_ff] */
  /* variants (all 0: the form above) */
  int32_t router_kind;      /* 0: weight = sigmoid(logit).  1: scores = softmax over all experts, the chosen scores are divided
                             * by their sum (+ 1e-20) and multiplied by route_scale */
  int32_t weight_output;    /* 0: the weight multiplies the expert's input, 1: its output */
  int32_t expert_act;       /* 0: the clamped gated unit.  else a b200_ff_act applied to up·h alone (no gate rows, no clamp);
                             * the shared expert has the same form: w_ff_in [up8(shared_ff), width] */
  int32_t shared_plain;     /* 0: shared expert × sigmoid(sg·h).  1: added as it is (no gate row) */
  float route_scale;
} b200_moe_desc;

/* What happens to q | k | v of an attention mixer between the in-projection and the cache, per token, in fp32:
 *   qk_norm: q (all heads·dim entries at once) and k (all kv_heads·dim) are RMS-normed and multiplied by q_norm / k_norm;
 *   rot_dims > 0: entry i < rot_dims/2 of every head of q and k is paired with entry i + rot_dims/2 and turned by the angle
 *     whose {cos, sin} is rot_table[pos][i] (the entries from rot_dims on pass unchanged);
 *   v_norm: every head's value is divided by its root mean square;
 *   v_mix 1: this layer's values are kept for the later layers of the pass.  v_mix 2: v <- (1 − lambda)·v + lambda·(the values
 *     the v_mix 1 layer kept for the same token), lambda read from mix_lambda on the device.
 * What this leaves in the projection rows is what is cached and attended. */
typedef struct b200_attn_prep_desc {
  int32_t qk_norm, rot_dims, v_norm, v_mix;
  const float* q_norm;      /* [heads·dim] */
  const float* k_norm;      /* [kv_heads·dim] */
  const float* rot_table;   /* [max_ctx][rot_dims/2][2] fp32 */
  const float* mix_lambda;  /* [1] */
  int32_t rot_interleaved;  /* 1: pair i is entries (2i, 2i+1) of the head instead of (i, i + rot_dims/2) */
} b200_attn_prep_desc;

/* Generalized delta rule (sizes heads / dim / vdim in b200_attn_desc).  w_in rows [r | k | v | out gate: heads·vdim |
 * removal logits: heads·dim | decay bottleneck: rank] at off_q / off_k / off_v / off_g / off_gate / off_up (the removal bias
 * in b_in).  Per head and key channel: decay w = exp(−decay_scale·sigmoid(w2·tanh(bottleneck) + w0)), removal a =
 * sigmoid(logit); u = k / sqrt(Σk² + unit_eps);  S_t = diag(w) S − (a∘u)(uᵀS) + k vᵀ (both terms read the old S), o = Sᵀr;
 * then o / rms(o) per head · head_norm · sigmoid(out gate). */
typedef struct b200_delta_desc {
  int32_t rank;
  float decay_scale, unit_eps;
  const void* w2;           /* [heads·dim, up8(rank)] (padding columns zero) */
  const float* w0;          /* [heads·dim] */
  const float* head_norm;   /* [heads·vdim] */
} b200_delta_desc;

/* Mamba-2 (heads, vdim in b200_attn_desc; dim = state).  w_in rows [z: inner | x: inner | B: groups·state | C: groups·state
 * | dt: heads] at off_g / off_v / off_k / off_q / off_gate, inner = heads·vdim; x | B | C are contiguous (off_k = off_v +
 * inner, off_q = off_k + groups·state) and pass a causal convolution of `taps` taps per channel (conv_w [channels, taps],
 * last column the current token's; conv_b) and SiLU.  dt = softplus(dt + dt_bias); per head (group h / (heads / groups)):
 * S_t = exp(−exp(A_log)·dt) S + dt·B xᵀ, y = SᵀC + D x; then y·silu(z), an RMS norm in norm_groups equal parts, · norm. */
typedef struct b200_mamba_desc {
  int32_t state, groups, taps, norm_groups;
  const float* conv_w;      /* [inner + 2·groups·state, taps] */
  const float* conv_b;      /* [inner + 2·groups·state] */
  const float* dt_bias;     /* [heads] */
  const float* A_log;       /* [heads] */
  const float* D;           /* [heads] */
  const float* norm;        /* [inner] */
} b200_mamba_desc;

/* Gated delta rule (heads = value heads, kv_heads = query / key heads, dim, vdim in b200_attn_desc; value head h reads
 * query / key head h / (heads / kv_heads)).  w_in rows [q: kv_heads·dim | k: kv_heads·dim | v: heads·vdim | out gate:
 * heads·vdim | write strength: heads | decay logit: heads] at off_q / off_k / off_v / off_g / off_gate / off_up.  q, k and v
 * pass a causal convolution of `taps` taps per channel (conv_w [channels, taps] over q | k | v, last column the current
 * token's, no bias; zeros before the sequence) and SiLU; q and k become unit vectors per head, x / sqrt(Σx² + unit_eps), q
 * also times dim^(−1/2).  beta = sigmoid(strength), g = exp(−exp(A_log)·softplus(decay logit + dt_bias)).  Per head:
 * S <- g·S;  u = beta·(v − Sᵀk);  S <- S + k uᵀ;  o = Sᵀq.  Then o / rms(o) · head_norm · silu(out gate).  The state S (fp32)
 * and the convolutions' last taps − 1 inputs live in the slot. */
typedef struct b200_gdelta_desc {
  int32_t taps;
  float unit_eps;
  const float* conv_w;      /* [2·kv_heads·dim + heads·vdim, taps] */
  const float* A_log;       /* [heads] */
  const float* dt_bias;     /* [heads] */
  const float* head_norm;   /* [vdim], shared by the heads */
} b200_gdelta_desc;

typedef struct b200_stack_layer {
  b200_attn_desc attn;
  int32_t ff;          /* feed-forward width; 0 = the layer has none */
  int32_t ff_act;      /* b200_ff_act */
  int32_t off_q, off_k, off_v, off_g, off_gate, off_up, n_in; /* first row of each segment of w_in; n_in = all rows */
  int32_t off_act, k_out; /* w_out columns: [0, heads·vdim) attention, [off_act, off_act + ff) feed-forward; k_out = all
                           * (sandwich blocks: k_out = heads·vdim, the mixer alone) */
  const float* norm;   /* [width] */
  const void* w_in;    /* [n_in, width] */
  const float* b_in;   /* [n_in] (0 where a segment has no bias) or NULL */
  const void* w_out;   /* [width, k_out] */
  int32_t side_col;    /* first column of this layer's part of the side table */
  const void* side_gate; /* [side_dim, width] or NULL: no side input */
  const void* side_proj; /* [width, side_dim] */
  const float* side_norm; /* [width] */
  /* ---- sandwich blocks (zero / NULL for parallel blocks) */
  int32_t mixer;         /* b200_mixer_kind */
  int32_t ff_kind;       /* b200_ff_kind */
  const float* post_norm;    /* [width] norm of the mixer's output */
  const float* ff_norm;      /* [width] norm before the feed-forward */
  const float* ff_post_norm; /* [width] norm of the feed-forward's output */
  /* feed-forward of a sandwich block: DENSE w_ff_in [ff, width], w_ff_out [width, ff]; MOE with a shared expert:
   * w_ff_in [up8(2·shared_ff + 1), width] = [gate | up | shared-gate logit row], w_ff_out [width, shared_ff] */
  const void* w_ff_in;
  const void* w_ff_out;
  b200_latent_desc lat;
  b200_mlstm_desc rec;
  b200_moe_desc moe;
  b200_attn_prep_desc prep;
  b200_delta_desc delta;
  b200_mamba_desc mamba;
  b200_gdelta_desc gdelta;
  const float* b_out;    /* [width] bias of the mixer's out-projection, or NULL */
  int32_t kv_share;      /* attention mixers: > 0: this layer has no key / value rows in w_in and no cache of its own — it
                          * reads the rows that layer kv_share − 1 (an earlier attention layer with equal kv_heads, dim and
                          * vdim) cached for the same positions */
} b200_stack_layer;

typedef struct b200_stack_desc {
  int32_t dtype;         /* b200_dtype of matrices, caches and activations */
  int32_t block;         /* b200_block_kind */
  int32_t width, vocab, n_layers, n_runs;
  const int32_t* run_layer_host;  /* [n_runs] which layer each run executes (a looped layer appears once per pass) */
  const int32_t* run_mix_host;    /* [n_runs] 1: before this run x <- mix_in·[x; x0] (x0 = the embedding output) */
  float embed_scale, residual_mult, norm_eps;
  float norm_offset;     /* block and final norms multiply by (norm_offset + w) */
  int32_t side_dim, side_stride;  /* columns per layer / per row of side_table */
  int32_t max_ctx, max_slots;
  const void* embed;     /* [vocab, width] */
  const void* mix_in;    /* [width, 2·width] or NULL */
  const void* side_table; /* [vocab, side_stride] or NULL */
  const float* final_norm; /* [width] */
  const void* head;      /* [vocab, width] */
  const b200_stack_layer* layers_host;
  int32_t norm_kind;     /* b200_norm_kind of the block and final norms */
  float logit_softcap;   /* > 0: logits <- cap·tanh(logits / cap) */
} b200_stack_desc;

/* Build a stack engine (single GPU).  Borrows the weights; owns the caches [slot][run][max_ctx][kv_heads·dim | ·vdim],
 * the per-slot positions / current tokens / token logs and a workspace that grows with the largest step. */
int b200_engine_create_stack(const b200_stack_desc* desc, b200_engine** out);

/* Ragged step: sequence i (slot slots_host[i]) consumes counts_host[i] new tokens, taken in order from ids_host; every
 * token attends to its slot's cache and to the earlier tokens of its own sequence in this step.  want_host lists flat
 * indices into ids_host whose logits are written, in that order, to logits_out_dev (fp32 [n_want, vocab], device).
 * greedy != 0: the argmax (or the configured sampler) of the LAST token of every sequence becomes that slot's current
 * token, so b200_engine_decode can go on, and the sequences become the engine's active batch.
 * The logits at a position depend neither on how its prompt was cut into steps nor on the other sequences of a step.
 * Host arrays may be freed on return. */
int b200_engine_step(b200_engine* eng, int64_t n_seq, const int32_t* slots_host, const int32_t* counts_host,
                     const int64_t* ids_host, int64_t n_want, const int32_t* want_host, float* logits_out_dev,
                     int greedy, void* stream);
/* Give a slot back: its position returns to 0 and its cache rows are overwritten by the next sequence. */
int b200_engine_slot_reset(b200_engine* eng, int64_t slot, void* stream);
int64_t b200_engine_slot_position(const b200_engine* eng, int64_t slot);
int64_t b200_engine_max_slots(const b200_engine* eng);

/* The stack engine's mechanisms as stand-alone ops (dtype = b200_dtype of T; fp32 where the name says so), exported so
 * that parity tests drive the kernels the engine runs. */
/* y[r,:] = T( x[r,:] · rsqrt(mean(x[r,:]²) + eps) · (offset + w[:]) ), x fp32 */
int b200_stack_rmsnorm(void* y, const float* x, const float* w, int64_t rows, int64_t dim, float eps, float offset,
                       int dtype, void* stream);
/* C[M,N] = A[M,K]·W[N,K]ᵀ (+ bias[N]) with fp32 accumulation; A, W, C of dtype T (any M, N, K) */
int b200_stack_linear(void* C, const void* A, const void* W, const float* bias_or_null, int64_t M, int64_t N, int64_t K,
                      int dtype, void* stream);
/* Attention of n_tok new tokens over per-slot caches: token t (slot[t], position pos[t]) reads its q (and gate logit)
 * from `proj` (row stride ld_proj, segments at off_q / off_g) and the keys of its slot's cache
 * kcache[slot·k_slot_stride + j·kv_heads·dim …], j visible under (window, keep_first); out[t, h·vdim …] (row stride
 * ld_out).  The rows of this step's own tokens must already be in the cache (b200_stack_kv_store). */
int b200_stack_attention(void* out, int64_t ld_out, const void* proj, int64_t ld_proj, int64_t off_q, int64_t off_g,
                         const void* kcache, const void* vcache, int64_t k_slot_stride, int64_t v_slot_stride,
                         const int32_t* slot, const int32_t* pos, int64_t n_tok, const b200_attn_desc* attn, int dtype,
                         void* stream);
int b200_stack_kv_store(void* kcache, void* vcache, int64_t k_slot_stride, int64_t v_slot_stride, const void* proj,
                        int64_t ld_proj, int64_t off_k, int64_t off_v, const int32_t* slot, const int32_t* pos,
                        int64_t n_tok, const b200_attn_desc* attn, int dtype, void* stream);
/* y[r, j] = T( act(g[r, j]) · u[r, j] ) over row-strided operands */
int b200_stack_act_mul(void* y, int64_t ld_y, const void* g, const void* u, int64_t ld_gu, int64_t rows, int64_t n,
                       int act, int dtype, void* stream);
/* x[r,:] += mult · y[r,:] · rsqrt(mean(y[r,:]²) + eps) · w[:]   (all fp32) */
int b200_stack_rms_add(float* x, const float* y, const float* w, int64_t rows, int64_t dim, float eps, float mult,
                       void* stream);
/* y[r,:] = T( norm(x[r,:]) · w ) with norm of b200_norm_kind `kind`, x fp32;  add != 0: xadd[r,:] += that (fp32, y unused) */
int b200_stack_norm(void* y, float* xadd, const float* x, const float* w, int64_t rows, int64_t dim, float eps, int kind,
                    int add, int dtype, void* stream);
/* Latent attention over per-slot caches, everything between the in-projection and the out-projection: `proj` rows hold
 * [q | down] (q at column 0, down at off_down); the cache rows [c | rotated key] of the new tokens are written, then every
 * token attends to rows 0 … pos of its slot; out[t, h·vdim …] (row stride ld_out). */
int b200_stack_latent_attention(void* out, int64_t ld_out, const void* proj, int64_t ld_proj, int64_t off_down, void* cache,
                                int64_t slot_stride, const int32_t* slot, const int32_t* pos, int64_t n_tok,
                                const b200_attn_desc* attn, const b200_latent_desc* lat, float eps, int dtype, void* stream);
/* mLSTM recurrence of n_seq sequences laid side by side: sequence s brings rows [row0[s], row0[s] + count[s]) of `proj`
 * (q | k | v at off_q / off_k / off_v) and `gates` (fp32 [rows, 2·heads] raw logits), continues the state of its slot
 * (slot / pos are per ROW; a sequence whose first row has pos 0 starts from zero) and leaves it advanced.
 * out fp32 [rows, heads, vdim + 2]: numerators Sᵀq', then n·q', then m.  State of a slot: b200_stack_mlstm_state_floats. */
int b200_stack_mlstm(float* out, const void* proj, int64_t ld_proj, int64_t off_q, int64_t off_k, int64_t off_v,
                     const float* gates, float* state, int64_t slot_stride, const int32_t* row0, const int32_t* count,
                     const int32_t* slot, const int32_t* pos, int64_t n_seq, int64_t n_rows, const b200_attn_desc* sizes,
                     float gate_cap, int dtype, void* stream);
int64_t b200_stack_mlstm_state_floats(int64_t heads, int64_t dim, int64_t vdim);
/* Routed experts on h [rows, width] (T): y fp32 [rows, width] = Σ_chosen expert_e(score_e · h); `chosen` (int32
 * [rows, top]) and `scores` (fp32 [rows, top]) receive the routing when not NULL.  Synchronises (allocates its workspace). */
int b200_stack_moe(float* y, const void* h, int64_t rows, int64_t width, const b200_moe_desc* moe, int32_t* chosen,
                   float* scores, int dtype, void* stream);
/* The linear recurrence of n_seq sequences laid side by side (rows [row0[s], row0[s] + count[s]) in order), all operands fp32
 * rows of stride ld: per head h and value column j, with s the dk entries of column j of S,
 *   s <- d∘s − p·(q·s) + b·(v_j·vscale),  out[row, h·dv + j] = s·r.
 * d [heads·dk] per row, or (d_scalar) [heads]; p, q [heads·dk] or both NULL (no removal); b, r [heads/share][dk] (`share`
 * consecutive heads read one vector); v [heads·dv]; vscale [heads] or NULL.  State of a slot: [heads][dk][dv] fp32 at
 * state + slot·slot_stride (slot / pos per ROW; a sequence whose first row has pos 0 starts from zero). */
int b200_stack_lin_scan(float* out, const float* d, const float* p, const float* q, const float* b, const float* r, const float* v,
                        const float* vscale, int64_t ld, int64_t heads, int64_t dk, int64_t dv, int64_t share, int64_t d_scalar,
                        float* state, int64_t slot_stride, const int32_t* row0, const int32_t* count, const int32_t* slot,
                        const int32_t* pos, int64_t n_seq, int64_t n_rows, void* stream);
/* The preparation of an attention mixer's q | k | v (b200_attn_prep_desc), in place in proj's rows (row stride ld_proj, segments
 * at off_q / off_k / off_v); vkeep (T [n_tok, ld_keep]) is written by a v_mix 1 layer and read by a v_mix 2 layer. */
int b200_stack_attn_prep(void* proj, int64_t ld_proj, int64_t off_q, int64_t off_k, int64_t off_v, const int32_t* pos,
                         int64_t n_tok, const b200_attn_desc* attn, const b200_attn_prep_desc* prep, void* vkeep,
                         int64_t ld_keep, float eps, int dtype, void* stream);
/* y[r, j] = T( min(g, limit)·sigmoid(1.702·min(g, limit))·(clamp(u, ±limit) + 1) ), g = gu[r, j], u = gu[r, n + j] */
int b200_stack_glu_clamp(void* y, const void* gu, int64_t rows, int64_t n, float limit, int dtype, void* stream);

/* ---- tensor parallel (one process per GPU; the caller exchanges the handles with torch.distributed) ---------- */

#define B200_IPC_HANDLE_BYTES 64
/* Size in bytes of the per-rank exchange window the engine wants mapped on every peer. */
int64_t b200_tp_window_bytes(const b200_model_desc* desc);
/* Allocate this rank's window and export its IPC handle. */
int b200_tp_window_create(int64_t bytes, void** window_out, uint8_t handle_out[B200_IPC_HANDLE_BYTES]);
/* Map a peer's window. */
int b200_tp_window_open(const uint8_t handle[B200_IPC_HANDLE_BYTES], void** peer_window_out);
int b200_tp_window_close(void* peer_window);
int b200_tp_window_destroy(void* window);
/* Like b200_engine_create, for rank desc->tp_rank of desc->tp_world: `windows_host[r]` is rank r's window as mapped
 * in this process (windows_host[tp_rank] is the local one).  The hidden-vector reductions after o_proj and
 * down_proj are done by the GEMV epilogue pushing fp32 partials into every peer's window over NVLink and the next
 * kernel's prologue summing them (no separate collective kernel). */
int b200_engine_create_tp(const b200_model_desc* desc, const b200_weight_table* weights, void* const* windows_host,
                          b200_engine** out);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* B200_DECODE_H_ */
