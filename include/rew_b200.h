/* rew_b200 — C ABI of the B200 (sm_100a) backend for Rechenwerk's (bitstormFA/rew)
 * transformer-decoder inference path.
 *
 * Conventions
 *   - Every function returns an int status: REWB200_OK (0) or REWB200_ERR.  After
 *     an error rewb200_last_error() returns a thread-local message.  Nothing
 *     throws or aborts across this boundary, and no call blocks without bound
 *     (device-side waits are bounded and report through the status).
 *   - Plain pointers and sizes only.  Host pointers are ordinary host memory
 *     unless a parameter says "device".
 *   - dtype codes are the ordinals of rew's DType enum (src/rew/dtype.nim:10-32).
 *   - Tensors are dense row-major; weights of a Linear are [in, out] as in
 *     src/rew/nn/linear.nim:21-25.
 *   - A rew Nim binding stores a rewb200_buffer* in BufferHandle.raw
 *     (src/rew/buffer.nim:42-65) and calls rewb200_buffer_release from the
 *     BufferReleaser (src/rew/buffer.nim:33).
 */
#ifndef REW_B200_H
#define REW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with hidden visibility */
#endif

#define REWB200_OK 0
#define REWB200_ERR 1

/* DType ordinals, src/rew/dtype.nim:10-32. */
enum {
  REWB200_BOOL = 0,
  REWB200_I8 = 1,
  REWB200_I16 = 2,
  REWB200_I32 = 3,
  REWB200_I64 = 4,
  REWB200_U8 = 5,
  REWB200_F16 = 9,
  REWB200_BF16 = 10,
  REWB200_F32 = 11,
  REWB200_F64 = 12
};

typedef struct rewb200_buffer rewb200_buffer;
typedef struct rewb200_model rewb200_model;
typedef struct rewb200_session rewb200_session;
typedef struct rewb200_nf4 rewb200_nf4;

/* ---- runtime ------------------------------------------------------------
 * Replaces client creation in installEagerBackend (src/rew/eager.nim:1769-1772)
 * and the PJRT client cache (src/rew/eager.nim:78-140).  `device_ordinals`
 * lists the CUDA devices this process drives (slot i <-> ordinal i). */
int rewb200_init(const int* device_ordinals, int n);
int rewb200_shutdown(void);
const char* rewb200_last_error(void);
/* Waits for all queued work of a slot; fails after timeout_ms or when a kernel
 * recorded a device-side status (bounded wait expired, bad index). */
int rewb200_sync(int slot, int timeout_ms);
/* Run-time switches (also read from the environment at init):
 *   "linear" = "mma" | "tc_prefill" | "tc"   bf16 Linear on mma.sync, on tcgen05 for more than 32
 *                                            rows, or on tcgen05 always   (REW_B200_LINEAR)
 *   "pdl"    = "0" | "1"                     programmatic dependent launch (REW_B200_PDL)
 *   "prefill" = "pair" | "persistent" | "tile"   Linear launches of 256-token tiles: persistent CTA pairs on 256 x 256 tiles
 *                                            (tcgen05 cta_group::2; default, widths that are multiples of 256), one
 *                                            persistent CTA per SM with the epilogue overlapped, or one CTA per tile
 *   "profile_linears" = "1".."31"            which launches rewb200_session_profile_linears times: bit 0 q|k|v, 1 o,
 *                                            2 gate|up, 3 down, 4 lm_head (default 31, all)
 *   "ep_exchange" = "auto" | "prefix" | "capacity"   expert-parallel all-to-all: auto (default) = over the peer heap when
 *                                            one is attached and the step fits (rewb200_comm_peer_alloc), else NCCL as under
 *                                            "prefix" from 4 ranks on; prefix = NCCL, pair counts first and then only the
 *                                            occupied prefix of every slot array (steps of 64+ pairs outside a captured
 *                                            graph); capacity = NCCL, always the worst-case capacity
 *   "tp_exchange" = "auto" | "one" | "two"   tensor-parallel all-reduce of decode-size steps over the peer heap: every rank
 *                                            stores its partial to every peer (one hop), or to the owner of the columns,
 *                                            which returns the sum (two hops, fewer bytes; measured slower at 2 and at
 *                                            8 ranks); auto = one hop
 *   "gate_up_split" = "on" | "off"           decode-size gate|up launches with too few feature tiles to fill the GPU split K
 *                                            and finish in a small sum + SwiGLU launch (default), or stay one launch
 *   "qkv_post" = "attention" | "attention_always" | "launch"
 *                                            bf16 decode steps: bias, RoPE and the KV-cache append of the new token inside the
 *                                            attention kernel when its grid is at most one wave (default) / whatever the
 *                                            grid, or in a launch of their own before it
 *   "nf4_gemv" = "tc" | "cuda"               NF4 weight-only Linear, steps of up to four rows: the tensor-core kernel that
 *                                            serves every step up to 32 rows (default), or a CUDA-core code streamer
 *                                            (fp16 pair lookups + HFMA2; measured slower, kept for comparison)
 *   "tp_allreduce" = "heap" | "nccl"         tensor-parallel steps of more than 64 rows (prefill): two-shot all-reduce over
 *                                            the peer heap when its bulk region holds the step (default), or NCCL always
 *   "record_routing" = "0" | "1"             test aid: sessions created afterwards keep every MoE layer's top-k expert ids
 *                                            of their last forward for rewb200_session_routing
 *   "inject_alloc_fail" = "n"                test hook: the n-th activation-buffer allocation from now fails on the host
 *   "moe_overlap" = "on" | "off"             MoE layers on one rank, steps of at most 64 rows: the shared experts run on a
 *                                            second stream beside the routed experts (default on)
 *   "splitk_min_blocks" = "1".."64"          fewest 64-wide K blocks a split-K slice keeps (default 8)
 *   "splitk_rows" = "0".."256"               largest step, in rows, whose Linear launches may split K (default 256)
 *   "splitk" = "slabs" | "cluster" | "qkv" | "out"   decode-size split-K: f32 slabs summed by the next kernel (default),
 *                                            or summed inside thread-block clusters through distributed shared memory
 *                                            (all launches, only q|k|v with its RoPE / cache-write epilogue, or only the others)
 *   "norm" = "cluster" | "row"               decode-size residual+norm: four CTAs per row exchanging the row
 *                                            statistics through distributed shared memory (default), or one CTA per row
 *   "attention_merge" = "launch" | "fused"   split-KV decode attention: a second launch combines the splits (default),
 *                                            or the last CTA of a (sequence, kv head) does
 *   "attention" = "tc" | "tc1" | "tc2" | "mma"   prefill attention with head_dim 128: tcgen05, one query tile per CTA below
 *                                            3072 query rows and two from there up (default); always one; two from 256
 *                                            rows up; mma.sync
 *   "sampling" = "bucket" | "radix"          top-k / top-p selection: bucket histograms with the
 *                                            radix select as the exact fallback (default), or
 *                                            the radix select always
 * Takes effect for later launches; sessions re-capture their decode graph on the next decode. */
int rewb200_set_option(int slot, const char* key, const char* value);
/* Number of kernels this library has launched on the slot since init. */
int64_t rewb200_launch_count(int slot);

/* ---- device buffers -------------------------------------------------------
 * transferToDevice / transferToHost (src/rew/eager.nim:229-247), fromHost /
 * toHost (src/rew/eager.nim:360-377,558-595), BufferReleaser
 * (src/rew/buffer.nim:33,69-82: nil-safe, idempotent per handle). */
int rewb200_buffer_from_host(int slot, const void* src, int dtype, const int64_t* dims, int ndims,
                             rewb200_buffer** out);
int rewb200_buffer_alloc(int slot, int dtype, const int64_t* dims, int ndims, rewb200_buffer** out);
int rewb200_buffer_to_host(const rewb200_buffer* buf, void* dst, size_t nbytes);
int rewb200_buffer_info(const rewb200_buffer* buf, int* dtype, int64_t* dims, int* ndims);
void* rewb200_buffer_device_ptr(const rewb200_buffer* buf);
void rewb200_buffer_release(rewb200_buffer* buf);

/* ---- Tier A: per-op eager dispatch ---------------------------------------
 * The EagerBackend proc slot (src/rew/dispatch.nim:47-49,65-85) as a C call:
 * op name, operand buffers, stringly-typed attributes in the wire format of
 * src/rew/eager.nim:934-948 ("[1,2]" and "@[1, 2]" both accepted), one result.
 * Ops: add sub mul divide neg exp sqrt rsqrt logistic maximum reshape transpose
 * broadcastTo dotGeneral reduceSum reduceMax slice concat iota compare select
 * astype topK. */
int rewb200_dispatch(const char* op, rewb200_buffer* const* operands, int n_operands,
                     const char* const* attr_keys, const char* const* attr_vals, int n_attrs,
                     rewb200_buffer** out, int* n_out);

/* ---- Tier B: fused layer entry points --------------------------------------
 * Same argument meaning as the rew.nn forwards they stand behind. */

/* Linear.forward, src/rew/nn/linear.nim:43-49.  x [N,in], w [in,out], b [out]
 * (f32 when w is f32; f32 bias with bf16 x/w). y has x's dtype. */
int rewb200_linear(const rewb200_buffer* x, const rewb200_buffer* w, const rewb200_buffer* b,
                   rewb200_buffer** y);
/* rmsNorm, src/rew/nn/norm.nim:204-224. */
int rewb200_rmsnorm(const rewb200_buffer* x, const rewb200_buffer* gamma, float eps, rewb200_buffer** y);
/* LayerNorm.forward, src/rew/nn/norm.nim:41-84 (last axis). */
int rewb200_layernorm(const rewb200_buffer* x, const rewb200_buffer* gamma, const rewb200_buffer* beta,
                      float eps, rewb200_buffer** y);
/* initRotaryPositionEncoding tables, src/rew/nn/rope.nim:112-145: two f32
 * buffers [max_seq, head_dim], computed on the host exactly as the reference. */
int rewb200_rope_tables(int slot, int head_dim, int max_seq, double theta, rewb200_buffer** cos_out,
                        rewb200_buffer** sin_out);
/* RotaryPositionEncoding.forward, src/rew/nn/rope.nim:153-179.  x [...,S,hd]. */
int rewb200_rope(const rewb200_buffer* x, const rewb200_buffer* cos_t, const rewb200_buffer* sin_t,
                 int64_t offset, rewb200_buffer** y);
/* scaledDotProductAttention with the GQA head expansion folded in
 * (src/rew/nn/attention.nim:36-81, src/rew/nn/groupedqueryattention.nim:126-133).
 * q [B,nh,S,hd], k,v [B,kvh,L,hd] -> [B,nh,S,hd].  mask_kind 0 = makeCausalMask
 * as written (attention.nim:18-34), 1 = conventional causal. */
int rewb200_gqa_attention(const rewb200_buffer* q, const rewb200_buffer* k, const rewb200_buffer* v,
                          int causal, int mask_kind, rewb200_buffer** out);
/* Measurement aid: the same call, then the attention launch `iters` more times
 * between two CUDA events; *ms_per_call = their mean device time. */
int rewb200_gqa_attention_timed(const rewb200_buffer* q, const rewb200_buffer* k, const rewb200_buffer* v,
                                int causal, int mask_kind, int iters, float* ms_per_call, rewb200_buffer** out);
/* GatedFeedForward.forward, src/rew/nn/gated_ffn.nim:46-67.  x [N,d]. */
int rewb200_swiglu_ffn(const rewb200_buffer* x, const rewb200_buffer* gate_w, const rewb200_buffer* gate_b,
                       const rewb200_buffer* up_w, const rewb200_buffer* up_b, const rewb200_buffer* down_w,
                       const rewb200_buffer* down_b, rewb200_buffer** y);
/* Embedding.forward on token ids instead of one-hot rows
 * (src/rew/nn/embedding.nim:39-62).  ids int32 [N] -> [N,d]. */
int rewb200_embed_gather(const rewb200_buffer* ids, const rewb200_buffer* table, rewb200_buffer** y);
/* Router of DeepSeekMoE.forward, src/rew/models/deepseek.nim:132-138:
 * softmax over experts, top-k, renormalise.  x [N,d] f32/bf16, router_w [d,E],
 * router_b [E] -> weights f32 [N,k], indices int32 [N,k]. */
int rewb200_moe_route(const rewb200_buffer* x, const rewb200_buffer* router_w, const rewb200_buffer* router_b,
                      int top_k, rewb200_buffer** weights, rewb200_buffer** indices);

/* ---- stateful layer pieces ---------------------------------------------------
 * For a backend-aware GroupedQueryAttention.forward / DeepSeekMoE.forward / generate loop written against
 * single layers instead of the whole-model engine below. */
typedef struct rewb200_kv rewb200_kv;
typedef struct rewb200_experts rewb200_experts;
typedef struct rewb200_sampler rewb200_sampler;
/* KvCache (src/rew/nn/kv_cache.nim:13-24): K and V of one attention layer, [batch, kv_heads, max_len,
 * head_dim], f32 or bf16, with one length for all sequences.  `append` (kv_cache.nim:47-77) is done by
 * rewb200_qkv_rope_kvappend in place instead of by concatenation. */
int rewb200_kv_create(int slot, int dtype, int batch, int kv_heads, int head_dim, int max_len, rewb200_kv** out);
void rewb200_kv_free(rewb200_kv* kv);
int rewb200_kv_length(const rewb200_kv* kv);   /* KvCache.length; -1 for NULL */
int rewb200_kv_reset(rewb200_kv* kv);
/* First half of GroupedQueryAttention.forward with a cache (src/rew/nn/groupedqueryattention.nim:94-122):
 * q / k / v Linear of x [batch, S, embedDim], RoPE of q and k at offset = cache length (tables from
 * rewb200_rope_tables), K and V appended to the cache.  q_out [batch, S, heads*head_dim].  Biases may be NULL. */
int rewb200_qkv_rope_kvappend(const rewb200_buffer* x, const rewb200_buffer* wq, const rewb200_buffer* bq,
                              const rewb200_buffer* wk, const rewb200_buffer* bk, const rewb200_buffer* wv,
                              const rewb200_buffer* bv, const rewb200_buffer* cos_t, const rewb200_buffer* sin_t,
                              rewb200_kv* kv, rewb200_buffer** q_out);
/* Second half (groupedqueryattention.nim:126-137 before outProj): the queries of the last append attend over
 * everything cached so far; q and out are [batch, S, heads*head_dim]; mask_kind as rewb200_gqa_attention. */
int rewb200_gqa_attention_cached(const rewb200_buffer* q, const rewb200_kv* kv, int causal, int mask_kind,
                                 rewb200_buffer** out);
/* The routed experts of a DeepSeekMoE layer (src/rew/models/deepseek.nim:36-52,74-78): n_experts triples of
 * gate / up [hidden, intermediate] and down [intermediate, hidden] weights (device buffers, all f32 or all
 * bf16) and optional f32 biases (array or entry NULL = zero), copied once into the fused device layout. */
int rewb200_experts_create(int slot, int n_experts, const rewb200_buffer* const* gate_w, const rewb200_buffer* const* gate_b,
                           const rewb200_buffer* const* up_w, const rewb200_buffer* const* up_b,
                           const rewb200_buffer* const* down_w, const rewb200_buffer* const* down_b, rewb200_experts** out);
void rewb200_experts_free(rewb200_experts* h);
/* DeepSeekMoE.forward after the router (deepseek.nim:140-144): y[t] = sum_j weights[t][j] *
 * expert_{indices[t][j]}(x[t]).  x [tokens, hidden]; weights f32 and indices int32 [tokens, k] as
 * rewb200_moe_route returns them; y has x's shape and dtype.  bf16: tokens sorted by expert, two grouped
 * GEMMs (SwiGLU in the first one's epilogue; tcgen05 for groups of more than 64 rows); f32: every expert on
 * every token, masked, as the reference computes it. */
int rewb200_moe_experts(const rewb200_experts* h, const rewb200_buffer* x, const rewb200_buffer* weights,
                        const rewb200_buffer* indices, rewb200_buffer** y);
/* Sampling state of `batch` sequences (GenerationConfig + Key of generate, src/rew/infer/generate.nim:12-58,
 * 231-265): per-sequence Threefry key (initKey(seed), folded with the step after every token), step counter
 * and the tokens seen so far (for repetitionPenalty), all on the device.  max_tokens bounds prompt +
 * generated tokens per sequence.  seeds: host uint64 [batch] or NULL (key 0). */
int rewb200_sampler_create(int slot, int batch, int vocab, int max_tokens, float temperature, int top_k, float top_p,
                           float min_p, float repetition_penalty, int do_sample, const uint64_t* seeds, rewb200_sampler** out);
void rewb200_sampler_free(rewb200_sampler* s);
/* Adds n_per_row tokens per sequence (host int32 [batch, n_per_row], e.g. the prompt) to the tokens seen. */
int rewb200_sampler_observe(rewb200_sampler* s, const int32_t* ids, int n_per_row);
/* lmHead + lastLogits + applySamplingConfig + sampleGreedy / sampleTopK / sampleTopP (generate.nim:92-190):
 * x [batch, d] (the last position's hidden state), lm_w [d, vocab], lm_b f32 [vocab] or NULL.  sampler NULL
 * = greedy argmax, first maximum.  next_ids host int32 [batch]; logits_out host f32 [batch, vocab] or NULL. */
int rewb200_lmhead_sample(const rewb200_buffer* x, const rewb200_buffer* lm_w, const rewb200_buffer* lm_b,
                          rewb200_sampler* sampler, int32_t* next_ids, float* logits_out);

/* ---- NF4 weight-only Linear (QLoRA base projection) -------------------------
 * nf4Quantize / nf4Dequantize (src/rew/quantize/codecs.nim:13-70) and
 * QloraLinear (src/rew/nn/lora.nim:173-191,331-431).  The reference dequantises
 * the frozen weight once on the host and multiplies in fp32; here the 4-bit
 * codes stay in device memory (0.5625 bytes per weight with the scales) and are
 * dequantised inside the matrix-vector kernel. */
/* initQloraLinearFromF32's quantisation step: w [in,out] f32 or bf16 on the
 * device, blocks of 64 along the flat index; in and out must be multiples of 64. */
int rewb200_nf4_pack(const rewb200_buffer* w, rewb200_nf4** out);
void rewb200_nf4_free(rewb200_nf4* h);
int rewb200_nf4_info(const rewb200_nf4* h, int64_t* in_features, int64_t* out_features);
/* The reference's representation of the same weight: packed [in*out/2] bytes
 * (even flat index in the low nibble) and scales [in*out/64], both on the host. */
int rewb200_nf4_unpack(const rewb200_nf4* h, uint8_t* packed, float* scales);
/* nf4Dequantize into a new bf16 [in,out] device buffer. */
int rewb200_nf4_dequantize(const rewb200_nf4* h, rewb200_buffer** w_out);
/* QloraLinear.forward (lora.nim:410-431): x [...,in] bf16 -> [...,out] bf16 =
 * x @ dequant(w) + bias + scaling * (x @ A^T) @ B^T.  bias f32 [out] or NULL;
 * A f32 [rank,in] and B f32 [out,rank], or both NULL for the base projection. */
int rewb200_qlora_linear(const rewb200_buffer* x, const rewb200_nf4* h, const rewb200_buffer* bias,
                         const rewb200_buffer* A, const rewb200_buffer* B, float scaling, rewb200_buffer** y);

/* Linear for callers that cannot allocate device memory (no counterpart in the
 * reference, which always allocates through its PJRT client).  Same math as
 * rewb200_linear for bf16 with M <= 32: y[M,N] = x[M,K] @ w[K,N] + bias, but on
 * raw device pointers the caller owns and with the split-K partial sums kept in
 * a fixed 8 MiB array inside the library image instead of pool memory, so the
 * call performs no cudaMalloc / cudaFree / pool allocation.  Meant for hosts
 * whose own allocator holds the whole device heap, and for sections where the
 * device-wide synchronisation of cudaMalloc is not acceptable.  Sizes with
 * M*N*4 bytes above 8 MiB are rejected.  Every call shares the one array:
 * calls that overlap on the GPU race; calls on one slot are stream-ordered.
 * rewb200_init resolves the array's address on each device it opens and loads
 * the kernels this call launches (the driver allocates the array when it loads
 * that code), so the call itself loads nothing.  The GEMM is the one the slot's
 * "linear" option selects (tcgen05 by default).  bias may be NULL. */
int rewb200_linear_noalloc(int slot, const void* x_bf16, const void* w_bf16, const float* bias, void* y_bf16,
                           int64_t M, int64_t K, int64_t N);

/* ---- model + generate ------------------------------------------------------
 * LlamaForCausalLM / DeepSeekForCausalLM (src/rew/models/llama.nim:13-44,
 * src/rew/models/deepseek.nim:20-63) as one object with fused device layouts. */
typedef struct rewb200_config {
  int32_t vocab, d_model, n_layers, n_heads, n_kv_heads, head_dim, ffn, max_seq;
  double theta;
  float eps;
  int32_t norm_kind;    /* 0 rmsNorm math, 1 LayerNorm (what LlamaDecoderLayer calls) */
  int32_t mask_kind;    /* 0 makeCausalMask as written, 1 conventional causal */
  int32_t n_routed, n_shared, top_k, moe_ffn, first_dense; /* n_routed == 0: dense Llama block */
  int32_t dtype;        /* REWB200_F32 or REWB200_BF16: weight/activation storage */
  int32_t tp_rank, tp_size; /* tensor parallel shard of heads / FFN columns */
  int32_t ep_rank, ep_size; /* expert parallel shard of routed experts */
  int32_t weight_quant; /* 0: weights in `dtype`; 1: the decoder blocks' Linear weights as NF4 codes in
                         * blocks of 64 (nf4Quantize, src/rew/quantize/codecs.nim:31-57), quantised at
                         * rewb200_model_finalize; needs dtype bf16 and a dense (non-MoE) model */
} rewb200_config;

int rewb200_model_create(int slot, const rewb200_config* cfg, rewb200_model** out);
void rewb200_model_free(rewb200_model* m);
/* Number and canonical order of the logical tensors (see rew_b200/weights.py):
 * embed; per layer ln1.gamma ln1.beta q.w q.b k.w k.b v.w v.b o.w o.b ln2.gamma
 * ln2.beta then gate.w gate.b up.w up.b down.w down.b (dense) or router.w
 * router.b + 6 per expert (shared first); norm.gamma norm.beta lm_head.w lm_head.b. */
int64_t rewb200_model_tensor_count(const rewb200_model* m);
/* Uploads logical tensor `index` from host f32 data of the FULL (unsharded)
 * shape; the library slices for tp/ep rank, converts and fuses. */
int rewb200_model_set_tensor(rewb200_model* m, int64_t index, const float* host, int64_t numel);
/* The sharding vocabulary of src/rew/sharding.nim for this model: where logical tensor `index` lives on this
 * rank.  global_shape / local_shape / offsets (ndims entries each, at most 2) follow shardLayout's block rule
 * (sharding.nim:255-270: localShape[dim] = shape[dim] / factor, offset = coord * local) on the tensor-parallel
 * axis: the q / k / v / gate / up / lm_head weights are PartitionSpec(["", "tp"]) (column-parallel,
 * *partitioned_dim = 1), their biases (["tp"]), the o / down weights (["tp", ""]) (row-parallel, dim 0), the rest
 * replicated (-1).  A routed expert that another expert-parallel rank owns has local_shape all zero. */
int rewb200_model_tensor_layout(const rewb200_model* m, int64_t index, int* ndims, int64_t* global_shape,
                                int64_t* local_shape, int64_t* offsets, int* partitioned_dim);
/* fromHostShards (src/rew/eager.nim:427-505) for one tensor: uploads exactly this rank's block (host f32 of
 * local_shape, at offsets; both must equal what rewb200_model_tensor_layout reports), so a sharded checkpoint
 * goes shard -> rank without the full tensor ever being assembled on a host. */
int rewb200_model_set_tensor_shard(rewb200_model* m, int64_t index, const float* host_local, const int64_t* local_shape,
                                   const int64_t* offsets, int ndims);
/* Device-side N(0,std) weights, zero biases, unit gammas (synthetic benchmarks). */
int rewb200_model_init_random(rewb200_model* m, uint64_t seed, float std);
int rewb200_model_finalize(rewb200_model* m);
int64_t rewb200_model_weight_bytes(const rewb200_model* m);

/* A batch of sequences with a paged KV cache (KvCache, src/rew/nn/kv_cache.nim:13-77;
 * PagedKvCache, src/rew/infer/generate.nim:63-88). */
int rewb200_session_create(rewb200_model* m, int batch, int max_len, rewb200_session** out);
void rewb200_session_free(rewb200_session* s);
int rewb200_session_reset(rewb200_session* s);
/* Feeds `S` new tokens per sequence (host int32 [batch,S]) at the current
 * offset, appends K/V, returns greedy next ids (host int32 [batch]) and, when
 * logits_out != NULL, the last-position logits (host f32 [batch,vocab]). */
int rewb200_session_forward(rewb200_session* s, const int32_t* ids, int S, int32_t* next_ids, float* logits_out);
/* `n_steps` greedy decode steps entirely on the device starting from the ids
 * the last forward produced; host out_ids [batch,n_steps]. */
int rewb200_session_decode(rewb200_session* s, int n_steps, int32_t* out_ids, float* last_logits);
/* generate (src/rew/infer/generate.nim:231-265), greedy, batched: prompt host
 * int32 [batch,S]; out_ids host int32 [batch,n_new]; stops early when eos >= 0
 * and every sequence has produced it. last_logits optional [batch,vocab]. */
int rewb200_generate(rewb200_session* s, const int32_t* prompt, int S, int n_new, int eos, int32_t* out_ids,
                     float* last_logits);
/* The same with GenerationConfig.stopTokenIds (generate.nim:21,263): a sequence ends with the first token
 * that is in stop_ids (host int32 [n_stop]) or equals eos (ignored when negative); ids after it are -1. */
int rewb200_generate_stop(rewb200_session* s, const int32_t* prompt, int S, int n_new, int eos, const int32_t* stop_ids,
                          int n_stop, int32_t* out_ids, float* last_logits);
/* ---- paged lanes: continuous batching --------------------------------------
 * PagedKvCache (src/rew/infer/generate.nim:63-88: blockSize, numBlocks,
 * freeBlocks) made operational.  The session owns `num_blocks` KV blocks of 64
 * tokens shared by `lanes` sequences; block 0 is the scratch block idle lanes
 * write to, the others are handed out on demand as a lane's sequence grows and
 * return to the free list when the lane is released.  Sequences join and leave
 * between decode steps, each with its own length; the decode step is the same
 * captured CUDA graph over all lanes (idle lanes report -1).  Not available on
 * tensor- or expert-parallel models. */
int rewb200_session_create_paged(rewb200_model* m, int lanes, int max_len, int num_blocks, rewb200_session** out);
/* Free blocks left in the pool (-1 when the session is not paged). */
int rewb200_session_free_blocks(const rewb200_session* s);
/* Tokens in the cache of an active lane (-1: idle lane or bad argument). */
int rewb200_lane_length(const rewb200_session* s, int lane);
/* Starts a sequence in an idle lane: reserves blocks for the S prompt tokens
 * (host int32 [S]), prefills that lane alone and returns its first new token.
 * With sampling set, the lane's key restarts from initKey(seed). */
int rewb200_lane_admit(rewb200_session* s, int lane, const int32_t* ids, int S, uint64_t seed, int32_t* next_id);
/* n_steps decode steps for every active lane; out_ids host int32
 * [lanes,n_steps], -1 for idle lanes.  Fails without side effects when the pool
 * cannot cover the growth of every active lane ("out of free blocks"). */
int rewb200_lanes_step(rewb200_session* s, int n_steps, int32_t* out_ids);
/* Ends a lane's sequence and returns its blocks to the pool (idempotent). */
int rewb200_lane_release(rewb200_session* s, int lane);

/* GenerationConfig sampling on the device (src/rew/infer/generate.nim:12-58 for
 * the fields and their checks, :92-159 sampleTopK / sampleTopP / sampleGreedy,
 * :192-218 applySamplingConfig, :231-265 the loop).  After this call forward,
 * decode and rewb200_generate pick each next token as generate() does:
 * repetition penalty over prompt + generated tokens, temperature, min-p, then
 * greedy (do_sample == 0 or temperature <= 0.01), top-k (top_k > 0, at most
 * 1024) or top-p.  Sequence b draws from Key = initKey(seeds[b]) (seeds NULL:
 * all 0, the reference's default key) and folds the step number in after every
 * token (src/rew/rng.nim:33-80).  Keys and step counters restart at
 * rewb200_session_reset, hence at every rewb200_generate.  On a paged session
 * call it before admitting lanes (each rewb200_lane_admit restarts its lane
 * from its own seed).  Not available on a tensor-parallel model. */
int rewb200_session_set_sampling(rewb200_session* s, float temperature, int top_k, float top_p, float min_p,
                                 float repetition_penalty, int do_sample, const uint64_t* seeds);
/* Back to plain greedy argmax. */
int rewb200_session_clear_sampling(rewb200_session* s);
/* logProbOf (generate.nim:220-227) of the first n tokens sampled since the last
 * reset, host f32 [batch,n]. */
int rewb200_session_logprobs(rewb200_session* s, int n, float* out);
/* Device-time of the last forward / decode call in milliseconds (CUDA events). */
int rewb200_session_last_ms(const rewb200_session* s, float* prefill_ms, float* decode_ms);
/* Kernels in one captured decode step (0 before the first decode). */
int rewb200_session_graph_kernels(const rewb200_session* s);
/* Test aid (option record_routing): the expert ids MoE layer `moe_layer` (0-based among the MoE layers) chose for
 * the `rows` tokens of the session's last forward, host int32 [rows, top_k], in the router's order. */
int rewb200_session_routing(rewb200_session* s, int moe_layer, int32_t* topi_out, int64_t rows);
/* Measurement aid: one decode step issued as plain launches with a CUDA event after every category of
 * launches; ms_by_category (host, n >= 11 floats) receives the device time per category, summed over the
 * layers: 0 embedding + first norm, 1 q|k|v Linear, 2 bias + RoPE + cache write, 3 attention, 4 o Linear,
 * 5 residual + norm after attention (with the tensor-parallel exchange), 6 gate|up Linear, 7 down Linear,
 * 8 routed experts (MoE), 9 residual + norm after the FFN (with the exchange), 10 lm_head + next-token.  The
 * events keep kernels from overlapping their neighbours, so the sum exceeds a replayed step; the step
 * advances the session by one token like rewb200_session_decode(s, 1, ...). */
int rewb200_session_trace_step(rewb200_session* s, float* ms_by_category, int n);
/* Measurement aid: runs only the Linear launches of one decode step (same
 * buffers, tiles and split-K as the real step) `iters` times between CUDA
 * events; reports milliseconds, algorithmic bytes and launches per step. */
int rewb200_session_profile_linears(rewb200_session* s, int iters, float* ms_per_step, int64_t* bytes_per_step,
                                    int* launches_per_step);
/* Full no-cache forward, logits for every position, as LlamaForCausalLM.forward
 * (src/rew/models/llama.nim:131-140): ids host [batch,S] -> logits host [batch,S,vocab]. */
int rewb200_model_forward_all(rewb200_session* s, const int32_t* ids, int S, int64_t offset, int causal,
                              float* logits_out);

/* ---- tensor / expert parallel communication -------------------------------
 * allReduce / allToAll (src/rew/ops/distributed.nim:62-83,106-128) executed
 * with NCCL over NVLink; one process per GPU. */
int rewb200_comm_unique_id(void* id128);                  /* 128 bytes, created on rank 0 */
int rewb200_comm_init(int slot, const void* id128, int rank, int world);
int rewb200_comm_allreduce_f32(int slot, void* device_ptr, int64_t n);
/* allToAll with equal counts (src/rew/ops/distributed.nim:106-128): bytes [p*bytes_per_peer, (p+1)*bytes_per_peer)
 * of the device send buffer go to rank p, and rank p's block for this rank lands at the same offset of the
 * device receive buffer.  Waits for completion and reports NCCL's asynchronous errors. */
int rewb200_comm_alltoall(int slot, const void* send_device, void* recv_device, int64_t bytes_per_peer);
/* Peer heap: exchange memory that the other ranks of the node write into directly over NVLink (plain peer
 * stores from inside this library's kernels; nothing is read from a peer and no library kernel is handed a
 * peer pointer).  Each rank allocates its heap and exports a 64-byte CUDA IPC handle; after the host has
 * gathered every rank's handle (rank order, world*64 bytes), attach maps the peers.  Sessions created
 * afterwards use it for
 *   - the tensor-parallel all-reduce (src/rew/ops/distributed.nim:62-83).  Steps up to 64 rows with
 *     rows*d_model*(4 for bf16 models, 8 for f32) <= allreduce_bytes: fused into the residual+norm kernel (each
 *     thread stores its partial into every rank's heap as 16-byte lines that carry the payload and a flag
 *     together, polls with a bound for the peers' lines in its own heap and sums the
 *     partials in rank order).  Larger steps whose partial fits twice into alltoall_bytes: two-shot (every rank
 *     stores slice p of its partial into rank p's heap, rank p stores the sum of the slices into every rank's
 *     heap).  Anything else goes through NCCL (bf16 payload on bf16 models);
 *   - the expert-parallel all-to-all (src/rew/ops/distributed.nim:106-128) whenever the slot arrays of a
 *     step (pairs*world rows of d_model activations, their expert ids and the f32 results) fit into
 *     alltoall_bytes: dispatch and return kernels store the occupied rows straight into the owner's heap
 *     and hand over the pair counts on the device, so neither a count exchange through the host nor
 *     padding crosses NVLink.  Larger steps go through NCCL send/recv.
 * Either size may be 0 (alltoall_bytes is one bulk region that serves whichever of the two a model uses: a
 * model is never both tensor- and expert-parallel).  The heap holds 16 KiB + 2*world*allreduce_bytes +
 * alltoall_bytes. */
int rewb200_comm_peer_alloc(int slot, int64_t allreduce_bytes, int64_t alltoall_bytes, void* handle64);
int rewb200_comm_peer_attach(int slot, const void* handles_all);
/* Free every session of the slot first: a captured decode graph keeps the communicator in use and
 * NCCL waits for it. */
int rewb200_comm_destroy(int slot);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif
