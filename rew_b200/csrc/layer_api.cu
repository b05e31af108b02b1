// Tier-B entry points for the parts of the decoder that hold state or take many weights: a backend-aware
// rew.nn forward can be written against these without going through the whole-model engine.
//   rewb200_kv_*               KvCache (src/rew/nn/kv_cache.nim:13-24,47-77) written in place
//   rewb200_qkv_rope_kvappend  first half of GroupedQueryAttention.forward with a cache
//                              (src/rew/nn/groupedqueryattention.nim:94-122): q/k/v Linear, RoPE at the
//                              cache length, K and V appended
//   rewb200_gqa_attention_cached  second half: attention of the new queries over the cache
//   rewb200_experts_* / rewb200_moe_experts  the routed experts of DeepSeekMoE.forward
//                              (src/rew/models/deepseek.nim:74-78,140-144) for already-routed tokens
//   rewb200_sampler_* / rewb200_lmhead_sample  lm_head + sampleGreedy / sampleTopK / sampleTopP
//                              (src/rew/infer/generate.nim:92-159,172-190)
// All of them run the engine's kernels; nothing here is a second implementation.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

using namespace rewb;

namespace rewb {
int moe_group_local_launch(Ctx* c, const void* x, int dtype, const int* topi, int64_t tokens, int k, int64_t d, int n_experts,
                           int* offsets, void* xs, int* pair_pos);
int moe_reset_launch(Ctx* c, int* cursor, int n_cursor, int* count, int n_count, int* meta, int n_meta);
int moe_dispatch_launch(Ctx* c, const void* x, int dtype, const int* topi, int64_t tokens, int k, int64_t d,
                        int experts_per_rank, int capacity, int* cursor, void* send_x, int* send_meta, int* pair_slot);
int moe_group_launch(Ctx* c, const void* recv_x, int dtype, const int* recv_meta, int n_slots, int64_t d, int n_experts,
                     int* count, int* offsets, int* cursor2, void* xs, int* slot_pos);
int moe_return_launch(Ctx* c, const float* ys, const int* slot_pos, int n_slots, int64_t d, float* ret);
int moe_combine_launch(Ctx* c, const float* back, const int* pair_slot, const float* topw, int64_t tokens, int k, int64_t d,
                       float* out, int accumulate);
int sample_launch(Ctx* c, const float* logits, float* work, int64_t B, int64_t V, int* hist, int* hist_len, int hist_cap,
                  uint32_t* keys, int* steps, int* next, float* logprob, int logprob_cap, float temperature, int top_k,
                  float top_p, float min_p, float rep_penalty, int do_sample, const int* active);

namespace {

// dst[r][map(c)] = src[r][c] with map(c) = (c / gran) * gstride + c % gran + off; src f32 or bf16, dst f32 or bf16
template <typename TS, typename TD>
__global__ void place_cols_kernel(const TS* src, int64_t rows, int64_t cols, TD* dst, int64_t ldd, int64_t gran, int64_t gstride,
                                  int64_t off) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const int64_t r = i / cols, c = i % cols;
  float v;
  if constexpr (sizeof(TS) == 2) v = __bfloat162float(src[i]);
  else v = src[i];
  const int64_t dc = (c / gran) * gstride + (c % gran) + off;
  if constexpr (sizeof(TD) == 2) dst[r * ldd + dc] = __float2bfloat16_rn(v);
  else dst[r * ldd + dc] = v;
}

int place_cols(Ctx* c, const rewb200_buffer* src, int64_t rows, int64_t cols, void* dst, int dst_dtype, int64_t ldd, int64_t gran,
               int64_t gstride, int64_t off) {
  const int64_t n = rows * cols;
  if (n == 0) return REWB200_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  const bool s16 = src->dtype == REWB200_BF16, d16 = dst_dtype == REWB200_BF16;
  RB_REQUIRE(s16 || src->dtype == REWB200_F32, "weights must be f32 or bf16");
  if (s16 && d16) place_cols_kernel<bf16, bf16><<<blocks, 256, 0, c->stream>>>((const bf16*)src->ptr, rows, cols, (bf16*)dst, ldd, gran, gstride, off);
  else if (s16) place_cols_kernel<bf16, float><<<blocks, 256, 0, c->stream>>>((const bf16*)src->ptr, rows, cols, (float*)dst, ldd, gran, gstride, off);
  else if (d16) place_cols_kernel<float, bf16><<<blocks, 256, 0, c->stream>>>((const float*)src->ptr, rows, cols, (bf16*)dst, ldd, gran, gstride, off);
  else place_cols_kernel<float, float><<<blocks, 256, 0, c->stream>>>((const float*)src->ptr, rows, cols, (float*)dst, ldd, gran, gstride, off);
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

// f32 parity path of the experts: out[t] (+)= w_e(t) * y[t] with w_e(t) = sum_j topw[t][j] * (topi[t][j] == e)
// (routedWeightForExpert, src/rew/models/deepseek.nim:114-120,140-144)
__global__ void expert_acc_kernel(const float* y, const float* topw, const int* topi, int k, int e, int64_t rows, int64_t d,
                                  float* out, int accumulate) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const int64_t t = i / d;
  float w = 0.f;
  for (int j = 0; j < k; ++j) w += topw[t * k + j] * (topi[t * k + j] == e ? 1.f : 0.f);
  const float v = y[i] * w;
  out[i] = accumulate ? out[i] + v : v;
}

// Scratch of one call from the stream-ordered pool; freed (stream-ordered) when the call returns.
struct Pool {
  Ctx* c;
  std::vector<void*> ptrs;
  explicit Pool(Ctx* ctx) : c(ctx) {}
  ~Pool() {
    for (void* p : ptrs) cudaFreeAsync(p, c->stream);
  }
  template <typename T>
  int get(T** out, size_t bytes) {
    void* p = nullptr;
    RB_CUDA(cudaMallocAsync(&p, std::max<size_t>(bytes, 256), c->stream));
    ptrs.push_back(p);
    *out = (T*)p;
    return REWB200_OK;
  }
};

}  // namespace
}  // namespace rewb

// ---------------------------------------------------------------- KvCache

struct rewb200_kv {
  int slot = 0, dtype = 0, B = 0, kvh = 0, hd = 0, max_len = 0;
  int len = 0;       // tokens held (all sequences advance together, as KvCache.length)
  int last_S = 0;    // tokens of the last append; their queries attend from position len - last_S
  void *k = nullptr, *v = nullptr;  // [B][kvh][max_len][hd]
  int* d_pos = nullptr;             // [B] position of the last append's first token
  CUtensorMap tmK, tmV;
};

extern "C" {

int rewb200_kv_create(int slot, int dtype, int batch, int kv_heads, int head_dim, int max_len, rewb200_kv** out) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(out, "initKvCache: NULL output");
  RB_REQUIRE(dtype == REWB200_F32 || dtype == REWB200_BF16, "initKvCache: dtype must be f32 or bf16");
  RB_REQUIRE(batch > 0 && kv_heads > 0 && head_dim > 0 && max_len > 0, "initKvCache: batch, heads, headDim and maxLen must be positive");
  RB_REQUIRE(head_dim % 2 == 0, "initKvCache: headDim must be even (RoPE pairs)");
  RB_REQUIRE(dtype == REWB200_F32 || head_dim == 64 || head_dim == 128, "bf16 caches support head_dim 64 and 128");
  RB_CUDA(cudaSetDevice(c->device));
  rewb200_kv* kv = new rewb200_kv();
  kv->slot = slot; kv->dtype = dtype; kv->B = batch; kv->kvh = kv_heads; kv->hd = head_dim; kv->max_len = max_len;
  const size_t bytes = (size_t)batch * kv_heads * max_len * head_dim * dtype_size(dtype);
  cudaError_t e = cudaMalloc(&kv->k, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->v, bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&kv->d_pos, batch * sizeof(int));
  if (e == cudaSuccess) e = cudaMemsetAsync(kv->k, 0, bytes, c->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(kv->v, 0, bytes, c->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(kv->d_pos, 0, batch * sizeof(int), c->stream);
  int st = e == cudaSuccess ? REWB200_OK : fail(std::string("initKvCache: ") + cudaGetErrorString(e));
  if (st == REWB200_OK && dtype == REWB200_BF16) {
    const uint64_t rows = (uint64_t)batch * kv_heads * max_len;
    st = make_tmap_2d_bf16(&kv->tmK, kv->k, head_dim, rows, (uint64_t)head_dim * 2, 64, 64);
    if (st == REWB200_OK) st = make_tmap_2d_bf16(&kv->tmV, kv->v, head_dim, rows, (uint64_t)head_dim * 2, 64, 64);
  }
  if (st != REWB200_OK) {
    cudaFree(kv->k);
    cudaFree(kv->v);
    cudaFree(kv->d_pos);
    delete kv;
    return st;
  }
  *out = kv;
  return REWB200_OK;
}

void rewb200_kv_free(rewb200_kv* kv) {
  if (!kv) return;
  Ctx* c = ctx_get(kv->slot);
  if (c) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
  }
  cudaFree(kv->k);
  cudaFree(kv->v);
  cudaFree(kv->d_pos);
  delete kv;
}

int rewb200_kv_length(const rewb200_kv* kv) { return kv ? kv->len : -1; }

int rewb200_kv_reset(rewb200_kv* kv) {
  RB_REQUIRE(kv, "KvCache: NULL handle");
  kv->len = 0;
  kv->last_S = 0;
  return REWB200_OK;
}

int rewb200_qkv_rope_kvappend(const rewb200_buffer* x, const rewb200_buffer* wq, const rewb200_buffer* bq,
                              const rewb200_buffer* wk, const rewb200_buffer* bk, const rewb200_buffer* wv,
                              const rewb200_buffer* bv, const rewb200_buffer* cos_t, const rewb200_buffer* sin_t,
                              rewb200_kv* kv, rewb200_buffer** q_out) {
  RB_REQUIRE(x && wq && wk && wv && cos_t && sin_t && kv && q_out, "GroupedQueryAttention.forward: NULL argument");
  RB_REQUIRE(x->ndims == 3, "GroupedQueryAttention.forward: query must be rank 3 [batch, seqLen, embedDim]");
  const int64_t B = x->dims[0], S = x->dims[1], d = x->dims[2];
  const int dt = x->dtype;
  RB_REQUIRE(dt == kv->dtype && wq->dtype == dt && wk->dtype == dt && wv->dtype == dt, "GroupedQueryAttention.forward: dtypes differ");
  RB_REQUIRE(B == kv->B, "KvCache.append: batch " + std::to_string(B) + " does not match the cache's " + std::to_string(kv->B));
  RB_REQUIRE(wq->ndims == 2 && wk->ndims == 2 && wv->ndims == 2 && wq->dims[0] == d && wk->dims[0] == d && wv->dims[0] == d,
             "GroupedQueryAttention.forward: projection weights must be [embedDim, out]");
  const int64_t nq = wq->dims[1], nkv = wk->dims[1];
  RB_REQUIRE(nkv == (int64_t)kv->kvh * kv->hd && wv->dims[1] == nkv && nq % kv->hd == 0 && (nq / kv->hd) % kv->kvh == 0,
             "GroupedQueryAttention.forward: projection widths do not match the cache's heads");
  RB_REQUIRE(kv->len + S <= kv->max_len, "KvCache.append: total length " + std::to_string(kv->len + S) + " exceeds maxLen " +
                                             std::to_string(kv->max_len));
  RB_REQUIRE(cos_t->ndims == 2 && cos_t->dims[1] == kv->hd && sin_t->ndims == 2 && sin_t->dims[1] == kv->hd &&
                 cos_t->dtype == REWB200_F32 && sin_t->dtype == REWB200_F32,
             "RotaryPositionEncoding.forward: tables must be f32 [maxSeqLen, headDim]");
  RB_REQUIRE(kv->len + S <= cos_t->dims[0], "RotaryPositionEncoding.forward: position " + std::to_string(kv->len + S) +
                                                " exceeds maxSeqLen " + std::to_string(cos_t->dims[0]));
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t rows = B * S, ntot = nq + 2 * nkv;
  Pool pool(c);
  float* fused = nullptr;  // [rows][nq | nkv | nkv] f32, biases added
  RB_TRY(pool.get(&fused, (size_t)rows * ntot * sizeof(float)));
  // the three projections through the same entry point the Linear layer uses, then side by side in one row
  const rewb200_buffer* ws[3] = {wq, wk, wv};
  const rewb200_buffer* bs[3] = {bq, bk, bv};
  const int64_t widths[3] = {nq, nkv, nkv}, offs[3] = {0, nq, nq + nkv};
  rewb200_buffer x2 = *x;  // [rows, d] view
  x2.ndims = 2;
  x2.dims[0] = rows;
  x2.dims[1] = d;
  x2.owned = false;
  for (int i = 0; i < 3; ++i) {
    rewb200_buffer* y = nullptr;
    RB_TRY(rewb200_linear(&x2, ws[i], bs[i], &y));
    const int st = place_cols(c, y, rows, widths[i], fused, REWB200_F32, ntot, widths[i], widths[i], offs[i]);
    rewb200_buffer_release(y);
    RB_TRY(st);
  }
  const int64_t qd[3] = {B, S, nq};
  RB_TRY(buffer_new(c, dt, qd, 3, q_out));
  std::vector<int> pos((size_t)B, kv->len);
  RB_CUDA(cudaMemcpyAsync(kv->d_pos, pos.data(), B * sizeof(int), cudaMemcpyHostToDevice, c->stream));
  RB_CUDA(cudaStreamSynchronize(c->stream));  // `pos` is pageable host memory
  QkvPostArgs qa;
  memset(&qa, 0, sizeof(qa));
  qa.partial = fused;
  qa.nsplit = 1;
  qa.split_stride = rows * ntot;
  qa.bias = nullptr;
  qa.cosT = (const float*)cos_t->ptr;
  qa.sinT = (const float*)sin_t->ptr;
  qa.pos0 = kv->d_pos;
  qa.S = (int)S;
  qa.rope_shift = 0;
  qa.kv_capacity = kv->max_len;
  qa.nh = (int)(nq / kv->hd);
  qa.kvh = kv->kvh;
  qa.hd = kv->hd;
  qa.max_seq = (int)cos_t->dims[0];
  qa.q_out = (*q_out)->ptr;
  qa.act_dtype = dt;
  qa.kv.k = kv->k;
  qa.kv.v = kv->v;
  qa.kv.block_table = nullptr;
  qa.kv.page = 64;
  qa.kv.kvh = kv->kvh;
  qa.kv.hd = kv->hd;
  qa.kv.contiguous_len = kv->max_len;
  qa.kv.dtype = dt;
  qa.status = c->d_status;
  const bool pdl = c->use_pdl;
  c->use_pdl = false;  // the predecessors are plain launches of this call
  const int st = qkv_post_launch(c, qa, B);
  c->use_pdl = pdl;
  RB_TRY(st);
  kv->len += (int)S;
  kv->last_S = (int)S;
  return REWB200_OK;
}

int rewb200_gqa_attention_cached(const rewb200_buffer* q, const rewb200_kv* kv, int causal, int mask_kind,
                                 rewb200_buffer** out) {
  RB_REQUIRE(q && kv && out, "scaledDotProductAttention: NULL argument");
  RB_REQUIRE(q->ndims == 3 && q->dims[0] == kv->B && q->dims[2] % kv->hd == 0,
             "scaledDotProductAttention: q must be [batch, seqLen, heads * headDim] of the cache's batch");
  RB_REQUIRE(q->dtype == kv->dtype, "scaledDotProductAttention: dtypes differ");
  const int64_t B = q->dims[0], S = q->dims[1], nq = q->dims[2];
  const int nh = (int)(nq / kv->hd);
  RB_REQUIRE(nh % kv->kvh == 0, "initGroupedQueryAttention: numHeads " + std::to_string(nh) + " must be divisible by numKVHeads " +
                                    std::to_string(kv->kvh));
  RB_REQUIRE(S == kv->last_S && kv->len >= S, "the queries must be those of the cache's last append");
  Ctx* c = ctx_get(q->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(buffer_new(c, q->dtype, q->dims, 3, out));
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q->ptr;
  a.q_sb = S * nq; a.q_ss = nq; a.q_sh = kv->hd;
  a.out = (*out)->ptr;
  a.o_sb = a.q_sb; a.o_ss = a.q_ss; a.o_sh = a.q_sh;
  a.kv.k = kv->k;
  a.kv.v = kv->v;
  a.kv.block_table = nullptr;
  a.kv.page = 64;
  a.kv.kvh = kv->kvh;
  a.kv.hd = kv->hd;
  a.kv.contiguous_len = kv->max_len;
  a.kv.dtype = kv->dtype;
  a.pos0 = kv->d_pos;  // context before these queries
  a.B = B;
  a.S = (int)S;
  a.nh = nh;
  a.causal = causal;
  a.mask_kind = mask_kind;
  a.kv_len_fixed = -1;
  a.max_kv_len = kv->max_len;
  a.dtype = kv->dtype;
  Pool pool(c);
  if (kv->dtype == REWB200_BF16) {
    a.tmK = &kv->tmK;
    a.tmV = &kv->tmV;
    a.scratch_bytes = attn_scratch_bytes(B, nh, kv->hd, 16);
    RB_TRY(pool.get(&a.scratch, a.scratch_bytes));
  }
  const bool pdl = c->use_pdl;
  c->use_pdl = false;
  const int st = attn_launch(c, a);
  c->use_pdl = pdl;
  return st;
}

}  // extern "C"

// ---------------------------------------------------------------- routed experts

struct rewb200_experts {
  int slot = 0, dtype = 0, E = 0;
  int64_t d = 0, f = 0;
  // bf16: gate|up of an expert fused into [d][2f] with gate / up columns interleaved in groups of 8 (the
  // layout the SwiGLU epilogue reads); f32: gate and up kept apart
  void *gu = nullptr, *down = nullptr, *gate32 = nullptr, *up32 = nullptr;
  float *gu_b = nullptr, *down_b = nullptr, *gate_b32 = nullptr, *up_b32 = nullptr;
  LinearBf16Plan plan_gu, plan_down;
};

extern "C" {

void rewb200_experts_free(rewb200_experts* h) {
  if (!h) return;
  Ctx* c = ctx_get(h->slot);
  if (c) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
  }
  void* ptrs[] = {h->gu, h->down, h->gate32, h->up32, h->gu_b, h->down_b, h->gate_b32, h->up_b32};
  for (void* p : ptrs) cudaFree(p);
  delete h;
}

int rewb200_experts_create(int slot, int n_experts, const rewb200_buffer* const* gate_w, const rewb200_buffer* const* gate_b,
                           const rewb200_buffer* const* up_w, const rewb200_buffer* const* up_b,
                           const rewb200_buffer* const* down_w, const rewb200_buffer* const* down_b, rewb200_experts** out) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(out && gate_w && up_w && down_w && n_experts >= 1 && n_experts <= 256, "initDeepSeekMoE: 1..256 routed experts");
  for (int e = 0; e < n_experts; ++e)
    RB_REQUIRE(gate_w[e] && up_w[e] && down_w[e] && gate_w[e]->ndims == 2 && up_w[e]->ndims == 2 && down_w[e]->ndims == 2,
               "initDeepSeekExpert: every expert needs gate, up and down weights [in, out]");
  const int dt = gate_w[0]->dtype;
  const int64_t d = gate_w[0]->dims[0], f = gate_w[0]->dims[1];
  RB_REQUIRE(dt == REWB200_F32 || dt == REWB200_BF16, "experts must be f32 or bf16");
  for (int e = 0; e < n_experts; ++e) {
    RB_REQUIRE(gate_w[e]->dtype == dt && up_w[e]->dtype == dt && down_w[e]->dtype == dt, "experts: dtypes differ");
    RB_REQUIRE(gate_w[e]->dims[0] == d && gate_w[e]->dims[1] == f && up_w[e]->dims[0] == d && up_w[e]->dims[1] == f &&
                   down_w[e]->dims[0] == f && down_w[e]->dims[1] == d,
               "initDeepSeekExpert: gate / up must be [hiddenSize, intermediateSize] and down the transpose shape");
  }
  if (dt == REWB200_BF16) RB_REQUIRE(d % 8 == 0 && f % 8 == 0, "bf16 experts need hiddenSize and intermediateSize multiples of 8");
  RB_CUDA(cudaSetDevice(c->device));
  rewb200_experts* h = new rewb200_experts();
  h->slot = slot; h->dtype = dt; h->E = n_experts; h->d = d; h->f = f;
  const size_t es = dtype_size(dt), E = (size_t)n_experts;
  auto body = [&]() -> int {
    RB_CUDA(cudaMalloc(&h->down, E * f * d * es));
    RB_CUDA(cudaMalloc((void**)&h->down_b, E * d * sizeof(float)));
    RB_CUDA(cudaMemsetAsync(h->down_b, 0, E * d * sizeof(float), c->stream));
    if (dt == REWB200_BF16) {
      RB_CUDA(cudaMalloc(&h->gu, E * d * 2 * f * es));
      RB_CUDA(cudaMalloc((void**)&h->gu_b, E * 2 * f * sizeof(float)));
      RB_CUDA(cudaMemsetAsync(h->gu_b, 0, E * 2 * f * sizeof(float), c->stream));
    } else {
      RB_CUDA(cudaMalloc(&h->gate32, E * d * f * es));
      RB_CUDA(cudaMalloc(&h->up32, E * d * f * es));
      RB_CUDA(cudaMalloc((void**)&h->gate_b32, E * f * sizeof(float)));
      RB_CUDA(cudaMalloc((void**)&h->up_b32, E * f * sizeof(float)));
      RB_CUDA(cudaMemsetAsync(h->gate_b32, 0, E * f * sizeof(float), c->stream));
      RB_CUDA(cudaMemsetAsync(h->up_b32, 0, E * f * sizeof(float), c->stream));
    }
    for (int e = 0; e < n_experts; ++e) {
      RB_TRY(place_cols(c, down_w[e], f, d, (char*)h->down + (size_t)e * f * d * es, dt, d, d, d, 0));
      if (down_b && down_b[e]) RB_TRY(place_cols(c, down_b[e], 1, d, h->down_b + (size_t)e * d, REWB200_F32, d, d, d, 0));
      if (dt == REWB200_BF16) {
        char* gw = (char*)h->gu + (size_t)e * d * 2 * f * es;
        float* gb = h->gu_b + (size_t)e * 2 * f;
        RB_TRY(place_cols(c, gate_w[e], d, f, gw, dt, 2 * f, 8, 16, 0));
        RB_TRY(place_cols(c, up_w[e], d, f, gw, dt, 2 * f, 8, 16, 8));
        if (gate_b && gate_b[e]) RB_TRY(place_cols(c, gate_b[e], 1, f, gb, REWB200_F32, 2 * f, 8, 16, 0));
        if (up_b && up_b[e]) RB_TRY(place_cols(c, up_b[e], 1, f, gb, REWB200_F32, 2 * f, 8, 16, 8));
      } else {
        RB_TRY(place_cols(c, gate_w[e], d, f, (char*)h->gate32 + (size_t)e * d * f * es, dt, f, f, f, 0));
        RB_TRY(place_cols(c, up_w[e], d, f, (char*)h->up32 + (size_t)e * d * f * es, dt, f, f, f, 0));
        if (gate_b && gate_b[e]) RB_TRY(place_cols(c, gate_b[e], 1, f, h->gate_b32 + (size_t)e * f, REWB200_F32, f, f, f, 0));
        if (up_b && up_b[e]) RB_TRY(place_cols(c, up_b[e], 1, f, h->up_b32 + (size_t)e * f, REWB200_F32, f, f, f, 0));
      }
    }
    if (dt == REWB200_BF16) {
      RB_TRY(linear_bf16_plan(&h->plan_gu, (const bf16*)h->gu, d, 2 * f, n_experts));
      RB_TRY(linear_bf16_plan(&h->plan_down, (const bf16*)h->down, f, d, n_experts));
    }
    RB_CUDA(cudaStreamSynchronize(c->stream));
    return REWB200_OK;
  };
  const int st = body();
  if (st != REWB200_OK) {
    const std::string why = rewb200_last_error();
    rewb200_experts_free(h);
    set_error(why);
    return st;
  }
  *out = h;
  return REWB200_OK;
}

int rewb200_moe_experts(const rewb200_experts* h, const rewb200_buffer* x, const rewb200_buffer* weights,
                        const rewb200_buffer* indices, rewb200_buffer** y) {
  RB_REQUIRE(h && x && weights && indices && y, "DeepSeekMoE.forward: NULL argument");
  RB_REQUIRE(x->ndims == 2 && x->dims[1] == h->d && x->dtype == h->dtype, "DeepSeekMoE.forward: hidden must be [tokens, hiddenSize] of the experts' dtype");
  RB_REQUIRE(weights->ndims == 2 && indices->ndims == 2 && weights->dtype == REWB200_F32 && indices->dtype == REWB200_I32 &&
                 weights->dims[0] == x->dims[0] && indices->dims[0] == x->dims[0] && weights->dims[1] == indices->dims[1],
             "DeepSeekMoE.forward: routing weights f32 [tokens, k] and indices int32 [tokens, k]");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t T = x->dims[0], d = h->d, f = h->f;
  const int k = (int)weights->dims[1], E = h->E;
  RB_REQUIRE(k >= 1 && k <= E, "initDeepSeekMoE: numExpertsPerTok must be in 1..numRouted");
  RB_TRY(buffer_new(c, x->dtype, x->dims, 2, y));
  if (T == 0) return REWB200_OK;
  const float* topw = (const float*)weights->ptr;
  const int* topi = (const int*)indices->ptr;
  Pool pool(c);
  const bool pdl = c->use_pdl;
  struct Restore {
    Ctx* c;
    bool v;
    ~Restore() { c->use_pdl = v; }
  } restore{c, pdl};
  c->use_pdl = false;  // scratch comes from the stream-ordered pool: plain stream order throughout
  if (h->dtype == REWB200_F32) {
    // the reference's own schedule: every expert on every token, masked by its routing weight
    float *g = nullptr, *u = nullptr, *hh = nullptr, *t = nullptr;
    RB_TRY(pool.get(&g, (size_t)T * f * 4));
    RB_TRY(pool.get(&u, (size_t)T * f * 4));
    RB_TRY(pool.get(&hh, (size_t)T * f * 4));
    RB_TRY(pool.get(&t, (size_t)T * d * 4));
    for (int e = 0; e < E; ++e) {
      RB_TRY(gemm_f32_launch(c, (const float*)x->ptr, (const float*)h->gate32 + (size_t)e * d * f, h->gate_b32 + (size_t)e * f, g, T, d, f));
      RB_TRY(gemm_f32_launch(c, (const float*)x->ptr, (const float*)h->up32 + (size_t)e * d * f, h->up_b32 + (size_t)e * f, u, T, d, f));
      RB_TRY(swiglu_f32_launch(c, g, u, hh, T * f));
      RB_TRY(gemm_f32_launch(c, hh, (const float*)h->down + (size_t)e * f * d, h->down_b + (size_t)e * d, t, T, f, d));
      const int64_t n = T * d;
      expert_acc_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(t, topw, topi, k, e, T, d, (float*)(*y)->ptr, e > 0 ? 1 : 0);
      RB_CUDA(cudaGetLastError());
      ++g_launch_total;
    }
    return ctx_check_status(c);
  }
  // bf16: rows sorted by expert, two grouped GEMMs (SwiGLU in the first one's epilogue), weighted combine
  const int64_t cap = T * k;
  bf16 *xs = nullptr, *hs = nullptr;
  float *ys = nullptr, *acc = nullptr;
  int* ints = nullptr;
  RB_TRY(pool.get(&xs, (size_t)(cap + 256) * d * 2));
  RB_TRY(pool.get(&hs, (size_t)(cap + 256) * f * 2));
  RB_TRY(pool.get(&ys, (size_t)cap * d * 4));
  RB_TRY(pool.get(&acc, (size_t)T * d * 4));
  RB_TRY(pool.get(&ints, (size_t)(1 + 3 * (E + 1) + 4 * cap) * sizeof(int)));
  RB_CUDA(cudaMemsetAsync(xs + cap * d, 0, (size_t)256 * d * 2, c->stream));   // rows a ragged last tile reads past the end
  RB_CUDA(cudaMemsetAsync(hs + cap * f, 0, (size_t)256 * f * 2, c->stream));
  int* cursor = ints;
  int* count = cursor + 1;
  int* offsets = count + (E + 1);
  int* cursor2 = offsets + (E + 1);
  int* meta = cursor2 + (E + 1);
  int* slot_pos = meta + cap;
  int* pair_slot = slot_pos + cap;
  const int max_rows = (int)std::min<int64_t>(T, cap);  // an expert sees each token at most once
  const float* back = ys;
  const bool sorted_in_place = cap <= 2048;  // one kernel sorts the pairs by expert; larger steps go through slot arrays
  if (sorted_in_place) {
    RB_TRY(moe_group_local_launch(c, x->ptr, REWB200_BF16, topi, T, k, d, E, offsets, xs, pair_slot));
  } else {
    bf16* send = nullptr;
    RB_TRY(pool.get(&send, (size_t)cap * d * 2));
    RB_TRY(moe_reset_launch(c, cursor, 1, count, E + 1, meta, (int)cap));
    RB_TRY(moe_dispatch_launch(c, x->ptr, REWB200_BF16, topi, T, k, d, E, (int)cap, cursor, send, meta, pair_slot));
    RB_TRY(moe_group_launch(c, send, REWB200_BF16, meta, (int)cap, d, E, count, offsets, cursor2, xs, slot_pos));
  }
  RB_TRY(linear_bf16_launch(c, h->plan_gu, xs, d, cap, EPI_SWIGLU_BF16, 1, hs, f, h->gu_b, offsets, max_rows));
  RB_TRY(linear_bf16_launch(c, h->plan_down, hs, f, cap, EPI_BIAS_F32, 1, ys, d, h->down_b, offsets, max_rows));
  if (!sorted_in_place) {
    float* ret = nullptr;
    RB_TRY(pool.get(&ret, (size_t)cap * d * 4));
    RB_TRY(moe_return_launch(c, ys, slot_pos, (int)cap, d, ret));
    back = ret;
  }
  RB_TRY(moe_combine_launch(c, back, pair_slot, topw, T, k, d, acc, 0));
  RB_TRY(cast_launch(c, acc, REWB200_F32, (*y)->ptr, REWB200_BF16, T * d));
  return ctx_check_status(c);
}

}  // extern "C"

// ---------------------------------------------------------------- lm_head + sampling

struct rewb200_sampler {
  int slot = 0, B = 0, V = 0, cap = 0;
  float temperature = 1.f, top_p = 1.f, min_p = 0.f, rep = 1.f;
  int top_k = 0, do_sample = 1;
  int *hist = nullptr, *hist_len = nullptr, *steps = nullptr, *next = nullptr;
  uint32_t* keys = nullptr;
  float *work = nullptr, *logprob = nullptr;
};

extern "C" {

void rewb200_sampler_free(rewb200_sampler* s) {
  if (!s) return;
  Ctx* c = ctx_get(s->slot);
  if (c) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
  }
  void* ptrs[] = {s->hist, s->hist_len, s->steps, s->next, s->keys, s->work, s->logprob};
  for (void* p : ptrs) cudaFree(p);
  delete s;
}

int rewb200_sampler_create(int slot, int batch, int vocab, int max_tokens, float temperature, int top_k, float top_p,
                           float min_p, float repetition_penalty, int do_sample, const uint64_t* seeds, rewb200_sampler** out) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(out && batch > 0 && vocab > 0 && max_tokens > 0, "initGenerationConfig: batch, vocabulary and token budget must be positive");
  // initGenerationConfig's checks (generate.nim:30-49)
  RB_REQUIRE(temperature >= 0.f, "initGenerationConfig: temperature must be non-negative");
  RB_REQUIRE(top_k >= 0, "initGenerationConfig: topK must be non-negative");
  RB_REQUIRE(top_p > 0.f && top_p <= 1.f, "initGenerationConfig: topP must be in (0, 1]");
  RB_REQUIRE(min_p >= 0.f && min_p <= 1.f, "initGenerationConfig: minP must be in [0, 1]");
  RB_REQUIRE(repetition_penalty > 0.f, "initGenerationConfig: repetitionPenalty must be positive");
  RB_REQUIRE(top_k <= 1024, "device sampling keeps at most 1024 top-k candidates");
  RB_CUDA(cudaSetDevice(c->device));
  rewb200_sampler* s = new rewb200_sampler();
  s->slot = slot; s->B = batch; s->V = vocab; s->cap = max_tokens;
  s->temperature = temperature; s->top_k = top_k; s->top_p = top_p; s->min_p = min_p; s->rep = repetition_penalty;
  s->do_sample = do_sample ? 1 : 0;
  auto body = [&]() -> int {
    RB_CUDA(cudaMalloc((void**)&s->hist, (size_t)batch * max_tokens * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->hist_len, batch * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->steps, batch * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->next, batch * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->keys, (size_t)batch * 2 * sizeof(uint32_t)));
    RB_CUDA(cudaMalloc((void**)&s->work, (size_t)batch * vocab * sizeof(float)));
    RB_CUDA(cudaMalloc((void**)&s->logprob, (size_t)batch * max_tokens * sizeof(float)));
    std::vector<uint32_t> k((size_t)batch * 2, 0u);  // initKey (src/rew/rng.nim:60-64)
    for (int b = 0; b < batch && seeds; ++b) {
      k[2 * b] = (uint32_t)(seeds[b] & 0xFFFFFFFFull);
      k[2 * b + 1] = (uint32_t)(seeds[b] >> 32);
    }
    RB_CUDA(cudaMemcpy(s->keys, k.data(), k.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
    RB_CUDA(cudaMemset(s->steps, 0, batch * sizeof(int)));
    RB_CUDA(cudaMemset(s->hist_len, 0, batch * sizeof(int)));
    return REWB200_OK;
  };
  const int st = body();
  if (st != REWB200_OK) {
    const std::string why = rewb200_last_error();
    rewb200_sampler_free(s);
    set_error(why);
    return st;
  }
  *out = s;
  return REWB200_OK;
}

int rewb200_sampler_observe(rewb200_sampler* s, const int32_t* ids, int n_per_row) {
  RB_REQUIRE(s && ids && n_per_row >= 0, "sampler: NULL argument");
  Ctx* c = ctx_get(s->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  std::vector<int> len((size_t)s->B);
  RB_CUDA(cudaMemcpy(len.data(), s->hist_len, s->B * sizeof(int), cudaMemcpyDeviceToHost));
  for (int b = 0; b < s->B; ++b) {
    RB_REQUIRE(len[b] + n_per_row <= s->cap, "sampler: more tokens than its budget");
    RB_CUDA(cudaMemcpy(s->hist + (size_t)b * s->cap + len[b], ids + (size_t)b * n_per_row, (size_t)n_per_row * sizeof(int),
                       cudaMemcpyHostToDevice));
    len[b] += n_per_row;
  }
  RB_CUDA(cudaMemcpy(s->hist_len, len.data(), s->B * sizeof(int), cudaMemcpyHostToDevice));
  return REWB200_OK;
}

int rewb200_lmhead_sample(const rewb200_buffer* x, const rewb200_buffer* lm_w, const rewb200_buffer* lm_b,
                          rewb200_sampler* sampler, int32_t* next_ids, float* logits_out) {
  RB_REQUIRE(x && lm_w && next_ids, "generate: NULL argument");
  RB_REQUIRE(x->ndims == 2 && lm_w->ndims == 2 && x->dims[1] == lm_w->dims[0], "lmHead: hidden [batch, d] and weight [d, vocab] do not agree");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t B = x->dims[0], V = lm_w->dims[1];
  RB_REQUIRE(!sampler || (sampler->B == B && sampler->V == V), "sampler was created for another batch or vocabulary");
  rewb200_buffer* logits = nullptr;
  RB_TRY(rewb200_linear(x, lm_w, lm_b, &logits));
  Pool pool(c);
  float* lf = (float*)logits->ptr;
  int st = REWB200_OK;
  if (logits->dtype == REWB200_BF16) {  // the samplers need f32 logits (generate.nim:173-175)
    st = pool.get(&lf, (size_t)B * V * 4);
    if (st == REWB200_OK) st = cast_launch(c, logits->ptr, REWB200_BF16, lf, REWB200_F32, B * V);
  }
  int* next = nullptr;
  void* scratch = nullptr;
  const bool pdl = c->use_pdl;
  c->use_pdl = false;
  if (st == REWB200_OK && sampler) {
    next = sampler->next;
    st = sample_launch(c, lf, sampler->work, B, V, sampler->hist, sampler->hist_len, sampler->cap, sampler->keys, sampler->steps,
                       next, sampler->logprob, sampler->cap, sampler->temperature, sampler->top_k, sampler->top_p, sampler->min_p,
                       sampler->rep, sampler->do_sample, nullptr);
  } else if (st == REWB200_OK) {
    st = pool.get(&next, (size_t)B * sizeof(int));
    if (st == REWB200_OK) st = pool.get(&scratch, (size_t)B * 64 * 8);
    if (st == REWB200_OK) st = argmax_launch(c, lf, B, V, next, scratch, (size_t)B * 64 * 8);
  }
  c->use_pdl = pdl;
  if (st == REWB200_OK && cudaMemcpyAsync(next_ids, next, B * sizeof(int), cudaMemcpyDeviceToHost, c->stream) != cudaSuccess)
    st = fail("copy of the sampled ids failed");
  if (st == REWB200_OK && logits_out &&
      cudaMemcpyAsync(logits_out, lf, (size_t)B * V * 4, cudaMemcpyDeviceToHost, c->stream) != cudaSuccess)
    st = fail("copy of the logits failed");
  if (st == REWB200_OK && cudaStreamSynchronize(c->stream) != cudaSuccess) st = fail("stream synchronisation failed");
  rewb200_buffer_release(logits);
  if (st != REWB200_OK) return st;
  return ctx_check_status(c);
}

}  // extern "C"
