// Tier-B C entry points: one call per rew.nn forward, on opaque device buffers.
// Each validates shapes with the reference's error wording where it has one
// and forwards to the kernels the engine uses.
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

using namespace rewb;

namespace rewb {
namespace {

template <typename T>
__global__ void rope_kernel(const T* x, T* y, const float* cosT, const float* sinT, int64_t lead, int64_t S, int hd,
                            int64_t offset) {
  const int half = hd / 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= lead * S * half) return;
  const int p = (int)(i % half);
  const int64_t row = i / half;
  const int64_t s = row % S;
  const float c0 = cosT[(offset + s) * hd + 2 * p], s0 = sinT[(offset + s) * hd + 2 * p];
  float x0, x1;
  if constexpr (sizeof(T) == 2) {
    x0 = __bfloat162float(x[row * hd + 2 * p]);
    x1 = __bfloat162float(x[row * hd + 2 * p + 1]);
    y[row * hd + 2 * p] = __float2bfloat16_rn(rope_even(c0, s0, x0, x1));
    y[row * hd + 2 * p + 1] = __float2bfloat16_rn(rope_odd(c0, s0, x0, x1));
  } else {
    x0 = x[row * hd + 2 * p];
    x1 = x[row * hd + 2 * p + 1];
    y[row * hd + 2 * p] = rope_even(c0, s0, x0, x1);
    y[row * hd + 2 * p + 1] = rope_odd(c0, s0, x0, x1);
  }
}

template <typename T>
__global__ void gather_rows_kernel(const int* ids, const T* table, T* out, int64_t N, int64_t V, int64_t d,
                                   int* status) {
  const int64_t row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(status, KS_BAD_INDEX);
    id = 0;
  }
  for (int64_t i = threadIdx.x; i < d; i += blockDim.x) out[row * d + i] = table[(int64_t)id * d + i];
}

int same_slot(const rewb200_buffer* a, const rewb200_buffer* b) {
  RB_REQUIRE(a->slot == b->slot, "cross-device operands forbidden");
  return REWB200_OK;
}

int alloc_like(Ctx* c, const rewb200_buffer* x, rewb200_buffer** y) { return buffer_new(c, x->dtype, x->dims, x->ndims, y); }

int norm_common(const rewb200_buffer* x, const rewb200_buffer* gamma, const rewb200_buffer* beta, float eps, int kind,
                rewb200_buffer** y) {
  RB_REQUIRE(x && gamma && y, "norm: NULL argument");
  RB_REQUIRE(x->ndims >= 1, "rmsNorm: input must have at least 1 dimension");
  RB_REQUIRE(x->dtype == REWB200_F32 || x->dtype == REWB200_BF16, "norm: x must be f32 or bf16");
  const int64_t d = x->dims[x->ndims - 1];
  RB_REQUIRE(gamma->dtype == REWB200_F32 && gamma->numel() == d, "norm: gamma must be f32 of the last dimension's size");
  RB_REQUIRE(kind == 0 || (beta && beta->dtype == REWB200_F32 && beta->numel() == d), "LayerNorm: beta must be f32 [d]");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(alloc_like(c, x, y));
  NormArgs a;
  memset(&a, 0, sizeof(a));
  a.embed = x->ptr;
  a.embed_dtype = x->dtype;
  a.gamma = (const float*)gamma->ptr;
  a.beta = beta ? (const float*)beta->ptr : nullptr;
  a.eps = eps;
  a.norm_kind = kind;
  a.d = d;
  a.out = (*y)->ptr;
  a.out_dtype = x->dtype;
  a.status = c->d_status;
  return residual_norm_launch(c, a, d ? x->numel() / d : 0);
}

}  // namespace
}  // namespace rewb

extern "C" {

int rewb200_linear(const rewb200_buffer* x, const rewb200_buffer* w, const rewb200_buffer* b, rewb200_buffer** y) {
  RB_REQUIRE(x && w && y, "Linear.forward: NULL argument");
  RB_REQUIRE(x->ndims == 2 && w->ndims == 2,
             "matmul: expected rank-2 operands, got ranks " + std::to_string(x->ndims) + " and " + std::to_string(w->ndims));
  RB_REQUIRE(x->dims[1] == w->dims[0], "matmul: inner dim mismatch: [" + std::to_string(x->dims[0]) + "," +
                                           std::to_string(x->dims[1]) + "] * [" + std::to_string(w->dims[0]) + "," +
                                           std::to_string(w->dims[1]) + "]");
  RB_REQUIRE(x->dtype == w->dtype, "Linear.forward: x and weight dtypes differ");
  RB_TRY(same_slot(x, w));
  RB_REQUIRE(!b || (b->dtype == REWB200_F32 && b->numel() == w->dims[1]), "Linear.forward: bias must be f32 [out]");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t M = x->dims[0], K = x->dims[1], N = w->dims[1];
  const int64_t od[2] = {M, N};
  RB_TRY(buffer_new(c, x->dtype, od, 2, y));
  const float* bias = b ? (const float*)b->ptr : nullptr;
  if (x->dtype == REWB200_F32)
    return gemm_f32_launch(c, (const float*)x->ptr, (const float*)w->ptr, bias, (float*)(*y)->ptr, M, K, N);
  RB_REQUIRE(x->dtype == REWB200_BF16, "Linear.forward: dtype must be f32 or bf16");
  LinearBf16Plan plan;
  RB_TRY(linear_bf16_plan(&plan, (const bf16*)w->ptr, K, N, 0));
  return linear_bf16_launch(c, plan, (const bf16*)x->ptr, K, M, EPI_BIAS_BF16, 1, (*y)->ptr, N, bias, nullptr, 0);
}

int rewb200_rmsnorm(const rewb200_buffer* x, const rewb200_buffer* gamma, float eps, rewb200_buffer** y) {
  return norm_common(x, gamma, nullptr, eps, 0, y);
}

int rewb200_layernorm(const rewb200_buffer* x, const rewb200_buffer* gamma, const rewb200_buffer* beta, float eps,
                      rewb200_buffer** y) {
  RB_REQUIRE(beta, "LayerNorm.forward: beta is NULL");
  return norm_common(x, gamma, beta, eps, 1, y);
}

int rewb200_rope_tables(int slot, int head_dim, int max_seq, double theta, rewb200_buffer** cos_out,
                        rewb200_buffer** sin_out) {
  RB_REQUIRE(cos_out && sin_out, "rope tables: NULL output");
  std::vector<float> ct, st;
  RB_TRY(rope_tables_host(head_dim, max_seq, theta, &ct, &st));
  const int64_t dims[2] = {max_seq, head_dim};
  RB_TRY(rewb200_buffer_from_host(slot, ct.data(), REWB200_F32, dims, 2, cos_out));
  return rewb200_buffer_from_host(slot, st.data(), REWB200_F32, dims, 2, sin_out);
}

int rewb200_rope(const rewb200_buffer* x, const rewb200_buffer* cos_t, const rewb200_buffer* sin_t, int64_t offset,
                 rewb200_buffer** y) {
  RB_REQUIRE(x && cos_t && sin_t && y, "RotaryPositionEncoding.forward: NULL argument");
  RB_REQUIRE(x->ndims >= 2, "RotaryPositionEncoding.forward: input rank must be at least 2");
  const int64_t S = x->dims[x->ndims - 2], hd = x->dims[x->ndims - 1];
  RB_REQUIRE(cos_t->ndims == 2 && sin_t->ndims == 2 && cos_t->dtype == REWB200_F32 && sin_t->dtype == REWB200_F32,
             "RotaryPositionEncoding.forward: tables must be f32 [maxSeqLen, headDim]");
  RB_REQUIRE(hd == cos_t->dims[1], "RotaryPositionEncoding.forward: headDim mismatch " + std::to_string(hd) + " vs " +
                                       std::to_string(cos_t->dims[1]));
  RB_REQUIRE(offset >= 0 && offset + S <= cos_t->dims[0], "RotaryPositionEncoding.forward: position " +
                                                              std::to_string(offset + S) + " exceeds maxSeqLen " +
                                                              std::to_string(cos_t->dims[0]));
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(alloc_like(c, x, y));
  const int64_t lead = (S * hd) ? x->numel() / (S * hd) : 0;
  const int64_t n = lead * S * (hd / 2);
  if (n == 0) return REWB200_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (x->dtype == REWB200_F32)
    rope_kernel<float><<<blocks, 256, 0, c->stream>>>((const float*)x->ptr, (float*)(*y)->ptr, (const float*)cos_t->ptr,
                                                      (const float*)sin_t->ptr, lead, S, (int)hd, offset);
  else if (x->dtype == REWB200_BF16)
    rope_kernel<bf16><<<blocks, 256, 0, c->stream>>>((const bf16*)x->ptr, (bf16*)(*y)->ptr, (const float*)cos_t->ptr,
                                                     (const float*)sin_t->ptr, lead, S, (int)hd, offset);
  else
    return fail("RotaryPositionEncoding.forward: dtype must be f32 or bf16");
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

static int gqa_attention_impl(const rewb200_buffer* q, const rewb200_buffer* k, const rewb200_buffer* v, int causal,
                              int mask_kind, rewb200_buffer** out, int iters, float* ms_per_call) {
  RB_REQUIRE(q && k && v && out, "scaledDotProductAttention: NULL argument");
  RB_REQUIRE(q->ndims == 4 && k->ndims == 4 && v->ndims == 4,
             "scaledDotProductAttention: operands must be [batch, heads, len, headDim]");
  RB_REQUIRE(q->dtype == k->dtype && q->dtype == v->dtype, "scaledDotProductAttention: dtypes differ");
  const int64_t B = q->dims[0], nh = q->dims[1], S = q->dims[2], hd = q->dims[3];
  const int64_t kvh = k->dims[1], L = k->dims[2];
  RB_REQUIRE(k->dims[0] == B && v->dims[0] == B && k->dims[3] == hd && v->dims[3] == hd && v->dims[1] == kvh &&
                 v->dims[2] == L,
             "scaledDotProductAttention: q/k/v shapes do not agree");
  RB_REQUIRE(kvh > 0 && nh % kvh == 0, "initGroupedQueryAttention: numHeads " + std::to_string(nh) +
                                           " must be divisible by numKVHeads " + std::to_string(kvh));
  RB_REQUIRE(L >= 1, "scaledDotProductAttention: need at least one key");
  RB_REQUIRE(!causal || mask_kind == 0 || L >= S, "conventional causal mask needs kvLen >= seqLen");
  Ctx* c = ctx_get(q->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(alloc_like(c, q, out));
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q->ptr;
  a.q_sb = nh * S * hd; a.q_ss = hd; a.q_sh = S * hd;
  a.out = (*out)->ptr;
  a.o_sb = a.q_sb; a.o_ss = a.q_ss; a.o_sh = a.q_sh;
  a.kv.k = k->ptr;
  a.kv.v = v->ptr;
  a.kv.block_table = nullptr;
  a.kv.page = 64;
  a.kv.kvh = (int)kvh;
  a.kv.hd = (int)hd;
  a.kv.contiguous_len = L;
  a.kv.dtype = q->dtype;
  a.pos0 = nullptr;
  a.B = B;
  a.S = (int)S;
  a.nh = (int)nh;
  a.causal = causal;
  a.mask_kind = mask_kind;
  a.kv_len_fixed = L;
  a.max_kv_len = L;
  a.dtype = q->dtype;
  CUtensorMap tmK, tmV;
  float* scratch = nullptr;
  if (q->dtype == REWB200_BF16) {
    RB_REQUIRE(hd == 64 || hd == 128, "bf16 attention supports head_dim 64 and 128");
    RB_TRY(make_tmap_2d_bf16(&tmK, k->ptr, hd, B * kvh * L, hd * 2, 64, 64));
    RB_TRY(make_tmap_2d_bf16(&tmV, v->ptr, hd, B * kvh * L, hd * 2, 64, 64));
    a.tmK = &tmK;
    a.tmV = &tmV;
    a.scratch_bytes = attn_scratch_bytes(B, (int)nh, (int)hd, 16);
    RB_CUDA(cudaMallocAsync((void**)&scratch, a.scratch_bytes, c->stream));
    a.scratch = scratch;
  }
  int st = attn_launch(c, a);
  if (st == REWB200_OK && iters > 0 && ms_per_call) {
    // measurement aid: the same launch `iters` more times between two CUDA events
    cudaEvent_t e0, e1;
    RB_CUDA(cudaEventCreate(&e0));
    RB_CUDA(cudaEventCreate(&e1));
    RB_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters && st == REWB200_OK; ++i) st = attn_launch(c, a);
    RB_CUDA(cudaEventRecord(e1, c->stream));
    RB_CUDA(cudaStreamSynchronize(c->stream));
    float ms = 0.f;
    RB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    *ms_per_call = ms / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  if (scratch) cudaFreeAsync(scratch, c->stream);
  return st;
}

int rewb200_gqa_attention(const rewb200_buffer* q, const rewb200_buffer* k, const rewb200_buffer* v, int causal,
                          int mask_kind, rewb200_buffer** out) {
  return gqa_attention_impl(q, k, v, causal, mask_kind, out, 0, nullptr);
}

int rewb200_gqa_attention_timed(const rewb200_buffer* q, const rewb200_buffer* k, const rewb200_buffer* v, int causal,
                                int mask_kind, int iters, float* ms_per_call, rewb200_buffer** out) {
  RB_REQUIRE(iters > 0 && ms_per_call, "rewb200_gqa_attention_timed: iters must be positive and ms_per_call non-NULL");
  return gqa_attention_impl(q, k, v, causal, mask_kind, out, iters, ms_per_call);
}

int rewb200_swiglu_ffn(const rewb200_buffer* x, const rewb200_buffer* gate_w, const rewb200_buffer* gate_b,
                       const rewb200_buffer* up_w, const rewb200_buffer* up_b, const rewb200_buffer* down_w,
                       const rewb200_buffer* down_b, rewb200_buffer** y) {
  RB_REQUIRE(x && gate_w && up_w && down_w && y, "GatedFeedForward.forward: NULL argument");
  RB_REQUIRE(x->ndims == 2, "GatedFeedForward.forward: x must be [rows, embedDim] here");
  RB_REQUIRE(gate_w->ndims == 2 && up_w->ndims == 2 && down_w->ndims == 2 && gate_w->dims[1] == up_w->dims[1] &&
                 down_w->dims[0] == gate_w->dims[1],
             "GatedFeedForward.forward: projection shapes do not agree");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t M = x->dims[0], f = gate_w->dims[1];
  rewb200_buffer *g = nullptr, *u = nullptr, *h = nullptr;
  int st = rewb200_linear(x, gate_w, gate_b, &g);
  if (st == REWB200_OK) st = rewb200_linear(x, up_w, up_b, &u);
  if (st == REWB200_OK) {
    const int64_t hd[2] = {M, f};
    st = buffer_new(c, x->dtype, hd, 2, &h);
  }
  if (st == REWB200_OK) {
    if (x->dtype == REWB200_F32) {
      st = swiglu_f32_launch(c, (const float*)g->ptr, (const float*)u->ptr, (float*)h->ptr, M * f);
    } else {
      // bf16 Tier-B call: activation in f32 on the rounded projections, rounded once more
      float *gf = nullptr, *uf = nullptr;
      if (cudaMallocAsync((void**)&gf, (size_t)M * f * 8 + 256, c->stream) != cudaSuccess) st = fail("allocation failed");
      if (st == REWB200_OK) {
        uf = gf + M * f;
        st = cast_launch(c, g->ptr, REWB200_BF16, gf, REWB200_F32, M * f);
        if (st == REWB200_OK) st = cast_launch(c, u->ptr, REWB200_BF16, uf, REWB200_F32, M * f);
        if (st == REWB200_OK) st = swiglu_f32_launch(c, gf, uf, gf, M * f);
        if (st == REWB200_OK) st = cast_launch(c, gf, REWB200_F32, h->ptr, REWB200_BF16, M * f);
        cudaFreeAsync(gf, c->stream);
      }
    }
  }
  if (st == REWB200_OK) st = rewb200_linear(h, down_w, down_b, y);
  rewb200_buffer_release(g);
  rewb200_buffer_release(u);
  rewb200_buffer_release(h);
  return st;
}

int rewb200_embed_gather(const rewb200_buffer* ids, const rewb200_buffer* table, rewb200_buffer** y) {
  RB_REQUIRE(ids && table && y, "Embedding.forward: NULL argument");
  RB_REQUIRE(ids->dtype == REWB200_I32, "oneHot: indices must be an int32 tensor");
  RB_REQUIRE(table->ndims == 2, "Embedding.forward: table must be [vocabSize, embedDim]");
  Ctx* c = ctx_get(table->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t N = ids->numel(), V = table->dims[0], d = table->dims[1];
  int64_t od[8];
  for (int i = 0; i < ids->ndims; ++i) od[i] = ids->dims[i];
  od[ids->ndims] = d;
  RB_REQUIRE(ids->ndims < 8, "Embedding.forward: too many dimensions");
  RB_TRY(buffer_new(c, table->dtype, od, ids->ndims + 1, y));
  if (N == 0) return REWB200_OK;
  if (table->dtype == REWB200_F32)
    gather_rows_kernel<float><<<(unsigned)N, 256, 0, c->stream>>>((const int*)ids->ptr, (const float*)table->ptr,
                                                                  (float*)(*y)->ptr, N, V, d, c->d_status);
  else if (table->dtype == REWB200_BF16)
    gather_rows_kernel<bf16><<<(unsigned)N, 256, 0, c->stream>>>((const int*)ids->ptr, (const bf16*)table->ptr,
                                                                 (bf16*)(*y)->ptr, N, V, d, c->d_status);
  else
    return fail("Embedding.forward: table must be f32 or bf16");
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

}  // extern "C"
