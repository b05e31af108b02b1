// Model + session engine: LlamaForCausalLM / DeepSeekForCausalLM
// (src/rew/models/llama.nim:106-140, src/rew/models/deepseek.nim:198-231) with a
// paged KV cache (src/rew/nn/kv_cache.nim, src/rew/infer/generate.nim:63-88) and
// the generate loop (src/rew/infer/generate.nim:231-265) driven on the device.
//
// Device layouts (chosen for B200, not the reference's per-tensor buffers):
//   - q|k|v projection weights concatenated along `out` into one [d, nq+2nkv]
//     matrix so one GEMM streams them; gate|up concatenated the same way, with
//     the bf16 variant interleaving gate/up columns in groups of 8 so the GEMM
//     epilogue can apply SiLU(gate)*up in registers.
//   - The residual stream stays f32; GEMM inputs are the model dtype.
//   - Row-parallel outputs (o-proj, down-proj) are written as f32 split-K
//     partials and summed by the residual+norm kernel, which is also where a
//     tensor-parallel all-reduce result lands.
//   - KV cache pages of 64 tokens: [page][kv_head][64][head_dim].
//   - One decode step (batch fixed, positions read from device memory) is
//     captured once into a CUDA graph and replayed; token ids, positions and
//     the step counter live on the device, so a run of n steps needs no host
//     round trip until the ids are copied back.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

using namespace rewb;

namespace rewb {

int comm_world(int slot);
int comm_rank(int slot);
int comm_allreduce_sum(Ctx* c, int slot, void* ptr, int64_t n, int dtype);
int comm_allgather_bytes(Ctx* c, int slot, const void* send, void* recv, size_t bytes_per_rank);
int comm_check_async(int slot);
int slab_sum_launch(Ctx* c, float* part, int nsplit, int64_t slab_elems);
int epoch_bump_launch(Ctx* c, int* epoch, int by);
int comm_alltoall_bytes(Ctx* c, int slot, const void* send, void* recv, size_t bytes_per_peer);
int comm_alltoallv_rows(Ctx* c, int slot, const void* send, void* recv, size_t peer_stride_bytes, size_t row_bytes,
                        const int* send_rows, const int* recv_rows);
int moe_route_launch(Ctx* c, const float* logits, int64_t N, int E, int k, float* topw, int* topi);
int moe_route_slabs_launch(Ctx* c, const float* logits, int nsplit, int64_t split_stride, const float* bias, int64_t N, int E,
                           int k, float* topw, int* topi, int* zero, int n_zero);
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
int moe_dispatch_peer_launch(Ctx* c, const void* x, int dtype, const int* topi, int64_t tokens, int k, int64_t d,
                             int experts_per_rank, int capacity, int* cursor, int* pair_slot, const A2aArgs& a);
int moe_group_peer_launch(Ctx* c, int dtype, int n_slots, int capacity, int64_t d, int n_experts, int* count, int* offsets,
                          int* cursor2, void* xs, int* slot_pos, const A2aArgs& a);
int moe_return_peer_launch(Ctx* c, const float* ys, const int* slot_pos, int n_slots, int capacity, int64_t d, const A2aArgs& a);
int moe_combine_peer_launch(Ctx* c, const int* pair_slot, const float* topw, int64_t tokens, int k, int64_t d, float* out,
                            int accumulate, const A2aArgs& a);
int sample_launch(Ctx* c, const float* logits, float* work, int64_t B, int64_t V, int* hist, int* hist_len, int hist_cap,
                  uint32_t* keys, int* steps, int* next, float* logprob, int logprob_cap, float temperature, int top_k,
                  float top_p, float min_p, float rep_penalty, int do_sample, const int* active);
int argmax_partial_launch(Ctx* c, const float* logits, int64_t rows, int64_t V, int idx_offset, int nchunks, float* pv, int* pi);
int argmax_gathered_launch(Ctx* c, const void* gathered, int world, int64_t rows, int nchunks, int* out);

namespace {

constexpr int PAGE = 64;

struct LinW {
  void* w = nullptr;   // [K,N] model dtype (for a quantised Linear: the shared dequantisation scratch)
  float* b = nullptr;  // [N]
  int64_t K = 0, N = 0;
  LinearBf16Plan plan;
  bool quant = false;  // weight held as NF4 codes
  Nf4W nf4;
  ColMap cm = {1, 1, 1, 0};  // logical column (the reference's [in,out]) -> device column of `w`
};

// Routed experts of one DeepSeekMoE layer held by this rank (src/rew/models/deepseek.nim:36-52).
struct MoeDev {
  LinW router;                 // gate: [d, n_routed]
  void* gu = nullptr;          // [E_l][d][2f]  gate|up per expert (bf16: interleaved in groups of 8)
  float* gu_b = nullptr;       // [E_l][2f]
  void* down = nullptr;        // [E_l][f][d]
  float* down_b = nullptr;     // [E_l][d]
  LinearBf16Plan plan_gu, plan_down;
  int E_l = 0;
  int64_t f = 0;
  std::vector<float> shared_down_bias;  // sum of the shared experts' down biases (uploaded at finalize)
};

struct LayerDev {
  float *ln1g = nullptr, *ln1b = nullptr, *ln2g = nullptr, *ln2b = nullptr;
  LinW qkv, o, gu, down;       // for a MoE layer gu/down are the fused SHARED experts (width n_shared * moe_ffn)
  int64_t ffn_local = 0;
  bool moe = false;
  MoeDev x;
};

// f32 path: out[t] (+)= w_e(t) * y[t], w_e(t) = sum_j topw[t][j] * (topi[t][j] == e)
// (routedWeightForExpert, src/rew/models/deepseek.nim:114-120,140-144)
__global__ void moe_dense_acc_kernel(const float* y, const float* topw, const int* topi, int k, int e, int64_t rows,
                                     int64_t d, float* out, int accumulate) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const int64_t t = i / d;
  float w = 0.f;
  for (int j = 0; j < k; ++j) w += topw[t * k + j] * (topi[t * k + j] == e ? 1.f : 0.f);
  const float v = y[i] * w;
  out[i] = accumulate ? out[i] + v : v;
}

__global__ void scatter_cols_f32_kernel(const float* src, int64_t src_ld, int64_t row0, int64_t col0, int64_t rows,
                                        int64_t cols, void* dst, int dst_bf16, int64_t ldd, int64_t gran,
                                        int64_t gstride, int64_t off) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const int64_t r = i / cols, c = i % cols;
  const float v = src[(row0 + r) * src_ld + col0 + c];
  const int64_t dc = (c / gran) * gstride + (c % gran) + off;
  if (dst_bf16) reinterpret_cast<bf16*>(dst)[r * ldd + dc] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(dst)[r * ldd + dc] = v;
}

// f32 path: out[r][c] = silu(gu[r][c]) * gu[r][f + c]   (src/rew/nn/gated_ffn.nim:55-59)
__global__ void swiglu_rows_f32_kernel(const float* gu, float* out, int64_t rows, int64_t f) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * f) return;
  const int64_t r = i / f, c = i % f;
  const float x = gu[r * 2 * f + c];
  const float sig = 1.0f / (1.0f + expf(-x));
  out[i] = (x * sig) * gu[r * 2 * f + f + c];
}

// Quantised gate|up: sums the split-K slabs of the LOGICAL [rows][gate(f) | up(f)] projection, adds the
// biases (stored in the bf16 engine's interleaved order: groups of 8 gate, 8 up) and applies SwiGLU
// (src/rew/nn/gated_ffn.nim:55-59).
__global__ void swiglu_slabs_kernel(const float* part, int ksplit, int64_t rows, int64_t f, const float* bias_il, bf16* out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * f) return;
  const int64_t r = i / f, c = i % f;
  float g = 0.f, u = 0.f;
  for (int s = 0; s < ksplit; ++s) {
    const float* p = part + ((int64_t)s * rows + r) * 2 * f;
    g += p[c];
    u += p[f + c];
  }
  const int64_t bi = (c / 8) * 16 + (c % 8);
  g += bias_il[bi];
  u += bias_il[bi + 8];
  const float sig = 1.0f / (1.0f + expf(-g));
  out[i] = __float2bfloat16_rn((g * sig) * u);
}

// bf16 gate|up launched with split-K: sums the slabs, which hold the engine's interleaved column order
// (groups of 8 gate columns followed by their 8 up columns), adds the biases and applies SwiGLU.
// One thread per group of eight outputs.
__global__ void swiglu_slabs_il_kernel(const float* part, int ksplit, int64_t rows, int64_t f, const float* bias_il, bf16* out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // group index
  const int64_t gpr = f / 8;
  if (i >= rows * gpr) return;
  const int64_t r = i / gpr, gidx = i % gpr;
  float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < ksplit; ++s) {
    const float4* p = reinterpret_cast<const float4*>(part + ((int64_t)s * rows + r) * 2 * f + gidx * 16);
    const float4 a0 = p[0], a1 = p[1], b0 = p[2], b1 = p[3];
    g[0] += a0.x; g[1] += a0.y; g[2] += a0.z; g[3] += a0.w; g[4] += a1.x; g[5] += a1.y; g[6] += a1.z; g[7] += a1.w;
    u[0] += b0.x; u[1] += b0.y; u[2] += b0.z; u[3] += b0.w; u[4] += b1.x; u[5] += b1.y; u[6] += b1.z; u[7] += b1.w;
  }
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    float v[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float gg = g[j + h] + (bias_il ? bias_il[gidx * 16 + j + h] : 0.f);
      const float uu = u[j + h] + (bias_il ? bias_il[gidx * 16 + 8 + j + h] : 0.f);
      v[h] = gg * (1.0f / (1.0f + __expf(-gg))) * uu;
    }
    const __nv_bfloat162 pk = __floats2bfloat162_rn(v[0], v[1]);
    o[j / 2] = *reinterpret_cast<const uint32_t*>(&pk);
  }
  *reinterpret_cast<uint4*>(out + r * f + gidx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void fill_i32_kernel(int* p, int n, int v) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

// End of a step: publish the sampled ids, make them the next step's input,
// advance positions and the step counter.
// `active` (optional): lanes with 0 keep their token and position and report -1.
__global__ void advance_kernel(const int* next, int* ids, int* pos, int* out_ids, int* step, const int* active, int B,
                               int S, int max_steps) {
  pdl_launch_dependents();
  pdl_wait();
  const int st = *step;
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const bool on = active == nullptr || active[b] != 0;
    if (on) {
      ids[b] = next[b];
      pos[b] += S;
    }
    if (out_ids && st < max_steps) out_ids[(int64_t)st * B + b] = on ? next[b] : -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) *step = st + 1;
}

}  // namespace
}  // namespace rewb

struct rewb200_model {
  Ctx* c = nullptr;
  int slot = 0;
  rewb200_config cfg;
  int nh_l = 0, kvh_l = 0;      // local heads under tensor parallelism
  int64_t vocab_l = 0;          // local slice of the vocabulary (lm_head is vocab-parallel)
  int64_t nq = 0, nkv = 0, nqkv = 0;
  void* embed = nullptr;
  std::vector<LayerDev> layers;
  float *ng = nullptr, *nb = nullptr;
  LinW lm;
  float *cosT = nullptr, *sinT = nullptr;
  float* stage = nullptr;       // f32 upload staging
  size_t stage_bytes = 0;
  bool finalized = false;
  int64_t weight_bytes = 0;
  std::vector<void*> allocs;
};

struct rewb200_session {
  rewb200_model* m = nullptr;
  int B = 0, max_len = 0, max_pages = 0;
  std::vector<void*> kc, vc;           // per layer
  std::vector<CUtensorMap> tmK, tmV;   // per layer (bf16)
  int* block_table = nullptr;
  int *d_pos = nullptr, *d_ids = nullptr, *d_next = nullptr, *d_out = nullptr, *d_step = nullptr;
  int out_capacity = 0;
  int32_t* h_ids = nullptr;            // pinned
  // activations, sized for `rows_cap` rows
  int64_t rows_cap = 0;
  float* x_res = nullptr;
  void* xn = nullptr;
  void* q = nullptr;
  void* attn = nullptr;
  void* h = nullptr;
  float* part = nullptr;               // split-K partials (largest user)
  size_t part_bytes = 0;
  float* gu32 = nullptr;               // f32 path: gate|up GEMM output
  float* logits = nullptr;             // [B or rows][V]
  int64_t logits_rows = 0;
  float* attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  void* argmax_scratch = nullptr;      // [B][64] (value, index) partials
  void* gather_scratch = nullptr;      // tensor parallel: all-gathered argmax partials / logits
  size_t gather_bytes = 0;
  // MoE scratch, sized for rows_cap tokens (capacity = tokens * top_k slots per peer)
  float* moe_logits = nullptr;
  float* moe_topw = nullptr;
  int* moe_topi = nullptr;
  int* moe_ints = nullptr;             // cursor | count | offsets | cursor2 | send_meta | recv_meta | pair_slot | slot_pos | recv counts
  size_t moe_ints_n = 0;
  void *moe_send = nullptr, *moe_recv = nullptr, *moe_xs = nullptr, *moe_hs = nullptr;
  float *moe_ys = nullptr, *moe_ret = nullptr, *moe_back = nullptr, *moe_tmp = nullptr;
  int* route_rec = nullptr;            // option record_routing: every MoE layer's top-k expert ids of the last forward, [n_moe][rows_cap][k]
  int64_t route_rows = 0;              // rows of the forward recorded last
  cudaGraphExec_t graph = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float prefill_ms = 0.f, decode_ms = 0.f;
  int host_pos = 0;                    // tokens so far (all sequences advance together)
  int graph_kernels = 0;               // kernels in one captured decode step
  int graph_epoch = -1;                // option epoch the graph was captured under
  // GenerationConfig sampling (generate.nim:12-58); off = greedy argmax
  bool samp_on = false;
  float samp_temperature = 1.f, samp_top_p = 1.f, samp_min_p = 0.f, samp_rep = 1.f;
  int samp_top_k = 0, samp_do_sample = 0;
  std::vector<uint64_t> samp_seeds;    // one per sequence; keys restart from these on reset
  int *samp_hist = nullptr, *samp_hist_len = nullptr, *samp_steps = nullptr;  // [B][max_len], [B], [B]
  uint32_t* samp_keys = nullptr;       // [B][2]
  float *samp_work = nullptr, *samp_logprob = nullptr;  // [B][V], [B][max_len]
  // Paged lanes (continuous batching): a shared pool of KV pages handed out on demand
  bool paged = false;
  int num_blocks = 0;                  // pages in the pool; page 0 is the scratch page of idle lanes
  std::vector<int> free_blocks;        // as PagedKvCache.freeBlocks (generate.nim:75,86-88)
  std::vector<int> lane_len;           // tokens in the cache per lane
  std::vector<char> lane_active;
  std::vector<std::vector<int>> lane_pages;
  int* d_active = nullptr;             // [B] or nullptr (every lane active)
  int* d_ids_prefill = nullptr;        // ids of a single-lane prefill
};

namespace rewb {
namespace {

// Sampling restarts with every generate call: keys back to initKey(seed), step counters to zero.
int samp_restart(rewb200_session* s) {
  Ctx* c = s->m->c;
  std::vector<uint32_t> k((size_t)s->B * 2);
  for (int b = 0; b < s->B; ++b) {  // initKey (src/rew/rng.nim:60-64)
    k[2 * b] = (uint32_t)(s->samp_seeds[b] & 0xFFFFFFFFull);
    k[2 * b + 1] = (uint32_t)(s->samp_seeds[b] >> 32);
  }
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaMemcpy(s->samp_keys, k.data(), k.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
  RB_CUDA(cudaMemset(s->samp_steps, 0, s->B * sizeof(int)));
  RB_CUDA(cudaMemset(s->samp_hist_len, 0, s->B * sizeof(int)));
  return REWB200_OK;
}

int dev_alloc(rewb200_model* m, void** p, size_t bytes) {
  RB_CUDA(cudaMalloc(p, std::max<size_t>(bytes, 256)));
  m->allocs.push_back(*p);
  m->weight_bytes += (int64_t)bytes;
  return REWB200_OK;
}

bool layer_is_moe(const rewb200_config& c, int l) { return c.n_routed > 0 && !(c.first_dense > 0 && l == 0); }

int alloc_lin(rewb200_model* m, LinW* w, int64_t K, int64_t N) {
  w->K = K;
  w->N = N;
  RB_TRY(dev_alloc(m, &w->w, (size_t)K * N * dtype_size(m->cfg.dtype)));
  RB_TRY(dev_alloc(m, (void**)&w->b, (size_t)N * sizeof(float)));
  RB_CUDA(cudaMemsetAsync(w->b, 0, (size_t)N * sizeof(float), m->c->stream));
  return REWB200_OK;
}

// Tensor index -> (layer, slot).  Slots follow the canonical order in the header.
struct TensorRef {
  int layer;  // -1: embed, -2: final
  int slot;
};
int locate(const rewb200_model* m, int64_t index, TensorRef* out) {
  const rewb200_config& c = m->cfg;
  if (index == 0) {
    *out = {-1, 0};
    return REWB200_OK;
  }
  int64_t i = 1;
  for (int l = 0; l < c.n_layers; ++l) {
    const int64_t n = 12 + (layer_is_moe(c, l) ? 2 + 6 * (int64_t)(c.n_shared + c.n_routed) : 6);
    if (index < i + n) {
      *out = {l, (int)(index - i)};
      return REWB200_OK;
    }
    i += n;
  }
  if (index < i + 4) {
    *out = {-2, (int)(index - i)};
    return REWB200_OK;
  }
  return fail("tensor index " + std::to_string(index) + " out of range");
}

int upload_stage(rewb200_model* m, const float* host, int64_t numel) {
  Ctx* c = m->c;
  const size_t bytes = (size_t)numel * sizeof(float);
  if (bytes > m->stage_bytes) {
    if (m->stage) RB_CUDA(cudaFree(m->stage));
    RB_CUDA(cudaMalloc((void**)&m->stage, bytes));
    m->stage_bytes = bytes;
  }
  size_t off = 0;
  while (off < bytes) {
    const size_t n = std::min(c->pinned_bytes, bytes - off);
    memcpy(c->pinned, (const char*)host + off, n);
    RB_CUDA(cudaMemcpyAsync((char*)m->stage + off, c->pinned, n, cudaMemcpyHostToDevice, c->stream));
    RB_CUDA(cudaStreamSynchronize(c->stream));
    off += n;
  }
  return REWB200_OK;
}

// Copies a [rows, cols] window of the staged f32 tensor into a device matrix
// with column mapping dst_col = (c / gran) * gstride + c % gran + off.
int scatter(rewb200_model* m, int64_t src_ld, int64_t row0, int64_t col0, int64_t rows, int64_t cols, void* dst,
            bool dst_model_dtype, int64_t ldd, int64_t gran, int64_t gstride, int64_t off) {
  const int64_t n = rows * cols;
  if (n == 0) return REWB200_OK;
  const int bf = (dst_model_dtype && m->cfg.dtype == REWB200_BF16) ? 1 : 0;
  scatter_cols_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, m->c->stream>>>(m->stage, src_ld, row0, col0, rows, cols,
                                                                                dst, bf, ldd, gran, gstride, off);
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

// cudaMalloc of one activation buffer.  The option "inject_alloc_fail" = n makes the n-th call from now
// fail on the host without touching the device (a test hook for the failed-growth path).
int acts_alloc(Ctx* c, void** p, size_t bytes) {
  if (c->inject_alloc_fail > 0 && --c->inject_alloc_fail == 0) return fail("cudaMalloc: out of memory (injected)");
  RB_CUDA(cudaMalloc(p, bytes));
  return REWB200_OK;
}
template <typename T>
int acts_alloc(Ctx* c, T** p, size_t bytes) {
  return acts_alloc(c, (void**)p, bytes);
}

int ensure_acts(rewb200_session* s, int64_t rows, int64_t logits_rows) {
  rewb200_model* m = s->m;
  const rewb200_config& c = m->cfg;
  const size_t es = dtype_size(c.dtype);
  if (rows > s->rows_cap) {
    RB_CUDA(cudaStreamSynchronize(m->c->stream));
    void** ptrs[] = {(void**)&s->x_res, &s->xn, &s->q, &s->attn, &s->h, (void**)&s->part, (void**)&s->gu32,
                     (void**)&s->moe_logits, (void**)&s->moe_topw, (void**)&s->moe_topi, (void**)&s->moe_ints, &s->moe_send,
                     &s->moe_recv, &s->moe_xs, &s->moe_hs, (void**)&s->moe_ys, (void**)&s->moe_ret, (void**)&s->moe_back,
                     (void**)&s->moe_tmp, (void**)&s->route_rec};
    // From here until every allocation below has succeeded the session holds no activation buffers: a failed
    // growth must leave it in a state where the next call allocates again instead of launching on NULL.
    s->rows_cap = 0;
    s->part_bytes = 0;
    if (s->graph) {
      cudaGraphExecDestroy(s->graph);
      s->graph = nullptr;
    }
    for (void** p : ptrs)
      if (*p) {
        void* q = *p;
        *p = nullptr;
        RB_CUDA(cudaFree(q));
      }
    int64_t fmax = 0;
    for (const LayerDev& L : m->layers) fmax = std::max(fmax, L.ffn_local);
    if (c.n_routed > 0) fmax = std::max<int64_t>(fmax, c.moe_ffn);
    RB_TRY(acts_alloc(m->c, (void**)&s->x_res, (size_t)rows * c.d_model * sizeof(float)));
    RB_TRY(acts_alloc(m->c, &s->xn, (size_t)rows * c.d_model * es));
    RB_TRY(acts_alloc(m->c, &s->q, (size_t)rows * std::max<int64_t>(m->nq, 1) * es));
    RB_TRY(acts_alloc(m->c, &s->attn, (size_t)rows * std::max<int64_t>(m->nq, 1) * es));
    RB_TRY(acts_alloc(m->c, &s->h, (size_t)rows * std::max<int64_t>(fmax, 1) * es));
    const int64_t widest = std::max<int64_t>(m->nqkv, c.d_model);
    // up to 16 split-K slabs of the widest residual-side Linear, or 4 of gate|up, at steps of at most 64 rows
    const size_t small_rows = (size_t)std::min<int64_t>(rows, 64);
    s->part_bytes = small_rows * std::max<size_t>(16 * widest, 4 * 2 * fmax) * sizeof(float);
    s->part_bytes = std::max(s->part_bytes, (size_t)std::min<int64_t>(rows, 256) * 4 * widest * sizeof(float));  // 4 slabs up to 256 rows
    s->part_bytes = std::max(s->part_bytes, (size_t)rows * widest * sizeof(float));
    if (c.weight_quant)  // the quantised gate|up GEMV leaves up to 4 slabs of [32][2f] here at decode sizes
      s->part_bytes = std::max(s->part_bytes, (size_t)32 * std::max<size_t>(16 * widest, 4 * 2 * fmax) * sizeof(float));
    RB_TRY(acts_alloc(m->c, (void**)&s->part, s->part_bytes));
    if (c.dtype == REWB200_F32) RB_TRY(acts_alloc(m->c, (void**)&s->gu32, (size_t)rows * 2 * std::max<int64_t>(fmax, 1) * sizeof(float)));
    if (c.n_routed > 0) {
      const int ep = c.ep_size, k = c.top_k, E_l = c.n_routed / ep;
      const int64_t cap = rows * k, slots = cap * ep;
      RB_TRY(acts_alloc(m->c, (void**)&s->moe_logits, (size_t)std::max<int64_t>(rows, 8 * std::min<int64_t>(rows, 64)) * c.n_routed * sizeof(float)));  // or 8 split-K slabs of a small step
      RB_TRY(acts_alloc(m->c, (void**)&s->moe_topw, (size_t)rows * k * sizeof(float)));
      RB_TRY(acts_alloc(m->c, (void**)&s->moe_topi, (size_t)rows * k * sizeof(int)));
      // the last 16 ints hold the per-peer counts this rank receives (prefix exchange of large steps)
      s->moe_ints_n = (size_t)(ep + 3 * (E_l + 1) + 3 * slots + rows * k) + 16;
      RB_TRY(acts_alloc(m->c, (void**)&s->moe_ints, s->moe_ints_n * sizeof(int)));
      RB_TRY(acts_alloc(m->c, (void**)&s->moe_tmp, (size_t)rows * c.d_model * sizeof(float)));
      if (m->c->record_routing) RB_TRY(acts_alloc(m->c, (void**)&s->route_rec, (size_t)c.n_layers * rows * k * sizeof(int)));
      if (c.dtype == REWB200_BF16) {
        RB_TRY(acts_alloc(m->c, &s->moe_send, (size_t)slots * c.d_model * es));
        if (ep > 1) RB_TRY(acts_alloc(m->c, &s->moe_recv, (size_t)slots * c.d_model * es));
        RB_TRY(acts_alloc(m->c, &s->moe_xs, (size_t)(slots + 128) * c.d_model * es));
        RB_TRY(acts_alloc(m->c, &s->moe_hs, (size_t)(slots + 128) * c.moe_ffn * es));
        RB_CUDA(cudaMemset(s->moe_xs, 0, (size_t)(slots + 128) * c.d_model * es));
        RB_CUDA(cudaMemset(s->moe_hs, 0, (size_t)(slots + 128) * c.moe_ffn * es));
        RB_TRY(acts_alloc(m->c, (void**)&s->moe_ys, (size_t)slots * c.d_model * sizeof(float)));
        RB_TRY(acts_alloc(m->c, (void**)&s->moe_ret, (size_t)slots * c.d_model * sizeof(float)));
        if (ep > 1) RB_TRY(acts_alloc(m->c, (void**)&s->moe_back, (size_t)slots * c.d_model * sizeof(float)));
      }
    }
    s->rows_cap = rows;
  }
  if (logits_rows > s->logits_rows) {
    RB_CUDA(cudaStreamSynchronize(m->c->stream));
    s->logits_rows = 0;
    if (s->graph) {
      cudaGraphExecDestroy(s->graph);
      s->graph = nullptr;
    }
    if (s->logits) {
      float* q = s->logits;
      s->logits = nullptr;
      RB_CUDA(cudaFree(q));
    }
    RB_TRY(acts_alloc(m->c, (void**)&s->logits, (size_t)logits_rows * m->vocab_l * sizeof(float)));
    s->logits_rows = logits_rows;
  }
  return REWB200_OK;
}

// y = x @ W for the model dtype.  `partial` selects the f32 split-K slab
// output (bias deferred to the consumer) over a finished output with bias.
int run_linear(rewb200_session* s, const LinW& w, const void* x, int64_t ldx, int64_t rows, bool partial, int epi,
               void* out, int64_t ldo, int* ksplit_out, const QkvPostArgs* fuse_qkv = nullptr, bool* fused = nullptr) {
  Ctx* c = s->m->c;
  if (fused) *fused = false;
  if (w.quant && rows <= 32) {
    // weight-only NF4: codes dequantised inside the GEMV, f32 split-K slabs
    int ks = nf4_pick_ksplit(c, w.K, w.N, rows);
    while (ks > 1 && (size_t)ks * rows * w.N * sizeof(float) > s->part_bytes) --ks;
    RB_REQUIRE((size_t)ks * rows * w.N * sizeof(float) <= s->part_bytes, "split-K scratch too small for the quantised Linear");
    RB_TRY(nf4_gemv_launch(c, w.nf4, (const bf16*)x, ldx, rows, ks, s->part));
    if (partial) {
      if (ksplit_out) *ksplit_out = ks;
      return REWB200_OK;
    }
    RB_REQUIRE(epi == EPI_SWIGLU_BF16, "quantised Linear: only the SwiGLU epilogue is fused");
    const int64_t n = rows * (w.N / 2);
    RB_CUDA(launch_k(swiglu_slabs_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, c->stream, c->use_pdl,
                     (const float*)s->part, ks, rows, w.N / 2, (const float*)w.b, (bf16*)out));
    ++g_launch_total;
    return REWB200_OK;
  }
  if (w.quant)  // prefill: expand the codes into the shared bf16 scratch (device column order), then the dense Linear
    RB_TRY(nf4_dequant_launch(c, w.nf4, (bf16*)w.w, w.N, w.cm));
  if (s->m->cfg.dtype == REWB200_BF16) {
    int ks = 1;
    if (partial) {
      ks = linear_bf16_pick_ksplit(c, rows, w.K, w.N);
      if (rows > 64 && c->linear_impl != 2) ks = 1;  // split-K above 64 rows is exercised on the tcgen05 Linear only
      while (ks > 1 && (size_t)ks * rows * ldo * sizeof(float) > s->part_bytes) ks /= 2;
      // decode-size steps: sum the K slices inside thread-block clusters, one slab (or finished q|k|v) comes out
      const int kc = std::min(ks, 8);
      if ((c->splitk_cluster & (fuse_qkv ? 1 : 2)) && linear_tc_cluster_ok(c, w.plan, rows, kc)) {
        if (ksplit_out) *ksplit_out = 1;
        if (fused) *fused = fuse_qkv != nullptr;
        return linear_tc_cluster_launch(c, w.plan, (const bf16*)x, ldx, rows, kc, (float*)out, ldo, fuse_qkv);
      }
    }
    if (ksplit_out) *ksplit_out = ks;
    if (!partial && epi == EPI_SWIGLU_BF16 && rows <= 64 && w.N % 16 == 0 && c->gu_split) {
      // a gate|up with too few feature tiles to fill the GPU: split K, then sum + SwiGLU in a second small launch
      int kg = std::min(4, linear_bf16_pick_ksplit(c, rows, w.K, w.N));
      while (kg > 1 && (size_t)kg * rows * w.N * sizeof(float) > s->part_bytes) kg /= 2;
      if (kg > 1) {
        RB_TRY(linear_bf16_launch(c, w.plan, (const bf16*)x, ldx, rows, EPI_PARTIAL_F32, kg, s->part, w.N, nullptr, nullptr, 0));
        const int64_t n = rows * (w.N / 16);
        RB_REQUIRE(ldo == w.N / 2, "SwiGLU output rows must be dense");
        RB_CUDA(launch_k(swiglu_slabs_il_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, c->stream, c->use_pdl,
                         (const float*)s->part, kg, rows, w.N / 2, (const float*)w.b, (bf16*)out));
        ++g_launch_total;
        return REWB200_OK;
      }
    }
    return linear_bf16_launch(c, w.plan, (const bf16*)x, ldx, rows, partial ? EPI_PARTIAL_F32 : epi, ks, out, ldo,
                              partial ? nullptr : w.b, nullptr, 0);
  }
  if (ksplit_out) *ksplit_out = 1;
  RB_REQUIRE(ldx == w.K && ldo == w.N, "f32 Linear expects dense rows");
  return gemm_f32_launch(c, (const float*)x, (const float*)w.w, partial ? nullptr : w.b, (float*)out, rows, w.K, w.N);
}

// Routed experts of one MoE layer for the normalised rows in s->xn: router, top-k, dispatch to the
// owning ranks, grouped expert GEMMs, return, weighted combine into slab 0 of s->part
// (DeepSeekMoE.forward, src/rew/models/deepseek.nim:132-144).
// Bytes of the peer heap's all-to-all region a step of `slots` slot rows needs (activations, expert ids, f32 results).
size_t a2a_need(int64_t slots, int64_t d, size_t es, int64_t* off_meta, int64_t* off_back) {
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t x = up((size_t)slots * d * es), meta = up((size_t)slots * sizeof(int));
  if (off_meta) *off_meta = (int64_t)x;
  if (off_back) *off_back = (int64_t)(x + meta);
  return x + meta + up((size_t)slots * d * sizeof(float));
}

// Whether the expert-parallel exchange of a step of `rows` tokens runs over the peer heap.
bool ep_uses_peer_heap(const rewb200_model* m, int64_t rows) {
  const rewb200_config& cf = m->cfg;
  if (cf.ep_size <= 1 || m->c->ep_prefix == 0 || m->c->ep_prefix == 1) return false;  // options capacity / prefix: NCCL
  const PeerInfo* pi = comm_peer_info(m->slot);
  return pi != nullptr && pi->world == cf.ep_size && pi->a2a[pi->rank] != nullptr &&
         a2a_need(rows * cf.top_k * cf.ep_size, cf.d_model, dtype_size(cf.dtype), nullptr, nullptr) <= pi->a2a_bytes;
}

int moe_routed(rewb200_session* s, LayerDev& L, int64_t rows, bool accumulate, float* out = nullptr, int moe_index = 0) {
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  const rewb200_config& cf = m->cfg;
  MoeDev& X = L.x;
  const int64_t d = cf.d_model, f = X.f;
  const int k = cf.top_k, ep = cf.ep_size, E_l = X.E_l;
  const int dt = cf.dtype;
  // expert parallel over the peer heap: the routing kernel also clears the dispatch kernel's per-peer cursors
  const bool peer = ep_uses_peer_heap(m, rows);
  int* const clear = peer ? s->moe_ints : nullptr;
  bool cleared = false;
  if (dt == REWB200_BF16 && rows <= 64) {
    // the router has one feature tile: split K over several CTAs, the routing kernel sums the slabs
    const int nkb = (int)((d + 63) / 64);
    int ks = 1;
    while (ks < 8 && nkb / (ks * 2) >= 4) ks *= 2;
    RB_TRY(linear_bf16_launch(c, X.router.plan, (const bf16*)s->xn, d, rows, EPI_PARTIAL_F32, ks, s->moe_logits, cf.n_routed,
                              nullptr, nullptr, 0));
    RB_TRY(moe_route_slabs_launch(c, s->moe_logits, ks, rows * cf.n_routed, X.router.b, rows, cf.n_routed, k, s->moe_topw,
                                  s->moe_topi, clear, peer ? ep : 0));
    cleared = peer;
  } else {
    if (dt == REWB200_BF16)
      RB_TRY(linear_bf16_launch(c, X.router.plan, (const bf16*)s->xn, d, rows, EPI_BIAS_F32, 1, s->moe_logits, cf.n_routed,
                                X.router.b, nullptr, 0));
    else
      RB_TRY(gemm_f32_launch(c, (const float*)s->xn, (const float*)X.router.w, X.router.b, s->moe_logits, rows, d, cf.n_routed));
    RB_TRY(moe_route_launch(c, s->moe_logits, rows, cf.n_routed, k, s->moe_topw, s->moe_topi));
  }
  if (s->route_rec) {
    RB_CUDA(cudaMemcpyAsync(s->route_rec + (size_t)moe_index * s->rows_cap * k, s->moe_topi, (size_t)rows * k * sizeof(int),
                            cudaMemcpyDeviceToDevice, c->stream));
    s->route_rows = rows;
  }
  if (dt == REWB200_F32) {
    // parity path: every local expert on every token, masked by its routing weight, as the reference does
    for (int e = 0; e < E_l; ++e) {
      const float* gw = (const float*)X.gu + (size_t)e * d * 2 * f;
      const float* dw = (const float*)X.down + (size_t)e * f * d;
      RB_TRY(gemm_f32_launch(c, (const float*)s->xn, gw, X.gu_b + (size_t)e * 2 * f, s->gu32, rows, d, 2 * f));
      const int64_t n = rows * f;
      swiglu_rows_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(s->gu32, (float*)s->h, rows, f);
      RB_CUDA(cudaGetLastError());
      RB_TRY(gemm_f32_launch(c, (const float*)s->h, dw, X.down_b + (size_t)e * d, s->moe_tmp, rows, f, d));
      const int64_t nd = rows * d;
      moe_dense_acc_kernel<<<(unsigned)((nd + 255) / 256), 256, 0, c->stream>>>(s->moe_tmp, s->moe_topw, s->moe_topi, k, e, rows,
                                                                                d, s->part, (accumulate || e > 0) ? 1 : 0);
      RB_CUDA(cudaGetLastError());
      g_launch_total += 2;
    }
    return REWB200_OK;
  }
  const int64_t cap = rows * k, slots = cap * ep;
  int* cursor = s->moe_ints;
  int* count = cursor + ep;
  int* offsets = count + (E_l + 1);
  int* cursor2 = offsets + (E_l + 1);
  int* send_meta = cursor2 + (E_l + 1);
  int* recv_meta = send_meta + slots;
  int* slot_pos = recv_meta + slots;
  int* pair_slot = slot_pos + slots;
  if (ep == 1 && cap <= 2048) {
    // every expert is local and the step is small: one kernel sorts the pairs by expert and copies the
    // rows, the combine reads the expert outputs in place (no slot arrays, no atomics, no return copy)
    RB_TRY(moe_group_local_launch(c, s->xn, dt, s->moe_topi, rows, k, d, E_l, offsets, s->moe_xs, pair_slot));
    const int max_rows_l = (int)std::min<int64_t>(rows, cap);
    RB_TRY(linear_bf16_launch(c, X.plan_gu, (const bf16*)s->moe_xs, d, cap, EPI_SWIGLU_BF16, 1, s->moe_hs, f, X.gu_b, offsets,
                              max_rows_l));
    RB_TRY(linear_bf16_launch(c, X.plan_down, (const bf16*)s->moe_hs, f, cap, EPI_BIAS_F32, 1, s->moe_ys, d, X.down_b, offsets,
                              max_rows_l));
    return moe_combine_launch(c, s->moe_ys, pair_slot, s->moe_topw, rows, k, d, out ? out : s->part, accumulate ? 1 : 0);
  }
  if (peer) {
    const PeerInfo* pi = comm_peer_info(m->slot);
    A2aArgs a;
    memset(&a, 0, sizeof(a));
    a.world = ep;
    a.my_rank = pi->rank;
    for (int r = 0; r < ep; ++r) {
      a.cells[r] = pi->a2a_flags[r];
      a.region[r] = pi->a2a[r];
    }
    a.off_x = 0;
    a2a_need(slots, d, dtype_size(dt), &a.off_meta, &a.off_back);
    a.arrive = pi->epoch + 2;
    a.epoch = pi->epoch + 1;
    a.offset = moe_index + 1;
    a.status = c->d_status;
    // large steps count with atomics: clear the counters; small ones need only the cursors, cleared by the routing kernel
    if (!cleared || slots > 4096) RB_TRY(moe_reset_launch(c, cursor, ep, count, E_l + 1, send_meta, 0));
    RB_TRY(moe_dispatch_peer_launch(c, s->xn, dt, s->moe_topi, rows, k, d, E_l, (int)cap, cursor, pair_slot, a));
    RB_TRY(moe_group_peer_launch(c, dt, (int)slots, (int)cap, d, E_l, count, offsets, cursor2, s->moe_xs, slot_pos, a));
    const int max_rows_p = (int)std::min<int64_t>(rows * ep, slots);
    RB_TRY(linear_bf16_launch(c, X.plan_gu, (const bf16*)s->moe_xs, d, slots, EPI_SWIGLU_BF16, 1, s->moe_hs, f, X.gu_b, offsets,
                              max_rows_p));
    RB_TRY(linear_bf16_launch(c, X.plan_down, (const bf16*)s->moe_hs, f, slots, EPI_BIAS_F32, 1, s->moe_ys, d, X.down_b, offsets,
                              max_rows_p));
    RB_TRY(moe_return_peer_launch(c, s->moe_ys, slot_pos, (int)slots, (int)cap, d, a));
    return moe_combine_peer_launch(c, pair_slot, s->moe_topw, rows, k, d, out ? out : s->part, accumulate ? 1 : 0, a);
  }
  RB_TRY(moe_reset_launch(c, cursor, ep, count, E_l + 1, send_meta, (int)slots));
  RB_TRY(moe_dispatch_launch(c, s->xn, dt, s->moe_topi, rows, k, d, E_l, (int)cap, cursor, s->moe_send, send_meta, pair_slot));
  const void* rx = s->moe_send;
  const int* rmeta = send_meta;
  // Large steps outside a captured graph (prefill): exchange the per-peer pair counts first and move only the
  // occupied prefix of every slot array instead of its worst-case capacity.  Decode steps keep the fixed-size
  // exchange, which needs no host round trip and can be captured.
  cudaStreamCaptureStatus cap_st = cudaStreamCaptureStatusNone;
  RB_CUDA(cudaStreamIsCapturing(c->stream, &cap_st));
  const bool prefix = ep > 1 && ep <= 16 && (c->ep_prefix == 1 || (c->ep_prefix >= 2 && ep >= 4)) &&
                      cap_st == cudaStreamCaptureStatusNone && cap >= 64;
  int* h_send_rows = c->h_status + 16;  // pinned: [16 send | 16 recv]
  int* h_recv_rows = c->h_status + 32;
  if (prefix) {
    int* recv_cnt = s->moe_ints + s->moe_ints_n - 16;
    RB_TRY(comm_alltoall_bytes(c, m->slot, cursor, recv_cnt, sizeof(int)));
    RB_CUDA(cudaMemcpyAsync(h_send_rows, cursor, ep * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    RB_CUDA(cudaMemcpyAsync(h_recv_rows, recv_cnt, ep * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    RB_CUDA(cudaMemsetAsync(recv_meta, 0xFF, (size_t)slots * sizeof(int), c->stream));  // -1: slots past a prefix stay empty
    RB_CUDA(cudaStreamSynchronize(c->stream));
    for (int p = 0; p < ep; ++p)
      RB_REQUIRE(h_send_rows[p] >= 0 && h_send_rows[p] <= cap && h_recv_rows[p] >= 0 && h_recv_rows[p] <= cap,
                 "expert-parallel dispatch: pair count out of range");
    RB_TRY(comm_alltoallv_rows(c, m->slot, s->moe_send, s->moe_recv, (size_t)cap * d * dtype_size(dt), (size_t)d * dtype_size(dt),
                               h_send_rows, h_recv_rows));
    RB_TRY(comm_alltoallv_rows(c, m->slot, send_meta, recv_meta, (size_t)cap * sizeof(int), sizeof(int), h_send_rows, h_recv_rows));
    rx = s->moe_recv;
    rmeta = recv_meta;
  } else if (ep > 1) {
    RB_TRY(comm_alltoall_bytes(c, m->slot, s->moe_send, s->moe_recv, (size_t)cap * d * dtype_size(dt)));
    RB_TRY(comm_alltoall_bytes(c, m->slot, send_meta, recv_meta, (size_t)cap * sizeof(int)));
    rx = s->moe_recv;
    rmeta = recv_meta;
  }
  RB_TRY(moe_group_launch(c, rx, dt, rmeta, (int)slots, d, E_l, count, offsets, cursor2, s->moe_xs, slot_pos));
  // an expert receives each token at most once: at most rows * ep rows per group
  const int max_rows = (int)std::min<int64_t>(rows * ep, slots);
  RB_TRY(linear_bf16_launch(c, X.plan_gu, (const bf16*)s->moe_xs, d, slots, EPI_SWIGLU_BF16, 1, s->moe_hs, f, X.gu_b, offsets,
                            max_rows));
  RB_TRY(linear_bf16_launch(c, X.plan_down, (const bf16*)s->moe_hs, f, slots, EPI_BIAS_F32, 1, s->moe_ys, d, X.down_b, offsets,
                            max_rows));
  RB_TRY(moe_return_launch(c, s->moe_ys, slot_pos, (int)slots, d, s->moe_ret));
  const float* back = s->moe_ret;
  if (prefix) {  // results go back the way the pairs came: what peer p sent here returns to p
    RB_TRY(comm_alltoallv_rows(c, m->slot, s->moe_ret, s->moe_back, (size_t)cap * d * sizeof(float), (size_t)d * sizeof(float),
                               h_recv_rows, h_send_rows));
    back = s->moe_back;
  } else if (ep > 1) {
    RB_TRY(comm_alltoall_bytes(c, m->slot, s->moe_ret, s->moe_back, (size_t)cap * d * sizeof(float)));
    back = s->moe_back;
  }
  return moe_combine_launch(c, back, pair_slot, s->moe_topw, rows, k, d, out ? out : s->part, accumulate ? 1 : 0);
}

// Copies the last-position logits [B, vocab] to the host; under tensor parallelism the
// vocabulary slices are all-gathered first and re-interleaved on the host.
int fetch_logits(rewb200_session* s, int64_t rows, float* host) {
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  const int tp = m->cfg.tp_size;
  if (tp == 1) {
    RB_CUDA(cudaMemcpyAsync(host, s->logits, (size_t)rows * m->cfg.vocab * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    RB_CUDA(cudaStreamSynchronize(c->stream));
    return REWB200_OK;
  }
  const size_t per = (size_t)rows * m->vocab_l * sizeof(float);
  RB_REQUIRE(per * tp <= s->gather_bytes, "logit gather buffer too small for this many rows");
  RB_TRY(comm_allgather_bytes(c, m->slot, s->logits, s->gather_scratch, per));
  std::vector<float> tmp((size_t)rows * m->cfg.vocab);
  RB_CUDA(cudaMemcpyAsync(tmp.data(), s->gather_scratch, per * tp, cudaMemcpyDeviceToHost, c->stream));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  for (int r = 0; r < tp; ++r)
    for (int64_t i = 0; i < rows; ++i)
      memcpy(host + i * m->cfg.vocab + r * m->vocab_l, tmp.data() + ((size_t)r * rows + i) * m->vocab_l, m->vocab_l * sizeof(float));
  return REWB200_OK;
}

// Per-category device times of one forward (REW_B200_TRACE-style measurement aid): an event after the
// launches of each category, elapsed times summed per category after a synchronisation.  Events between
// kernels switch programmatic dependent launch off at those points, so the sum exceeds the untraced step;
// the split is what it is for.
enum TraceCat : int { TC_EMBED = 0, TC_QKV, TC_QKV_POST, TC_ATTN, TC_O, TC_NORM_ATTN, TC_GATE_UP, TC_DOWN, TC_MOE, TC_NORM_FFN, TC_HEAD, TC_COUNT };
struct Trace {
  std::vector<cudaEvent_t> ev;
  std::vector<int> cat;
  cudaStream_t st = nullptr;
  int begin(cudaStream_t s) {
    st = s;
    return mark(-1);
  }
  int mark(int c) {
    cudaEvent_t e;
    RB_CUDA(cudaEventCreate(&e));
    RB_CUDA(cudaEventRecord(e, st));
    ev.push_back(e);
    cat.push_back(c);
    return REWB200_OK;
  }
  int finish(float* ms) {  // ms[TC_COUNT]
    for (int i = 0; i < TC_COUNT; ++i) ms[i] = 0.f;
    RB_CUDA(cudaStreamSynchronize(st));
    for (size_t i = 1; i < ev.size(); ++i) {
      float t = 0.f;
      RB_CUDA(cudaEventElapsedTime(&t, ev[i - 1], ev[i]));
      if (cat[i] >= 0 && cat[i] < TC_COUNT) ms[cat[i]] += t;
    }
    return REWB200_OK;
  }
  ~Trace() {
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
  }
};

struct FwdOpts {
  Trace* trace = nullptr;     // when set, an event follows every category of launches
  int S = 1;
  int rope_shift = 0;
  int causal = 1;
  bool all_logits = false;  // lm_head on every row instead of the last position
  bool from_device_ids = false;
  // Lanes [b0, b0 + nb) of the session only (nb < 0: all).  The per-lane arrays (positions, block table,
  // next ids, logits rows, sampling state) are indexed from b0; ids_src overrides where the nb*S input
  // ids are read, so that a single-lane prefill does not disturb the other lanes' pending tokens.
  int b0 = 0, nb = -1;
  const int* ids_src = nullptr;
  bool record_out = true;    // append the new ids to the session's [step][B] output buffer
};

// Enqueues one forward over rows = B*S tokens whose ids are in s->d_ids.
int enqueue_forward(rewb200_session* s, const FwdOpts& o) {
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  const rewb200_config& cf = m->cfg;
  const int b0 = o.b0, nb = o.nb < 0 ? s->B : o.nb;
  const int64_t rows = (int64_t)nb * o.S;
  const int64_t d = cf.d_model;
  int* const pos = s->d_pos + b0;
  const int* const block_table = s->block_table + (size_t)b0 * s->max_pages;
  float* const logits = o.all_logits ? s->logits : s->logits + (size_t)b0 * m->vocab_l;
  int* const next = s->d_next + b0;
  const int dt = cf.dtype;

  // A captured decode step is replayed as one graph launch: positions, block tables and all cache rows but
  // the newest were written before that launch, which is what lets two kernels read them ahead of their
  // stream dependency.  Plain launches (prefill, REW_B200_NO_GRAPH) chain across calls and get no such promise.
  cudaStreamCaptureStatus cap_st = cudaStreamCaptureStatusNone;
  RB_CUDA(cudaStreamIsCapturing(c->stream, &cap_st));
  const bool in_graph = cap_st == cudaStreamCaptureStatusActive && o.S == 1;
  NormArgs na;
  memset(&na, 0, sizeof(na));
  na.x_res = s->x_res;
  na.d = d;
  na.eps = cf.eps;
  na.norm_kind = cf.norm_kind;
  na.out = s->xn;
  na.out_dtype = dt;
  na.vocab = cf.vocab;
  na.status = c->d_status;
  na.embed_dtype = dt;

  // embedding gather + first norm
  {
    NormArgs a = na;
    a.embed = m->embed;
    a.ids = o.ids_src ? o.ids_src : s->d_ids;
    a.gamma = m->layers[0].ln1g;
    a.beta = m->layers[0].ln1b;
    if (o.trace) RB_TRY(o.trace->begin(c->stream));
    RB_TRY(residual_norm_launch(c, a, rows));
    if (o.trace) RB_TRY(o.trace->mark(TC_EMBED));
  }
  // Tensor parallel: steps of up to 64 rows sum the row-parallel partials inside residual_norm (each CTA
  // pushes its columns to every rank's heap and adds the peers' in rank order); larger ones go through
  // NCCL, bf16 models with a bf16 payload (the o / down projections then write one bf16 slab, no bias).
  const PeerInfo* pi = cf.tp_size > 1 ? comm_peer_info(m->slot) : nullptr;
  // a slot holds the step as 16-byte lines of 8 payload bytes each
  const bool oneshot = pi != nullptr && pi->buf_bytes > 0 && d % 4 == 0 && rows <= 64 &&
                       (size_t)rows * d * dtype_size(dt) * 2 <= pi->buf_bytes && pi->world == cf.tp_size;
  // (steps above 256 rows never split K, so a bf16 model's o / down projections write one bf16 slab there on one GPU
  // too: half the bytes between the GEMM and the residual+norm kernel, rounded where the reference's bf16 Linear rounds)
  const bool tp_bf16_slab = (cf.tp_size > 1 ? rows > 64 : (rows > 256 && cf.n_routed == 0)) && !oneshot && dt == REWB200_BF16 && d % 4 == 0;  // smaller steps keep split-K slabs
  // ... and when the heap's bulk region holds a scatter and a gather buffer of the step, the sum itself runs
  // over the heap too (two-shot: reduce-scatter and all-gather by peer stores) instead of through NCCL
  const size_t pay = dtype_size(dt);
  const bool twoshot = cf.tp_size > 1 && !oneshot && rows > 64 && pi != nullptr && pi->world == cf.tp_size &&
                       pi->a2a[pi->rank] != nullptr && d % ((int64_t)cf.tp_size * (16 / pay)) == 0 &&
                       2 * (size_t)rows * d * pay <= pi->a2a_bytes && c->tp_twoshot;
  auto tp_reduce = [&](int l, int which, int& ks, NormArgs& a) -> int {
    if (cf.tp_size <= 1) {
      if (tp_bf16_slab) {
        ks = 1;
        a.nsplit = 1;
        a.partial_bf16 = 1;
      }
      return REWB200_OK;
    }
    if (oneshot) {
      a.n_peers = pi->world;
      a.my_rank = pi->rank;
      a.payload_bf16 = dt == REWB200_BF16 ? 1 : 0;
      a.two_shot = c->tp_exchange == 2 && d % (4 * (int64_t)pi->world) == 0 ? 1 : 0;  // measured slower at 2 and at 8 ranks: off by default
      a.slot_lines = (int64_t)(pi->buf_bytes / 16);
      for (int r = 0; r < pi->world; ++r) a.peer_buf[r] = pi->bufs[which][r];
      a.epoch = pi->epoch;
      a.barrier_offset = 2 * l + which + 1;
      return REWB200_OK;
    }
    if (!tp_bf16_slab) RB_TRY(slab_sum_launch(c, s->part, ks, rows * d));  // one slab: bf16 from the GEMM, or f32 summed here
    ks = 1;
    a.nsplit = 1;
    a.partial_bf16 = tp_bf16_slab ? 1 : 0;
    if (twoshot) {
      Tp2Args t;
      memset(&t, 0, sizeof(t));
      t.world = pi->world;
      t.my_rank = pi->rank;
      for (int r = 0; r < pi->world; ++r) {
        t.cells[r] = pi->a2a_flags[r];
        t.region[r] = pi->a2a[r];
      }
      t.off_gather = (int64_t)((size_t)rows * d * pay);
      t.arrive = pi->epoch + 2;
      t.epoch = pi->epoch + 1;
      t.offset = 2 * l + which + 1;
      t.status = c->d_status;
      t.partial = s->part;
      t.rows = rows;
      t.d = d;
      t.payload_bf16 = dt == REWB200_BF16 ? 1 : 0;
      RB_TRY(tp2_allreduce_launch(c, t));
      a.partial = reinterpret_cast<const float*>(pi->a2a[pi->rank] + t.off_gather);
      a.wait_cells = pi->a2a_flags[pi->rank] + 16;
      a.wait_n = pi->world;
      a.wait_epoch = pi->epoch + 1;
      a.wait_offset = t.offset;
      return REWB200_OK;
    }
    RB_TRY(comm_allreduce_sum(c, m->slot, s->part, rows * d, tp_bf16_slab ? REWB200_BF16 : REWB200_F32));
    return REWB200_OK;
  };
  // o-proj / down-proj: f32 split-K slabs for the consumer kernel, or one bf16 slab ahead of a bf16 NCCL sum
  auto run_row_parallel = [&](const LinW& w, const void* x, int64_t ldx, int* ks) -> int {
    if (!tp_bf16_slab || (w.quant && rows <= 32)) return run_linear(s, w, x, ldx, rows, true, 0, s->part, d, ks);
    *ks = 1;
    if (w.quant) RB_TRY(nf4_dequant_launch(c, w.nf4, (bf16*)w.w, w.N, w.cm));
    return linear_bf16_launch(c, w.plan, (const bf16*)x, ldx, rows, EPI_BIAS_BF16, 1, s->part, d, nullptr, nullptr, 0);
  };
  int moe_seen = 0;  // MoE layers so far: numbers the flags of the peer-heap all-to-all
  for (int l = 0; l < cf.n_layers; ++l) {
    LayerDev& L = m->layers[l];
    int ks = 1;
    bool qkv_done = false;
    QkvPostArgs qa;
    memset(&qa, 0, sizeof(qa));
    qa.partial = s->part;
    qa.nsplit = ks;
    qa.split_stride = rows * m->nqkv;
    qa.bias = L.qkv.b;
    qa.cosT = m->cosT;
    qa.sinT = m->sinT;
    qa.pos0 = pos;
    qa.S = o.S;
    qa.rope_shift = o.rope_shift;
    qa.nh = m->nh_l;
    qa.kvh = m->kvh_l;
    qa.hd = cf.head_dim;
    qa.max_seq = cf.max_seq;
    qa.q_out = s->q;
    qa.act_dtype = dt;
    qa.kv.k = s->kc[l];
    qa.kv.v = s->vc[l];
    qa.kv.block_table = block_table;
    qa.kv.max_pages = s->max_pages;
    qa.kv.page = PAGE;
    qa.kv.kvh = m->kvh_l;
    qa.kv.hd = cf.head_dim;
    qa.kv.dtype = dt;
    qa.kv_capacity = s->max_len;
    qa.status = c->d_status;
    qa.early_lookup = in_graph ? 1 : 0;
    RB_TRY(run_linear(s, L.qkv, s->xn, d, rows, true, 0, s->part, m->nqkv, &ks, dt == REWB200_BF16 ? &qa : nullptr, &qkv_done));
    if (o.trace) RB_TRY(o.trace->mark(TC_QKV));
    // decode steps: the attention kernel finishes q / k / v of the new token from the slabs itself
    // ... when its grid is at most one wave of two CTAs per SM (measured: with several waves the prologue in front of
    // every CTA costs more than the launch it saves: l8 batch 128 5.69 -> 6.08 ms, the MoE model 7.07 -> 7.28 ms)
    const bool fuse_into_attn = !qkv_done && o.S == 1 && dt == REWB200_BF16 && c->attn_fuse_qkv && m->nh_l / m->kvh_l <= 16 &&
                                (c->attn_fuse_qkv_always ||
                                 (int64_t)nb * m->kvh_l * decode_splits(c, nb, m->kvh_l) <= 2 * (int64_t)c->sm_count);
    qa.nsplit = ks;
    if (!qkv_done && !fuse_into_attn) RB_TRY(qkv_post_launch(c, qa, nb));
    if (o.trace) RB_TRY(o.trace->mark(TC_QKV_POST));

    AttnArgs aa;
    memset(&aa, 0, sizeof(aa));
    aa.q = s->q;
    aa.q_sb = (int64_t)o.S * m->nq;
    aa.q_ss = m->nq;
    aa.q_sh = cf.head_dim;
    aa.out = s->attn;
    aa.o_sb = aa.q_sb;
    aa.o_ss = aa.q_ss;
    aa.o_sh = aa.q_sh;
    aa.kv = qa.kv;
    aa.pos0 = pos;
    aa.B = nb;
    aa.S = o.S;
    aa.nh = m->nh_l;
    aa.causal = o.causal;
    aa.mask_kind = cf.mask_kind;
    aa.kv_len_fixed = -1;
    aa.max_kv_len = s->max_len;
    aa.scale = 0.f;
    aa.dtype = dt;
    aa.kv_tail_only = in_graph ? 1 : 0;  // inside the captured step only the newest cache row is written
    aa.scratch = s->attn_scratch;
    aa.scratch_bytes = s->attn_scratch_bytes;
    if (dt == REWB200_BF16) {
      aa.tmK = &s->tmK[l];
      aa.tmV = &s->tmV[l];
    }
    if (fuse_into_attn) aa.fuse_qkv = &qa;
    RB_TRY(attn_launch(c, aa));
    if (o.trace) RB_TRY(o.trace->mark(TC_ATTN));

    RB_TRY(run_row_parallel(L.o, s->attn, m->nq, &ks));
    if (o.trace) RB_TRY(o.trace->mark(TC_O));
    {
      NormArgs a = na;
      a.partial = s->part;
      a.nsplit = ks;
      a.split_stride = rows * d;
      a.bias = L.o.b;
      a.gamma = L.ln2g;
      a.beta = L.ln2b;
      RB_TRY(tp_reduce(l, 0, ks, a));
      RB_TRY(residual_norm_launch(c, a, rows));
      if (o.trace) RB_TRY(o.trace->mark(TC_NORM_ATTN));
    }
    ks = 0;  // slabs of s->part that hold FFN output so far
    // MoE layer with shared experts on one rank, small step: the shared experts (three short launches)
    // run on a second stream beside the routed path (router, sort, two HBM-bound grouped GEMMs, combine).
    // Their slabs sit behind the gate|up scratch, the routed sum in the slab after them.
    const size_t gu_scratch = (size_t)4 * rows * 2 * L.ffn_local;  // floats the split gate|up may use at the head of s->part
    const bool fork = L.moe && L.ffn_local > 0 && dt == REWB200_BF16 && (cf.ep_size == 1 || ep_uses_peer_heap(m, rows)) &&
                      cf.tp_size == 1 && rows <= 64 &&
                      c->moe_overlap && (gu_scratch + (size_t)17 * rows * d) * sizeof(float) <= s->part_bytes;
    if (fork) {
      float* base = s->part + gu_scratch;
      RB_CUDA(cudaEventRecord(c->ev_fork, c->stream));
      RB_CUDA(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
      cudaStream_t main_stream = c->stream;
      const bool pdl = c->use_pdl;
      c->stream = c->side;
      c->use_pdl = false;  // first launch behind an event wait: a plain dependency
      int st = run_linear(s, L.gu, s->xn, d, rows, false, EPI_SWIGLU_BF16, s->h, L.ffn_local, nullptr);
      c->use_pdl = pdl;
      if (st == REWB200_OK) st = run_linear(s, L.down, s->h, L.ffn_local, rows, true, 0, base, d, &ks);
      c->stream = main_stream;
      RB_TRY(st);
      RB_CUDA(cudaEventRecord(c->ev_join, c->side));
      RB_TRY(moe_routed(s, L, rows, false, base + (size_t)ks * rows * d, moe_seen++));
      RB_CUDA(cudaStreamWaitEvent(c->stream, c->ev_join, 0));
      NormArgs a = na;
      a.partial = base;
      a.nsplit = ks + 1;
      a.split_stride = rows * d;
      a.bias = L.down.b;
      const bool last = (l + 1 == cf.n_layers);
      a.gamma = last ? m->ng : m->layers[l + 1].ln1g;
      a.beta = last ? m->nb : m->layers[l + 1].ln1b;
      c->use_pdl = false;  // two predecessors (combine and the shared down projection): a plain dependency
      st = residual_norm_launch(c, a, rows);
      c->use_pdl = pdl;
      RB_TRY(st);
      if (o.trace) RB_TRY(o.trace->mark(TC_MOE));
      continue;
    }
    if (L.ffn_local > 0) {  // dense FFN, or the fused shared experts of a MoE layer
      if (dt == REWB200_BF16) {
        RB_TRY(run_linear(s, L.gu, s->xn, d, rows, false, EPI_SWIGLU_BF16, s->h, L.ffn_local, nullptr));
      } else {
        RB_TRY(run_linear(s, L.gu, s->xn, d, rows, false, EPI_BIAS_F32, s->gu32, 2 * L.ffn_local, nullptr));
        const int64_t n = rows * L.ffn_local;
        swiglu_rows_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(s->gu32, (float*)s->h, rows, L.ffn_local);
        RB_CUDA(cudaGetLastError());
        ++g_launch_total;
      }
      if (o.trace) RB_TRY(o.trace->mark(TC_GATE_UP));
      RB_TRY(run_row_parallel(L.down, s->h, L.ffn_local, &ks));
      if (o.trace) RB_TRY(o.trace->mark(TC_DOWN));
    }
    if (L.moe) {
      RB_TRY(moe_routed(s, L, rows, ks > 0, nullptr, moe_seen++));
      if (ks == 0) ks = 1;
      if (o.trace) RB_TRY(o.trace->mark(TC_MOE));
    }
    {
      NormArgs a = na;
      a.partial = s->part;
      a.nsplit = ks;
      a.split_stride = rows * d;
      a.bias = L.ffn_local > 0 ? L.down.b : nullptr;
      const bool last = (l + 1 == cf.n_layers);
      a.gamma = last ? m->ng : m->layers[l + 1].ln1g;
      a.beta = last ? m->nb : m->layers[l + 1].ln1b;
      RB_TRY(tp_reduce(l, 1, ks, a));
      RB_TRY(residual_norm_launch(c, a, rows));
      if (o.trace) RB_TRY(o.trace->mark(TC_NORM_FFN));
    }
  }
  if (oneshot) RB_TRY(epoch_bump_launch(c, pi->epoch, 2 * cf.n_layers));  // same on every rank
  if (moe_seen > 0 && ep_uses_peer_heap(m, rows)) RB_TRY(epoch_bump_launch(c, comm_peer_info(m->slot)->epoch + 1, moe_seen));
  if (twoshot) RB_TRY(epoch_bump_launch(c, pi->epoch + 1, 2 * cf.n_layers));
  // lm_head: last position of every sequence (generate.nim:172-190) or every row.
  const int64_t lrows = o.all_logits ? rows : nb;
  const char* xl = (const char*)s->xn + (o.all_logits ? 0 : (size_t)(o.S - 1) * d * dtype_size(dt));
  const int64_t ldx = o.all_logits ? d : (int64_t)o.S * d;
  if (dt == REWB200_BF16) {
    RB_TRY(linear_bf16_launch(c, m->lm.plan, (const bf16*)xl, ldx, lrows, EPI_BIAS_F32, 1, logits, m->vocab_l, m->lm.b,
                              nullptr, 0));
  } else {
    if (o.all_logits || o.S == 1) {
      RB_TRY(gemm_f32_launch(c, (const float*)xl, (const float*)m->lm.w, m->lm.b, logits, lrows, d, m->vocab_l));
    } else {
      // gather the last rows into the head of q (free at this point), then GEMM
      for (int b = 0; b < nb; ++b)
        RB_CUDA(cudaMemcpyAsync((float*)s->q + (size_t)b * d, (const float*)s->xn + ((size_t)b * o.S + o.S - 1) * d,
                                d * sizeof(float), cudaMemcpyDeviceToDevice, c->stream));
      RB_TRY(gemm_f32_launch(c, (const float*)s->q, (const float*)m->lm.w, m->lm.b, logits, lrows, d, m->vocab_l));
    }
  }
  if (!o.all_logits) {
    if (cf.tp_size > 1) {
      RB_REQUIRE(b0 == 0 && nb == s->B, "lane ranges are not available on a tensor-parallel model");
      // vocab-parallel: per-rank (value, index) partials, all-gathered, then the same first-max rule
      const int nch = 16;
      float* pv = (float*)s->argmax_scratch;
      int* pi = (int*)((char*)s->argmax_scratch + (size_t)s->B * nch * 4);
      RB_TRY(argmax_partial_launch(c, s->logits, s->B, m->vocab_l, (int)(cf.tp_rank * m->vocab_l), nch, pv, pi));
      RB_TRY(comm_allgather_bytes(c, m->slot, s->argmax_scratch, s->gather_scratch, (size_t)s->B * nch * 8));
      RB_TRY(argmax_gathered_launch(c, s->gather_scratch, cf.tp_size, s->B, nch, s->d_next));
    } else if (s->samp_on) {
      const int* act = s->d_active ? s->d_active + b0 : nullptr;
      RB_TRY(sample_launch(c, logits, s->samp_work + (size_t)b0 * cf.vocab, nb, cf.vocab, s->samp_hist + (size_t)b0 * s->max_len,
                           s->samp_hist_len + b0, s->max_len, s->samp_keys + 2 * b0, s->samp_steps + b0, next,
                           s->samp_logprob + (size_t)b0 * s->max_len, s->max_len, s->samp_temperature, s->samp_top_k,
                           s->samp_top_p, s->samp_min_p, s->samp_rep, s->samp_do_sample, act));
    } else {
      RB_TRY(argmax_launch(c, logits, nb, cf.vocab, next, s->argmax_scratch, (size_t)s->B * 64 * 8));
    }
    RB_CUDA(launch_k(advance_kernel, dim3(1), dim3(256), 0, c->stream, c->use_pdl, (const int*)next, s->d_ids + b0, pos,
                     o.record_out ? s->d_out : (int*)nullptr, s->d_step, (const int*)(s->d_active ? s->d_active + b0 : nullptr),
                     nb, o.S, s->out_capacity));
    ++g_launch_total;
  }
  if (o.trace) RB_TRY(o.trace->mark(TC_HEAD));
  return REWB200_OK;
}

}  // namespace
}  // namespace rewb

extern "C" {

int rewb200_model_create(int slot, const rewb200_config* cfg, rewb200_model** out) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(cfg && out, "rewb200_model_create: NULL argument");
  RB_CUDA(cudaSetDevice(c->device));
  RB_REQUIRE(cfg->dtype == REWB200_F32 || cfg->dtype == REWB200_BF16, "model dtype must be f32 or bf16");
  RB_REQUIRE(cfg->weight_quant == 0 || cfg->weight_quant == 1, "weight_quant must be 0 or 1 (NF4)");
  if (cfg->weight_quant == 1) {
    RB_REQUIRE(cfg->dtype == REWB200_BF16 && cfg->n_routed == 0, "NF4 weights need a dense bf16 model");
    RB_REQUIRE(cfg->d_model % 64 == 0 && (cfg->ffn / std::max(1, cfg->tp_size)) % 64 == 0 && cfg->head_dim % 64 == 0,
               "NF4 weights need d_model, head_dim and the local ffn width to be multiples of 64");
  }
  RB_REQUIRE(cfg->vocab > 0 && cfg->d_model > 0 && cfg->n_layers > 0 && cfg->head_dim > 0 && cfg->max_seq > 0,
             "model dimensions must be positive");
  RB_REQUIRE(cfg->n_kv_heads > 0 && cfg->n_heads % cfg->n_kv_heads == 0,
             "initGroupedQueryAttention: numHeads " + std::to_string(cfg->n_heads) + " must be divisible by numKVHeads " +
                 std::to_string(cfg->n_kv_heads));
  RB_REQUIRE(cfg->head_dim % 2 == 0, "initRotaryPositionEncoding: headDim must be positive and even, got " +
                                         std::to_string(cfg->head_dim));
  const int tp = std::max(1, cfg->tp_size);
  RB_REQUIRE(cfg->tp_rank >= 0 && cfg->tp_rank < tp, "tp_rank out of range");
  RB_REQUIRE(cfg->n_heads % tp == 0 && cfg->n_kv_heads % tp == 0 && cfg->ffn % tp == 0,
             "shardLayout: heads, kv heads and FFN width must be divisible by the tensor-parallel size");
  const int ep = std::max(1, cfg->ep_size);
  if (cfg->n_routed > 0) {
    RB_REQUIRE(tp == 1, "MoE models shard by experts (ep_size), not by tensor parallelism");
    RB_REQUIRE(cfg->ep_rank >= 0 && cfg->ep_rank < ep && cfg->n_routed % ep == 0, "initDeepSeekMoE: numRouted must divide by ep_size");
    RB_REQUIRE(cfg->n_shared >= 0, "initDeepSeekMoE: numShared must be non-negative");
    RB_REQUIRE(cfg->top_k >= 1 && cfg->top_k <= cfg->n_routed, "initDeepSeekMoE: numExpertsPerTok must be in 1..numRouted");
    RB_REQUIRE(cfg->moe_ffn > 0 && cfg->n_routed <= 256, "initDeepSeekMoE: hiddenSize and intermediateSize must be positive");
    RB_REQUIRE(cfg->dtype == REWB200_BF16 || ep == 1, "expert parallelism is built for bf16 models");
    if (cfg->dtype == REWB200_BF16)
      RB_REQUIRE(cfg->moe_ffn % 8 == 0 && cfg->n_routed % 8 == 0, "bf16 MoE needs moe_ffn and numRouted multiples of 8");
  } else {
    RB_REQUIRE(ep == 1, "ep_size > 1 needs a MoE model");
  }
  rewb200_model* m = new rewb200_model();
  m->c = c;
  m->slot = slot;
  m->cfg = *cfg;
  m->cfg.tp_size = tp;
  m->cfg.ep_size = std::max(1, cfg->ep_size);
  RB_REQUIRE(cfg->vocab % tp == 0, "shardLayout: vocabulary must be divisible by the tensor-parallel size");
  m->vocab_l = cfg->vocab / tp;
  m->nh_l = cfg->n_heads / tp;
  m->kvh_l = cfg->n_kv_heads / tp;
  m->nq = (int64_t)m->nh_l * cfg->head_dim;
  m->nkv = (int64_t)m->kvh_l * cfg->head_dim;
  m->nqkv = m->nq + 2 * m->nkv;
  const int64_t d = cfg->d_model;
  if (cfg->dtype == REWB200_BF16)
    RB_REQUIRE(d % 8 == 0 && m->nqkv % 8 == 0 && (cfg->ffn / tp) % 8 == 0 && (cfg->vocab / tp) % 8 == 0 &&
                   (cfg->head_dim == 64 || cfg->head_dim == 128),
               "bf16 models need d_model, ffn/tp, vocab multiples of 8 and head_dim 64 or 128");
  const size_t es = dtype_size(cfg->dtype);
  RB_TRY(dev_alloc(m, &m->embed, (size_t)cfg->vocab * d * es));
  m->layers.resize(cfg->n_layers);
  auto alloc_vec = [&](float** p, float v) -> int {
    RB_TRY(dev_alloc(m, (void**)p, d * sizeof(float)));
    return fill_const_launch(c, *p, REWB200_F32, d, v);
  };
  for (int l = 0; l < cfg->n_layers; ++l) {
    LayerDev& L = m->layers[l];
    RB_TRY(alloc_vec(&L.ln1g, 1.f));
    RB_TRY(alloc_vec(&L.ln1b, 0.f));
    RB_TRY(alloc_vec(&L.ln2g, 1.f));
    RB_TRY(alloc_vec(&L.ln2b, 0.f));
    L.moe = layer_is_moe(*cfg, l);
    if (L.moe) L.ffn_local = (int64_t)cfg->n_shared * cfg->moe_ffn;
    else if (cfg->n_routed > 0 && cfg->first_dense > 0) L.ffn_local = cfg->first_dense;
    else L.ffn_local = cfg->ffn / tp;
    RB_TRY(alloc_lin(m, &L.qkv, d, m->nqkv));
    RB_TRY(alloc_lin(m, &L.o, m->nq, d));
    if (L.ffn_local > 0) {
      RB_TRY(alloc_lin(m, &L.gu, d, 2 * L.ffn_local));
      RB_TRY(alloc_lin(m, &L.down, L.ffn_local, d));
    }
    if (L.moe) {
      MoeDev& X = L.x;
      X.E_l = cfg->n_routed / m->cfg.ep_size;
      X.f = cfg->moe_ffn;
      X.shared_down_bias.assign(d, 0.f);
      RB_TRY(alloc_lin(m, &X.router, d, cfg->n_routed));
      RB_TRY(dev_alloc(m, &X.gu, (size_t)X.E_l * d * 2 * X.f * es));
      RB_TRY(dev_alloc(m, &X.down, (size_t)X.E_l * X.f * d * es));
      RB_TRY(dev_alloc(m, (void**)&X.gu_b, (size_t)X.E_l * 2 * X.f * sizeof(float)));
      RB_TRY(dev_alloc(m, (void**)&X.down_b, (size_t)X.E_l * d * sizeof(float)));
      RB_CUDA(cudaMemsetAsync(X.gu_b, 0, (size_t)X.E_l * 2 * X.f * sizeof(float), c->stream));
      RB_CUDA(cudaMemsetAsync(X.down_b, 0, (size_t)X.E_l * d * sizeof(float), c->stream));
    }
  }
  RB_TRY(alloc_vec(&m->ng, 1.f));
  RB_TRY(alloc_vec(&m->nb, 0.f));
  RB_TRY(alloc_lin(m, &m->lm, d, m->vocab_l));
  std::vector<float> ct, st;
  RB_TRY(rope_tables_host(cfg->head_dim, cfg->max_seq, cfg->theta, &ct, &st));
  RB_TRY(dev_alloc(m, (void**)&m->cosT, ct.size() * sizeof(float)));
  RB_TRY(dev_alloc(m, (void**)&m->sinT, st.size() * sizeof(float)));
  RB_CUDA(cudaMemcpyAsync(m->cosT, ct.data(), ct.size() * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  RB_CUDA(cudaMemcpyAsync(m->sinT, st.data(), st.size() * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  *out = m;
  return REWB200_OK;
}

void rewb200_model_free(rewb200_model* m) {
  if (!m) return;
  cudaSetDevice(m->c->device);
  cudaStreamSynchronize(m->c->stream);
  for (void* p : m->allocs) cudaFree(p);
  if (m->stage) cudaFree(m->stage);
  delete m;
}

int64_t rewb200_model_tensor_count(const rewb200_model* m) {
  if (!m) return 0;
  int64_t n = 1;
  for (int l = 0; l < m->cfg.n_layers; ++l)
    n += 12 + (layer_is_moe(m->cfg, l) ? 2 + 6 * (int64_t)(m->cfg.n_shared + m->cfg.n_routed) : 6);
  return n + 4;
}

int64_t rewb200_model_weight_bytes(const rewb200_model* m) { return m ? m->weight_bytes : 0; }

}  // extern "C"

namespace rewb {
namespace {

// Which dimension of logical tensor `index` the tensor-parallel axis splits (PartitionSpec(["", "tp"]) for the
// column-parallel q / k / v / gate / up / lm_head weights, (["tp", ""]) for the row-parallel o / down weights,
// (["tp"]) for the biases of column-parallel layers), following shardLayout's block rule
// (src/rew/sharding.nim:255-270).  dim = -1: replicated.  Routed-expert tensors are whole tensors owned by
// one expert-parallel rank: *owner_ep is that rank, -1 for everything else.
int tensor_partition(const rewb200_model* m, int64_t index, int* dim, int* ndims, int64_t* shape, int* owner_ep) {
  const rewb200_config& c = m->cfg;
  TensorRef r;
  RB_TRY(locate(m, index, &r));
  const int64_t d = c.d_model, hd = c.head_dim;
  const int64_t NQ = (int64_t)c.n_heads * hd, NKV = (int64_t)c.n_kv_heads * hd;
  *dim = -1;
  *owner_ep = -1;
  auto mat = [&](int64_t rows, int64_t cols, int split) { *ndims = 2; shape[0] = rows; shape[1] = cols; *dim = split; };
  auto vec = [&](int64_t n, bool split) { *ndims = 1; shape[0] = n; *dim = split ? 0 : -1; };
  if (r.layer == -1) { mat(c.vocab, d, -1); return REWB200_OK; }
  if (r.layer == -2) {
    switch (r.slot) {
      case 0: case 1: vec(d, false); break;
      case 2: mat(d, c.vocab, 1); break;
      default: vec(c.vocab, true); break;
    }
    return REWB200_OK;
  }
  const LayerDev& L = m->layers[r.layer];
  const int64_t F = (c.n_routed > 0 && c.first_dense > 0) ? c.first_dense : c.ffn;
  if (!(L.moe && r.slot >= 12)) {
    switch (r.slot) {
      case 0: case 1: case 10: case 11: case 9: case 17: vec(d, false); break;
      case 2: mat(d, NQ, 1); break;
      case 3: vec(NQ, true); break;
      case 4: case 6: mat(d, NKV, 1); break;
      case 5: case 7: vec(NKV, true); break;
      case 8: mat(NQ, d, 0); break;
      case 12: case 14: mat(d, F, 1); break;
      case 13: case 15: vec(F, true); break;
      case 16: mat(F, d, 0); break;
      default: return fail("tensor slot not supported for this layer kind");
    }
    return REWB200_OK;
  }
  const int64_t f = L.x.f, E = c.n_routed;
  if (r.slot == 12) { mat(d, E, -1); return REWB200_OK; }
  if (r.slot == 13) { vec(E, false); return REWB200_OK; }
  const int idx = r.slot - 14, ei = idx / 6, which = idx % 6;
  RB_REQUIRE(ei < c.n_shared + c.n_routed, "expert index out of range");
  switch (which) {
    case 0: case 2: mat(d, f, -1); break;
    case 1: case 3: vec(f, false); break;
    case 4: mat(f, d, -1); break;
    default: vec(d, false); break;
  }
  if (ei >= c.n_shared) *owner_ep = (ei - c.n_shared) / L.x.E_l;
  return REWB200_OK;
}

int set_tensor_impl(rewb200_model* m, int64_t index, const float* host, int64_t numel, bool shard);

}  // namespace
}  // namespace rewb

extern "C" {

int rewb200_model_set_tensor(rewb200_model* m, int64_t index, const float* host, int64_t numel) {
  RB_REQUIRE(m && host, "rewb200_model_set_tensor: NULL argument");
  return set_tensor_impl(m, index, host, numel, false);
}

int rewb200_model_tensor_layout(const rewb200_model* m, int64_t index, int* ndims, int64_t* global_shape,
                                int64_t* local_shape, int64_t* offsets, int* partitioned_dim) {
  RB_REQUIRE(m && ndims && global_shape && local_shape && offsets, "rewb200_model_tensor_layout: NULL argument");
  int dim = -1, owner = -1;
  RB_TRY(tensor_partition(m, index, &dim, ndims, global_shape, &owner));
  for (int i = 0; i < *ndims; ++i) {
    local_shape[i] = global_shape[i];
    offsets[i] = 0;
  }
  const int tp = m->cfg.tp_size;
  if (dim >= 0 && tp > 1) {  // shardLayout: localShape[dim] = shape[dim] / factor, offset = coord * local
    local_shape[dim] = global_shape[dim] / tp;
    offsets[dim] = (int64_t)m->cfg.tp_rank * local_shape[dim];
  }
  if (owner >= 0 && m->cfg.ep_size > 1 && owner != m->cfg.ep_rank)
    for (int i = 0; i < *ndims; ++i) local_shape[i] = 0;  // another rank's expert: nothing of it lives here
  if (partitioned_dim) *partitioned_dim = (dim >= 0 && tp > 1) ? dim : -1;
  return REWB200_OK;
}

int rewb200_model_set_tensor_shard(rewb200_model* m, int64_t index, const float* host_local, const int64_t* local_shape,
                                   const int64_t* offsets, int ndims) {
  RB_REQUIRE(m && host_local && local_shape && offsets, "rewb200_model_set_tensor_shard: NULL argument");
  int nd = 0, pdim = -1;
  int64_t gs[4], ls[4], off[4];
  RB_TRY(rewb200_model_tensor_layout(m, index, &nd, gs, ls, off, &pdim));
  RB_REQUIRE(nd == ndims, "fromHostShards: shard rank " + std::to_string(ndims) + " does not match the tensor's " + std::to_string(nd));
  int64_t numel = 1;
  for (int i = 0; i < nd; ++i) {
    RB_REQUIRE(local_shape[i] == ls[i] && offsets[i] == off[i],
               "fromHostShards: tensor " + std::to_string(index) + " dim " + std::to_string(i) + ": this rank holds [" +
                   std::to_string(off[i]) + ", " + std::to_string(off[i] + ls[i]) + "), the shard given covers [" +
                   std::to_string(offsets[i]) + ", " + std::to_string(offsets[i] + local_shape[i]) + ")");
    numel *= ls[i];
  }
  if (numel == 0) return REWB200_OK;
  return set_tensor_impl(m, index, host_local, numel, true);
}

}  // extern "C"

namespace rewb {
namespace {

// shard = false: `host` is the FULL logical tensor and the rank's block is cut out of it; shard = true: `host`
// is exactly this rank's block (rewb200_model_tensor_layout), nothing else crosses the host interface.
int set_tensor_impl(rewb200_model* m, int64_t index, const float* host, int64_t numel, bool shard) {
  RB_REQUIRE(!m->finalized, "model already finalized");
  RB_CUDA(cudaSetDevice(m->c->device));
  const rewb200_config& c = m->cfg;
  TensorRef r;
  RB_TRY(locate(m, index, &r));
  const int64_t d = c.d_model, hd = c.head_dim;
  const int tp = c.tp_size, rk = shard ? 0 : c.tp_rank;
  const int64_t NQ = (int64_t)c.n_heads * hd / (shard ? tp : 1), NKV = (int64_t)c.n_kv_heads * hd / (shard ? tp : 1);
  const int64_t VOC = (int64_t)c.vocab / (shard ? tp : 1);
  const bool bf = c.dtype == REWB200_BF16;
  auto expect = [&](int64_t n) -> int {
    RB_REQUIRE(numel == n, "tensor " + std::to_string(index) + ": expected " + std::to_string(n) + " elements, got " +
                               std::to_string(numel));
    return upload_stage(m, host, numel);
  };
  auto vec = [&](float* dst, int64_t n_full, int64_t off, int64_t n) -> int {
    RB_TRY(expect(n_full));
    return scatter(m, n_full, 0, off, 1, n, dst, false, n, n, n, 0);
  };
  if (r.layer == -1) {
    RB_TRY(expect((int64_t)c.vocab * d));
    return scatter(m, d, 0, 0, c.vocab, d, m->embed, true, d, d, d, 0);
  }
  if (r.layer == -2) {
    switch (r.slot) {
      case 0: return vec(m->ng, d, 0, d);
      case 1: return vec(m->nb, d, 0, d);
      case 2: RB_TRY(expect(d * VOC)); return scatter(m, VOC, 0, rk * m->vocab_l, d, m->vocab_l, m->lm.w, true, m->vocab_l, m->vocab_l, m->vocab_l, 0);
      default: return vec(m->lm.b, VOC, rk * m->vocab_l, m->vocab_l);
    }
  }
  LayerDev& L = m->layers[r.layer];
  const int64_t nq = m->nq, nkv = m->nkv, nqkv = m->nqkv, fl = L.ffn_local;
  // gate/up column mapping: bf16 interleaves groups of 8 (gate at +0, up at +8 of each 16); f32 concatenates.
  const int64_t ggran = bf ? 8 : fl, gstride = bf ? 16 : fl;
  const int64_t F = ((c.n_routed > 0 && c.first_dense > 0) ? c.first_dense : c.ffn) / (shard ? tp : 1);  // dense block width
  if (!(L.moe && r.slot >= 12)) switch (r.slot) {
    case 0: return vec(L.ln1g, d, 0, d);
    case 1: return vec(L.ln1b, d, 0, d);
    case 2: RB_TRY(expect(d * NQ)); return scatter(m, NQ, 0, rk * nq, d, nq, L.qkv.w, true, nqkv, nq, nq, 0);
    case 3: RB_TRY(expect(NQ)); return scatter(m, NQ, 0, rk * nq, 1, nq, L.qkv.b, false, nqkv, nq, nq, 0);
    case 4: RB_TRY(expect(d * NKV)); return scatter(m, NKV, 0, rk * nkv, d, nkv, L.qkv.w, true, nqkv, nkv, nkv, nq);
    case 5: RB_TRY(expect(NKV)); return scatter(m, NKV, 0, rk * nkv, 1, nkv, L.qkv.b, false, nqkv, nkv, nkv, nq);
    case 6: RB_TRY(expect(d * NKV)); return scatter(m, NKV, 0, rk * nkv, d, nkv, L.qkv.w, true, nqkv, nkv, nkv, nq + nkv);
    case 7: RB_TRY(expect(NKV)); return scatter(m, NKV, 0, rk * nkv, 1, nkv, L.qkv.b, false, nqkv, nkv, nkv, nq + nkv);
    case 8: RB_TRY(expect(NQ * d)); return scatter(m, d, rk * nq, 0, nq, d, L.o.w, true, d, d, d, 0);
    case 9: return vec(L.o.b, d, 0, d);
    case 10: return vec(L.ln2g, d, 0, d);
    case 11: return vec(L.ln2b, d, 0, d);
    case 12: RB_TRY(expect(d * F)); return scatter(m, F, 0, rk * fl, d, fl, L.gu.w, true, 2 * fl, ggran, gstride, 0);
    case 13: RB_TRY(expect(F)); return scatter(m, F, 0, rk * fl, 1, fl, L.gu.b, false, 2 * fl, ggran, gstride, 0);
    case 14: RB_TRY(expect(d * F)); return scatter(m, F, 0, rk * fl, d, fl, L.gu.w, true, 2 * fl, ggran, gstride, bf ? 8 : fl);
    case 15: RB_TRY(expect(F)); return scatter(m, F, 0, rk * fl, 1, fl, L.gu.b, false, 2 * fl, ggran, gstride, bf ? 8 : fl);
    case 16: RB_TRY(expect(F * d)); return scatter(m, d, rk * fl, 0, fl, d, L.down.w, true, d, d, d, 0);
    case 17: return vec(L.down.b, d, 0, d);
    default: break;
  }
  (void)tp;
  RB_REQUIRE(L.moe, "tensor slot not supported for this layer kind");
  {
    MoeDev& X = L.x;
    const int64_t f = X.f, E = c.n_routed;
    if (r.slot == 12) {
      RB_TRY(expect(d * E));
      return scatter(m, E, 0, 0, d, E, X.router.w, true, E, E, E, 0);
    }
    if (r.slot == 13) return vec(X.router.b, E, 0, E);
    const int idx = r.slot - 14, ei = idx / 6, which = idx % 6;
    RB_REQUIRE(ei < c.n_shared + c.n_routed, "expert index out of range");
    // column mapping of gate / up inside a fused [.., 2*width] block
    const int64_t gran = bf ? 8 : f, gstr = bf ? 16 : f;
    if (ei < c.n_shared) {
      const int64_t ns = c.n_shared, W2 = 2 * ns * f;
      const int64_t g_off = bf ? ei * 2 * f : ei * f, u_off = bf ? ei * 2 * f + 8 : ns * f + ei * f;
      switch (which) {
        case 0: RB_TRY(expect(d * f)); return scatter(m, f, 0, 0, d, f, L.gu.w, true, W2, gran, gstr, g_off);
        case 1: RB_TRY(expect(f)); return scatter(m, f, 0, 0, 1, f, L.gu.b, false, W2, gran, gstr, g_off);
        case 2: RB_TRY(expect(d * f)); return scatter(m, f, 0, 0, d, f, L.gu.w, true, W2, gran, gstr, u_off);
        case 3: RB_TRY(expect(f)); return scatter(m, f, 0, 0, 1, f, L.gu.b, false, W2, gran, gstr, u_off);
        case 4: RB_TRY(expect(f * d));
          return scatter(m, d, 0, 0, f, d, (char*)L.down.w + (size_t)ei * f * d * dtype_size(c.dtype), true, d, d, d, 0);
        default:
          RB_REQUIRE(numel == d, "expert down bias must have d_model elements");
          for (int64_t i = 0; i < d; ++i) X.shared_down_bias[i] += host[i];
          return REWB200_OK;
      }
    }
    const int e = ei - c.n_shared;
    if (e / X.E_l != c.ep_rank) return REWB200_OK;  // another rank's expert
    const int64_t le = e % X.E_l;
    const size_t es2 = dtype_size(c.dtype);
    char* gw = (char*)X.gu + (size_t)le * d * 2 * f * es2;
    float* gb = X.gu_b + le * 2 * f;
    const int64_t u_off = bf ? 8 : f;
    switch (which) {
      case 0: RB_TRY(expect(d * f)); return scatter(m, f, 0, 0, d, f, gw, true, 2 * f, gran, gstr, 0);
      case 1: RB_TRY(expect(f)); return scatter(m, f, 0, 0, 1, f, gb, false, 2 * f, gran, gstr, 0);
      case 2: RB_TRY(expect(d * f)); return scatter(m, f, 0, 0, d, f, gw, true, 2 * f, gran, gstr, u_off);
      case 3: RB_TRY(expect(f)); return scatter(m, f, 0, 0, 1, f, gb, false, 2 * f, gran, gstr, u_off);
      case 4: RB_TRY(expect(f * d)); return scatter(m, d, 0, 0, f, d, (char*)X.down + (size_t)le * f * d * es2, true, d, d, d, 0);
      default: RB_TRY(expect(d)); return scatter(m, d, 0, 0, 1, d, X.down_b + le * d, false, d, d, d, 0);
    }
  }
}

}  // namespace
}  // namespace rewb

extern "C" {

int rewb200_model_init_random(rewb200_model* m, uint64_t seed, float std) {
  RB_REQUIRE(m, "rewb200_model_init_random: NULL model");
  RB_REQUIRE(!m->finalized, "model already finalized");
  RB_CUDA(cudaSetDevice(m->c->device));
  Ctx* c = m->c;
  const int dt = m->cfg.dtype;
  // replicated tensors (the embedding) use the seed alone; sharded ones also mix in the rank
  uint64_t k = seed * 1000003ull;
  RB_TRY(fill_normal_launch(c, m->embed, dt, (int64_t)m->cfg.vocab * m->cfg.d_model, ++k, std));
  k += (uint64_t)m->cfg.tp_rank * 7919ull;
  for (LayerDev& L : m->layers) {
    RB_TRY(fill_normal_launch(c, L.qkv.w, dt, L.qkv.K * L.qkv.N, ++k, std));
    RB_TRY(fill_normal_launch(c, L.o.w, dt, L.o.K * L.o.N, ++k, std));
    if (L.ffn_local > 0) {
      RB_TRY(fill_normal_launch(c, L.gu.w, dt, L.gu.K * L.gu.N, ++k, std));
      RB_TRY(fill_normal_launch(c, L.down.w, dt, L.down.K * L.down.N, ++k, std));
    }
    if (L.moe) {
      const uint64_t router_seed = seed * 1000003ull + 500000ull + (uint64_t)(&L - &m->layers[0]);  // same on every rank
      RB_TRY(fill_normal_launch(c, L.x.router.w, dt, L.x.router.K * L.x.router.N, router_seed, std));
      // experts differ per rank; everything else above must be identical on every rank
      const uint64_t ke = (router_seed * 31ull + 7ull) ^ ((uint64_t)(m->cfg.ep_rank + 1) << 40);
      RB_TRY(fill_normal_launch(c, L.x.gu, dt, (int64_t)L.x.E_l * m->cfg.d_model * 2 * L.x.f, ke + 1, std));
      RB_TRY(fill_normal_launch(c, L.x.down, dt, (int64_t)L.x.E_l * L.x.f * m->cfg.d_model, ke + 2, std));
    }
  }
  RB_TRY(fill_normal_launch(c, m->lm.w, dt, m->lm.K * m->lm.N, ++k, std));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  return REWB200_OK;
}

int rewb200_model_finalize(rewb200_model* m) {
  RB_REQUIRE(m, "rewb200_model_finalize: NULL model");
  if (m->finalized) return REWB200_OK;
  RB_CUDA(cudaSetDevice(m->c->device));
  if (m->cfg.weight_quant == 1) {
    // nf4Quantize every decoder-block Linear from its bf16 device copy, drop that copy, and let all of
    // them share one bf16 scratch (the largest matrix) for prefill-size launches.
    Ctx* c = m->c;
    size_t scratch = 0;
    for (LayerDev& L : m->layers)
      for (LinW* w : {&L.qkv, &L.o, &L.gu, &L.down}) scratch = std::max(scratch, (size_t)w->K * w->N * sizeof(bf16));
    void* shared = nullptr;
    RB_CUDA(cudaMalloc(&shared, scratch));
    m->allocs.push_back(shared);
    for (LayerDev& L : m->layers) {
      L.gu.cm = ColMap{L.ffn_local, 8, 16, 8};  // bf16 engine layout: gate/up interleaved in groups of 8
      for (LinW* w : {&L.qkv, &L.o, &L.down}) w->cm = ColMap{w->N, w->N, w->N, 0};
      for (LinW* w : {&L.qkv, &L.o, &L.gu, &L.down}) {
        RB_TRY(nf4_alloc(c, w->K, w->N, &w->nf4));
        m->allocs.push_back(w->nf4.q);
        m->allocs.push_back(w->nf4.sc);
        m->allocs.push_back(w->nf4.sc2);
        RB_TRY(nf4_quantize_launch(c, w->w, REWB200_BF16, w->N, w->cm, w->nf4));
        RB_CUDA(cudaStreamSynchronize(c->stream));
        auto it = std::find(m->allocs.begin(), m->allocs.end(), w->w);
        if (it != m->allocs.end()) m->allocs.erase(it);
        RB_CUDA(cudaFree(w->w));
        m->weight_bytes += (int64_t)(w->K * w->N / 2 + w->K * (w->N / 64) * 6) - (int64_t)(w->K * w->N * 2);
        w->w = shared;
        w->quant = true;
      }
    }
  }
  if (m->cfg.dtype == REWB200_BF16) {
    for (LayerDev& L : m->layers) {
      RB_TRY(linear_bf16_plan(&L.qkv.plan, (const bf16*)L.qkv.w, L.qkv.K, L.qkv.N, 0));
      RB_TRY(linear_bf16_plan(&L.o.plan, (const bf16*)L.o.w, L.o.K, L.o.N, 0));
      if (L.ffn_local > 0) {
        RB_TRY(linear_bf16_plan(&L.gu.plan, (const bf16*)L.gu.w, L.gu.K, L.gu.N, 0));
        RB_TRY(linear_bf16_plan(&L.down.plan, (const bf16*)L.down.w, L.down.K, L.down.N, 0));
      }
      if (L.moe) {
        RB_TRY(linear_bf16_plan(&L.x.router.plan, (const bf16*)L.x.router.w, L.x.router.K, L.x.router.N, 0));
        RB_TRY(linear_bf16_plan(&L.x.plan_gu, (const bf16*)L.x.gu, m->cfg.d_model, 2 * L.x.f, L.x.E_l));
        RB_TRY(linear_bf16_plan(&L.x.plan_down, (const bf16*)L.x.down, L.x.f, m->cfg.d_model, L.x.E_l));
      }
    }
    RB_TRY(linear_bf16_plan(&m->lm.plan, (const bf16*)m->lm.w, m->lm.K, m->lm.N, 0));
  }
  for (LayerDev& L : m->layers)  // shared experts' down biases were summed on the host
    if (L.moe && L.ffn_local > 0)
      RB_CUDA(cudaMemcpyAsync(L.down.b, L.x.shared_down_bias.data(), m->cfg.d_model * sizeof(float), cudaMemcpyHostToDevice,
                              m->c->stream));
  if (m->stage) {
    RB_CUDA(cudaStreamSynchronize(m->c->stream));
    RB_CUDA(cudaFree(m->stage));
    m->stage = nullptr;
    m->stage_bytes = 0;
  }
  RB_CUDA(cudaStreamSynchronize(m->c->stream));
  m->finalized = true;
  return REWB200_OK;
}

static int session_fill(rewb200_session* s, int batch, int max_len, int num_blocks);

static int session_create_impl(rewb200_model* m, int batch, int max_len, int num_blocks, rewb200_session** out) {
  RB_REQUIRE(m && out, "rewb200_session_create: NULL argument");
  RB_REQUIRE(m->finalized, "rewb200_session_create: call rewb200_model_finalize first");
  RB_REQUIRE(batch > 0 && max_len > 0, "initKvCache: batch and maxLen must be positive");
  RB_REQUIRE(max_len <= m->cfg.max_seq, "KvCache maxLen " + std::to_string(max_len) + " exceeds maxSeqLen " +
                                            std::to_string(m->cfg.max_seq) + " of the RoPE tables");
  Ctx* c = m->c;
  RB_CUDA(cudaSetDevice(c->device));
  rewb200_session* s = new rewb200_session();
  s->m = m;
  const int st = session_fill(s, batch, max_len, num_blocks);
  if (st != REWB200_OK) {
    const std::string why = rewb200_last_error();  // freeing must not replace the message of the failure
    rewb200_session_free(s);
    set_error(why);
    return st;
  }
  *out = s;
  return REWB200_OK;
}

// Allocates everything a new session owns; on an error the caller frees what has been allocated so far.
static int session_fill(rewb200_session* s, int batch, int max_len, int num_blocks) {
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  s->B = batch;
  s->max_len = max_len;
  s->max_pages = (max_len + PAGE - 1) / PAGE;
  s->paged = num_blocks > 0;
  s->num_blocks = num_blocks;
  const int64_t n_pages = s->paged ? (int64_t)num_blocks : (int64_t)batch * s->max_pages;
  const size_t es = dtype_size(m->cfg.dtype);
  const int64_t cache_rows = n_pages * m->kvh_l * PAGE;
  const size_t cache_bytes = (size_t)cache_rows * m->cfg.head_dim * es;
  s->kc.resize(m->cfg.n_layers);
  s->vc.resize(m->cfg.n_layers);
  s->tmK.resize(m->cfg.n_layers);
  s->tmV.resize(m->cfg.n_layers);
  for (int l = 0; l < m->cfg.n_layers; ++l) {
    RB_CUDA(cudaMalloc(&s->kc[l], cache_bytes));
    RB_CUDA(cudaMalloc(&s->vc[l], cache_bytes));
    RB_CUDA(cudaMemsetAsync(s->kc[l], 0, cache_bytes, c->stream));
    RB_CUDA(cudaMemsetAsync(s->vc[l], 0, cache_bytes, c->stream));
    if (m->cfg.dtype == REWB200_BF16) {
      RB_TRY(make_tmap_2d_bf16(&s->tmK[l], s->kc[l], m->cfg.head_dim, cache_rows, (uint64_t)m->cfg.head_dim * 2, 64, 64));
      RB_TRY(make_tmap_2d_bf16(&s->tmV[l], s->vc[l], m->cfg.head_dim, cache_rows, (uint64_t)m->cfg.head_dim * 2, 64, 64));
    }
  }
  const int64_t n_bt = (int64_t)batch * s->max_pages;
  std::vector<int> bt((size_t)n_bt, 0);
  if (!s->paged)
    for (int64_t i = 0; i < n_bt; ++i) bt[i] = (int)i;  // sequence b owns pages [b*max_pages, (b+1)*max_pages)
  RB_CUDA(cudaMalloc((void**)&s->block_table, n_bt * sizeof(int)));
  RB_CUDA(cudaMemcpyAsync(s->block_table, bt.data(), n_bt * sizeof(int), cudaMemcpyHostToDevice, c->stream));
  if (s->paged) {
    // every lane idle on the scratch page 0; blocks 1.. are free (PagedKvCache.freeBlocks, generate.nim:86-88)
    for (int i = num_blocks - 1; i >= 1; --i) s->free_blocks.push_back(i);
    s->lane_len.assign(batch, 0);
    s->lane_active.assign(batch, 0);
    s->lane_pages.assign(batch, {});
    RB_CUDA(cudaMalloc((void**)&s->d_active, batch * sizeof(int)));
    RB_CUDA(cudaMemsetAsync(s->d_active, 0, batch * sizeof(int), c->stream));
    RB_CUDA(cudaMalloc((void**)&s->d_ids_prefill, (size_t)max_len * sizeof(int)));
  }
  RB_CUDA(cudaMalloc((void**)&s->d_pos, batch * sizeof(int)));
  RB_CUDA(cudaMalloc((void**)&s->d_next, batch * sizeof(int)));
  RB_CUDA(cudaMalloc((void**)&s->d_step, sizeof(int)));
  RB_CUDA(cudaMalloc((void**)&s->d_ids, (size_t)batch * max_len * sizeof(int)));
  RB_CUDA(cudaMemsetAsync(s->d_ids, 0, (size_t)batch * max_len * sizeof(int), c->stream));  // idle lanes decode token 0
  s->out_capacity = max_len;
  RB_CUDA(cudaMalloc((void**)&s->d_out, (size_t)batch * s->out_capacity * sizeof(int)));
  RB_CUDA(cudaMallocHost((void**)&s->h_ids, (size_t)batch * max_len * sizeof(int)));
  RB_CUDA(cudaMemsetAsync(s->d_pos, 0, batch * sizeof(int), c->stream));
  RB_CUDA(cudaMemsetAsync(s->d_step, 0, sizeof(int), c->stream));
  s->attn_scratch_bytes = attn_scratch_bytes(batch, m->nh_l, m->cfg.head_dim, 16);
  RB_CUDA(cudaMalloc((void**)&s->attn_scratch, s->attn_scratch_bytes));
  RB_CUDA(cudaMalloc(&s->argmax_scratch, (size_t)batch * 64 * 8));
  if (m->cfg.tp_size > 1) {
    RB_REQUIRE(comm_world(m->slot) == m->cfg.tp_size && comm_rank(m->slot) == m->cfg.tp_rank,
               "tensor-parallel model needs rewb200_comm_init with the same rank and world size first");
    s->gather_bytes = std::max<size_t>((size_t)batch * 64 * 8 * m->cfg.tp_size, (size_t)batch * m->cfg.vocab * sizeof(float));
    RB_CUDA(cudaMalloc(&s->gather_scratch, s->gather_bytes));
  }
  RB_CUDA(cudaEventCreate(&s->ev0));
  RB_CUDA(cudaEventCreate(&s->ev1));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  return REWB200_OK;
}

int rewb200_session_create(rewb200_model* m, int batch, int max_len, rewb200_session** out) {
  return session_create_impl(m, batch, max_len, 0, out);
}

int rewb200_session_create_paged(rewb200_model* m, int lanes, int max_len, int num_blocks, rewb200_session** out) {
  RB_REQUIRE(m && out, "rewb200_session_create_paged: NULL argument");
  RB_REQUIRE(num_blocks >= 2, "initPagedKvCache: numBlocks must be at least 2 (block 0 is the idle lanes' scratch block)");
  RB_REQUIRE(m->cfg.tp_size <= 1 && m->cfg.ep_size <= 1, "paged lanes are not available on a sharded model");
  return session_create_impl(m, lanes, max_len, num_blocks, out);
}

void rewb200_session_free(rewb200_session* s) {
  if (!s) return;
  Ctx* c = s->m->c;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  if (s->graph) cudaGraphExecDestroy(s->graph);
  for (void* p : s->kc) cudaFree(p);
  for (void* p : s->vc) cudaFree(p);
  void* ptrs[] = {s->d_active, s->d_ids_prefill, s->block_table, s->d_pos, s->d_ids, s->d_next, s->d_out, s->d_step, s->x_res, s->xn, s->q,
                  s->attn, s->h, s->part, s->gu32, s->logits, s->attn_scratch, s->argmax_scratch, s->gather_scratch,
                  s->samp_hist, s->samp_hist_len, s->samp_steps, s->samp_keys, s->samp_work, s->samp_logprob, s->moe_logits, s->moe_topw, s->moe_topi, s->moe_ints,
                  s->moe_send, s->moe_recv, s->moe_xs, s->moe_hs, s->moe_ys, s->moe_ret, s->moe_back, s->moe_tmp, s->route_rec};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  if (s->h_ids) cudaFreeHost(s->h_ids);
  if (s->ev0) cudaEventDestroy(s->ev0);
  if (s->ev1) cudaEventDestroy(s->ev1);
  delete s;
}

int rewb200_session_reset(rewb200_session* s) {
  RB_REQUIRE(s, "rewb200_session_reset: NULL session");
  Ctx* c = s->m->c;
  RB_CUDA(cudaSetDevice(c->device));
  if (s->paged)
    for (int b = 0; b < s->B; ++b) RB_TRY(rewb200_lane_release(s, b));
  RB_CUDA(cudaMemsetAsync(s->d_pos, 0, s->B * sizeof(int), c->stream));
  RB_CUDA(cudaMemsetAsync(s->d_step, 0, sizeof(int), c->stream));
  s->host_pos = 0;
  if (s->samp_on) RB_TRY(samp_restart(s));
  return REWB200_OK;
}

int rewb200_session_forward(rewb200_session* s, const int32_t* ids, int S, int32_t* next_ids, float* logits_out) {
  RB_REQUIRE(s && ids, "rewb200_session_forward: NULL argument");
  RB_REQUIRE(!s->paged, "rewb200_session_forward: a paged session is driven by rewb200_lane_admit / rewb200_lanes_step");
  RB_REQUIRE(S > 0, "generate: tokenIds must not be empty");
  RB_REQUIRE(s->host_pos + S <= s->max_len, "KvCache.append: total length " + std::to_string(s->host_pos + S) +
                                                " exceeds maxLen " + std::to_string(s->max_len));
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t rows = (int64_t)s->B * S;
  for (int64_t i = 0; i < rows; ++i)
    RB_REQUIRE(ids[i] >= 0 && ids[i] < m->cfg.vocab, "generate: token id out of range at index " + std::to_string(i));
  RB_TRY(ensure_acts(s, rows, s->B));
  memcpy(s->h_ids, ids, rows * sizeof(int32_t));
  RB_CUDA(cudaEventRecord(s->ev0, c->stream));
  RB_CUDA(cudaMemcpyAsync(s->d_ids, s->h_ids, rows * sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
  RB_CUDA(cudaMemsetAsync(s->d_step, 0, sizeof(int), c->stream));
  if (s->samp_on) {
    // tokens seen so far = everything fed to the model (generate.nim:248 `tokenIds & generated`)
    RB_CUDA(cudaMemcpy2DAsync(s->samp_hist + s->host_pos, (size_t)s->max_len * sizeof(int), s->d_ids, (size_t)S * sizeof(int),
                              (size_t)S * sizeof(int), s->B, cudaMemcpyDeviceToDevice, c->stream));
    // on the slot's stream (a copy on the legacy stream would not be ordered against this non-blocking stream)
    fill_i32_kernel<<<(unsigned)((s->B + 255) / 256), 256, 0, c->stream>>>(s->samp_hist_len, s->B, s->host_pos + S);
    RB_CUDA(cudaGetLastError());
    ++g_launch_total;
  }
  FwdOpts o;
  o.S = S;
  RB_TRY(enqueue_forward(s, o));
  RB_CUDA(cudaEventRecord(s->ev1, c->stream));
  if (next_ids)
    RB_CUDA(cudaMemcpyAsync(next_ids, s->d_next, s->B * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  if (logits_out) RB_TRY(fetch_logits(s, s->B, logits_out));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaEventElapsedTime(&s->prefill_ms, s->ev0, s->ev1));
  s->host_pos += S;
  if (m->cfg.tp_size > 1 || m->cfg.ep_size > 1) RB_TRY(comm_check_async(m->slot));
  return ctx_check_status(c);
}

// n_steps decode steps for every lane of the session (captured once into a CUDA graph, then replayed).
static int decode_core(rewb200_session* s, int n_steps, int32_t* out_ids, float* last_logits) {
  RB_REQUIRE(n_steps <= s->out_capacity, "too many decode steps for the session's id buffer");
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(ensure_acts(s, std::max<int64_t>(s->B, s->rows_cap), s->B));
  FwdOpts o;
  o.S = 1;
  const char* nograph = getenv("REW_B200_NO_GRAPH");
  const bool use_graph = !(nograph && nograph[0] == '1');
  if (s->graph && s->graph_epoch != c->option_epoch) {
    cudaGraphExecDestroy(s->graph);
    s->graph = nullptr;
  }
  if (use_graph && !s->graph && n_steps > 0) {
    s->graph_epoch = c->option_epoch;
    cudaGraph_t g;
    const int64_t before = g_launch_total;
    RB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int st = enqueue_forward(s, o);
    s->graph_kernels = (int)(g_launch_total - before);
    cudaError_t e = cudaStreamEndCapture(c->stream, &g);
    if (st != REWB200_OK) {
      if (e == cudaSuccess) cudaGraphDestroy(g);
      return st;
    }
    RB_CUDA(e);
    RB_CUDA(cudaGraphInstantiate(&s->graph, g, 0));
    RB_CUDA(cudaGraphDestroy(g));
  }
  RB_CUDA(cudaMemsetAsync(s->d_step, 0, sizeof(int), c->stream));
  RB_CUDA(cudaEventRecord(s->ev0, c->stream));
  for (int i = 0; i < n_steps; ++i) {
    if (use_graph) {
      RB_CUDA(cudaGraphLaunch(s->graph, c->stream));
      g_launch_total += s->graph_kernels;
    } else {
      RB_TRY(enqueue_forward(s, o));
    }
  }
  RB_CUDA(cudaEventRecord(s->ev1, c->stream));
  if (out_ids && n_steps > 0) {
    // device layout [step][B] -> host [B][n_steps]
    std::vector<int32_t> tmp((size_t)n_steps * s->B);
    RB_CUDA(cudaMemcpyAsync(tmp.data(), s->d_out, tmp.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
    RB_CUDA(cudaStreamSynchronize(c->stream));
    for (int st = 0; st < n_steps; ++st)
      for (int b = 0; b < s->B; ++b) out_ids[(size_t)b * n_steps + st] = tmp[(size_t)st * s->B + b];
  }
  if (last_logits) RB_TRY(fetch_logits(s, s->B, last_logits));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaEventElapsedTime(&s->decode_ms, s->ev0, s->ev1));
  if (m->cfg.tp_size > 1 || m->cfg.ep_size > 1) RB_TRY(comm_check_async(m->slot));
  return ctx_check_status(c);
}

int rewb200_session_decode(rewb200_session* s, int n_steps, int32_t* out_ids, float* last_logits) {
  RB_REQUIRE(s, "rewb200_session_decode: NULL session");
  RB_REQUIRE(!s->paged, "rewb200_session_decode: a paged session is driven by rewb200_lane_admit / rewb200_lanes_step");
  RB_REQUIRE(n_steps >= 0, "n_steps must be non-negative");
  RB_REQUIRE(s->host_pos > 0, "rewb200_session_decode: feed a prompt with rewb200_session_forward first");
  RB_REQUIRE(s->host_pos + n_steps <= s->max_len, "KvCache.append: total length " +
                                                      std::to_string(s->host_pos + n_steps) + " exceeds maxLen " +
                                                      std::to_string(s->max_len));
  RB_TRY(decode_core(s, n_steps, out_ids, last_logits));
  s->host_pos += n_steps;
  return REWB200_OK;
}

int rewb200_generate_stop(rewb200_session* s, const int32_t* prompt, int S, int n_new, int eos, const int32_t* stop_ids,
                          int n_stop, int32_t* out_ids, float* last_logits) {
  RB_REQUIRE(s && prompt && out_ids, "rewb200_generate: NULL argument");
  RB_REQUIRE(!s->paged, "rewb200_generate: a paged session is driven by rewb200_lane_admit / rewb200_lanes_step");
  RB_REQUIRE(n_new >= 1, "generate: maxNewTokens must be positive");
  RB_REQUIRE(n_stop >= 0 && (n_stop == 0 || stop_ids != nullptr), "generate: stopTokenIds missing");
  // `nextToken in config.stopTokenIds or nextToken == eosTokenId` (generate.nim:263)
  auto is_stop = [&](int32_t id) {
    if (eos >= 0 && id == eos) return true;
    for (int i = 0; i < n_stop; ++i)
      if (id == stop_ids[i]) return true;
    return false;
  };
  const bool stops = eos >= 0 || n_stop > 0;
  RB_TRY(rewb200_session_reset(s));
  std::vector<int32_t> first(s->B);
  RB_TRY(rewb200_session_forward(s, prompt, S, first.data(), n_new == 1 ? last_logits : nullptr));
  for (int b = 0; b < s->B; ++b) out_ids[(size_t)b * n_new] = first[b];
  if (n_new == 1) return REWB200_OK;
  auto all_done = [&](int upto) {
    for (int b = 0; b < s->B; ++b) {
      bool hit = false;
      for (int t = 0; t < upto; ++t) hit |= is_stop(out_ids[(size_t)b * n_new + t]);
      if (!hit) return false;
    }
    return true;
  };
  if (!stops) {
    std::vector<int32_t> rest((size_t)s->B * (n_new - 1));
    RB_TRY(rewb200_session_decode(s, n_new - 1, rest.data(), last_logits));
    for (int b = 0; b < s->B; ++b)
      for (int t = 1; t < n_new; ++t) out_ids[(size_t)b * n_new + t] = rest[(size_t)b * (n_new - 1) + t - 1];
    return REWB200_OK;
  }
  // With stop tokens the host looks at the ids every 8 steps.
  int done = 1;
  for (int b = 0; b < s->B; ++b)
    for (int t = 1; t < n_new; ++t) out_ids[(size_t)b * n_new + t] = -1;
  while (done < n_new && !all_done(done)) {
    const int chunk = std::min(8, n_new - done);
    std::vector<int32_t> rest((size_t)s->B * chunk);
    RB_TRY(rewb200_session_decode(s, chunk, rest.data(), last_logits));
    for (int b = 0; b < s->B; ++b)
      for (int t = 0; t < chunk; ++t) out_ids[(size_t)b * n_new + done + t] = rest[(size_t)b * chunk + t];
    done += chunk;
  }
  // ids after a sequence's first stop token are not part of its output (generate.nim:263-264)
  for (int b = 0; b < s->B; ++b) {
    bool hit = false;
    for (int t = 0; t < n_new; ++t) {
      if (hit) out_ids[(size_t)b * n_new + t] = -1;
      else if (is_stop(out_ids[(size_t)b * n_new + t])) hit = true;
    }
  }
  return REWB200_OK;
}

int rewb200_generate(rewb200_session* s, const int32_t* prompt, int S, int n_new, int eos, int32_t* out_ids,
                     float* last_logits) {
  return rewb200_generate_stop(s, prompt, S, n_new, eos, nullptr, 0, out_ids, last_logits);
}


// ---- paged lanes: continuous batching over a shared pool of KV blocks -----------------------------

namespace {

// Makes sure `lane` owns blocks for `new_len` tokens and uploads its block-table row when it grew.
int lane_reserve(rewb200_session* s, int lane, int new_len) {
  Ctx* c = s->m->c;
  const int need = (new_len + PAGE - 1) / PAGE;
  std::vector<int>& pages = s->lane_pages[lane];
  if ((int)pages.size() >= need) return REWB200_OK;
  RB_REQUIRE((int)s->free_blocks.size() >= need - (int)pages.size(),
             "PagedKvCache: out of free blocks (lane " + std::to_string(lane) + " needs " +
                 std::to_string(need - (int)pages.size()) + ", " + std::to_string(s->free_blocks.size()) + " free)");
  while ((int)pages.size() < need) {
    pages.push_back(s->free_blocks.back());
    s->free_blocks.pop_back();
  }
  std::vector<int> row((size_t)s->max_pages, 0);
  for (size_t i = 0; i < pages.size(); ++i) row[i] = pages[i];
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaMemcpy(s->block_table + (size_t)lane * s->max_pages, row.data(), row.size() * sizeof(int), cudaMemcpyHostToDevice));
  return REWB200_OK;
}

int lane_check(const rewb200_session* s, int lane, const char* who) {
  RB_REQUIRE(s, std::string(who) + ": NULL session");
  RB_REQUIRE(s->paged, std::string(who) + ": the session was not created with rewb200_session_create_paged");
  RB_REQUIRE(lane >= 0 && lane < s->B, std::string(who) + ": lane " + std::to_string(lane) + " out of range");
  return REWB200_OK;
}

}  // namespace

int rewb200_session_free_blocks(const rewb200_session* s) { return (s && s->paged) ? (int)s->free_blocks.size() : -1; }

int rewb200_lane_length(const rewb200_session* s, int lane) {
  if (!s || !s->paged || lane < 0 || lane >= s->B || !s->lane_active[lane]) return -1;
  return s->lane_len[lane];
}

int rewb200_lane_admit(rewb200_session* s, int lane, const int32_t* ids, int S, uint64_t seed, int32_t* next_id) {
  RB_TRY(lane_check(s, lane, "rewb200_lane_admit"));
  RB_REQUIRE(ids, "rewb200_lane_admit: NULL ids");
  RB_REQUIRE(!s->lane_active[lane], "rewb200_lane_admit: lane " + std::to_string(lane) + " is busy; release it first");
  RB_REQUIRE(S > 0, "generate: tokenIds must not be empty");
  RB_REQUIRE(S < s->max_len, "KvCache.append: total length " + std::to_string(S + 1) + " exceeds maxLen " + std::to_string(s->max_len));
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  RB_CUDA(cudaSetDevice(c->device));
  for (int i = 0; i < S; ++i)
    RB_REQUIRE(ids[i] >= 0 && ids[i] < m->cfg.vocab, "generate: token id out of range at index " + std::to_string(i));
  RB_TRY(lane_reserve(s, lane, S));
  RB_TRY(ensure_acts(s, std::max<int64_t>(std::max<int64_t>(S, s->B), s->rows_cap), s->B));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  const int one = 1, zero = 0;
  RB_CUDA(cudaMemcpy(s->d_ids_prefill, ids, (size_t)S * sizeof(int), cudaMemcpyHostToDevice));
  RB_CUDA(cudaMemcpy(s->d_pos + lane, &zero, sizeof(int), cudaMemcpyHostToDevice));
  RB_CUDA(cudaMemcpy(s->d_active + lane, &one, sizeof(int), cudaMemcpyHostToDevice));
  if (s->samp_on) {
    // this lane's generate() starts over: Key = initKey(seed), step 0, seen = the prompt
    s->samp_seeds[lane] = seed;
    const uint32_t k[2] = {(uint32_t)(seed & 0xFFFFFFFFull), (uint32_t)(seed >> 32)};
    RB_CUDA(cudaMemcpy(s->samp_keys + 2 * lane, k, sizeof(k), cudaMemcpyHostToDevice));
    RB_CUDA(cudaMemcpy(s->samp_steps + lane, &zero, sizeof(int), cudaMemcpyHostToDevice));
    RB_CUDA(cudaMemcpy(s->samp_hist + (size_t)lane * s->max_len, ids, (size_t)S * sizeof(int), cudaMemcpyHostToDevice));
    RB_CUDA(cudaMemcpy(s->samp_hist_len + lane, &S, sizeof(int), cudaMemcpyHostToDevice));
  }
  RB_CUDA(cudaEventRecord(s->ev0, c->stream));
  FwdOpts o;
  o.S = S;
  o.b0 = lane;
  o.nb = 1;
  o.ids_src = s->d_ids_prefill;
  o.record_out = false;
  RB_TRY(enqueue_forward(s, o));
  RB_CUDA(cudaEventRecord(s->ev1, c->stream));
  int32_t first = -1;
  RB_CUDA(cudaMemcpyAsync(&first, s->d_next + lane, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaEventElapsedTime(&s->prefill_ms, s->ev0, s->ev1));
  s->lane_active[lane] = 1;
  s->lane_len[lane] = S;
  if (next_id) *next_id = first;
  return ctx_check_status(c);
}

int rewb200_lanes_step(rewb200_session* s, int n_steps, int32_t* out_ids) {
  RB_TRY(lane_check(s, 0, "rewb200_lanes_step"));
  RB_REQUIRE(n_steps >= 0, "n_steps must be non-negative");
  int need_blocks = 0;
  for (int b = 0; b < s->B; ++b) {
    if (!s->lane_active[b]) continue;
    RB_REQUIRE(s->lane_len[b] + n_steps <= s->max_len, "KvCache.append: total length " +
                                                           std::to_string(s->lane_len[b] + n_steps) + " of lane " +
                                                           std::to_string(b) + " exceeds maxLen " + std::to_string(s->max_len));
    need_blocks += std::max(0, (s->lane_len[b] + n_steps + PAGE - 1) / PAGE - (int)s->lane_pages[b].size());
  }
  // all or nothing: no lane grows unless every lane can
  RB_REQUIRE(need_blocks <= (int)s->free_blocks.size(), "PagedKvCache: out of free blocks (" + std::to_string(need_blocks) +
                                                            " needed for " + std::to_string(n_steps) + " steps, " +
                                                            std::to_string(s->free_blocks.size()) + " free)");
  for (int b = 0; b < s->B; ++b)
    if (s->lane_active[b]) RB_TRY(lane_reserve(s, b, s->lane_len[b] + n_steps));
  RB_TRY(decode_core(s, n_steps, out_ids, nullptr));
  for (int b = 0; b < s->B; ++b)
    if (s->lane_active[b]) s->lane_len[b] += n_steps;
  return REWB200_OK;
}

int rewb200_lane_release(rewb200_session* s, int lane) {
  RB_TRY(lane_check(s, lane, "rewb200_lane_release"));
  if (!s->lane_active[lane] && s->lane_pages[lane].empty()) return REWB200_OK;  // idempotent
  Ctx* c = s->m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  const int zero = 0;
  RB_CUDA(cudaMemcpy(s->d_active + lane, &zero, sizeof(int), cudaMemcpyHostToDevice));
  RB_CUDA(cudaMemcpy(s->d_pos + lane, &zero, sizeof(int), cudaMemcpyHostToDevice));
  std::vector<int> row((size_t)s->max_pages, 0);  // back on the scratch block
  RB_CUDA(cudaMemcpy(s->block_table + (size_t)lane * s->max_pages, row.data(), row.size() * sizeof(int), cudaMemcpyHostToDevice));
  for (int pg : s->lane_pages[lane]) s->free_blocks.push_back(pg);
  s->lane_pages[lane].clear();
  s->lane_active[lane] = 0;
  s->lane_len[lane] = 0;
  return REWB200_OK;
}

int rewb200_session_set_sampling(rewb200_session* s, float temperature, int top_k, float top_p, float min_p,
                                 float repetition_penalty, int do_sample, const uint64_t* seeds) {
  RB_REQUIRE(s, "rewb200_session_set_sampling: NULL session");
  // initGenerationConfig's checks (generate.nim:30-49)
  RB_REQUIRE(temperature >= 0.f, "initGenerationConfig: temperature must be non-negative");
  RB_REQUIRE(top_k >= 0, "initGenerationConfig: topK must be non-negative");
  RB_REQUIRE(top_p > 0.f && top_p <= 1.f, "initGenerationConfig: topP must be in (0, 1]");
  RB_REQUIRE(min_p >= 0.f && min_p <= 1.f, "initGenerationConfig: minP must be in [0, 1]");
  RB_REQUIRE(repetition_penalty > 0.f, "initGenerationConfig: repetitionPenalty must be positive");
  RB_REQUIRE(top_k <= 1024, "device sampling keeps at most 1024 top-k candidates");
  rewb200_model* m = s->m;
  RB_REQUIRE(m->cfg.tp_size <= 1, "device sampling is not available on a vocabulary-sharded (tensor-parallel) model");
  Ctx* c = m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  if (!s->samp_hist) {
    RB_CUDA(cudaMalloc((void**)&s->samp_hist, (size_t)s->B * s->max_len * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->samp_hist_len, s->B * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->samp_steps, s->B * sizeof(int)));
    RB_CUDA(cudaMalloc((void**)&s->samp_keys, (size_t)s->B * 2 * sizeof(uint32_t)));
    RB_CUDA(cudaMalloc((void**)&s->samp_work, (size_t)s->B * m->cfg.vocab * sizeof(float)));
    RB_CUDA(cudaMalloc((void**)&s->samp_logprob, (size_t)s->B * s->max_len * sizeof(float)));
  }
  s->samp_seeds.assign((size_t)s->B, 0);
  if (seeds)
    for (int b = 0; b < s->B; ++b) s->samp_seeds[b] = seeds[b];
  s->samp_temperature = temperature;
  s->samp_top_k = top_k;
  s->samp_top_p = top_p;
  s->samp_min_p = min_p;
  s->samp_rep = repetition_penalty;
  s->samp_do_sample = do_sample ? 1 : 0;
  s->samp_on = true;
  if (s->graph) {  // the captured decode step carries the old sampling arguments
    cudaGraphExecDestroy(s->graph);
    s->graph = nullptr;
  }
  return samp_restart(s);
}

int rewb200_session_clear_sampling(rewb200_session* s) {
  RB_REQUIRE(s, "rewb200_session_clear_sampling: NULL session");
  Ctx* c = s->m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  s->samp_on = false;
  if (s->graph) {
    cudaGraphExecDestroy(s->graph);
    s->graph = nullptr;
  }
  return REWB200_OK;
}

int rewb200_session_logprobs(rewb200_session* s, int n, float* out) {
  RB_REQUIRE(s && out, "rewb200_session_logprobs: NULL argument");
  RB_REQUIRE(s->samp_on, "rewb200_session_logprobs: call rewb200_session_set_sampling first");
  RB_REQUIRE(n >= 0 && n <= s->max_len, "rewb200_session_logprobs: n out of range");
  if (n == 0) return REWB200_OK;
  Ctx* c = s->m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaMemcpy2D(out, (size_t)n * sizeof(float), s->samp_logprob, (size_t)s->max_len * sizeof(float),
                       (size_t)n * sizeof(float), s->B, cudaMemcpyDeviceToHost));
  return REWB200_OK;
}

int rewb200_session_last_ms(const rewb200_session* s, float* prefill_ms, float* decode_ms) {
  RB_REQUIRE(s, "rewb200_session_last_ms: NULL session");
  if (prefill_ms) *prefill_ms = s->prefill_ms;
  if (decode_ms) *decode_ms = s->decode_ms;
  return REWB200_OK;
}

// Times only the Linear launches of one decode step (q|k|v, o, gate|up, down of
// every layer and lm_head, same buffers and split-K choices as the real step),
// `iters` times back to back, with CUDA events on the launching stream.
int rewb200_session_profile_linears(rewb200_session* s, int iters, float* ms_per_step, int64_t* bytes_per_step,
                                    int* launches_per_step) {
  RB_REQUIRE(s && ms_per_step && iters > 0, "rewb200_session_profile_linears: bad argument");
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  RB_REQUIRE(m->cfg.dtype == REWB200_BF16, "linear profiling is for bf16 models");
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(ensure_acts(s, std::max<int64_t>(s->B, s->rows_cap), s->B));
  const int64_t rows = s->B, d = m->cfg.d_model;
  int64_t bytes = 0;
  int launches = 0;
  const int pm = c->profile_mask;  // option profile_linears: which of the launches to time
  auto one_step = [&](bool count) -> int {
    for (LayerDev& L : m->layers) {
      if (L.moe || L.ffn_local == 0) return fail("linear profiling covers dense decoder blocks only");
      // algorithmic bytes of one Linear: weights (bf16, or NF4 codes + scales) + activations in + result out
      auto wbytes = [&](const LinW& w) { return w.quant ? w.K * w.N / 2 + w.K * (w.N / 64) * 2 : w.K * w.N * 2; };  // codes + bf16 scale pairs
      int ks = 1;
      if (pm & 1) {
        RB_TRY(run_linear(s, L.qkv, s->xn, d, rows, true, 0, s->part, m->nqkv, &ks));
        if (count) bytes += wbytes(L.qkv) + rows * L.qkv.K * 2 + (int64_t)ks * rows * L.qkv.N * 4;
        if (count) ++launches;
      }
      if (pm & 2) {
        RB_TRY(run_linear(s, L.o, s->attn, m->nq, rows, true, 0, s->part, d, &ks));
        if (count) bytes += wbytes(L.o) + rows * L.o.K * 2 + (int64_t)ks * rows * L.o.N * 4;
        if (count) ++launches;
      }
      if (pm & 4) {
        RB_TRY(run_linear(s, L.gu, s->xn, d, rows, false, EPI_SWIGLU_BF16, s->h, L.ffn_local, nullptr));
        if (count) bytes += wbytes(L.gu) + rows * L.gu.K * 2 + rows * L.ffn_local * 2;
        if (count) ++launches;
      }
      if (pm & 8) {
        RB_TRY(run_linear(s, L.down, s->h, L.ffn_local, rows, true, 0, s->part, d, &ks));
        if (count) bytes += wbytes(L.down) + rows * L.down.K * 2 + (int64_t)ks * rows * L.down.N * 4;
        if (count) ++launches;
      }
    }
    if (pm & 16) {
      RB_TRY(linear_bf16_launch(c, m->lm.plan, (const bf16*)s->xn, d, rows, EPI_BIAS_F32, 1, s->logits, m->vocab_l, m->lm.b,
                                nullptr, 0));
      if (count) {
        bytes += (m->lm.K * m->lm.N + rows * m->lm.K) * 2 + rows * m->lm.N * 4;
        launches += 1;
      }
    }
    return REWB200_OK;
  };
  RB_TRY(one_step(true));  // warm-up, also counts bytes
  RB_CUDA(cudaEventRecord(s->ev0, c->stream));
  for (int i = 0; i < iters; ++i) RB_TRY(one_step(false));
  RB_CUDA(cudaEventRecord(s->ev1, c->stream));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  float ms = 0.f;
  RB_CUDA(cudaEventElapsedTime(&ms, s->ev0, s->ev1));
  *ms_per_step = ms / iters;
  if (bytes_per_step) *bytes_per_step = bytes;
  if (launches_per_step) *launches_per_step = launches;
  return ctx_check_status(c);
}

int rewb200_session_graph_kernels(const rewb200_session* s) { return s ? s->graph_kernels : 0; }

int rewb200_session_routing(rewb200_session* s, int moe_layer, int32_t* topi_out, int64_t rows) {
  RB_REQUIRE(s && topi_out, "rewb200_session_routing: NULL argument");
  RB_REQUIRE(s->route_rec != nullptr, "rewb200_session_routing: set option record_routing=1 before the session's first forward");
  int n_moe = 0;
  for (const LayerDev& L : s->m->layers) n_moe += L.moe ? 1 : 0;
  RB_REQUIRE(moe_layer >= 0 && moe_layer < n_moe && rows == s->route_rows, "rewb200_session_routing: layer or row count does not match the last forward");
  Ctx* c = s->m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  RB_CUDA(cudaMemcpy(topi_out, s->route_rec + (size_t)moe_layer * s->rows_cap * s->m->cfg.top_k,
                     (size_t)rows * s->m->cfg.top_k * sizeof(int), cudaMemcpyDeviceToHost));
  return REWB200_OK;
}

int rewb200_session_trace_step(rewb200_session* s, float* ms_by_category, int n) {
  RB_REQUIRE(s && ms_by_category && n >= TC_COUNT, "rewb200_session_trace_step: needs room for 11 categories");
  RB_REQUIRE(!s->paged && s->host_pos > 0 && s->host_pos + 1 <= s->max_len, "rewb200_session_trace_step: feed a prompt first");
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(ensure_acts(s, std::max<int64_t>(s->B, s->rows_cap), s->B));
  Trace tr;
  FwdOpts o;
  o.S = 1;
  o.trace = &tr;
  RB_TRY(enqueue_forward(s, o));
  RB_TRY(tr.finish(ms_by_category));
  s->host_pos += 1;
  for (int i = TC_COUNT; i < n; ++i) ms_by_category[i] = 0.f;
  return ctx_check_status(c);
}

int rewb200_model_forward_all(rewb200_session* s, const int32_t* ids, int S, int64_t offset, int causal,
                              float* logits_out) {
  RB_REQUIRE(s && ids && logits_out, "rewb200_model_forward_all: NULL argument");
  RB_REQUIRE(S > 0 && S <= s->max_len, "sequence length out of range for this session");
  rewb200_model* m = s->m;
  Ctx* c = m->c;
  RB_REQUIRE(offset >= 0 && offset + S <= m->cfg.max_seq, "RotaryPositionEncoding.forward: position " +
                                                             std::to_string(offset + S) + " exceeds maxSeqLen " +
                                                             std::to_string(m->cfg.max_seq));
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t rows = (int64_t)s->B * S;
  for (int64_t i = 0; i < rows; ++i)
    RB_REQUIRE(ids[i] >= 0 && ids[i] < m->cfg.vocab, "token id out of range at index " + std::to_string(i));
  RB_TRY(rewb200_session_reset(s));
  RB_TRY(ensure_acts(s, rows, rows));
  memcpy(s->h_ids, ids, rows * sizeof(int32_t));
  RB_CUDA(cudaMemcpyAsync(s->d_ids, s->h_ids, rows * sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
  FwdOpts o;
  o.S = S;
  o.rope_shift = (int)offset;
  o.causal = causal;
  o.all_logits = true;
  RB_TRY(enqueue_forward(s, o));
  RB_TRY(fetch_logits(s, rows, logits_out));
  return ctx_check_status(c);
}

}  // extern "C"
