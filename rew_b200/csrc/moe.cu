// Mixture-of-experts routing for DeepSeekMoE.forward
// (src/rew/models/deepseek.nim:122-145).
//
// moe_route_kernel: one warp per token does what the reference spends a
// softmax chain and two full stable sorts on (deepseek.nim:132-138,
// src/rew/ops/sort.nim:36-90): softmax over the E router logits, the k largest
// probabilities in descending order (exact ties resolved towards the lower
// expert index), renormalised by their sum.
#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "ptx.cuh"

namespace rewb {
namespace {

constexpr int MAX_E_PER_LANE = 8;  // E <= 256

// logits: nsplit slabs [N][E] split_stride apart, summed in slab order, plus bias (may be null).
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int nsplit, int64_t split_stride,
                                                        const float* __restrict__ bias, int64_t N, int E, int k,
                                                        float* __restrict__ topw, int* __restrict__ topi, int* zero, int n_zero) {
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.x == 0 && (int)threadIdx.x < n_zero) zero[threadIdx.x] = 0;  // the dispatch kernel's per-peer cursors
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= N) return;
  const float* lr = logits + tok * E;
  float p[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    float v = -INFINITY;
    if (e < E) {
      v = 0.f;
      for (int sp = 0; sp < nsplit; ++sp) v += lr[sp * split_stride + e];
      if (bias) v += bias[e];
    }
    p[i] = v;
    mx = fmaxf(mx, p[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = (e < E) ? expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = (e < E) ? p[i] / sum : -1.f;  // probabilities are >= 0; -1 marks "absent / taken"
  }
  float denom = 0.f;
  float myw = 0.f;
  int myi = 0;
  for (int j = 0; j < k; ++j) {
    float bv = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (p[i] > bv || (p[i] == bv && e < be)) {
        bv = p[i];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    denom += bv;
    if (lane == j % 32) {
      myw = bv;
      myi = be;
    }
    if ((be & 31) == lane) p[be >> 5] = -1.f;
    if (j % 32 == 31 || j == k - 1) {
      // flush up to 32 selections held one per lane
      const int base = (j / 32) * 32;
      if (base + lane <= j) {
        topw[tok * k + base + lane] = myw;
        topi[tok * k + base + lane] = myi;
      }
    }
  }
  __syncwarp();
  for (int j = lane; j < k; j += 32) topw[tok * k + j] = topw[tok * k + j] / denom;
}


// ---- dispatch / gather / combine around the grouped expert GEMMs -------------
// Pairs (token, j) are sent to the rank that owns expert topi[token][j] into
// fixed-capacity per-peer slot arrays (capacity = tokens * k, the worst case), so
// an expert-parallel all-to-all needs no count exchange.  Slot order inside a
// peer comes from an atomic counter and may vary between runs; results do not
// depend on it because every pair is computed independently and each token sums
// its k results in the fixed order j = 0..k-1.

__global__ void moe_reset_kernel(int* cursor, int n_cursor, int* count, int n_count, int* meta, int n_meta) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_cursor) cursor[i] = 0;
  if (i < n_count) count[i] = 0;
  if (i < n_meta) meta[i] = -1;
}

template <typename T>
__global__ void __launch_bounds__(128) moe_dispatch_kernel(const T* __restrict__ x, const int* __restrict__ topi, int k,
                                                           int64_t d, int experts_per_rank, int capacity, int* cursor,
                                                           T* send_x, int* send_meta, int* pair_slot) {
  __shared__ int s_slot;
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  if (threadIdx.x == 0) {
    const int e = topi[pair];
    const int p = e / experts_per_rank;
    const int slot = p * capacity + atomicAdd(&cursor[p], 1);
    send_meta[slot] = e % experts_per_rank;
    pair_slot[pair] = slot;
    s_slot = slot;
  }
  __syncthreads();
  const int tok = pair / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)tok * d);
  uint4* dst = reinterpret_cast<uint4*>(send_x + (int64_t)s_slot * d);
  const int n16 = (int)(d * sizeof(T) / 16);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
}

__global__ void moe_count_kernel(const int* __restrict__ meta, int n_slots, int* count) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_slots && meta[i] >= 0) atomicAdd(&count[meta[i]], 1);
}

__global__ void moe_scan_kernel(const int* count, int n_experts, int* offsets, int* cursor2) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = acc;
      cursor2[e] = acc;
      acc += count[e];
    }
    offsets[n_experts] = acc;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(const T* __restrict__ recv_x, const int* __restrict__ recv_meta,
                                                         int64_t d, int* cursor2, T* xs, int* slot_pos) {
  __shared__ int s_pos;
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  const int e = recv_meta[slot];
  if (e < 0) {
    if (threadIdx.x == 0) slot_pos[slot] = -1;
    return;
  }
  if (threadIdx.x == 0) {
    s_pos = atomicAdd(&cursor2[e], 1);
    slot_pos[slot] = s_pos;
  }
  __syncthreads();
  const uint4* src = reinterpret_cast<const uint4*>(recv_x + (int64_t)slot * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + (int64_t)s_pos * d);
  const int n16 = (int)(d * sizeof(T) / 16);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
}

template <typename T>
__global__ void __launch_bounds__(128) moe_group_local_kernel(const T* __restrict__ x, const int* __restrict__ topi, int n_pairs,
                                                              int k, int64_t d, int n_experts, int* offsets, T* xs,
                                                              int* pair_pos) {
  __shared__ int s_red[4];
  __shared__ int s_hist[32 * MAX_E_PER_LANE + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  const int e = topi[pair];
  int before = 0;  // pairs of lower experts, and earlier pairs of the same expert
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int ep = topi[p];
    before += (ep < e || (ep == e && p < pair)) ? 1 : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = before;
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i <= n_experts; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  const int pos = s_red[0] + s_red[1] + s_red[2] + s_red[3];
  if (threadIdx.x == 0) pair_pos[pair] = pos;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(pair / k) * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + (int64_t)pos * d);
  const int n16 = (int)(d * sizeof(T) / 16);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
  if (blockIdx.x == 0) {
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&s_hist[topi[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int i = 0; i < n_experts; ++i) {
        offsets[i] = acc;
        acc += s_hist[i];
      }
      offsets[n_experts] = acc;
    }
  }
}

// ret[slot] = ys[slot_pos[slot]] for occupied slots: results back in the sender's slot order.
__global__ void __launch_bounds__(128) moe_return_kernel(const float* __restrict__ ys, const int* __restrict__ slot_pos,
                                                         int64_t d, float* ret) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  const int pos = slot_pos[slot];
  float4* dst = reinterpret_cast<float4*>(ret + (int64_t)slot * d);
  const int n4 = (int)(d / 4);
  if (pos < 0) return;  // empty slot: nobody reads its row (the combine follows pair_slot, which names occupied slots only)
  const float4* src = reinterpret_cast<const float4*>(ys + (int64_t)pos * d);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = src[i];
}

// out[token] (+)= sum_j topw[token][j] * back[pair_slot[token][j]]   (deepseek.nim:140-144 for the
// experts a token actually selected; the others have weight 0 in the reference).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ back, const int* __restrict__ pair_slot,
                                                          const float* __restrict__ topw, int k, int64_t d, float* out,
                                                          int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x;
  const int n4 = (int)(d / 4);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      const float w = topw[tok * k + j];
      const float4 v = reinterpret_cast<const float4*>(back + (int64_t)pair_slot[tok * k + j] * d)[i];
      acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    float4* o = reinterpret_cast<float4*>(out + (int64_t)tok * d) + i;
    if (accumulate) {
      const float4 p = *o;
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    *o = acc;
  }
}

// ---- the same steps with the all-to-all done by peer stores (A2aArgs) ------------------------------
// Slot numbering is unchanged: slot = owner_rank * capacity + index on the asking side,
// source_rank * capacity + index on the owning side.

template <typename T>
__global__ void __launch_bounds__(128) moe_dispatch_peer_kernel(const T* __restrict__ x, const int* __restrict__ topi, int k,
                                                                int64_t d, int experts_per_rank, int capacity, int* cursor,
                                                                int* pair_slot, A2aArgs a) {
  __shared__ int s_p, s_idx;
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  if (threadIdx.x == 0) {
    const int e = topi[pair];
    const int p = e / experts_per_rank;
    const int idx = atomicAdd(&cursor[p], 1);
    reinterpret_cast<int*>(a.region[p] + a.off_meta)[(int64_t)a.my_rank * capacity + idx] = e % experts_per_rank;
    pair_slot[pair] = p * capacity + idx;
    s_p = p;
    s_idx = idx;
  }
  __syncthreads();
  const int tok = pair / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)tok * d);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.region[s_p] + a.off_x) + ((int64_t)a.my_rank * capacity + s_idx) * d);
  const int n16 = (int)(d * sizeof(T) / 16);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
  if (grid_last_cta(a.arrive)) {
    // every pair of this rank has been stored: hand each owner its pair count, then the flag
    if ((int)threadIdx.x < a.world) {
      const int p = threadIdx.x;
      const int n = atomicAdd(&cursor[p], 0);
      *reinterpret_cast<volatile int*>(a.cells[p] + a.my_rank) = n;
      peer_flag_release(a.cells[p] + 8 + a.my_rank, *a.epoch + a.offset);
    }
  }
}

// count[e] = pairs for local expert e among the occupied slots; waits for every rank's dispatch flag first.
__global__ void __launch_bounds__(256) moe_count_peer_kernel(int n_slots, int capacity, int* count, A2aArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  peer_flags_wait(a.cells[a.my_rank] + 8, 1, a.world, -1, *a.epoch + a.offset, a.status);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_slots) return;
  const int src = i / capacity, idx = i % capacity;
  if (idx >= __ldcg(a.cells[a.my_rank] + src)) return;
  const int e = __ldcg(reinterpret_cast<const int*>(a.region[a.my_rank] + a.off_meta) + i);
  atomicAdd(&count[e], 1);
}

template <typename T>
__global__ void __launch_bounds__(128) moe_gather_peer_kernel(int64_t d, int capacity, int* cursor2, T* xs, int* slot_pos,
                                                              A2aArgs a) {
  __shared__ int s_pos;
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  const int src = slot / capacity, idx = slot % capacity;
  if (idx >= __ldcg(a.cells[a.my_rank] + src)) {
    if (threadIdx.x == 0) slot_pos[slot] = -1;
    return;
  }
  if (threadIdx.x == 0) {
    const int e = __ldcg(reinterpret_cast<const int*>(a.region[a.my_rank] + a.off_meta) + slot);
    s_pos = atomicAdd(&cursor2[e], 1);
    slot_pos[slot] = s_pos;
  }
  __syncthreads();
  const uint4* src_row = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.region[a.my_rank] + a.off_x) + (int64_t)slot * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + (int64_t)s_pos * d);
  const int n16 = (int)(d * sizeof(T) / 16);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldcg(src_row + i);
}

// Small steps (decode): count, scan and gather in ONE kernel and without atomics.  One CTA per slot; it waits
// for the dispatch flags, looks at every occupied slot's expert id and places its own row behind all rows of
// lower experts and the lower-numbered slots of its own expert (a fixed order), CTA 0 writes the experts' row
// offsets.  n_slots * 4 bytes of ids per CTA out of L2: meant for a few thousand slots at most.
template <typename T>
__global__ void __launch_bounds__(128) moe_group_small_peer_kernel(int n_slots, int capacity, int64_t d, int n_experts,
                                                                   int* offsets, T* xs, int* slot_pos, A2aArgs a) {
  __shared__ int s_cnt[8];
  __shared__ int s_red[4];
  __shared__ int s_hist[32 * MAX_E_PER_LANE + 1];
  pdl_launch_dependents();
  pdl_wait();
  peer_flags_wait(a.cells[a.my_rank] + 8, 1, a.world, -1, *a.epoch + a.offset, a.status);
  if ((int)threadIdx.x < a.world) s_cnt[threadIdx.x] = __ldcg(a.cells[a.my_rank] + threadIdx.x);
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i <= n_experts; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  const int* meta = reinterpret_cast<const int*>(a.region[a.my_rank] + a.off_meta);
  const int slot = blockIdx.x;
  const bool mine = (slot % capacity) < s_cnt[slot / capacity];
  const int e = mine ? __ldcg(meta + slot) : -1;
  int before = 0;
  for (int p = threadIdx.x; p < n_slots; p += blockDim.x) {
    if ((p % capacity) >= s_cnt[p / capacity]) continue;
    const int ep = __ldcg(meta + p);
    before += (ep < e || (ep == e && p < slot)) ? 1 : 0;
    if (blockIdx.x == 0) atomicAdd(&s_hist[ep], 1);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = before;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < n_experts; ++i) {
      offsets[i] = acc;
      acc += s_hist[i];
    }
    offsets[n_experts] = acc;
  }
  if (!mine) {
    if (threadIdx.x == 0) slot_pos[slot] = -1;
    return;
  }
  const int pos = s_red[0] + s_red[1] + s_red[2] + s_red[3];
  if (threadIdx.x == 0) slot_pos[slot] = pos;
  const uint4* src_row = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.region[a.my_rank] + a.off_x) + (int64_t)slot * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + (int64_t)pos * d);
  const int n16 = (int)(d * sizeof(T) / 16);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldcg(src_row + i);
}

// Expert outputs back to the rank that asked, in its slot order; the last CTA raises the return flags.
__global__ void __launch_bounds__(128) moe_return_peer_kernel(const float* __restrict__ ys, const int* __restrict__ slot_pos,
                                                              int64_t d, int capacity, A2aArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x;
  const int pos = slot_pos[slot];
  if (pos >= 0) {
    const int src = slot / capacity, idx = slot % capacity;
    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.region[src] + a.off_back) + ((int64_t)a.my_rank * capacity + idx) * d);
    const float4* from = reinterpret_cast<const float4*>(ys + (int64_t)pos * d);
    const int n4 = (int)(d / 4);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = from[i];
  }
  if (grid_last_cta(a.arrive + 1)) {
    if ((int)threadIdx.x < a.world) peer_flag_release(a.cells[threadIdx.x] + 16 + a.my_rank, *a.epoch + a.offset);
  }
}

__global__ void __launch_bounds__(256) moe_combine_peer_kernel(const int* __restrict__ pair_slot, const float* __restrict__ topw,
                                                               int k, int64_t d, float* out, int accumulate, A2aArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  peer_flags_wait(a.cells[a.my_rank] + 16, 1, a.world, -1, *a.epoch + a.offset, a.status);
  const float* back = reinterpret_cast<const float*>(a.region[a.my_rank] + a.off_back);
  const int tok = blockIdx.x;
  const int n4 = (int)(d / 4);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      const float w = topw[tok * k + j];
      const float4 v = __ldcg(reinterpret_cast<const float4*>(back + (int64_t)pair_slot[tok * k + j] * d) + i);
      acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    float4* o = reinterpret_cast<float4*>(out + (int64_t)tok * d) + i;
    if (accumulate) {
      const float4 p = *o;
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    *o = acc;
  }
}

}  // namespace

#define RB_LAUNCH(kernel, grid, block, ...)                                                   \
  do {                                                                                        \
    RB_CUDA(launch_k(kernel, dim3((unsigned)(grid)), dim3(block), 0, c->stream, c->use_pdl, __VA_ARGS__)); \
    ++g_launch_total;                                                                         \
  } while (0)

int moe_reset_launch(Ctx* c, int* cursor, int n_cursor, int* count, int n_count, int* meta, int n_meta) {
  const int n = std::max(n_cursor, std::max(n_count, n_meta));
  RB_LAUNCH(moe_reset_kernel, (n + 255) / 256, 256, cursor, n_cursor, count, n_count, meta, n_meta);
  return REWB200_OK;
}
int moe_dispatch_launch(Ctx* c, const void* x, int dtype, const int* topi, int64_t tokens, int k, int64_t d,
                        int experts_per_rank, int capacity, int* cursor, void* send_x, int* send_meta, int* pair_slot) {
  if (tokens == 0) return REWB200_OK;
  RB_REQUIRE((d * dtype_size(dtype)) % 16 == 0, "MoE dispatch needs rows that are multiples of 16 bytes");
  if (dtype == REWB200_BF16)
    RB_LAUNCH(moe_dispatch_kernel<bf16>, tokens * k, 128, (const bf16*)x, topi, k, d, experts_per_rank, capacity, cursor,
              (bf16*)send_x, send_meta, pair_slot);
  else
    RB_LAUNCH(moe_dispatch_kernel<float>, tokens * k, 128, (const float*)x, topi, k, d, experts_per_rank, capacity, cursor,
              (float*)send_x, send_meta, pair_slot);
  return REWB200_OK;
}
int moe_group_launch(Ctx* c, const void* recv_x, int dtype, const int* recv_meta, int n_slots, int64_t d, int n_experts,
                     int* count, int* offsets, int* cursor2, void* xs, int* slot_pos) {
  if (n_slots == 0) return REWB200_OK;
  RB_LAUNCH(moe_count_kernel, (n_slots + 255) / 256, 256, recv_meta, n_slots, count);
  RB_LAUNCH(moe_scan_kernel, 1, 32, (const int*)count, n_experts, offsets, cursor2);
  if (dtype == REWB200_BF16)
    RB_LAUNCH(moe_gather_kernel<bf16>, n_slots, 128, (const bf16*)recv_x, recv_meta, d, cursor2, (bf16*)xs, slot_pos);
  else
    RB_LAUNCH(moe_gather_kernel<float>, n_slots, 128, (const float*)recv_x, recv_meta, d, cursor2, (float*)xs, slot_pos);
  return REWB200_OK;
}
int moe_return_launch(Ctx* c, const float* ys, const int* slot_pos, int n_slots, int64_t d, float* ret) {
  if (n_slots == 0) return REWB200_OK;
  RB_LAUNCH(moe_return_kernel, n_slots, 128, ys, slot_pos, d, ret);
  return REWB200_OK;
}
int moe_combine_launch(Ctx* c, const float* back, const int* pair_slot, const float* topw, int64_t tokens, int k, int64_t d,
                       float* out, int accumulate) {
  if (tokens == 0) return REWB200_OK;
  RB_LAUNCH(moe_combine_kernel, tokens, 256, back, pair_slot, topw, k, d, out, accumulate);
  return REWB200_OK;
}

// Peer-heap variants (bf16 or f32 activations).  `cursor` (world ints) and `count` (n_experts + 1 ints) must be zero.
int moe_dispatch_peer_launch(Ctx* c, const void* x, int dtype, const int* topi, int64_t tokens, int k, int64_t d,
                             int experts_per_rank, int capacity, int* cursor, int* pair_slot, const A2aArgs& a) {
  RB_REQUIRE(tokens > 0, "expert-parallel dispatch needs at least one token on every rank");
  RB_REQUIRE((d * dtype_size(dtype)) % 16 == 0, "MoE dispatch needs rows that are multiples of 16 bytes");
  if (dtype == REWB200_BF16)
    RB_LAUNCH(moe_dispatch_peer_kernel<bf16>, tokens * k, 128, (const bf16*)x, topi, k, d, experts_per_rank, capacity, cursor,
              pair_slot, a);
  else
    RB_LAUNCH(moe_dispatch_peer_kernel<float>, tokens * k, 128, (const float*)x, topi, k, d, experts_per_rank, capacity, cursor,
              pair_slot, a);
  return REWB200_OK;
}
int moe_group_peer_launch(Ctx* c, int dtype, int n_slots, int capacity, int64_t d, int n_experts, int* count, int* offsets,
                          int* cursor2, void* xs, int* slot_pos, const A2aArgs& a) {
  if (n_slots <= 4096 && n_experts <= 32 * MAX_E_PER_LANE) {  // decode sizes: one kernel, fixed row order
    if (dtype == REWB200_BF16)
      RB_LAUNCH(moe_group_small_peer_kernel<bf16>, n_slots, 128, n_slots, capacity, d, n_experts, offsets, (bf16*)xs, slot_pos, a);
    else
      RB_LAUNCH(moe_group_small_peer_kernel<float>, n_slots, 128, n_slots, capacity, d, n_experts, offsets, (float*)xs, slot_pos, a);
    return REWB200_OK;
  }
  RB_LAUNCH(moe_count_peer_kernel, (n_slots + 255) / 256, 256, n_slots, capacity, count, a);
  RB_LAUNCH(moe_scan_kernel, 1, 32, (const int*)count, n_experts, offsets, cursor2);
  if (dtype == REWB200_BF16)
    RB_LAUNCH(moe_gather_peer_kernel<bf16>, n_slots, 128, d, capacity, cursor2, (bf16*)xs, slot_pos, a);
  else
    RB_LAUNCH(moe_gather_peer_kernel<float>, n_slots, 128, d, capacity, cursor2, (float*)xs, slot_pos, a);
  return REWB200_OK;
}
int moe_return_peer_launch(Ctx* c, const float* ys, const int* slot_pos, int n_slots, int capacity, int64_t d, const A2aArgs& a) {
  RB_LAUNCH(moe_return_peer_kernel, n_slots, 128, ys, slot_pos, d, capacity, a);
  return REWB200_OK;
}
int moe_combine_peer_launch(Ctx* c, const int* pair_slot, const float* topw, int64_t tokens, int k, int64_t d, float* out,
                            int accumulate, const A2aArgs& a) {
  RB_LAUNCH(moe_combine_peer_kernel, tokens, 256, pair_slot, topw, k, d, out, accumulate, a);
  return REWB200_OK;
}

int moe_route_slabs_launch(Ctx* c, const float* logits, int nsplit, int64_t split_stride, const float* bias, int64_t N, int E,
                           int k, float* topw, int* topi, int* zero, int n_zero) {
  RB_REQUIRE(E >= 1 && E <= 32 * MAX_E_PER_LANE, "MoE routing supports up to 256 experts");
  RB_REQUIRE(k >= 1 && k <= E, "initDeepSeekMoE: numExpertsPerTok must be in 1..numRouted");
  RB_REQUIRE(n_zero >= 0 && n_zero <= 128, "at most 128 counters can be cleared by the routing kernel");
  if (N == 0) return REWB200_OK;
  RB_CUDA(launch_k(moe_route_kernel, dim3((unsigned)((N + 3) / 4)), dim3(128), 0, c->stream, c->use_pdl, logits, nsplit,
                   split_stride, bias, N, E, k, topw, topi, zero, n_zero));
  ++g_launch_total;
  return REWB200_OK;
}
int moe_route_launch(Ctx* c, const float* logits, int64_t N, int E, int k, float* topw, int* topi) {
  return moe_route_slabs_launch(c, logits, 1, 0, nullptr, N, E, k, topw, topi, nullptr, 0);
}

// One rank owning every expert: pos[pair] = row of pair (token, j) in the expert-sorted activation matrix
// (experts ascending, pairs ascending inside an expert, so the order is the same on every run), the row
// is copied there, and block 0 writes the experts' row offsets for the grouped GEMMs.
int moe_group_local_launch(Ctx* c, const void* x, int dtype, const int* topi, int64_t tokens, int k, int64_t d, int n_experts,
                           int* offsets, void* xs, int* pair_pos) {
  if (tokens == 0) return REWB200_OK;
  RB_REQUIRE((d * dtype_size(dtype)) % 16 == 0, "MoE dispatch needs rows that are multiples of 16 bytes");
  RB_REQUIRE(n_experts <= 32 * MAX_E_PER_LANE, "MoE routing supports up to 256 experts");
  if (dtype == REWB200_BF16)
    RB_LAUNCH(moe_group_local_kernel<bf16>, tokens * k, 128, (const bf16*)x, topi, (int)(tokens * k), k, d, n_experts, offsets,
              (bf16*)xs, pair_pos);
  else
    RB_LAUNCH(moe_group_local_kernel<float>, tokens * k, 128, (const float*)x, topi, (int)(tokens * k), k, d, n_experts, offsets,
              (float*)xs, pair_pos);
  return REWB200_OK;
}

}  // namespace rewb

using namespace rewb;

extern "C" int rewb200_moe_route(const rewb200_buffer* x, const rewb200_buffer* router_w, const rewb200_buffer* router_b,
                                 int top_k, rewb200_buffer** weights, rewb200_buffer** indices) {
  RB_REQUIRE(x && router_w && weights && indices, "DeepSeekMoE.forward: NULL argument");
  RB_REQUIRE(x->ndims == 2 && router_w->ndims == 2 && x->dims[1] == router_w->dims[0],
             "DeepSeekMoE.forward: hidden [tokens, d] and gate weight [d, experts] do not agree");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t N = x->dims[0], E = router_w->dims[1];
  RB_REQUIRE(top_k >= 1 && top_k <= E, "initDeepSeekMoE: numExpertsPerTok must be in 1..numRouted");
  rewb200_buffer* logits = nullptr;
  RB_TRY(rewb200_linear(x, router_w, router_b, &logits));
  float* lf = (float*)logits->ptr;
  float* tmp = nullptr;
  int st = REWB200_OK;
  if (logits->dtype == REWB200_BF16) {
    if (cudaMallocAsync((void**)&tmp, (size_t)N * E * 4 + 256, c->stream) != cudaSuccess) st = fail("allocation failed");
    if (st == REWB200_OK) st = cast_launch(c, logits->ptr, REWB200_BF16, tmp, REWB200_F32, N * E);
    lf = tmp;
  }
  const int64_t od[2] = {N, top_k};
  if (st == REWB200_OK) st = buffer_new(c, REWB200_F32, od, 2, weights);
  if (st == REWB200_OK) st = buffer_new(c, REWB200_I32, od, 2, indices);
  if (st == REWB200_OK) st = moe_route_launch(c, lf, N, (int)E, top_k, (float*)(*weights)->ptr, (int*)(*indices)->ptr);
  if (tmp) cudaFreeAsync(tmp, c->stream);
  rewb200_buffer_release(logits);
  return st;
}
