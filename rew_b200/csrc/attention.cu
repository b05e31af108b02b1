// Grouped-query attention over a (paged or contiguous) KV cache.
//
// Restates scaledDotProductAttention (src/rew/nn/attention.nim:36-81) with the
// GQA head expansion of src/rew/nn/groupedqueryattention.nim:126-133 folded into
// indexing (query head h reads kv head h / group; nothing is materialised):
//   scores = q.k ; scores *= 1/sqrt(hd) ; + mask ; softmax(max, exp, sum, div) ; @ v
// mask_kind 0 is makeCausalMask exactly as written (attention.nim:18-34: key j is
// visible to query i iff i <= j); mask_kind 1 is the conventional causal mask
// for a query block that ends at the last key.
//
// Three kernels:
//   attn_f32_kernel      any head_dim, f32, CUDA cores (the f32 parity path)
//   attn_decode_kernel   bf16, one query token: split-KV flash-decode.  K/V tiles
//                        of 64 tokens arrive by TMA (128-byte swizzle) in a
//                        3-stage mbarrier ring; the kv head's query group forms
//                        the M rows of mma.sync tiles so each K/V byte is read
//                        once per group; softmax state lives in registers
//                        (quad shuffles), warps and splits merge by log-sum-exp.
//   attn_prefill_kernel  bf16, S > 1: flash-attention forward, 64 queries per CTA.
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tc.cuh"

namespace rewb {

extern int64_t g_launch_total;

namespace {

constexpr int TILE = 64;  // tokens per K/V tile == tokens per cache page

struct AttnDev {
  const void* q;
  int64_t q_sb, q_ss, q_sh;   // element strides of q: batch, position, head
  void* out;
  int64_t o_sb, o_ss, o_sh;
  const void* k;
  const void* v;
  const int* pos0;
  const int* block_table;
  int max_pages;
  int kvh, nh, group, S, hd;
  int64_t kv_len_fixed;
  int64_t contiguous_len;
  int causal, mask_kind;
  float scale;
  float* part_o;    // [B][nh][nsplit][hd]
  float* part_ml;   // [B][nh][nsplit][2]
  int nsplit;
  int early_kv;     // see AttnArgs::kv_tail_only
  int* tickets;     // [B][kvh] zero between launches: the last split of a (sequence, kv head) merges; nullptr: separate merge launch
  int* status;
  // Decode only (S == 1), optional: q, k and v of the new token are not read from memory but finished here from
  // the f32 split-K slabs of the q|k|v projection (sum in slab order, bias, interleaved-pair RoPE, bf16), exactly
  // as qkv_post_kernel would have done one launch earlier; the CTA whose tile range ends the sequence also writes
  // the new K / V row into the cache before it requests that tile.
  const float* f_partial;  // [f_ks][B][f_ntot]; nullptr: q comes from `q`, the cache is complete
  int f_ks;
  int64_t f_stride;
  const float* f_bias;     // [f_ntot] or nullptr
  const float* f_cos;      // [f_max_seq][hd]
  const float* f_sin;
  int f_rope_shift, f_max_seq, f_capacity, f_ntot;
};

__device__ __forceinline__ int kv_len_of(const AttnDev& a, int b) {
  return a.kv_len_fixed >= 0 ? (int)a.kv_len_fixed : a.pos0[b] + a.S;
}
__device__ __forceinline__ bool visible(const AttnDev& a, int i, int j, int ctx) {
  if (!a.causal) return true;
  return a.mask_kind == 0 ? (i <= j) : (j <= i + ctx);
}
// Row index (in units of head_dim elements) of key j of kv head h of sequence b.
__device__ __forceinline__ int64_t kv_row(const AttnDev& a, int b, int h, int j) {
  if (a.block_table) {
    const int page = a.block_table[(int64_t)b * a.max_pages + j / TILE];
    return ((int64_t)page * a.kvh + h) * TILE + j % TILE;
  }
  return ((int64_t)b * a.kvh + h) * a.contiguous_len + j;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------ f32
// One CTA per (query i, head h, sequence b).  Dynamic smem: kv_len scores +
// 128 floats of reduction space.
__global__ void __launch_bounds__(128) attn_f32_kernel(AttnDev a) {
  extern __shared__ float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kv_len = kv_len_of(a, b), ctx = kv_len - a.S;
  const int hd = a.hd, hk = h / a.group;
  float* scores = sm;
  float* red = sm + kv_len;
  const float* q = reinterpret_cast<const float*>(a.q) + b * a.q_sb + i * a.q_ss + h * a.q_sh;
  const float* K = reinterpret_cast<const float*>(a.k);
  const float* V = reinterpret_cast<const float*>(a.v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;

  for (int j = warp; j < kv_len; j += nw) {
    const float* kr = K + kv_row(a, b, hk, j) * hd;
    float d = 0.f;
    for (int e = lane; e < hd; e += 32) d += q[e] * kr[e];
    d = warp_sum(d);
    if (lane == 0) {
      float s = d * a.scale;
      if (a.causal) s = s + (visible(a, i, j, ctx) ? 0.0f : -1e9f);
      scores[j] = s;
    }
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < kv_len; j += blockDim.x) mx = fmaxf(mx, scores[j]);
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < nw; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < kv_len; j += blockDim.x) {
    const float e = expf(scores[j] - mx);
    scores[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < nw; ++w) sum += red[w];
  __syncthreads();
  for (int j = threadIdx.x; j < kv_len; j += blockDim.x) scores[j] = scores[j] / sum;
  __syncthreads();
  // attn @ v: thread (grp, d) sums keys grp, grp+ngroups, ...
  const int ngroups = max(1, (int)blockDim.x / hd);
  float* outp = reinterpret_cast<float*>(a.out) + b * a.o_sb + i * a.o_ss + h * a.o_sh;
  for (int d0 = 0; d0 < hd; d0 += blockDim.x) {
    const int d = d0 + (threadIdx.x % min(hd, (int)blockDim.x));
    const int grp = threadIdx.x / min(hd, (int)blockDim.x);
    float acc = 0.f;
    if (d < hd && grp < ngroups)
      for (int j = grp; j < kv_len; j += ngroups) acc += scores[j] * V[kv_row(a, b, hk, j) * hd + d];
    red[threadIdx.x] = acc;
    __syncthreads();
    if (grp == 0 && d < hd) {
      float t = 0.f;
      for (int g2 = 0; g2 < ngroups; ++g2) t += red[g2 * min(hd, (int)blockDim.x) + (d - d0)];
      outp[d] = t;
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ bf16 shared pieces
constexpr int ATT_STAGES = 3;

template <int HD>
struct ATile {
  static constexpr int BOXES = HD / 64;
  static constexpr int BOX_BYTES = TILE * 128;
  static constexpr int KV_BYTES = BOXES * BOX_BYTES;  // one of K or V
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int SMEM = ATT_STAGES * STAGE_BYTES + 1024 + 128;
};

// Issues the TMA loads of one 64-token K/V tile.
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* stage, uint64_t* bar, const CUtensorMap* tmK,
                                          const CUtensorMap* tmV, int64_t row0) {
  using T = ATile<HD>;
  mbar_expect_tx(bar, T::STAGE_BYTES);
#pragma unroll
  for (int bx = 0; bx < T::BOXES; ++bx) {
    tma_load_2d(stage + bx * T::BOX_BYTES, tmK, bar, bx * 64, (int)row0);
    tma_load_2d(stage + T::KV_BYTES + bx * T::BOX_BYTES, tmV, bar, bx * 64, (int)row0);
  }
}

__device__ __forceinline__ int64_t tile_row0(const AttnDev& a, int b, int hk, int tile) {
  if (a.block_table) {
    const int page = a.block_table[(int64_t)b * a.max_pages + tile];
    return ((int64_t)page * a.kvh + hk) * TILE;
  }
  return ((int64_t)b * a.kvh + hk) * a.contiguous_len + (int64_t)tile * TILE;
}

template <int HD>
__device__ __forceinline__ uint32_t kv_addr(uint32_t base, uint32_t row, uint32_t chunk) {
  return base + (chunk >> 3) * ATile<HD>::BOX_BYTES + swz128(row, chunk & 7);
}

// ------------------------------------------------------------------ bf16 decode (S == 1)
// grid (nsplit, kvh, B), 128 threads.  Warp w owns tokens 16w..16w+15 of every tile.
// Combines the split-KV partials of one (sequence, head) for output element d: log-sum-exp weights, splits in
// ascending order.  All loads of a phase are issued before the first use (up to 16 splits, fully unrolled), so a
// merge costs two L2 round trips instead of one per split; partials were written by other SMs: read through L2.
__device__ __forceinline__ float merge_splits(const float* __restrict__ part_ml, const float* __restrict__ part_o, int64_t base,
                                              int nsplit, int hd, int d) {
  float ms[16], ls[16], os[16];
#pragma unroll
  for (int sp = 0; sp < 16; ++sp) {
    const bool in = sp < nsplit;
    const float2 ml = in ? __ldcg(reinterpret_cast<const float2*>(part_ml + (base + sp) * 2)) : make_float2(-INFINITY, 0.f);
    ms[sp] = ml.x;
    ls[sp] = ml.y;
    os[sp] = in ? __ldcg(part_o + (base + sp) * hd + d) : 0.f;
  }
  float M = -INFINITY;
#pragma unroll
  for (int sp = 0; sp < 16; ++sp) M = fmaxf(M, ms[sp]);
  const float Mu = (M == -INFINITY) ? 0.f : M;
  float L = 0.f, acc = 0.f;
#pragma unroll
  for (int sp = 0; sp < 16; ++sp) {
    if (sp < nsplit) {
      const float f = __expf(ms[sp] - Mu);
      L += ls[sp] * f;
      acc += os[sp] * f;
    }
  }
  return L > 0.f ? acc / L : 0.f;
}

template <int HD>
__global__ void __launch_bounds__(128) attn_decode_kernel(const __grid_constant__ CUtensorMap tmK,
                                                          const __grid_constant__ CUtensorMap tmV, AttnDev a) {
  using T = ATile<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + ATT_STAGES * T::STAGE_BYTES);

  __shared__ uint32_t sQ[16 * (HD / 2)];  // fused q|k|v: this kv head's query group as bf16 pairs [row][HD / 2]
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3, l8 = lane & 7, lq = lane >> 3;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ATT_STAGES; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    pdl_launch_dependents();
  }
  __syncthreads();

  // Inside the engine's step, sequence lengths and block tables were written at least two kernels back
  // in the stream (every kernel of the chain waits on its predecessor before it ends), and the kernel
  // just before this one writes only the newest cache row, which lies in the last tile.  Then (early_kv)
  // every other K/V tile can be requested before griddepcontrol.wait, while that predecessor still runs.
  if (!a.early_kv) pdl_wait();
  const int kv_len = kv_len_of(a, b);
  const int ntiles = (kv_len + TILE - 1) / TILE;
  const int tps = (ntiles + a.nsplit - 1) / a.nsplit;
  const int t0 = split * tps, t1 = min(ntiles, t0 + tps);
  const int nt_local = max(0, t1 - t0);
  int early = 0;
  if (threadIdx.x == 0 && a.early_kv)
    for (; early < min(ATT_STAGES - 1, nt_local) && t0 + early < ntiles - 1; ++early)
      load_tile<HD>(smem + early * T::STAGE_BYTES, &full[early], &tmK, &tmV, tile_row0(a, b, hk, t0 + early));
  pdl_wait();

  if (a.f_partial) {
    // ---- finish q (all CTAs) and the new K / V row (the CTA that owns the sequence's last tile) from the slabs
    const int pos = kv_len - 1, rpos = pos + a.f_rope_shift;
    const bool pos_ok = pos >= 0 && pos < a.f_capacity && rpos >= 0 && rpos < a.f_max_seq;
    if (!pos_ok && threadIdx.x == 0) atomicExch(a.status, KS_BAD_INDEX);
    const float* pr = a.f_partial + (int64_t)b * a.f_ntot;
    const float* cr = a.f_cos + (int64_t)(pos_ok ? rpos : 0) * HD;
    const float* sr = a.f_sin + (int64_t)(pos_ok ? rpos : 0) * HD;
    const int nq = a.nh * HD, nkv = a.kvh * HD;
    auto pair_at = [&](int col, bool rope, int e) -> uint32_t {  // e: element index of the pair inside its head
      float v0 = 0.f, v1 = 0.f;
      for (int sp = 0; sp < a.f_ks; ++sp) {
        const float2 p2 = *reinterpret_cast<const float2*>(pr + sp * a.f_stride + col);
        v0 += p2.x;
        v1 += p2.y;
      }
      if (a.f_bias) {
        v0 += a.f_bias[col];
        v1 += a.f_bias[col + 1];
      }
      if (rope) {
        const float c0 = cr[e], s0 = sr[e];
        const float r0 = rope_even(c0, s0, v0, v1), r1 = rope_odd(c0, s0, v0, v1);
        v0 = r0;
        v1 = r1;
      }
      return pack_bf16(v0, v1);
    };
    for (int p = threadIdx.x; p < a.group * (HD / 2); p += blockDim.x) {
      const int row = p / (HD / 2), e = 2 * (p % (HD / 2));
      sQ[p] = pair_at((hk * a.group + row) * HD + e, true, e);
    }
    const bool owns_last = ntiles > 0 && t0 <= ntiles - 1 && ntiles - 1 < t1;
    if (owns_last && pos_ok) {
      const int64_t crow = kv_row(a, b, hk, pos) * HD;
      for (int p = threadIdx.x; p < HD; p += blockDim.x) {  // HD / 2 pairs of k, then HD / 2 pairs of v
        const bool is_k = p < HD / 2;
        const int e = 2 * (is_k ? p : p - HD / 2);
        const uint32_t pk = pair_at((is_k ? nq : nq + nkv) + hk * HD + e, is_k, e);
        bf16* dst = reinterpret_cast<bf16*>(const_cast<void*>(is_k ? a.k : a.v)) + crow + e;
        *reinterpret_cast<uint32_t*>(dst) = pk;
      }
      // the row is read back by the bulk tensor copy of the last tile (async proxy): order the stores before it
      __threadfence();
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    __syncthreads();
  }

  // Q fragments: rows = heads of this kv head's group (rows >= group are zero).
  uint32_t qf[HD / 16][4];
  {
    const bf16* qb = reinterpret_cast<const bf16*>(a.q) + b * a.q_sb;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = g + (r & 1) * 8;
        const int dim = kk * 16 + (r >> 1) * 8 + 2 * t;
        uint32_t v = 0;
        if (row < a.group) {
          if (a.f_partial) v = sQ[row * (HD / 2) + dim / 2];
          else v = *reinterpret_cast<const uint32_t*>(qb + (hk * a.group + row) * a.q_sh + dim);
        }
        qf[kk][r] = v;
      }
  }

  if (threadIdx.x == 0)
    for (int i = early; i < min(ATT_STAGES - 1, nt_local); ++i)
      load_tile<HD>(smem + i * T::STAGE_BYTES, &full[i], &tmK, &tmV, tile_row0(a, b, hk, t0 + i));

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int r = 0; r < 4; ++r) o[i][r] = 0.f;

  const uint32_t smem_base = smem_u32(smem);
  bool ok = true;
  for (int it = 0; it < nt_local; ++it) {
    const int s = it % ATT_STAGES;
    if (threadIdx.x == 0 && it + ATT_STAGES - 1 < nt_local) {
      const int nx = it + ATT_STAGES - 1;
      load_tile<HD>(smem + (nx % ATT_STAGES) * T::STAGE_BYTES, &full[nx % ATT_STAGES], &tmK, &tmV,
                    tile_row0(a, b, hk, t0 + nx));
    }
    ok = mbar_wait(&full[s], (it / ATT_STAGES) & 1, a.status);
    if (!ok) break;
    const uint32_t kb = smem_base + s * T::STAGE_BYTES;
    const uint32_t vb = kb + T::KV_BYTES;

    float sc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int r = 0; r < 4; ++r) sc[i][r] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
      uint32_t k0, k1, k2, k3;
      ldmatrix_x4(k0, k1, k2, k3, kv_addr<HD>(kb, warp * 16 + (lq >> 1) * 8 + l8, kk * 2 + (lq & 1)));
      mma_bf16_16816(sc[0], qf[kk], k0, k1);
      mma_bf16_16816(sc[1], qf[kk], k2, k3);
    }
    const int jbase = (t0 + it) * TILE + warp * 16;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int j = jbase + nt * 8 + 2 * t + (r & 1);
        sc[nt][r] = (j < kv_len) ? sc[nt][r] * a.scale : -INFINITY;
      }
    uint32_t pa[4];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float mx = fmaxf(fmaxf(sc[0][2 * hf], sc[0][2 * hf + 1]), fmaxf(sc[1][2 * hf], sc[1][2 * hf + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hf], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = __expf(m_run[hf] - m_use);
      const float p00 = __expf(sc[0][2 * hf] - m_use), p01 = __expf(sc[0][2 * hf + 1] - m_use);
      const float p10 = __expf(sc[1][2 * hf] - m_use), p11 = __expf(sc[1][2 * hf + 1] - m_use);
      l_run[hf] = l_run[hf] * alpha + (p00 + p01 + p10 + p11);
      m_run[hf] = m_new;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][2 * hf] *= alpha;
        o[i][2 * hf + 1] *= alpha;
      }
      pa[hf] = pack_bf16(p00, p01);
      pa[2 + hf] = pack_bf16(p10, p11);
    }
#pragma unroll
    for (int jp = 0; jp < HD / 16; ++jp) {
      uint32_t v0, v1, v2, v3;
      ldmatrix_x4_trans(v0, v1, v2, v3, kv_addr<HD>(vb, warp * 16 + (lq & 1) * 8 + l8, 2 * jp + (lq >> 1)));
      mma_bf16_16816(o[2 * jp], pa, v0, v1);
      mma_bf16_16816(o[2 * jp + 1], pa, v2, v3);
    }
    __syncthreads();  // everyone is done with stage s before it is refilled
  }
  if (!ok) return;

  // ---- merge the four warps (log-sum-exp) through shared memory
  __syncthreads();
  float* sO = reinterpret_cast<float*>(smem);             // [4][16][HD]
  float* sM = sO + 4 * 16 * HD;                           // [4][16]
  float* sL = sM + 64;                                    // [4][16]
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    float l = l_run[hf];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = g + hf * 8;
    if (t == 0) {
      sM[warp * 16 + row] = m_run[hf];
      sL[warp * 16 + row] = l;
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      float* dst = sO + ((warp * 16 + row) * HD) + i * 8 + 2 * t;
      dst[0] = o[i][2 * hf];
      dst[1] = o[i][2 * hf + 1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < a.group * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 16 + row]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = __expf(sM[w * 16 + row] - Mu);
      L += sL[w * 16 + row] * f;
      acc += sO[(w * 16 + row) * HD + d] * f;
    }
    const int head = hk * a.group + row;
    if (a.nsplit == 1) {
      bf16* op = reinterpret_cast<bf16*>(a.out) + b * a.o_sb + head * a.o_sh;
      op[d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const int64_t pi = ((int64_t)b * a.nh + head) * a.nsplit + split;
      a.part_o[pi * HD + d] = acc;
      if (d == 0) {
        a.part_ml[pi * 2] = M;
        a.part_ml[pi * 2 + 1] = L;
      }
    }
  }
  if (a.nsplit == 1 || a.tickets == nullptr) return;
  // ---- the CTA that finishes last for this (sequence, kv head) combines the splits: no second launch.
  // Every CTA publishes its partials, then takes a ticket; the last ticket holder sees all of them.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = a.tickets + (int64_t)b * a.kvh + hk;
    const int tkt = atomicAdd(tk, 1);
    s_last = (tkt == a.nsplit - 1) ? 1 : 0;
    if (s_last) *tk = 0;  // every other split has already taken its ticket: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < a.group * HD; idx += blockDim.x) {
    const int row = idx / HD, d = idx % HD;
    const int head = hk * a.group + row;
    const int64_t base = ((int64_t)b * a.nh + head) * a.nsplit;
    bf16* op = reinterpret_cast<bf16*>(a.out) + b * a.o_sb + head * a.o_sh;
    op[d] = __float2bfloat16_rn(merge_splits(a.part_ml, a.part_o, base, a.nsplit, HD, d));
  }
}

// grid (nh, B), HD threads: combine split partials.
__global__ void attn_merge_kernel(AttnDev a) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int64_t base = ((int64_t)b * a.nh + head) * a.nsplit;
  bf16* op = reinterpret_cast<bf16*>(a.out) + b * a.o_sb + head * a.o_sh;
  op[d] = __float2bfloat16_rn(merge_splits(a.part_ml, a.part_o, base, a.nsplit, a.hd, d));
}

// ------------------------------------------------------------------ bf16 prefill (S > 1)
// grid (ceil(S/64), nh, B), 128 threads; warp w owns query rows 16w..16w+15 of the block.
template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const __grid_constant__ CUtensorMap tmK,
                                                           const __grid_constant__ CUtensorMap tmV, AttnDev a) {
  using T = ATile<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + ATT_STAGES * T::STAGE_BYTES);

  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / a.group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3, l8 = lane & 7, lq = lane >> 3;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ATT_STAGES; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    pdl_launch_dependents();
  }
  __syncthreads();
  pdl_wait();

  const int kv_len = kv_len_of(a, b), ctx = kv_len - a.S;
  const int ntiles = (kv_len + TILE - 1) / TILE;
  int t_lo = 0, t_hi = ntiles;
  if (a.causal) {
    if (a.mask_kind == 0) t_lo = min(ntiles, (qb * 64) / TILE);
    else t_hi = min(ntiles, (min(a.S - 1, qb * 64 + 63) + ctx) / TILE + 1);
  }
  const int nt_local = max(0, t_hi - t_lo);

  const int i0 = qb * 64 + warp * 16;  // first query row of this warp
  uint32_t qf[HD / 16][4];
  {
    const bf16* qbase = reinterpret_cast<const bf16*>(a.q) + b * a.q_sb + h * a.q_sh;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int i = i0 + g + (r & 1) * 8;
        const int dim = kk * 16 + (r >> 1) * 8 + 2 * t;
        qf[kk][r] = (i < a.S) ? *reinterpret_cast<const uint32_t*>(qbase + i * a.q_ss + dim) : 0u;
      }
  }

  if (threadIdx.x == 0)
    for (int i = 0; i < min(ATT_STAGES - 1, nt_local); ++i)
      load_tile<HD>(smem + i * T::STAGE_BYTES, &full[i], &tmK, &tmV, tile_row0(a, b, hk, t_lo + i));

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int r = 0; r < 4; ++r) o[i][r] = 0.f;

  const uint32_t smem_base = smem_u32(smem);
  bool ok = true;
  for (int it = 0; it < nt_local; ++it) {
    const int s = it % ATT_STAGES;
    if (threadIdx.x == 0 && it + ATT_STAGES - 1 < nt_local) {
      const int nx = it + ATT_STAGES - 1;
      load_tile<HD>(smem + (nx % ATT_STAGES) * T::STAGE_BYTES, &full[nx % ATT_STAGES], &tmK, &tmV,
                    tile_row0(a, b, hk, t_lo + nx));
    }
    ok = mbar_wait(&full[s], (it / ATT_STAGES) & 1, a.status);
    if (!ok) break;
    const uint32_t kb = smem_base + s * T::STAGE_BYTES;
    const uint32_t vb = kb + T::KV_BYTES;

    float sc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int r = 0; r < 4; ++r) sc[i][r] = 0.f;
#pragma unroll
    for (int np = 0; np < 4; ++np)
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t k0, k1, k2, k3;
        ldmatrix_x4(k0, k1, k2, k3, kv_addr<HD>(kb, np * 16 + (lq >> 1) * 8 + l8, kk * 2 + (lq & 1)));
        mma_bf16_16816(sc[2 * np], qf[kk], k0, k1);
        mma_bf16_16816(sc[2 * np + 1], qf[kk], k2, k3);
      }
    const int jbase = (t_lo + it) * TILE;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int j = jbase + nt * 8 + 2 * t + (r & 1);
        const int i = i0 + g + (r >> 1) * 8;
        const bool vis = (j < kv_len) && visible(a, i, j, ctx);
        sc[nt][r] = vis ? sc[nt][r] * a.scale : -INFINITY;
      }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(sc[nt][2 * hf], sc[nt][2 * hf + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hf], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = __expf(m_run[hf] - m_use);
      float ls = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        sc[nt][2 * hf] = __expf(sc[nt][2 * hf] - m_use);
        sc[nt][2 * hf + 1] = __expf(sc[nt][2 * hf + 1] - m_use);
        ls += sc[nt][2 * hf] + sc[nt][2 * hf + 1];
      }
      l_run[hf] = l_run[hf] * alpha + ls;
      m_run[hf] = m_new;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][2 * hf] *= alpha;
        o[i][2 * hf + 1] *= alpha;
      }
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t pa[4];
      pa[0] = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
      pa[1] = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
      pa[2] = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
      pa[3] = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
      for (int jp = 0; jp < HD / 16; ++jp) {
        uint32_t v0, v1, v2, v3;
        ldmatrix_x4_trans(v0, v1, v2, v3, kv_addr<HD>(vb, ks * 16 + (lq & 1) * 8 + l8, 2 * jp + (lq >> 1)));
        mma_bf16_16816(o[2 * jp], pa, v0, v1);
        mma_bf16_16816(o[2 * jp + 1], pa, v2, v3);
      }
    }
    __syncthreads();
  }
  if (!ok) return;

#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    float l = l_run[hf];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int i = i0 + g + hf * 8;
    if (i >= a.S) continue;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    bf16* op = reinterpret_cast<bf16*>(a.out) + b * a.o_sb + i * a.o_ss + h * a.o_sh;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<uint32_t*>(op + nt * 8 + 2 * t) = pack_bf16(o[nt][2 * hf] * inv, o[nt][2 * hf + 1] * inv);
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill attention on the 5th-generation tensor core (head_dim 128, conventional causal or no mask).
// CTA = 128 queries of one head; a softmax thread owns half of query row i = TMEM lane i.
//   warp 0   TMA: K and V tiles of 128 keys (one stage each; four 64x64 boxes, 128-byte swizzle)
//   warp 1   one thread issues S = Q K^T (8 x tcgen05.mma, both operands K-major in shared memory,
//            S[128 queries][128 keys] f32 in TMEM) and O += P V (8 x tcgen05.mma, A = P read from
//            TMEM as bf16, B = V MN-major from shared memory, O[128][128] f32 in TMEM)
//   warps 2-9 online softmax in the exp2 domain, two warps per lane quarter, each on 64 of the 128 keys:
//            read the scores once into registers, exchange the half-row maxima through shared memory,
//            write P over the columns of S (after a barrier: the other half's warp may still be
//            reading them), rescale their half of O only when some row's maximum moved; at the end
//            normalise O and store bf16 rows
// 256 TMEM columns and 96 KB of shared memory per CTA: two CTAs per SM, so one CTA's softmax runs
// under the other's matrix products.  Every wait is bounded.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Named barrier of 64 threads with a literal id (a register id makes ptxas reserve all 16 barriers of the SM).
__device__ __forceinline__ void pair_sync(int id) {
  switch (id) {
    case 1: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 3: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    case 4: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    case 5: asm volatile("bar.sync 5, 64;" ::: "memory"); break;
    case 6: asm volatile("bar.sync 6, 64;" ::: "memory"); break;
    case 7: asm volatile("bar.sync 7, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 8, 64;" ::: "memory"); break;
  }
}

// Online softmax of one query tile of the tcgen05 prefill kernels, as run by one warp: lane quarter `quarter` (the 32
// tensor-memory lanes = query rows this warp may touch), keys 64 half .. +63 of every 128-key tile.  S (f32 scores)
// sits at s_addr, O (f32) at o_addr.  The two warps of a lane quarter exchange their half-row maxima through
// shared memory and meet at their own named barrier `pair_bar` (64 threads): P (bf16 pairs) overwrites the score
// columns, and half 1's P lands on columns whose scores belong to half 0, so half 0 must have read them first.
// The four quarters of a tile never wait for each other, which keeps their exp2 phases apart.
// Both kernels call this, so they return the same bits.
__device__ __forceinline__ void fa_softmax_warp(const AttnDev& a, uint32_t s_addr, uint32_t o_addr, float* xmax, float* xsum,
                                                uint64_t* s_full, uint64_t* p_full, uint64_t* o_done, int ntiles, int q0t,
                                                int ctx, int kv_len, int quarter, int half, int lane, int pair_bar, int b,
                                                int head) {
  constexpr int BKV = 128;
  const int row = quarter * 32 + lane;
  const int qi = q0t + row;
  const int qlim = a.causal ? qi + ctx : 0x7fffffff;   // last visible key
  const float sl2 = a.scale * 1.4426950408889634f;
  float m = -INFINITY, l = 0.f;   // l: this half's share of the row sum (both halves share m)
  bool ok = true;
  for (int j = 0; j < ntiles; ++j) {
    if (ok) ok = mbar_wait(s_full, j & 1, a.status);
    __syncwarp();  // the tensor-memory accesses below are warp-collective
    tc::fence_after();
    const int k0 = j * BKV + half * 64;
    // only the last tile or two of a query block contain masked keys; the test is the same for every
    // thread of the tile, so the common tile runs without a compare per element
    const bool edge = (a.causal && j * BKV + BKV - 1 > q0t + ctx) || (j * BKV + BKV > kv_len);
    uint32_t r0[32], r1[32];
    tc::ld32_issue(s_addr + half * 64, r0);
    tc::ld32_issue(s_addr + half * 64 + 32, r1);
    tc::wait_ld();
    float mraw;   // maximum of the raw scores (the scale is positive)
    if (edge) {
      mraw = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        if (k0 + e <= qlim && k0 + e < kv_len) mraw = fmaxf(mraw, __uint_as_float(r0[e]));
        if (k0 + 32 + e <= qlim && k0 + 32 + e < kv_len) mraw = fmaxf(mraw, __uint_as_float(r1[e]));
      }
    } else {
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains of three-input maxima
#pragma unroll
      for (int e = 0; e < 32; e += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = max3(mx4[u], __uint_as_float(r0[e + u]), __uint_as_float(r1[e + u]));
      }
      mraw = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    }
    float* xm = xmax + (j & 1) * 256;
    xm[half * 128 + row] = mraw;
    // after this barrier both warps of the quarter hold their scores in registers and both half maxima are visible
    pair_sync(pair_bar);
    mraw = fmaxf(mraw, xm[(half ^ 1) * 128 + row]);
    const float mx = fmaxf(m, mraw * sl2);
    const float m_use = (mx == -INFINITY) ? 0.f : mx;
    const float alpha = ex2_approx(m - m_use);   // 0 on the first tile (m = -inf)
    float ls[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t pk[32];
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const uint32_t* rr = cc ? r1 : r0;
      if (edge) {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const int key = k0 + cc * 32 + e;
          const float p0 = (key <= qlim && key < kv_len) ? ex2_approx(fmaf(__uint_as_float(rr[e]), sl2, -m_use)) : 0.f;
          const float p1 = (key + 1 <= qlim && key + 1 < kv_len) ? ex2_approx(fmaf(__uint_as_float(rr[e + 1]), sl2, -m_use)) : 0.f;
          ls[(e >> 1) & 3] += p0 + p1;
          pk[cc * 16 + (e >> 1)] = pack_bf16(p0, p1);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(rr[e]), sl2, -m_use));
          const float p1 = ex2_approx(fmaf(__uint_as_float(rr[e + 1]), sl2, -m_use));
          ls[(e >> 1) & 3] += p0 + p1;
          pk[cc * 16 + (e >> 1)] = pack_bf16(p0, p1);
        }
      }
    }
    // P (bf16 pairs): keys 64 half .. +63 -> columns 32 half .. +31 of this tile's S
    tc::st32(s_addr + half * 32, pk);
    l = l * alpha + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
    m = mx;
    // O must be rescaled when this row's maximum moved; skip the TMEM round trip when no row of the warp needs it.
    // s_full(j) was committed after P V of tile j - 1 was issued, so that product has landed in O by now.
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
      tc::ld32_issue(o_addr + half * 64, r0);
      tc::ld32_issue(o_addr + half * 64 + 32, r1);
      tc::wait_ld();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        r0[e] = __float_as_uint(__uint_as_float(r0[e]) * alpha);
        r1[e] = __float_as_uint(__uint_as_float(r1[e]) * alpha);
      }
      tc::st32_issue(o_addr + half * 64, r0);
      tc::st32_issue(o_addr + half * 64 + 32, r1);
      tc::wait_st();
    }
    tc::fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(p_full);
  }
  // ---------------- epilogue: O / l -> bf16 row (this warp's 64 of the 128 output columns)
  xsum[half * 128 + row] = l;
  pair_sync(pair_bar);
  l += xsum[(half ^ 1) * 128 + row];
  if (ntiles > 0 && ok) ok = mbar_wait(o_done, (ntiles - 1) & 1, a.status);
  __syncwarp();
  tc::fence_after();
  // tcgen05.ld is warp-collective: every lane takes part, only the rows that exist are stored
  const bool store = qi < a.S && ok;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  bf16* op = reinterpret_cast<bf16*>(a.out) + (int64_t)b * a.o_sb + (int64_t)min(qi, a.S - 1) * a.o_ss + (int64_t)head * a.o_sh +
             half * 64;
  uint32_t r[32];
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    if (ntiles > 0) {
      tc::ld32(o_addr + half * 64 + c * 32, r);
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) r[e] = 0u;
    }
    if (store) {
#pragma unroll
      for (int e = 0; e < 32; e += 8) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
        v.y = pack_bf16(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
        v.z = pack_bf16(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
        v.w = pack_bf16(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
        *reinterpret_cast<uint4*>(op + c * 32 + e) = v;
      }
    }
  }
}

namespace fa {
constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = BKV * HD * 2;            // 32 KB: [hd half][128 rows][64 elements]
constexpr int XCH = 3 * 2 * 128 * 4;                // row maxima (two buffers) and row sums exchanged by the two column halves
constexpr int SMEM = 3 * TILE_BYTES + XCH + 256 + 1024;   // Q, K, V + exchange + barriers + alignment slack
constexpr int THREADS = 10 * 32;
}  // namespace fa

__global__ void __launch_bounds__(fa::THREADS, 2) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmV, AttnDev a) {
  using namespace fa;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;
  uint8_t* sV = smem + 2 * TILE_BYTES;
  float* xmax = reinterpret_cast<float*>(smem + 3 * TILE_BYTES);   // [2 buffers][2 halves][128 rows]
  float* xsum = xmax + 2 * 2 * 128;                                 // [2 halves][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * TILE_BYTES + XCH);
  uint64_t *k_full = bars, *k_empty = bars + 1, *v_full = bars + 2, *v_empty = bars + 3, *s_full = bars + 4, *p_full = bars + 5,
           *o_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;   // the long (late) query tiles first
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh_idx = head / a.group;
  const int q0 = qt * BQ;
  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);   // the eight softmax warps
    mbar_init(o_done, 1);
    fence_barrier_init();
    pdl_launch_dependents();
  }
  if (warp == 1) tc::alloc(tmem_slot, 256);
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // q, k, v and positions come from the previous kernels

  const int kv_len = kv_len_of(a, b);
  const int ctx = kv_len - a.S;
  // keys this query tile can see: all of them, or up to its last query's position
  const int last_q = min(a.S, q0 + BQ) - 1;
  const int kv_end = a.causal ? min(kv_len, last_q + ctx + 1) : kv_len;
  const int ntiles = (kv_end + BKV - 1) / BKV;

  if (warp >= 2) {
    // stage Q: 128 rows x 256 bytes into [hd half][row][64 elements] with the 128-byte swizzle TMA would apply;
    // 256 threads, half a row each
    const int r = (threadIdx.x - 64) & 127, hh = (threadIdx.x - 64) >> 7;
    const int qi = q0 + r;
    const bf16* qp = reinterpret_cast<const bf16*>(a.q) + (int64_t)b * a.q_sb + (int64_t)min(qi, a.S - 1) * a.q_ss + (int64_t)head * a.q_sh;
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {  // eight 16-byte chunks: one 64-element half of the row
      uint4 v = make_uint4(0, 0, 0, 0);
      if (qi < a.S) v = *reinterpret_cast<const uint4*>(qp + hh * 64 + c8 * 8);
      *reinterpret_cast<uint4*>(sQ + hh * (TILE_BYTES / 2) + swz128((uint32_t)r, (uint32_t)c8)) = v;
    }
    fence_proxy_async();  // the tensor core reads these bytes through the async proxy
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        for (int kv = 0; kv < 2 && ok; ++kv) {  // K first, then V
          uint64_t* full = kv ? v_full : k_full;
          uint64_t* empty = kv ? v_empty : k_empty;
          if (j > 0 && !mbar_wait(empty, (j - 1) & 1, a.status)) {
            ok = false;
            break;
          }
          uint8_t* dst = kv ? sV : sK;
          mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int t = min(j * BKV + half * 64, kv_len - 1) & ~63;   // a half tile past the end re-reads a valid page
            const int row = (int)kv_row(a, b, kvh_idx, t);
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d(dst + c * (TILE_BYTES / 2) + half * 8192, kv ? &tmV : &tmK, full, c * 64, row);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // D f32, A/B bf16, M = 128, N = 128; QK^T: both K-major; PV: A from TMEM (K-major), B = V MN-major
      const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_pv = idesc_qk | (1u << 16);
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        ok = mbar_wait(k_full, j & 1, a.status);
        if (!ok) break;
        tc::fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // head_dim in steps of 16: two 64-element halves of four steps
          const uint32_t off = (kk >> 2) * (TILE_BYTES / 2) + (kk & 3) * 32;
          tc::umma_bf16_ss(tmem_base, tc::smem_desc(q_addr + off, 16, 1024), tc::smem_desc(k_addr + off, 16, 1024), idesc_qk,
                           kk > 0 ? 1u : 0u);
        }
        tc::commit(s_full);
        tc::commit(k_empty);
        ok = mbar_wait(p_full, j & 1, a.status) && mbar_wait(v_full, j & 1, a.status);
        if (!ok) break;
        tc::fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // keys in steps of 16 = two 8-row swizzle atoms
          tc::umma_bf16_ta(tmem_base + 128, tmem_base + kk * 8, tc::smem_desc(v_addr + kk * 2048, TILE_BYTES / 2, 1024), idesc_pv,
                           (j > 0 || kk > 0) ? 1u : 0u);
        tc::commit(o_done);
        tc::commit(v_empty);
      }
    }
  } else {
    // ---------------- softmax warps: lane quarter = warp % 4, keys 64 half .. +63 of every key tile
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    fa_softmax_warp(a, lane_addr, lane_addr + 128, xmax, xsum, s_full, p_full, o_done, ntiles, q0, ctx, kv_len, quarter, half,
                    lane, 1 + quarter, b, head);
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill attention, two query tiles per CTA ("ping-pong"): 256 queries of one head share every K / V tile.
// Tensor memory (all 512 columns, one CTA per SM): S0 | S1 | O0 | O1, 128 columns each.
//   warp 0        TMA: K and V tiles of 128 keys, two stages each
//   warp 1        one thread issues, per key tile j:  O0 += P0(j) V(j);  S0 = Q0 K(j+1)^T;  O1 += P1(j) V(j);
//                 S1 = Q1 K(j+1)^T.  While the softmax warps of tile 0 work on S0(j+1) the tensor core runs tile 1's
//                 products and the other way round, so neither the tensor pipe nor the exp unit waits for a whole
//                 QK^T -> softmax -> PV chain as in the one-tile kernel.
//   warps 2-9     softmax of query tile 0, warps 10-17 of query tile 1: the same code and the same per-row
//                 arithmetic as attn_prefill_tc_kernel (two warps per lane quarter, 64 keys each), so both kernels
//                 return the same bits.
// Under the conventional causal mask tile 0 sees one key tile fewer than tile 1.  Every wait is bounded.
namespace fa2 {
constexpr int BQ = 256, BKV = 128;
constexpr int TILE_BYTES = fa::TILE_BYTES;
constexpr int XCH = 2 * fa::XCH;                       // one exchange area per query tile
constexpr int SMEM = 6 * TILE_BYTES + XCH + 256 + 1024;   // Q0, Q1, 2 x K, 2 x V
constexpr int THREADS = 18 * 32;
}  // namespace fa2

__global__ void __launch_bounds__(fa2::THREADS, 1) attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                        const __grid_constant__ CUtensorMap tmV, AttnDev a) {
  using namespace fa2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // [2 query tiles]
  uint8_t* sK = smem + 2 * TILE_BYTES;      // [2 stages]
  uint8_t* sV = smem + 4 * TILE_BYTES;      // [2 stages]
  float* xch = reinterpret_cast<float*>(smem + 6 * TILE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES + XCH);
  uint64_t *k_full = bars, *k_empty = bars + 2, *v_full = bars + 4, *v_empty = bars + 6, *s_full = bars + 8, *p_full = bars + 10,
           *o_done = bars + 12;   // two of each: ring stage for K / V, query tile for S / P / O
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;   // the long (late) query tiles first
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh_idx = head / a.group;
  const int q0 = qt * BQ;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
      mbar_init(s_full + i, 1);
      mbar_init(p_full + i, 8);   // the eight softmax warps of a query tile
      mbar_init(o_done + i, 1);
    }
    fence_barrier_init();
    pdl_launch_dependents();
  }
  if (warp == 1) tc::alloc(tmem_slot, 512);
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // q, k, v and positions come from the previous kernels

  const int kv_len = kv_len_of(a, b);
  const int ctx = kv_len - a.S;
  // key tiles each query tile can see: all of them, or up to its last query's position; none for a tile past S
  int nt[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int first = q0 + t * 128;
    const int last_q = min(a.S, first + 128) - 1;
    const int kv_end = a.causal ? min(kv_len, last_q + ctx + 1) : kv_len;
    nt[t] = first < a.S ? (kv_end + BKV - 1) / BKV : 0;
  }
  const int nt_max = max(nt[0], nt[1]);

  if (warp >= 2) {
    // stage Q: 2 x 128 rows x 256 bytes into [tile][hd half][row][64 elements] with the 128-byte swizzle TMA would
    // apply; 512 threads, half a row each
    const int idx = threadIdx.x - 64;
    const int r = idx & 127, hh = (idx >> 7) & 1, t = idx >> 8;
    const int qi = q0 + t * 128 + r;
    const bf16* qp = reinterpret_cast<const bf16*>(a.q) + (int64_t)b * a.q_sb + (int64_t)min(qi, a.S - 1) * a.q_ss + (int64_t)head * a.q_sh;
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (qi < a.S) v = *reinterpret_cast<const uint4*>(qp + hh * 64 + c8 * 8);
      *reinterpret_cast<uint4*>(sQ + t * TILE_BYTES + hh * (TILE_BYTES / 2) + swz128((uint32_t)r, (uint32_t)c8)) = v;
    }
    fence_proxy_async();  // the tensor core reads these bytes through the async proxy
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      bool ok = true;
      for (int j = 0; j < nt_max && ok; ++j) {
        const int st = j & 1;
        for (int kv = 0; kv < 2 && ok; ++kv) {  // K first, then V
          uint64_t* full = (kv ? v_full : k_full) + st;
          uint64_t* empty = (kv ? v_empty : k_empty) + st;
          if (j >= 2 && !mbar_wait(empty, ((j >> 1) - 1) & 1, a.status)) {
            ok = false;
            break;
          }
          uint8_t* dst = (kv ? sV : sK) + st * TILE_BYTES;
          mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int tk = min(j * BKV + half * 64, kv_len - 1) & ~63;   // a half tile past the end re-reads a valid page
            const int row = (int)kv_row(a, b, kvh_idx, tk);
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d(dst + c * (TILE_BYTES / 2) + half * 8192, kv ? &tmV : &tmK, full, c * 64, row);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_pv = idesc_qk | (1u << 16);
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = true;
      // S_t = Q_t K(j)^T into columns t * 128
      // descriptor words once; inside the loops an operand moves by one 32-bit add
      constexpr uint32_t hi = tc::desc_hi(1024);
      const uint32_t q_lo = tc::desc_lo(q_addr, 16), k_lo = tc::desc_lo(k_addr, 16), v_lo = tc::desc_lo(v_addr, TILE_BYTES / 2);
      auto issue_qk = [&](int t, int j) {
        const uint32_t qa = q_lo + t * (TILE_BYTES >> 4), ka = k_lo + (j & 1) * (TILE_BYTES >> 4);
        const uint32_t d = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // head_dim in steps of 16: two 64-element halves of four steps
          constexpr uint32_t half_step = (TILE_BYTES / 2) >> 4;
          const uint32_t off = (kk >> 2) * half_step + (kk & 3) * 2;
          tc::umma_bf16_ss_lh(d, qa + off, ka + off, hi, idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc::commit(s_full + t);
      };
      if (nt_max > 0) {
        ok = mbar_wait(k_full, 0, a.status);
        if (ok) {
          tc::fence_after();
          for (int t = 0; t < 2; ++t)
            if (nt[t] > 0) issue_qk(t, 0);
          tc::commit(k_empty);
        }
      }
      for (int j = 0; j < nt_max && ok; ++j) {
        const int st = j & 1, ph = (j >> 1) & 1;
        bool v_ready = false, k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < nt[t]) {
            ok = mbar_wait(p_full + t, j & 1, a.status);
            if (ok && !v_ready) ok = v_ready = mbar_wait(v_full + st, ph, a.status);
            if (!ok) break;
            tc::fence_after();
            const uint32_t va = v_lo + st * (TILE_BYTES >> 4);
            const uint32_t pa = tmem_base + t * 128, od = tmem_base + 256 + t * 128;
            const uint32_t acc0 = j > 0 ? 1u : 0u;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // keys in steps of 16 = two 8-row swizzle atoms
              tc::umma_bf16_ta_lh(od, pa + kk * 8, va + kk * (2048 >> 4), hi, idesc_pv, kk > 0 ? 1u : acc0);
            tc::commit(o_done + t);
          }
          if (j + 1 < nt[t]) {
            if (!k_ready) ok = k_ready = mbar_wait(k_full + ((j + 1) & 1), ((j + 1) >> 1) & 1, a.status);
            if (!ok) break;
            tc::fence_after();
            issue_qk(t, j + 1);
          }
        }
        if (!ok) break;
        tc::commit(v_empty + st);
        if (j + 1 < nt_max) tc::commit(k_empty + ((j + 1) & 1));
      }
    }
  } else {
    // ---------------- softmax warps: query tile t, lane quarter = warp % 4, keys 64 half .. +63 of every key tile
    const int t = (warp - 2) >> 3;
    const int quarter = warp & 3, half = ((warp - 2) >> 2) & 1;
    const uint32_t s_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + t * 128;
    const uint32_t o_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + 256 + t * 128;
    float* xmax = xch + t * (fa::XCH / 4);      // [2 buffers][2 halves][128 rows]
    float* xsum = xmax + 2 * 2 * 128;           // [2 halves][128 rows]
    fa_softmax_warp(a, s_addr, o_addr, xmax, xsum, s_full + t, p_full + t, o_done + t, nt[t], q0 + t * 128, ctx, kv_len, quarter,
                    half, lane, 1 + t * 4 + quarter, b, head);
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem_base, 512);
  }
}

}  // namespace

int decode_splits(Ctx* c, int64_t B, int kvh) {
  if (const char* e = getenv("REW_B200_ATTN_SPLITS")) {  // tuning override
    const int v = atoi(e);
    if (v >= 1 && v <= 16) return v;
  }
  const int64_t base = B * kvh;
  if (base >= c->sm_count) return 1;
  // two CTAs fit an SM: fill those slots once (rounding up would leave a short second wave)
  const int64_t s = std::max<int64_t>(1, 2 * c->sm_count / base);
  return (int)std::min<int64_t>(s, 16);
}



size_t attn_scratch_bytes(int64_t B, int nh, int hd, int max_splits) {
  return (size_t)B * nh * max_splits * (hd + 2) * sizeof(float);
}

int attn_launch(Ctx* c, const AttnArgs& h) {
  if (h.B == 0 || h.S == 0) return REWB200_OK;
  AttnDev a;
  a.q = h.q; a.q_sb = h.q_sb; a.q_ss = h.q_ss; a.q_sh = h.q_sh;
  a.out = h.out; a.o_sb = h.o_sb; a.o_ss = h.o_ss; a.o_sh = h.o_sh;
  a.k = h.kv.k; a.v = h.kv.v;
  a.pos0 = h.pos0;
  a.block_table = h.kv.block_table;
  a.max_pages = h.kv.max_pages;
  a.kvh = h.kv.kvh; a.nh = h.nh; a.group = h.nh / h.kv.kvh; a.S = h.S; a.hd = h.kv.hd;
  a.kv_len_fixed = h.kv_len_fixed;
  a.contiguous_len = h.kv.contiguous_len;
  a.causal = h.causal; a.mask_kind = h.mask_kind;
  a.scale = h.scale != 0.f ? h.scale : 1.0f / sqrtf((float)h.kv.hd);
  a.part_o = nullptr; a.part_ml = nullptr; a.nsplit = 1;
  a.early_kv = (h.kv_tail_only && h.S == 1) ? 1 : 0;
  a.tickets = nullptr;
  a.status = c->d_status;
  a.f_partial = nullptr;
  a.f_ks = 0; a.f_stride = 0; a.f_bias = nullptr; a.f_cos = nullptr; a.f_sin = nullptr;
  a.f_rope_shift = 0; a.f_max_seq = 0; a.f_capacity = 0; a.f_ntot = 0;
  if (h.fuse_qkv) {
    const QkvPostArgs& f = *h.fuse_qkv;
    RB_REQUIRE(h.S == 1 && h.dtype == REWB200_BF16 && h.pos0 != nullptr && f.hd == h.kv.hd && f.kvh == h.kv.kvh && f.nh == h.nh &&
                   f.hd % 2 == 0 && h.nh / h.kv.kvh <= 16,
               "fused q|k|v needs a bf16 decode step with per-sequence positions");
    a.f_partial = f.partial; a.f_ks = f.nsplit; a.f_stride = f.split_stride; a.f_bias = f.bias;
    a.f_cos = f.cosT; a.f_sin = f.sinT; a.f_rope_shift = f.rope_shift; a.f_max_seq = f.max_seq; a.f_capacity = f.kv_capacity;
    a.f_ntot = (f.nh + 2 * f.kvh) * f.hd;
  }
  RB_REQUIRE(h.nh % h.kv.kvh == 0, "numHeads must be divisible by numKVHeads");
  RB_REQUIRE(h.pos0 != nullptr || h.kv_len_fixed >= 0, "attention needs per-sequence positions or a fixed key length");
  RB_REQUIRE(!h.kv.block_table || h.kv.page == TILE, "paged KV cache must use 64-token pages");

  if (h.dtype == REWB200_F32) {
    RB_REQUIRE(h.max_kv_len > 0, "f32 attention needs the maximum key length");
    const size_t smem = ((size_t)h.max_kv_len + 128 + 32) * sizeof(float);
    RB_REQUIRE(smem <= 200 * 1024, "f32 attention supports at most ~50k keys per sequence");
    RB_REQUIRE(a.hd <= 128 || a.hd % 128 == 0, "f32 attention: head_dim above 128 must be a multiple of 128");
    static size_t cur = 48 * 1024;
    if (smem > cur) {
      RB_CUDA(cudaFuncSetAttribute(attn_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      cur = smem;
    }
    RB_CUDA(launch_k(attn_f32_kernel, dim3((unsigned)h.S, (unsigned)h.nh, (unsigned)h.B), dim3(128), smem, c->stream,
                     c->use_pdl, a));
    ++g_launch_total;
    return REWB200_OK;
  }
  RB_REQUIRE(h.dtype == REWB200_BF16, "attention supports f32 and bf16");
  RB_REQUIRE(a.hd == 128 || a.hd == 64, "bf16 attention supports head_dim 64 and 128, got " + std::to_string(a.hd));
  RB_REQUIRE(h.q_sh % 2 == 0 && h.q_sb % 2 == 0 && h.q_ss % 2 == 0, "bf16 attention: q strides must be even");
  RB_REQUIRE(h.tmK != nullptr && h.tmV != nullptr, "bf16 attention needs K/V tensor maps");
  static bool attrs = false;
  if (!attrs) {
    RB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATile<128>::SMEM));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATile<64>::SMEM));
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATile<128>::SMEM));
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATile<64>::SMEM));
    attrs = true;
  }
  if (h.S == 1) {
    RB_REQUIRE(a.group <= 16, "bf16 decode attention supports query groups of at most 16 heads");
    int nsplit = decode_splits(c, h.B, a.kvh);
    if (nsplit > 1) {
      const size_t need = attn_scratch_bytes(h.B, h.nh, a.hd, nsplit);
      RB_REQUIRE(h.scratch != nullptr && h.scratch_bytes >= need, "attention scratch too small for split-KV decode");
      a.part_o = h.scratch;
      a.part_ml = h.scratch + (size_t)h.B * h.nh * nsplit * a.hd;
    }
    a.nsplit = nsplit;
    a.tickets = (nsplit > 1 && c->attn_fused_merge && h.B * a.kvh <= Ctx::kTickets) ? c->d_tickets : nullptr;
    dim3 grid((unsigned)nsplit, (unsigned)a.kvh, (unsigned)h.B);
    if (a.hd == 128)
      RB_CUDA(launch_k(attn_decode_kernel<128>, grid, dim3(128), (size_t)ATile<128>::SMEM, c->stream, c->use_pdl, *h.tmK, *h.tmV, a));
    else
      RB_CUDA(launch_k(attn_decode_kernel<64>, grid, dim3(128), (size_t)ATile<64>::SMEM, c->stream, c->use_pdl, *h.tmK, *h.tmV, a));
    ++g_launch_total;
    if (nsplit > 1 && a.tickets == nullptr) {
      RB_CUDA(launch_k(attn_merge_kernel, dim3((unsigned)h.nh, (unsigned)h.B), dim3((unsigned)a.hd), 0, c->stream, c->use_pdl, a));
      ++g_launch_total;
    }
    return REWB200_OK;
  }
  if (c->attn_tc && a.hd == 128 && h.S >= 128 && (!a.causal || a.mask_kind == 1) && h.q_ss % 8 == 0 && h.q_sh % 8 == 0 &&
      h.q_sb % 8 == 0 && h.o_ss % 8 == 0 && h.o_sh % 8 == 0 && h.o_sb % 8 == 0) {
    static bool tc_attr = false;
    if (!tc_attr) {
      RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::SMEM));
      RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
      tc_attr = true;
    }
    // two query tiles per CTA pay from about 4096 query rows (a K / V tile then serves 256 rows and the L2 -> SM
    // traffic halves); below that the one-tile kernel with two CTAs per SM hides its prologue and tail better
    if (c->attn_pingpong && h.S >= c->attn_pingpong_min_rows) {
      static bool tc2_attr = false;
      if (!tc2_attr) {
        RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa2::SMEM));
        tc2_attr = true;
      }
      dim3 pgrid((unsigned)((h.S + fa2::BQ - 1) / fa2::BQ), (unsigned)h.nh, (unsigned)h.B);
      RB_CUDA(launch_k(attn_prefill_tc2_kernel, pgrid, dim3(fa2::THREADS), (size_t)fa2::SMEM, c->stream, c->use_pdl, *h.tmK, *h.tmV, a));
      ++g_launch_total;
      return REWB200_OK;
    }
    dim3 tgrid((unsigned)((h.S + fa::BQ - 1) / fa::BQ), (unsigned)h.nh, (unsigned)h.B);
    RB_CUDA(launch_k(attn_prefill_tc_kernel, tgrid, dim3(fa::THREADS), (size_t)fa::SMEM, c->stream, c->use_pdl, *h.tmK, *h.tmV, a));
    ++g_launch_total;
    return REWB200_OK;
  }
  dim3 grid((unsigned)((h.S + 63) / 64), (unsigned)h.nh, (unsigned)h.B);
  if (a.hd == 128)
    RB_CUDA(launch_k(attn_prefill_kernel<128>, grid, dim3(128), (size_t)ATile<128>::SMEM, c->stream, c->use_pdl, *h.tmK, *h.tmV, a));
  else
    RB_CUDA(launch_k(attn_prefill_kernel<64>, grid, dim3(128), (size_t)ATile<64>::SMEM, c->stream, c->use_pdl, *h.tmK, *h.tmV, a));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace rewb
