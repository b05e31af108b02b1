// bf16 Linear on the 5th-generation tensor cores (tcgen05.mma, accumulator in
// tensor memory): y[M,N] = x[M,K] @ W[K,N] (+ b), src/rew/nn/linear.nim:43-49.
//
// Operand roles follow the reference's weight layout.  W is [in,out] row-major,
// i.e. `out` is contiguous, which is an MN-major UMMA operand: W is the A
// operand (UMMA M = 128 output features per CTA), the activations x[token][k]
// (k contiguous, K-major) are the B operand (UMMA N = TN tokens).  The f32
// accumulator D[feature][token] lives in TMEM: lane = output feature, column =
// token.
//
// Roles inside the CTA (192 threads):
//   warp 0   TMA producer: cp.async.bulk.tensor boxes of W (64 k x 64 features,
//            two per stage) and x (64 k x TN tokens), 128-byte swizzle, into a
//            multi-stage mbarrier ring; W loads are issued before
//            griddepcontrol.wait so the ramp overlaps the previous kernel.
//   warp 1   allocates TMEM, then one elected thread issues four
//            tcgen05.mma.kind::f16 (K = 16 each) per stage from shared-memory
//            descriptors and releases the stage with tcgen05.commit.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp owns 32 lanes),
//            apply bias / SwiGLU, store.
// All waits are bounded; on a timeout the roles fall through to the common
// exit, where TMEM is released.
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tc.cuh"

namespace rewb {
namespace {

constexpr int BM = 128;  // output features per CTA
constexpr int BK = 64;
constexpr int A_BYTES = 2 * BK * 64 * 2;  // two 64x64 boxes

template <int TN>
struct TcCfg {
  // 32 tokens: 5 x 20 KB, 64: 4 x 24 KB, 128: 3 x 32 KB, so that two CTAs share an SM (these tiles serve steps
  // with a single token tile, where a launch has only as many CTAs as feature tiles x splits); 256: 4 x 48 KB
  static constexpr int STAGES = TN <= 32 ? 5 : (TN <= 64 ? 4 : (TN <= 128 ? 3 : 4));
  static constexpr int B_BYTES = TN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = TN < 32 ? 32 : TN;
};

struct TcArgs {
  int64_t M, N, K;
  int kb_per_split;
  int epi;
  void* out;
  int64_t ldo;
  int64_t split_stride;
  const float* bias;
  int* status;
  const int* row_offsets;  // grouped launches (persistent kernel): rows of group g = [row_offsets[g], row_offsets[g+1])
  int groups;
  int fuse_qkv;       // cluster kernel: finish q|k|v in the epilogue (bias, RoPE, cache write) instead of one f32 slab
  QkvPostArgs qp;     // what qkv_post_kernel would have been given (partial / nsplit unused)
};

// ---- thread-block cluster pieces of the split-K kernel
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t saddr, uint32_t rank) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(saddr), "r"(rank));
  return ra;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
  return v;
}

__device__ __forceinline__ float silu_f(float x) { return x * (1.0f / (1.0f + __expf(-x))); }

// Second half of the cluster split-K epilogue, run by the four epilogue warps of every CTA after the
// cluster barrier: this CTA finishes tokens [rank * 32/KS, (rank+1) * 32/KS) of the tile.  All loads of
// the peers' tiles are issued before the first add, and the sum runs in split order, so the result
// equals what the slab consumer kernels compute.
template <int KS>
__device__ __forceinline__ void cluster_finish(const TcArgs& a, uint8_t* smem, int q, int lane, int col0, int row0,
                                               bool epi_ok) {
  constexpr int TPR = 32 / KS;  // tokens this CTA finishes
  const uint32_t cr = cluster_ctarank();
  const int64_t feat = (int64_t)col0 + q * 32 + lane;
  const bool feat_ok = feat < a.N;
  const int j0 = (int)cr * TPR;
  const uint32_t soff = smem_u32(smem) + (uint32_t)(j0 * BM + q * 32 + lane) * 4u;
  float v[TPR];
  {
    float t[KS][TPR];
#pragma unroll
    for (int rr = 0; rr < KS; ++rr) {
      const uint32_t ra = dsmem_addr(soff, (uint32_t)rr);
#pragma unroll
      for (int jj = 0; jj < TPR; ++jj) t[rr][jj] = ld_dsmem_f32(ra + (uint32_t)jj * (BM * 4u));
    }
#pragma unroll
    for (int jj = 0; jj < TPR; ++jj) {
      v[jj] = 0.f;
#pragma unroll
      for (int rr = 0; rr < KS; ++rr) v[jj] += t[rr][jj];  // split order
    }
  }
  if (!a.fuse_qkv) {
    if (feat_ok && epi_ok) {
#pragma unroll
      for (int jj = 0; jj < TPR; ++jj) {
        const int64_t grow = (int64_t)row0 + j0 + jj;
        if (grow < a.M) reinterpret_cast<float*>(a.out)[grow * a.ldo + feat] = v[jj];
      }
    }
    return;
  }
  // ---- q|k|v: bias, RoPE on interleaved pairs, q to its buffer, k / v into the cache.
  // Lane t < TPR looks up token t's position and cache row once; everyone reads them by shuffle.
  const QkvPostArgs& p = a.qp;
  const int hd = p.hd, nq = p.nh * hd, nkv = p.kvh * hd;
  int m_rpos = -1;          // RoPE table row, -1: row outside the launch or a bad index
  long long m_crb = 0;      // cache row of kv head 0
  const int64_t head_stride = p.kv.block_table ? p.kv.page : p.kv.contiguous_len;
  if (lane < TPR) {
    const int64_t grow = (int64_t)row0 + j0 + lane;
    if (grow < a.M) {
      const int b = (int)(grow / p.S), sidx = (int)(grow % p.S);
      const int pos = p.pos0[b] + sidx, rpos = pos + p.rope_shift;
      if (pos < 0 || pos >= p.kv_capacity || rpos < 0 || rpos >= p.max_seq) {
        atomicExch(p.status, KS_BAD_INDEX);
      } else {
        m_rpos = rpos;
        if (p.kv.block_table) {
          const int page = p.kv.block_table[(int64_t)b * p.kv.max_pages + pos / p.kv.page];
          m_crb = ((long long)page * p.kvh) * p.kv.page + pos % p.kv.page;
        } else {
          m_crb = ((long long)b * p.kvh) * p.kv.contiguous_len + pos;
        }
      }
    }
  }
  const int col = (int)feat;
  const bool rot = col < nq + nkv;
  const int e = rot ? col % hd : (col - nq - nkv) % hd;
  const int hkv = col < nq ? 0 : (rot ? (col - nq) / hd : (col - nq - nkv) / hd);
  const float bias_v = (p.bias && feat_ok) ? p.bias[feat] : 0.f;
  int rpos[TPR];
  long long crb[TPR];
  float cs[TPR], sn[TPR];
#pragma unroll
  for (int jj = 0; jj < TPR; ++jj) {
    rpos[jj] = __shfl_sync(0xffffffffu, m_rpos, jj);
    crb[jj] = __shfl_sync(0xffffffffu, m_crb, jj);
  }
#pragma unroll
  for (int jj = 0; jj < TPR; ++jj) {
    cs[jj] = 1.f;
    sn[jj] = 0.f;
    if (rot && feat_ok && rpos[jj] >= 0) {
      cs[jj] = p.cosT[(int64_t)rpos[jj] * hd + e];
      sn[jj] = p.sinT[(int64_t)rpos[jj] * hd + e];
    }
  }
#pragma unroll
  for (int jj = 0; jj < TPR; ++jj) {
    const float x = v[jj] + bias_v;
    const float pr = __shfl_xor_sync(0xffffffffu, x, 1);  // the other element of the pair
    if (!feat_ok || !epi_ok || rpos[jj] < 0) continue;
    const int64_t grow = (int64_t)row0 + j0 + jj;
    if (rot) {
      const float r = (e & 1) ? rope_odd(cs[jj], sn[jj], pr, x) : rope_even(cs[jj], sn[jj], x, pr);
      if (col < nq)
        reinterpret_cast<bf16*>(p.q_out)[grow * nq + col] = __float2bfloat16_rn(r);
      else
        reinterpret_cast<bf16*>(p.kv.k)[(crb[jj] + hkv * head_stride) * hd + e] = __float2bfloat16_rn(r);
    } else {
      reinterpret_cast<bf16*>(p.kv.v)[(crb[jj] + hkv * head_stride) * hd + e] = __float2bfloat16_rn(x);
    }
  }
}

// CL = 1 (decode tile only): the CTAs of one feature tile that split K form a thread-block cluster
// along z and sum their accumulators through distributed shared memory, each finishing 32 / ksplit
// of the tile's tokens, so the launch leaves one finished slab (or finished q / k / v) instead of
// ksplit partial slabs for the next kernel to add up.
template <int TN, int CL>
__global__ void __launch_bounds__(192) linear_tc_kernel(const __grid_constant__ CUtensorMap tmW,
                                                         const __grid_constant__ CUtensorMap tmX, TcArgs a) {
  static_assert(CL == 0 || TN == 32, "the cluster reduction is written for the decode tile");
  using C = TcCfg<TN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tmem_full = empty + C::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Tile order: with several token tiles the CTAs walk groups of 8 token tiles per feature tile,
  // so a wave touches ~8 x-tiles and ~18 W-tiles instead of one x-tile and every W-tile; without
  // this a weight matrix larger than L2 is re-streamed from HBM once per token tile.
  int tile_n = blockIdx.x, tile_m = blockIdx.y;
  if (gridDim.y > 1) {
    constexpr int GROUP_M = 8;
    const int lin = blockIdx.x + gridDim.x * blockIdx.y;
    const int per_group = GROUP_M * gridDim.x;
    const int group = lin / per_group;
    const int first_m = group * GROUP_M;
    const int group_rows = min(GROUP_M, (int)gridDim.y - first_m);
    const int in_group = lin - group * per_group;
    tile_m = first_m + in_group % group_rows;
    tile_n = in_group / group_rows;
  }
  const int col0 = tile_n * BM;              // first output feature of the tile
  const int row0 = tile_m * TN;              // first token of the tile
  const int split = blockIdx.z;
  const int rows_valid = (int)min((int64_t)TN, a.M - row0);
  const int nkb_total = (int)((a.K + BK - 1) / BK);
  const int kb0 = split * a.kb_per_split;
  const int nkb = max(0, min(a.kb_per_split, nkb_total - kb0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    fence_barrier_init();
    pdl_launch_dependents();
  }
  if (warp == 1) {
    tc::alloc(tmem_slot, (uint32_t)C::TMEM_COLS);
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool epi_ok = true;
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      const int pre = min(C::STAGES, nkb);
      for (int kb = 0; kb < pre; ++kb) {
        uint8_t* st = smem + kb * C::STAGE_BYTES;
        mbar_expect_tx(&full[kb], C::STAGE_BYTES);
        const int k = (kb0 + kb) * BK;
        tma_load_2d_hint(st, &tmW, &full[kb], col0, k, pol_w);
        tma_load_2d_hint(st + A_BYTES / 2, &tmW, &full[kb], col0 + 64, k, pol_w);
      }
      pdl_wait();
      for (int kb = 0; kb < pre; ++kb)
        tma_load_2d_hint(smem + kb * C::STAGE_BYTES + A_BYTES, &tmX, &full[kb], (kb0 + kb) * BK, row0, pol_x);
      for (int kb = pre; kb < nkb; ++kb) {
        const int s = kb % C::STAGES;
        if (!mbar_wait(&empty[s], ((kb / C::STAGES) - 1) & 1, a.status)) break;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        const int k = (kb0 + kb) * BK;
        tma_load_2d_hint(st, &tmW, &full[s], col0, k, pol_w);
        tma_load_2d_hint(st + A_BYTES / 2, &tmW, &full[s], col0 + 64, k, pol_w);
        tma_load_2d_hint(st + A_BYTES, &tmX, &full[s], k, row0, pol_x);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
      // instruction descriptor: D f32, A/B bf16, A MN-major, B K-major, N = TN, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(TN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      const uint32_t smem_base = smem_u32(smem);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % C::STAGES;
        ok = mbar_wait(&full[s], (kb / C::STAGES) & 1, a.status);
        if (!ok) break;
        tc::fence_after();
        const uint32_t sa = smem_base + s * C::STAGE_BYTES;
        const uint32_t sb = sa + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          // A: 16 k-rows of 128 bytes = two 8-row swizzle atoms 1024 B apart (SBO); the second
          //    64-feature box is 8192 B further (LBO).  B: rows of 128 B, 8-row atoms 1024 B apart.
          const uint64_t da = tc::smem_desc(sa + kk * 2048, A_BYTES / 2, 1024);
          const uint64_t db = tc::smem_desc(sb + kk * 32, 16, 1024);
          tc::umma_bf16_ss(tmem_base, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
        }
        tc::commit(&empty[s]);  // stage is free once these MMAs have read it
      }
      if (ok) tc::commit(tmem_full);
    }
  } else {
    // ---------------- epilogue warps 2..5; TMEM lanes 32*(warp%4) .. +31
    // The accumulator is D[feature][token]; the output is [token][feature].  Each thread owns one
    // feature, so the tile is transposed through shared memory (the pipeline stages are free once
    // tmem_full fires) and then written with 16-byte, fully coalesced stores.
    const int q = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
    bool ok = true;
    if (nkb > 0) {
      ok = mbar_wait(tmem_full, 0, a.status);
      tc::fence_after();
    }
    pdl_wait();
    if constexpr (CL == 1) {
      // own partial tile -> shared memory as [token][feature] f32 (the pipeline stages are free by now)
      uint32_t r[32];
      ok = __all_sync(0xffffffffu, ok);  // the tensor-memory load below is warp-collective
      if (ok && nkb > 0) {
        tc::ld32(tmem_base + ((uint32_t)(q * 32) << 16), r);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      float* stg = reinterpret_cast<float*>(smem);
#pragma unroll
      for (int j = 0; j < 32; ++j) stg[j * BM + q * 32 + lane] = __uint_as_float(r[j]);
      epi_ok = ok;
    } else if constexpr (TN == 32) {
      // decode-size tile: the output is a few KB, direct stores (32 lanes = 32 consecutive features)
      if (ok) {
        const int64_t feat = (int64_t)col0 + q * 32 + lane;
        const bool feat_ok = feat < a.N;
        const float bias_v = (a.bias && feat_ok && a.epi != EPI_PARTIAL_F32) ? a.bias[feat] : 0.f;
        uint32_t r[32];
        if (nkb > 0) {
          tc::ld32(tmem_base + ((uint32_t)(q * 32) << 16), r);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (a.epi == EPI_SWIGLU_BF16) {
          const bool is_gate = (lane & 15) < 8;
          const int64_t oc = ((int64_t)col0 + q * 32) / 2 + (lane >> 4) * 8 + (lane & 7);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = __uint_as_float(r[j]) + bias_v;
            const float up = __shfl_down_sync(0xffffffffu, v, 8);
            if (is_gate && feat_ok && j < rows_valid)
              reinterpret_cast<bf16*>(a.out)[(int64_t)(row0 + j) * a.ldo + oc] = __float2bfloat16_rn(silu_f(v) * up);
          }
        } else if (feat_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j >= rows_valid) break;
            const float v = __uint_as_float(r[j]) + bias_v;
            const int64_t grow = row0 + j;
            if (a.epi == EPI_PARTIAL_F32)
              reinterpret_cast<float*>(a.out)[split * a.split_stride + grow * a.ldo + feat] = v;
            else if (a.epi == EPI_BIAS_F32)
              reinterpret_cast<float*>(a.out)[grow * a.ldo + feat] = v;
            else
              reinterpret_cast<bf16*>(a.out)[grow * a.ldo + feat] = __float2bfloat16_rn(v);
          }
        }
      }
    } else {
      const bool swiglu = a.epi == EPI_SWIGLU_BF16;
      const bool out_f32 = a.epi == EPI_PARTIAL_F32 || a.epi == EPI_BIAS_F32;
      const int tile_cols = swiglu ? 64 : 128;
      const int row_bytes = tile_cols * (out_f32 ? 4 : 2);
      uint8_t* stg = smem;
      if (ok) {
        const int64_t feat = (int64_t)col0 + q * 32 + lane;
        const bool feat_ok = feat < a.N;
        const float bias_v = (a.bias && feat_ok && a.epi != EPI_PARTIAL_F32) ? a.bias[feat] : 0.f;
        // gate features sit in lanes with (lane % 16) < 8, their up partners 8 lanes higher
        const bool is_gate = (lane & 15) < 8;
        const int hcol = q * 16 + (lane >> 4) * 8 + (lane & 7);
  #pragma unroll 1
        for (int c0 = 0; c0 < TN; c0 += 32) {
          if (c0 >= rows_valid) break;
          uint32_t r[32];
          if (nkb > 0) {
            tc::ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
          } else {
  #pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (swiglu) {
  #pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float v = __uint_as_float(r[j]) + bias_v;
              const float up = __shfl_down_sync(0xffffffffu, v, 8);
              if (is_gate) reinterpret_cast<bf16*>(stg + (c0 + j) * row_bytes)[hcol] = __float2bfloat16_rn(silu_f(v) * up);
            }
          } else if (out_f32) {
  #pragma unroll
            for (int j = 0; j < 32; ++j)
              reinterpret_cast<float*>(stg + (c0 + j) * row_bytes)[q * 32 + lane] = __uint_as_float(r[j]) + bias_v;
          } else {
  #pragma unroll
            for (int j = 0; j < 32; ++j)
              reinterpret_cast<bf16*>(stg + (c0 + j) * row_bytes)[q * 32 + lane] = __float2bfloat16_rn(__uint_as_float(r[j]) + bias_v);
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
      if (ok) {
        const int chunks_per_row = row_bytes / 16;           // 32 (f32), 16 (bf16), 8 (SwiGLU)
        const int elems_per_chunk = out_f32 ? 4 : 8;
        const int64_t out_col0 = swiglu ? col0 / 2 : col0;
        const int64_t out_cols = swiglu ? a.N / 2 : a.N;
        const size_t esz = out_f32 ? 4 : 2;
        uint8_t* obase = reinterpret_cast<uint8_t*>(a.out) + (a.epi == EPI_PARTIAL_F32 ? (size_t)split * a.split_stride * 4 : 0);
        const int total = rows_valid * chunks_per_row;
        for (int i = et; i < total; i += 128) {
          const int row = i / chunks_per_row, ch = i % chunks_per_row;
          const int64_t col = out_col0 + (int64_t)ch * elems_per_chunk;
          if (col >= out_cols) continue;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + row * row_bytes + ch * 16);
          *reinterpret_cast<uint4*>(obase + ((size_t)(row0 + row) * a.ldo + col) * esz) = v;
        }
      }

    }
  }
  (void)epi_ok;
  if constexpr (CL == 1) {
    (void)rows_valid;
    __syncwarp();
    cluster_sync_all();  // every CTA of the cluster has staged its partial tile
    if (warp >= 2) {
      const int q = warp & 3;
      switch (gridDim.z) {
        case 2: cluster_finish<2>(a, smem, q, lane, col0, row0, epi_ok); break;
        case 4: cluster_finish<4>(a, smem, q, lane, col0, row0, epi_ok); break;
        default: cluster_finish<8>(a, smem, q, lane, col0, row0, epi_ok); break;
      }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its tile
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem_base, (uint32_t)C::TMEM_COLS);
  }
}

// ---- persistent variant for prefill-size launches (256-token tiles, no split-K) -------------------
// One CTA per SM walks its share of the output tiles.  The accumulator is double-buffered in TMEM
// (2 x 256 columns), so the epilogue warps drain tile j while the MMA warp already accumulates tile
// j + 1 and the TMA ring keeps running across tile boundaries; the per-tile cost becomes
// max(main loop, epilogue) instead of their sum.  The epilogue transposes 32 tokens at a time through
// two small staging buffers, which leaves room for the same four pipeline stages.
struct PersistCfg {
  static constexpr int TN = 256;
  static constexpr int STAGES = 4;
  static constexpr int B_BYTES = TN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 48 KB
  static constexpr int STG_LD = 528;                      // bytes per staged token row (512 + 16: no bank conflicts)
  static constexpr int STG_BYTES = 32 * STG_LD;           // 32 tokens x 128 features x 4 bytes
  static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STG_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
};

// GROUPED: the weights are `groups` stacked matrices (3-D tensor map, third coordinate = group, e.g. the
// routed experts of a MoE layer) and group g owns the rows [row_offsets[g], row_offsets[g+1]) of x and of the
// output; the offsets are device data from an earlier kernel of the step.  The tile list is then built on
// the device: token tiles are numbered group by group (a group's last tile may be ragged), and a tile loads a
// full box of rows (the surplus belongs to the next group or is out of range) but stores only its own.
constexpr int kMaxGroups = 256;
constexpr int kMaxPersistCtas = 256;
// Per-CTA list "token tiles ahead of each group" of the grouped launches.  The kernel's shared memory is full
// (four 48 KB stages, two staging buffers), so each CTA keeps its copy in global memory, where it stays in L1.
static __device__ int g_first_tile[kMaxPersistCtas][kMaxGroups + 1];

template <bool GROUPED>
__global__ void __launch_bounds__(192) linear_tc_persist_kernel(const __grid_constant__ CUtensorMap tmW,
                                                                 const __grid_constant__ CUtensorMap tmX, TcArgs a,
                                                                 int tiles_n, int tiles_m) {
  using C = PersistCfg;
  constexpr int TN = C::TN;
  int* const s_first_tile = g_first_tile[blockIdx.x % kMaxPersistCtas];  // this CTA's copy (grouped launches only)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stg_base = smem + C::STAGES * C::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(stg_base + 2 * C::STG_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tmem_full = empty + C::STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (int)((a.K + BK - 1) / BK);
  if constexpr (GROUPED) {
    pdl_wait();  // the row offsets come from an earlier kernel of the step
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int g = 0; g < a.groups; ++g) {
        s_first_tile[g] = acc;
        acc += (a.row_offsets[g + 1] - a.row_offsets[g] + TN - 1) / TN;
      }
      s_first_tile[a.groups] = acc;
      __threadfence_block();
    }
    __syncthreads();
    tiles_m = s_first_tile[a.groups];
  }
  const int total_tiles = tiles_n * tiles_m;
  // Dense: same tile order as the one-tile kernel, groups of 8 token tiles per feature tile.  Grouped:
  // feature tiles fastest, so the CTAs of a wave work on a few token tiles of one or two experts.
  // row0 = first row of the tile, rows_valid = rows of it that belong to the output, grp = weight matrix.
  auto tile_coords = [&](int lin, int& tile_n, int& row0, int& rows_valid, int& grp) {
    if constexpr (GROUPED) {
      const int gm = lin / tiles_n;
      tile_n = lin - gm * tiles_n;
      int lo = 0, hi = a.groups;  // the group g with s_first_tile[g] <= gm < s_first_tile[g + 1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_first_tile[mid] <= gm) lo = mid;
        else hi = mid;
      }
      grp = lo;
      row0 = a.row_offsets[lo] + (gm - s_first_tile[lo]) * TN;
      rows_valid = min(TN, a.row_offsets[lo + 1] - row0);
    } else {
      constexpr int GROUP_M = 8;
      const int per_group = GROUP_M * tiles_n;
      const int group = lin / per_group;
      const int first_m = group * GROUP_M;
      const int group_rows = min(GROUP_M, tiles_m - first_m);
      const int in_group = lin - group * per_group;
      const int tile_m = first_m + in_group % group_rows;
      tile_n = in_group / group_rows;
      row0 = tile_m * TN;
      rows_valid = (int)min((int64_t)TN, a.M - row0);
      grp = 0;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 1);
    }
    fence_barrier_init();
    pdl_launch_dependents();
  }
  if (warp == 1) {
    tc::alloc(tmem_slot, (uint32_t)C::TMEM_COLS);
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      pdl_wait();  // the activations come from the previous kernel
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tile_n, row0, rows_valid, grp;
        tile_coords(t, tile_n, row0, rows_valid, grp);
        const int col0 = tile_n * BM;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % C::STAGES;
          if (it >= C::STAGES && !mbar_wait(&empty[s], ((it / C::STAGES) - 1) & 1, a.status)) {
            ok = false;
            break;
          }
          uint8_t* st = smem + s * C::STAGE_BYTES;
          mbar_expect_tx(&full[s], C::STAGE_BYTES);
          const int k = kb * BK;
          if constexpr (GROUPED) {
            tma_load_3d_hint(st, &tmW, &full[s], col0, k, grp, pol_x);  // an expert's weights serve several token tiles: keep them in L2
            tma_load_3d_hint(st + A_BYTES / 2, &tmW, &full[s], col0 + 64, k, grp, pol_x);
          } else {
            tma_load_2d_hint(st, &tmW, &full[s], col0, k, pol_w);
            tma_load_2d_hint(st + A_BYTES / 2, &tmW, &full[s], col0 + 64, k, pol_w);
          }
          tma_load_2d_hint(st + A_BYTES, &tmX, &full[s], k, row0, pol_x);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(TN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      const uint32_t smem_base = smem_u32(smem);
      int it = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++j) {
        const int buf = j & 1;
        if (j >= 2) {  // the epilogue must have drained this accumulator (tile j - 2)
          ok = mbar_wait(&tmem_empty[buf], ((j >> 1) - 1) & 1, a.status);
          if (!ok) break;
          tc::fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * TN);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % C::STAGES;
          ok = mbar_wait(&full[s], (it / C::STAGES) & 1, a.status);
          if (!ok) break;
          tc::fence_after();
          const uint32_t sa = smem_base + s * C::STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = tc::smem_desc(sa + kk * 2048, A_BYTES / 2, 1024);
            const uint64_t db = tc::smem_desc(sb + kk * 32, 16, 1024);
            tc::umma_bf16_ss(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc::commit(&empty[s]);
        }
        if (ok) tc::commit(&tmem_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue warps 2..5; TMEM lanes 32*(warp%4) .. +31
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    const bool swiglu = a.epi == EPI_SWIGLU_BF16;
    const bool out_f32 = a.epi == EPI_PARTIAL_F32 || a.epi == EPI_BIAS_F32;
    const int tile_cols = swiglu ? 64 : 128;
    const int row_bytes = tile_cols * (out_f32 ? 4 : 2);
    const int chunks_per_row = row_bytes / 16;
    const int elems_per_chunk = out_f32 ? 4 : 8;
    const size_t esz = out_f32 ? 4 : 2;
    const int64_t out_cols = swiglu ? a.N / 2 : a.N;
    pdl_wait();  // the output buffer may still be read by the previous kernel
    int j = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++j) {
      int tile_n, row0, rows_valid, grp;
      tile_coords(t, tile_n, row0, rows_valid, grp);
      const int col0 = tile_n * BM;
      const int buf = j & 1;
      if (ok) ok = mbar_wait(&tmem_full[buf], (j >> 1) & 1, a.status);
      tc::fence_after();
      const int64_t feat = (int64_t)col0 + q * 32 + lane;
      const bool feat_ok = feat < a.N;
      // grouped launches keep one bias row per group: [groups][N]
      const float bias_v = (a.bias && feat_ok && a.epi != EPI_PARTIAL_F32) ? a.bias[(int64_t)grp * a.N + feat] : 0.f;
      const int64_t out_col0 = swiglu ? col0 / 2 : col0;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 32) {
        if (c0 >= rows_valid) break;  // uniform over the four warps
        uint8_t* stg = stg_base + ((c0 >> 5) & 1) * C::STG_BYTES;
        if (ok) {
          uint32_t r[32];
          tc::ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * TN + c0), r);
          if (swiglu || out_f32) {
            // f32 [token][feature]; SwiGLU is applied on the way out, by all 128 threads
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              reinterpret_cast<float*>(stg + jj * C::STG_LD)[q * 32 + lane] = __uint_as_float(r[jj]) + bias_v;
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              reinterpret_cast<bf16*>(stg + jj * C::STG_LD)[q * 32 + lane] = __float2bfloat16_rn(__uint_as_float(r[jj]) + bias_v);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
        if (ok) {
          const int rows_here = min(32, rows_valid - c0);
          const int total = rows_here * chunks_per_row;
          uint8_t* obase = reinterpret_cast<uint8_t*>(a.out);
          for (int i = et; i < total; i += 128) {
            const int row = i / chunks_per_row, ch = i % chunks_per_row;
            const int64_t col = out_col0 + (int64_t)ch * elems_per_chunk;
            if (col >= out_cols) continue;
            uint4 v;
            if (swiglu) {
              // features ch*16 .. +7 are gates, +8 .. +15 their up partners (the engine's interleave)
              const float4* gp = reinterpret_cast<const float4*>(stg + row * C::STG_LD + ch * 64);
              const float4 g0 = gp[0], g1 = gp[1], u0 = gp[2], u1 = gp[3];
              v.x = pack_bf16(silu_f(g0.x) * u0.x, silu_f(g0.y) * u0.y);
              v.y = pack_bf16(silu_f(g0.z) * u0.z, silu_f(g0.w) * u0.w);
              v.z = pack_bf16(silu_f(g1.x) * u1.x, silu_f(g1.y) * u1.y);
              v.w = pack_bf16(silu_f(g1.z) * u1.z, silu_f(g1.w) * u1.w);
            } else {
              v = *reinterpret_cast<const uint4*>(stg + row * C::STG_LD + ch * 16);
            }
            *reinterpret_cast<uint4*>(obase + ((size_t)(row0 + c0 + row) * a.ldo + col) * esz) = v;
          }
        }
      }
      // every epilogue warp has read its part of the accumulator: hand the buffer back
      tc::fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) mbar_arrive(&tmem_empty[buf]);
    }
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem_base, (uint32_t)C::TMEM_COLS);
  }
}

// ---- two-CTA variant of the persistent kernel (prefill, dense weights) -------------------------------
// A cluster of two CTAs on neighbouring SMs works on one 256-feature x 256-token output tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 features of W (A operand) and its own 128 tokens of x
// (half of the B operand), the tensor cores of both SMs read both halves, and each CTA's tensor memory
// receives the accumulator rows of its own 128 features for all 256 tokens.  Per CTA a stage is 32 KB
// instead of 48 KB for the same tensor-core work, which takes the kernel off the shared-memory bandwidth
// limit of the one-CTA tile (48 KB written and read per 512 tensor cycles = 188 B/cycle against 128).
// Protocol: the bulk tensor loads of both CTAs complete on the LEADER's (even CTA's) `full` barrier (the
// cta_group::2 form of the load; no multicast: every CTA loads only what it alone needs); the leader's MMA
// thread issues for both and releases a stage by committing to the `empty` barrier of each CTA; finished
// accumulators are announced to both CTAs' epilogue warps the same way; the leader reuses an accumulator
// buffer once the epilogues of both CTAs have arrived on its `tmem_empty` barrier.
struct PairCfg {
  static constexpr int TN = 256;                          // tokens per tile (both CTAs together)
  static constexpr int STAGES = 6;
  static constexpr int B_BYTES = (TN / 2) * 128;          // this CTA's 128 tokens x 64 k
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB
  static constexpr int STG_LD = 528;
  static constexpr int STG_BYTES = 32 * STG_LD;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STG_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
};

constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the bit that tells the two CTAs of a pair apart in a shared::cluster address

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const void* tmap, uint64_t* leader_bar, int x, int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(leader_bar) & kPeerBitMask), "r"(x), "r"(y),
      "l"(policy)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrives on the barrier at shared::cluster address `bar_cluster_addr` once every tcgen05 operation this thread
// has issued so far is complete
__device__ __forceinline__ void commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192) linear_tc_pair_kernel(const __grid_constant__ CUtensorMap tmW,
                                                                                        const __grid_constant__ CUtensorMap tmX,
                                                                                        TcArgs a, int tiles_n, int tiles_m) {
  using C = PairCfg;
  constexpr int TN = C::TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stg_base = smem + C::STAGES * C::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(stg_base + 2 * C::STG_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tmem_full = empty + C::STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0: leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_tiles = tiles_n * tiles_m;  // tiles of 256 features x 256 tokens
  const int nkb = (int)((a.K + BK - 1) / BK);
  auto tile_coords = [&](int lin, int& tile_n, int& tile_m) {
    constexpr int GROUP_M = 8;
    const int per_group = GROUP_M * tiles_n;
    const int group = lin / per_group;
    const int first_m = group * GROUP_M;
    const int group_rows = min(GROUP_M, tiles_m - first_m);
    const int in_group = lin - group * per_group;
    tile_m = first_m + in_group % group_rows;
    tile_n = in_group / group_rows;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2);  // the epilogues of both CTAs
    }
    fence_barrier_init();
    pdl_launch_dependents();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc::fence_before();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival, and both allocations are done
  tc::fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      pdl_wait();  // the activations come from the previous kernel
      int it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += n_pairs) {
        int tile_n, tile_m;
        tile_coords(t, tile_n, tile_m);
        const int col0 = tile_n * 256 + (int)rank * BM, row0 = tile_m * TN + (int)rank * (TN / 2);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % C::STAGES;
          if (it >= C::STAGES && !mbar_wait(&empty[s], ((it / C::STAGES) - 1) & 1, a.status)) {
            ok = false;
            break;
          }
          uint8_t* st = smem + s * C::STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * C::STAGE_BYTES);  // this CTA's stage and the peer's
          const int k = kb * BK;
          tma_load_2d_pair(st, &tmW, &full[s], col0, k, pol_w);
          tma_load_2d_pair(st + A_BYTES / 2, &tmW, &full[s], col0 + 64, k, pol_w);
          tma_load_2d_pair(st + A_BYTES, &tmX, &full[s], k, row0, pol_x);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // D f32, A/B bf16, A MN-major, B K-major, N = 256 tokens, M = 256 features over the pair
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      const uint32_t smem_base = smem_u32(smem);
      int it = 0, j = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += n_pairs, ++j) {
        const int buf = j & 1;
        if (j >= 2) {  // both epilogues must have drained this accumulator (tile j - 2)
          ok = mbar_wait(&tmem_empty[buf], ((j >> 1) - 1) & 1, a.status);
          if (!ok) break;
          tc::fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * TN);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % C::STAGES;
          ok = mbar_wait(&full[s], (it / C::STAGES) & 1, a.status);
          if (!ok) break;
          tc::fence_after();
          const uint32_t sa = smem_base + s * C::STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = tc::smem_desc(sa + kk * 2048, A_BYTES / 2, 1024);
            const uint64_t db = tc::smem_desc(sb + kk * 32, 16, 1024);
            umma_bf16_ss_pair(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          commit_pair(smem_u32(&empty[s]));
          commit_pair(dsmem_addr(smem_u32(&empty[s]), 1));
        }
        if (ok) {
          commit_pair(smem_u32(&tmem_full[buf]));
          commit_pair(dsmem_addr(smem_u32(&tmem_full[buf]), 1));
        }
      }
    }
  } else {
    // ---------------- epilogue warps 2..5 of each CTA; TMEM lanes 32*(warp%4) .. +31 = this CTA's 128 features
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    const bool swiglu = a.epi == EPI_SWIGLU_BF16;
    const bool out_f32 = a.epi == EPI_PARTIAL_F32 || a.epi == EPI_BIAS_F32;
    const int tile_cols = swiglu ? 64 : 128;
    const int row_bytes = tile_cols * (out_f32 ? 4 : 2);
    const int chunks_per_row = row_bytes / 16;
    const int elems_per_chunk = out_f32 ? 4 : 8;
    const size_t esz = out_f32 ? 4 : 2;
    const int64_t out_cols = swiglu ? a.N / 2 : a.N;
    const uint32_t leader_tmem_empty0 = dsmem_addr(smem_u32(&tmem_empty[0]), 0);
    pdl_wait();  // the output buffer may still be read by the previous kernel
    int j = 0;
    bool ok = true;
    for (int t = pair; t < total_tiles; t += n_pairs, ++j) {
      int tile_n, tile_m;
      tile_coords(t, tile_n, tile_m);
      const int col0 = tile_n * 256 + (int)rank * BM, row0 = tile_m * TN;
      const int rows_valid = (int)min((int64_t)TN, a.M - row0);
      const int buf = j & 1;
      if (ok) ok = mbar_wait(&tmem_full[buf], (j >> 1) & 1, a.status);
      tc::fence_after();
      const int64_t feat = (int64_t)col0 + q * 32 + lane;
      const bool feat_ok = feat < a.N;
      const float bias_v = (a.bias && feat_ok && a.epi != EPI_PARTIAL_F32) ? a.bias[feat] : 0.f;
      const int64_t out_col0 = swiglu ? col0 / 2 : col0;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 32) {
        if (c0 >= rows_valid) break;  // uniform over the four warps
        uint8_t* stg = stg_base + ((c0 >> 5) & 1) * C::STG_BYTES;
        if (ok) {
          uint32_t r[32];
          tc::ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * TN + c0), r);
          if (swiglu || out_f32) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              reinterpret_cast<float*>(stg + jj * C::STG_LD)[q * 32 + lane] = __uint_as_float(r[jj]) + bias_v;
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              reinterpret_cast<bf16*>(stg + jj * C::STG_LD)[q * 32 + lane] = __float2bfloat16_rn(__uint_as_float(r[jj]) + bias_v);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
        if (ok) {
          const int rows_here = min(32, rows_valid - c0);
          const int total = rows_here * chunks_per_row;
          uint8_t* obase = reinterpret_cast<uint8_t*>(a.out);
          for (int i = et; i < total; i += 128) {
            const int row = i / chunks_per_row, ch = i % chunks_per_row;
            const int64_t col = out_col0 + (int64_t)ch * elems_per_chunk;
            if (col >= out_cols) continue;
            uint4 v;
            if (swiglu) {
              const float4* gp = reinterpret_cast<const float4*>(stg + row * C::STG_LD + ch * 64);
              const float4 g0 = gp[0], g1 = gp[1], u0 = gp[2], u1 = gp[3];
              v.x = pack_bf16(silu_f(g0.x) * u0.x, silu_f(g0.y) * u0.y);
              v.y = pack_bf16(silu_f(g0.z) * u0.z, silu_f(g0.w) * u0.w);
              v.z = pack_bf16(silu_f(g1.x) * u1.x, silu_f(g1.y) * u1.y);
              v.w = pack_bf16(silu_f(g1.z) * u1.z, silu_f(g1.w) * u1.w);
            } else {
              v = *reinterpret_cast<const uint4*>(stg + row * C::STG_LD + ch * 16);
            }
            *reinterpret_cast<uint4*>(obase + ((size_t)(row0 + c0 + row) * a.ldo + col) * esz) = v;
          }
        }
      }
      // every epilogue warp of this CTA has read its part of the accumulator: tell the leader
      tc::fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) mbar_arrive_cluster(leader_tmem_empty0 + (uint32_t)buf * 8u);
    }
  }
  tc::fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves (or frees tensor memory) while the peer may still use this CTA's memory or barriers
  if (warp == 1) {
    tc::fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

template <int TN>
int launch_tn(Ctx* c, const LinearBf16Plan& plan, const CUtensorMap& tmX, const TcArgs& a, dim3 grid) {
  using C = TcCfg<TN>;
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA(cudaFuncSetAttribute(linear_tc_kernel<TN, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_set = true;
  }
  RB_CUDA(launch_k(linear_tc_kernel<TN, 0>, grid, dim3(192), (size_t)C::SMEM, c->stream, c->use_pdl, plan.tmW, tmX, a));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace

bool linear_tc_cluster_ok(Ctx* c, const LinearBf16Plan& plan, int64_t M, int ksplit) {
  return c->splitk_cluster != 0 && c->linear_impl == 2 && plan.groups == 0 && M >= 1 && M <= 32 &&
         (ksplit == 2 || ksplit == 4 || ksplit == 8);
}

int linear_tc_cluster_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int ksplit,
                             float* out, int64_t ldo, const QkvPostArgs* fuse_qkv) {
  RB_REQUIRE(linear_tc_cluster_ok(c, plan, M, ksplit), "cluster split-K: at most 32 rows and 2, 4 or 8 splits");
  RB_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "bf16 Linear: activations must be 16-byte aligned rows");
  using C = TcCfg<32>;
  CUtensorMap tmX;
  RB_TRY(make_tmap_2d_bf16(&tmX, x, (uint64_t)plan.K, (uint64_t)M, (uint64_t)ldx * 2, 64, 32));
  TcArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M;
  a.N = plan.N;
  a.K = plan.K;
  const int nkb = (int)((plan.K + BK - 1) / BK);
  a.kb_per_split = (nkb + ksplit - 1) / ksplit;
  a.epi = EPI_PARTIAL_F32;
  a.out = out;
  a.ldo = ldo;
  a.split_stride = 0;
  a.bias = nullptr;
  a.status = c->d_status;
  if (fuse_qkv) {
    RB_REQUIRE(fuse_qkv->act_dtype == REWB200_BF16 && fuse_qkv->hd % 2 == 0 &&
                   (int64_t)(fuse_qkv->nh + 2 * fuse_qkv->kvh) * fuse_qkv->hd == plan.N,
               "fused q|k|v epilogue: bf16 activations and a weight of nq + 2 nkv columns");
    a.fuse_qkv = 1;
    a.qp = *fuse_qkv;
  }
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA(cudaFuncSetAttribute(linear_tc_kernel<32, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_set = true;
  }
  dim3 grid((unsigned)((plan.N + BM - 1) / BM), 1u, (unsigned)ksplit);
  RB_CUDA(launch_k_cluster(linear_tc_kernel<32, 1>, grid, dim3(192), (size_t)C::SMEM, c->stream, c->use_pdl,
                           dim3(1, 1, (unsigned)ksplit), plan.tmW, tmX, a));
  ++g_launch_total;
  return REWB200_OK;
}

// Grouped launch (plan.groups stacked weight matrices, rows of group g = [row_offsets[g], row_offsets[g+1]) of
// x / out, bias [groups][N] or NULL): the persistent kernel with its tile list built on the device.  For
// groups of prefill size (MoE experts with hundreds of rows each); smaller ones stay on the HBM-bound
// mma.sync kernel of linear_bf16.cu.
int linear_tc_grouped_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int epi, void* out,
                             int64_t ldo, const float* bias, const int* row_offsets) {
  RB_REQUIRE(plan.groups >= 1 && plan.groups <= kMaxGroups && row_offsets != nullptr, "grouped tcgen05 Linear: 1..256 groups and row offsets");
  RB_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "bf16 Linear: activations must be 16-byte aligned rows");
  RB_REQUIRE(epi != EPI_PARTIAL_F32, "grouped Linear does not split K");
  RB_REQUIRE(epi != EPI_SWIGLU_BF16 || plan.N % 16 == 0, "SwiGLU epilogue needs interleaved width % 16 == 0");
  if (M == 0) return REWB200_OK;
  CUtensorMap tmX;
  RB_TRY(make_tmap_2d_bf16(&tmX, x, (uint64_t)plan.K, (uint64_t)M, (uint64_t)ldx * 2, 64, PersistCfg::TN));
  TcArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M;
  a.N = plan.N;
  a.K = plan.K;
  a.kb_per_split = (int)((plan.K + BK - 1) / BK);
  a.epi = epi;
  a.out = out;
  a.ldo = ldo;
  a.split_stride = M * ldo;
  a.bias = bias;
  a.status = c->d_status;
  a.row_offsets = row_offsets;
  a.groups = plan.groups;
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA(cudaFuncSetAttribute(linear_tc_persist_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PersistCfg::SMEM));
    attr_set = true;
  }
  const int tiles_n = (int)((plan.N + BM - 1) / BM);
  // at most ceil(M / TN) + groups token tiles exist; one CTA per SM walks them
  const int64_t max_tiles = (int64_t)tiles_n * ((M + PersistCfg::TN - 1) / PersistCfg::TN + plan.groups);
  const int ctas = (int)std::min<int64_t>(std::min<int64_t>(max_tiles, c->sm_count), kMaxPersistCtas);
  RB_CUDA(launch_k(linear_tc_persist_kernel<true>, dim3((unsigned)ctas), dim3(192), (size_t)PersistCfg::SMEM, c->stream, c->use_pdl,
                   plan.tmW, tmX, a, tiles_n, 0));
  ++g_launch_total;
  return REWB200_OK;
}

// Loads this file's module on the current device and prepares the decode-size kernel (M <= 32), so that a
// later launch of it neither loads code nor changes function attributes.
int linear_tc_preload() {
  RB_CUDA(cudaFuncSetAttribute(linear_tc_kernel<32, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<32>::SMEM));
  cudaFuncAttributes fa;
  RB_CUDA(cudaFuncGetAttributes(&fa, linear_tc_kernel<32, 0>));
  return REWB200_OK;
}

// Same contract as linear_bf16_launch (ungrouped).
int linear_tc_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int epi, int ksplit,
                     void* out, int64_t ldo, const float* bias) {
  RB_REQUIRE(plan.groups == 0, "the tcgen05 Linear does not take grouped weights");
  RB_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "bf16 Linear: activations must be 16-byte aligned rows");
  RB_REQUIRE(ksplit >= 1 && (ksplit == 1 || epi == EPI_PARTIAL_F32), "split-K needs the partial epilogue");
  RB_REQUIRE(epi != EPI_SWIGLU_BF16 || plan.N % 16 == 0, "SwiGLU epilogue needs interleaved width % 16 == 0");
  if (M == 0) return REWB200_OK;
  const int TN = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
  CUtensorMap tmX;
  RB_TRY(make_tmap_2d_bf16(&tmX, x, (uint64_t)plan.K, (uint64_t)M, (uint64_t)ldx * 2, 64, TN));
  TcArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M;
  a.N = plan.N;
  a.K = plan.K;
  const int nkb = (int)((plan.K + BK - 1) / BK);
  a.kb_per_split = (nkb + ksplit - 1) / ksplit;
  a.epi = epi;
  a.out = out;
  a.ldo = ldo;
  a.split_stride = M * ldo;
  a.bias = bias;
  a.status = c->d_status;
  dim3 grid((unsigned)((plan.N + BM - 1) / BM), (unsigned)((M + TN - 1) / TN), (unsigned)ksplit);
  if (TN == 256 && ksplit == 1 && c->prefill_persistent && c->prefill_pair && plan.N % 256 == 0 && c->sm_count % 2 == 0 &&
      (int64_t)grid.x * grid.y >= 2 * (int64_t)c->sm_count) {
    // two-CTA tiles: 256 features x 256 tokens per pair of SMs
    CUtensorMap tmXh;
    RB_TRY(make_tmap_2d_bf16(&tmXh, x, (uint64_t)plan.K, (uint64_t)M, (uint64_t)ldx * 2, 64, PairCfg::TN / 2));
    static bool pair_attr = false;
    if (!pair_attr) {
      RB_CUDA(cudaFuncSetAttribute(linear_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM));
      pair_attr = true;
    }
    const int tiles_n = (int)(plan.N / 256), tiles_m = (int)grid.y;
    const int ctas = (int)std::min<int64_t>(2 * (int64_t)tiles_n * tiles_m, c->sm_count);
    RB_CUDA(launch_k(linear_tc_pair_kernel, dim3((unsigned)(ctas & ~1)), dim3(192), (size_t)PairCfg::SMEM, c->stream, c->use_pdl,
                     plan.tmW, tmXh, a, tiles_n, tiles_m));
    ++g_launch_total;
    return REWB200_OK;
  }
  if (TN == 256 && ksplit == 1 && c->prefill_persistent && (int64_t)grid.x * grid.y >= 2 * (int64_t)c->sm_count) {
    static bool attr_set = false;
    if (!attr_set) {
      RB_CUDA(cudaFuncSetAttribute(linear_tc_persist_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PersistCfg::SMEM));
      attr_set = true;
    }
    const int ctas = (int)std::min<int64_t>((int64_t)grid.x * grid.y, c->sm_count);
    RB_CUDA(launch_k(linear_tc_persist_kernel<false>, dim3((unsigned)ctas), dim3(192), (size_t)PersistCfg::SMEM, c->stream, c->use_pdl,
                     plan.tmW, tmX, a, (int)grid.x, (int)grid.y));
    ++g_launch_total;
    return REWB200_OK;
  }
  switch (TN) {
    case 32: return launch_tn<32>(c, plan, tmX, a, grid);
    case 64: return launch_tn<64>(c, plan, tmX, a, grid);
    case 128: return launch_tn<128>(c, plan, tmX, a, grid);
    default: return launch_tn<256>(c, plan, tmX, a, grid);
  }
}

}  // namespace rewb
