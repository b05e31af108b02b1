// bf16 Linear (src/rew/nn/linear.nim:43-49): y[M,N] = x[M,K] @ W[K,N] (+ b).
//
// Decode regime (M <= 32 rows) is bound by streaming W from HBM once; the kernel
// is a TMA-fed, mbarrier-pipelined weight streamer:
//   - W keeps the reference's [in,out] row-major layout.  A CTA owns 128 output
//     columns and a K range; one producer warp issues cp.async.bulk.tensor loads
//     of 64(k) x 64(n) bf16 boxes (128-byte swizzle) into a STAGES-deep ring.
//   - 4 consumer warps (32 columns each) read the swizzled boxes with
//     ldmatrix(.trans for W) and accumulate in f32 with mma.sync m16n8k16.
//   - The weight loads of the first STAGES stages are issued BEFORE
//     griddepcontrol.wait, so under programmatic dependent launch the ramp-up of
//     this kernel overlaps the tail of the previous one; only the activation
//     loads and the epilogue wait for the producer kernel.
//   - Split-K partials (f32) go to scratch and are summed by the consumer
//     kernel (residual+norm or QKV post-processing), never by atomics, so
//     results are deterministic.
// The default bf16 Linear is the tcgen05 kernel of linear_tc.cu; this mma.sync
// kernel serves the grouped launches of the MoE experts (blockIdx.z = expert,
// 3-D tensor map, device-side row offsets) and stays selectable for everything
// else with the option linear = "mma" (128-row tiles for more than 64 rows).
#include "common.cuh"
#include "ptx.cuh"

namespace rewb {

extern int64_t g_launch_total;

namespace {

constexpr int BN = 128;   // output columns per CTA
constexpr int BK = 64;    // k per stage (one 128-byte swizzle row of x)
constexpr int W_BOX_BYTES = BK * 64 * 2;  // 64 k-rows x 64 cols
constexpr int CONSUMER_WARPS = 4;

template <int ROWS>
struct Cfg {
  static constexpr int STAGES = (ROWS <= 32) ? 5 : 4;
  static constexpr int X_BYTES = ROWS * 128;
  static constexpr int STAGE_BYTES = 2 * W_BOX_BYTES + X_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int MT = ROWS / 16;
};

struct LinArgs {
  int64_t M, N, K;
  int kb_per_split;        // k-blocks (of 64) each split handles
  int epi;
  void* out;
  int64_t ldo;             // elements between output rows
  int64_t split_stride;    // elements between split slabs (EPI_PARTIAL_F32)
  const float* bias;
  const int* row_offsets;  // grouped: rows of group g = [row_offsets[g], row_offsets[g+1])
  int grouped;
  int* status;
};

__device__ __forceinline__ float silu_f(float x) { return x * (1.0f / (1.0f + __expf(-x))); }

template <int ROWS>
__global__ void __launch_bounds__(160) linear_bf16_kernel(const __grid_constant__ CUtensorMap tmW,
                                                           const __grid_constant__ CUtensorMap tmX, LinArgs a) {
  using C = Cfg<ROWS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = blockIdx.x * BN;
  int row0, rows_valid, group = 0;
  if (a.grouped) {
    // the row offsets are produced by earlier kernels of the same step: under programmatic
    // dependent launch they may only be read after griddepcontrol.wait
    pdl_wait();
    group = blockIdx.z;
    const int r_begin = a.row_offsets[group], r_end = a.row_offsets[group + 1];
    row0 = r_begin + blockIdx.y * ROWS;
    rows_valid = r_end - row0;
    if (rows_valid <= 0) return;   // uniform for the CTA: no barrier has been touched yet
    if (rows_valid > ROWS) rows_valid = ROWS;
  } else {
    row0 = blockIdx.y * ROWS;
    rows_valid = (int)min((int64_t)ROWS, a.M - row0);
  }
  const int split = a.grouped ? 0 : blockIdx.z;
  const int nkb_total = (int)((a.K + BK - 1) / BK);
  const int kb0 = split * a.kb_per_split;
  const int nkb = max(0, min(a.kb_per_split, nkb_total - kb0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CONSUMER_WARPS);
    }
    fence_barrier_init();
    pdl_launch_dependents();
  }
  __syncthreads();

  if (warp == CONSUMER_WARPS) {
    // ---------------- producer: one lane drives TMA
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
        if (a.grouped) {
          tma_load_3d_hint(st, &tmW, &full[kb], col0, k, group, pol_w);
          tma_load_3d_hint(st + W_BOX_BYTES, &tmW, &full[kb], col0 + 64, k, group, pol_w);
        } else {
          tma_load_2d_hint(st, &tmW, &full[kb], col0, k, pol_w);
          tma_load_2d_hint(st + W_BOX_BYTES, &tmW, &full[kb], col0 + 64, k, pol_w);
        }
      }
      pdl_wait();  // activations come from the previous kernel
      for (int kb = 0; kb < pre; ++kb) {
        uint8_t* st = smem + kb * C::STAGE_BYTES;
        tma_load_2d_hint(st + 2 * W_BOX_BYTES, &tmX, &full[kb], (kb0 + kb) * BK, row0, pol_x);
      }
      bool ok = true;
      for (int kb = pre; kb < nkb && ok; ++kb) {
        const int s = kb % C::STAGES;
        ok = mbar_wait(&empty[s], ((kb / C::STAGES) - 1) & 1, a.status);
        if (!ok) break;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        const int k = (kb0 + kb) * BK;
        if (a.grouped) {
          tma_load_3d_hint(st, &tmW, &full[s], col0, k, group, pol_w);
          tma_load_3d_hint(st + W_BOX_BYTES, &tmW, &full[s], col0 + 64, k, group, pol_w);
        } else {
          tma_load_2d_hint(st, &tmW, &full[s], col0, k, pol_w);
          tma_load_2d_hint(st + W_BOX_BYTES, &tmW, &full[s], col0 + 64, k, pol_w);
        }
        tma_load_2d_hint(st + 2 * W_BOX_BYTES, &tmX, &full[s], k, row0, pol_x);
      }
    }
    return;
  }

  // ---------------- consumers
  float acc[C::MT][4][4];
#pragma unroll
  for (int i = 0; i < C::MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;

  const uint32_t smem_base = smem_u32(smem);
  // W: this warp's 32 columns live in box (warp/2), 16-byte chunks 4*(warp%2)..+3
  const uint32_t w_box_off = (warp >> 1) * W_BOX_BYTES;
  const uint32_t w_chunk0 = (warp & 1) * 4;
  const uint32_t l8 = lane & 7, lq = lane >> 3;  // row within 8x8 matrix, matrix index

  bool ok = true;
  for (int kb = 0; kb < nkb; ++kb) {
    const int s = kb % C::STAGES;
    ok = mbar_wait(&full[s], (kb / C::STAGES) & 1, a.status);
    if (!ok) break;
    const uint32_t st = smem_base + s * C::STAGE_BYTES;
    const uint32_t wb = st + w_box_off;
    const uint32_t xb = st + 2 * W_BOX_BYTES;
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      // B fragments (W): matrices (k 0-7,n-tile j) (k 8-15,j) (k 0-7,j+1) (k 8-15,j+1)
      uint32_t b[4][2];
      {
        const uint32_t krow = kk * 16 + (lq & 1) * 8 + l8;
        ldmatrix_x4_trans(b[0][0], b[0][1], b[1][0], b[1][1], wb + swz128(krow, w_chunk0 + 0 + (lq >> 1)));
        ldmatrix_x4_trans(b[2][0], b[2][1], b[3][0], b[3][1], wb + swz128(krow, w_chunk0 + 2 + (lq >> 1)));
      }
#pragma unroll
      for (int mt = 0; mt < C::MT; ++mt) {
        // A fragment (x rows 16mt..): (rows 0-7,k 0-7) (rows 8-15,k 0-7) (rows 0-7,k 8-15) (rows 8-15,k 8-15)
        uint32_t af[4];
        const uint32_t xrow = mt * 16 + (lq & 1) * 8 + l8;
        ldmatrix_x4(af[0], af[1], af[2], af[3], xb + swz128(xrow, kk * 2 + (lq >> 1)));
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma_bf16_16816(acc[mt][nt], af, b[nt][0], b[nt][1]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  // ---------------- epilogue (writes wait for the previous kernel's readers)
  pdl_wait();
  if (!ok) return;
  // grouped launches keep one bias row per group: [groups][N]
  const float* bias = a.bias ? a.bias + (a.grouped ? (int64_t)group * a.N : 0) : nullptr;
  const int g = lane >> 2, t = lane & 3;
  const int wcol0 = col0 + warp * 32;
#pragma unroll
  for (int mt = 0; mt < C::MT; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mt * 16 + g + half * 8;
      if (r >= rows_valid) continue;
      const int64_t grow = row0 + r;
      if (a.epi == EPI_SWIGLU_BF16) {
#pragma unroll
        for (int nt = 0; nt < 4; nt += 2) {
          const int64_t cg = wcol0 + nt * 8 + 2 * t;  // gate column in the interleaved matrix
          if (cg >= a.N) continue;
          const float g0 = acc[mt][nt][half * 2 + 0] + (bias ? bias[cg] : 0.f);
          const float g1 = acc[mt][nt][half * 2 + 1] + (bias ? bias[cg + 1] : 0.f);
          const float u0 = acc[mt][nt + 1][half * 2 + 0] + (bias ? bias[cg + 8] : 0.f);
          const float u1 = acc[mt][nt + 1][half * 2 + 1] + (bias ? bias[cg + 9] : 0.f);
          const int64_t oc = (wcol0 + nt * 8) / 2 + 2 * t;
          uint32_t v = pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
          *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(a.out) + grow * a.ldo + oc) = v;
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int64_t c = wcol0 + nt * 8 + 2 * t;
          if (c >= a.N) continue;
          float v0 = acc[mt][nt][half * 2 + 0], v1 = acc[mt][nt][half * 2 + 1];
          if (a.epi == EPI_PARTIAL_F32) {
            float* o = reinterpret_cast<float*>(a.out) + split * a.split_stride + grow * a.ldo + c;
            *reinterpret_cast<float2*>(o) = make_float2(v0, v1);
          } else {
            if (bias) {
              v0 += bias[c];
              v1 += bias[c + 1];
            }
            if (a.epi == EPI_BIAS_F32) {
              float* o = reinterpret_cast<float*>(a.out) + grow * a.ldo + c;
              *reinterpret_cast<float2*>(o) = make_float2(v0, v1);
            } else {
              bf16* o = reinterpret_cast<bf16*>(a.out) + grow * a.ldo + c;
              *reinterpret_cast<uint32_t*>(o) = pack_bf16(v0, v1);
            }
          }
        }
      }
    }
  }
}

template <int ROWS>
int launch_rows(Ctx* c, const LinearBf16Plan& plan, const CUtensorMap& tmX, const LinArgs& a, dim3 grid) {
  using C = Cfg<ROWS>;
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA(cudaFuncSetAttribute(linear_bf16_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_set = true;
  }
  RB_CUDA(launch_k(linear_bf16_kernel<ROWS>, grid, dim3(160), (size_t)C::SMEM, c->stream, c->use_pdl, plan.tmW, tmX, a));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace

int linear_bf16_plan(LinearBf16Plan* plan, const bf16* W, int64_t K, int64_t N, int groups) {
  RB_REQUIRE(N % 8 == 0, "bf16 Linear needs out features % 8 == 0 (TMA row stride of 16 bytes), got " + std::to_string(N));
  plan->K = K;
  plan->N = N;
  plan->groups = groups;
  if (groups >= 1)  // grouped (one weight matrix per expert); 0 = a single matrix
    return make_tmap_3d_bf16(&plan->tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)groups, (uint64_t)N * 2,
                             (uint64_t)K * N * 2, 64, BK);
  return make_tmap_2d_bf16(&plan->tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)N * 2, 64, BK);
}

// Enough CTAs to keep two resident per SM, but never K slices shorter than 8
// k-blocks (512 rows): shorter slices spend their time filling the pipeline.
// As linear_tc_preload, for the mma.sync kernel of steps of up to 32 rows (option linear=mma).
int linear_bf16_preload() {
  RB_CUDA(cudaFuncSetAttribute(linear_bf16_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<32>::SMEM));
  cudaFuncAttributes fa;
  RB_CUDA(cudaFuncGetAttributes(&fa, linear_bf16_kernel<32>));
  return REWB200_OK;
}

int linear_bf16_pick_ksplit(Ctx* c, int64_t M, int64_t K, int64_t N) {
  if (M > 256 || M > c->splitk_max_rows) return 1;  // up to here one token tile covers the step: the weights are streamed once either way
  const int tiles = (int)((N + BN - 1) / BN);
  const int nkb = (int)((K + BK - 1) / BK);
  const int target = 2 * c->sm_count;
  // every split is another f32 slab of M rows that the consumer kernel reads back: fewer of them as the step grows
  const int cap = M <= 64 ? 16 : (M <= 128 ? 4 : 2);
  int split = 1;
  // stop doubling once the CTA count would overshoot the resident slots by more than a quarter
  while (tiles * split * 2 <= target + target / 4 && nkb / (split * 2) >= c->splitk_min_blocks && split < cap) split *= 2;
  // a launch that still leaves SMs empty (narrow layers of a tensor-parallel shard) may cut K finer
  while (tiles * split < c->sm_count && nkb / (split * 2) >= std::min(4, c->splitk_min_blocks) && split < cap) split *= 2;
  return split;
}

int linear_bf16_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int epi,
                       int ksplit, void* out, int64_t ldo, const float* bias, const int* row_offsets,
                       int max_rows_per_group) {
  RB_REQUIRE(ldx % 8 == 0, "bf16 Linear needs the activation row stride % 8 == 0");
  RB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, "bf16 Linear: activation pointer must be 16-byte aligned");
  RB_REQUIRE(ksplit >= 1 && (ksplit == 1 || epi == EPI_PARTIAL_F32), "split-K needs the partial epilogue");
  RB_REQUIRE(epi != EPI_SWIGLU_BF16 || plan.N % 16 == 0, "SwiGLU epilogue needs interleaved width % 16 == 0");
  if (M == 0) return REWB200_OK;
  const bool grouped = plan.groups >= 1;
  if (!grouped && (c->linear_impl == 2 || (c->linear_impl == 1 && M > 32)))
    return linear_tc_launch(c, plan, x, ldx, M, epi, ksplit, out, ldo, bias);
  RB_REQUIRE(!grouped || (row_offsets != nullptr && ksplit == 1), "grouped Linear needs row offsets and no split-K");
  // groups of prefill size are contractions for the tcgen05 pipe; small ones (decode) stream weights from HBM here
  if (grouped && max_rows_per_group > 64 && c->linear_impl != 0 && plan.groups <= 256 && epi != EPI_PARTIAL_F32)
    return linear_tc_grouped_launch(c, plan, x, ldx, M, epi, out, ldo, bias, row_offsets);
  const int64_t rows_for_tile = grouped ? max_rows_per_group : M;
  const bool small = rows_for_tile <= 64;  // 33..64 rows: two 32-row tiles keep two CTAs per SM
  const int ROWS = small ? 32 : 128;
  CUtensorMap tmX;
  RB_TRY(make_tmap_2d_bf16(&tmX, x, (uint64_t)plan.K, (uint64_t)M, (uint64_t)ldx * 2, 64, ROWS));
  LinArgs a;
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
  a.row_offsets = row_offsets;
  a.grouped = grouped ? 1 : 0;
  a.status = c->d_status;
  dim3 grid((unsigned)((plan.N + BN - 1) / BN), (unsigned)((rows_for_tile + ROWS - 1) / ROWS),
            (unsigned)(grouped ? plan.groups : ksplit));
  if (small) return launch_rows<32>(c, plan, tmX, a, grid);
  return launch_rows<128>(c, plan, tmX, a, grid);
}

}  // namespace rewb
