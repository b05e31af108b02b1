// Weight-only NF4 Linear: the frozen base projection of QloraLinear (src/rew/nn/lora.nim:410-431) with
// the weights kept in their 4-bit codes in HBM and dequantised inside the GEMV, instead of the
// reference's dequantise-once-on-the-host-then-fp32-matmul (lora.nim:347-349).
//
// Codec as src/rew/quantize/codecs.nim:13-70: blocks of 64 consecutive elements of the flat row-major
// [in, out] weight (= 64 consecutive output features of one input row when out % 64 == 0), scale =
// max(1e-10, absmax), code = nearest of the 16 NF4 levels (first one on a tie), value = level * scale.
//
// Device layout (this library's own; rewb200_nf4_unpack gives back the reference's bytes):
//   q  [N/64][K/64][4 k16 steps][32 lanes] uint4   one 16-byte load per lane and k16 step: word w holds
//        the column tiles j = 2w and 2w+1; nibble (j&1)*4 + r of a word is W[k][n] with
//        k = 64 kb + 16 i + {2t, 2t+1, 2t+8, 2t+9}[r], n = 64 g + 8 j + lane/4, t = lane % 4 -- byte b of
//        a word is therefore one B register (two consecutive k) of mma.m16n8k16 for one tile
//   sc [N/64][K] f32                                the scales of one 64-column group, contiguous along k
// GEMV (rows <= 32): a warp owns one 64-column group over a slice of K.  A byte (two codes) indexes a
// shared-memory table of bf16 level PAIRS, replicated once per lane so that lane l only ever touches
// bank l: one conflict-free LDS yields a whole B register.  (Integer byte-permute lookups were tried
// first: 11 ALU operations per four weights saturate the half-rate integer pipe at 0.17 of the HBM
// roofline.)  The register is multiplied by the bf16 pair of its two rows' scales (HMUL2) and fed to the
// tensor core; activations are staged per warp with cp.async, double-buffered.  The 8 warps of a CTA
// split the CTA's K range and add their accumulators through shared memory; CTAs of different K ranges
// leave f32 slabs [ksplit][M][N] that the consumer sums, as for the bf16 Linear.
#include <cuda_bf16.h>

#include <algorithm>
#include <string>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace rewb {
namespace {

__constant__ float kNf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                               -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                               0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                               0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
// the same levels rounded to bf16 (round to nearest even)
__constant__ uint16_t kNf4Bf16[16] = {0xBF80, 0xBF32, 0xBF06, 0xBECA, 0xBE92, 0xBE3D, 0xBDBA, 0x0000,
                                      0x3DA3, 0x3E25, 0x3E7C, 0x3EAD, 0x3EE2, 0x3F10, 0x3F39, 0x3F80};

__device__ __forceinline__ int64_t map_col(const ColMap& cm, int64_t n) {
  const int64_t seg = n / cm.seg_len, within = n % cm.seg_len;
  return (within / cm.gran) * cm.gstride + (within % cm.gran) + seg * cm.seg_off;
}

// position of W[64 kb + kk][64 g + nn] inside the (g, kb) tile: k16 step, lane, word, nibble
__device__ __forceinline__ void tile_pos(int kk, int nn, int& i, int& lane, int& word, int& nib) {
  i = kk >> 4;
  const int k16 = kk & 15, j = nn >> 3, c = nn & 7;
  const int t = (k16 & 7) >> 1, r = (k16 & 1) + ((k16 >> 3) << 1);
  lane = c * 4 + t;
  word = j >> 1;
  nib = (j & 1) * 4 + r;
}

// grid (N/64, K/64), 64 threads: thread r quantises row kb*64 + r of the group, then the tile is packed.
template <typename T>
__global__ void __launch_bounds__(64) nf4_quantize_kernel(const T* src, int64_t ld, ColMap cm, uint4* q, float* sc, int64_t K,
                                                          int64_t N) {
  __shared__ uint32_t tile[4][32][4];  // [k16 step][lane][word]
  const int g = blockIdx.x, kb = blockIdx.y, r = threadIdx.x;
  const int64_t k = (int64_t)kb * 64 + r;
  for (int i = threadIdx.x; i < 4 * 32 * 4; i += 64) (&tile[0][0][0])[i] = 0u;
  __syncthreads();
  float v[64];
  float absMax = 1e-10f;
#pragma unroll 8
  for (int n = 0; n < 64; ++n) {
    v[n] = (float)src[k * ld + map_col(cm, (int64_t)g * 64 + n)];
    absMax = fmaxf(absMax, fabsf(v[n]));
  }
  sc[(int64_t)g * K + k] = absMax;
#pragma unroll 4
  for (int n = 0; n < 64; ++n) {
    const float normalized = fminf(1.0f, fmaxf(-1.0f, v[n] / absMax));
    float minDist = 1e10f;
    int code = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float dist = fabsf(normalized - kNf4[i]);
      if (dist < minDist) {
        minDist = dist;
        code = i;
      }
    }
    int i, lane, word, nib;
    tile_pos(r, n, i, lane, word, nib);
    atomicOr(&tile[i][lane][word], (uint32_t)code << (4 * nib));
  }
  __syncthreads();
  const int KB = (int)(K / 64);
  uint4* dst = q + ((int64_t)g * KB + kb) * 128;
  for (int e = threadIdx.x; e < 128; e += 64) {
    const uint32_t* w = &tile[e >> 5][e & 31][0];
    dst[e] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// dst (bf16, column-mapped) = level * scale, or codes_out (uint8 [K][N]) = code
__global__ void __launch_bounds__(128) nf4_expand_kernel(const uint4* q, const float* sc, int64_t K, int64_t N, bf16* dst,
                                                         int64_t ld, ColMap cm, uint8_t* codes_out) {
  const int g = blockIdx.x, kb = blockIdx.y;
  const int KB = (int)(K / 64);
  const uint32_t* tile = reinterpret_cast<const uint32_t*>(q + ((int64_t)g * KB + kb) * 128);
  for (int e = threadIdx.x; e < 64 * 64; e += 128) {
    const int kk = e >> 6, nn = e & 63;
    int i, lane, word, nib;
    tile_pos(kk, nn, i, lane, word, nib);
    const int code = (tile[(i * 32 + lane) * 4 + word] >> (4 * nib)) & 15;
    const int64_t k = (int64_t)kb * 64 + kk, n = (int64_t)g * 64 + nn;
    if (codes_out) codes_out[k * N + n] = (uint8_t)code;
    else dst[k * ld + map_col(cm, n)] = __float2bfloat16_rn(kNf4[code] * sc[(int64_t)g * K + k]);
  }
}

constexpr int GW = 8;      // warps per CTA
constexpr int XS_LD = 72;  // bf16 elements per staged row: 144 bytes keeps ldmatrix free of bank conflicts

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

template <int MT>
__global__ void __launch_bounds__(GW * 32, 2) nf4_gemv_kernel(const uint4* __restrict__ q, const float* __restrict__ sc,
                                                              const bf16* __restrict__ x, int64_t ldx, int M, int64_t K,
                                                              int64_t N, int kb_per_cta, float* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* lut = reinterpret_cast<uint32_t*>(smem);                      // [256 byte values][32 lanes]
  bf16* xs_all = reinterpret_cast<bf16*>(smem + 256 * 32 * 4);            // [GW][2][16*MT][XS_LD]
  constexpr int XT = 16 * MT * XS_LD;                                     // elements of one staged tile
  float* ss_all = reinterpret_cast<float*>(smem + 256 * 32 * 4 + (size_t)GW * 2 * XT * sizeof(bf16));  // [GW][2][64] scales
  const int split = blockIdx.y, G = (int)(N / 64);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (int)(K / 64);
  const int kb0 = split * kb_per_cta, kb1 = min(KB, kb0 + kb_per_cta);
  const int per = (max(kb1 - kb0, 0) + GW - 1) / GW;
  const int wk0 = min(kb1, kb0 + warp * per), wk1 = min(kb1, wk0 + per);

  // pair table: entry e = (level[e & 15], level[e >> 4]) as bf16x2, one copy per lane (bank = lane)
  for (int idx = threadIdx.x; idx < 256 * 8; idx += GW * 32) {  // 16 bytes = four lanes' copies per store
    const int e = idx >> 3;
    const uint32_t v = (uint32_t)kNf4Bf16[e & 15] | ((uint32_t)kNf4Bf16[e >> 4] << 16);
    reinterpret_cast<uint4*>(lut)[idx] = make_uint4(v, v, v, v);
  }
  bool first = true;
  // a CTA walks the column groups blockIdx.x, blockIdx.x + gridDim.x, ...: the table is built once
  for (int g = blockIdx.x; g < G; g += gridDim.x) {
  const uint4* qp = q + ((int64_t)g * KB) * 128 + lane;
  uint4 qv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) qv[i] = make_uint4(0, 0, 0, 0);
  if (wk0 < wk1) {  // the weights do not depend on the previous kernel: fetch before waiting for it
#pragma unroll
    for (int i = 0; i < 4; ++i) qv[i] = qp[(int64_t)wk0 * 128 + i * 32];
  }
  if (first) {
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();
    first = false;
  }

  float acc[MT][8][4];
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[a][j][e] = 0.f;

  bf16* xs = xs_all + (size_t)warp * 2 * XT;
  float* ss = ss_all + (size_t)warp * 2 * 64;
  // this warp copies its own activation tile (16*MT rows of 128 bytes) and its group's 64 scales
  auto stage = [&](int kb, int buf) {
#pragma unroll
    for (int e = lane; e < 16 * MT * 8; e += 32) {
      const int row = e >> 3, seg = e & 7;
      const bf16* src = x + (int64_t)min(row, M - 1) * ldx + (int64_t)kb * 64 + seg * 8;
      cp_async16(smem_u32(xs + (size_t)buf * XT + row * XS_LD + seg * 8), src, row < M ? 16 : 0);  // rows >= M: zeros
    }
    if (lane < 16) cp_async16(smem_u32(ss + buf * 64 + lane * 4), sc + (int64_t)g * K + (int64_t)kb * 64 + lane * 4, 16);
  };
  if (wk0 < wk1) stage(wk0, 0);
  cp_async_commit();
  const unsigned char* lut_bytes = reinterpret_cast<const unsigned char*>(lut);
  const uint32_t lane4 = (uint32_t)lane * 4;
  const int t = lane & 3;
  for (int kb = wk0; kb < wk1; ++kb) {
    const int buf = (kb - wk0) & 1;
    const bool more = kb + 1 < wk1;
    if (more) stage(kb + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();  // everything but the tile just requested has landed
    __syncwarp();
    const bf16* xt = xs + (size_t)buf * XT;
    // scales for the four k16 steps: rows 2t, 2t+1 and 2t+8, 2t+9 as bf16 pairs
    uint32_t spair[4][2];
    {
      const float* sp = ss + buf * 64 + 2 * t;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = *reinterpret_cast<const float2*>(sp + 16 * i);
        const float2 b = *reinterpret_cast<const float2*>(sp + 16 * i + 8);
        spair[i][0] = pack_bf16(a.x, a.y);
        spair[i][1] = pack_bf16(b.x, b.y);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t af[MT][4];
#pragma unroll
      for (int a = 0; a < MT; ++a) {
        const int arow = a * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, acol = 16 * i + (lane >> 4) * 8;
        ldmatrix_x4(af[a][0], af[a][1], af[a][2], af[a][3], smem_u32(xt + arow * XS_LD + acol));
      }
      const uint32_t words[4] = {qv[i].x, qv[i].y, qv[i].z, qv[i].w};
      // the codes of this step are in `words`: refill the register with the same step of the next block
      if (more) qv[i] = qp[(int64_t)(kb + 1) * 128 + i * 32];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t u = words[w];
        // byte b of the word = one B register.  Pair e of this lane's table copy sits at byte offset
        // e * 128 + lane * 4: a shift, one (x & mask) | lane4, one LDS.
        const uint32_t o0 = ((u << 7) & 0x7F80u) | lane4, o1 = ((u >> 1) & 0x7F80u) | lane4;
        const uint32_t o2 = ((u >> 9) & 0x7F80u) | lane4, o3 = ((u >> 17) & 0x7F80u) | lane4;
        const uint32_t b00 = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o0), spair[i][0]);
        const uint32_t b01 = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o1), spair[i][1]);
        const uint32_t b10 = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o2), spair[i][0]);
        const uint32_t b11 = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o3), spair[i][1]);
#pragma unroll
        for (int a = 0; a < MT; ++a) {
          mma_bf16_16816(acc[a][2 * w], af[a], b00, b01);
          mma_bf16_16816(acc[a][2 * w + 1], af[a], b10, b11);
        }
      }
    }
    __syncwarp();  // all lanes are done with this tile before it is overwritten two iterations on
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its staging area: reuse it for the reduction
  float* red = reinterpret_cast<float*>(xs_all);  // [GW][16*MT][64]
  const int c = lane >> 2;
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float* rp = red + ((size_t)warp * 16 * MT + a * 16 + c) * 64 + 8 * j + 2 * t;
      *reinterpret_cast<float2*>(rp) = make_float2(acc[a][j][0], acc[a][j][1]);
      *reinterpret_cast<float2*>(rp + 8 * 64) = make_float2(acc[a][j][2], acc[a][j][3]);
    }
  __syncthreads();
  float* op = out + (int64_t)split * M * N + (int64_t)g * 64;
  for (int e = threadIdx.x; e < 16 * MT * 16; e += GW * 32) {  // float4 per thread
    const int m = e >> 4, n4 = (e & 15) * 4;
    if (m >= M) continue;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < GW; ++w) {
      const float4 v = *reinterpret_cast<const float4*>(red + ((size_t)w * 16 * MT + m) * 64 + n4);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    *reinterpret_cast<float4*>(op + (int64_t)m * N + n4) = s;
  }
  __syncthreads();  // the reduction area is staging area again
  }  // column groups
}

template <int MT>
constexpr size_t gemv_smem() {
  return 256 * 32 * 4 + (size_t)GW * 2 * 16 * MT * XS_LD * sizeof(bf16) + (size_t)GW * 2 * 64 * sizeof(float);
}

}  // namespace

int nf4_alloc(Ctx* c, int64_t K, int64_t N, Nf4W* w) {
  (void)c;
  RB_REQUIRE(K > 0 && N > 0 && K % 64 == 0 && N % 64 == 0, "NF4 weights need in and out features that are multiples of 64");
  w->K = K;
  w->N = N;
  RB_CUDA(cudaMalloc((void**)&w->q, (size_t)K * N / 2));
  RB_CUDA(cudaMalloc((void**)&w->sc, (size_t)K * (N / 64) * sizeof(float)));
  return REWB200_OK;
}

void nf4_free(Nf4W* w) {
  if (w->q) cudaFree(w->q);
  if (w->sc) cudaFree(w->sc);
  w->q = nullptr;
  w->sc = nullptr;
}

int nf4_quantize_launch(Ctx* c, const void* src, int src_dtype, int64_t ld, ColMap cm, const Nf4W& w) {
  const dim3 grid((unsigned)(w.N / 64), (unsigned)(w.K / 64));
  if (src_dtype == REWB200_BF16)
    nf4_quantize_kernel<bf16><<<grid, 64, 0, c->stream>>>((const bf16*)src, ld, cm, w.q, w.sc, w.K, w.N);
  else if (src_dtype == REWB200_F32)
    nf4_quantize_kernel<float><<<grid, 64, 0, c->stream>>>((const float*)src, ld, cm, w.q, w.sc, w.K, w.N);
  else
    return fail("nf4 quantise: weights must be f32 or bf16");
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

int nf4_dequant_launch(Ctx* c, const Nf4W& w, bf16* dst, int64_t ld, ColMap cm) {
  const dim3 grid((unsigned)(w.N / 64), (unsigned)(w.K / 64));
  nf4_expand_kernel<<<grid, 128, 0, c->stream>>>(w.q, w.sc, w.K, w.N, dst, ld, cm, nullptr);
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

int nf4_codes_launch(Ctx* c, const Nf4W& w, uint8_t* codes) {
  const dim3 grid((unsigned)(w.N / 64), (unsigned)(w.K / 64));
  ColMap cm{w.N, w.N, w.N, 0};
  nf4_expand_kernel<<<grid, 128, 0, c->stream>>>(w.q, w.sc, w.K, w.N, nullptr, 0, cm, codes);
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

// CTAs along K: each of a CTA's 8 warps should own about 4 blocks of 64 rows, but the grid should
// still cover the GPU about twice.  (Fewer, longer-lived CTAs walking several column groups measured
// slower: the drain and refill of the per-warp pipeline at every group costs more than the table build.)
int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N) {
  const int groups = (int)(N / 64), KB = (int)(K / 64);
  int ks = std::max(1, KB / (GW * 4));
  while (ks < KB / GW && groups * ks < 2 * c->sm_count) ++ks;
  return std::max(1, std::min(ks, KB));
}

int nf4_gemv_launch(Ctx* c, const Nf4W& w, const bf16* x, int64_t ldx, int64_t M, int ksplit, float* out) {
  RB_REQUIRE(M >= 1 && M <= 32, "nf4 GEMV handles 1 to 32 rows");
  RB_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "nf4 GEMV needs 16-byte aligned activation rows");
  const int KB = (int)(w.K / 64);
  ksplit = std::max(1, std::min(ksplit, KB));
  const int per = (KB + ksplit - 1) / ksplit;
  // one CTA per (column group, K slice); the kernel also accepts fewer CTAs than groups
  const dim3 grid((unsigned)(w.N / 64), (unsigned)ksplit);
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemv_smem<1>()));
    RB_CUDA(cudaFuncSetAttribute(nf4_gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemv_smem<2>()));
    attr_set = true;
  }
  if (M <= 16)
    RB_CUDA(launch_k(nf4_gemv_kernel<1>, grid, dim3(GW * 32), gemv_smem<1>(), c->stream, c->use_pdl, (const uint4*)w.q,
                     (const float*)w.sc, x, ldx, (int)M, w.K, w.N, per, out));
  else
    RB_CUDA(launch_k(nf4_gemv_kernel<2>, grid, dim3(GW * 32), gemv_smem<2>(), c->stream, c->use_pdl, (const uint4*)w.q,
                     (const float*)w.sc, x, ldx, (int)M, w.K, w.N, per, out));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace rewb

// ---- C ABI: QloraLinear on packed weights ------------------------------------------------------

struct rewb200_nf4 {
  int slot = 0;
  rewb::Nf4W w;
};

namespace rewb {
namespace {

// xa[m][r] = sum_k x[m][k] * A[r][k]   (x @ A^T, lora.nim:421-422); one warp per (m, r)
__global__ void lora_xa_kernel(const bf16* x, int64_t ldx, const float* A, int64_t M, int64_t K, int rank, float* xa) {
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= M * rank) return;
  const int64_t m = wid / rank, r = wid % rank;
  float s = 0.f;
  for (int64_t k = lane; k < K; k += 32) s += __bfloat162float(x[m * ldx + k]) * A[r * K + k];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) xa[wid] = s;
}

// y = sum of the split-K slabs + bias + scaling * (xa @ B^T)   (lora.nim:418-428)
__global__ void qlora_finish_kernel(const float* part, int ksplit, int64_t M, int64_t N, const float* bias, const float* xa,
                                    const float* B, int rank, float scaling, bf16* y) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  const int64_t m = i / N, n = i % N;
  float v = 0.f;
  for (int s = 0; s < ksplit; ++s) v += part[(int64_t)s * M * N + i];
  if (bias) v += bias[n];
  if (xa) {
    float dlt = 0.f;
    for (int r = 0; r < rank; ++r) dlt += xa[m * rank + r] * B[n * rank + r];
    v += scaling != 1.0f ? dlt * scaling : dlt;
  }
  y[i] = __float2bfloat16_rn(v);
}

}  // namespace
}  // namespace rewb

extern "C" {

using namespace rewb;

int rewb200_nf4_pack(const rewb200_buffer* w, rewb200_nf4** out) {
  RB_REQUIRE(w && out, "rewb200_nf4_pack: NULL argument");
  RB_REQUIRE(w->ndims == 2, "initQloraLinearFromF32: weight must be [inFeatures, outFeatures]");
  RB_REQUIRE(w->dtype == REWB200_F32 || w->dtype == REWB200_BF16, "rewb200_nf4_pack: weight must be f32 or bf16");
  Ctx* c = ctx_get(w->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  rewb200_nf4* h = new rewb200_nf4();
  h->slot = w->slot;
  int st = nf4_alloc(c, w->dims[0], w->dims[1], &h->w);
  if (st == REWB200_OK) st = nf4_quantize_launch(c, w->ptr, w->dtype, w->dims[1], ColMap{w->dims[1], w->dims[1], w->dims[1], 0}, h->w);
  if (st != REWB200_OK) {
    nf4_free(&h->w);
    delete h;
    return st;
  }
  *out = h;
  return REWB200_OK;
}

void rewb200_nf4_free(rewb200_nf4* h) {
  if (!h) return;
  Ctx* c = ctx_get(h->slot);
  if (c) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
  }
  nf4_free(&h->w);
  delete h;
}

int rewb200_nf4_info(const rewb200_nf4* h, int64_t* in_features, int64_t* out_features) {
  RB_REQUIRE(h, "rewb200_nf4_info: NULL handle");
  if (in_features) *in_features = h->w.K;
  if (out_features) *out_features = h->w.N;
  return REWB200_OK;
}

int rewb200_nf4_unpack(const rewb200_nf4* h, uint8_t* packed, float* scales) {
  RB_REQUIRE(h && packed && scales, "rewb200_nf4_unpack: NULL argument");
  Ctx* c = ctx_get(h->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t K = h->w.K, N = h->w.N, G = N / 64;
  uint8_t* d_codes = nullptr;
  RB_CUDA(cudaMalloc((void**)&d_codes, (size_t)K * N));
  int st = nf4_codes_launch(c, h->w, d_codes);
  std::vector<uint8_t> codes((size_t)K * N);
  std::vector<float> sc((size_t)K * G);
  if (st == REWB200_OK) {
    cudaError_t e = cudaMemcpyAsync(codes.data(), d_codes, codes.size(), cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(sc.data(), h->w.sc, sc.size() * sizeof(float), cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) st = fail(std::string("rewb200_nf4_unpack: ") + cudaGetErrorString(e));
  }
  cudaFree(d_codes);
  RB_TRY(st);
  // the reference's order: two codes per byte along the flat [in, out] index, one scale per flat block
  for (int64_t i = 0; i < K * N; i += 2) packed[i / 2] = (uint8_t)(codes[i] | (codes[i + 1] << 4));
  for (int64_t k = 0; k < K; ++k)
    for (int64_t g = 0; g < G; ++g) scales[k * G + g] = sc[g * K + k];
  return REWB200_OK;
}

int rewb200_nf4_dequantize(const rewb200_nf4* h, rewb200_buffer** w_out) {
  RB_REQUIRE(h && w_out, "rewb200_nf4_dequantize: NULL argument");
  Ctx* c = ctx_get(h->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t dims[2] = {h->w.K, h->w.N};
  rewb200_buffer* b = nullptr;
  RB_TRY(buffer_new(c, REWB200_BF16, dims, 2, &b));
  b->slot = h->slot;
  int st = nf4_dequant_launch(c, h->w, (bf16*)b->ptr, h->w.N, ColMap{h->w.N, h->w.N, h->w.N, 0});
  if (st != REWB200_OK) {
    rewb200_buffer_release(b);
    return st;
  }
  *w_out = b;
  return REWB200_OK;
}

int rewb200_qlora_linear(const rewb200_buffer* x, const rewb200_nf4* h, const rewb200_buffer* bias, const rewb200_buffer* A,
                         const rewb200_buffer* B, float scaling, rewb200_buffer** y) {
  RB_REQUIRE(x && h && y, "rewb200_qlora_linear: NULL argument");
  RB_REQUIRE(x->dtype == REWB200_BF16, "rewb200_qlora_linear: activations must be bf16");
  RB_REQUIRE(x->ndims >= 1 && x->dims[x->ndims - 1] == h->w.K,
             "QloraLinear.forward: last dimension " + std::to_string(x->ndims ? x->dims[x->ndims - 1] : 0) +
                 " does not match inFeatures " + std::to_string(h->w.K));
  RB_REQUIRE(x->slot == h->slot, "rewb200_qlora_linear: operands live on different devices");
  const int64_t K = h->w.K, N = h->w.N, M = x->numel() / K;
  int rank = 0;
  if (A || B) {
    RB_REQUIRE(A && B && A->dtype == REWB200_F32 && B->dtype == REWB200_F32 && A->ndims == 2 && B->ndims == 2,
               "rewb200_qlora_linear: A [rank,in] and B [out,rank] must both be f32 matrices");
    rank = (int)A->dims[0];
    RB_REQUIRE(A->dims[1] == K && B->dims[0] == N && B->dims[1] == rank, "rewb200_qlora_linear: LoRA factor shapes do not match");
  }
  if (bias) RB_REQUIRE(bias->dtype == REWB200_F32 && bias->numel() == N, "rewb200_qlora_linear: bias must be f32 [out]");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  int64_t dims[8];
  for (int i = 0; i < x->ndims; ++i) dims[i] = x->dims[i];
  dims[x->ndims - 1] = N;
  rewb200_buffer* out = nullptr;
  RB_TRY(buffer_new(c, REWB200_BF16, dims, x->ndims, &out));
  out->slot = x->slot;
  if (M == 0) {
    *y = out;
    return REWB200_OK;
  }
  const int ks = nf4_pick_ksplit(c, K, N);
  float *part = nullptr, *xa = nullptr;
  cudaError_t e = cudaMalloc((void**)&part, (size_t)ks * 32 * N * sizeof(float));
  if (e == cudaSuccess && rank > 0) e = cudaMalloc((void**)&xa, (size_t)M * rank * sizeof(float));
  int st = e == cudaSuccess ? REWB200_OK : fail(std::string("rewb200_qlora_linear: ") + cudaGetErrorString(e));
  if (st == REWB200_OK && rank > 0) {
    const int64_t threads = M * rank * 32;
    lora_xa_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, c->stream>>>((const bf16*)x->ptr, K, (const float*)A->ptr, M, K,
                                                                            rank, xa);
    ++g_launch_total;
  }
  for (int64_t m0 = 0; m0 < M && st == REWB200_OK; m0 += 32) {
    const int64_t rows = std::min<int64_t>(32, M - m0);
    st = nf4_gemv_launch(c, h->w, (const bf16*)x->ptr + m0 * K, K, rows, ks, part);
    if (st != REWB200_OK) break;
    const int64_t n = rows * N;
    qlora_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(
        part, ks, rows, N, bias ? (const float*)bias->ptr : nullptr, rank > 0 ? xa + m0 * rank : nullptr,
        rank > 0 ? (const float*)B->ptr : nullptr, rank, scaling, (bf16*)out->ptr + m0 * N);
    ++g_launch_total;
  }
  if (st == REWB200_OK) {
    e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) st = fail(std::string("rewb200_qlora_linear: ") + cudaGetErrorString(e));
  }
  if (part) cudaFree(part);
  if (xa) cudaFree(xa);
  if (st != REWB200_OK) {
    rewb200_buffer_release(out);
    return st;
  }
  *y = out;
  return ctx_check_status(c);
}

}  // extern "C"
