// Weight-only NF4 Linear: the frozen base projection of QloraLinear (src/rew/nn/lora.nim:410-431) with
// the weights kept in their 4-bit codes in HBM and dequantised inside the GEMV, instead of the
// reference's dequantise-once-on-the-host-then-fp32-matmul (lora.nim:347-349).
//
// Codec as src/rew/quantize/codecs.nim:13-70: blocks of 64 consecutive elements of the flat row-major
// [in, out] weight (= 64 consecutive output features of one input row when out % 64 == 0), scale =
// max(1e-10, absmax), code = nearest of the 16 NF4 levels (first one on a tie), value = level * scale.
//
// Device layout (this library's own; rewb200_nf4_unpack gives back the reference's bytes):
//   q  [N/64][K/64][4 warps][32 lanes] uint4   one 16-byte load per lane and 64 input rows: word i is
//        k16 step i; nibble j*4+r of a word is W[k][n] with k = 16 i + {2t, 2t+1, 2t+8, 2t+9}[r],
//        n = 64 g + 16 warp + 8 j + lane/4, t = lane % 4 -- exactly the B fragment of mma.m16n8k16
//   sc [N/64][K] f32                           the scales of one 64-column group, contiguous along k
// GEMV (rows <= 32): CTA = one 64-column group x a slice of K; the scale depends on (k, group), so it
// is folded into the ACTIVATIONS of the CTA (x'[m][k] = x[m][k] * sc[g][k], staged in shared memory)
// and the B operand is the bare NF4 level, looked up with byte permutes: three PRMT per byte plane
// (levels 0-7, levels 8-15, select by bit 3) for four codes at once.  f32 accumulation, split-K
// partials [ksplit][M][N] summed by the consumer as for the bf16 Linear.
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

__device__ __forceinline__ int64_t map_col(const ColMap& cm, int64_t n) {
  const int64_t seg = n / cm.seg_len, within = n % cm.seg_len;
  return (within / cm.gran) * cm.gstride + (within % cm.gran) + seg * cm.seg_off;
}

// grid (N/64, K/64), 64 threads: thread r quantises row kb*64 + r of the group, then the tile is packed.
template <typename T>
__global__ void __launch_bounds__(64) nf4_quantize_kernel(const T* src, int64_t ld, ColMap cm, uint4* q, float* sc, int64_t K,
                                                          int64_t N) {
  __shared__ uint8_t codes[64][64 + 4];
  const int g = blockIdx.x, kb = blockIdx.y, r = threadIdx.x;
  const int64_t k = (int64_t)kb * 64 + r;
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
    codes[r][n] = (uint8_t)code;
  }
  __syncthreads();
  const int KB = (int)(K / 64);
  for (int pair = threadIdx.x; pair < 128; pair += 64) {
    const int warp = pair >> 5, lane = pair & 31, t = lane & 3, c = lane >> 2;
    uint32_t words[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t u = 0;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          const int kk = 16 * i + 2 * t + (rr & 1) + ((rr >> 1) ? 8 : 0);
          const int nn = 16 * warp + 8 * j + c;
          u |= (uint32_t)codes[kk][nn] << (4 * (j * 4 + rr));
        }
      words[i] = u;
    }
    q[(((int64_t)g * KB + kb) * 4 + warp) * 32 + lane] = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// mode 0: dst (bf16, column-mapped) = level * scale; mode 1: dst (uint8 [K][N]) = code
__global__ void __launch_bounds__(128) nf4_expand_kernel(const uint4* q, const float* sc, int64_t K, int64_t N, bf16* dst,
                                                         int64_t ld, ColMap cm, uint8_t* codes_out) {
  const int g = blockIdx.x, kb = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = lane & 3, c = lane >> 2;
  const int KB = (int)(K / 64);
  const uint4 qv = q[(((int64_t)g * KB + kb) * 4 + warp) * 32 + lane];
  const uint32_t words[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        const int code = (words[i] >> (4 * (j * 4 + rr))) & 15;
        const int64_t k = (int64_t)kb * 64 + 16 * i + 2 * t + (rr & 1) + ((rr >> 1) ? 8 : 0);
        const int64_t n = (int64_t)g * 64 + 16 * warp + 8 * j + c;
        if (codes_out) codes_out[k * N + n] = (uint8_t)code;
        else dst[k * ld + map_col(cm, n)] = __float2bfloat16_rn(kNf4[code] * sc[(int64_t)g * K + k]);
      }
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// bf16 bit patterns of the 16 levels, split into a low-byte and a high-byte plane of four words each
// (levels 0-3, 4-7, 8-11, 12-15): bf16(-1) = 0xBF80, bf16(-0.6962) = 0xBF32, ...
struct Nf4Planes {
  uint32_t lo[4], hi[4];
};
__host__ __device__ constexpr uint16_t nf4_bf16_bits(int i) {
  // round-to-nearest-even bf16 of the table, written out so that host and device agree
  constexpr uint16_t bits[16] = {0xBF80, 0xBF32, 0xBF06, 0xBECA, 0xBE92, 0xBE3D, 0xBDBA, 0x0000,
                                 0x3DA3, 0x3E25, 0x3E7C, 0x3EAD, 0x3EE2, 0x3F10, 0x3F39, 0x3F80};
  return bits[i];
}
__device__ __forceinline__ Nf4Planes nf4_planes() {
  Nf4Planes p;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      lo |= (uint32_t)(nf4_bf16_bits(4 * w + b) & 0xFF) << (8 * b);
      hi |= (uint32_t)(nf4_bf16_bits(4 * w + b) >> 8) << (8 * b);
    }
    p.lo[w] = lo;
    p.hi[w] = hi;
  }
  return p;
}

// Four codes (the low 16 bits of q16, code r in nibble r) -> two bf16x2 registers
// (level[r0] | level[r1] << 16, level[r2] | level[r3] << 16).
__device__ __forceinline__ void nf4_lookup4(uint32_t q16, const Nf4Planes& p, uint32_t& r01, uint32_t& r23) {
  const uint32_t s7 = q16 & 0x7777u;                        // index within a half of the table
  const uint32_t pick = ((q16 >> 1) & 0x4444u) | 0x3210u;   // byte i from the low (bit 3 = 0) or the high half
  const uint32_t lo = prmt(prmt(p.lo[0], p.lo[1], s7), prmt(p.lo[2], p.lo[3], s7), pick);
  const uint32_t hi = prmt(prmt(p.hi[0], p.hi[1], s7), prmt(p.hi[2], p.hi[3], s7), pick);
  r01 = prmt(lo, hi, 0x5140u);
  r23 = prmt(lo, hi, 0x7362u);
}

constexpr int XS_LD = 72;  // bf16 elements per staged row: 144 bytes keeps ldmatrix free of bank conflicts

template <int MT>
__global__ void __launch_bounds__(128) nf4_gemv_kernel(const uint4* __restrict__ q, const float* __restrict__ sc,
                                                       const bf16* __restrict__ x, int64_t ldx, int M, int64_t K, int64_t N,
                                                       int kb_per_split, float* __restrict__ out) {
  __shared__ __align__(16) bf16 xs[2][16 * MT][XS_LD];
  const int g = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (int)(K / 64);
  const int kb0 = split * kb_per_split, kb1 = min(KB, kb0 + kb_per_split);
  const uint4* qp = q + (((int64_t)g * KB) * 4 + warp) * 32 + lane;
  const Nf4Planes planes = nf4_planes();
  float acc[MT][2][4];
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[a][j][e] = 0.f;

  // the weights do not depend on the previous kernel: start fetching before waiting for it
  uint4 qv = make_uint4(0, 0, 0, 0);
  if (kb0 < kb1) qv = qp[(int64_t)kb0 * 128];
  pdl_launch_dependents();
  pdl_wait();

  // staging role: 16*MT rows x 64 k, 16 consecutive k per thread
  const int srow = threadIdx.x >> 2, sseg = (threadIdx.x & 3) * 16;
  for (int kb = kb0; kb < kb1; ++kb) {
    const int buf = (kb - kb0) & 1;
    uint4 qn = make_uint4(0, 0, 0, 0);
    if (kb + 1 < kb1) qn = qp[(int64_t)(kb + 1) * 128];
    for (int row = srow; row < 16 * MT; row += 32) {
      uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
      const int64_t k0 = (int64_t)kb * 64 + sseg;
      if (row < M) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + (int64_t)row * ldx + k0);
        xa = xp[0];
        xb = xp[1];
      }
      const float4* sp = reinterpret_cast<const float4*>(sc + (int64_t)g * K + k0);
      const float4 s0 = sp[0], s1 = sp[1], s2 = sp[2], s3 = sp[3];
      const float sv[16] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w, s2.x, s2.y, s2.z, s2.w, s3.x, s3.y, s3.z, s3.w};
      const uint32_t xin[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
      uint32_t xo[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float lo = __uint_as_float(xin[e] << 16) * sv[2 * e];
        const float hi = __uint_as_float(xin[e] & 0xFFFF0000u) * sv[2 * e + 1];
        xo[e] = pack_bf16(lo, hi);
      }
      uint4* dp = reinterpret_cast<uint4*>(&xs[buf][row][sseg]);
      dp[0] = make_uint4(xo[0], xo[1], xo[2], xo[3]);
      dp[1] = make_uint4(xo[4], xo[5], xo[6], xo[7]);
    }
    __syncthreads();
    const uint32_t words[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t b[2][2];
      nf4_lookup4(words[i], planes, b[0][0], b[0][1]);
      nf4_lookup4(words[i] >> 16, planes, b[1][0], b[1][1]);
#pragma unroll
      for (int a = 0; a < MT; ++a) {
        uint32_t af[4];
        const int arow = a * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, acol = 16 * i + (lane >> 4) * 8;
        ldmatrix_x4(af[0], af[1], af[2], af[3], smem_u32(&xs[buf][arow][acol]));
        mma_bf16_16816(acc[a][0], af, b[0][0], b[0][1]);
        mma_bf16_16816(acc[a][1], af, b[1][0], b[1][1]);
      }
    }
    qv = qn;
  }
  const int t = lane & 3, c = lane >> 2;
  float* op = out + (int64_t)split * M * N;
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t n = (int64_t)g * 64 + 16 * warp + 8 * j + 2 * t;
      const int m0 = a * 16 + c, m1 = m0 + 8;
      if (m0 < M) *reinterpret_cast<float2*>(op + (int64_t)m0 * N + n) = make_float2(acc[a][j][0], acc[a][j][1]);
      if (m1 < M) *reinterpret_cast<float2*>(op + (int64_t)m1 * N + n) = make_float2(acc[a][j][2], acc[a][j][3]);
    }
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

int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N) {
  const int groups = (int)(N / 64), KB = (int)(K / 64);
  int ks = (c->sm_count * 6 + groups - 1) / groups;
  ks = std::max(1, std::min(ks, std::max(1, KB / 4)));
  return ks;
}

int nf4_gemv_launch(Ctx* c, const Nf4W& w, const bf16* x, int64_t ldx, int64_t M, int ksplit, float* out) {
  RB_REQUIRE(M >= 1 && M <= 32, "nf4 GEMV handles 1 to 32 rows");
  RB_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "nf4 GEMV needs 16-byte aligned activation rows");
  const int KB = (int)(w.K / 64);
  ksplit = std::max(1, std::min(ksplit, KB));
  const int per = (KB + ksplit - 1) / ksplit;
  const dim3 grid((unsigned)(w.N / 64), (unsigned)ksplit);
  if (M <= 16)
    RB_CUDA(launch_k(nf4_gemv_kernel<1>, grid, dim3(128), 0, c->stream, c->use_pdl, (const uint4*)w.q, (const float*)w.sc, x, ldx,
                     (int)M, w.K, w.N, per, out));
  else
    RB_CUDA(launch_k(nf4_gemv_kernel<2>, grid, dim3(128), 0, c->stream, c->use_pdl, (const uint4*)w.q, (const float*)w.sc, x, ldx,
                     (int)M, w.K, w.N, per, out));
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
