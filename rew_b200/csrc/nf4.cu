// Weight-only NF4 Linear: the frozen base projection of QloraLinear (src/rew/nn/lora.nim:410-431) with
// the weights kept in their 4-bit codes in HBM and dequantised inside the GEMV, instead of the
// reference's dequantise-once-on-the-host-then-fp32-matmul (lora.nim:347-349).
//
// Codec as src/rew/quantize/codecs.nim:13-70: blocks of 64 consecutive elements of the flat row-major
// [in, out] weight (= 64 consecutive output features of one input row when out % 64 == 0), scale =
// max(1e-10, absmax), code = nearest of the 16 NF4 levels (first one on a tie), value = level * scale.
//
// Device layout (this library's own; rewb200_nf4_unpack gives back the reference's bytes):
//   q   [ceil(N/128)][K/64][128 features][32 bytes]  the 64 codes of one feature and one block of 64 input
//         rows, byte j = (code of row 2j) | (code of row 2j+1) << 4; features past N hold code 7 (= 0.0)
//   sc  [N/64][K] f32      the scales of one 64-feature group, contiguous along k
//   sc2 [N/64][K/2] u32    the same scales as bf16 pairs (rows 2j, 2j+1): what the GEMV multiplies by
// GEMV (rows <= 32) on the 5th-generation tensor core with the WEIGHT operand in tensor memory:
//   D[128 features][32 tokens] (TMEM, f32) += A[128 features][64 k] (TMEM, bf16) * B[64 k][32 tokens] (smem)
//   warp 0      TMA producer, two rings: 14 stages of the tile's 4 KB of codes + the scale pairs of its two
//               groups (bulk copies out of HBM, 56 KB in flight per CTA), 4 stages of the activation tile
//               (32 tokens x 64 k, 128-byte swizzle, out of L2)
//   warp 1      one thread issues four tcgen05.mma (K = 16 each) per block of 64 rows, A read from TMEM
//   warps 2-9   dequantisers: a warp owns the 32 TMEM lanes (features) of its lane quarter and every
//               other block; a lane reads its feature's 32 code bytes from the stage, turns each byte into a bf16 pair
//               with ONE conflict-free LDS from a shared-memory pair table (one copy per lane), multiplies
//               by the scale pair (HMUL2) and stores its 32 columns with one tcgen05.st into one of four
//               A buffers.  The dequantised weights never touch shared memory.
//   epilogue    warps 2-5 read D (tcgen05.ld) and store the f32 split-K slab [ksplit][M][N]
// (Two earlier versions fed mma.sync from registers: byte-permute lookups saturated the half-rate
// integer pipe at 0.17 of the HBM roofline; the pair table with per-warp cp.async staging reached 0.22.
// A variant of this kernel with 512 features per CTA, i.e. four times the codes in flight, was slower.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <string>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"
#include "tc.cuh"

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

// byte offset of the pair byte of W[k][n] inside q
__device__ __forceinline__ int64_t code_byte(int64_t k, int64_t n, int64_t KB) {
  return (((n >> 7) * KB + (k >> 6)) * 128 + (n & 127)) * 32 + ((k & 63) >> 1);
}

// grid (N/64, K/64), 64 threads: thread r quantises the 64 features of group g for input row kb*64 + r.
template <typename T>
__global__ void __launch_bounds__(64) nf4_quantize_kernel(const T* src, int64_t ld, ColMap cm, uint8_t* q, float* sc,
                                                          uint32_t* sc2, int64_t K, int64_t N) {
  __shared__ uint8_t codes[64][64 + 4];  // [row][feature]
  __shared__ float srow[64];
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
  srow[r] = absMax;
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
  const int64_t KB = K / 64;
  // thread r now packs feature r: 32 bytes, two rows per byte
  const int64_t n = (int64_t)g * 64 + r;
  uint32_t words[8];
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    uint32_t u = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int j = 4 * w + b;
      u |= (uint32_t)(codes[2 * j][r] | (codes[2 * j + 1][r] << 4)) << (8 * b);
    }
    words[w] = u;
  }
  uint4* dst = reinterpret_cast<uint4*>(q + code_byte((int64_t)kb * 64, n, KB));
  dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
  dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
  if (r < 32) sc2[(int64_t)g * (K / 2) + (int64_t)kb * 32 + r] = pack_bf16(srow[2 * r], srow[2 * r + 1]);
}

// dst (bf16, column-mapped) = level * scale, or codes_out (uint8 [K][N]) = code
__global__ void __launch_bounds__(128) nf4_expand_kernel(const uint8_t* q, const float* sc, int64_t K, int64_t N, bf16* dst,
                                                         int64_t ld, ColMap cm, uint8_t* codes_out) {
  const int g = blockIdx.x, kb = blockIdx.y;
  const int64_t KB = K / 64;
  for (int e = threadIdx.x; e < 64 * 64; e += 128) {
    const int kk = e >> 6, nn = e & 63;
    const int64_t k = (int64_t)kb * 64 + kk, n = (int64_t)g * 64 + nn;
    const int code = (q[code_byte(k, n, KB)] >> (4 * (kk & 1))) & 15;
    if (codes_out) codes_out[k * N + n] = (uint8_t)code;
    else dst[k * ld + map_col(cm, n)] = __float2bfloat16_rn(kNf4[code] * sc[(int64_t)g * K + k]);
  }
}

constexpr int NT_XST = 4;                    // activation stages: they come out of L2, a short ring is enough
constexpr int NT_CST = 14;                   // code stages: 56 KB of packed weights in flight per CTA hide the HBM latency
constexpr int NT_XBYTES = 32 * 128;          // activations of a block: 32 tokens x 64 k bf16 (128-byte swizzle)
constexpr int NT_CBYTES = 128 * 32;          // codes of a block: 128 features x 32 bytes
constexpr int NT_SBYTES = 2 * 32 * 4;        // scale pairs of a block: 2 groups x 32 pairs
constexpr int NT_CSTAGE = NT_CBYTES + NT_SBYTES;   // code stage = codes | scale pairs
constexpr int NT_DEQ = 8;                    // dequantiser warps
constexpr int NT_THREADS = (2 + NT_DEQ) * 32;
constexpr int NT_ABUF = 4;                   // weight-operand buffers in tensor memory
constexpr int NT_TMEM_COLS = 256;            // D: columns 0-31; A buffer b: columns 32 + 32 b .. +31
constexpr int NT_LUT_BYTES = 256 * 32 * 4;
constexpr int NT_SMEM = NT_XST * NT_XBYTES + NT_CST * NT_CSTAGE + NT_LUT_BYTES + 512 + 1024;

__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

__global__ void __launch_bounds__(NT_THREADS) nf4_tc_kernel(const __grid_constant__ CUtensorMap tmX, const uint8_t* __restrict__ q,
                                                            const uint32_t* __restrict__ sc2, int M, int64_t K, int64_t N,
                                                            int kb_per_split, float* __restrict__ out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* xs = smem;                                                    // [NT_XST] activation tiles
  uint8_t* cs = smem + NT_XST * NT_XBYTES;                               // [NT_CST]{codes | scale pairs}
  uint32_t* lut = reinterpret_cast<uint32_t*>(cs + NT_CST * NT_CSTAGE);  // [256 byte values][32 lanes]
  uint64_t* x_full = reinterpret_cast<uint64_t*>(lut + 256 * 32);
  uint64_t* x_empty = x_full + NT_XST;
  uint64_t* c_full = x_empty + NT_XST;      // [NT_CST]
  uint64_t* c_empty = c_full + NT_CST;      // [NT_CST]
  uint64_t* a_full = c_empty + NT_CST;      // [NT_ABUF]
  uint64_t* a_empty = a_full + NT_ABUF;     // [NT_ABUF]
  uint64_t* d_full = a_empty + NT_ABUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int KB = (int)(K / 64);
  const int kb0 = split * kb_per_split;
  const int nkb = max(0, min(kb_per_split, KB - kb0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < NT_XST; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&x_empty[s], 1);
    }
    for (int s = 0; s < NT_CST; ++s) {
      mbar_init(&c_full[s], 1);
      mbar_init(&c_empty[s], 4);  // the four lane quarters of the parity that dequantises the block
    }
    for (int b = 0; b < NT_ABUF; ++b) {
      mbar_init(&a_full[b], 4);   // the four lane quarters
      mbar_init(&a_empty[b], 1);
    }
    mbar_init(d_full, 1);
    fence_barrier_init();
    pdl_launch_dependents();
  }
  if (warp == 1) tc::alloc(tmem_slot, NT_TMEM_COLS);
  // pair table: entry e = (level[e & 15], level[e >> 4]) as bf16x2, one copy per lane (bank = lane)
  for (int idx = threadIdx.x; idx < 256 * 8; idx += NT_THREADS) {
    const int e = idx >> 3;
    const uint32_t v = (uint32_t)kNf4Bf16[e & 15] | ((uint32_t)kNf4Bf16[e >> 4] << 16);
    reinterpret_cast<uint4*>(lut)[idx] = make_uint4(v, v, v, v);
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      const uint64_t pol_x = policy_evict_last();
      // Two rings.  Codes (4 KB per block, plain bulk copy) and the scale pairs of the tile's two
      // 64-feature groups come from HBM: 14 stages, 56 KB in flight per CTA.  The activation tile of a
      // block (tensor copy) comes out of L2: 4 stages.  Codes and scales do not depend on the previous
      // kernel: the first ring-full is requested before waiting for it.
      const int64_t g0 = ((int64_t)tile * 128) >> 6, G = N >> 6;
      auto load_codes = [&](int kb) {
        const int s = kb % NT_CST;
        uint8_t* st = cs + s * NT_CSTAGE;
        mbar_expect_tx(&c_full[s], NT_CSTAGE);
        bulk_load_1d(st, q + ((int64_t)tile * KB + kb0 + kb) * NT_CBYTES, NT_CBYTES, &c_full[s]);
        for (int h = 0; h < 2; ++h) {
          const int64_t g = min(g0 + h, G - 1);  // a half tile past N re-reads the last group (its lanes are never stored)
          bulk_load_1d(st + NT_CBYTES + h * 128, sc2 + g * (K / 2) + (int64_t)(kb0 + kb) * 32, 128, &c_full[s]);
        }
      };
      auto load_x = [&](int kb) {
        const int s = kb % NT_XST;
        mbar_expect_tx(&x_full[s], NT_XBYTES);
        tma_load_2d_hint(xs + s * NT_XBYTES, &tmX, &x_full[s], (kb0 + kb) * 64, 0, pol_x);
      };
      for (int kb = 0; kb < min(NT_CST, nkb); ++kb) load_codes(kb);
      pdl_wait();  // the activations come from the previous kernel
      for (int kb = 0; kb < min(NT_XST, nkb); ++kb) load_x(kb);
      // block t, once consumed, frees the activation slot of block t + NT_XST and the code slot of t + NT_CST
      for (int t = 0; t < nkb; ++t) {
        const int xk = t + NT_XST, ck = t + NT_CST;
        if (xk >= nkb && ck >= nkb) break;
        if (xk < nkb) {
          if (!mbar_wait(&x_empty[xk % NT_XST], ((xk / NT_XST) - 1) & 1, status)) break;
          load_x(xk);
        }
        if (ck < nkb) {
          if (!mbar_wait(&c_empty[ck % NT_CST], ((ck / NT_CST) - 1) & 1, status)) break;
          load_codes(ck);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
      // instruction descriptor: D f32, A and B bf16, both K-major (A lives in tensor memory), N = 32, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(32 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t xs_addr = smem_u32(xs);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int p = kb % NT_ABUF, s = kb % NT_XST;
        ok = mbar_wait(&a_full[p], (kb / NT_ABUF) & 1, status) && mbar_wait(&x_full[s], (kb / NT_XST) & 1, status);
        if (!ok) break;
        tc::fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t db = tc::smem_desc(xs_addr + s * NT_XBYTES + kk * 32, 16, 1024);
          tc::umma_bf16_ta(tmem_base, tmem_base + 32 + p * 32 + kk * 8, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
        }
        tc::commit(&x_empty[s]);
        tc::commit(&a_empty[p]);
      }
      if (ok) tc::commit(d_full);
    }
  } else {
    // ---------------- dequantisers: lane quarter = warp % 4 (the TMEM lanes a warp may touch), parity = which blocks
    const int dw = warp - 2, p = dw >> 2, quarter = warp & 3;
    const int64_t n_feat = (int64_t)tile * 128 + quarter * 32 + lane;
    const bool valid = (int64_t)tile * 128 + quarter * 32 < N;  // N % 64 == 0: a quarter is all in or all out
    const uint8_t* lut_bytes = reinterpret_cast<const uint8_t*>(lut);
    const uint32_t lane4 = (uint32_t)lane * 4;
    const uint32_t a_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + 32;
    bool ok = true;
    for (int kb = p; kb < nkb; kb += 2) {
      const int s = kb % NT_CST, ab = kb % NT_ABUF, use = kb / NT_ABUF;
      if (ok) ok = mbar_wait(&c_full[s], (kb / NT_CST) & 1, status);
      const uint8_t* st = cs + s * NT_CSTAGE;
      const uint4* cp = reinterpret_cast<const uint4*>(st + (quarter * 32 + lane) * 32);
      const uint4 qa = cp[0], qb = cp[1];
      const uint4* sp4 = reinterpret_cast<const uint4*>(st + NT_CBYTES + (quarter >> 1) * 128);
      const uint32_t words[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      uint32_t r[32];
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const uint4 s4 = sp4[w];  // the same address for every lane: a broadcast
        const uint32_t u = words[w];
        // pair e of this lane's table copy sits at byte offset e * 128 + lane * 4
        const uint32_t o0 = ((u << 7) & 0x7F80u) | lane4, o1 = ((u >> 1) & 0x7F80u) | lane4;
        const uint32_t o2 = ((u >> 9) & 0x7F80u) | lane4, o3 = ((u >> 17) & 0x7F80u) | lane4;
        r[4 * w + 0] = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o0), s4.x);
        r[4 * w + 1] = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o1), s4.y);
        r[4 * w + 2] = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o2), s4.z);
        r[4 * w + 3] = hmul2_bf16(*reinterpret_cast<const uint32_t*>(lut_bytes + o3), s4.w);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&c_empty[s]);  // codes and scales are in registers: the stage may be refilled
      if (use >= 1 && ok) {  // the tensor core must have consumed this buffer's previous contents
        ok = mbar_wait(&a_empty[ab], (use - 1) & 1, status);
        tc::fence_after();
      }
      if (valid) tc::st32(a_lane + ab * 32, r);
      tc::fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[ab]);
    }
    if (p == 0) {
      // ---------------- epilogue: D[feature = lane][token = column] -> out[split][token][feature]
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
      if (nkb > 0) {
        ok = mbar_wait(d_full, 0, status) && ok;
        ok = __all_sync(0xffffffffu, ok);  // the load below is warp-collective
        tc::fence_after();
        if (ok) tc::ld32(tmem_base + ((uint32_t)(quarter * 32) << 16), r);
      }
      pdl_wait();  // the slab buffer may still be read by the previous kernel
      if (valid && ok) {
        float* op = out + (int64_t)split * M * N + n_feat;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < M) op[(int64_t)j * N] = __uint_as_float(r[j]);
      }
    }
  }
  tc::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::dealloc(tmem_base, NT_TMEM_COLS);
  }
}

}  // namespace

int nf4_alloc(Ctx* c, int64_t K, int64_t N, Nf4W* w) {
  (void)c;
  RB_REQUIRE(K > 0 && N > 0 && K % 64 == 0 && N % 64 == 0, "NF4 weights need in and out features that are multiples of 64");
  w->K = K;
  w->N = N;
  const int64_t tiles = (N + 127) / 128;
  RB_CUDA(cudaMalloc((void**)&w->q, (size_t)tiles * 128 * K / 2));
  RB_CUDA(cudaMemset(w->q, 0x77, (size_t)tiles * 128 * K / 2));  // code 7 = 0.0 for the features past N
  RB_CUDA(cudaMalloc((void**)&w->sc, (size_t)K * (N / 64) * sizeof(float)));
  RB_CUDA(cudaMalloc((void**)&w->sc2, (size_t)(K / 2) * (N / 64) * sizeof(uint32_t)));
  return REWB200_OK;
}

void nf4_free(Nf4W* w) {
  if (w->q) cudaFree(w->q);
  if (w->sc) cudaFree(w->sc);
  if (w->sc2) cudaFree(w->sc2);
  w->q = nullptr;
  w->sc = nullptr;
  w->sc2 = nullptr;
}

int nf4_quantize_launch(Ctx* c, const void* src, int src_dtype, int64_t ld, ColMap cm, const Nf4W& w) {
  const dim3 grid((unsigned)(w.N / 64), (unsigned)(w.K / 64));
  if (src_dtype == REWB200_BF16)
    nf4_quantize_kernel<bf16><<<grid, 64, 0, c->stream>>>((const bf16*)src, ld, cm, w.q, w.sc, w.sc2, w.K, w.N);
  else if (src_dtype == REWB200_F32)
    nf4_quantize_kernel<float><<<grid, 64, 0, c->stream>>>((const float*)src, ld, cm, w.q, w.sc, w.sc2, w.K, w.N);
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

// CTAs along K: two CTAs fit an SM; fill those slots once (a second, partial wave costs a whole CTA
// lifetime) and keep at least 4 blocks of 64 rows per CTA.
// ---- GEMV for one to four rows on the CUDA cores ---------------------------------------------------------
// With so few rows the tensor core has nothing to do and the kernel is a stream of codes: 0.5 byte per weight
// against 2 for bf16, so the instruction count per code byte is what matters.  A CTA owns 128 features and a
// range of 64-row blocks; thread t owns feature t and reads its 32 code bytes of a block with two 16-byte
// loads (consecutive threads, consecutive 32 bytes: the tile's 4 KB are one contiguous run); the next block's
// codes are requested before this block's are consumed.  A code byte (two weights) costs one lookup in a
// 256-entry table of fp16 level PAIRS (eight copies side by side, so that lanes rarely share a bank) and one HFMA2 per row with the
// matching pair of activations, which are staged once per block already multiplied by the group's scales
// (xs[row][j] = (x[2j] * s[2j], x[2j+1] * s[2j+1]) as fp16).  The 32 products of a block are summed in fp16
// and the block sums in f32, which keeps the rounding error of the sum at the 1e-3 level; fp16's range holds
// activations up to ~6e4 / scale.  Output: the same f32 split-K slabs [ksplit][M][N] the tensor-core kernel
// leaves.
template <int MR>
__global__ void __launch_bounds__(128) nf4_gemv_small_kernel(const uint8_t* __restrict__ q, const float* __restrict__ sc,
                                                             const bf16* __restrict__ x, int64_t ldx, int M, int64_t K,
                                                             int64_t N, int kb_per_split, float* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t nf4s_smem[];
  __half2* tab = reinterpret_cast<__half2*>(nf4s_smem);                         // [256][8]: eight copies, lane & 7 picks one
  __half2* xs = reinterpret_cast<__half2*>(nf4s_smem + 256 * 8 * 4);            // [2 buffers][2 groups][MR][32]
  pdl_launch_dependents();
  const int tile = blockIdx.x, split = blockIdx.y, t = threadIdx.x, lane = t & 31;
  const int KB = (int)(K / 64);
  const int kb0 = split * kb_per_split;
  const int nkb = max(0, min(kb_per_split, KB - kb0));
  for (int i = t; i < 256 * 8; i += 128) {
    const int byte = i >> 3;
    tab[i] = __floats2half2_rn(kNf4[byte & 15], kNf4[byte >> 4]);
  }
  const int cp = lane & 7;
  const uint4* qp = reinterpret_cast<const uint4*>(q) + (((int64_t)tile * KB + kb0) * 128 + t) * 2;
  uint4 c0 = make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u), c1 = c0, n0 = c0, n1 = c0, m0 = c0, m1 = c0;  // code 7 = 0.0
  if (nkb > 0) {  // the weights do not depend on the previous kernel: three blocks are requested before the wait
    c0 = __ldcs(qp);
    c1 = __ldcs(qp + 1);
  }
  if (nkb > 1) {
    n0 = __ldcs(qp + 256);
    n1 = __ldcs(qp + 257);
  }
  pdl_wait();
  // staging: thread t prepares pair (t & 31) of group (t >> 5) & 1 for rows (t >> 6), (t >> 6) + 2
  const int sg = (t >> 5) & 1, sj = t & 31, sm0 = t >> 6;
  const int64_t sgi = (int64_t)tile * 2 + sg;
  const bool sg_ok = sgi * 64 < N;
  // Staging is software-pipelined: the scales and activations of block kb + 2 are requested while block kb is
  // consumed and written to shared memory one iteration later, so no iteration waits for a global load.
  constexpr int SL = (MR + 1) / 2;  // rows this thread stages
  float2 s2_reg = make_float2(0.f, 0.f);
  uint32_t x_reg[SL];
  auto fetch = [&](int kb) {
    const int64_t k = (int64_t)(kb0 + kb) * 64 + 2 * sj;
    s2_reg = sg_ok ? *reinterpret_cast<const float2*>(sc + sgi * K + k) : make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < SL; ++i) {
      const int m = sm0 + 2 * i;
      x_reg[i] = (m < M && m < MR) ? *reinterpret_cast<const uint32_t*>(x + (int64_t)m * ldx + k) : 0u;
    }
  };
  auto put = [&](int buf) {
#pragma unroll
    for (int i = 0; i < SL; ++i) {
      const int m = sm0 + 2 * i;
      if (m < MR) {
        const __nv_bfloat162 xb = *reinterpret_cast<const __nv_bfloat162*>(&x_reg[i]);
        xs[((buf * 2 + sg) * MR + m) * 32 + sj] = __floats2half2_rn(__low2float(xb) * s2_reg.x, __high2float(xb) * s2_reg.y);
      }
    }
  };
  float acc[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) acc[m] = 0.f;
  if (nkb > 0) {
    fetch(0);
    put(0);
  }
  if (nkb > 1) fetch(1);
  __syncthreads();
  const int g = t >> 6;
  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 2 < nkb) {
      m0 = __ldcs(qp + (int64_t)(kb + 2) * 256);
      m1 = __ldcs(qp + (int64_t)(kb + 2) * 256 + 1);
    }
    if (kb + 1 < nkb) put(buf ^ 1);     // block kb + 1, requested one iteration ago
    if (kb + 2 < nkb) fetch(kb + 2);
    const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    __half2 hs[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) hs[m] = __float2half2_rn(0.f);
    const __half2* xg = xs + (buf * 2 + g) * MR * 32;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) {
      __half2 lv[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) lv[b] = tab[((w[wi] >> (8 * b)) & 0xFFu) * 8 + cp];
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xg + m * 32 + 4 * wi);  // the pairs of rows 8wi .. 8wi+7
        hs[m] = __hfma2(lv[0], *reinterpret_cast<const __half2*>(&xv.x), hs[m]);
        hs[m] = __hfma2(lv[1], *reinterpret_cast<const __half2*>(&xv.y), hs[m]);
        hs[m] = __hfma2(lv[2], *reinterpret_cast<const __half2*>(&xv.z), hs[m]);
        hs[m] = __hfma2(lv[3], *reinterpret_cast<const __half2*>(&xv.w), hs[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      const float2 f = __half22float2(hs[m]);
      acc[m] += f.x + f.y;
    }
    __syncthreads();  // xs[buf] is free again and xs[buf ^ 1] is complete
    c0 = n0;
    c1 = n1;
    n0 = m0;
    n1 = m1;
  }
  const int64_t n = (int64_t)tile * 128 + t;
  if (n < N)
    for (int m = 0; m < M && m < MR; ++m) out[((int64_t)split * M + m) * N + n] = acc[m];
}

template <int MR>
constexpr int nf4_small_smem() { return 256 * 8 * 4 + 2 * 2 * MR * 32 * 4; }

constexpr int kNf4SmallRows = 4;

int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N);

int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N, int64_t M) {
  if (M <= kNf4SmallRows && c->nf4_small) {  // many small CTAs (8 per SM resident): about eight waves' worth keeps the stream smooth
    const int tiles = (int)((N + 127) / 128), KB = (int)(K / 64);
    int ks = std::max(1, 8 * c->sm_count / tiles);
    ks = std::min(ks, std::max(1, KB / 4));  // at least four blocks per CTA: the table and pipeline start-up are per CTA
    return std::max(1, std::min(ks, 16));
  }
  return nf4_pick_ksplit(c, K, N);
}

int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N) {
  const int tiles = (int)((N + 127) / 128), KB = (int)(K / 64), slots = 2 * c->sm_count;
  int ks = std::max(1, slots / tiles);
  ks = std::min(ks, std::max(1, KB / 4));
  return std::max(1, std::min(ks, 16));
}

int nf4_gemv_launch(Ctx* c, const Nf4W& w, const bf16* x, int64_t ldx, int64_t M, int ksplit, float* out) {
  RB_REQUIRE(M >= 1 && M <= 32, "nf4 GEMV handles 1 to 32 rows");
  RB_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "nf4 GEMV needs 16-byte aligned activation rows");
  const int KB = (int)(w.K / 64);
  ksplit = std::max(1, std::min(ksplit, KB));
  const int per = (KB + ksplit - 1) / ksplit;
  const dim3 grid((unsigned)((w.N + 127) / 128), (unsigned)ksplit);
  if (M <= kNf4SmallRows && c->nf4_small) {
    static bool small_attr = false;
    if (!small_attr) {
      RB_CUDA(cudaFuncSetAttribute(nf4_gemv_small_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, nf4_small_smem<1>()));
      RB_CUDA(cudaFuncSetAttribute(nf4_gemv_small_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, nf4_small_smem<2>()));
      RB_CUDA(cudaFuncSetAttribute(nf4_gemv_small_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, nf4_small_smem<4>()));
      small_attr = true;
    }
#define RB_NF4S(MR)                                                                                                    \
  RB_CUDA(launch_k(nf4_gemv_small_kernel<MR>, grid, dim3(128), (size_t)nf4_small_smem<MR>(), c->stream, c->use_pdl,    \
                   (const uint8_t*)w.q, (const float*)w.sc, x, ldx, (int)M, w.K, w.N, per, out))
    if (M == 1) RB_NF4S(1);
    else if (M == 2) RB_NF4S(2);
    else RB_NF4S(4);
#undef RB_NF4S
    ++g_launch_total;
    return REWB200_OK;
  }
  CUtensorMap tmX;
  RB_TRY(make_tmap_2d_bf16(&tmX, x, (uint64_t)w.K, (uint64_t)M, (uint64_t)ldx * 2, 64, 32));
  static bool attr_set = false;
  if (!attr_set) {
    RB_CUDA(cudaFuncSetAttribute(nf4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, NT_SMEM));
    RB_CUDA(cudaFuncSetAttribute(nf4_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    attr_set = true;
  }
  RB_CUDA(launch_k(nf4_tc_kernel, grid, dim3(NT_THREADS), (size_t)NT_SMEM, c->stream, c->use_pdl, tmX, (const uint8_t*)w.q,
                   (const uint32_t*)w.sc2, (int)M, w.K, w.N, per, out, c->d_status));
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
  const int ks = nf4_pick_ksplit(c, K, N, std::min<int64_t>(M, 32));
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
