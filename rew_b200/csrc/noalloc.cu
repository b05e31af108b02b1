// rewb200_linear_noalloc: the decode-size bf16 Linear for callers that cannot
// allocate device memory.  The GEMM is the kernel the slot's "linear" option
// selects for rewb200_linear too: the tcgen05 weight streamer of linear_tc.cu by
// default, the mma.sync one of linear_bf16.cu under linear=mma; both leave f32
// split-K slabs that a small kernel here sums.
//
// Who that is: a host runtime that has handed the whole device heap to its own
// allocator (for example a serving process that reserves all free HBM for KV
// pages at start-up), and code running in a latency-critical section where the
// device-wide synchronisation cudaMalloc / cudaFree imply is not acceptable.
// For them this entry point touches no allocator at all: the split-K partial
// sums, which the other entry points keep in pool memory, live in a fixed
// array that is part of the library image.
//
// Cost and limits: the array is kNoAllocScratchBytes (8 MiB) of device memory
// on every GPU that loads the library, held until the process exits.  A call
// needs ksplit * M * N * 4 bytes of it and is rejected when even ksplit = 1 does
// not fit.  All calls share the one array and it keeps the previous call's
// contents; nothing has to be cleared because every slab entry a call reads
// was written by that same call's GEMM first.  Two calls that overlap on the
// GPU (different streams or slots of one device) would race on it; calls on
// one slot are ordered by the slot's stream and are safe.
#include "common.cuh"
#include "ptx.cuh"

namespace rewb {
namespace {

constexpr size_t kNoAllocScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Host-side cache of the array's device address, per device ordinal, filled by
// noalloc_setup under rewb200_init's lock.  The symbol's name is only a host
// stand-in; kernels must be given this address.
float* g_scratch_addr[64] = {nullptr};

__global__ void __launch_bounds__(256) sum_partials_kernel(const float* __restrict__ part, int nsplit, int64_t slab,
                                                           const float* __restrict__ bias, bf16* __restrict__ y,
                                                           int64_t M, int64_t N) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  float acc = 0.f;
  for (int s = 0; s < nsplit; ++s) acc += part[s * slab + i];
  if (bias) acc += bias[i % N];
  y[i] = __float2bfloat16_rn(acc);
}

int scratch_address(Ctx* c, float** out) {
  RB_REQUIRE(c->device >= 0 && c->device < 64 && g_scratch_addr[c->device] != nullptr,
             "rewb200_linear_noalloc: the scratch array was not resolved for this device (rewb200_init does that)");
  *out = g_scratch_addr[c->device];
  return REWB200_OK;
}

}  // namespace

int linear_tc_preload();
int linear_bf16_preload();

// Called by rewb200_init for every device it opens, with that device current.  CUDA loads modules
// lazily: the first cudaGetSymbolAddress of the array and the first launch of a kernel load the module
// that holds them, and loading the module with the 8 MiB array allocates device memory inside the driver.
// All of that happens here, so that no call of rewb200_linear_noalloc loads code or reserves memory.
int noalloc_setup(Ctx* c) {
  RB_REQUIRE(c->device >= 0 && c->device < 64, "device ordinal out of range");
  void* p = nullptr;
  RB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
  RB_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null address for the scratch array");
  g_scratch_addr[c->device] = (float*)p;
  cudaFuncAttributes fa;
  RB_CUDA(cudaFuncGetAttributes(&fa, sum_partials_kernel));
  RB_TRY(linear_tc_preload());
  RB_TRY(linear_bf16_preload());
  return REWB200_OK;
}

}  // namespace rewb

using namespace rewb;

// y[M,N] (bf16) = x[M,K] (bf16) @ w[K,N] (bf16) + bias[N] (f32, may be NULL).
// All pointers are device pointers the caller owns; M <= 32.
// rewb200_init has resolved the scratch array's address (cudaGetSymbolAddress,
// with the device current) and loaded the kernels used here, so no call loads a
// module; no cudaMalloc, cudaFree, pool or library allocation happens in any call.
extern "C" int rewb200_linear_noalloc(int slot, const void* x, const void* w, const float* bias, void* y, int64_t M,
                                      int64_t K, int64_t N) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(x && w && y, "rewb200_linear_noalloc: NULL pointer");
  RB_REQUIRE(M >= 1 && M <= 32 && K >= 1 && N >= 1, "rewb200_linear_noalloc: needs 1 <= M <= 32 and positive K, N");
  RB_REQUIRE(K % 8 == 0 && N % 8 == 0, "rewb200_linear_noalloc: K and N must be multiples of 8 (16-byte TMA rows)");
  RB_CUDA(cudaSetDevice(c->device));
  const size_t slab_bytes = (size_t)M * N * sizeof(float);
  RB_REQUIRE(slab_bytes <= kNoAllocScratchBytes,
             "rewb200_linear_noalloc: M*N*4 = " + std::to_string(slab_bytes) + " bytes exceeds the fixed scratch of " +
                 std::to_string(kNoAllocScratchBytes) + " bytes; use rewb200_linear for this size");
  float* scratch = nullptr;
  RB_TRY(scratch_address(c, &scratch));
  int ks = linear_bf16_pick_ksplit(c, M, K, N);
  while (ks > 1 && (size_t)ks * slab_bytes > kNoAllocScratchBytes) ks /= 2;
  LinearBf16Plan plan;
  RB_TRY(linear_bf16_plan(&plan, (const bf16*)w, K, N, 0));
  RB_TRY(linear_bf16_launch(c, plan, (const bf16*)x, K, M, EPI_PARTIAL_F32, ks, scratch, N, nullptr, nullptr, 0));
  const int64_t n = M * N;
  sum_partials_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(scratch, ks, M * N, bias, (bf16*)y, M, N);
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}
