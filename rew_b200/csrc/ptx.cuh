// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor,
// never with cluster multicast), ldmatrix, mma.sync, programmatic dependent
// launch.  Every wait is bounded: after kSpinLimit polls the waiter records an
// error code in a status word and gives up, so a kernel can never hang the GPU.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rewb {

constexpr uint32_t kSpinLimit = 1u << 24;  // ~ a second of polling at most

enum KernelStatus : int {
  KS_OK = 0,
  KS_MBAR_TIMEOUT = 1,
  KS_BAD_INDEX = 2,
  KS_TMEM_TIMEOUT = 3,
  KS_PEER_TIMEOUT = 4,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false (and records KS_MBAR_TIMEOUT) if the phase never completed.
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// The bound is both an iteration count and ~2 s of wall time (try_wait may
// itself block for an implementation-defined slice).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 127u) == 127u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) break;
    }
  }
  if (status) atomicExch(status, KS_MBAR_TIMEOUT);
  return false;
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2D tiled load, global -> this CTA's shared memory, completion on an mbarrier.
// x (innermost coordinate) * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const void* tmap, uint64_t* bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y),
      "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(void* dst, const void* tmap, uint64_t* bar, int x, int y, int z,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "l"(policy)
      : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue early / wait until every prior kernel's writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- flags between the ranks of a node (peer heap) ------------------------------------------------
// Writer: every thread of the CTA has issued its stores into the peer's memory; after the CTA barrier
// the flag store (release, system scope) orders them before the flag.  Reader: polls a cell of its OWN
// memory with acquire loads.  Flag values only grow; `v - target >= 0` also accepts a later round.
__device__ __forceinline__ void peer_flag_release(int* cell, int value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(cell), "r"(value) : "memory");
}
__device__ __forceinline__ int peer_flag_acquire(const int* cell) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(cell) : "memory");
  return v;
}
// Threads 0..n-1 (except `skip`) each wait for one cell; bounded by 2 s, and cut short once any wait on
// this GPU has already timed out, so a lost peer costs one timeout per step and never a hang.  Ends with a
// CTA barrier: afterwards every thread may read what the peers stored before raising their flags.
__device__ __forceinline__ void peer_flags_wait(const int* cells, int stride, int n, int skip, int target, int* status) {
  if ((int)threadIdx.x < n && (int)threadIdx.x != skip) {
    const int* cell = cells + (int64_t)threadIdx.x * stride;
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
      if (peer_flag_acquire(cell) - target >= 0) break;
      if ((it & 63u) == 63u) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > 2000000000ull || *reinterpret_cast<volatile int*>(status) == KS_PEER_TIMEOUT) {
          atomicExch(status, KS_PEER_TIMEOUT);
          break;
        }
      }
    }
  }
  __syncthreads();
}

// Last CTA of a grid to arrive (every CTA calls this exactly once, after its peer stores): returns true in all
// threads of that CTA.  The fence before the arrival makes the CTA's stores visible system-wide first; the
// counter is left at zero for the next launch.
__device__ __forceinline__ bool grid_last_cta(int* arrive) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int t = atomicAdd(arrive, 1);
    s_last = (t == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) ? 1 : 0;
    if (s_last) {
      __threadfence_system();
      *arrive = 0;
    }
  }
  __syncthreads();
  return s_last != 0;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One RoPE pair (v0, v1) -> (c v0 - s v1, s v0 + c v1) with a fixed rounding sequence (one product rounded, then one
// fused multiply-add).  Left to the compiler, the contraction can differ from kernel to kernel; with this, every
// kernel that rotates q / k returns the same bits.
__device__ __forceinline__ float rope_even(float c, float s, float v0, float v1) { return __fmaf_rn(c, v0, -__fmul_rn(s, v1)); }
__device__ __forceinline__ float rope_odd(float c, float s, float v0, float v1) { return __fmaf_rn(s, v0, __fmul_rn(c, v1)); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a TMA box whose rows
// are 128 bytes and which was written with CU_TENSOR_MAP_SWIZZLE_128B (box base
// aligned to 1024 bytes).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace rewb
