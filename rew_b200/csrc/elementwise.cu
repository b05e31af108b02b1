// Row-wise kernels between the GEMMs of a decoder block, each replacing a chain
// of single-op dispatches in the reference:
//   residual_norm  : split-K / tensor-parallel partial sum + bias + residual add
//                    + rmsNorm (src/rew/nn/norm.nim:204-224) or LayerNorm
//                    (src/rew/nn/norm.nim:41-84); or embedding row gather
//                    (src/rew/nn/embedding.nim:39-62) + norm for the first layer.
//   qkv_post       : partial sum + bias + interleaved-pair RoPE from the host
//                    tables (src/rew/nn/rope.nim:56-108,153-179) + KV-cache append
//                    (src/rew/nn/kv_cache.nim:47-77) written straight into pages.
//   argmax         : sampleGreedy, first maximum (src/rew/infer/generate.nim:152-159).
#include <math.h>

#include <algorithm>

#include <cooperative_groups.h>

#include "common.cuh"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace rewb {

int64_t g_launch_total = 0;

namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_PER_THREAD = 64;  // d <= 16384

template <typename TE, typename TO>
__global__ void __launch_bounds__(NORM_THREADS) residual_norm_kernel(NormArgs a) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int64_t d = a.d;
  float vals[NORM_MAX_PER_THREAD];
  int cnt = 0;
  float* xr = a.x_res + row * d;
  const TE* erow = nullptr;
  if (a.embed) {
    int64_t id = row;  // without ids the table is read row by row (a plain typed input)
    if (a.ids) {
      id = a.ids[row];
      if (id < 0 || id >= a.vocab) {
        if (threadIdx.x == 0) atomicExch(a.status, KS_BAD_INDEX);
        id = 0;
      }
    }
    erow = reinterpret_cast<const TE*>(a.embed) + id * d;
  }
  for (int64_t i = threadIdx.x; i < d; i += NORM_THREADS, ++cnt) {
    float v = erow ? to_f<TE>(erow[i]) : xr[i];  // x_res is required when there is no table
    if (a.partial) {
      float p = 0.f;
      for (int s = 0; s < a.nsplit; ++s) p += a.partial[s * a.split_stride + row * d + i];
      if (a.bias) p += a.bias[i];
      v += p;
    }
    vals[cnt] = v;
    if (a.x_res && (erow || a.partial)) xr[i] = v;
  }
  if (a.norm_kind < 0) return;
  TO* orow = reinterpret_cast<TO*>(a.out) + row * d;
  if (a.norm_kind == 0) {
    float ss = 0.f;
    for (int k = 0; k < cnt; ++k) ss += vals[k] * vals[k];
    ss = block_sum(ss, red);
    const float rms = sqrtf(ss / (float)d + a.eps);
    cnt = 0;
    for (int64_t i = threadIdx.x; i < d; i += NORM_THREADS, ++cnt)
      orow[i] = from_f<TO>(a.gamma[i] * (vals[cnt] / rms));
  } else {
    float s1 = 0.f;
    for (int k = 0; k < cnt; ++k) s1 += vals[k];
    const float mean = block_sum(s1, red) / (float)d;
    float s2 = 0.f;
    for (int k = 0; k < cnt; ++k) {
      const float c = vals[k] - mean;
      s2 += c * c;
    }
    const float var = block_sum(s2, red) / (float)d;
    const float inv = 1.0f / sqrtf(var + a.eps);
    cnt = 0;
    for (int64_t i = threadIdx.x; i < d; i += NORM_THREADS, ++cnt)
      orow[i] = from_f<TO>(a.gamma[i] * ((vals[cnt] - mean) * inv) + a.beta[i]);
  }
}

// Vectorised variant for d % 4 == 0: 512 threads, each owning NCH float4 chunks
// held in registers; the split-K slab loads of a chunk are independent and
// issued together, so the kernel is bound by L2 bandwidth, not by a chain of
// dependent loads.
constexpr int NORMV_THREADS = 512;

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    uint2 u;
    u.x = pack_bf16(v.x, v.y);
    u.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

// Sum of the split-K slabs at element offset `idx` (a multiple of 4), in slab order.
__device__ __forceinline__ float4 partial_sum4(const NormArgs& a, int64_t idx) {
  float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
  if (a.partial_bf16) {
    const bf16* pp = reinterpret_cast<const bf16*>(a.partial) + idx;
    for (int s = 0; s < a.nsplit; ++s) {
      const uint2 u = __ldcg(reinterpret_cast<const uint2*>(pp + s * a.split_stride));  // may have been written by a peer
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
      p.x += __low2float(lo); p.y += __high2float(lo); p.z += __low2float(hi); p.w += __high2float(hi);
    }
    return p;
  }
  const float* pp = a.partial + idx;
  if (a.wait_n > 0) return __ldcg(reinterpret_cast<const float4*>(pp));  // one slab, written by the peers
  int s = 0;
  for (; s + 4 <= a.nsplit; s += 4) {
    const float4 p0 = *reinterpret_cast<const float4*>(pp + (s + 0) * a.split_stride);
    const float4 p1 = *reinterpret_cast<const float4*>(pp + (s + 1) * a.split_stride);
    const float4 p2 = *reinterpret_cast<const float4*>(pp + (s + 2) * a.split_stride);
    const float4 p3 = *reinterpret_cast<const float4*>(pp + (s + 3) * a.split_stride);
    p.x += p0.x; p.y += p0.y; p.z += p0.z; p.w += p0.w;
    p.x += p1.x; p.y += p1.y; p.z += p1.z; p.w += p1.w;
    p.x += p2.x; p.y += p2.y; p.z += p2.z; p.w += p2.w;
    p.x += p3.x; p.y += p3.y; p.z += p3.z; p.w += p3.w;
  }
  for (; s < a.nsplit; ++s) {
    const float4 p0 = *reinterpret_cast<const float4*>(pp + s * a.split_stride);
    p.x += p0.x; p.y += p0.y; p.z += p0.z; p.w += p0.w;
  }
  return p;
}

// One 16-byte line of the one-shot exchange: two 4-byte payload words, each followed by the flag of this
// all-reduce ({w0, flag, w1, flag}).  A line is stored with one 16-byte store; should the link split it, each
// 8-byte half still carries its own flag, so a reader that sees both flags has both words.
__device__ __forceinline__ void ll_store(void* line, uint32_t w0, uint32_t w1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(line), "r"(w0), "r"(flag), "r"(w1), "r"(flag) : "memory");
}
// Polls a line of this GPU's own memory until both flags match; bounded by 2 s, and cut short once any wait
// on this GPU has already timed out.
__device__ __forceinline__ uint2 ll_poll(const void* line, uint32_t flag, int* status) {
  uint32_t x, fx, y, fy;
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(fx), "=r"(y), "=r"(fy) : "l"(line) : "memory");
    if (fx == flag && fy == flag) break;
    if ((it & 255u) == 255u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > 2000000000ull || *reinterpret_cast<volatile int*>(status) == KS_PEER_TIMEOUT) {
        atomicExch(status, KS_PEER_TIMEOUT);
        break;
      }
    }
  }
  return make_uint2(x, y);
}

// Tensor-parallel all-reduce of this thread's columns (see NormArgs): p[c] holds this rank's partial of the
// float4 at element offset idx[c] (idx[c] < 0: none) and comes back as the sum over all ranks, added in rank
// order from the values that crossed NVLink, so every rank ends up with the same bits.  Payload and flag
// travel in the same store (no fence, no separate flag round trip): bf16 payload = one line per float4, f32
// payload = two.  The same thread of every rank handles the same columns, so each thread waits only for
// the lines it reads itself.
template <int NCH>
__device__ __forceinline__ void tp_exchange4(const NormArgs& a, float4 (&p)[NCH], const int64_t (&idx)[NCH]) {
  const uint32_t flag = (uint32_t)(*a.epoch + a.barrier_offset);
  const int64_t mine = (int64_t)a.my_rank * a.slot_lines;
  if (a.payload_bf16) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (idx[c] < 0) continue;
      const uint32_t w0 = pack_bf16(p[c].x, p[c].y), w1 = pack_bf16(p[c].z, p[c].w);
      for (int r = 0; r < a.n_peers; ++r)
        if (r != a.my_rank) ll_store(reinterpret_cast<uint4*>(a.peer_buf[r]) + mine + (idx[c] >> 2), w0, w1, flag);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&w0), hi = *reinterpret_cast<const __nv_bfloat162*>(&w1);
      p[c] = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));  // what the peers see
    }
  } else {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (idx[c] < 0) continue;
      for (int r = 0; r < a.n_peers; ++r)
        if (r != a.my_rank) {
          uint4* line = reinterpret_cast<uint4*>(a.peer_buf[r]) + mine + (idx[c] >> 1);
          ll_store(line, __float_as_uint(p[c].x), __float_as_uint(p[c].y), flag);
          ll_store(line + 1, __float_as_uint(p[c].z), __float_as_uint(p[c].w), flag);
        }
    }
  }
  const uint4* local = reinterpret_cast<const uint4*>(a.peer_buf[a.my_rank]);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    if (idx[c] < 0) continue;
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.n_peers; ++r) {
      float4 q = p[c];
      if (r != a.my_rank) {
        if (a.payload_bf16) {
          const uint2 u = ll_poll(local + (int64_t)r * a.slot_lines + (idx[c] >> 2), flag, a.status);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
          q = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
        } else {
          const uint4* line = local + (int64_t)r * a.slot_lines + (idx[c] >> 1);
          const uint2 u0 = ll_poll(line, flag, a.status), u1 = ll_poll(line + 1, flag, a.status);
          q = make_float4(__uint_as_float(u0.x), __uint_as_float(u0.y), __uint_as_float(u1.x), __uint_as_float(u1.y));
        }
      }
      t.x += q.x; t.y += q.y; t.z += q.z; t.w += q.w;
    }
    p[c] = t;
  }
}

// The same all-reduce in two hops (NormArgs::two_shot): the columns of a row are owned by the ranks in blocks of
// d / n_peers.  A thread stores its partial of a float4 to the owner only (slot `my_rank` of the owner's buffer);
// the owner's thread polls the other ranks' partials, adds all of them in rank order and stores the sum into slot
// `my_rank` of every peer (the lines of its own columns, which no partial uses); the other ranks poll that line.
// Same threads handle the same columns on every rank, a thread sends all its partials before its first poll, and
// an owner's polls depend on those sends only, so no wait can depend on itself.  Every rank ends up with the
// owner's value (rounded to the payload type), so ranks stay bit-identical.
template <int NCH>
__device__ __forceinline__ void tp_exchange4_two(const NormArgs& a, float4 (&p)[NCH], const int64_t (&idx)[NCH]) {
  const uint32_t flag = (uint32_t)(*a.epoch + a.barrier_offset);
  const int64_t mine = (int64_t)a.my_rank * a.slot_lines;
  const int64_t dn = a.d / a.n_peers;
  const uint4* local = reinterpret_cast<const uint4*>(a.peer_buf[a.my_rank]);
  const int sh = a.payload_bf16 ? 2 : 1;   // a float4 is one line (bf16) or two (f32)
  auto send = [&](int r, int64_t line, const float4& v) {
    uint4* dst = reinterpret_cast<uint4*>(a.peer_buf[r]) + mine + line;
    if (a.payload_bf16) {
      ll_store(dst, pack_bf16(v.x, v.y), pack_bf16(v.z, v.w), flag);
    } else {
      ll_store(dst, __float_as_uint(v.x), __float_as_uint(v.y), flag);
      ll_store(dst + 1, __float_as_uint(v.z), __float_as_uint(v.w), flag);
    }
  };
  auto recv = [&](int r, int64_t line) -> float4 {
    const uint4* src = local + (int64_t)r * a.slot_lines + line;
    if (a.payload_bf16) {
      const uint2 u = ll_poll(src, flag, a.status);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
      return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
    }
    const uint2 u0 = ll_poll(src, flag, a.status), u1 = ll_poll(src + 1, flag, a.status);
    return make_float4(__uint_as_float(u0.x), __uint_as_float(u0.y), __uint_as_float(u1.x), __uint_as_float(u1.y));
  };
  auto rounded = [&](const float4& v) -> float4 {   // what a value looks like after crossing a link
    if (!a.payload_bf16) return v;
    const uint32_t w0 = pack_bf16(v.x, v.y), w1 = pack_bf16(v.z, v.w);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&w0), hi = *reinterpret_cast<const __nv_bfloat162*>(&w1);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
  };
  int owner[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    owner[c] = -1;
    if (idx[c] < 0) continue;
    owner[c] = (int)((idx[c] % a.d) / dn);
    if (owner[c] != a.my_rank) send(owner[c], idx[c] >> sh, p[c]);
    else p[c] = rounded(p[c]);
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    if (idx[c] < 0) continue;
    const int64_t line = idx[c] >> sh;
    if (owner[c] == a.my_rank) {
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < a.n_peers; ++r) {
        const float4 q = r == a.my_rank ? p[c] : recv(r, line);
        t.x += q.x; t.y += q.y; t.z += q.z; t.w += q.w;
      }
      t = rounded(t);
      for (int r = 0; r < a.n_peers; ++r)
        if (r != a.my_rank) send(r, line, t);
      p[c] = t;
    } else {
      p[c] = recv(owner[c], line);
    }
  }
}

template <typename TE, typename TO, int NCH>
__global__ void __launch_bounds__(NORMV_THREADS) residual_norm_vec_kernel(NormArgs a) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  if (a.wait_n > 0) peer_flags_wait(a.wait_cells, 1, a.wait_n, -1, *a.wait_epoch + a.wait_offset, a.status);
  const int64_t row = blockIdx.x;
  const int64_t d = a.d;
  float* xr = a.x_res + row * d;
  const TE* erow = nullptr;
  if (a.embed) {
    int64_t id = row;
    if (a.ids) {
      id = a.ids[row];
      if (id < 0 || id >= a.vocab) {
        if (threadIdx.x == 0) atomicExch(a.status, KS_BAD_INDEX);
        id = 0;
      }
    }
    erow = reinterpret_cast<const TE*>(a.embed) + id * d;
  }
  float4 vals[NCH];
  const bool summed = a.partial != nullptr;
  if (summed) {
    int64_t idx[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int64_t i = ((int64_t)c * NORMV_THREADS + threadIdx.x) * 4;
      idx[c] = i < d ? row * d + i : -1;
      vals[c] = i < d ? partial_sum4(a, idx[c]) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (a.n_peers > 0) {
      if (a.two_shot) tp_exchange4_two<NCH>(a, vals, idx);
      else tp_exchange4<NCH>(a, vals, idx);
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int64_t i = ((int64_t)c * NORMV_THREADS + threadIdx.x) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < d) {
      v = erow ? Vec4<TE>::load(erow + i) : *reinterpret_cast<const float4*>(xr + i);
      if (summed) {
        float4 p = vals[c];
        if (a.bias) {
          const float4 b = *reinterpret_cast<const float4*>(a.bias + i);
          p.x += b.x; p.y += b.y; p.z += b.z; p.w += b.w;
        }
        v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
      }
      if (a.x_res && (erow || summed)) *reinterpret_cast<float4*>(xr + i) = v;
    }
    vals[c] = v;
  }
  if (a.norm_kind < 0) return;
  TO* orow = reinterpret_cast<TO*>(a.out) + row * d;
  float mean = 0.f, scale;
  if (a.norm_kind == 0) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) ss += vals[c].x * vals[c].x + vals[c].y * vals[c].y + vals[c].z * vals[c].z + vals[c].w * vals[c].w;
    ss = block_sum(ss, red);
    scale = sqrtf(ss / (float)d + a.eps);  // rmsNorm divides by this
  } else {
    float s1 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) s1 += vals[c].x + vals[c].y + vals[c].z + vals[c].w;
    mean = block_sum(s1, red) / (float)d;
    float s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int64_t i = ((int64_t)c * NORMV_THREADS + threadIdx.x) * 4;
      if (i < d) {
        const float cx = vals[c].x - mean, cy = vals[c].y - mean, cz = vals[c].z - mean, cw = vals[c].w - mean;
        s2 += cx * cx + cy * cy + cz * cz + cw * cw;
      }
    }
    const float var = block_sum(s2, red) / (float)d;
    scale = 1.0f / sqrtf(var + a.eps);    // LayerNorm multiplies by this
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int64_t i = ((int64_t)c * NORMV_THREADS + threadIdx.x) * 4;
    if (i >= d) continue;
    const float4 g = *reinterpret_cast<const float4*>(a.gamma + i);
    float4 o;
    if (a.norm_kind == 0) {
      o.x = g.x * (vals[c].x / scale); o.y = g.y * (vals[c].y / scale);
      o.z = g.z * (vals[c].z / scale); o.w = g.w * (vals[c].w / scale);
    } else {
      const float4 b = *reinterpret_cast<const float4*>(a.beta + i);
      o.x = g.x * ((vals[c].x - mean) * scale) + b.x; o.y = g.y * ((vals[c].y - mean) * scale) + b.y;
      o.z = g.z * ((vals[c].z - mean) * scale) + b.z; o.w = g.w * ((vals[c].w - mean) * scale) + b.w;
    }
    Vec4<TO>::store(orow + i, o);
  }
}

// Decode-size variant: a cluster of four CTAs per row, each on a quarter of the columns; the row
// statistics meet through distributed shared memory.  With 32 rows the one-CTA-per-row kernel keeps 32
// SMs busy reading 8 slabs of 16 KB each; this one spreads the same reads over 128 SMs.
template <typename TE, int NCH>
__global__ void __cluster_dims__(4, 1, 1) __launch_bounds__(256) residual_norm_cluster_kernel(NormArgs a) {
  __shared__ float red[33];
  __shared__ float part[2];
  cg::cluster_group cl = cg::this_cluster();
  const unsigned rank = cl.block_rank();
  pdl_launch_dependents();
  const int64_t row = blockIdx.x >> 2;
  const int64_t d = a.d, dq = d >> 2, col0 = (int64_t)rank * dq;
  float* xr = a.x_res + row * d;
  float4 vals[NCH];
  pdl_wait();
  const TE* erow = nullptr;
  if (a.embed) {
    int64_t id = row;
    if (a.ids) {
      id = a.ids[row];
      if (id < 0 || id >= a.vocab) {
        if (threadIdx.x == 0 && rank == 0) atomicExch(a.status, KS_BAD_INDEX);
        id = 0;
      }
    }
    erow = reinterpret_cast<const TE*>(a.embed) + id * d;
  }
  const bool summed = a.partial != nullptr;
  // the residual (or embedding) row is requested first, so that its latency runs under the slab loads and,
  // with tensor parallelism, under the exchange
  float4 xin[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int64_t off = ((int64_t)c * 256 + threadIdx.x) * 4;
    xin[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (off < dq) xin[c] = erow ? Vec4<TE>::load(erow + col0 + off) : *reinterpret_cast<const float4*>(xr + col0 + off);
  }
  if (summed) {
    int64_t idx[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int64_t off = ((int64_t)c * 256 + threadIdx.x) * 4;
      idx[c] = off < dq ? row * d + col0 + off : -1;
      vals[c] = off < dq ? partial_sum4(a, idx[c]) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (a.n_peers > 0) {
      if (a.two_shot) tp_exchange4_two<NCH>(a, vals, idx);
      else tp_exchange4<NCH>(a, vals, idx);
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int64_t off = ((int64_t)c * 256 + threadIdx.x) * 4;
    const int64_t i = col0 + off;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (off < dq) {
      v = xin[c];
      if (summed) {
        float4 p = vals[c];
        if (a.bias) {
          const float4 b = *reinterpret_cast<const float4*>(a.bias + i);
          p.x += b.x; p.y += b.y; p.z += b.z; p.w += b.w;
        }
        v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
      }
      if (a.x_res && (erow || summed)) *reinterpret_cast<float4*>(xr + i) = v;
    }
    vals[c] = v;
  }
  // sum over the row = sum over the four CTAs' block sums, added in rank order by every CTA alike
  auto row_sum = [&](float local, int slot) -> float {
    const float bs = block_sum(local, red);
    if (threadIdx.x == 0) part[slot] = bs;
    cl.sync();
    float t = 0.f;
    for (unsigned r = 0; r < 4; ++r) t += *cl.map_shared_rank(&part[slot], r);
    return t;
  };
  bf16* orow = reinterpret_cast<bf16*>(a.out) + row * d;
  float mean = 0.f, scale;
  if (a.norm_kind == 0) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) ss += vals[c].x * vals[c].x + vals[c].y * vals[c].y + vals[c].z * vals[c].z + vals[c].w * vals[c].w;
    scale = sqrtf(row_sum(ss, 0) / (float)d + a.eps);  // rmsNorm divides by this
  } else {
    float s1 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) s1 += vals[c].x + vals[c].y + vals[c].z + vals[c].w;
    mean = row_sum(s1, 0) / (float)d;
    float s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int64_t off = ((int64_t)c * 256 + threadIdx.x) * 4;
      if (off < dq) {
        const float cx = vals[c].x - mean, cy = vals[c].y - mean, cz = vals[c].z - mean, cw = vals[c].w - mean;
        s2 += cx * cx + cy * cy + cz * cz + cw * cw;
      }
    }
    scale = 1.0f / sqrtf(row_sum(s2, 1) / (float)d + a.eps);  // LayerNorm multiplies by this
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int64_t off = ((int64_t)c * 256 + threadIdx.x) * 4;
    if (off >= dq) continue;
    const int64_t i = col0 + off;
    const float4 g = *reinterpret_cast<const float4*>(a.gamma + i);
    float4 o;
    if (a.norm_kind == 0) {
      o.x = g.x * (vals[c].x / scale); o.y = g.y * (vals[c].y / scale);
      o.z = g.z * (vals[c].z / scale); o.w = g.w * (vals[c].w / scale);
    } else {
      const float4 b = *reinterpret_cast<const float4*>(a.beta + i);
      o.x = g.x * ((vals[c].x - mean) * scale) + b.x; o.y = g.y * ((vals[c].y - mean) * scale) + b.y;
      o.z = g.z * ((vals[c].z - mean) * scale) + b.z; o.w = g.w * ((vals[c].w - mean) * scale) + b.w;
    }
    Vec4<bf16>::store(orow + i, o);
  }
  cl.sync();  // no CTA leaves while another may still read its block sums
}

template <typename TA>
__device__ __forceinline__ void store8(TA* dst, const float* r);
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* r) {
  *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(r[4], r[5], r[6], r[7]);
}
template <>
__device__ __forceinline__ void store8<bf16>(bf16* dst, const float* r) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]), pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
}

// Same work as qkv_post_kernel, eight consecutive columns (four RoPE pairs) per thread with 16-byte
// accesses; needs head_dim % 8 == 0.  Prefill-size launches are bandwidth-bound on the f32 partials.
template <typename TA>
__global__ void __launch_bounds__(256) qkv_post_vec_kernel(QkvPostArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int b = (int)(row / a.S), s = (int)(row % a.S);
  const int pos = a.pos0[b] + s;
  const int hd = a.hd;
  const int nq = a.nh * hd, nkv = a.kvh * hd, ntot = nq + 2 * nkv;
  const int rpos = pos + a.rope_shift;
  if (pos < 0 || pos >= a.kv_capacity || rpos < 0 || rpos >= a.max_seq) {
    if (threadIdx.x == 0) atomicExch(a.status, KS_BAD_INDEX);
    return;
  }
  const int col = 8 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (col >= ntot) return;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const float* pp = a.partial + row * ntot + col;
  for (int sp = 0; sp < a.nsplit; ++sp) {
    const float4 t0 = *reinterpret_cast<const float4*>(pp + sp * a.split_stride);
    const float4 t1 = *reinterpret_cast<const float4*>(pp + sp * a.split_stride + 4);
    v[0] += t0.x; v[1] += t0.y; v[2] += t0.z; v[3] += t0.w;
    v[4] += t1.x; v[5] += t1.y; v[6] += t1.z; v[7] += t1.w;
  }
  if (a.bias) {
    const float4 b0 = *reinterpret_cast<const float4*>(a.bias + col), b1 = *reinterpret_cast<const float4*>(a.bias + col + 4);
    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
    v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
  }
  int64_t cache_row_base, head_stride;
  if (a.kv.block_table) {
    const int page = a.kv.block_table[(int64_t)b * a.kv.max_pages + pos / a.kv.page];
    cache_row_base = ((int64_t)page * a.kvh) * a.kv.page + pos % a.kv.page;
    head_stride = a.kv.page;
  } else {
    cache_row_base = ((int64_t)b * a.kvh) * a.kv.contiguous_len + pos;
    head_stride = a.kv.contiguous_len;
  }
  if (col < nq + nkv) {
    // the tables hold each angle's value twice (elements 2i and 2i+1), so element 2j of the chunk is pair j's
    const int e0 = col % hd;
    const float* cr = a.cosT + (int64_t)rpos * hd + e0;
    const float* sr = a.sinT + (int64_t)rpos * hd + e0;
    const float4 c0 = *reinterpret_cast<const float4*>(cr), c1 = *reinterpret_cast<const float4*>(cr + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sr), s1 = *reinterpret_cast<const float4*>(sr + 4);
    const float cs[4] = {c0.x, c0.z, c1.x, c1.z}, sn[4] = {s0.x, s0.z, s1.x, s1.z};
    float r[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      r[2 * j] = rope_even(cs[j], sn[j], v[2 * j], v[2 * j + 1]);
      r[2 * j + 1] = rope_odd(cs[j], sn[j], v[2 * j], v[2 * j + 1]);
    }
    if (col < nq) {
      store8<TA>(reinterpret_cast<TA*>(a.q_out) + row * nq + col, r);
    } else {
      const int h = (col - nq) / hd, e = (col - nq) % hd;
      store8<TA>(reinterpret_cast<TA*>(a.kv.k) + (cache_row_base + h * head_stride) * hd + e, r);
    }
  } else {
    const int h = (col - nq - nkv) / hd, e = (col - nq - nkv) % hd;
    store8<TA>(reinterpret_cast<TA*>(a.kv.v) + (cache_row_base + h * head_stride) * hd + e, v);
  }
}

// One CTA per (token row, chunk of 256 column pairs) of the fused q|k|v row.
template <typename TA>
__global__ void __launch_bounds__(256) qkv_post_kernel(QkvPostArgs a) {
  pdl_launch_dependents();
  // Inside a captured decode step (early_lookup) positions, block tables and RoPE tables were written
  // before the graph was launched: look them up while the q|k|v Linear drains; only its slabs have to
  // wait.  Elsewhere a kernel still in flight may be their producer (a dependent launch starts as soon
  // as its predecessor has STARTED, so "several launches back" proves nothing): wait first.
  if (!a.early_lookup) pdl_wait();
  const int64_t row = blockIdx.x;
  const int b = (int)(row / a.S), s = (int)(row % a.S);
  const int pos = a.pos0[b] + s;
  const int hd = a.hd, half = hd / 2;
  const int nq = a.nh * hd, nkv = a.kvh * hd, ntot = nq + 2 * nkv;
  const int rpos = pos + a.rope_shift;
  if (pos < 0 || pos >= a.kv_capacity || rpos < 0 || rpos >= a.max_seq) {
    if (threadIdx.x == 0) atomicExch(a.status, KS_BAD_INDEX);
    return;
  }
  const float* cr = a.cosT + (int64_t)rpos * hd;
  const float* sr = a.sinT + (int64_t)rpos * hd;
  // destination rows of this token in the cache
  int64_t cache_row_base;  // row index for kv head 0; kv head h adds h * stride
  int64_t head_stride;
  if (a.kv.block_table) {
    const int page = a.kv.block_table[(int64_t)b * a.kv.max_pages + pos / a.kv.page];
    cache_row_base = ((int64_t)page * a.kvh) * a.kv.page + pos % a.kv.page;
    head_stride = a.kv.page;
  } else {
    cache_row_base = ((int64_t)b * a.kvh) * a.kv.contiguous_len + pos;
    head_stride = a.kv.contiguous_len;
  }
  TA* q_out = reinterpret_cast<TA*>(a.q_out) + row * nq;
  TA* kc = reinterpret_cast<TA*>(a.kv.k);
  TA* vc = reinterpret_cast<TA*>(a.kv.v);
  const int npairs = ntot / 2;
  {
    const int p = blockIdx.y * blockDim.x + threadIdx.x;
    if (p >= npairs) return;
    const int col = 2 * p;
    float c0 = 1.f, s0 = 0.f;
    if (col < nq + nkv) {
      const int i = (col % hd) / 2;
      c0 = cr[2 * i];
      s0 = sr[2 * i];
    }
    const float b0 = a.bias ? a.bias[col] : 0.f, b1 = a.bias ? a.bias[col + 1] : 0.f;
    pdl_wait();
    float v0 = 0.f, v1 = 0.f;
    const float* pp = a.partial + row * ntot + col;
    int sp = 0;
    for (; sp + 4 <= a.nsplit; sp += 4) {
      const float2 t0 = *reinterpret_cast<const float2*>(pp + (sp + 0) * a.split_stride);
      const float2 t1 = *reinterpret_cast<const float2*>(pp + (sp + 1) * a.split_stride);
      const float2 t2 = *reinterpret_cast<const float2*>(pp + (sp + 2) * a.split_stride);
      const float2 t3 = *reinterpret_cast<const float2*>(pp + (sp + 3) * a.split_stride);
      v0 += t0.x; v1 += t0.y;
      v0 += t1.x; v1 += t1.y;
      v0 += t2.x; v1 += t2.y;
      v0 += t3.x; v1 += t3.y;
    }
    for (; sp < a.nsplit; ++sp) {
      const float2 t = *reinterpret_cast<const float2*>(pp + sp * a.split_stride);
      v0 += t.x;
      v1 += t.y;
    }
    if (a.bias) {
      v0 += b0;
      v1 += b1;
    }
    if (col < nq + nkv) {
      const float r0 = rope_even(c0, s0, v0, v1);
      const float r1 = rope_odd(c0, s0, v0, v1);
      if (col < nq) {
        q_out[col] = from_f<TA>(r0);
        q_out[col + 1] = from_f<TA>(r1);
      } else {
        const int h = (col - nq) / hd, e = (col - nq) % hd;
        TA* dst = kc + (cache_row_base + h * head_stride) * hd + e;
        dst[0] = from_f<TA>(r0);
        dst[1] = from_f<TA>(r1);
      }
    } else {
      const int h = (col - nq - nkv) / hd, e = (col - nq - nkv) % hd;
      TA* dst = vc + (cache_row_base + h * head_stride) * hd + e;
      dst[0] = from_f<TA>(v0);
      dst[1] = from_f<TA>(v1);
    }
  }
  (void)half;
}

// First maximum of each row (sampleGreedy).  grid (rows, chunks): each CTA scans
// one column chunk; with more than one chunk the (value, index) partials are
// merged by argmax_final_kernel.
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int64_t V, int64_t chunk_w,
                                                      int* out, float* part_v, int* part_i) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_launch_dependents();
  pdl_wait();
  const float* r = logits + (int64_t)blockIdx.x * V;
  const int64_t c0 = (int64_t)blockIdx.y * chunk_w, c1 = min(V, c0 + chunk_w);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
    const float v = r[i];
    if (v > best || (v == best && (int)i < bi)) {
      best = v;
      bi = (int)i;
    }
  }
  // NaN-free inputs assumed, as in the reference's host loop (a NaN never wins a '>' test).
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
        best = sv[w];
        bi = si[w];
      }
    if (gridDim.y == 1) {
      out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    } else {
      part_v[blockIdx.x * gridDim.y + blockIdx.y] = best;
      part_i[blockIdx.x * gridDim.y + blockIdx.y] = bi;
    }
  }
}

__global__ void __launch_bounds__(32) argmax_final_kernel(const float* part_v, const int* part_i, int nchunks, int* out) {
  pdl_launch_dependents();
  pdl_wait();
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nchunks; i += 32) {
    const float v = part_v[blockIdx.x * nchunks + i];
    const int ix = part_i[blockIdx.x * nchunks + i];
    if (v > best || (v == best && ix < bi)) {
      best = v;
      bi = ix;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
}

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits, int64_t V, int64_t chunk_w,
                                                              int idx_offset, float* part_v, int* part_i) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_launch_dependents();
  pdl_wait();
  const float* r = logits + (int64_t)blockIdx.x * V;
  const int64_t c0 = (int64_t)blockIdx.y * chunk_w, c1 = min(V, c0 + chunk_w);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
    const float v = r[i];
    if (v > best || (v == best && (int)i < bi)) {
      best = v;
      bi = (int)i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
        best = sv[w];
        bi = si[w];
      }
    part_v[blockIdx.x * gridDim.y + blockIdx.y] = best;
    part_i[blockIdx.x * gridDim.y + blockIdx.y] = (bi == 0x7fffffff) ? 0x7fffffff : bi + idx_offset;
  }
}

__global__ void __launch_bounds__(32) argmax_gathered_kernel(const void* gathered, int world, int rows, int nchunks, int* out) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t per_rank = (size_t)rows * nchunks * 8;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < world * nchunks; i += 32) {
    const int r = i / nchunks, ch = i % nchunks;
    const char* base = (const char*)gathered + (size_t)r * per_rank;
    const float v = ((const float*)base)[blockIdx.x * nchunks + ch];
    const int ix = ((const int*)(base + (size_t)rows * nchunks * 4))[blockIdx.x * nchunks + ch];
    if (v > best || (v == best && ix < bi)) {
      best = v;
      bi = ix;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
}

// ---- two-shot tensor-parallel all-reduce (Tp2Args) ----------------------------------------------------
// 16-byte chunks: CE payload elements each.  Scatter: chunk (row, col) of the local partial goes to the rank
// that owns its column slice.
template <typename T>
__global__ void __launch_bounds__(256) tp2_scatter_kernel(Tp2Args a) {
  constexpr int CE = 16 / sizeof(T);
  pdl_launch_dependents();
  pdl_wait();
  const int64_t cpr = a.d / CE, dn = a.d / a.world;
  const int64_t total = a.rows * cpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / cpr, col = (i % cpr) * CE;
    const int p = (int)(col / dn);
    if (p == a.my_rank) continue;
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.partial) + row * a.d + col);
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.region[p]) + ((int64_t)a.my_rank * a.rows + row) * dn + (col - p * dn)) = v;
  }
  if (grid_last_cta(a.arrive)) {
    if ((int)threadIdx.x < a.world) peer_flag_release(a.cells[threadIdx.x] + 8 + a.my_rank, *a.epoch + a.offset);
  }
}

__device__ __forceinline__ void acc_chunk(float (&acc)[8], uint4 v, bf16) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
    acc[2 * j] += __low2float(h);
    acc[2 * j + 1] += __high2float(h);
  }
}
__device__ __forceinline__ void acc_chunk(float (&acc)[8], uint4 v, float) {
  acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y); acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
}

// Reduce + gather: this rank adds the world copies of its column slice in rank order and stores the sum into
// every rank's gather buffer (its own included).
template <typename T>
__global__ void __launch_bounds__(256) tp2_reduce_kernel(Tp2Args a) {
  constexpr int CE = 16 / sizeof(T);
  pdl_launch_dependents();
  pdl_wait();
  peer_flags_wait(a.cells[a.my_rank] + 8, 1, a.world, -1, *a.epoch + a.offset, a.status);
  const int64_t dn = a.d / a.world, cps = dn / CE;
  const int64_t total = a.rows * cps;
  const T* scat = reinterpret_cast<const T*>(a.region[a.my_rank]);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / cps, c0 = (i % cps) * CE;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < a.world; ++r) {
      uint4 v;
      if (r == a.my_rank) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.partial) + row * a.d + a.my_rank * dn + c0);
      else v = __ldcg(reinterpret_cast<const uint4*>(scat + ((int64_t)r * a.rows + row) * dn + c0));
      acc_chunk(acc, v, T());
    }
    uint4 o;
    if constexpr (sizeof(T) == 2) {
      o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    } else {
      o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
    }
    const int64_t at = row * a.d + a.my_rank * dn + c0;
    for (int r = 0; r < a.world; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.region[r] + a.off_gather) + at) = o;
  }
  if (grid_last_cta(a.arrive + 1)) {
    if ((int)threadIdx.x < a.world) peer_flag_release(a.cells[threadIdx.x] + 16 + a.my_rank, *a.epoch + a.offset);
  }
}

__global__ void epoch_bump_kernel(int* epoch, int by) {
  pdl_launch_dependents();
  pdl_wait();
  *epoch += by;
}

// part[0][i] += part[1][i] + ... (before a tensor-parallel all-reduce of one slab)
__global__ void __launch_bounds__(256) slab_sum_kernel(float* part, int nsplit, int64_t slab, int64_t n4) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 a = reinterpret_cast<float4*>(part)[i];
  for (int s = 1; s < nsplit; ++s) {
    const float4 b = reinterpret_cast<const float4*>(part + s * slab)[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  reinterpret_cast<float4*>(part)[i] = a;
}

__global__ void swiglu_f32_kernel(const float* g, const float* u, float* out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  // src/rew/nn/activation.nim:28-38: x * (1 / (1 + exp(-x)))
  const float x = g[i];
  const float sig = 1.0f / (1.0f + expf(-x));
  out[i] = (x * sig) * u[i];
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* src, TD* dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<TD>(to_f<TS>(src[i]));
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Counter-based N(0,std): Box-Muller on two hashed uniforms per element pair.
template <typename T>
__global__ void fill_normal_kernel(T* dst, int64_t n, uint64_t seed, float std) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t i = 2 * p;
  if (i >= n) return;
  const uint64_t h = splitmix64(seed ^ splitmix64((uint64_t)p));
  const float u1 = ((uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);
  const float u2 = (uint32_t)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
  const float r = sqrtf(-2.0f * logf(u1)) * std;
  float s, c;
  sincospif(2.0f * u2, &s, &c);
  dst[i] = from_f<T>(r * c);
  if (i + 1 < n) dst[i + 1] = from_f<T>(r * s);
}

template <typename T>
__global__ void fill_const_kernel(T* dst, int64_t n, float v) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(v);
}

}  // namespace

int residual_norm_launch(Ctx* c, const NormArgs& a, int64_t rows) {
  if (rows == 0) return REWB200_OK;
  RB_REQUIRE(a.d <= (int64_t)NORM_THREADS * NORM_MAX_PER_THREAD, "norm width above 16384 is not supported");
  const bool e16 = a.embed_dtype == REWB200_BF16, o16 = a.out_dtype == REWB200_BF16;
  cudaError_t e;
  RB_REQUIRE(a.n_peers == 0 || (a.d % 4 == 0 && a.partial != nullptr && rows <= 64 && a.n_peers <= 8 &&
                                rows * a.d / (a.payload_bf16 ? 4 : 2) <= a.slot_lines),
             "the fused all-reduce needs d_model % 4 == 0, local partials, at most 64 rows and a slot that holds the step");
  RB_REQUIRE(!a.partial_bf16 || a.d % 4 == 0, "bf16 partials need d_model % 4 == 0");
  if (o16 && a.norm_kind >= 0 && rows <= 64 && a.d % 16 == 0 && a.d <= 16384 && c->norm_cluster) {
    const int nch = (int)((a.d / 16 + 255) / 256);  // float4 per thread over a quarter row
    dim3 g((unsigned)(rows * 4)), b(256);
#define RB_NORMC(TE)                                                                                  \
  (nch <= 1   ? launch_k(residual_norm_cluster_kernel<TE, 1>, g, b, 0, c->stream, c->use_pdl, a)          \
   : nch <= 2 ? launch_k(residual_norm_cluster_kernel<TE, 2>, g, b, 0, c->stream, c->use_pdl, a)          \
              : launch_k(residual_norm_cluster_kernel<TE, 4>, g, b, 0, c->stream, c->use_pdl, a))
    e = e16 ? RB_NORMC(bf16) : RB_NORMC(float);
#undef RB_NORMC
    RB_CUDA(e);
    ++g_launch_total;
    return REWB200_OK;
  }
  if (a.d % 4 == 0) {
    const int nch = (int)((a.d / 4 + NORMV_THREADS - 1) / NORMV_THREADS);
    dim3 g((unsigned)rows), b(NORMV_THREADS);
#define RB_NORMV(TE, TO)                                                                                   \
  (nch <= 1   ? launch_k(residual_norm_vec_kernel<TE, TO, 1>, g, b, 0, c->stream, c->use_pdl, a)             \
   : nch <= 2 ? launch_k(residual_norm_vec_kernel<TE, TO, 2>, g, b, 0, c->stream, c->use_pdl, a)             \
   : nch <= 4 ? launch_k(residual_norm_vec_kernel<TE, TO, 4>, g, b, 0, c->stream, c->use_pdl, a)             \
              : launch_k(residual_norm_vec_kernel<TE, TO, 8>, g, b, 0, c->stream, c->use_pdl, a))
    if (e16 && o16) e = RB_NORMV(bf16, bf16);
    else if (e16) e = RB_NORMV(bf16, float);
    else if (o16) e = RB_NORMV(float, bf16);
    else e = RB_NORMV(float, float);
#undef RB_NORMV
    RB_CUDA(e);
    ++g_launch_total;
    return REWB200_OK;
  }
  dim3 grid((unsigned)rows), block(NORM_THREADS);
  if (e16 && o16) e = launch_k(residual_norm_kernel<bf16, bf16>, grid, block, 0, c->stream, c->use_pdl, a);
  else if (e16) e = launch_k(residual_norm_kernel<bf16, float>, grid, block, 0, c->stream, c->use_pdl, a);
  else if (o16) e = launch_k(residual_norm_kernel<float, bf16>, grid, block, 0, c->stream, c->use_pdl, a);
  else e = launch_k(residual_norm_kernel<float, float>, grid, block, 0, c->stream, c->use_pdl, a);
  RB_CUDA(e);
  ++g_launch_total;
  return REWB200_OK;
}

int qkv_post_launch(Ctx* c, const QkvPostArgs& a, int64_t B) {
  const int64_t rows = B * a.S;
  if (rows == 0) return REWB200_OK;
  RB_REQUIRE(a.hd % 2 == 0, "head_dim must be even for RoPE");
  cudaError_t e;
  const int npairs = (a.nh + 2 * a.kvh) * a.hd / 2;
  if (a.hd % 8 == 0 && rows > 64) {  // prefill sizes: eight columns per thread
    const int nchunk = (a.nh + 2 * a.kvh) * a.hd / 8;
    dim3 vgrid((unsigned)rows, (unsigned)((nchunk + 255) / 256));
    if (a.act_dtype == REWB200_BF16)
      e = launch_k(qkv_post_vec_kernel<bf16>, vgrid, dim3(256), 0, c->stream, c->use_pdl, a);
    else
      e = launch_k(qkv_post_vec_kernel<float>, vgrid, dim3(256), 0, c->stream, c->use_pdl, a);
    RB_CUDA(e);
    ++g_launch_total;
    return REWB200_OK;
  }
  dim3 grid((unsigned)rows, (unsigned)((npairs + 255) / 256));
  if (a.act_dtype == REWB200_BF16)
    e = launch_k(qkv_post_kernel<bf16>, grid, dim3(256), 0, c->stream, c->use_pdl, a);
  else
    e = launch_k(qkv_post_kernel<float>, grid, dim3(256), 0, c->stream, c->use_pdl, a);
  RB_CUDA(e);
  ++g_launch_total;
  return REWB200_OK;
}

int argmax_launch(Ctx* c, const float* logits, int64_t rows, int64_t V, int* out_ids, void* scratch, size_t scratch_bytes) {
  if (rows == 0) return REWB200_OK;
  int nchunks = 1;
  if (scratch && V >= 8192) {
    nchunks = (int)std::min<int64_t>(64, (V + 4095) / 4096);
    while (nchunks > 1 && (size_t)rows * nchunks * 8 > scratch_bytes) nchunks /= 2;
  }
  const int64_t chunk_w = (V + nchunks - 1) / nchunks;
  float* pv = (float*)scratch;
  int* pi = (int*)((char*)scratch + (size_t)rows * nchunks * 4);
  RB_CUDA(launch_k(argmax_kernel, dim3((unsigned)rows, (unsigned)nchunks), dim3(256), 0, c->stream, c->use_pdl, logits, V,
                   chunk_w, out_ids, pv, pi));
  ++g_launch_total;
  if (nchunks > 1) {
    RB_CUDA(launch_k(argmax_final_kernel, dim3((unsigned)rows), dim3(32), 0, c->stream, c->use_pdl, (const float*)pv,
                     (const int*)pi, nchunks, out_ids));
    ++g_launch_total;
  }
  return REWB200_OK;
}

// Stage 1 only: per-chunk (value, global index) partials, for the vocab-parallel lm_head.
int argmax_partial_launch(Ctx* c, const float* logits, int64_t rows, int64_t V, int idx_offset, int nchunks, float* pv, int* pi) {
  if (rows == 0) return REWB200_OK;
  const int64_t chunk_w = (V + nchunks - 1) / nchunks;
  RB_CUDA(launch_k(argmax_partial_kernel, dim3((unsigned)rows, (unsigned)nchunks), dim3(256), 0, c->stream, c->use_pdl, logits,
                   V, chunk_w, idx_offset, pv, pi));
  ++g_launch_total;
  return REWB200_OK;
}

// gathered: per rank [rows*nchunks floats | rows*nchunks ints]; first maximum by (value desc, index asc).
int argmax_gathered_launch(Ctx* c, const void* gathered, int world, int64_t rows, int nchunks, int* out) {
  if (rows == 0) return REWB200_OK;
  RB_CUDA(launch_k(argmax_gathered_kernel, dim3((unsigned)rows), dim3(32), 0, c->stream, c->use_pdl, gathered, world,
                   (int)rows, nchunks, out));
  ++g_launch_total;
  return REWB200_OK;
}

int tp2_allreduce_launch(Ctx* c, const Tp2Args& a) {
  const int ce = a.payload_bf16 ? 8 : 4;
  RB_REQUIRE(a.world >= 2 && a.world <= 8 && a.d % ((int64_t)a.world * ce) == 0, "two-shot all-reduce: d_model must split into 16-byte chunks per rank");
  const int64_t chunks = a.rows * (a.d / ce);
  const unsigned g1 = (unsigned)std::min<int64_t>((chunks + 255) / 256, (int64_t)c->sm_count * 16);
  const unsigned g2 = (unsigned)std::min<int64_t>((chunks / a.world + 255) / 256, (int64_t)c->sm_count * 16);
  if (a.payload_bf16) {
    RB_CUDA(launch_k(tp2_scatter_kernel<bf16>, dim3(g1), dim3(256), 0, c->stream, c->use_pdl, a));
    RB_CUDA(launch_k(tp2_reduce_kernel<bf16>, dim3(std::max(g2, 1u)), dim3(256), 0, c->stream, c->use_pdl, a));
  } else {
    RB_CUDA(launch_k(tp2_scatter_kernel<float>, dim3(g1), dim3(256), 0, c->stream, c->use_pdl, a));
    RB_CUDA(launch_k(tp2_reduce_kernel<float>, dim3(std::max(g2, 1u)), dim3(256), 0, c->stream, c->use_pdl, a));
  }
  g_launch_total += 2;
  return REWB200_OK;
}

int epoch_bump_launch(Ctx* c, int* epoch, int by) {
  RB_CUDA(launch_k(epoch_bump_kernel, dim3(1), dim3(1), 0, c->stream, c->use_pdl, epoch, by));
  ++g_launch_total;
  return REWB200_OK;
}

int slab_sum_launch(Ctx* c, float* part, int nsplit, int64_t slab_elems) {
  if (nsplit <= 1 || slab_elems == 0) return REWB200_OK;
  RB_REQUIRE(slab_elems % 4 == 0, "slab size must be a multiple of 4 floats");
  const int64_t n4 = slab_elems / 4;
  RB_CUDA(launch_k(slab_sum_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, c->stream, c->use_pdl, part, nsplit,
                   slab_elems, n4));
  ++g_launch_total;
  return REWB200_OK;
}

int swiglu_f32_launch(Ctx* c, const float* g, const float* u, float* out, int64_t n) {
  if (n == 0) return REWB200_OK;
  swiglu_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(g, u, out, n);
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

int cast_launch(Ctx* c, const void* src, int sd, void* dst, int dd, int64_t n) {
  if (n == 0) return REWB200_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (sd == REWB200_F32 && dd == REWB200_BF16)
    cast_kernel<float, bf16><<<blocks, 256, 0, c->stream>>>((const float*)src, (bf16*)dst, n);
  else if (sd == REWB200_BF16 && dd == REWB200_F32)
    cast_kernel<bf16, float><<<blocks, 256, 0, c->stream>>>((const bf16*)src, (float*)dst, n);
  else if (sd == REWB200_F32 && dd == REWB200_F32)
    cast_kernel<float, float><<<blocks, 256, 0, c->stream>>>((const float*)src, (float*)dst, n);
  else if (sd == REWB200_BF16 && dd == REWB200_BF16)
    cast_kernel<bf16, bf16><<<blocks, 256, 0, c->stream>>>((const bf16*)src, (bf16*)dst, n);
  else
    return fail("cast: only f32 and bf16 are supported");
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

int fill_normal_launch(Ctx* c, void* dst, int dtype, int64_t n, uint64_t seed, float std) {
  if (n == 0) return REWB200_OK;
  const int64_t pairs = (n + 1) / 2;
  const unsigned blocks = (unsigned)((pairs + 255) / 256);
  if (dtype == REWB200_BF16) fill_normal_kernel<bf16><<<blocks, 256, 0, c->stream>>>((bf16*)dst, n, seed, std);
  else if (dtype == REWB200_F32) fill_normal_kernel<float><<<blocks, 256, 0, c->stream>>>((float*)dst, n, seed, std);
  else return fail("fill_normal: only f32 and bf16 are supported");
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

int fill_const_launch(Ctx* c, void* dst, int dtype, int64_t n, float v) {
  if (n == 0) return REWB200_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == REWB200_BF16) fill_const_kernel<bf16><<<blocks, 256, 0, c->stream>>>((bf16*)dst, n, v);
  else if (dtype == REWB200_F32) fill_const_kernel<float><<<blocks, 256, 0, c->stream>>>((float*)dst, n, v);
  else return fail("fill_const: only f32 and bf16 are supported");
  RB_CUDA(cudaGetLastError());
  ++g_launch_total;
  return REWB200_OK;
}

// src/rew/nn/rope.nim:123-138, computed on the host as the reference does
// (double pow, float angle, float cos/sin, each value stored twice).
int rope_tables_host(int hd, int max_seq, double theta, std::vector<float>* cosT, std::vector<float>* sinT) {
  RB_REQUIRE(hd > 0 && hd % 2 == 0, "initRotaryPositionEncoding: headDim must be positive and even, got " + std::to_string(hd));
  RB_REQUIRE(max_seq > 0, "initRotaryPositionEncoding: maxSeqLen must be positive");
  const int half = hd / 2;
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i) inv[i] = 1.0f / (float)pow(theta, (double)(2 * i) / (double)hd);
  cosT->resize((size_t)max_seq * hd);
  sinT->resize((size_t)max_seq * hd);
  for (int p = 0; p < max_seq; ++p) {
    const float fp = (float)p;
    for (int i = 0; i < half; ++i) {
      const float angle = fp * inv[i];
      const float cv = cosf(angle), sv = sinf(angle);
      const size_t base = (size_t)p * hd + 2 * i;
      (*cosT)[base] = cv;
      (*cosT)[base + 1] = cv;
      (*sinT)[base] = sv;
      (*sinT)[base + 1] = sv;
    }
  }
  return REWB200_OK;
}

}  // namespace rewb
