// Token sampling on the device for generate (src/rew/infer/generate.nim:92-159,192-265).
// The reference copies every step's logits to the host, sorts the whole vocabulary there and
// samples in Nim loops; here a cluster of four CTAs per sequence does it next to the lm_head output:
//   applySamplingConfig  repetition penalty once per occurrence among the tokens seen so far (a bitmap in
//                        shared memory finds the seen ids, the thread holding a token's first occurrence
//                        counts the others), temperature, min-p               (generate.nim:192-218)
//   greedy               first maximum                                        (:152-159)
//   sampleTopK           the k largest, sorted (value descending, index ascending = Nim's stable sort),
//                        exp WITHOUT max subtraction, sequential cumulative sum, u <= cum   (:92-116)
//   sampleTopP           "first rank whose cumulative probability reaches t", once for the nucleus
//                        cutoff (t = topP) and once for the draw (t = u * nucleus mass)     (:118-150)
//   keys                 Threefry-2x32 as src/rew/rng.nim:33-80; u = unit float of foldIn(key, 0).a;
//                        after each token key = foldIn(key, step)
// No full sort: both selections first narrow the vocabulary with histograms over a monotone 24-bit
// code of (max - value) (three 8-bit levels, quarter-logit buckets at the top level, per-warp private
// histograms so that shared-memory atomics do not pile up on one address), gather the at most 4096
// survivors into the first CTA's shared memory and sort only those.  Each CTA of the cluster walks a
// quarter of the vocabulary row; partial histograms and candidates travel through distributed shared
// memory, and the first CTA takes every decision so that the four can never disagree on how many
// cluster barriers follow.  Inputs that the buckets cannot separate (thousands of equal values, more
// than k tokens at -inf) take the exact path in the first CTA: a radix select over the
// order-preserving bits of the float itself with ties resolved by index.  Probability-mass histograms
// add floats with atomics and the cumulative sums run as parallel scans, so a draw within rounding of
// the boundary between two tokens may resolve either way; the rest is deterministic.
#include <cooperative_groups.h>
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace rewb {
namespace {

constexpr int ST = 1024;       // threads per CTA
constexpr int NW = ST / 32;    // warps
constexpr int CS = 4;          // CTAs per sequence (one cluster)
constexpr int MAX_TOPK = 1024;
constexpr int CAP = 4096;      // candidates gathered and sorted in shared memory
constexpr unsigned FULL = 0xffffffffu;

struct SampleArgs {
  const float* logits;   // [B][V]
  float* work;           // [B][V] transformed logits
  int64_t V;
  int* hist;             // [B][hist_cap] tokens seen so far (prompt + generated)
  int* hist_len;         // [B]
  int hist_cap;
  uint32_t* keys;        // [B][2]
  int* steps;            // [B] tokens sampled so far in this generate call (the reference's `step`)
  int* next;             // [B] sampled ids
  float* logprob;        // [B][logprob_cap], indexed by step
  int logprob_cap;
  float temperature, top_p, min_p, rep_penalty;
  int top_k, do_sample;
  int exact_only;        // skip the bucket path (testing aid)
  const int* active;     // [B] or nullptr: sequences with 0 are skipped
  int* status;
};

__device__ __forceinline__ uint32_t rotl32(uint32_t x, uint32_t r) { return (x << r) | (x >> (32u - r)); }
__device__ void threefry2x32(uint32_t ka, uint32_t kb, uint32_t ca, uint32_t cb, uint32_t* oa, uint32_t* ob) {
  const uint32_t rot[4] = {13u, 15u, 26u, 6u};
  const uint32_t k2 = ka ^ kb ^ 0x1BD11BDAu;
  uint32_t x0 = ca + ka, x1 = cb + kb;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    x0 = x0 + x1;
    x1 = rotl32(x1, rot[r]);
    x1 = x1 ^ x0;
  }
  *oa = x0 + kb;
  *ob = x1 + k2 + 1u;
}

// order-preserving map float -> uint32 (larger float = larger key; -inf lowest)
__device__ __forceinline__ uint32_t fkey(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Monotone 24-bit code of the distance from the maximum: a larger value never has a larger code.
// Level 0 digit = quarter-logit buckets over [M - 63.75, M]; levels 1 and 2 split a bucket 256 ways
// each.  (d - l1) and (t - l2) are exact in float, so the order survives.  Everything farther than
// the range (including -inf) gets the last code.
__device__ __forceinline__ uint32_t bcode(float v, float M) {
  const float d = (M - v) * 4.0f;
  if (!(d < 255.0f)) return 0xFFFFFFu;
  const int l1 = (int)d;
  const float t = (d - (float)l1) * 256.0f;
  const int l2 = min(255, (int)t);
  const float t2 = (t - (float)l2) * 256.0f;
  const int l3 = min(255, max(0, (int)t2));
  return ((uint32_t)l1 << 16) | ((uint32_t)l2 << 8) | (uint32_t)l3;
}

// Visits every (index, value) of p[lo..hi) once, block-strided.  One CTA walks its part of a
// vocabulary row out of L2, so the loads must overlap: 16-byte loads, four in flight per thread.
template <typename F>
__device__ __forceinline__ void for_each_value(const float* p, int64_t lo, int64_t hi, F f) {
  if (((lo | hi) & 3) == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const int64_t j_lo = lo >> 2, j_hi = hi >> 2;
    const float4* p4 = reinterpret_cast<const float4*>(p);
    for (int64_t j0 = j_lo + threadIdx.x; j0 < j_hi; j0 += (int64_t)ST * 4) {
      float4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t j = j0 + (int64_t)u * ST;
        if (j < j_hi) r[u] = p4[j];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t j = j0 + (int64_t)u * ST;
        if (j < j_hi) {
          f(4 * j, r[u].x);
          f(4 * j + 1, r[u].y);
          f(4 * j + 2, r[u].z);
          f(4 * j + 3, r[u].w);
        }
      }
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += ST) f(i, p[i]);
  }
}

__device__ float block_reduce_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(FULL, t, o);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Exclusive prefix sum of one int per thread over the block; `total` gets the block sum.
__device__ int block_exclusive_scan(int v, int* scan, int* total) {
  __syncthreads();
  scan[threadIdx.x] = v;
  __syncthreads();
  for (int off = 1; off < ST; off <<= 1) {
    const int t = (threadIdx.x >= off) ? scan[threadIdx.x - off] : 0;
    __syncthreads();
    scan[threadIdx.x] += t;
    __syncthreads();
  }
  *total = scan[ST - 1];
  return scan[threadIdx.x] - v;
}

struct Decision {        // taken by the first CTA, copied by the others
  uint32_t prefix;       // digits of the code picked so far
  int level;
  int above_cnt;         // elements / mass in buckets before the picked one
  float above_mass;
  int ok;                // the picked bucket fits CAP
  float target;          // mass still to cover inside the picked bucket
  int need;              // elements still to take inside the picked bucket
};

struct Shared {
  float red[33];
  int hist_i[256];       // exact path: counts per digit
  int scan[ST];
  int part_cnt[256];     // this CTA's share of a histogram level
  float part_mass[256];
  int cnt1[256];         // first CTA: level-0 totals, kept for the second selection
  float mass1[256];
  int cntw[256];         // first CTA: totals of the level being refined
  float massw[256];
  float part_f[2];       // scalars exchanged across the cluster
  int part_i[2];
  int wsum_c[32];
  float wsum_m[32];
  Decision dec;
  uint32_t sel_prefix;   // exact path
  int sel_need;
  float sel_target;
  float sel_above;
  int slot;
  int result;
  int pick;
  int last_nonempty;
  int first;
  float nucleus;
};

struct Dyn {             // carved out of dynamic shared memory
  uint32_t* bitmap;      // V bits
  int* hc;               // [NW][256] per-warp counts
  float* hm;             // [NW][256] per-warp masses
  float* cval;           // [CAP]
  int* cidx;             // [CAP]
};

// ---- bucket path ---------------------------------------------------------------------------------

// Folds the per-warp private histograms into this CTA's share (sh.part_cnt / sh.part_mass).
__device__ void fold_private_hists(const Dyn& dy, Shared& sh) {
  __syncthreads();
  if (threadIdx.x < 256) {
    int c = 0;
    float m = 0.f;
    for (int x = 0; x < NW; ++x) {
      c += dy.hc[x * 256 + threadIdx.x];
      m += dy.hm[x * 256 + threadIdx.x];
    }
    sh.part_cnt[threadIdx.x] = c;
    sh.part_mass[threadIdx.x] = m;
  }
  __syncthreads();
}

// This CTA's share of one level of the code histogram.
__device__ void bucket_hist_partial(const float* w, int64_t lo, int64_t hi, float M, int level, uint32_t prefix,
                                    const Dyn& dy, Shared& sh) {
  for (int i = threadIdx.x; i < NW * 256; i += ST) {
    dy.hc[i] = 0;
    dy.hm[i] = 0.f;
  }
  __syncthreads();
  const int wp = threadIdx.x >> 5;
  const int sh_hi = 24 - 8 * level, sh_d = 16 - 8 * level;
  for_each_value(w, lo, hi, [&](int64_t, float v) {
    const uint32_t c = bcode(v, M);
    if ((c >> sh_hi) == prefix) {
      const int bin = (int)((c >> sh_d) & 255u);
      atomicAdd(&dy.hc[wp * 256 + bin], 1);
      atomicAdd(&dy.hm[wp * 256 + bin], expf(v - M));
    }
  });
  fold_private_hists(dy, sh);
}

// First CTA: adds the four shares of a level (call between two cluster barriers).
__device__ void total_hists(cg::cluster_group& cl, Shared& sh, int* cnt_out, float* mass_out) {
  if (threadIdx.x < 256) {
    int c = 0;
    float m = 0.f;
    for (unsigned r = 0; r < CS; ++r) {
      const Shared* rs = cl.map_shared_rank(&sh, r);
      c += rs->part_cnt[threadIdx.x];
      m += rs->part_mass[threadIdx.x];
    }
    cnt_out[threadIdx.x] = c;
    mass_out[threadIdx.x] = m;
  }
  __syncthreads();
}

// First CTA: picks the bucket of one level.  MASS: the first bucket (largest values first) in which the
// running mass reaches dec.target; otherwise the bucket that holds the dec.need-th largest element.
template <bool MASS>
__device__ void pick_bucket(const int* cnt, const float* mass, int level, bool include_above, Shared& sh) {
  const int t = threadIdx.x, lane = t & 31, wp = t >> 5;
  int c = 0;
  float m = 0.f;
  if (t < 256) {
    c = cnt[t];
    m = mass[t];
  }
  int ic = c;
  float im = m;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int oc = __shfl_up_sync(FULL, ic, o);
    const float om = __shfl_up_sync(FULL, im, o);
    if (lane >= o) {
      ic += oc;
      im += om;
    }
  }
  if (t < 256 && lane == 31) {
    sh.wsum_c[wp] = ic;
    sh.wsum_m[wp] = im;
  }
  if (t == 0) {
    sh.pick = 256;
    sh.last_nonempty = -1;
  }
  __syncthreads();
  if (t < 256) {
    for (int x = 0; x < wp; ++x) {
      ic += sh.wsum_c[x];
      im += sh.wsum_m[x];
    }
    const bool hit = MASS ? (m > 0.f && im >= sh.dec.target) : (ic >= sh.dec.need);
    if (hit) atomicMin(&sh.pick, t);
    if (MASS && m > 0.f) atomicMax(&sh.last_nonempty, t);
  }
  __syncthreads();
  int pick = sh.pick;
  // MASS: rounding can leave the target just above the total; take the last bucket with any mass
  if (pick == 256) pick = MASS ? max(sh.last_nonempty, 0) : 255;
  if (t == pick) {
    const int accc = ic - c;
    const float accm = im - m;
    if (MASS) sh.dec.target -= accm;
    else sh.dec.need -= accc;
    sh.dec.above_cnt += accc;
    sh.dec.above_mass += accm;
    sh.dec.prefix = (sh.dec.prefix << 8) | (uint32_t)pick;
    sh.dec.level = level;
    sh.dec.ok = (c + (include_above ? sh.dec.above_cnt : 0)) <= CAP;
  }
  __syncthreads();
}

// Narrows the vocabulary to one bucket of the code; true when that bucket (plus everything above it
// when include_above) fits CAP.  The first CTA needs sh.cnt1 / sh.mass1 (level 0).  Result in sh.dec of
// every CTA.  Every CTA of the cluster must call it with the same arguments.
template <bool MASS>
__device__ bool bucket_select(cg::cluster_group& cl, unsigned rank, const float* w, int64_t lo, int64_t hi, float M,
                              float target_mass, int target_cnt, bool include_above, const Dyn& dy, Shared& sh) {
  if (threadIdx.x == 0) {
    Decision d;
    d.prefix = 0; d.level = 0; d.above_cnt = 0; d.above_mass = 0.f; d.ok = 0; d.target = target_mass; d.need = target_cnt;
    sh.dec = d;
  }
  __syncthreads();
  for (int level = 0; level < 3; ++level) {
    if (level > 0) {
      bucket_hist_partial(w, lo, hi, M, level, sh.dec.prefix, dy, sh);
      cl.sync();  // every share is complete
    }
    if (rank == 0) {
      if (level > 0) total_hists(cl, sh, sh.cntw, sh.massw);
      pick_bucket<MASS>(level == 0 ? sh.cnt1 : sh.cntw, level == 0 ? sh.mass1 : sh.massw, level, include_above, sh);
    }
    cl.sync();  // the decision is published; shares may be overwritten
    if (rank != 0) {
      if (threadIdx.x == 0) sh.dec = *cl.map_shared_rank(&sh.dec, 0);
      __syncthreads();
    }
    if (sh.dec.ok) return true;
  }
  return false;
}

// Bitonic sort of the first n2 (a power of two) candidates: value descending, index ascending.
__device__ void sort_candidates(const Dyn& dy, int n2) {
  for (int size = 2; size <= n2; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n2; i += ST) {
        const int j = i ^ stride;
        if (j > i) {
          const bool up = (i & size) == 0;
          const float vi = dy.cval[i], vj = dy.cval[j];
          const int ii = dy.cidx[i], ij = dy.cidx[j];
          const bool i_first = (vi > vj) || (vi == vj && ii < ij);  // i belongs before j
          if (up ? !i_first : i_first) {
            dy.cval[i] = vj; dy.cval[j] = vi;
            dy.cidx[i] = ij; dy.cidx[j] = ii;
          }
        }
      }
      __syncthreads();
    }
}

// Every CTA sends its elements of the selected bucket (and of everything above it when include_above)
// to the first CTA, which sorts them.  Returns the number gathered (meaningful in the first CTA).
__device__ int bucket_gather(cg::cluster_group& cl, unsigned rank, const float* w, int64_t lo, int64_t hi, float M,
                             bool include_above, const Dyn& dy, Shared& sh) {
  const uint32_t prefix = sh.dec.prefix;
  const int shift = 16 - 8 * sh.dec.level;
  if (rank == 0 && threadIdx.x == 0) sh.slot = 0;
  cl.sync();
  int* slot0 = cl.map_shared_rank(&sh.slot, 0);
  float* cval0 = cl.map_shared_rank(dy.cval, 0);
  int* cidx0 = cl.map_shared_rank(dy.cidx, 0);
  for_each_value(w, lo, hi, [&](int64_t i, float v) {
    const uint32_t c = bcode(v, M) >> shift;
    if (include_above ? c <= prefix : c == prefix) {
      const int s = atomicAdd(slot0, 1);
      if (s < CAP) {
        cval0[s] = v;
        cidx0[s] = (int)i;
      }
    }
  });
  cl.sync();
  if (rank != 0) return 0;
  const int n = min(sh.slot, CAP);
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  for (int i = n + threadIdx.x; i < n2; i += ST) {
    dy.cval[i] = -INFINITY;
    dy.cidx[i] = 0x7fffffff;
  }
  __syncthreads();
  sort_candidates(dy, n2);
  return n;
}

// First CTA: first position of the sorted candidates at which base + running mass reaches target
// (the last position when it never does); *cum_at = base + mass through that position.
__device__ int cum_find(const Dyn& dy, int n, float M, float base, float target, float* cum_at, Shared& sh) {
  const int t = threadIdx.x, lane = t & 31, wp = t >> 5;
  float e[CAP / ST];
  float run = 0.f;
#pragma unroll
  for (int u = 0; u < CAP / ST; ++u) {
    const int i = t * (CAP / ST) + u;
    run += (i < n) ? expf(dy.cval[i] - M) : 0.f;
    e[u] = run;  // inclusive within the thread
  }
  float inc = run;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float other = __shfl_up_sync(FULL, inc, o);
    if (lane >= o) inc += other;
  }
  if (lane == 31) sh.wsum_m[wp] = inc;
  if (t == 0) sh.first = 0x7fffffff;
  __syncthreads();
  float off = base + (inc - run);
  for (int x = 0; x < wp; ++x) off += sh.wsum_m[x];
#pragma unroll
  for (int u = 0; u < CAP / ST; ++u) {
    const int i = t * (CAP / ST) + u;
    if (i < n && off + e[u] >= target) {
      atomicMin(&sh.first, i);
      break;
    }
  }
  __syncthreads();
  int first = sh.first;
  if (first == 0x7fffffff) first = n - 1;
  if (first < 0 && t == 0) sh.nucleus = base;
#pragma unroll
  for (int u = 0; u < CAP / ST; ++u)
    if (first == t * (CAP / ST) + u) sh.nucleus = off + e[u];
  __syncthreads();
  *cum_at = sh.nucleus;
  return first;
}

// ---- exact path: radix select over the bits of the float itself --------------------------------

// Index of the `need`-th (1-based) element, in ascending index order, whose key equals `key`.
__device__ int nth_tie(const float* w, int64_t V, uint32_t key, int need, Shared& sh) {
  const int64_t chunk = (V + ST - 1) / ST;
  const int64_t lo = (int64_t)threadIdx.x * chunk, hi = min(V, lo + chunk);
  int cnt = 0;
  for (int64_t i = lo; i < hi; ++i) cnt += (fkey(w[i]) == key);
  int total;
  const int before = block_exclusive_scan(cnt, sh.scan, &total);
  if (threadIdx.x == 0) sh.result = -1;
  __syncthreads();
  if (need > total) need = total;
  if (need >= 1 && before < need && before + cnt >= need) {
    int seen = before;
    for (int64_t i = lo; i < hi; ++i)
      if (fkey(w[i]) == key && ++seen == need) {
        sh.result = (int)i;
        break;
      }
  }
  __syncthreads();
  return sh.result;
}

// First rank, in (value descending, index ascending) order, whose cumulative mass
// sum exp(w - M) reaches `target`.  Returns the token; *cum_out = mass through it.
__device__ int mass_select(const float* w, int64_t V, float M, float target, float* cum_out, const Dyn& dy, Shared& sh) {
  if (threadIdx.x == 0) {
    sh.sel_prefix = 0;
    sh.sel_target = target;
    sh.sel_above = 0.f;
  }
  __syncthreads();
  const int wp = threadIdx.x >> 5;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const uint32_t prefix = sh.sel_prefix;
    const uint32_t pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < NW * 256; i += ST) dy.hm[i] = 0.f;
    __syncthreads();
    for_each_value(w, 0, V, [&](int64_t, float v) {
      const uint32_t k = fkey(v);
      if ((k & pmask) == prefix) atomicAdd(&dy.hm[wp * 256 + ((k >> shift) & 255u)], expf(v - M));
    });
    __syncthreads();
    if (threadIdx.x < 256) {
      float m = 0.f;
      for (int x = 0; x < NW; ++x) m += dy.hm[x * 256 + threadIdx.x];
      sh.massw[threadIdx.x] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = 0.f;
      int pick = -1, last_nonempty = -1;
      for (int dgt = 255; dgt >= 0; --dgt) {
        const float m = sh.massw[dgt];
        if (m > 0.f) last_nonempty = dgt;
        if (acc + m >= sh.sel_target && m > 0.f) {
          pick = dgt;
          break;
        }
        acc += m;
      }
      if (pick < 0) {  // rounding left the target just above the total: take the lowest populated bin
        pick = max(last_nonempty, 0);
        acc -= sh.massw[pick];
      }
      sh.sel_target -= acc;
      sh.sel_above += acc;
      sh.sel_prefix = prefix | ((uint32_t)pick << shift);
    }
    __syncthreads();
  }
  // all elements with this exact key share one mass value
  const uint32_t key = sh.sel_prefix;
  const uint32_t kb = (key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key;
  const float mass = expf(__uint_as_float(kb) - M);
  int need = 1;
  if (mass > 0.f) need = max(1, (int)ceilf(sh.sel_target / mass));
  const float above = sh.sel_above;
  const int tok = nth_tie(w, V, key, need, sh);
  if (cum_out) *cum_out = above + (float)need * mass;
  return tok;
}

// The k largest (value descending, index ascending) into dy.cval / dy.cidx, sorted.
__device__ void exact_top_k(const float* w, int64_t V, int k, const Dyn& dy, Shared& sh) {
  // counting radix select: key T with count(key > T) < k <= count(key >= T)
  if (threadIdx.x == 0) {
    sh.sel_prefix = 0;
    sh.sel_need = k;
  }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const uint32_t prefix = sh.sel_prefix;
    const uint32_t pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    if (threadIdx.x < 256) sh.hist_i[threadIdx.x] = 0;
    __syncthreads();
    for_each_value(w, 0, V, [&](int64_t, float v) {
      const uint32_t kk = fkey(v);
      if ((kk & pmask) == prefix) {
        // one atomic per distinct digit in the warp: equal values would otherwise serialise
        const int bin = (int)((kk >> shift) & 255u);
        const unsigned act = __activemask();
        const unsigned same = __match_any_sync(act, bin);
        if ((int)(threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&sh.hist_i[bin], __popc(same));
      }
    });
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, pick = 0;
      for (int dgt = 255; dgt >= 0; --dgt) {
        if (acc + sh.hist_i[dgt] >= sh.sel_need) {
          pick = dgt;
          break;
        }
        acc += sh.hist_i[dgt];
      }
      sh.sel_need -= acc;
      sh.sel_prefix = prefix | ((uint32_t)pick << shift);
    }
    __syncthreads();
  }
  const uint32_t T = sh.sel_prefix;
  const int ties_needed = sh.sel_need;  // how many elements with key == T belong to the top k
  if (threadIdx.x == 0) sh.slot = 0;
  for (int i = threadIdx.x; i < MAX_TOPK; i += ST) {
    dy.cval[i] = -INFINITY;
    dy.cidx[i] = 0x7fffffff;
  }
  __syncthreads();
  for_each_value(w, 0, V, [&](int64_t i, float v) {
    if (fkey(v) > T) {
      const int s = atomicAdd(&sh.slot, 1);
      if (s < MAX_TOPK) {
        dy.cval[s] = v;
        dy.cidx[s] = (int)i;
      }
    }
  });
  __syncthreads();
  {  // ties in ascending index order: the first `ties_needed` of them
    const int64_t chunk = (V + ST - 1) / ST;
    const int64_t lo = (int64_t)threadIdx.x * chunk, hi = min(V, lo + chunk);
    int cnt = 0;
    for (int64_t i = lo; i < hi; ++i) cnt += (fkey(w[i]) == T);
    int total;
    int before = block_exclusive_scan(cnt, sh.scan, &total);
    const int base = sh.slot;
    for (int64_t i = lo; i < hi && before < ties_needed; ++i)
      if (fkey(w[i]) == T) {
        if (base + before < MAX_TOPK) {
          dy.cval[base + before] = w[i];
          dy.cidx[base + before] = (int)i;
        }
        ++before;
      }
  }
  __syncthreads();
  int n2 = 1;
  while (n2 < k) n2 <<= 1;
  sort_candidates(dy, n2);
}


// ---- the kernel --------------------------------------------------------------------------------

__global__ void __cluster_dims__(CS, 1, 1) __launch_bounds__(ST) sample_kernel(SampleArgs a) {
  extern __shared__ __align__(16) unsigned char dyn_raw[];
  __shared__ Shared sh;
  cg::cluster_group cl = cg::this_cluster();
  const unsigned rank = cl.block_rank();
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x / CS;
  if (a.active && a.active[b] == 0) return;  // an idle lane: the whole cluster leaves together
  const int64_t V = a.V;
  const int nwords = (int)((V + 31) / 32);
  Dyn dy;
  dy.bitmap = (uint32_t*)dyn_raw;
  dy.hc = (int*)(dyn_raw + (((size_t)nwords * 4 + 15) & ~(size_t)15));
  dy.hm = (float*)(dy.hc + NW * 256);
  dy.cval = dy.hm + NW * 256;
  dy.cidx = (int*)(dy.cval + CAP);
  const float* lg = a.logits + (int64_t)b * V;
  float* w = a.work + (int64_t)b * V;
  const int* hrow = a.hist + (int64_t)b * a.hist_cap;
  const int nseen = a.hist_len[b];
  const bool greedy = !a.do_sample || a.temperature <= 0.01f;
  const int wp = threadIdx.x >> 5;
  // this CTA's quarter of the row (whole float4s when the row allows 16-byte loads)
  const int64_t q = (V & 3) == 0 ? ((V / 4 + CS - 1) / CS) * 4 : (V + CS - 1) / CS;
  const int64_t lo = min(V, (int64_t)rank * q), hi = min(V, lo + q);

  const bool use_pen = a.rep_penalty != 1.0f;
  if (use_pen) {
    for (int i = threadIdx.x; i < nwords; i += ST) dy.bitmap[i] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < nseen; i += ST) {
      const int t = hrow[i];
      if (t >= 0 && t < V) atomicOr(&dy.bitmap[t >> 5], 1u << (t & 31));
    }
    __syncthreads();
  }

  // applySamplingConfig: penalty, temperature; then the maximum for min-p / softmax
  const float temp = fmaxf(a.temperature, 1e-6f);
  float mx = -INFINITY;
  for_each_value(lg, lo, hi, [&](int64_t i, float x) {
    if (use_pen && (dy.bitmap[i >> 5] >> (i & 31)) & 1u) return;  // seen tokens: below
    x = x / temp;
    w[i] = x;
    mx = fmaxf(mx, x);
  });
  if (use_pen) {
    // The reference walks the seen list, so a token is penalised once per occurrence.  The thread that
    // holds a token's first occurrence counts the others and writes that token's value.
    for (int j = threadIdx.x; j < nseen; j += ST) {
      const int t = hrow[j];
      if (t < lo || t >= hi) continue;  // another CTA's quarter (or out of range)
      bool first = true;
      for (int p = 0; p < j; ++p) first &= (hrow[p] != t);
      if (!first) continue;
      int cnt = 1;
      for (int p = j + 1; p < nseen; ++p) cnt += (hrow[p] == t);
      float x = lg[t];
      for (int r = 0; r < cnt; ++r) x = (x < 0.f) ? x * a.rep_penalty : x / a.rep_penalty;
      x = x / temp;
      w[t] = x;
      mx = fmaxf(mx, x);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
  if ((threadIdx.x & 31) == 0) sh.red[wp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = sh.red[0];
    for (int i = 1; i < 32; ++i) m = fmaxf(m, sh.red[i]);
    sh.part_f[0] = m;
  }
  cl.sync();
  mx = cl.map_shared_rank(&sh, 0)->part_f[0];
  for (unsigned r = 1; r < CS; ++r) mx = fmaxf(mx, cl.map_shared_rank(&sh, r)->part_f[0]);

  // min-p, the softmax denominator and (when sampling) the level-0 bucket histograms in one pass
  if (!greedy)
    for (int i = threadIdx.x; i < NW * 256; i += ST) {
      dy.hc[i] = 0;
      dy.hm[i] = 0.f;
    }
  __syncthreads();
  float sum = 0.f;
  const float thresh = a.min_p > 0.f ? mx + logf(a.min_p) : -INFINITY;
  for_each_value(w, lo, hi, [&](int64_t i, float x) {
    if (a.min_p > 0.f && x < thresh) {
      x = -INFINITY;
      w[i] = x;
    }
    const float e = expf(x - mx);
    sum += e;
    if (!greedy) {
      const int bin = (int)(bcode(x, mx) >> 16);
      atomicAdd(&dy.hc[wp * 256 + bin], 1);
      atomicAdd(&dy.hm[wp * 256 + bin], e);
    }
  });
  const float part_sum = block_reduce_sum(sum, sh.red);
  if (!greedy) fold_private_hists(dy, sh);
  if (threadIdx.x == 0) sh.part_f[1] = part_sum;
  cl.sync();  // (the maxima in part_f[0] have been read by everyone before this barrier)
  float sumExp = 0.f;
  for (unsigned r = 0; r < CS; ++r) sumExp += cl.map_shared_rank(&sh, r)->part_f[1];
  if (!greedy && rank == 0) total_hists(cl, sh, sh.cnt1, sh.mass1);
  cl.sync();  // shares may be overwritten from here on

  int tok = -1;  // meaningful in the first CTA
  if (greedy) {
    // sampleGreedy: first maximum
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for_each_value(w, lo, hi, [&](int64_t i, float v) {
      if (v > bv || (v == bv && (int)i < bi)) {
        bv = v;
        bi = (int)i;
      }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(FULL, bv, o);
      const int oi = __shfl_xor_sync(FULL, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
      sh.red[wp] = bv;
      sh.scan[wp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < 32; ++i)
        if (sh.red[i] > bv || (sh.red[i] == bv && sh.scan[i] < bi)) {
          bv = sh.red[i];
          bi = sh.scan[i];
        }
      sh.part_f[0] = bv;
      sh.part_i[0] = bi;
    }
    cl.sync();
    if (rank == 0) {
      if (threadIdx.x == 0) {
        float bv0 = -INFINITY;
        int bi0 = 0x7fffffff;
        for (unsigned r = 0; r < CS; ++r) {
          const Shared* rs = cl.map_shared_rank(&sh, r);
          const float v = rs->part_f[0];
          const int i = rs->part_i[0];
          if (v > bv0 || (v == bv0 && i < bi0)) {
            bv0 = v;
            bi0 = i;
          }
        }
        sh.result = (bi0 == 0x7fffffff) ? 0 : bi0;
      }
      __syncthreads();
      tok = sh.result;
    }
  } else {
    // u = uniformF32(key, 1, 0, 1)[0] = unit float of foldIn(key, 0).a
    uint32_t ua, ub;
    threefry2x32(a.keys[2 * b], a.keys[2 * b + 1], 0u, 0u, &ua, &ub);
    const float u = (float)(ua >> 8) * (1.0f / 16777216.0f);
    if (a.top_k > 0) {
      const int k = (int)min((int64_t)min(a.top_k, MAX_TOPK), V);
      if (!a.exact_only && bucket_select<false>(cl, rank, w, lo, hi, mx, 0.f, k, true, dy, sh)) {
        // everything down to the bucket of the k-th value, sorted in the first CTA
        bucket_gather(cl, rank, w, lo, hi, mx, true, dy, sh);
      } else if (rank == 0) {
        exact_top_k(w, V, k, dy, sh);
      }
      if (rank == 0) {
        if (threadIdx.x == 0) {
          // sampleTopK: exp without max subtraction, sequential sums, u <= cum
          float sumE = 0.f;
          for (int i = 0; i < k; ++i) sumE += expf(dy.cval[i]);
          float cum = 0.f;
          int pick = dy.cidx[k - 1];
          for (int i = 0; i < k; ++i) {
            cum += expf(dy.cval[i]) / sumE;
            if (u <= cum) {
              pick = dy.cidx[i];
              break;
            }
          }
          sh.result = pick;
        }
        __syncthreads();
        tok = sh.result;
      }
    } else {
      // sampleTopP: nucleus cutoff, then the draw inside the nucleus
      bool done = false;
      const float t1 = a.top_p * sumExp;
      if (!a.exact_only && bucket_select<true>(cl, rank, w, lo, hi, mx, t1, 0, false, dy, sh)) {
        int n = bucket_gather(cl, rank, w, lo, hi, mx, false, dy, sh);
        if (rank == 0) {
          float cum;
          cum_find(dy, n, mx, sh.dec.above_mass, t1, &cum, sh);  // leaves the nucleus mass in sh.nucleus
        }
        cl.sync();
        const float t2 = u * cl.map_shared_rank(&sh, 0)->nucleus;
        if (bucket_select<true>(cl, rank, w, lo, hi, mx, t2, 0, false, dy, sh)) {
          n = bucket_gather(cl, rank, w, lo, hi, mx, false, dy, sh);
          if (rank == 0) {
            float cum;
            const int at = cum_find(dy, n, mx, sh.dec.above_mass, t2, &cum, sh);
            tok = at >= 0 ? dy.cidx[at] : -1;
          }
          done = true;
        }
      }
      if (!done && rank == 0) {
        float nucleus = 0.f;
        mass_select(w, V, mx, t1, &nucleus, dy, sh);
        __syncthreads();
        nucleus = fminf(nucleus, sumExp);
        tok = mass_select(w, V, mx, u * nucleus, nullptr, dy, sh);
      }
    }
  }
  if (rank == 0) {
    __syncthreads();
    if (tok < 0 || tok >= V) {
      if (threadIdx.x == 0) atomicExch(a.status, KS_BAD_INDEX);
      tok = 0;
    }
    if (threadIdx.x == 0) {
      a.next[b] = tok;
      const int st = a.steps[b];
      a.steps[b] = st + 1;
      // w[tok] may have been written by another CTA of the cluster: read it from L2
      if (a.logprob && st < a.logprob_cap) a.logprob[(int64_t)b * a.logprob_cap + st] = __ldcg(&w[tok]) - mx - logf(sumExp);
      if (nseen < a.hist_cap) {
        a.hist[(int64_t)b * a.hist_cap + nseen] = tok;
        a.hist_len[b] = nseen + 1;
      }
      uint32_t na, nb;  // key = foldIn(key, step)
      threefry2x32(a.keys[2 * b], a.keys[2 * b + 1], (uint32_t)st, 0u, &na, &nb);
      a.keys[2 * b] = na;
      a.keys[2 * b + 1] = nb;
    }
  }
  cl.sync();  // no CTA leaves while another may still read its shared memory
}

}  // namespace

int sample_launch(Ctx* c, const float* logits, float* work, int64_t B, int64_t V, int* hist, int* hist_len, int hist_cap,
                  uint32_t* keys, int* steps, int* next, float* logprob, int logprob_cap, float temperature, int top_k,
                  float top_p, float min_p, float rep_penalty, int do_sample, const int* active) {
  if (B == 0) return REWB200_OK;
  SampleArgs a;
  a.logits = logits; a.work = work; a.V = V; a.hist = hist; a.hist_len = hist_len; a.hist_cap = hist_cap; a.keys = keys;
  a.steps = steps; a.next = next; a.logprob = logprob; a.logprob_cap = logprob_cap;
  a.temperature = temperature; a.top_p = top_p; a.min_p = min_p; a.rep_penalty = rep_penalty;
  a.top_k = top_k; a.do_sample = do_sample; a.exact_only = c->sampling_exact ? 1 : 0; a.active = active; a.status = c->d_status;
  const size_t bitmap_bytes = ((size_t)((V + 31) / 32) * 4 + 15) & ~(size_t)15;
  const size_t smem = bitmap_bytes + (size_t)NW * 256 * 8 + (size_t)CAP * 8;
  RB_REQUIRE(smem <= 200 * 1024, "sampling supports vocabularies up to about 800 000 tokens");
  static size_t cur = 0;
  if (smem > cur) {
    RB_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cur = smem;
  }
  RB_CUDA(launch_k(sample_kernel, dim3((unsigned)(B * CS)), dim3(ST), smem, c->stream, c->use_pdl, a));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace rewb
