// CPU restatement of Rechenwerk's (bitstormFA/rew) transformer-decoder inference
// path.  TEST INFRASTRUCTURE ONLY: this file is the parity checker and the timed
// CPU baseline.  The CUDA library never links, loads or calls it.
//
// Parity status: the primitive ops (add/mul/neg/exp/matmul/reduceSum/transpose/
// iota/broadcast) are pinned against the known-answer vectors in the
// reference's tests/teager_dispatch.nim and the generate loop against
// tests/tgenerate.nim.  For everything above the primitives (RoPE, norms,
// softmax, attention, GQA, SwiGLU, MoE routing, logits) the reference holds no
// golden vector and cannot be executed without its Nim toolchain and the XLA
// PJRT plugin, so for those layers: PARITY UNPINNED.  Each function restates
// the op sequence of the cited reference body, in the same order of
// elementwise operations; only the accumulation order inside dot products and
// reductions is this file's own (the reference leaves it to XLA).
//
// All tensors are row-major float32.  Sums run in double when accum64 is set
// (default) and in float, left to right, otherwise.

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

int g_accum64 = 1;

// ---------------------------------------------------------------- primitives

// src/rew/ops/linalg.nim:239-252 (matmul = dotGeneral contracting a.1 with b.0)
void matmul(const float* a, const float* b, float* out, int64_t M, int64_t K, int64_t N) {
  // Threads split the output columns, row blocks of 32 keep the accumulators in
  // cache; every (m, n) still sums over k in ascending order.
  constexpr int64_t NB = 128, MB = 32;
  const int64_t nblocks = (N + NB - 1) / NB;
#pragma omp parallel for schedule(dynamic)
  for (int64_t nb = 0; nb < nblocks; ++nb) {
    const int64_t n0 = nb * NB, nw = std::min(NB, N - n0);
    for (int64_t m0 = 0; m0 < M; m0 += MB) {
      const int64_t mw = std::min(MB, M - m0);
      if (g_accum64) {
        double acc[MB][NB];
        for (int64_t i = 0; i < mw; ++i)
          for (int64_t n = 0; n < nw; ++n) acc[i][n] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
          const float* br = b + k * N + n0;
          for (int64_t i = 0; i < mw; ++i) {
            const double av = a[(m0 + i) * K + k];
            for (int64_t n = 0; n < nw; ++n) acc[i][n] += av * (double)br[n];
          }
        }
        for (int64_t i = 0; i < mw; ++i)
          for (int64_t n = 0; n < nw; ++n) out[(m0 + i) * N + n0 + n] = (float)acc[i][n];
      } else {
        float acc[MB][NB];
        for (int64_t i = 0; i < mw; ++i)
          for (int64_t n = 0; n < nw; ++n) acc[i][n] = 0.f;
        for (int64_t k = 0; k < K; ++k) {
          const float* br = b + k * N + n0;
          for (int64_t i = 0; i < mw; ++i) {
            const float av = a[(m0 + i) * K + k];
            for (int64_t n = 0; n < nw; ++n) acc[i][n] += av * br[n];
          }
        }
        for (int64_t i = 0; i < mw; ++i)
          for (int64_t n = 0; n < nw; ++n) out[(m0 + i) * N + n0 + n] = acc[i][n];
      }
    }
  }
}

float sum_f(const float* x, int64_t n) {
  if (g_accum64) {
    double s = 0;
    for (int64_t i = 0; i < n; ++i) s += x[i];
    return (float)s;
  }
  float s = 0;
  for (int64_t i = 0; i < n; ++i) s += x[i];
  return s;
}

float dot_f(const float* a, const float* b, int64_t n) {
  if (g_accum64) {
    double s = 0;
    for (int64_t i = 0; i < n; ++i) s += (double)a[i] * (double)b[i];
    return (float)s;
  }
  float s = 0;
  for (int64_t i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

// src/rew/nn/linear.nim:43-49: matmul, broadcast bias over rows, add.
void linear(const float* x, const float* W, const float* b, float* y, int64_t N, int64_t in,
            int64_t out) {
  matmul(x, W, y, N, in, out);
  for (int64_t n = 0; n < N; ++n)
    for (int64_t o = 0; o < out; ++o) y[n * out + o] = y[n * out + o] + b[o];
}

// src/rew/nn/norm.nim:204-224: sq = x*x; meanSq = sum(sq)/float32(d)
// (ops/reduce.nim:132-150); rms = sqrt(meanSq + eps); out = gamma * (x / rms).
void rmsnorm(const float* x, const float* gamma, float eps, float* out, int64_t rows, int64_t d) {
  std::vector<float> sq(d);
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * d;
    for (int64_t i = 0; i < d; ++i) sq[i] = xr[i] * xr[i];
    const float meanSq = sum_f(sq.data(), d) / (float)d;
    const float rms = std::sqrt(meanSq + eps);
    for (int64_t i = 0; i < d; ++i) out[r * d + i] = gamma[i] * (xr[i] / rms);
  }
}

// src/rew/nn/norm.nim:41-84: mean; centered; biased variance; rsqrt(var+eps);
// gamma * (centered * invStd) + beta.
void layernorm(const float* x, const float* gamma, const float* beta, float eps, float* out,
               int64_t rows, int64_t d) {
  std::vector<float> c(d), sq(d);
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * d;
    const float mean = sum_f(xr, d) / (float)d;
    for (int64_t i = 0; i < d; ++i) {
      c[i] = xr[i] - mean;
      sq[i] = c[i] * c[i];
    }
    const float var = sum_f(sq.data(), d) / (float)d;
    const float invStd = 1.0f / std::sqrt(var + eps);
    for (int64_t i = 0; i < d; ++i) out[r * d + i] = gamma[i] * (c[i] * invStd) + beta[i];
  }
}

void norm_any(int kind, const float* x, const float* g, const float* b, float eps, float* out,
              int64_t rows, int64_t d) {
  if (kind == 0) rmsnorm(x, g, eps, out, rows, d);
  else layernorm(x, g, b, eps, out, rows, d);
}

// src/rew/nn/rope.nim:112-145: invFreq_i = 1f / float32(pow(theta, 2i/hd)) with
// the pow in double; angle = float32(pos) * invFreq in float; cos/sin of the
// float angle; each value stored twice (positions 2i and 2i+1).
void rope_tables(int hd, int maxSeq, double theta, float* cosT, float* sinT) {
  const int half = hd / 2;
  std::vector<float> invFreq(half);
  for (int i = 0; i < half; ++i) {
    const double exponent = (double)(2 * i) / (double)hd;
    invFreq[i] = 1.0f / (float)std::pow(theta, exponent);
  }
  for (int pos = 0; pos < maxSeq; ++pos) {
    const float fp = (float)pos;
    for (int i = 0; i < half; ++i) {
      const float angle = fp * invFreq[i];
      const int64_t base = (int64_t)pos * hd + 2 * i;
      cosT[base] = std::cos(angle);
      cosT[base + 1] = std::cos(angle);
      sinT[base] = std::sin(angle);
      sinT[base + 1] = std::sin(angle);
    }
  }
}

// src/rew/nn/rope.nim:153-179 (table rows offset..offset+S) and :56-108
// (x0' = cos0*x0 - sin0*x1 ; x1' = sin0*x0 + cos0*x1 on interleaved pairs,
// cos0/sin0 = component 0 of the duplicated table).  x: [lead, S, hd].
void rope_apply(const float* x, float* out, const float* cosT, const float* sinT, int64_t lead,
                int64_t S, int hd, int64_t offset) {
  const int half = hd / 2;
  for (int64_t l = 0; l < lead; ++l)
    for (int64_t s = 0; s < S; ++s) {
      const float* xr = x + (l * S + s) * hd;
      float* orow = out + (l * S + s) * hd;
      const float* c = cosT + (offset + s) * hd;
      const float* sn = sinT + (offset + s) * hd;
      for (int i = 0; i < half; ++i) {
        const float x0 = xr[2 * i], x1 = xr[2 * i + 1];
        const float c0 = c[2 * i], s0 = sn[2 * i];
        orow[2 * i] = c0 * x0 - s0 * x1;
        orow[2 * i + 1] = s0 * x0 + c0 * x1;
      }
    }
}

// src/rew/nn/activation.nim:64-77: max, subtract, exp, sum, divide.
void softmax_rows(float* x, int64_t rows, int64_t n) {
  std::vector<float> e(n);
  for (int64_t r = 0; r < rows; ++r) {
    float* xr = x + r * n;
    float mx = -INFINITY;
    for (int64_t i = 0; i < n; ++i) mx = std::max(mx, xr[i]);
    for (int64_t i = 0; i < n; ++i) e[i] = std::exp(xr[i] - mx);
    const float s = sum_f(e.data(), n);
    for (int64_t i = 0; i < n; ++i) xr[i] = e[i] / s;
  }
}

// src/rew/nn/attention.nim:18-34 as written: 0 where row <= col, -1e9 where
// row > col.  mask_kind 1 is the conventional causal mask for a query block
// that ends at the last key: key j visible to query i iff j <= i + (L - S).
inline float mask_value(int mask_kind, int64_t i, int64_t j, int64_t S, int64_t L) {
  if (mask_kind == 0) return (i <= j) ? 0.0f : -1e9f;
  return (j <= i + (L - S)) ? 0.0f : -1e9f;
}

// src/rew/nn/attention.nim:36-81.  q [G,S,hd], k,v [G,L,hd] -> out [G,S,hd].
// scores = q.k ; scores *= 1/sqrt(hd) ; + mask ; softmax ; attn.v
void sdpa(const float* q, const float* k, const float* v, float* out, int64_t G, int64_t S,
          int64_t L, int hd, int causal, int mask_kind, float scale) {
  const float sc = (scale != 0.f) ? scale : 1.0f / std::sqrt((float)hd);
#pragma omp parallel for schedule(dynamic)
  for (int64_t g = 0; g < G; ++g) {
    std::vector<float> scores(S * L);
    for (int64_t i = 0; i < S; ++i)
      for (int64_t j = 0; j < L; ++j) {
        float s = dot_f(q + (g * S + i) * hd, k + (g * L + j) * hd, hd);
        s = s * sc;
        if (causal) s = s + mask_value(mask_kind, i, j, S, L);
        scores[i * L + j] = s;
      }
    softmax_rows(scores.data(), S, L);
    for (int64_t i = 0; i < S; ++i)
      for (int d = 0; d < hd; ++d) {
        if (g_accum64) {
          double acc = 0;
          for (int64_t j = 0; j < L; ++j) acc += (double)scores[i * L + j] * v[(g * L + j) * hd + d];
          out[(g * S + i) * hd + d] = (float)acc;
        } else {
          float acc = 0;
          for (int64_t j = 0; j < L; ++j) acc += scores[i * L + j] * v[(g * L + j) * hd + d];
          out[(g * S + i) * hd + d] = acc;
        }
      }
  }
}

// src/rew/nn/activation.nim:28-38: sigmoid = 1 / (1 + exp(-x)); silu = x * sigmoid.
inline float silu(float x) {
  const float e = std::exp(-x);
  const float sig = 1.0f / (1.0f + e);
  return x * sig;
}

// [N, H*hd] (projection output) -> [B,H,S,hd]; groupedqueryattention.nim:106-113.
void split_heads(const float* flat, float* out, int64_t B, int64_t S, int H, int hd) {
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int h = 0; h < H; ++h)
        std::memcpy(out + ((b * H + h) * S + s) * hd, flat + ((b * S + s) * H + h) * hd,
                    sizeof(float) * hd);
}

struct Cfg {
  int32_t vocab, d_model, n_layers, n_heads, n_kv_heads, head_dim, ffn, max_seq;
  double theta;
  float eps;
  int32_t norm_kind;   // 0 = rmsNorm math (nn/norm.nim:204-224), 1 = LayerNorm (nn/norm.nim:41-84)
  int32_t mask_kind;   // 0 = makeCausalMask as written, 1 = conventional causal
  int32_t n_routed, n_shared, top_k, moe_ffn, first_dense;  // n_routed == 0: dense Llama block
};

// Tensor order (every Linear has weight [in,out] then bias [out]):
//   0 embed [V,d]
//   per layer: ln1.gamma ln1.beta  q.w q.b k.w k.b v.w v.b o.w o.b  ln2.gamma ln2.beta
//              dense block:  gate.w gate.b up.w up.b down.w down.b
//              MoE block:    router.w router.b, then for each shared expert and each routed
//                            expert: gate.w gate.b up.w up.b down.w down.b
//   final: norm.gamma norm.beta lm_head.w lm_head.b
struct LayerW {
  const float *ln1g, *ln1b, *qw, *qb, *kw, *kb, *vw, *vb, *ow, *ob, *ln2g, *ln2b;
  bool moe;
  const float *gw, *gb, *uw, *ub, *dw, *db;  // dense
  const float *rw, *rb;                        // router
  std::vector<const float*> ex;                // experts: 6 pointers each, shared first
};

struct Model {
  Cfg c;
  const float* embed;
  std::vector<LayerW> layers;
  const float *ng, *nb, *lw, *lb;
  std::vector<float> cosT, sinT;
};

bool layer_is_moe(const Cfg& c, int l) { return c.n_routed > 0 && !(c.first_dense > 0 && l == 0); }

int64_t tensor_count(const Cfg& c) {
  int64_t n = 1;
  for (int l = 0; l < c.n_layers; ++l) {
    n += 12;
    if (layer_is_moe(c, l)) n += 2 + 6 * (int64_t)(c.n_shared + c.n_routed);
    else n += 6;
  }
  return n + 4;
}

Model build(const Cfg& c, const float* const* t) {
  Model m;
  m.c = c;
  int64_t i = 0;
  m.embed = t[i++];
  m.layers.resize(c.n_layers);
  for (int l = 0; l < c.n_layers; ++l) {
    LayerW& L = m.layers[l];
    L.ln1g = t[i++]; L.ln1b = t[i++];
    L.qw = t[i++]; L.qb = t[i++]; L.kw = t[i++]; L.kb = t[i++];
    L.vw = t[i++]; L.vb = t[i++]; L.ow = t[i++]; L.ob = t[i++];
    L.ln2g = t[i++]; L.ln2b = t[i++];
    L.moe = layer_is_moe(c, l);
    if (!L.moe) {
      L.gw = t[i++]; L.gb = t[i++]; L.uw = t[i++]; L.ub = t[i++]; L.dw = t[i++]; L.db = t[i++];
    } else {
      L.rw = t[i++]; L.rb = t[i++];
      for (int e = 0; e < 6 * (c.n_shared + c.n_routed); ++e) L.ex.push_back(t[i++]);
    }
  }
  m.ng = t[i++]; m.nb = t[i++]; m.lw = t[i++]; m.lb = t[i++];
  m.cosT.resize((size_t)c.max_seq * c.head_dim);
  m.sinT.resize((size_t)c.max_seq * c.head_dim);
  rope_tables(c.head_dim, c.max_seq, c.theta, m.cosT.data(), m.sinT.data());
  return m;
}

// src/rew/nn/gated_ffn.nim:46-67 and src/rew/models/deepseek.nim:74-78.
void gated_ffn(const float* x, const float* gw, const float* gb, const float* uw, const float* ub,
               const float* dw, const float* db, float* out, int64_t N, int64_t d, int64_t f) {
  std::vector<float> g(N * f), u(N * f);
  linear(x, gw, gb, g.data(), N, d, f);
  linear(x, uw, ub, u.data(), N, d, f);
  for (int64_t i = 0; i < N * f; ++i) g[i] = silu(g[i]) * u[i];
  linear(g.data(), dw, db, out, N, f, d);
}

// src/rew/ops/sort.nim:36-90: stable descending sort, first k.  The reference
// comparator is the non-strict GE under a stable sort, which leaves the order
// of exact ties to XLA; here ties keep ascending index order.
void topk_rows(const float* p, int64_t rows, int E, int k, float* vals, int32_t* idx) {
  std::vector<int32_t> order(E);
  for (int64_t r = 0; r < rows; ++r) {
    std::iota(order.begin(), order.end(), 0);
    const float* pr = p + r * E;
    std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return pr[a] > pr[b]; });
    for (int j = 0; j < k; ++j) {
      idx[r * k + j] = order[j];
      vals[r * k + j] = pr[order[j]];
    }
  }
}

// Router: src/rew/models/deepseek.nim:132-138 (softmax over experts, topK,
// divide by the sum of the selected probabilities).
void moe_route(const float* x, const float* rw, const float* rb, int64_t N, int64_t d, int E, int k,
               float* topw, int32_t* topi) {
  std::vector<float> logits(N * E);
  linear(x, rw, rb, logits.data(), N, d, E);
  softmax_rows(logits.data(), N, E);
  topk_rows(logits.data(), N, E, k, topw, topi);
  for (int64_t n = 0; n < N; ++n) {
    const float denom = sum_f(topw + n * k, k);
    for (int j = 0; j < k; ++j) topw[n * k + j] = topw[n * k + j] / denom;
  }
}

// src/rew/models/deepseek.nim:122-145: shared experts summed, then EVERY
// routed expert evaluated on every token and scaled by
// weight[n] = sum_j topW[n,j] * (topIdx[n,j] == e) (:114-120).
// Optional record of every MoE layer's routing during a forward (tests compare it with the device's).
struct RouteRec {
  std::vector<std::vector<int32_t>> topi;   // per MoE layer [N][k]
  std::vector<std::vector<float>> topw;
};
static RouteRec* g_route_rec = nullptr;

void moe_forward(const Cfg& c, const LayerW& L, const float* x, float* out, int64_t N) {
  const int64_t d = c.d_model, f = c.moe_ffn;
  std::vector<float> tmp(N * d);
  std::fill(out, out + N * d, 0.f);
  for (int s = 0; s < c.n_shared; ++s) {
    const float* const* e = &L.ex[6 * s];
    gated_ffn(x, e[0], e[1], e[2], e[3], e[4], e[5], tmp.data(), N, d, f);
    if (s == 0) std::copy(tmp.begin(), tmp.end(), out);
    else for (int64_t i = 0; i < N * d; ++i) out[i] = out[i] + tmp[i];
  }
  std::vector<float> topw(N * c.top_k);
  std::vector<int32_t> topi(N * c.top_k);
  moe_route(x, L.rw, L.rb, N, d, c.n_routed, c.top_k, topw.data(), topi.data());
  if (g_route_rec) {
    g_route_rec->topi.push_back(topi);
    g_route_rec->topw.push_back(topw);
  }
  std::vector<float> w(N);
  for (int e = 0; e < c.n_routed; ++e) {
    bool any = false;
    for (int64_t n = 0; n < N; ++n) {
      float s = 0.f;
      for (int j = 0; j < c.top_k; ++j) s += topw[n * c.top_k + j] * (topi[n * c.top_k + j] == e ? 1.f : 0.f);
      w[n] = s;
      any |= (s != 0.f);
    }
    // expert(x) * 0 adds exactly 0 for finite values, so idle experts are skipped.
    if (!any) continue;
    const float* const* p = &L.ex[6 * (c.n_shared + e)];
    gated_ffn(x, p[0], p[1], p[2], p[3], p[4], p[5], tmp.data(), N, d, f);
    for (int64_t n = 0; n < N; ++n)
      for (int64_t i = 0; i < d; ++i) out[n * d + i] = out[n * d + i] + tmp[n * d + i] * w[n];
  }
}

// Per-layer KV state of the composed cached driver ([B,kvh,len,hd] as
// src/rew/nn/kv_cache.nim:13-24; append = concatenate on dim 2, :47-77).
struct KV {
  std::vector<float> k, v;
  int64_t len = 0;
};

void kv_append(KV& c, const float* kNew, const float* vNew, int64_t B, int H, int64_t S, int hd) {
  const int64_t newLen = c.len + S;
  std::vector<float> k2(B * H * newLen * hd), v2(B * H * newLen * hd);
  for (int64_t g = 0; g < B * H; ++g) {
    std::memcpy(&k2[g * newLen * hd], c.k.data() + g * c.len * hd, sizeof(float) * c.len * hd);
    std::memcpy(&v2[g * newLen * hd], c.v.data() + g * c.len * hd, sizeof(float) * c.len * hd);
    std::memcpy(&k2[(g * newLen + c.len) * hd], kNew + g * S * hd, sizeof(float) * S * hd);
    std::memcpy(&v2[(g * newLen + c.len) * hd], vNew + g * S * hd, sizeof(float) * S * hd);
  }
  c.k.swap(k2);
  c.v.swap(v2);
  c.len = newLen;
}

// One attention block on hidden states h [B,S,d].  With kv == nullptr this is
// GroupedQueryAttention.forward as written (groupedqueryattention.nim:75-144):
// K/V come from the same S tokens.  With a cache it is the composition the
// reference leaves to the caller: project the new tokens, RoPE q and k at
// `offset`, append post-RoPE K and V to the cache, attend over the whole cache.
void gqa_block(const Model& m, const LayerW& L, const float* h, float* out, int64_t B, int64_t S,
               int64_t offset, int causal, KV* kv) {
  const Cfg& c = m.c;
  const int nh = c.n_heads, kvh = c.n_kv_heads, hd = c.head_dim, group = nh / kvh;
  const int64_t N = B * S, d = c.d_model;
  std::vector<float> qf(N * nh * hd), kf(N * kvh * hd), vf(N * kvh * hd);
  linear(h, L.qw, L.qb, qf.data(), N, d, nh * hd);
  linear(h, L.kw, L.kb, kf.data(), N, d, kvh * hd);
  linear(h, L.vw, L.vb, vf.data(), N, d, kvh * hd);
  std::vector<float> q(qf.size()), k(kf.size()), v(vf.size());
  split_heads(qf.data(), q.data(), B, S, nh, hd);
  split_heads(kf.data(), k.data(), B, S, kvh, hd);
  split_heads(vf.data(), v.data(), B, S, kvh, hd);
  std::vector<float> qr(q.size()), kr(k.size());
  rope_apply(q.data(), qr.data(), m.cosT.data(), m.sinT.data(), B * nh, S, hd, offset);
  rope_apply(k.data(), kr.data(), m.cosT.data(), m.sinT.data(), B * kvh, S, hd, offset);
  const float *kk = kr.data(), *vv = v.data();
  int64_t Lkv = S;
  if (kv) {
    kv_append(*kv, kr.data(), v.data(), B, kvh, S, hd);
    kk = kv->k.data();
    vv = kv->v.data();
    Lkv = kv->len;
  }
  // head expand (groupedqueryattention.nim:126-133): query head h uses kv head h / group.
  std::vector<float> kx(B * nh * Lkv * hd), vx(B * nh * Lkv * hd);
  for (int64_t b = 0; b < B; ++b)
    for (int hh = 0; hh < nh; ++hh) {
      std::memcpy(&kx[(b * nh + hh) * Lkv * hd], kk + (b * kvh + hh / group) * Lkv * hd, sizeof(float) * Lkv * hd);
      std::memcpy(&vx[(b * nh + hh) * Lkv * hd], vv + (b * kvh + hh / group) * Lkv * hd, sizeof(float) * Lkv * hd);
    }
  std::vector<float> a(B * nh * S * hd);
  sdpa(qr.data(), kx.data(), vx.data(), a.data(), B * nh, S, Lkv, hd, causal, c.mask_kind, 0.f);
  std::vector<float> flat(N * nh * hd);
  for (int64_t b = 0; b < B; ++b)
    for (int hh = 0; hh < nh; ++hh)
      for (int64_t s = 0; s < S; ++s)
        std::memcpy(&flat[((b * S + s) * nh + hh) * hd], &a[((b * nh + hh) * S + s) * hd], sizeof(float) * hd);
  linear(flat.data(), L.ow, L.ob, out, N, nh * hd, d);
}

// src/rew/models/llama.nim:106-117 and src/rew/models/deepseek.nim:198-215.
void decoder_layer(const Model& m, const LayerW& L, float* h, int64_t B, int64_t S, int64_t offset,
                   int causal, KV* kv) {
  const Cfg& c = m.c;
  const int64_t N = B * S, d = c.d_model;
  std::vector<float> normed(N * d), attn(N * d), mlp(N * d);
  norm_any(c.norm_kind, h, L.ln1g, L.ln1b, c.eps, normed.data(), N, d);
  gqa_block(m, L, normed.data(), attn.data(), B, S, offset, causal, kv);
  for (int64_t i = 0; i < N * d; ++i) h[i] = h[i] + attn[i];
  norm_any(c.norm_kind, h, L.ln2g, L.ln2b, c.eps, normed.data(), N, d);
  if (L.moe) moe_forward(c, L, normed.data(), mlp.data(), N);
  else gated_ffn(normed.data(), L.gw, L.gb, L.uw, L.ub, L.dw, L.db, mlp.data(), N, d,
                 (c.n_routed > 0 && c.first_dense > 0) ? c.first_dense : c.ffn);
  for (int64_t i = 0; i < N * d; ++i) h[i] = h[i] + mlp[i];
}

// Embedding.forward is one-hot @ table (src/rew/nn/embedding.nim:39-62).  Adding
// 0*w for every other row changes nothing for finite w, so this is a row copy.
void embed(const Model& m, const int32_t* ids, float* h, int64_t N) {
  for (int64_t n = 0; n < N; ++n)
    std::memcpy(h + n * m.c.d_model, m.embed + (int64_t)ids[n] * m.c.d_model, sizeof(float) * m.c.d_model);
}

// Backbone + final norm (llama.nim:119-129); hidden [B,S,d] returned in h.
void backbone(const Model& m, const int32_t* ids, float* h, int64_t B, int64_t S, int64_t offset,
              int causal, std::vector<KV>* kvs) {
  embed(m, ids, h, B * S);
  for (int l = 0; l < m.c.n_layers; ++l)
    decoder_layer(m, m.layers[l], h, B, S, offset, causal, kvs ? &(*kvs)[l] : nullptr);
  std::vector<float> out(B * S * m.c.d_model);
  norm_any(m.c.norm_kind, h, m.ng, m.nb, m.c.eps, out.data(), B * S, m.c.d_model);
  std::copy(out.begin(), out.end(), h);
}

// src/rew/infer/generate.nim:152-159: first maximum wins.
int32_t sample_greedy(const float* logits, int64_t n) {
  int64_t best = 0;
  for (int64_t i = 0; i < n; ++i)
    if (logits[i] > logits[best]) best = i;
  return (int32_t)best;
}

}  // namespace

// ------------------------------------------------------------------ C ABI

ORC_API void orc_set_accum64(int on) { g_accum64 = on; }
ORC_API int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Worker threads of the OpenMP loops (a launcher may have exported OMP_NUM_THREADS=1 for every rank).
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

// src/rew/ops/literal.nim:112-116: round-to-nearest-even on the bit pattern.
ORC_API void orc_bf16_round(const float* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t bits;
    std::memcpy(&bits, in + i, 4);
    const uint32_t roundBias = 0x7FFFu + ((bits >> 16) & 1u);
    bits += roundBias;
    bits &= 0xFFFF0000u;
    std::memcpy(out + i, &bits, 4);
  }
}

// Elementwise primitives (src/rew/ops/arith.nim:49-64, ops/unary.nim:29-40).
ORC_API void orc_binary(int op, const float* a, const float* b, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    switch (op) {
      case 0: out[i] = a[i] + b[i]; break;
      case 1: out[i] = a[i] - b[i]; break;
      case 2: out[i] = a[i] * b[i]; break;
      default: out[i] = a[i] / b[i]; break;
    }
  }
}
ORC_API void orc_unary(int op, const float* a, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    switch (op) {
      case 0: out[i] = -a[i]; break;
      case 1: out[i] = std::exp(a[i]); break;
      case 2: out[i] = std::sqrt(a[i]); break;
      case 3: out[i] = 1.0f / std::sqrt(a[i]); break;
      default: out[i] = 1.0f / (1.0f + std::exp(-a[i])); break;  // logistic
    }
  }
}
ORC_API void orc_matmul(const float* a, const float* b, float* out, int64_t M, int64_t K, int64_t N) {
  matmul(a, b, out, M, K, N);
}
ORC_API float orc_reduce_sum(const float* a, int64_t n) { return sum_f(a, n); }
// src/rew/ops/shape.nim:45-76 (rank-2 case).
ORC_API void orc_transpose2d(const float* a, float* out, int64_t R, int64_t C) {
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < C; ++c) out[c * R + r] = a[r * C + c];
}
// src/rew/ops/shape.nim:295-323 (rank-2 case): value = index along `dim`.
ORC_API void orc_iota2d(int32_t* out, int64_t R, int64_t C, int dim) {
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < C; ++c) out[r * C + c] = (int32_t)(dim == 0 ? r : c);
}

ORC_API void orc_linear(const float* x, const float* W, const float* b, float* y, int64_t N, int64_t in,
                        int64_t out) {
  linear(x, W, b, y, N, in, out);
}
ORC_API void orc_rmsnorm(const float* x, const float* g, float eps, float* out, int64_t rows, int64_t d) {
  rmsnorm(x, g, eps, out, rows, d);
}
ORC_API void orc_layernorm(const float* x, const float* g, const float* b, float eps, float* out,
                           int64_t rows, int64_t d) {
  layernorm(x, g, b, eps, out, rows, d);
}
ORC_API void orc_rope_tables(int hd, int maxSeq, double theta, float* cosT, float* sinT) {
  rope_tables(hd, maxSeq, theta, cosT, sinT);
}
ORC_API void orc_rope_apply(const float* x, float* out, const float* cosT, const float* sinT, int64_t lead,
                            int64_t S, int hd, int64_t offset) {
  rope_apply(x, out, cosT, sinT, lead, S, hd, offset);
}
ORC_API void orc_softmax(float* x, int64_t rows, int64_t n) { softmax_rows(x, rows, n); }
ORC_API void orc_causal_mask(float* out, int64_t S, int64_t L, int mask_kind) {
  for (int64_t i = 0; i < S; ++i)
    for (int64_t j = 0; j < L; ++j) out[i * L + j] = mask_value(mask_kind, i, j, S, L);
}
ORC_API void orc_sdpa(const float* q, const float* k, const float* v, float* out, int64_t G, int64_t S,
                      int64_t L, int hd, int causal, int mask_kind, float scale) {
  sdpa(q, k, v, out, G, S, L, hd, causal, mask_kind, scale);
}
// Attention over [B,nh,S,hd] queries and [B,kvh,L,hd] keys/values with the
// reference's head expansion (groupedqueryattention.nim:126-133).
ORC_API void orc_gqa_attention(const float* q, const float* k, const float* v, float* out, int64_t B, int nh,
                               int kvh, int64_t S, int64_t L, int hd, int causal, int mask_kind) {
  const int group = nh / kvh;
  std::vector<float> kx(B * nh * L * hd), vx(B * nh * L * hd);
  for (int64_t b = 0; b < B; ++b)
    for (int h = 0; h < nh; ++h) {
      std::memcpy(&kx[(b * nh + h) * L * hd], k + (b * kvh + h / group) * L * hd, sizeof(float) * L * hd);
      std::memcpy(&vx[(b * nh + h) * L * hd], v + (b * kvh + h / group) * L * hd, sizeof(float) * L * hd);
    }
  sdpa(q, kx.data(), vx.data(), out, B * nh, S, L, hd, causal, mask_kind, 0.f);
}
ORC_API void orc_silu(const float* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = silu(x[i]);
}
ORC_API void orc_gated_ffn(const float* x, const float* gw, const float* gb, const float* uw, const float* ub,
                           const float* dw, const float* db, float* out, int64_t N, int64_t d, int64_t f) {
  gated_ffn(x, gw, gb, uw, ub, dw, db, out, N, d, f);
}
// One-hot @ table, literally (nn/embedding.nim:39-62 with nn/activation.nim:205-228).
ORC_API void orc_embedding_onehot(const int32_t* ids, const float* table, float* out, int64_t N, int64_t V,
                                  int64_t d) {
  std::vector<float> onehot(N * V, 0.f);
  for (int64_t n = 0; n < N; ++n) onehot[n * V + ids[n]] = 1.f;
  matmul(onehot.data(), table, out, N, V, d);
}
ORC_API void orc_topk(const float* p, int64_t rows, int E, int k, float* vals, int32_t* idx) {
  topk_rows(p, rows, E, k, vals, idx);
}
ORC_API void orc_moe_route(const float* x, const float* rw, const float* rb, int64_t N, int64_t d, int E, int k,
                           float* topw, int32_t* topi) {
  moe_route(x, rw, rb, N, d, E, k, topw, topi);
}

ORC_API int64_t orc_tensor_count(const Cfg* c) { return tensor_count(*c); }

// Whole-model forward without a cache, as LlamaForCausalLM.forward /
// DeepSeekForCausalLM.forward are written (llama.nim:131-140,
// deepseek.nim:217-231): logits for every position, [B,S,V].
ORC_API void orc_model_forward(const Cfg* c, const float* const* tensors, const int32_t* ids, int64_t B,
                               int64_t S, int64_t offset, int causal, float* logits) {
  Model m = build(*c, tensors);
  std::vector<float> h(B * S * c->d_model);
  backbone(m, ids, h.data(), B, S, offset, causal, nullptr);
  linear(h.data(), m.lw, m.lb, logits, B * S, c->d_model, c->vocab);
}

// The same forward, returning what every MoE layer's router chose: topi / topw [n_moe_layers][B*S][k].
ORC_API void orc_model_routing(const Cfg* c, const float* const* tensors, const int32_t* ids, int64_t B, int64_t S,
                               int64_t offset, int causal, int32_t* topi, float* topw) {
  Model m = build(*c, tensors);
  std::vector<float> h(B * S * c->d_model);
  RouteRec rec;
  g_route_rec = &rec;
  backbone(m, ids, h.data(), B, S, offset, causal, nullptr);
  g_route_rec = nullptr;
  const size_t per = (size_t)B * S * c->top_k;
  for (size_t l = 0; l < rec.topi.size(); ++l) {
    std::memcpy(topi + l * per, rec.topi[l].data(), per * sizeof(int32_t));
    std::memcpy(topw + l * per, rec.topw[l].data(), per * sizeof(float));
  }
}

// Hidden states after the final norm for one MoE/dense block stack; used by tests.
ORC_API void orc_moe_layer(const Cfg* c, const float* const* tensors, int layer, const float* x, float* out,
                           int64_t N) {
  Model m = build(*c, tensors);
  moe_forward(*c, m.layers[layer], x, out, N);
}

// Greedy generation with a KV cache, composed as the reference's pieces allow:
// generate() (infer/generate.nim:231-265) feeds the whole prompt at offset 0,
// then one token at a time at offset = tokens so far; the forward is the
// cached composition described at gqa_block; only the last position's logits
// are used (generate.nim:172-190); greedy = first max (:152-159).  EOS and
// stop tokens are disabled when eos < 0.  prompt [B,S] -> out_ids [B,n_new];
// last_logits [B,V] = logits that chose the final token; all_logits (optional)
// [n_new,B,V].
ORC_API void orc_generate_greedy(const Cfg* c, const float* const* tensors, const int32_t* prompt, int64_t B,
                                 int64_t S, int n_new, int eos, int32_t* out_ids, float* last_logits,
                                 float* all_logits) {
  Model m = build(*c, tensors);
  const int64_t d = c->d_model, V = c->vocab;
  std::vector<KV> kvs(c->n_layers);
  std::vector<int32_t> cur(prompt, prompt + B * S);
  int64_t curS = S, offset = 0;
  std::vector<float> logits(B * V);
  for (int step = 0; step < n_new; ++step) {
    std::vector<float> h(B * curS * d), last(B * d);
    backbone(m, cur.data(), h.data(), B, curS, offset, /*causal=*/1, &kvs);
    for (int64_t b = 0; b < B; ++b) std::memcpy(&last[b * d], &h[(b * curS + curS - 1) * d], sizeof(float) * d);
    linear(last.data(), m.lw, m.lb, logits.data(), B, d, V);
    if (all_logits) std::memcpy(all_logits + (int64_t)step * B * V, logits.data(), sizeof(float) * B * V);
    std::vector<int32_t> next(B);
    bool stop = false;
    for (int64_t b = 0; b < B; ++b) {
      next[b] = sample_greedy(&logits[b * V], V);
      out_ids[b * n_new + step] = next[b];
      if (eos >= 0 && next[b] == eos) stop = true;
    }
    offset += curS;
    cur = next;
    curS = 1;
    if (stop) {
      for (int64_t b = 0; b < B; ++b)
        for (int s2 = step + 1; s2 < n_new; ++s2) out_ids[b * n_new + s2] = -1;
      break;
    }
  }
  if (last_logits) std::memcpy(last_logits, logits.data(), sizeof(float) * B * V);
}

// src/rew/infer/generate.nim:192-218 (repetition penalty, temperature, min-p)
// and :220-227 (log-probability of the chosen token).
ORC_API void orc_apply_sampling_config(float* logits, int64_t V, const int32_t* seen, int64_t n_seen,
                                       float temperature, float min_p, float repetition_penalty) {
  if (repetition_penalty != 1.0f)
    for (int64_t i = 0; i < n_seen; ++i) {
      const int32_t t = seen[i];
      if (t >= 0 && t < V) {
        if (logits[t] < 0.f) logits[t] *= repetition_penalty;
        else logits[t] /= repetition_penalty;
      }
    }
  const float temp = std::max(temperature, 1e-6f);
  for (int64_t i = 0; i < V; ++i) logits[i] = logits[i] / temp;
  if (min_p > 0.f) {
    float mx = -INFINITY;
    for (int64_t i = 0; i < V; ++i) mx = std::max(mx, logits[i]);
    const float threshold = mx + std::log(min_p);
    for (int64_t i = 0; i < V; ++i)
      if (logits[i] < threshold) logits[i] = -INFINITY;
  }
}
ORC_API int32_t orc_sample_greedy(const float* logits, int64_t V) { return sample_greedy(logits, V); }
ORC_API float orc_log_prob_of(const float* logits, int64_t V, int32_t token) {
  if (token < 0 || token >= V) return -INFINITY;
  float mx = -INFINITY;
  for (int64_t i = 0; i < V; ++i) mx = std::max(mx, logits[i]);
  float sumExp = 0.f;
  for (int64_t i = 0; i < V; ++i) sumExp += std::exp(logits[i] - mx);
  return logits[token] - mx - std::log(sumExp);
}

// The host loop of generate() driven by a caller-supplied forward, as the
// reference's own test drives it (tests/tgenerate.nim:21-52): records offsets
// and inputs; stops at eos or a stop token.
typedef void (*orc_forward_fn)(const int32_t* ids, int64_t n, int64_t offset, float* logits_out, void* user);
ORC_API int orc_generate_loop(orc_forward_fn fn, void* user, const int32_t* prompt, int64_t n_prompt, int64_t V,
                              int max_new, int eos, int32_t* out_tokens, float* out_logprobs) {
  std::vector<int32_t> gen;
  std::vector<float> logits(V);
  int64_t offset = 0;
  for (int step = 0; step < max_new; ++step) {
    std::vector<int32_t> in = (step == 0) ? std::vector<int32_t>(prompt, prompt + n_prompt)
                                          : std::vector<int32_t>{gen.back()};
    fn(in.data(), (int64_t)in.size(), offset, logits.data(), user);
    std::vector<int32_t> seen(prompt, prompt + n_prompt);
    seen.insert(seen.end(), gen.begin(), gen.end());
    orc_apply_sampling_config(logits.data(), V, seen.data(), (int64_t)seen.size(), 1.0f, 0.f, 1.0f);
    const int32_t next = sample_greedy(logits.data(), V);
    out_logprobs[gen.size()] = orc_log_prob_of(logits.data(), V, next);
    gen.push_back(next);
    out_tokens[gen.size() - 1] = next;
    offset += (int64_t)in.size();
    if (next == eos) break;
  }
  return (int)gen.size();
}

// Timed CPU baseline for the decode metric: fabricates a KV cache of `ctx`
// random entries per layer, then runs `n_steps` single-token steps
// (backbone with S = 1, lm_head on the last position, greedy argmax) for B
// sequences and returns the wall-clock seconds of those steps alone.
ORC_API double orc_decode_bench(const Cfg* c, const float* const* tensors, int64_t B, int64_t ctx, int n_steps,
                                int32_t* last_ids) {
  Model m = build(*c, tensors);
  const int64_t d = c->d_model, V = c->vocab;
  std::vector<KV> kvs(c->n_layers);
  uint64_t st = 0x243F6A8885A308D3ull;
  auto rnd = [&]() {
    st = st * 6364136223846793005ull + 1442695040888963407ull;
    return ((float)((st >> 40) & 0xFFFF) / 65536.0f - 0.5f) * 0.2f;
  };
  for (auto& kv : kvs) {
    kv.k.resize((size_t)B * c->n_kv_heads * ctx * c->head_dim);
    kv.v.resize(kv.k.size());
    for (auto& x : kv.k) x = rnd();
    for (auto& x : kv.v) x = rnd();
    kv.len = ctx;
  }
  std::vector<int32_t> cur(B);
  for (int64_t b = 0; b < B; ++b) cur[b] = (int32_t)((b * 7919) % V);
  std::vector<float> logits(B * V), h(B * d);
  const auto t0 = std::chrono::steady_clock::now();
  int64_t offset = ctx;
  for (int step = 0; step < n_steps; ++step) {
    backbone(m, cur.data(), h.data(), B, 1, offset, 1, &kvs);
    linear(h.data(), m.lw, m.lb, logits.data(), B, d, V);
    for (int64_t b = 0; b < B; ++b) cur[b] = sample_greedy(&logits[b * V], V);
    offset += 1;
  }
  const auto t1 = std::chrono::steady_clock::now();
  if (last_ids) std::memcpy(last_ids, cur.data(), sizeof(int32_t) * B);
  return std::chrono::duration<double>(t1 - t0).count();
}

// ---------------------------------------------------------------- sampling
// Threefry-2x32, four rounds, src/rew/rng.nim:33-56; foldIn :75-80; the unit
// float of src/rew/nn/init.nim:14-17; uniformF32(key, 1, 0, 1)[0] :19-27.
namespace {
struct Key { uint32_t a, b; };
inline uint32_t rotl32(uint32_t x, uint32_t r) { return (x << r) | (x >> (32u - r)); }
Key threefry2x32(Key key, Key ctr) {
  static const uint32_t rot[4] = {13u, 15u, 26u, 6u};
  const uint32_t k0 = key.a, k1 = key.b, k2 = k0 ^ k1 ^ 0x1BD11BDAu;
  uint32_t x0 = ctr.a + k0, x1 = ctr.b + k1;
  for (int r = 0; r < 4; ++r) {
    x0 = x0 + x1;
    x1 = rotl32(x1, rot[r]);
    x1 = x1 ^ x0;
  }
  x0 = x0 + k1;
  x1 = x1 + k2 + 1u;
  return Key{x0, x1};
}
Key init_key(uint64_t seed) { return Key{(uint32_t)(seed & 0xFFFFFFFFull), (uint32_t)(seed >> 32)}; }
Key fold_in(Key k, uint64_t data) { return threefry2x32(k, Key{(uint32_t)(data & 0xFFFFFFFFull), (uint32_t)(data >> 32)}); }
float unit_float(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }
float uniform01(Key key) { return 0.0f + (1.0f - 0.0f) * unit_float(fold_in(key, 0).a); }

// (value, index) sorted by value descending; equal values keep ascending index (Nim's sort is stable).
std::vector<std::pair<float, int>> sorted_desc(const float* logits, int64_t V) {
  std::vector<std::pair<float, int>> s(V);
  for (int64_t i = 0; i < V; ++i) s[i] = {logits[i], (int)i};
  std::stable_sort(s.begin(), s.end(), [](const std::pair<float, int>& x, const std::pair<float, int>& y) { return x.first > y.first; });
  return s;
}

// src/rew/infer/generate.nim:92-116
int sample_top_k(const float* logits, int64_t V, int topK, Key key) {
  auto s = sorted_desc(logits, V);
  const int k = (int)std::min<int64_t>(topK, V);
  std::vector<float> probs(k);
  float sumExp = 0.f;
  for (int i = 0; i < k; ++i) {
    probs[i] = std::exp(s[i].first);
    sumExp += probs[i];
  }
  for (int i = 0; i < k; ++i) probs[i] /= sumExp;
  const float u = uniform01(key);
  float cum = 0.f;
  for (int i = 0; i < k; ++i) {
    cum += probs[i];
    if (u <= cum) return s[i].second;
  }
  return s[k - 1].second;
}

// src/rew/infer/generate.nim:118-150
int sample_top_p(const float* logits, int64_t V, float topP, Key key) {
  auto s = sorted_desc(logits, V);
  const float maxLogit = s[0].first;
  std::vector<float> probs(V);
  float sumExp = 0.f;
  for (int64_t i = 0; i < V; ++i) {
    probs[i] = std::exp(s[i].first - maxLogit);
    sumExp += probs[i];
  }
  for (int64_t i = 0; i < V; ++i) probs[i] /= sumExp;
  float cum = 0.f;
  int64_t cutoff = V;
  for (int64_t i = 0; i < V; ++i) {
    cum += probs[i];
    if (cum >= topP) {
      cutoff = i + 1;
      break;
    }
  }
  float renorm = 0.f;
  for (int64_t i = 0; i < cutoff; ++i) renorm += probs[i];
  for (int64_t i = 0; i < cutoff; ++i) probs[i] /= renorm;
  const float u = uniform01(key);
  cum = 0.f;
  for (int64_t i = 0; i < cutoff; ++i) {
    cum += probs[i];
    if (u <= cum) return s[i].second;
  }
  return s[cutoff - 1].second;
}
}  // namespace

ORC_API void orc_threefry(uint32_t ka, uint32_t kb, uint32_t ca, uint32_t cb, uint32_t* out2) {
  const Key r = threefry2x32(Key{ka, kb}, Key{ca, cb});
  out2[0] = r.a;
  out2[1] = r.b;
}
ORC_API float orc_uniform01(uint64_t seed, int n_folds, const uint64_t* folds) {
  Key k = init_key(seed);
  for (int i = 0; i < n_folds; ++i) k = fold_in(k, folds[i]);
  return uniform01(k);
}
ORC_API int32_t orc_sample_top_k(const float* logits, int64_t V, int topK, uint64_t seed) {
  return sample_top_k(logits, V, topK, init_key(seed));
}
ORC_API int32_t orc_sample_top_p(const float* logits, int64_t V, float topP, uint64_t seed) {
  return sample_top_p(logits, V, topP, init_key(seed));
}

// generate() with a GenerationConfig (src/rew/infer/generate.nim:231-265), one key per sequence
// (the reference loop is batch-1; sequence b starts from initKey(seeds[b])).  Cached forward as in
// orc_generate_greedy.  out_ids [B,n_new], out_logprobs [B,n_new].
ORC_API void orc_generate_sampled(const Cfg* c, const float* const* tensors, const int32_t* prompt, int64_t B, int64_t S,
                                  int n_new, float temperature, int top_k, float top_p, float min_p,
                                  float repetition_penalty, int do_sample, const uint64_t* seeds, int32_t* out_ids,
                                  float* out_logprobs) {
  Model m = build(*c, tensors);
  const int64_t d = c->d_model, V = c->vocab;
  std::vector<KV> kvs(c->n_layers);
  std::vector<int32_t> cur(prompt, prompt + B * S);
  std::vector<std::vector<int32_t>> seen(B);
  std::vector<Key> keys(B);
  for (int64_t b = 0; b < B; ++b) {
    seen[b].assign(prompt + b * S, prompt + (b + 1) * S);
    keys[b] = init_key(seeds[b]);
  }
  int64_t curS = S, offset = 0;
  std::vector<float> logits(B * V);
  for (int step = 0; step < n_new; ++step) {
    std::vector<float> h(B * curS * d), last(B * d);
    backbone(m, cur.data(), h.data(), B, curS, offset, 1, &kvs);
    for (int64_t b = 0; b < B; ++b) std::memcpy(&last[b * d], &h[(b * curS + curS - 1) * d], sizeof(float) * d);
    linear(last.data(), m.lw, m.lb, logits.data(), B, d, V);
    std::vector<int32_t> next(B);
    for (int64_t b = 0; b < B; ++b) {
      float* lg = &logits[b * V];
      orc_apply_sampling_config(lg, V, seen[b].data(), (int64_t)seen[b].size(), temperature, min_p, repetition_penalty);
      int32_t tok;
      if (!do_sample || temperature <= 0.01f) tok = sample_greedy(lg, V);
      else if (top_k > 0) tok = sample_top_k(lg, V, top_k, keys[b]);
      else tok = sample_top_p(lg, V, top_p, keys[b]);
      next[b] = tok;
      out_ids[b * n_new + step] = tok;
      if (out_logprobs) out_logprobs[b * n_new + step] = orc_log_prob_of(lg, V, tok);
      seen[b].push_back(tok);
      keys[b] = fold_in(keys[b], (uint64_t)step);
    }
    offset += curS;
    cur = next;
    curS = 1;
  }
}

// ---------------------------------------------------------------------------------------------
// NF4 weight codec and the QLoRA Linear (src/rew/quantize/codecs.nim:13-74, src/rew/nn/lora.nim:217-256,
// 331-431).  Weights are the flat row-major [in, out] array; a block is `blockSize` consecutive flat
// elements; two codes per byte, the even element in the low nibble.
namespace {
const float kNf4Table[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                             -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                             0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                             0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
// codecs.nim:23-29: nearest table entry, the first one on a tie
int find_nf4_index(float value) {
  float minDist = 1e10f;
  int result = 0;
  for (int i = 0; i < 16; ++i) {
    const float dist = std::fabs(value - kNf4Table[i]);
    if (dist < minDist) {
      minDist = dist;
      result = i;
    }
  }
  return result;
}
}  // namespace

// codecs.nim:31-57.  packed: (n+1)/2 bytes, scales: ceil(n/blockSize) floats.
ORC_API void orc_nf4_quantize(const float* weights, int64_t n, int blockSize, uint8_t* packed, float* scales) {
  const int64_t numBlocks = (n + blockSize - 1) / blockSize;
  std::memset(packed, 0, (size_t)((n + 1) / 2));
  for (int64_t blk = 0; blk < numBlocks; ++blk) {
    const int64_t start = blk * blockSize, endPos = std::min<int64_t>(start + blockSize, n);
    float absMax = 1e-10f;
    for (int64_t i = start; i < endPos; ++i) absMax = std::max(absMax, std::fabs(weights[i]));
    scales[blk] = absMax;
    for (int64_t i = start; i < endPos; ++i) {
      float normalized = weights[i] / absMax;
      normalized = std::min(1.0f, std::max(-1.0f, normalized));
      const int code = find_nf4_index(normalized) & 0x0F;
      if ((i % 2) == 0) packed[i / 2] = (uint8_t)code;
      else packed[i / 2] = (uint8_t)(packed[i / 2] | (code << 4));
    }
  }
}

// codecs.nim:59-70 (lora.nim:217-256 computes the same values group by group)
ORC_API void orc_nf4_dequantize(const uint8_t* packed, const float* scales, int64_t n, int blockSize, float* out) {
  for (int64_t i = 0; i < n; ++i) {
    const int code = (i % 2) == 0 ? (packed[i / 2] & 0x0F) : ((packed[i / 2] >> 4) & 0x0F);
    out[i] = kNf4Table[code] * scales[i / blockSize];
  }
}

// QloraLinear.forward (lora.nim:410-431): x [M,in] @ dequantizedWeight [in,out] + bias + scaling * (x @ A^T) @ B^T,
// A [rank,in], B [out,rank]; bias may be NULL (hasBias = false).
ORC_API void orc_qlora_forward(const float* x, int64_t M, const uint8_t* packed, const float* scales, int64_t in, int64_t out,
                               int groupSize, const float* bias, const float* A, const float* B, int rank, float scaling,
                               float* y) {
  std::vector<float> W((size_t)in * out);
  orc_nf4_dequantize(packed, scales, in * out, groupSize, W.data());
  std::vector<float> base((size_t)M * out);
  matmul(x, W.data(), base.data(), M, in, out);
  if (bias)
    for (int64_t m = 0; m < M; ++m)
      for (int64_t o = 0; o < out; ++o) base[m * out + o] = base[m * out + o] + bias[o];
  std::vector<float> aT((size_t)in * rank), bT((size_t)rank * out), xA((size_t)M * rank), delta((size_t)M * out);
  for (int64_t r = 0; r < rank; ++r)
    for (int64_t i = 0; i < in; ++i) aT[i * rank + r] = A[r * in + i];
  for (int64_t o = 0; o < out; ++o)
    for (int64_t r = 0; r < rank; ++r) bT[r * out + o] = B[o * rank + r];
  matmul(x, aT.data(), xA.data(), M, in, rank);
  matmul(xA.data(), bT.data(), delta.data(), M, rank, out);
  for (int64_t i = 0; i < M * out; ++i) {
    const float dlt = scaling != 1.0f ? delta[i] * scaling : delta[i];
    y[i] = base[i] + dlt;
  }
}
