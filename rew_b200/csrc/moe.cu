// Mixture-of-experts routing for DeepSeekMoE.forward
// (src/rew/models/deepseek.nim:122-145).
//
// moe_route_kernel: one warp per token does what the reference spends a
// softmax chain and two full stable sorts on (deepseek.nim:132-138,
// src/rew/ops/sort.nim:36-90): softmax over the E router logits, the k largest
// probabilities in descending order (exact ties resolved towards the lower
// expert index), renormalised by their sum.
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"

namespace rewb {
namespace {

constexpr int MAX_E_PER_LANE = 8;  // E <= 256

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int64_t N, int E, int k,
                                                        float* __restrict__ topw, int* __restrict__ topi) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= N) return;
  const float* lr = logits + tok * E;
  float p[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = (e < E) ? lr[e] : -INFINITY;
    mx = fmaxf(mx, p[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = (e < E) ? expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = (e < E) ? p[i] / sum : -1.f;  // probabilities are >= 0; -1 marks "absent / taken"
  }
  float denom = 0.f;
  float myw = 0.f;
  int myi = 0;
  for (int j = 0; j < k; ++j) {
    float bv = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (p[i] > bv || (p[i] == bv && e < be)) {
        bv = p[i];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    denom += bv;
    if (lane == j % 32) {
      myw = bv;
      myi = be;
    }
    if ((be & 31) == lane) p[be >> 5] = -1.f;
    if (j % 32 == 31 || j == k - 1) {
      // flush up to 32 selections held one per lane
      const int base = (j / 32) * 32;
      if (base + lane <= j) {
        topw[tok * k + base + lane] = myw;
        topi[tok * k + base + lane] = myi;
      }
    }
  }
  __syncwarp();
  for (int j = lane; j < k; j += 32) topw[tok * k + j] = topw[tok * k + j] / denom;
}

}  // namespace

int moe_route_launch(Ctx* c, const float* logits, int64_t N, int E, int k, float* topw, int* topi) {
  RB_REQUIRE(E >= 1 && E <= 32 * MAX_E_PER_LANE, "MoE routing supports up to 256 experts");
  RB_REQUIRE(k >= 1 && k <= E, "initDeepSeekMoE: numExpertsPerTok must be in 1..numRouted");
  if (N == 0) return REWB200_OK;
  RB_CUDA(launch_k(moe_route_kernel, dim3((unsigned)((N + 3) / 4)), dim3(128), 0, c->stream, c->use_pdl, logits, N, E, k,
                   topw, topi));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace rewb

using namespace rewb;

extern "C" int rewb200_moe_route(const rewb200_buffer* x, const rewb200_buffer* router_w, const rewb200_buffer* router_b,
                                 int top_k, rewb200_buffer** weights, rewb200_buffer** indices) {
  RB_REQUIRE(x && router_w && weights && indices, "DeepSeekMoE.forward: NULL argument");
  RB_REQUIRE(x->ndims == 2 && router_w->ndims == 2 && x->dims[1] == router_w->dims[0],
             "DeepSeekMoE.forward: hidden [tokens, d] and gate weight [d, experts] do not agree");
  Ctx* c = ctx_get(x->slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  const int64_t N = x->dims[0], E = router_w->dims[1];
  RB_REQUIRE(top_k >= 1 && top_k <= E, "initDeepSeekMoE: numExpertsPerTok must be in 1..numRouted");
  rewb200_buffer* logits = nullptr;
  RB_TRY(rewb200_linear(x, router_w, router_b, &logits));
  float* lf = (float*)logits->ptr;
  float* tmp = nullptr;
  int st = REWB200_OK;
  if (logits->dtype == REWB200_BF16) {
    if (cudaMallocAsync((void**)&tmp, (size_t)N * E * 4 + 256, c->stream) != cudaSuccess) st = fail("allocation failed");
    if (st == REWB200_OK) st = cast_launch(c, logits->ptr, REWB200_BF16, tmp, REWB200_F32, N * E);
    lf = tmp;
  }
  const int64_t od[2] = {N, top_k};
  if (st == REWB200_OK) st = buffer_new(c, REWB200_F32, od, 2, weights);
  if (st == REWB200_OK) st = buffer_new(c, REWB200_I32, od, 2, indices);
  if (st == REWB200_OK) st = moe_route_launch(c, lf, N, (int)E, top_k, (float*)(*weights)->ptr, (int*)(*indices)->ptr);
  if (tmp) cudaFreeAsync(tmp, c->stream);
  rewb200_buffer_release(logits);
  return st;
}
