// Shared host-side declarations of the rew_b200 CUDA library: runtime context,
// device buffers, error convention, and the launchers each .cu file exports to
// the others.  Nothing here is part of the public C ABI (see include/rew_b200.h).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/rew_b200.h"

namespace rewb {

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------- errors
void set_error(const std::string& msg);
int fail(const std::string& msg);  // records msg, returns REWB200_ERR

#define RB_CUDA(expr)                                                                          \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return ::rewb::fail(std::string(#expr) + ": " + cudaGetErrorString(_e) + " at " __FILE__ \
                          ":" + std::to_string(__LINE__));                                     \
  } while (0)
#define RB_TRY(expr)            \
  do {                          \
    int _s = (expr);            \
    if (_s != REWB200_OK) return _s; \
  } while (0)
#define RB_REQUIRE(cond, msg)                       \
  do {                                              \
    if (!(cond)) return ::rewb::fail(msg);          \
  } while (0)

// ---------------------------------------------------------------- context
struct Ctx {
  int device = -1;
  cudaStream_t stream = nullptr;
  cudaStream_t side = nullptr;            // second stream for a branch that runs beside the main one (MoE shared experts)
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  bool moe_overlap = true;
  int ep_prefix = 2;          // expert-parallel exchange: 2 (auto) over the peer heap when one is attached and the step fits,
                              // else NCCL as under 1 from 4 ranks on; 1 NCCL, pair counts first, then only the occupied slot
                              // prefixes (outside a captured graph); 0 NCCL, always the worst-case capacity
  int* d_status = nullptr;   // kernels record KernelStatus codes here
  static constexpr int kTickets = 16384;
  int* d_tickets = nullptr;  // split-KV decode attention: one arrival counter per (sequence, kv head), zero between launches
  bool attn_fused_merge = false;  // measured slower than the separate merge launch (3.20 vs 3.06 ms per step at batch 1)
  int* h_status = nullptr;   // pinned, 64 ints: [0] mirror of d_status; [16..31] / [32..47] per-peer pair counts sent /
                             // received by the expert-parallel prefix exchange
  int sm_count = 0;
  bool use_pdl = true;
  int linear_impl = 2;       // bf16 Linear: 0 mma.sync, 1 tcgen05 when rows > 32, 2 tcgen05 always (default)
  bool prefill_persistent = true;  // 256-token Linear tiles on the persistent kernel with overlapped epilogue
  bool prefill_pair = true;        // ... on pairs of CTAs (tcgen05 cta_group::2, 256 x 256 tiles) when the width is a multiple of 256
  int splitk_min_blocks = 8;  // a K slice keeps at least this many 64-wide blocks (a CTA's pipeline needs a few to ramp)
  int splitk_max_rows = 256;  // largest step (rows) whose Linear launches may split K
  int profile_mask = 31;      // rewb200_session_profile_linears: bit 0 q|k|v, 1 o, 2 gate|up, 3 down, 4 lm_head
  int splitk_cluster = 0;     // decode-size split-K summed inside thread-block clusters instead of through f32 slabs: bit 0 the q|k|v launch, bit 1 the others (off: measured slower)
  bool norm_cluster = true;   // decode-size residual+norm on clusters of four CTAs per row
  bool attn_pingpong = true;  // ... with two query tiles per CTA sharing the K / V tiles, from this many query rows up
  int attn_pingpong_min_rows = 3072;
  bool attn_tc = true;        // prefill attention (head_dim 128, conventional causal) on the tcgen05 kernel
  bool sampling_exact = false; // samplers skip the bucket path and always run the full-vocabulary radix select
  int tp_exchange = 0;          // fused exchange of decode-size steps: 0 / 1 one hop (every rank stores to every peer), 2 two hops
  bool gu_split = true;         // decode-size gate|up launches with too few feature tiles split K (slabs + a sum-and-SwiGLU launch)
  bool attn_fuse_qkv_always = false;  // option qkv_post=attention_always: also with grids of several waves (tests)
  bool attn_fuse_qkv = true;    // decode steps: bias + RoPE + cache append of the new token inside the attention kernel
  bool nf4_small = false;       // NF4 GEMV of up to four rows on the CUDA-core streamer instead of the tensor-core kernel (measured slower: off)
  bool tp_twoshot = true;       // tensor-parallel steps above 64 rows: sum over the peer heap (two-shot) instead of NCCL
  bool record_routing = false;  // sessions keep every MoE layer's top-k expert ids of their last forward (a test aid)
  int inject_alloc_fail = 0;  // test hook: the n-th activation allocation from now fails on the host
  int option_epoch = 0;      // bumped by rewb200_set_option; captured graphs from older epochs are rebuilt
  void* pinned = nullptr;    // pinned host staging for H2D/D2H of buffers
  size_t pinned_bytes = 0;
};
Ctx* ctx_get(int slot);       // nullptr + error when not initialised
Ctx* ctx_current();           // slot 0
int ctx_check_status(Ctx* c); // reads d_status after a sync; non-zero -> error

size_t dtype_size(int dtype);

// Encodes a 2D row-major bf16 tensor map: `inner` contiguous elements per row,
// `outer` rows, `row_stride_bytes` between rows (multiple of 16), box =
// box_inner x box_outer elements, 128-byte swizzle (box_inner must be 64).
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);
// 3D variant (dim 2 = groups, e.g. experts) with box depth 1.
int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t groups,
                      uint64_t row_stride_bytes, uint64_t group_stride_bytes, uint32_t box_inner,
                      uint32_t box_outer);

// NF4 weight-only Linear (nf4.cu).  Column map: logical column n of the quantised matrix lives at
// device column (w / gran) * gstride + w % gran + (n / seg_len) * seg_off with w = n % seg_len
// (identity: seg_len = gran = gstride = N, seg_off = 0; the bf16 engine's gate|up interleave:
// seg_len = F, gran = 8, gstride = 16, seg_off = 8).
struct ColMap {
  int64_t seg_len, gran, gstride, seg_off;
};
struct Nf4W {
  uint8_t* q = nullptr;     // [ceil(N/128)][K/64][128][32] codes: feature-major, two input rows per byte
  float* sc = nullptr;      // [N/64][K] scales
  uint32_t* sc2 = nullptr;  // [N/64][K/2] the scales as bf16 pairs of consecutive input rows
  int64_t K = 0, N = 0;
};
int nf4_alloc(Ctx* c, int64_t K, int64_t N, Nf4W* w);
void nf4_free(Nf4W* w);
int nf4_quantize_launch(Ctx* c, const void* src, int src_dtype, int64_t ld, ColMap cm, const Nf4W& w);
int nf4_dequant_launch(Ctx* c, const Nf4W& w, bf16* dst, int64_t ld, ColMap cm);
int nf4_codes_launch(Ctx* c, const Nf4W& w, uint8_t* codes);
int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N);
int nf4_pick_ksplit(Ctx* c, int64_t K, int64_t N, int64_t M);  // rows of the step: up to four run on the CUDA-core GEMV
// out: [ksplit][M][N] f32 partial sums of x[M,K] @ W (no bias); 1 <= M <= 32
int nf4_gemv_launch(Ctx* c, const Nf4W& w, const bf16* x, int64_t ldx, int64_t M, int ksplit, float* out);

// Launch helper that optionally attaches the programmatic-stream-serialization
// attribute (the kernel then starts early and calls griddepcontrol.wait itself).
extern int64_t g_launch_total;  // kernels launched by this library since load

template <typename... KArgs, typename... Args>
cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Same, with the thread-block cluster shape given at launch.
template <typename... KArgs, typename... Args>
cudaError_t launch_k_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                             dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---------------------------------------------------------------- buffers
}  // namespace rewb

// Opaque to C callers.  One contiguous row-major device allocation.
struct rewb200_buffer {
  int slot = 0;
  int dtype = 0;
  int ndims = 0;
  int64_t dims[8] = {0};
  void* ptr = nullptr;
  size_t bytes = 0;
  bool owned = true;
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < ndims; ++i) n *= dims[i];
    return n;
  }
};

namespace rewb {

int buffer_new(Ctx* c, int dtype, const int64_t* dims, int ndims, rewb200_buffer** out);

// ---------------------------------------------------------------- launchers
enum Epilogue : int {
  EPI_PARTIAL_F32 = 0,  // out_f32[split][row][col] = acc
  EPI_BIAS_F32 = 1,     // out_f32[row][col] = acc + bias[col]
  EPI_BIAS_BF16 = 2,    // out_bf16[row][col] = acc + bias[col]
  EPI_SWIGLU_BF16 = 3,  // columns interleaved gate/up in groups of 8: out[row][col/2..] = silu(g+bg)*(u+bu)
};

struct LinearBf16Plan {
  CUtensorMap tmW;       // W [K rows][N cols] bf16 (reference layout [in,out]); 3D when groups > 1
  int64_t K = 0, N = 0;
  int groups = 0;        // 0: one matrix; >= 1: that many stacked matrices (experts), 3-D tensor map
};
// y = x @ W (+bias); x [M,K] bf16 row-major (ldx elements), W as planned.
// ksplit > 1 requires EPI_PARTIAL_F32 (out holds ksplit slabs of M*N floats).
// For grouped launches (plan.groups >= 1) group g uses rows
// [row_offsets[g], row_offsets[g+1]) of x/out (device array, groups+1 ints).
int linear_bf16_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int epi,
                       int ksplit, void* out, int64_t ldo, const float* bias, const int* row_offsets, int max_rows_per_group);
int linear_tc_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int epi, int ksplit,
                     void* out, int64_t ldo, const float* bias);
int linear_tc_grouped_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int epi, void* out,
                             int64_t ldo, const float* bias, const int* row_offsets);
// Decode-size split-K on thread-block clusters (M <= 32, ksplit in {2,4,8}): the CTAs that share a
// feature tile sum their accumulators through distributed shared memory and leave ONE f32 slab
// out[M][ldo] (bias still for the consumer), or, with fuse_qkv, finished q / k / v exactly as
// qkv_post_kernel would have left them (bf16 activations).
struct QkvPostArgs;
bool linear_tc_cluster_ok(Ctx* c, const LinearBf16Plan& plan, int64_t M, int ksplit);
int linear_tc_cluster_launch(Ctx* c, const LinearBf16Plan& plan, const bf16* x, int64_t ldx, int64_t M, int ksplit,
                             float* out, int64_t ldo, const QkvPostArgs* fuse_qkv);
int linear_bf16_plan(LinearBf16Plan* plan, const bf16* W, int64_t K, int64_t N, int groups);
int linear_bf16_pick_ksplit(Ctx* c, int64_t M, int64_t K, int64_t N);

// f32 path: C[M,N] = A[M,K] @ B[K,N] (+ bias[N]).
int gemm_f32_launch(Ctx* c, const float* A, const float* B, const float* bias, float* C, int64_t M, int64_t K,
                    int64_t N);

struct NormArgs {
  float* x_res;           // [rows,d] residual stream (in/out)
  const float* partial;   // [nsplit][rows][d] or nullptr
  int nsplit;
  int64_t split_stride;   // elements between partial slabs
  const float* bias;      // [d] or nullptr (added once)
  const void* embed;      // embedding table [V,d] (model dtype) or nullptr
  const int* ids;         // [rows] token ids when embed != nullptr
  int embed_dtype;
  const float* gamma;
  const float* beta;
  float eps;
  int norm_kind;          // 0 rms, 1 layernorm, -1 none (only update x_res)
  int64_t d;
  void* out;              // normalised output, out_dtype
  int out_dtype;
  int vocab;
  int* status;
  int partial_bf16;       // the partial slabs hold bf16 instead of f32 (a tensor-parallel sum that travelled as bf16)
  // The partial is the gather buffer of the two-shot tensor-parallel all-reduce (Tp2Args), written by the peers:
  // wait (bounded) until cell r of wait_cells has reached *wait_epoch + wait_offset for every rank r < wait_n.
  const int* wait_cells;
  int wait_n;
  const int* wait_epoch;
  int wait_offset;
  // One-shot tensor-parallel all-reduce fused into this kernel (n_peers > 0), push style: a thread sums its
  // columns of the local split-K slabs and stores that partial into slot `my_rank` of EVERY peer's exchange
  // buffer with plain peer stores, as 16-byte lines {payload, flag, payload, flag} (flag = `*epoch +
  // barrier_offset`, a value no earlier all-reduce has used), then polls (bounded) the same lines of the other
  // ranks' slots in its OWN memory until they carry that flag, and adds the partials in rank order, so every
  // rank computes the same bits.  Payload and flag arrive together: no fence and no flag round trip.
  int n_peers;
  int my_rank;
  int payload_bf16;       // partials cross NVLink as bf16 (bf16 models) or f32
  int two_shot;           // 1: columns are owned by ranks in blocks of d / n_peers: a partial goes to the owner only, the
                          // owner adds the n_peers values in rank order and stores the sum to every peer (one more hop,
                          // 2 (n - 1) / n of a partial over the links instead of n - 1 partials)
  void* peer_buf[8];      // rank r's exchange buffer of this all-reduce: [world][slot_lines] 16-byte lines
  int64_t slot_lines;     // lines between two writers' slots
  const int* epoch;       // device counter, advanced once per forward on every rank alike
  int barrier_offset;
};
int residual_norm_launch(Ctx* c, const NormArgs& a, int64_t rows);

struct KvLayout {
  void* k;                // [n_pages][kvh][page][hd]
  void* v;
  const int* block_table; // [B][max_pages] page ids, or nullptr for contiguous [B][kvh][L][hd]
  int max_pages;
  int page;               // tokens per page (64)
  int kvh, hd;
  int64_t contiguous_len; // L when block_table == nullptr
  int dtype;
};

struct QkvPostArgs {
  const float* partial;   // [nsplit][rows][nq+2nkv] f32 (bias not yet added)
  int nsplit;
  int64_t split_stride;
  const float* bias;      // [nq+2nkv]
  const float* cosT;      // [max_seq][hd]
  const float* sinT;
  const int* pos0;        // [B] position of each sequence's first new token
  int S;                  // new tokens per sequence (rows = B*S)
  int rope_shift;         // RoPE table row = cache position + rope_shift (the reference's `offset`)
  int kv_capacity;        // tokens the cache can hold per sequence
  int nh, kvh, hd;
  int max_seq;            // rows of the RoPE tables
  void* q_out;            // [rows][nh][hd], act dtype
  int act_dtype;
  KvLayout kv;
  int* status;
  int early_lookup;       // positions, block tables and RoPE tables predate every kernel that may still be in flight
                          // (a captured decode step): they may be read before the stream dependency resolves
};
int qkv_post_launch(Ctx* c, const QkvPostArgs& a, int64_t B);

struct AttnArgs {
  const void* q;          // element strides below: batch, position, head (head_dim contiguous)
  int64_t q_sb, q_ss, q_sh;
  void* out;
  int64_t o_sb, o_ss, o_sh;
  KvLayout kv;
  const int* pos0;        // [B] device: context length before these S queries, or nullptr
  int64_t B;
  int S;
  int nh;
  int causal;             // 0: every key visible
  int mask_kind;          // 0 as written (key j visible to query i iff i <= j), 1 conventional causal
  int64_t kv_len_fixed;   // >= 0: keys per sequence (used when pos0 == nullptr)
  int64_t max_kv_len;     // upper bound of keys per sequence (sizes the f32 kernel's shared memory)
  float scale;            // 0: 1/sqrt(head_dim)
  int dtype;
  int kv_tail_only;       // decode (S == 1): no kernel that may still be in flight writes K, V, pos0 or the block table,
                          // except for the newest cache row (a captured decode step: everything older predates the
                          // graph launch), so older K/V tiles may be requested before the stream dependency
                          // resolves.  A dependent launch starts once its predecessor has STARTED, so distance in
                          // the stream proves nothing: leave 0 outside a captured step.
  float* scratch;         // split-KV partials (bf16 decode)
  size_t scratch_bytes;
  const CUtensorMap* tmK; // bf16: TMA maps over the K / V rows ([rows][head_dim], box 64x64)
  const CUtensorMap* tmV;
  const QkvPostArgs* fuse_qkv;  // bf16 decode (S == 1), optional: the attention kernel finishes q / k / v of the new
                                // token from the q|k|v projection's split-K slabs itself (what qkv_post_launch would
                                // have done in a launch of its own) and appends K / V to the cache; `q` is not read
};
int attn_launch(Ctx* c, const AttnArgs& a);
int decode_splits(Ctx* c, int64_t B, int kvh);  // KV splits a decode attention launch of B sequences x kvh kv heads uses
size_t attn_scratch_bytes(int64_t B, int nh, int hd, int max_splits);

// scratch (optional): rows*64*8 bytes lets wide rows be scanned by several CTAs each
struct PeerInfo {
  int world = 0, rank = 0;
  size_t buf_bytes = 0;        // capacity of ONE writer's slot; an exchange buffer holds `world` of them
  char* bufs[2][8] = {};       // [which][rank]: the two alternating exchange buffers of every rank (own rank: local)
  int* epoch = nullptr;        // local device counter
  char* a2a[8] = {};           // [rank]: the expert-parallel all-to-all region of every rank (nullptr without one)
  size_t a2a_bytes = 0;
  int* a2a_flags[8] = {};      // [rank]: 4 x 8 ints, cell (phase, writer rank)
};
// Expert-parallel all-to-all over the peer heap (src/rew/ops/distributed.nim:106-128): the dispatch kernel
// stores every (token, expert) pair's row straight into the owning rank's region, the return kernel
// stores the expert outputs straight into the asking rank's region; pair counts and flags travel the
// same way, so no count exchange passes through the host and no padding crosses NVLink.
struct A2aArgs {
  int world, my_rank;
  int* cells[8];      // rank r's cells: pair counts [8] | dispatch flags [8] | return flags [8], indexed by writer rank
  char* region[8];    // rank r's all-to-all region; below, byte offsets inside it (the same on every rank)
  int64_t off_x;      // recv_x [world][cap][d] activations
  int64_t off_meta;   // recv_meta [world][cap] local expert ids
  int64_t off_back;   // back [world][cap][d] f32 expert outputs
  int* arrive;        // two local arrival counters (dispatch, return), zero between launches
  const int* epoch;   // local device counter; flag value of this layer = *epoch + offset
  int offset;
  int* status;
};
// Two-shot tensor-parallel all-reduce of a [rows, d] partial over the peer heap, for steps too large for the
// fused one-shot exchange (prefill): (1) every rank stores slice p (columns [p*d/world, (p+1)*d/world)) of its
// partial into rank p's scatter buffer, (2) rank p adds the world slices in rank order and stores the sum into
// EVERY rank's gather buffer, (3) the residual+norm kernel reads the local gather buffer.  Each rank moves
// 2*(world-1)/world of the partial over NVLink instead of (world-1) times all of it, and every rank reads the
// same sums.  Regions and cells are those of the expert-parallel all-to-all (a model is never both).
struct Tp2Args {
  int world, my_rank;
  int* cells[8];       // rank r's cells: [8 unused] | scatter flags [8] | gather flags [8], indexed by writer rank
  char* region[8];     // rank r's bulk region: scatter buffer [world][rows][d/world], then the gather buffer [rows][d]
  int64_t off_gather;  // byte offset of the gather buffer
  int* arrive;         // two local arrival counters, zero between launches
  const int* epoch;    // local device counter; flag value = *epoch + offset
  int offset;
  int* status;
  const void* partial; // this rank's [rows][d] partial, payload dtype
  int64_t rows, d;
  int payload_bf16;
};
int tp2_allreduce_launch(Ctx* c, const Tp2Args& a);
// nullptr when no peer heap has been attached for the slot
const PeerInfo* comm_peer_info(int slot);

int argmax_launch(Ctx* c, const float* logits, int64_t rows, int64_t V, int* out_ids, void* scratch, size_t scratch_bytes);
int swiglu_f32_launch(Ctx* c, const float* g, const float* u, float* out, int64_t n);
int cast_launch(Ctx* c, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n);
int fill_normal_launch(Ctx* c, void* dst, int dtype, int64_t n, uint64_t seed, float std);
int fill_const_launch(Ctx* c, void* dst, int dtype, int64_t n, float v);
int rope_tables_host(int hd, int max_seq, double theta, std::vector<float>* cosT, std::vector<float>* sinT);

}  // namespace rewb
