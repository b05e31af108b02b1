// Runtime of the rew_b200 library: per-slot device context (stream, status
// word, pinned staging), the stream-ordered CUDA allocator behind device
// buffers, host<->device transfers, the error convention and TMA descriptor
// encoding.  Stands where rew keeps its PJRT client cache and transfer helpers
// (src/rew/eager.nim:78-140,229-247) and BufferHandle releaser
// (src/rew/buffer.nim:33,69-82).
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace rewb {

static thread_local std::string g_last_error;
static std::vector<Ctx*> g_ctx;
static std::mutex g_mu;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(const std::string& msg) {
  g_last_error = msg;
  return REWB200_ERR;
}

Ctx* ctx_get(int slot) {
  if (slot < 0 || slot >= (int)g_ctx.size() || !g_ctx[slot]) {
    set_error("rew_b200: slot " + std::to_string(slot) + " is not initialised; call rewb200_init first");
    return nullptr;
  }
  return g_ctx[slot];
}
Ctx* ctx_current() { return ctx_get(0); }

size_t dtype_size(int dtype) {
  switch (dtype) {
    case REWB200_BOOL: case REWB200_I8: case REWB200_U8: return 1;
    case REWB200_I16: case REWB200_F16: case REWB200_BF16: return 2;
    case REWB200_I32: case REWB200_F32: return 4;
    case REWB200_I64: case REWB200_F64: return 8;
    default: return 0;
  }
}

int ctx_check_status(Ctx* c) {
  int st = 0;
  RB_CUDA(cudaMemcpyAsync(c->h_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  RB_CUDA(cudaStreamSynchronize(c->stream));
  st = *c->h_status;
  if (st != 0) {
    RB_CUDA(cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream));
    RB_CUDA(cudaMemsetAsync(c->d_tickets, 0, Ctx::kTickets * sizeof(int), c->stream));  // a kernel that gave up may have left counts behind
    const char* what = st == KS_MBAR_TIMEOUT ? "a bounded mbarrier wait expired"
                       : st == KS_BAD_INDEX  ? "an index was out of range (token id / page / position)"
                       : st == KS_TMEM_TIMEOUT ? "a bounded tensor-memory wait expired"
                       : st == KS_PEER_TIMEOUT ? "a bounded wait on a peer GPU expired"
                                               : "unknown device status";
    return fail(std::string("rew_b200 device status ") + std::to_string(st) + ": " + what);
  }
  return REWB200_OK;
}

// ---- TMA descriptors.  cuTensorMapEncodeTiled comes from the driver through
// the runtime's entry-point query, so the library has no link-time dependency
// on libcuda and still loads on a machine without a GPU.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int load_encode() {
  if (g_encode) return REWB200_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  RB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  RB_REQUIRE(fn != nullptr && qres == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled not available");
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return REWB200_OK;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  RB_TRY(load_encode());
  RB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base must be 16-byte aligned");
  RB_REQUIRE(row_stride_bytes % 16 == 0, "tensor map row stride must be a multiple of 16 bytes (dims % 8 for bf16)");
  RB_REQUIRE(box_inner * 2 == 128, "128-byte swizzle needs a 64-element bf16 inner box");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RB_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(2d) failed with code " + std::to_string((int)r));
  return REWB200_OK;
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t groups,
                      uint64_t row_stride_bytes, uint64_t group_stride_bytes, uint32_t box_inner,
                      uint32_t box_outer) {
  RB_TRY(load_encode());
  RB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base must be 16-byte aligned");
  RB_REQUIRE(row_stride_bytes % 16 == 0 && group_stride_bytes % 16 == 0, "tensor map strides must be multiples of 16 bytes");
  cuuint64_t dims[3] = {inner, outer, groups};
  cuuint64_t strides[2] = {row_stride_bytes, group_stride_bytes};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RB_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(3d) failed with code " + std::to_string((int)r));
  return REWB200_OK;
}

int noalloc_setup(Ctx* c);  // noalloc.cu

int buffer_new(Ctx* c, int dtype, const int64_t* dims, int ndims, rewb200_buffer** out) {
  RB_REQUIRE(ndims >= 0 && ndims <= 8, "buffer rank must be 0..8");
  const size_t es = dtype_size(dtype);
  RB_REQUIRE(es != 0, "unsupported dtype code " + std::to_string(dtype));
  rewb200_buffer* b = new rewb200_buffer();
  b->slot = 0;
  for (int i = 0; i < (int)g_ctx.size(); ++i)
    if (g_ctx[i] == c) b->slot = i;
  b->dtype = dtype;
  b->ndims = ndims;
  int64_t n = 1;
  for (int i = 0; i < ndims; ++i) {
    if (dims[i] < 0) {
      delete b;
      return fail("negative dimension");
    }
    b->dims[i] = dims[i];
    n *= dims[i];
  }
  b->bytes = (size_t)n * es;
  if (b->bytes > 0) {
    cudaError_t e = cudaMallocAsync(&b->ptr, (b->bytes + 255) & ~size_t(255), c->stream);
    if (e != cudaSuccess) {
      delete b;
      return fail(std::string("device allocation of ") + std::to_string(n * es) + " bytes failed: " +
                  cudaGetErrorString(e));
    }
  }
  *out = b;
  return REWB200_OK;
}

}  // namespace rewb

using namespace rewb;

extern "C" {

const char* rewb200_last_error(void) { return g_last_error.c_str(); }

int rewb200_init(const int* device_ordinals, int n) {
  std::lock_guard<std::mutex> lk(g_mu);
  RB_REQUIRE(n >= 1 && n <= 16 && device_ordinals, "rewb200_init: need 1..16 device ordinals");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(std::string("rewb200_init: no CUDA device available (") + cudaGetErrorString(e) +
                "); this backend has no CPU fallback");
  if (!g_ctx.empty()) return REWB200_OK;  // idempotent
  for (int i = 0; i < n; ++i) {
    const int dev = device_ordinals[i];
    RB_REQUIRE(dev >= 0 && dev < count, "rewb200_init: device ordinal out of range");
    RB_CUDA(cudaSetDevice(dev));
    cudaDeviceProp prop;
    RB_CUDA(cudaGetDeviceProperties(&prop, dev));
    RB_REQUIRE(prop.major == 10, std::string("rewb200_init: device '") + prop.name +
                                     "' is not compute capability 10.x; this library is built for sm_100a only");
    Ctx* c = new Ctx();
    c->device = dev;
    c->sm_count = prop.multiProcessorCount;
    RB_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    RB_CUDA(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
    RB_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
    RB_CUDA(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
    RB_CUDA(cudaMalloc(&c->d_status, 256));
    RB_CUDA(cudaMemset(c->d_status, 0, 256));
    RB_CUDA(cudaMalloc(&c->d_tickets, Ctx::kTickets * sizeof(int)));
    RB_CUDA(cudaMemset(c->d_tickets, 0, Ctx::kTickets * sizeof(int)));
    RB_CUDA(cudaMallocHost(&c->h_status, 256));
    c->pinned_bytes = 64u << 20;
    RB_CUDA(cudaMallocHost(&c->pinned, c->pinned_bytes));
    cudaMemPool_t pool;
    RB_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t thresh = UINT64_MAX;  // keep freed blocks cached in the pool
    RB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh));
    const char* pdl = getenv("REW_B200_PDL");
    c->use_pdl = !(pdl && pdl[0] == '0');
    const char* li = getenv("REW_B200_LINEAR");
    if (li) c->linear_impl = !strcmp(li, "mma") ? 0 : (!strcmp(li, "tc_prefill") ? 1 : 2);
    RB_TRY(noalloc_setup(c));  // resolves rewb200_linear_noalloc's scratch array and loads its kernels on this device
    g_ctx.push_back(c);
  }
  RB_CUDA(cudaSetDevice(g_ctx[0]->device));
  return REWB200_OK;
}

int rewb200_shutdown(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (Ctx* c : g_ctx) {
    if (!c) continue;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    cudaFree(c->d_status);
    cudaFree(c->d_tickets);
    cudaFreeHost(c->h_status);
    cudaFreeHost(c->pinned);
    cudaStreamDestroy(c->stream);
    cudaStreamDestroy(c->side);
    cudaEventDestroy(c->ev_fork);
    cudaEventDestroy(c->ev_join);
    delete c;
  }
  g_ctx.clear();
  return REWB200_OK;
}

int rewb200_sync(int slot, int timeout_ms) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  cudaEvent_t ev;
  RB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  RB_CUDA(cudaEventRecord(ev, c->stream));
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    cudaError_t q = cudaEventQuery(ev);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) {
      cudaEventDestroy(ev);
      return fail(std::string("rewb200_sync: ") + cudaGetErrorString(q));
    }
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (timeout_ms > 0 && ms > timeout_ms) {
      cudaEventDestroy(ev);
      return fail("rewb200_sync: timed out after " + std::to_string(timeout_ms) + " ms");
    }
  }
  cudaEventDestroy(ev);
  return ctx_check_status(c);
}

int rewb200_set_option(int slot, const char* key, const char* value) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(key && value, "rewb200_set_option: NULL argument");
  RB_CUDA(cudaStreamSynchronize(c->stream));
  const std::string k(key), v(value);
  if (k == "linear") {
    RB_REQUIRE(v == "mma" || v == "tc_prefill" || v == "tc", "option linear: expected mma, tc_prefill or tc");
    c->linear_impl = v == "tc" ? 2 : (v == "tc_prefill" ? 1 : 0);
  } else if (k == "pdl") {
    c->use_pdl = v != "0";
  } else if (k == "prefill") {
    RB_REQUIRE(v == "pair" || v == "persistent" || v == "tile", "option prefill: expected pair, persistent or tile");
    c->prefill_persistent = v != "tile";
    c->prefill_pair = v == "pair";
  } else if (k == "profile_linears") {
    const int mask = atoi(v.c_str());
    RB_REQUIRE(mask >= 1 && mask <= 31, "option profile_linears: a bit mask 1..31 (1 q|k|v, 2 o, 4 gate|up, 8 down, 16 lm_head)");
    c->profile_mask = mask;
  } else if (k == "attention_merge") {
    RB_REQUIRE(v == "fused" || v == "launch", "option attention_merge: expected fused or launch");
    c->attn_fused_merge = v == "fused";
  } else if (k == "ep_exchange") {
    RB_REQUIRE(v == "prefix" || v == "capacity" || v == "auto", "option ep_exchange: expected auto, prefix or capacity");
    c->ep_prefix = v == "prefix" ? 1 : (v == "capacity" ? 0 : 2);
  } else if (k == "tp_exchange") {
    RB_REQUIRE(v == "auto" || v == "one" || v == "two", "option tp_exchange: expected auto, one or two");
    c->tp_exchange = v == "one" ? 1 : (v == "two" ? 2 : 0);
  } else if (k == "gate_up_split") {
    RB_REQUIRE(v == "on" || v == "off", "option gate_up_split: expected on or off");
    c->gu_split = v == "on";
  } else if (k == "qkv_post") {
    RB_REQUIRE(v == "attention" || v == "attention_always" || v == "launch",
               "option qkv_post: expected attention, attention_always or launch");
    c->attn_fuse_qkv = v != "launch";
    c->attn_fuse_qkv_always = v == "attention_always";
  } else if (k == "nf4_gemv") {
    RB_REQUIRE(v == "cuda" || v == "tc", "option nf4_gemv: expected tc or cuda");
    c->nf4_small = v == "cuda";
  } else if (k == "tp_allreduce") {
    RB_REQUIRE(v == "heap" || v == "nccl", "option tp_allreduce: expected heap or nccl");
    c->tp_twoshot = v == "heap";
  } else if (k == "record_routing") {
    c->record_routing = v != "0";
  } else if (k == "inject_alloc_fail") {
    const int n = atoi(v.c_str());
    RB_REQUIRE(n >= 0, "option inject_alloc_fail: a non-negative count");
    c->inject_alloc_fail = n;
  } else if (k == "moe_overlap") {
    RB_REQUIRE(v == "on" || v == "off", "option moe_overlap: expected on or off");
    c->moe_overlap = v == "on";
  } else if (k == "splitk_rows") {
    const int r = atoi(v.c_str());
    RB_REQUIRE(r >= 0 && r <= 256, "option splitk_rows: 0..256");
    c->splitk_max_rows = r;
  } else if (k == "splitk_min_blocks") {
    const int r = atoi(v.c_str());
    RB_REQUIRE(r >= 1 && r <= 64, "option splitk_min_blocks: 1..64");
    c->splitk_min_blocks = r;
  } else if (k == "splitk") {
    RB_REQUIRE(v == "cluster" || v == "slabs" || v == "qkv" || v == "out", "option splitk: expected cluster, slabs, qkv or out");
    c->splitk_cluster = v == "cluster" ? 3 : v == "qkv" ? 1 : v == "out" ? 2 : 0;
  } else if (k == "norm") {
    RB_REQUIRE(v == "cluster" || v == "row", "option norm: expected cluster or row");
    c->norm_cluster = v == "cluster";
  } else if (k == "attention") {
    RB_REQUIRE(v == "tc" || v == "tc1" || v == "tc2" || v == "mma", "option attention: expected tc, tc1, tc2 or mma");
    c->attn_tc = v != "mma";
    c->attn_pingpong = v == "tc" || v == "tc2";
    c->attn_pingpong_min_rows = v == "tc2" ? 256 : 3072;
  } else if (k == "sampling") {
    RB_REQUIRE(v == "bucket" || v == "radix", "option sampling: expected bucket or radix");
    c->sampling_exact = v == "radix";
  } else {
    return fail("rewb200_set_option: unknown option '" + k + "'");
  }
  ++c->option_epoch;
  return REWB200_OK;
}

int64_t rewb200_launch_count(int slot) {
  (void)slot;  // one process drives one GPU; the counter is process-wide
  return g_launch_total;
}

int rewb200_buffer_alloc(int slot, int dtype, const int64_t* dims, int ndims, rewb200_buffer** out) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(out != nullptr, "rewb200_buffer_alloc: out is NULL");
  RB_CUDA(cudaSetDevice(c->device));
  return buffer_new(c, dtype, dims, ndims, out);
}

int rewb200_buffer_from_host(int slot, const void* src, int dtype, const int64_t* dims, int ndims,
                             rewb200_buffer** out) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(out != nullptr, "rewb200_buffer_from_host: out is NULL");
  RB_CUDA(cudaSetDevice(c->device));
  rewb200_buffer* b = nullptr;
  RB_TRY(buffer_new(c, dtype, dims, ndims, &b));
  if (b->bytes > 0) {
    RB_REQUIRE(src != nullptr, "rewb200_buffer_from_host: src is NULL");
    // Stage through pinned memory in chunks so the copy is a true async DMA.
    size_t off = 0;
    while (off < b->bytes) {
      const size_t n = std::min(c->pinned_bytes, b->bytes - off);
      memcpy(c->pinned, (const char*)src + off, n);
      RB_CUDA(cudaMemcpyAsync((char*)b->ptr + off, c->pinned, n, cudaMemcpyHostToDevice, c->stream));
      RB_CUDA(cudaStreamSynchronize(c->stream));
      off += n;
    }
  }
  *out = b;
  return REWB200_OK;
}

int rewb200_buffer_to_host(const rewb200_buffer* buf, void* dst, size_t nbytes) {
  RB_REQUIRE(buf != nullptr && (dst != nullptr || nbytes == 0), "rewb200_buffer_to_host: NULL argument");
  Ctx* c = ctx_get(buf->slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(nbytes <= buf->bytes, "rewb200_buffer_to_host: destination larger than the buffer (" +
                                       std::to_string(nbytes) + " > " + std::to_string(buf->bytes) + ")");
  RB_CUDA(cudaSetDevice(c->device));
  size_t off = 0;
  while (off < nbytes) {
    const size_t n = std::min(c->pinned_bytes, nbytes - off);
    RB_CUDA(cudaMemcpyAsync(c->pinned, (const char*)buf->ptr + off, n, cudaMemcpyDeviceToHost, c->stream));
    RB_CUDA(cudaStreamSynchronize(c->stream));
    memcpy((char*)dst + off, c->pinned, n);
    off += n;
  }
  if (nbytes == 0) RB_CUDA(cudaStreamSynchronize(c->stream));
  return ctx_check_status(c);
}

int rewb200_buffer_info(const rewb200_buffer* buf, int* dtype, int64_t* dims, int* ndims) {
  RB_REQUIRE(buf != nullptr, "rewb200_buffer_info: NULL buffer");
  if (dtype) *dtype = buf->dtype;
  if (ndims) *ndims = buf->ndims;
  if (dims)
    for (int i = 0; i < buf->ndims; ++i) dims[i] = buf->dims[i];
  return REWB200_OK;
}

void* rewb200_buffer_device_ptr(const rewb200_buffer* buf) { return buf ? buf->ptr : nullptr; }

void rewb200_buffer_release(rewb200_buffer* buf) {
  if (!buf) return;
  if (buf->owned && buf->ptr && buf->slot < (int)g_ctx.size() && g_ctx[buf->slot]) {
    Ctx* c = g_ctx[buf->slot];
    cudaSetDevice(c->device);
    cudaFreeAsync(buf->ptr, c->stream);
  }
  buf->ptr = nullptr;
  delete buf;
}

}  // extern "C"
