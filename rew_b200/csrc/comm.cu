// Tensor/expert-parallel communication: allReduce / allToAll of
// src/rew/ops/distributed.nim:62-83,106-128 executed with NCCL over NVLink, one
// process per GPU.  NCCL is resolved at run time (dlopen) so the library loads
// on hosts without it and shares the copy a host process may already have
// loaded.  Collectives run on the slot's stream, so they can be captured into
// the decode graph.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace rewb {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
};
static NcclApi g_nccl;

struct Comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
};
static Comm g_comm[16];

static int nccl_load() {
  if (g_nccl.handle) return REWB200_OK;
  // REW_B200_NCCL names a specific library; otherwise whatever libnccl.so.2 the process already
  // holds (or the system one) is used.
  const char* envp = getenv("REW_B200_NCCL");
  const char* names[] = {envp ? envp : "libnccl.so.2", "libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  RB_REQUIRE(h != nullptr, std::string("NCCL library not found (dlopen libnccl.so.2): ") + dlerror());
#define RB_SYM(field, name)                                                     \
  *(void**)(&g_nccl.field) = dlsym(h, name);                                    \
  RB_REQUIRE(g_nccl.field != nullptr, std::string("NCCL symbol missing: ") + name)
  RB_SYM(GetUniqueId, "ncclGetUniqueId");
  RB_SYM(CommInitRank, "ncclCommInitRank");
  RB_SYM(CommDestroy, "ncclCommDestroy");
  RB_SYM(CommAbort, "ncclCommAbort");
  RB_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
  RB_SYM(GetErrorString, "ncclGetErrorString");
  RB_SYM(AllReduce, "ncclAllReduce");
  RB_SYM(AllGather, "ncclAllGather");
  RB_SYM(Send, "ncclSend");
  RB_SYM(Recv, "ncclRecv");
  RB_SYM(GroupStart, "ncclGroupStart");
  RB_SYM(GroupEnd, "ncclGroupEnd");
#undef RB_SYM
  g_nccl.handle = h;
  return REWB200_OK;
}

#define RB_NCCL(expr)                                                                                   \
  do {                                                                                                  \
    ncclResult_t _r = (expr);                                                                           \
    if (_r != ncclSuccess) return fail(std::string(#expr) + ": " + g_nccl.GetErrorString(_r));          \
  } while (0)

int comm_world(int slot) { return (slot >= 0 && slot < 16 && g_comm[slot].comm) ? g_comm[slot].world : 1; }
int comm_rank(int slot) { return (slot >= 0 && slot < 16 && g_comm[slot].comm) ? g_comm[slot].rank : 0; }

int comm_allreduce_sum(Ctx* c, int slot, void* ptr, int64_t n, int dtype) {
  RB_REQUIRE(slot >= 0 && slot < 16 && g_comm[slot].comm, "rewb200_comm_init has not been called for this slot");
  RB_REQUIRE(dtype == REWB200_F32 || dtype == REWB200_BF16, "all-reduce payload must be f32 or bf16");
  RB_NCCL(g_nccl.AllReduce(ptr, ptr, (size_t)n, dtype == REWB200_F32 ? ncclFloat : ncclBfloat16, ncclSum, g_comm[slot].comm,
                           c->stream));
  return REWB200_OK;
}

int comm_allgather_bytes(Ctx* c, int slot, const void* send, void* recv, size_t bytes_per_rank) {
  RB_REQUIRE(slot >= 0 && slot < 16 && g_comm[slot].comm, "rewb200_comm_init has not been called for this slot");
  RB_NCCL(g_nccl.AllGather(send, recv, bytes_per_rank, ncclChar, g_comm[slot].comm, c->stream));
  return REWB200_OK;
}

// Equal-count all-to-all: rank r sends bytes [p*bytes, (p+1)*bytes) of `send` to peer p.
int comm_alltoall_bytes(Ctx* c, int slot, const void* send, void* recv, size_t bytes_per_peer) {
  RB_REQUIRE(slot >= 0 && slot < 16 && g_comm[slot].comm, "rewb200_comm_init has not been called for this slot");
  Comm& cm = g_comm[slot];
  RB_NCCL(g_nccl.GroupStart());
  for (int p = 0; p < cm.world; ++p) {
    RB_NCCL(g_nccl.Send((const char*)send + (size_t)p * bytes_per_peer, bytes_per_peer, ncclChar, p, cm.comm, c->stream));
    RB_NCCL(g_nccl.Recv((char*)recv + (size_t)p * bytes_per_peer, bytes_per_peer, ncclChar, p, cm.comm, c->stream));
  }
  RB_NCCL(g_nccl.GroupEnd());
  return REWB200_OK;
}

// All-to-all of row prefixes: the block for peer p starts at p * peer_stride_bytes in both buffers; this rank
// sends its first send_rows[p] rows of it and receives recv_rows[p] rows (host arrays; send_rows[p] here equals
// recv_rows[this rank] on peer p).
int comm_alltoallv_rows(Ctx* c, int slot, const void* send, void* recv, size_t peer_stride_bytes, size_t row_bytes,
                        const int* send_rows, const int* recv_rows) {
  RB_REQUIRE(slot >= 0 && slot < 16 && g_comm[slot].comm, "rewb200_comm_init has not been called for this slot");
  Comm& cm = g_comm[slot];
  RB_NCCL(g_nccl.GroupStart());
  for (int p = 0; p < cm.world; ++p) {
    if (send_rows[p] > 0)
      RB_NCCL(g_nccl.Send((const char*)send + (size_t)p * peer_stride_bytes, (size_t)send_rows[p] * row_bytes, ncclChar, p,
                          cm.comm, c->stream));
    if (recv_rows[p] > 0)
      RB_NCCL(g_nccl.Recv((char*)recv + (size_t)p * peer_stride_bytes, (size_t)recv_rows[p] * row_bytes, ncclChar, p, cm.comm,
                          c->stream));
  }
  RB_NCCL(g_nccl.GroupEnd());
  return REWB200_OK;
}

// ---- peer heap: exchange memory for the fused all-reduce and the expert-parallel all-to-all ----------
// One cudaMalloc per rank, exported with CUDA IPC and mapped by every other rank of the node:
//   [0, 16 KiB)   header: epoch counter (int 0), all-to-all epoch (int 1), arrival counters of the all-to-all
//                 kernels (ints 2, 3); at 256 the all-to-all cells: pair counts [8], dispatch flags [8],
//                 return flags [8]
//   then          two alternating all-reduce exchange buffers of world x buf_bytes each
//   then          the all-to-all region (a2a_bytes)
// Peers are written with plain stores and never read; every rank reads only its own memory.
constexpr size_t kHeapHeader = 16384;
constexpr size_t kHeapA2aCellsOff = 256;

struct PeerHeap {
  void* local = nullptr;
  void* mapped[8] = {};
  PeerInfo info;
  bool attached = false;
};
static PeerHeap g_heap[16];

static void heap_fill(PeerInfo* info, int r, char* base, bool own) {
  const size_t ar = (size_t)info->world * info->buf_bytes;
  info->bufs[0][r] = base + kHeapHeader;
  info->bufs[1][r] = base + kHeapHeader + ar;
  info->a2a_flags[r] = (int*)(base + kHeapA2aCellsOff);
  info->a2a[r] = info->a2a_bytes ? base + kHeapHeader + 2 * ar : nullptr;
  if (own) info->epoch = (int*)base;
}

// After a synchronisation of the slot's stream: reports an error NCCL raised asynchronously (a rank that went
// away, a transport fault) instead of leaving it to the next collective; the communicator is aborted then.
int comm_check_async(int slot) {
  if (slot < 0 || slot >= 16 || !g_comm[slot].comm) return REWB200_OK;
  ncclResult_t async = ncclSuccess;
  RB_NCCL(g_nccl.CommGetAsyncError(g_comm[slot].comm, &async));
  if (async != ncclSuccess) {
    g_nccl.CommAbort(g_comm[slot].comm);
    g_comm[slot].comm = nullptr;
    return fail(std::string("NCCL asynchronous error: ") + g_nccl.GetErrorString(async));
  }
  return REWB200_OK;
}

const PeerInfo* comm_peer_info(int slot) {
  return (slot >= 0 && slot < 16 && g_heap[slot].attached) ? &g_heap[slot].info : nullptr;
}

}  // namespace rewb

using namespace rewb;

extern "C" {

int rewb200_comm_peer_alloc(int slot, int64_t allreduce_bytes, int64_t alltoall_bytes, void* handle64) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(handle64 != nullptr && allreduce_bytes >= 0 && alltoall_bytes >= 0 && allreduce_bytes % 256 == 0 &&
                 alltoall_bytes % 256 == 0 && allreduce_bytes + alltoall_bytes > 0,
             "rewb200_comm_peer_alloc: sizes must be non-negative multiples of 256, not both zero");
  RB_REQUIRE(slot < 16 && g_comm[slot].comm, "rewb200_comm_peer_alloc: call rewb200_comm_init first");
  RB_REQUIRE(g_comm[slot].world <= 8, "the peer heap supports up to 8 ranks");
  RB_REQUIRE(!g_heap[slot].local, "rewb200_comm_peer_alloc: already allocated for this slot");
  RB_CUDA(cudaSetDevice(c->device));
  PeerHeap& h = g_heap[slot];
  const size_t total = kHeapHeader + 2 * (size_t)g_comm[slot].world * (size_t)allreduce_bytes + (size_t)alltoall_bytes;
  RB_CUDA(cudaMalloc(&h.local, total));
  RB_CUDA(cudaMemset(h.local, 0, kHeapHeader + 2 * (size_t)g_comm[slot].world * (size_t)allreduce_bytes));  // flag 0 = no data yet
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
  cudaIpcMemHandle_t ih;
  RB_CUDA(cudaIpcGetMemHandle(&ih, h.local));
  memcpy(handle64, &ih, 64);
  h.info.world = g_comm[slot].world;
  h.info.rank = g_comm[slot].rank;
  h.info.buf_bytes = (size_t)allreduce_bytes;
  h.info.a2a_bytes = (size_t)alltoall_bytes;
  return REWB200_OK;
}

int rewb200_comm_peer_attach(int slot, const void* handles_all) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(slot < 16 && g_heap[slot].local && handles_all, "rewb200_comm_peer_attach: call rewb200_comm_peer_alloc first");
  RB_REQUIRE(!g_heap[slot].attached, "rewb200_comm_peer_attach: already attached for this slot");
  RB_CUDA(cudaSetDevice(c->device));
  PeerHeap& h = g_heap[slot];
  for (int r = 0; r < h.info.world; ++r) {
    void* base = h.local;
    if (r != h.info.rank) {
      cudaIpcMemHandle_t ih;
      memcpy(&ih, (const char*)handles_all + (size_t)r * 64, 64);
      RB_CUDA(cudaIpcOpenMemHandle(&h.mapped[r], ih, cudaIpcMemLazyEnablePeerAccess));
      base = h.mapped[r];
    }
    heap_fill(&h.info, r, (char*)base, r == h.info.rank);
  }
  RB_CUDA(cudaDeviceSynchronize());
  h.attached = true;
  return REWB200_OK;
}

int rewb200_comm_unique_id(void* id128) {
  RB_REQUIRE(id128 != nullptr, "rewb200_comm_unique_id: NULL buffer");
  RB_TRY(nccl_load());
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  RB_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, 128);
  return REWB200_OK;
}

int rewb200_comm_init(int slot, const void* id128, int rank, int world) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(id128 != nullptr && world >= 1 && rank >= 0 && rank < world, "rewb200_comm_init: bad rank/world");
  RB_REQUIRE(slot < 16 && !g_comm[slot].comm, "rewb200_comm_init: communicator already exists for this slot");
  RB_TRY(nccl_load());
  RB_CUDA(cudaSetDevice(c->device));
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  RB_NCCL(g_nccl.CommInitRank(&g_comm[slot].comm, world, id, rank));
  g_comm[slot].rank = rank;
  g_comm[slot].world = world;
  return REWB200_OK;
}

static int comm_finish(Ctx* c, int slot);

int rewb200_comm_allreduce_f32(int slot, void* device_ptr, int64_t n) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_CUDA(cudaSetDevice(c->device));
  RB_TRY(comm_allreduce_sum(c, slot, device_ptr, n, REWB200_F32));
  return comm_finish(c, slot);
}

static int comm_finish(Ctx* c, int slot) {
  RB_CUDA(cudaStreamSynchronize(c->stream));
  return comm_check_async(slot);
}

int rewb200_comm_alltoall(int slot, const void* send_device, void* recv_device, int64_t bytes_per_peer) {
  Ctx* c = ctx_get(slot);
  if (!c) return REWB200_ERR;
  RB_REQUIRE(send_device && recv_device && bytes_per_peer >= 0, "allToAll: NULL buffer or negative size");
  RB_REQUIRE(send_device != recv_device, "allToAll: send and receive buffers must differ");
  RB_CUDA(cudaSetDevice(c->device));
  if (bytes_per_peer == 0) return REWB200_OK;
  RB_TRY(comm_alltoall_bytes(c, slot, send_device, recv_device, (size_t)bytes_per_peer));
  return comm_finish(c, slot);
}

int rewb200_comm_destroy(int slot) {
  if (slot < 0 || slot >= 16 || !g_comm[slot].comm) return REWB200_OK;
  Ctx* c = ctx_get(slot);
  if (c) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
  }
  PeerHeap& h = g_heap[slot];
  if (h.local) {
    for (int r = 0; r < 8; ++r)
      if (h.mapped[r]) cudaIpcCloseMemHandle(h.mapped[r]);
    cudaFree(h.local);
    h = PeerHeap();
  }
  g_nccl.CommDestroy(g_comm[slot].comm);
  g_comm[slot].comm = nullptr;
  return REWB200_OK;
}

}  // extern "C"
