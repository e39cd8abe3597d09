// Exchange + merge of the sequence-sharded decode partials over peer memory, one launch per call.
//
// Sequence sharding (no counterpart in the reference, whose decode call is
// src/ops/d_stage_kv_cache.py:219-303 on one GPU) leaves every rank with the un-normalised softmax state
// (m, l, acc) of its shard; the result is their log-sum-exp merge.  Instead of a collective followed by a merge
// kernel, every rank launches this one kernel.  Thread d of the block of row r stores element d of the row into
// slot [rank] of every peer's exchange buffer with plain 8-byte stores through NVLink (peer pointers, no multicast):
// each store carries the fp32 value and the call's sequence number, so a word is valid exactly when its upper half
// equals the sequence number and no fence or separate flag is needed.  The same thread then polls - with a time
// limit - the words the peers store for (r, d) in its own buffer and merges them.
//
// Exchange buffer of one rank (all ranks use the same layout):
//   [0, 256)                        header: word 0 = status (bit 1: a wait ran out)
//   local f32 [2][msg]              the rank's own state of a call, m [rows] | l [rows] | acc [rows][128], written by
//                                   the decode kernel (hq_peer_slot gives partial_m / partial_l / partial_acc)
//   recv  {f32, u32} [2][world][rows * 130]   what the peers store: the same elements, each with the sequence number
// Two parities (seq & 1): a rank can be at most one call ahead of a peer, because its wait needs the peer's words of
// the same call, and the peer stores them only after its kernel of the call before has finished (stream order).
#include <cstring>

#include "hq_peer.cuh"

namespace hq {

struct PeerParams {
  PeerGroup g;
  void* out; int out_dtype; int64_t out_stride;
};

// Grid: at most as many blocks as are resident at once; a block first stores all of its rows to the peers and only
// then waits, so every rank's words are on their way without depending on anything another rank does.
__global__ void __launch_bounds__(128)
peer_exchange_merge_kernel(const PeerParams p) {
  // Launched as a programmatic dependent of the kernel before it on the stream (the decode call that writes this
  // rank's state): its blocks may be resident before that kernel ends and wait here for its completion.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int d = threadIdx.x;
  const PeerGroup& g = p.g;
  const PeerLayout L = peer_layout(g.world, g.rows);
  const float* local = reinterpret_cast<const float*>(g.bufs[g.rank] + L.local_off) + (int64_t)(g.seq & 1u) * L.msg;

  for (int r = blockIdx.x; r < g.rows; r += gridDim.x) {
    const int64_t ia = 2 * (int64_t)g.rows + (int64_t)r * 128 + d;
    peer_push(g, L, ia, local[ia]);
    if (d < 2) peer_push(g, L, d * g.rows + r, local[d * g.rows + r]);      // thread 0: m, thread 1: l
  }
  bool expired = false;
  for (int r = blockIdx.x; r < g.rows; r += gridDim.x) {
    const float v = peer_merge(g, L, r, d, local[r], local[g.rows + r], local[2 * (int64_t)g.rows + (int64_t)r * 128 + d], &expired);
    store_out(p.out, (int64_t)r * p.out_stride + d, v, p.out_dtype);
  }
  if (expired) atomicOr(reinterpret_cast<int*>(g.bufs[g.rank]), 2);
}

}  // namespace hq

extern "C" int hq_peer_exchange_bytes(int world, int rows, int64_t* bytes) {
  using namespace hq;
  HQ_REQUIRE(bytes && world >= 1 && world <= kPeerMaxWorld && rows >= 1, HQ_ERR_INVALID,
             "hq_peer_exchange_bytes: 1 <= world <= %d and rows >= 1 required", kPeerMaxWorld);
  *bytes = peer_layout(world, rows).bytes;
  return HQ_OK;
}

extern "C" int hq_peer_slot(void* buf, int world, int rows, uint32_t seq, float** m, float** l, float** acc) {
  using namespace hq;
  HQ_REQUIRE(buf && m && l && acc && world >= 1 && world <= kPeerMaxWorld && rows >= 1, HQ_ERR_INVALID,
             "hq_peer_slot: bad argument");
  const PeerLayout L = peer_layout(world, rows);
  float* s = reinterpret_cast<float*>((uint8_t*)buf + L.local_off) + (int64_t)(seq & 1u) * L.msg;
  *m = s; *l = s + rows; *acc = s + 2 * (int64_t)rows;
  return HQ_OK;
}

extern "C" int hq_peer_recv_slot(void* buf, int world, int rows, uint32_t seq, int src_rank, void** words) {
  using namespace hq;
  HQ_REQUIRE(buf && words && world >= 1 && world <= kPeerMaxWorld && src_rank >= 0 && src_rank < world && rows >= 1,
             HQ_ERR_INVALID, "hq_peer_recv_slot: bad argument");
  const PeerLayout L = peer_layout(world, rows);
  *words = (uint8_t*)buf + L.recv_off + (((int64_t)(seq & 1u) * world + src_rank) * L.msg) * 8;
  return HQ_OK;
}

extern "C" int hq_peer_exchange_merge(const hq_peer_exchange_args* a, void* stream) {
  using namespace hq;
  HQ_REQUIRE(a != nullptr && a->struct_bytes == (int32_t)sizeof(hq_peer_exchange_args), HQ_ERR_INVALID,
             "hq_peer_exchange_merge: null args or struct_bytes mismatch");
  HQ_REQUIRE(a->world >= 1 && a->world <= kPeerMaxWorld && a->rank >= 0 && a->rank < a->world && a->rows >= 1, HQ_ERR_INVALID,
             "hq_peer_exchange_merge: world %d rank %d rows %d", a->world, a->rank, a->rows);
  HQ_REQUIRE(a->seq != 0 && a->out != nullptr, HQ_ERR_INVALID, "hq_peer_exchange_merge: seq starts at 1; out must be set");
  HQ_REQUIRE(a->out_dtype == HQ_BF16 || a->out_dtype == HQ_F16 || a->out_dtype == HQ_F32, HQ_ERR_UNSUPPORTED,
             "hq_peer_exchange_merge: out_dtype %d", a->out_dtype);
  PeerParams p{};
  for (int j = 0; j < a->world; ++j) {
    HQ_REQUIRE(a->bufs[j] != nullptr && ((uintptr_t)a->bufs[j] & 255) == 0, HQ_ERR_ALIGNMENT,
               "hq_peer_exchange_merge: buffer %d null or not 256-byte aligned", j);
    p.g.bufs[j] = (uint8_t*)a->bufs[j];
  }
  p.g.world = a->world; p.g.rank = a->rank; p.g.rows = a->rows; p.g.seq = a->seq;
  p.out = a->out; p.out_dtype = a->out_dtype; p.out_stride = a->out_stride;
  p.g.timeout_ns = a->timeout_ns > 0 ? a->timeout_ns : 2000000000ll;
  static thread_local int per_sm = 0;            // blocks of this kernel that are resident on one SM at a time
  if (per_sm == 0) {
    HQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_exchange_merge_kernel, 128, 0));
    if (per_sm < 1) per_sm = 1;
  }
  const int resident = per_sm * sm_count();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(a->rows < resident ? a->rows : resident));
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HQ_CUDA(cudaLaunchKernelEx(&cfg, peer_exchange_merge_kernel, p));
  return HQ_OK;
}

extern "C" int hq_peer_status(const void* buf, int* status) {
  using namespace hq;
  HQ_REQUIRE(buf && status, HQ_ERR_INVALID, "hq_peer_status: null pointer");
  HQ_CUDA(cudaMemcpy(status, buf, sizeof(int), cudaMemcpyDeviceToHost));     // synchronises with the device
  return HQ_OK;
}

// ---- exchange buffers shared between the processes of one node (CUDA IPC) ------------------------------------
extern "C" int hq_peer_buffer_create(int64_t bytes, void** ptr, void* handle64) {
  using namespace hq;
  HQ_REQUIRE(ptr && handle64 && bytes > 0, HQ_ERR_INVALID, "hq_peer_buffer_create: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  HQ_CUDA(cudaMalloc(&p, (size_t)bytes));
  HQ_CUDA(cudaMemset(p, 0, (size_t)bytes));
  cudaIpcMemHandle_t h;
  HQ_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, 64);
  *ptr = p;
  return HQ_OK;
}
extern "C" int hq_peer_buffer_open(const void* handle64, void** ptr) {
  using namespace hq;
  HQ_REQUIRE(ptr && handle64, HQ_ERR_INVALID, "hq_peer_buffer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  HQ_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return HQ_OK;
}
extern "C" int hq_peer_buffer_close(void* ptr) {
  using namespace hq;
  if (ptr) HQ_CUDA(cudaIpcCloseMemHandle(ptr));
  return HQ_OK;
}
extern "C" int hq_peer_buffer_destroy(void* ptr) {
  using namespace hq;
  if (ptr) HQ_CUDA(cudaFree(ptr));
  return HQ_OK;
}
