// Exchange + merge of the sequence-sharded decode partials over peer memory, one launch per call.
//
// Sequence sharding (no counterpart in the reference, whose decode call is
// src/ops/d_stage_kv_cache.py:219-303 on one GPU) leaves every rank with the un-normalised softmax state
// (m, l, acc) of its shard; the result is their log-sum-exp merge.  Instead of a collective followed by a merge
// kernel, every rank launches this one kernel: block r writes row r of the local state into slot [rank] of every
// peer's exchange buffer with plain stores through NVLink (peer pointers, no multicast), publishes it with a
// system-scope release store of the call's sequence number into the peer's flag word for (rank, r), waits - with a
// time limit - for the same flag from every peer, and merges row r from the slots of its own buffer.
//
// Exchange buffer of one rank (all ranks use the same layout):
//   [0, 256)                                  header: word 0 = status (bit 1: a wait ran out)
//   flags  u32 [2][world][rows_pad]           sequence number of the last call whose row has arrived
//   slots  f32 [2][world][msg]                msg = m [rows] | l [rows] | acc [rows][128], rounded up to 64 floats
// Two parities (seq & 1): a rank can be at most one call ahead of a peer, because its wait needs the peer's flags of the
// same call, and the peer raises them only after its kernel of the call before has finished (stream order).
//
// The local partial is produced directly in slot [seq & 1][rank] of the local buffer by the decode kernel
// (hq_peer_slot gives the pointers for partial_m / partial_l / partial_acc).
#include <cstring>

#include "hq_common.cuh"

namespace hq {

constexpr int kPeerMaxWorld = 16;
constexpr int kPeerHeaderBytes = 256;

struct PeerLayout {
  int64_t rows_pad, msg, flags_off, slots_off, bytes;
};
__host__ __device__ inline PeerLayout peer_layout(int world, int rows) {
  PeerLayout L;
  L.rows_pad = (rows + 31) / 32 * 32;
  L.msg = ((int64_t)rows * 130 + 63) / 64 * 64;
  L.flags_off = kPeerHeaderBytes;
  L.slots_off = L.flags_off + 2 * (int64_t)world * L.rows_pad * 4;
  L.slots_off = (L.slots_off + 255) / 256 * 256;
  L.bytes = L.slots_off + 2 * (int64_t)world * L.msg * 4;
  return L;
}

struct PeerParams {
  uint8_t* bufs[kPeerMaxWorld];
  int world, rank, rows;
  uint32_t seq;
  void* out; int out_dtype; int64_t out_stride;
  int64_t timeout_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Grid: at most as many blocks as are resident at once; a block first pushes and publishes all of its rows and only
// then waits, so every rank's flags are raised without depending on anything another rank does.
__global__ void __launch_bounds__(128)
peer_exchange_merge_kernel(const PeerParams p) {
  const int d = threadIdx.x;
  const PeerLayout L = peer_layout(p.world, p.rows);
  const int par = (int)(p.seq & 1u);
  uint8_t* mine = p.bufs[p.rank];
  const int64_t slot_of_me = ((int64_t)par * p.world + p.rank) * L.msg;
  const float* my_slot = reinterpret_cast<const float*>(mine + L.slots_off) + slot_of_me;
  uint8_t* peer = (d < p.world && d != p.rank) ? p.bufs[d] : nullptr;     // thread d publishes to / waits for rank d

  for (int r = blockIdx.x; r < p.rows; r += gridDim.x) {
    const float my_m = my_slot[r], my_l = my_slot[p.rows + r], my_a = my_slot[2 * (int64_t)p.rows + (int64_t)r * 128 + d];
    // 1. push row r to every peer
    for (int j = 0; j < p.world; ++j) {
      if (j == p.rank) continue;
      float* dst = reinterpret_cast<float*>(p.bufs[j] + L.slots_off) + slot_of_me;
      dst[2 * (int64_t)p.rows + (int64_t)r * 128 + d] = my_a;
      if (d == 0) { dst[r] = my_m; dst[p.rows + r] = my_l; }
    }
    __syncthreads();
    // 2. publish: the barrier orders every thread's stores before thread d's fence + release store
    if (peer != nullptr) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(peer + L.flags_off) + ((int64_t)par * p.world + p.rank) * L.rows_pad + r, p.seq);
    }
  }

  const float* slots = reinterpret_cast<const float*>(mine + L.slots_off) + (int64_t)par * p.world * L.msg;
  for (int r = blockIdx.x; r < p.rows; r += gridDim.x) {
    // 3. wait for row r of every peer, with a time limit
    if (peer != nullptr) {
      const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + L.flags_off) + ((int64_t)par * p.world + d) * L.rows_pad + r;
      const uint64_t t0 = global_timer_ns();
      bool ok = true;
      while (ld_acquire_sys(flag) != p.seq) {
        if ((int64_t)(global_timer_ns() - t0) > p.timeout_ns) { ok = false; break; }
        __nanosleep(20);
      }
      if (!ok) atomicOr(reinterpret_cast<int*>(mine), 2);
    }
    __syncthreads();
    // 4. merge row r over the ranks' slots in the local buffer
    float M = -INFINITY;
    for (int j = 0; j < p.world; ++j) M = fmaxf(M, __ldcg(slots + j * L.msg + r));
    float num = 0.f, den = 0.f;
    for (int j = 0; j < p.world; ++j) {
      const float* s = slots + j * L.msg;
      const float mj = __ldcg(s + r);
      const float w = (mj == -INFINITY) ? 0.f : ex2f(mj - M);
      num += w * __ldcg(s + 2 * (int64_t)p.rows + (int64_t)r * 128 + d);
      den += w * __ldcg(s + p.rows + r);
    }
    store_out(p.out, (int64_t)r * p.out_stride + d, den > 0.f ? num / den : 0.f, p.out_dtype);
  }
}

}  // namespace hq

extern "C" int hq_peer_exchange_bytes(int world, int rows, int64_t* bytes) {
  using namespace hq;
  HQ_REQUIRE(bytes && world >= 1 && world <= kPeerMaxWorld && rows >= 1, HQ_ERR_INVALID,
             "hq_peer_exchange_bytes: 1 <= world <= %d and rows >= 1 required", kPeerMaxWorld);
  *bytes = peer_layout(world, rows).bytes;
  return HQ_OK;
}

extern "C" int hq_peer_slot(void* buf, int world, int rows, uint32_t seq, int rank, float** m, float** l, float** acc) {
  using namespace hq;
  HQ_REQUIRE(buf && m && l && acc && world >= 1 && world <= kPeerMaxWorld && rank >= 0 && rank < world && rows >= 1,
             HQ_ERR_INVALID, "hq_peer_slot: bad argument");
  const PeerLayout L = peer_layout(world, rows);
  float* s = reinterpret_cast<float*>((uint8_t*)buf + L.slots_off) + ((int64_t)(seq & 1u) * world + rank) * L.msg;
  *m = s; *l = s + rows; *acc = s + 2 * (int64_t)rows;
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
    p.bufs[j] = (uint8_t*)a->bufs[j];
  }
  p.world = a->world; p.rank = a->rank; p.rows = a->rows; p.seq = a->seq;
  p.out = a->out; p.out_dtype = a->out_dtype; p.out_stride = a->out_stride;
  p.timeout_ns = a->timeout_ns > 0 ? a->timeout_ns : 2000000000ll;
  const int resident = 8 * sm_count();          // 128-thread blocks with 40 registers: at least 8 per SM
  peer_exchange_merge_kernel<<<a->rows < resident ? a->rows : resident, 128, 0, (cudaStream_t)stream>>>(p);
  HQ_CUDA(cudaGetLastError());
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
