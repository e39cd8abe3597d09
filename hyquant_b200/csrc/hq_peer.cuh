// Layout of a peer-exchange buffer and the device primitives of the exchange (see hq_peer.cu for the protocol).
#pragma once
#include "hq_common.cuh"

namespace hq {

constexpr int kPeerMaxWorld = 16;
constexpr int kPeerHeaderBytes = 256;

struct PeerLayout {
  int64_t elems, msg, local_off, recv_off, bytes;
};
__host__ __device__ inline PeerLayout peer_layout(int world, int rows) {
  PeerLayout L;
  L.elems = (int64_t)rows * 130;
  L.msg = (L.elems + 63) / 64 * 64;
  L.local_off = kPeerHeaderBytes;
  L.recv_off = L.local_off + 2 * L.msg * 4;
  L.bytes = L.recv_off + 2 * (int64_t)world * L.msg * 8;
  return L;
}

// What a kernel needs to take part in an exchange: every rank's buffer as addressable from this GPU.
struct PeerGroup {
  uint8_t* bufs[kPeerMaxWorld];
  int world, rank, rows;
  uint32_t seq;
  int64_t timeout_ns;
};

// A word of the exchange is {fp32 value, uint32 sequence number} and is valid exactly when its upper half equals the
// call's sequence number.  That needs the two halves to become visible together, so each word moves as ONE 8-byte
// scalar access (naturally aligned b64 accesses are single-copy atomic; the elements of a .v2.b32 access are not
// guaranteed to be).
__device__ __forceinline__ void st_pair_sys(uint2* p, float v, uint32_t seq) {
  const uint64_t w = (uint64_t)__float_as_uint(v) | ((uint64_t)seq << 32);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2* p) {
  uint64_t w;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Poll one word until it carries `seq`; gives up (returns 0 and sets *expired) after the time limit.
__device__ __forceinline__ float wait_pair(const uint2* p, uint32_t seq, int64_t timeout_ns, bool* expired) {
  uint2 v = ld_pair_sys(p);
  if (v.y != seq && !*expired) {
    const uint64_t t0 = global_timer_ns();
    int spins = 0;
    while ((v = ld_pair_sys(p)).y != seq) {
      if ((++spins & 63) == 0 && (int64_t)(global_timer_ns() - t0) > timeout_ns) { *expired = true; break; }
    }
  }
  return v.y == seq ? __uint_as_float(v.x) : 0.f;
}

// Store element `idx` (position in m [rows] | l [rows] | acc [rows][128]) of this rank's state into every peer's buffer.
__device__ __forceinline__ void peer_push(const PeerGroup& g, const PeerLayout& L, int64_t idx, float v) {
  const int64_t my_recv = ((int64_t)(g.seq & 1u) * g.world + g.rank) * L.msg;
  for (int j = 0; j < g.world; ++j) {
    if (j == g.rank) continue;
    st_pair_sys(reinterpret_cast<uint2*>(g.bufs[j] + L.recv_off) + my_recv + idx, v, g.seq);
  }
}

// Log-sum-exp merge of channel d of row r over all ranks: this rank's (m, l, a) from registers, the peers' from the
// words they store into this rank's buffer (polled with the time limit).  Returns the normalised value.
__device__ __forceinline__ float peer_merge(const PeerGroup& g, const PeerLayout& L, int r, int d, float my_m, float my_l,
                                            float my_a, bool* expired) {
  const uint2* recv = reinterpret_cast<const uint2*>(g.bufs[g.rank] + L.recv_off) + (int64_t)(g.seq & 1u) * g.world * L.msg;
  const int64_t ia = 2 * (int64_t)g.rows + (int64_t)r * 128 + d;
  // every peer's three words are requested before any is looked at: one round trip when they have all arrived
  uint2 wm[kPeerMaxWorld], wl[kPeerMaxWorld], wa[kPeerMaxWorld];
#pragma unroll
  for (int j = 0; j < kPeerMaxWorld; ++j) {
    if (j < g.world && j != g.rank) {
      wm[j] = ld_pair_sys(recv + j * L.msg + r);
      wl[j] = ld_pair_sys(recv + j * L.msg + g.rows + r);
      wa[j] = ld_pair_sys(recv + j * L.msg + ia);
    }
  }
  float M = my_m;
#pragma unroll
  for (int j = 0; j < kPeerMaxWorld; ++j) {
    if (j < g.world && j != g.rank) {
      if (wm[j].y != g.seq) wm[j].x = __float_as_uint(wait_pair(recv + j * L.msg + r, g.seq, g.timeout_ns, expired));
      if (wl[j].y != g.seq) wl[j].x = __float_as_uint(wait_pair(recv + j * L.msg + g.rows + r, g.seq, g.timeout_ns, expired));
      if (wa[j].y != g.seq) wa[j].x = __float_as_uint(wait_pair(recv + j * L.msg + ia, g.seq, g.timeout_ns, expired));
      M = fmaxf(M, __uint_as_float(wm[j].x));
    }
  }
  const float w0 = (my_m == -INFINITY) ? 0.f : ex2f(my_m - M);
  float num = w0 * my_a, den = w0 * my_l;
#pragma unroll
  for (int j = 0; j < kPeerMaxWorld; ++j) {
    if (j < g.world && j != g.rank) {
      const float mj = __uint_as_float(wm[j].x);
      const float w = (mj == -INFINITY) ? 0.f : ex2f(mj - M);
      num += w * __uint_as_float(wa[j].x);
      den += w * __uint_as_float(wl[j].x);
    }
  }
  return den > 0.f ? num / den : 0.f;
}

}  // namespace hq
