// Flag protocol of the symmetric-memory kernels: release / acquire words in every rank's flag block,
// bounded waits.  Shared by the collectives (comm_kernels.cu) and by the kernels that fuse a reduction
// over ranks with their own arithmetic (dion_fused.cu).
#pragma once

#include "kernels.h"
#include "umma.cuh"

namespace dion {

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Flag block layout (unsigned words): flags[channel * kMaxPeers + source_rank].
// `signal`: tell every peer that this rank reached `epoch` on `channel`.
__device__ __forceinline__ void signal_peers(const PeerTable& t, long long flag_off, int channel, int rank, int world,
                                             unsigned epoch, int lane) {
  if (lane < world) {
    unsigned* f = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(t.ptrs[lane]) + flag_off);
    st_release_sys(f + channel * kMaxPeers + rank, epoch);
  }
}
// `wait`: until every source rank reached `epoch` on `channel` in this rank's flag block.
// Returns false on timeout.  Epochs only grow, so ">= epoch" also accepts a later one.
__device__ __forceinline__ bool wait_peers(const PeerTable& t, long long flag_off, int channel, int rank, int world,
                                           unsigned epoch, int lane, unsigned long long budget_ns = kWaitBudgetNs) {
  bool ok = true;
  if (lane < world) {
    const unsigned* f = reinterpret_cast<const unsigned*>(reinterpret_cast<const char*>(t.ptrs[rank]) + flag_off) +
                        channel * kMaxPeers + lane;
    const unsigned long long t0 = global_timer_ns();
    while ((int)(ld_acquire_sys(f) - epoch) < 0) {
      if (global_timer_ns() - t0 > budget_ns) {
        ok = false;
        break;
      }
    }
  }
  return ok;
}
// one source rank only; every lane of the calling warp polls the same word
__device__ __forceinline__ bool wait_peer(const PeerTable& t, long long flag_off, int channel, int rank, int src,
                                          unsigned epoch, unsigned long long budget_ns) {
  const unsigned* f = reinterpret_cast<const unsigned*>(reinterpret_cast<const char*>(t.ptrs[rank]) + flag_off) +
                      channel * kMaxPeers + src;
  const unsigned long long t0 = global_timer_ns();
  while ((int)(ld_acquire_sys(f) - epoch) < 0) {
    if (global_timer_ns() - t0 > budget_ns) return false;
  }
  return true;
}

}  // namespace dion
