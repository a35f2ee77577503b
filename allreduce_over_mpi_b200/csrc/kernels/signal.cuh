// Cross-GPU rendezvous primitives for kernels that read each other's memory.
//
// Every rank owns an array of 64-bit flags in peer-visible memory, one per
// (lane, source rank); a lane is one CTA, and CTA number c of every rank works on the
// same sub-slice of every block, so a rendezvous only ever involves CTA c of each rank.
// A rendezvous number is `call * kCallStride + index`, where `call` counts the collective
// calls of the communicator (kept on the device, so a captured CUDA graph replays
// correctly).  Numbers only grow and waits compare ">=", so a flag is never reset and a
// lane that sat out many calls cannot be confused by a stale value.
//
// Signal = release store at system scope into the peer's flag; wait = acquire load of my
// own flag.  Data written before the signal (by any thread of the CTA: the signalling
// thread runs after a CTA barrier) is visible to the peer's reads after its wait.
//
// Every wait is bounded by wall time (%globaltimer).  On expiry the lane records
// {FT_ERR_TIMEOUT, rendezvous index, peer} in the status block, raises the CTA-wide
// abort flag and the kernel runs to its end without touching peer memory again.  This
// replaces the reference's MPI_Waitall + MPI_Barrier per stage
// (allreduce_over_mpi/mpi_mod.hpp:1576, :1594-1595, :1642-1643), which block forever
// when a peer dies.
#pragma once
#include <stdint.h>

#include "../api/ft_types.h"
#include "comm_dev.h"

namespace ftk {

__device__ __forceinline__ void st_release_sys(flag_t* p, flag_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ flag_t ld_acquire_sys(const flag_t* p) {
  flag_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Spin until *flag >= value or `timeout_ns` passes.  Returns false on expiry.
__device__ __forceinline__ bool wait_flag(const flag_t* flag, flag_t value, unsigned long long timeout_ns) {
  if (ld_acquire_sys(flag) >= value) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (ld_acquire_sys(flag) >= value) return true;
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

__device__ __forceinline__ void report(Status* st, int code, int index, int peer, int lane) {
  if (st && atomicCAS_system(&st->code, FT_OK, code) == FT_OK) {
    st->index = index;
    st->peer = peer;
    st->lane = lane;
    __threadfence_system();
  }
}

struct LaneSync {
  flag_t* const* peer_flags;    // peer_flags[r] = rank r's flag array as mapped here
  flag_t* my_flags;             // == peer_flags[rank]
  int rank, world, lane, max_ranks;
  unsigned long long timeout_ns;
  Status* status;
  int* abort;                   // shared-memory flag of this CTA
};

// Rendezvous of this lane with the ranks in `mask`.  All threads of the CTA must call it.
// Thread t < world handles peer t.  Returns with *abort set if a wait ran out.
__device__ __forceinline__ void lane_rendezvous(const LaneSync& s, unsigned long long mask, flag_t value, int index) {
  __syncthreads();  // everything this CTA wrote so far happens-before the signals below
  const int t = threadIdx.x;
  if (!*s.abort && t < s.world && t != s.rank && ((mask >> t) & 1ull)) {
    st_release_sys(s.peer_flags[t] + (size_t)s.lane * s.max_ranks + s.rank, value);
    if (!wait_flag(s.my_flags + (size_t)s.lane * s.max_ranks + t, value, s.timeout_ns)) {
      report(s.status, FT_ERR_TIMEOUT, index, t, s.lane);
      *s.abort = 1;
    }
  }
  __syncthreads();
}

}  // namespace ftk
