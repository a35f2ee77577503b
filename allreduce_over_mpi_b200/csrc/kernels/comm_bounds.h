// Range check of the collective kernels' addresses, for the debugging build (-DFT_BOUNDS).
//
// Every address a collective kernel forms is "base of rank r's symmetric heap + byte offset", for a
// run of `len` bytes.  In a build with FT_BOUNDS defined each such run is tested against the size of
// the heap before the first access: a run that leaves the heap is NOT touched; the lane records
// {FT_ERR_BOUNDS, where, rank, lane} in the communicator's status block (first failure wins) and
// skips that piece of work, so the kernel still ends normally and the host reads the report with
// ft_comm_status.  Nothing traps and no out-of-range address is ever dereferenced.  Without
// FT_BOUNDS the macro expands to nothing and the kernels are unchanged.
//
// The predicate itself is plain C++ usable on the host, where its failing branch is unit-tested
// (ft_bounds_check_host in comm.cpp); on the GPU the checked build is only ever run on correct plans.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FT_BOUNDS_HD __host__ __device__ __forceinline__
#else
#define FT_BOUNDS_HD inline
#endif

namespace ftk {

// Is [off, off + len) inside rank `rank`'s heap of `heap_bytes` bytes, in a world of `world` ranks?
FT_BOUNDS_HD bool range_in_heap(uint64_t heap_bytes, int rank, int world, uint64_t off, uint64_t len) {
  return rank >= 0 && rank < world && off <= heap_bytes && len <= heap_bytes - off;
}

}  // namespace ftk

#ifdef FT_BOUNDS
// `where`: a small integer naming the site (stage index, or 100+ for the one-pass kernels); `on_fail`: the
// statement that skips the work (continue / return / a flag), uniform across the CTA like the test itself.
#define FT_CHECK_RANGE(c, rank_, off_, len_, where_, lane_, on_fail)                                      \
  if (!ftk::range_in_heap((c).heap_bytes, (rank_), (c).world, (uint64_t)(off_), (uint64_t)(len_))) {      \
    if (threadIdx.x == 0) ftk::report((c).status, FT_ERR_BOUNDS, (where_), (rank_), (lane_));             \
    on_fail;                                                                                              \
  }
#else
#define FT_CHECK_RANGE(c, rank_, off_, len_, where_, lane_, on_fail)
#endif
