// Multi-GPU collective kernels over NVLink peer memory (sm_100a).
//
//  * staged_allreduce_kernel   executes a FlexTree plan (flat, multi-level tree, lonely
//    layouts, ring): per stage, rendezvous with the stage's peers, then for every pull
//    load the block from the listed peers' symmetric heaps with 16-byte loads over
//    NVSwitch, add them to the own copy in fp32 registers, store once.  Transfer and
//    reduction are one pass; there is no staging buffer and no library call.  This is
//    the device form of the reference's per-stage Isend/Irecv/Waitall + handle_reduce +
//    Barrier loop (allreduce_over_mpi/mpi_mod.hpp:1550-1596, :1620-1644).
//  * oneshot_allreduce_kernel  every rank publishes its input in a staging slot, one
//    rendezvous, every rank sums all N copies itself (latency-optimal for small sizes).
//  * nvls_kernel               multimem.ld_reduce / multimem.st through the NVSwitch
//    multicast mapping (in-switch reduction), where the box exposes it: all-reduce, and
//    its two halves (reduce-scatter, all-gather) as passes of their own.
//  * nvls_oneshot_kernel       publish, one rendezvous, every rank reduces the whole message inside the
//    switch (tens of KB to a few MB).
//  * hybrid_allreduce_kernel   both at once on disjoint parts of the message.
//  * push_allreduce_kernel     flat two-shot in one pass: pull + sum + posted writes to every rank.
//  * ll_allreduce_kernel       push protocol with the flag inside every 8-byte word, no
//    rendezvous at all (smallest messages).
//  * ll_tree_allreduce_kernel  any plan (tree, lonely, ring) with that protocol: one one-way NVLink
//    trip per stage instead of a rendezvous.
//
// Work split: CTA c ("lane" c) of every rank owns the same byte sub-range of every
// block, so all dependencies between ranks are lane-local and a rendezvous never needs
// a grid-wide barrier.  Remote data is read with plain per-thread loads; no TMA or
// multicast load ever targets another GPU's memory.
#include <cstdio>

#include "comm_dev.h"
#include "signal.cuh"
#include "comm_bounds.h"
#include "vec.cuh"

extern "C" void ft_count_launch(uint64_t n);

namespace ftk {

constexpr int kThreads = 512;
constexpr int kUnroll = 4;

// Read the communicator's call number; the last CTA to read it bumps it for the next
// kernel on the stream.  Returns the number of THIS call to every thread.
__device__ __forceinline__ unsigned long long begin_call(const CommDev& c, unsigned long long* smem_slot) {
  if (threadIdx.x == 0) {
    const unsigned long long call = *(volatile unsigned long long*)c.call_count;
    *smem_slot = call;
    __threadfence();
    if (atomicAdd(c.arrived, 1u) == gridDim.x - 1) {
      *(volatile unsigned int*)c.arrived = 0;
      *(volatile unsigned long long*)c.call_count = call + 1;
      if (c.status) c.status->calls = (unsigned int)(call + 1);
    }
  }
  __syncthreads();
  return *smem_slot;
}

// dst[i] = fin( init(p0[i]) + p1[i] + ... ) for 16-byte vectors i in [0, nvec_total) where
// the last vector may be partial (`total_bytes` not a multiple of 16).  ptrs[] live in
// shared memory.  dst_user (optional) receives the same result; it may be unaligned.
template <class P>
__device__ __forceinline__ void pull_range(const unsigned char* const* ptrs, int n, unsigned char* dst_work,
                                           unsigned char* dst_user, bool user_vec_ok, uint64_t total_bytes,
                                           uint32_t es, bool do_scale, float scale,
                                           unsigned char* const* push_dsts = nullptr, int n_push = 0) {
  const uint64_t nvec = (total_bytes + 15) / 16;
  const uint64_t step = (uint64_t)blockDim.x * kUnroll;
  const unsigned char* s0 = ptrs[0];
  const unsigned char* s1 = n > 1 ? ptrs[1] : nullptr;
  // The first two sources of the NEXT step are requested before this step's results are
  // stored, so loads stay in flight across steps (for fan-in 2 that is all of them).
  uint4 f0[kUnroll], f1[kUnroll];
  auto issue_first = [&](uint64_t base) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * blockDim.x + threadIdx.x;
      f0[u] = i < nvec ? ld_stream(s0 + i * 16) : make_uint4(0, 0, 0, 0);
    }
    if (s1) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * blockDim.x + threadIdx.x;
        f1[u] = i < nvec ? ld_stream(s1 + i * 16) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  issue_first(0);
  for (uint64_t base = 0; base < nvec; base += step) {
    uint64_t idx[kUnroll];
    bool ok[kUnroll];
    typename P::Acc acc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      idx[u] = base + (uint64_t)u * blockDim.x + threadIdx.x;
      ok[u] = idx[u] < nvec;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) P::init(acc[u], f0[u]);
    if (s1) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) P::add(acc[u], f1[u]);
    }
    int k = 2;
    for (; k + 2 <= n; k += 2) {
      uint4 v[2][kUnroll];
      const unsigned char* pa = ptrs[k];
      const unsigned char* pb = ptrs[k + 1];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[0][u] = ok[u] ? ld_stream(pa + idx[u] * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[1][u] = ok[u] ? ld_stream(pb + idx[u] * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) { P::add(acc[u], v[0][u]); P::add(acc[u], v[1][u]); }
    }
    if (k < n) {
      uint4 v[kUnroll];
      const unsigned char* pa = ptrs[k];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[u] = ok[u] ? ld_stream(pa + idx[u] * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) P::add(acc[u], v[u]);
    }
    if (base + step < nvec) issue_first(base + step);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (!ok[u]) continue;
      const uint4 out = do_scale ? P::fins(acc[u], scale) : P::fin(acc[u]);
      const uint64_t off = idx[u] * 16;
      const uint32_t valid = (uint32_t)(total_bytes - off < 16 ? total_bytes - off : 16);
      if (dst_work) {
        if (valid == 16) st_vec(dst_work + off, out);
        else st_partial(dst_work + off, out, valid, es);
      }
      if (dst_user) {
        if (valid == 16 && user_vec_ok) st_vec(dst_user + off, out);
        else st_partial(dst_user + off, out, valid, es);
      }
      for (int q = 0; q < n_push; ++q) {   // posted writes of the result into other ranks' buffers
        if (valid == 16) st_vec(push_dsts[q] + off, out);
        else st_partial(push_dsts[q] + off, out, valid, es);
      }
    }
  }
}

// Plain lane-sliced copy src -> dst (src may be unaligned user memory).
__device__ __forceinline__ void copy_range(const unsigned char* src, bool src_vec_ok, unsigned char* dst, bool dst_vec_ok,
                                           uint64_t total_bytes, uint32_t es) {
  const uint64_t nvec = (total_bytes + 15) / 16;
  for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint64_t off = i * 16;
    const uint32_t valid = (uint32_t)(total_bytes - off < 16 ? total_bytes - off : 16);
    const uint4 v = (valid == 16 && src_vec_ok) ? ld_stream(src + off) : ld_partial(src + off, valid, es);
    if (valid == 16 && dst_vec_ok) st_vec(dst + off, v);
    else st_partial(dst + off, v, valid, es);
  }
}

// One gather step of a stage: `ng` independent copies (one per source rank), all in flight
// together so that a small message pays one NVLink round trip for the whole stage and a
// large one pulls from every peer's link at once instead of queueing on one peer.
struct CopyJob { const unsigned char* src; unsigned char* dst_work; unsigned char* dst_user; uint64_t bytes; };
constexpr int kMaxGroup = FT_MAX_FANIN;

__device__ __forceinline__ void store_job(const CopyJob& jb, uint64_t off, uint4 v, bool user_vec_ok, uint32_t es) {
  const uint32_t valid = (uint32_t)(jb.bytes - off < 16 ? jb.bytes - off : 16);
  if (jb.dst_work) {
    if (valid == 16) st_vec(jb.dst_work + off, v);
    else st_partial(jb.dst_work + off, v, valid, es);
  }
  if (jb.dst_user) {
    if (valid == 16 && user_vec_ok) st_vec(jb.dst_user + off, v);
    else st_partial(jb.dst_user + off, v, valid, es);
  }
}

// JOBS jobs x VPT vectors per thread per step = 4 loads per step; the loads of the next step are
// issued before the stores of the current one (up to 8 in flight), so the wire never idles
// between steps.  `first` is the index of the first job of this batch.
template <int JOBS, int VPT>
__device__ __forceinline__ void copy_batch(const CopyJob* jobs, int first, int ng, uint64_t max_bytes, bool user_vec_ok, uint32_t es) {
  const uint64_t max_nvec = (max_bytes + 15) / 16;
  const uint64_t step = (uint64_t)blockDim.x * VPT;
  uint4 cur[JOBS][VPT], nxt[JOBS][VPT];
  auto issue = [&](uint64_t base, uint4 (&buf)[JOBS][VPT]) {
#pragma unroll
    for (int j = 0; j < JOBS; ++j)
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const uint64_t off = (base + (uint64_t)u * blockDim.x + threadIdx.x) * 16;
        const bool ok = first + j < ng && off < jobs[first + j < ng ? first + j : first].bytes;
        buf[j][u] = ok ? ld_stream(jobs[first + j].src + off) : make_uint4(0, 0, 0, 0);
      }
  };
  issue(0, cur);
  for (uint64_t base = 0; base < max_nvec; base += step) {
    if (base + step < max_nvec) issue(base + step, nxt);
#pragma unroll
    for (int j = 0; j < JOBS; ++j)
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const uint64_t off = (base + (uint64_t)u * blockDim.x + threadIdx.x) * 16;
        if (first + j < ng && off < jobs[first + j].bytes) store_job(jobs[first + j], off, cur[j][u], user_vec_ok, es);
      }
#pragma unroll
    for (int j = 0; j < JOBS; ++j)
#pragma unroll
      for (int u = 0; u < VPT; ++u) cur[j][u] = nxt[j][u];
  }
}

__device__ __forceinline__ void copy_group(const CopyJob* jobs, int ng, uint64_t max_bytes, bool user_vec_ok, uint32_t es) {
  if (ng == 1) { copy_batch<1, 4>(jobs, 0, ng, max_bytes, user_vec_ok, es); return; }
  if (ng == 2) { copy_batch<2, 2>(jobs, 0, ng, max_bytes, user_vec_ok, es); return; }
  if (ng <= 4) { copy_batch<4, 1>(jobs, 0, ng, max_bytes, user_vec_ok, es); return; }
  // many sources (flat plans): one pass with a load from every source in flight per thread
  const uint64_t max_nvec = (max_bytes + 15) / 16;
  constexpr int kWide = 8;
  for (uint64_t base = 0; base < max_nvec; base += blockDim.x) {
    const uint64_t off = (base + threadIdx.x) * 16;
    for (int j0 = 0; j0 < ng; j0 += kWide) {
      uint4 v[kWide];
      bool ok[kWide];
#pragma unroll
      for (int u = 0; u < kWide; ++u) {
        ok[u] = j0 + u < ng && off < jobs[j0 + u < ng ? j0 + u : 0].bytes;
        v[u] = ok[u] ? ld_stream(jobs[j0 + u].src + off) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kWide; ++u)
        if (ok[u]) store_job(jobs[j0 + u], off, v[u], user_vec_ok, es);
    }
  }
}

// Bytes of a region each lane takes.  Slices of large regions start on 1 KiB boundaries: a warp's 512-byte
// request (32 x 16 bytes) then never straddles one more 128-byte line than it has to - measured on 8 GPUs, NVLS
// all-reduce of 256 MiB: 806 GB/s with 32 or 64 lanes (slices of 2^k bytes), 707 GB/s with 48 (slices that start
// at odd multiples of 16 bytes).
__device__ __forceinline__ uint64_t lane_chunk(uint64_t region_bytes, int nlanes) {
  const uint64_t chunk = (region_bytes + nlanes - 1) / nlanes;
  const uint64_t a = chunk >= 4096 ? 1024 : 16;
  return (chunk + a - 1) & ~(a - 1);
}

struct LaneSlice { uint64_t off, bytes; };
// Sub-range of a region of `region_bytes` owned by `lane` of `nlanes` when every lane
// takes a 16-byte-aligned chunk of `chunk` bytes.
__device__ __forceinline__ LaneSlice lane_slice(uint64_t region_bytes, uint64_t chunk, int lane) {
  LaneSlice s;
  s.off = (uint64_t)lane * chunk;
  s.bytes = s.off >= region_bytes ? 0 : (region_bytes - s.off < chunk ? region_bytes - s.off : chunk);
  return s;
}

// ------------------------------------------------------------------------------- staged
template <int POL>
__global__ void __launch_bounds__(kThreads, 1) staged_allreduce_kernel(const __grid_constant__ CommDev c, const __grid_constant__ StagedArgs a) {
  using P = typename PolById<POL>::type;
  __shared__ const unsigned char* ptrs[2][FT_MAX_FANIN];
  __shared__ CopyJob jobs[kMaxGroup];
  __shared__ int abort_flag;
  __shared__ unsigned long long call_slot;
  const int lane = blockIdx.x, nlanes = gridDim.x;
  if (threadIdx.x == 0) abort_flag = 0;
  unsigned long long call = 0;
  if (a.do_sync) call = begin_call(c, &call_slot);
  else __syncthreads();

  LaneSync sync{c.flags, c.flags[c.rank], c.rank, c.world, lane, FT_MAX_RANKS, c.timeout_ns, c.status, &abort_flag};
  const uint32_t es = a.elem_size;
  const uint64_t block_bytes = a.block_elems * es;               // multiple of 16
  const uint64_t total_bytes = a.count * es;
  const uint64_t chunk = lane_chunk(block_bytes, nlanes);
  // staging mode alternates between two work buffers with the call parity, so that a rank
  // may refill one while a slow peer still gathers from the other
  const uint64_t work_off = a.work_off + (call & 1) * a.alt_stride;
  unsigned char* my_work = c.heap[c.rank] + work_off;

  auto block_len = [&](int b) -> uint64_t {   // bytes of block b that hold data
    const uint64_t lo = (uint64_t)b * block_bytes;
    return lo >= total_bytes ? 0 : (total_bytes - lo < block_bytes ? total_bytes - lo : block_bytes);
  };

  // stage the caller's input into the symmetric work buffer, lane-sliced like everything else
  if (a.user_in && a.stage_begin == 0) {
    for (int b = 0; b < c.world; ++b) {
      const LaneSlice s = lane_slice(block_len(b), chunk, lane);
      if (s.bytes) {
        const uint64_t off = (uint64_t)b * block_bytes + s.off;
        FT_CHECK_RANGE(c, c.rank, work_off + off, s.bytes, 200, lane, continue)
        copy_range((const unsigned char*)a.user_in + off, a.user_vec_ok, my_work + off, true, s.bytes, es);
      }
    }
  }

  int pp = 0;
  for (uint32_t s = a.stage_begin; s < a.stage_end; ++s) {
    const DevStage st = a.plan->stages[s];
    if (a.do_sync) {
      lane_rendezvous(sync, st.sync_mask, call * kCallStride + s + 1, (int)s);
      if (abort_flag) break;
    }
    // the very last stage's gathers are read by nobody: skip the work-buffer copy when the
    // caller takes the result elsewhere
    const bool need_work = !(a.user_out && s + 1 == a.plan->nstages);
    uint32_t q = st.pull_begin;
    while (q < st.pull_end) {
      const DevPull pl = a.pulls[q];
      if (pl.reduce) {
        ++q;
        const LaneSlice sl = lane_slice(block_len(pl.block), chunk, lane);
        if (!sl.bytes) continue;   // uniform across the CTA
        const uint64_t off = (uint64_t)pl.block * block_bytes + sl.off;
        const int n = pl.nsrc + 1;
#ifdef FT_BOUNDS
        {
          bool inside = true;
          FT_CHECK_RANGE(c, c.rank, work_off + off, sl.bytes, (int)s, lane, inside = false)
          for (int k = 0; k < pl.nsrc; ++k) FT_CHECK_RANGE(c, (int)pl.src[k], work_off + off, sl.bytes, (int)s, lane, inside = false)
          if (!inside) continue;
        }
#endif
        if ((int)threadIdx.x < n)
          ptrs[pp][threadIdx.x] = threadIdx.x == 0 ? my_work + off : c.heap[pl.src[threadIdx.x - 1]] + work_off + off;
        __syncthreads();
        // a block is final for this rank when its last reduction happens here
        pull_range<P>(ptrs[pp], n, need_work ? my_work + off : nullptr,
                      (a.user_out && st.last_rs) ? (unsigned char*)a.user_out + off : nullptr, a.user_vec_ok, sl.bytes, es,
                      st.last_rs != 0, a.scale);
        pp ^= 1;
        continue;
      }
      // a run of gathers: collect them and move them together
      int ng = 0;
      uint64_t max_bytes = 0;
      for (; q < st.pull_end && ng < kMaxGroup; ++q) {
        const DevPull g = a.pulls[q];
        if (g.reduce) break;
        const LaneSlice sl = lane_slice(block_len(g.block), chunk, lane);
        if (!sl.bytes) continue;
        const uint64_t off = (uint64_t)g.block * block_bytes + sl.off;
        FT_CHECK_RANGE(c, (int)g.src[0], work_off + off, sl.bytes, (int)s, lane, continue)
        FT_CHECK_RANGE(c, c.rank, work_off + off, sl.bytes, (int)s, lane, continue)
        if (threadIdx.x == 0) {
          jobs[ng].src = c.heap[g.src[0]] + work_off + off;
          jobs[ng].dst_work = need_work ? my_work + off : nullptr;
          jobs[ng].dst_user = a.user_out ? (unsigned char*)a.user_out + off : nullptr;
          jobs[ng].bytes = sl.bytes;
        }
        max_bytes = sl.bytes > max_bytes ? sl.bytes : max_bytes;
        ++ng;
      }
      __syncthreads();
      if (ng) copy_group(jobs, ng, max_bytes, a.user_vec_ok, es);
      __syncthreads();
    }
  }
  // closing rendezvous: the plan's own set after the last stage; every rank (end_sync == 2) when a
  // phase runs alone, since then the caller may rewrite any part of the buffer once the call returns
  if (a.do_sync && a.end_sync && !abort_flag && (a.end_sync == 2 || a.stage_end == a.plan->nstages)) {
    const unsigned long long everyone = c.world >= 64 ? ~0ull : ((1ull << c.world) - 1);
    lane_rendezvous(sync, a.end_sync == 2 ? everyone : a.plan->end_sync_mask, call * kCallStride + a.plan->nstages + 1,
                    (int)a.plan->nstages);
  }
}

// ------------------------------------------------------------------------------- one-shot
template <int POL>
__global__ void __launch_bounds__(kThreads) oneshot_allreduce_kernel(const __grid_constant__ CommDev c, const __grid_constant__ OneShotArgs a,
                                                                      uint64_t slot_bytes) {
  using P = typename PolById<POL>::type;
  __shared__ const unsigned char* ptrs[FT_MAX_RANKS];
  __shared__ int abort_flag;
  __shared__ unsigned long long call_slot;
  const int lane = blockIdx.x, nlanes = gridDim.x;
  if (threadIdx.x == 0) abort_flag = 0;
  unsigned long long call = 0;
  if (a.phase_mask & 2) call = begin_call(c, &call_slot);
  else { call = a.emu_call; __syncthreads(); }
  const uint32_t es = a.elem_size;
  const uint64_t total_bytes = a.count * es;
  const uint64_t chunk = lane_chunk(total_bytes, nlanes);
  const LaneSlice sl = lane_slice(total_bytes, chunk, lane);
  // two staging slots alternate with the call parity: a slot is rewritten only after every
  // rank has entered the call after its last readers
  const uint64_t slot = a.slot_off + (call & 1) * slot_bytes;

#ifdef FT_BOUNDS
  if (c.heap_bytes) {   // (0: a caller-built world without a heap size, e.g. the allocation-free entry point)
    bool inside = true;
    for (int r = 0; r < c.world; ++r) FT_CHECK_RANGE(c, r, slot + sl.off, sl.bytes, 100, lane, inside = false)
    if (!inside) return;
  }
#endif
  if ((a.phase_mask & 1) && sl.bytes)
    copy_range((const unsigned char*)a.user_in + sl.off, a.user_vec_ok, c.heap[c.rank] + slot + sl.off, true, sl.bytes, es);
  if (a.phase_mask & 2) {
    LaneSync sync{c.flags, c.flags[c.rank], c.rank, c.world, lane, FT_MAX_RANKS, c.timeout_ns, c.status, &abort_flag};
    unsigned long long all = c.world >= 64 ? ~0ull : ((1ull << c.world) - 1);
    lane_rendezvous(sync, all, call * kCallStride + 1, 0);
    if (abort_flag) return;
  }
  if ((a.phase_mask & 4) && sl.bytes) {
    if ((int)threadIdx.x < c.world) ptrs[threadIdx.x] = c.heap[threadIdx.x] + slot + sl.off;   // rank order: same sum order everywhere
    __syncthreads();
    pull_range<P>(ptrs, c.world, nullptr, (unsigned char*)a.user_out + sl.off, a.user_vec_ok, sl.bytes, es, a.scale != 1.0f, a.scale);
  }
}

// ------------------------------------------------------------------------------- low-latency push
// For messages of a few KB the cost is all latency.  Here nothing waits for a rendezvous:
// every rank pushes its input straight into a receive area in every peer's heap as 8-byte
// words {32 bits of data, 32-bit tag of this call}; 8-byte stores are single-copy atomic, so
// a word whose tag matches carries valid data.  Each rank then polls its own memory, sums the
// N contributions in rank order (identical bits on every rank) and writes the result.  Two
// receive areas alternate with the call parity; a peer cannot be two calls ahead because
// finishing a call needs this rank's data of that call.
__device__ __forceinline__ void st_ll(unsigned char* p, uint32_t d0, uint32_t d1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d0), "r"(tag), "r"(d1), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_ll(const unsigned char* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <int POL>
__global__ void __launch_bounds__(kThreads) ll_allreduce_kernel(const __grid_constant__ CommDev c, const __grid_constant__ LLArgs a) {
  using P = typename PolById<POL>::type;
  __shared__ unsigned long long call_slot;
  unsigned long long call;
  if (a.use_call_counter) call = begin_call(c, &call_slot);
  else call = a.emu_call;
  const uint32_t tag = (uint32_t)(call + 1) | 0x80000000u;   // never 0, differs between consecutive calls of a parity
  const uint32_t es = a.elem_size;
  const uint64_t total_bytes = a.count * es;
  const uint64_t nitems = (total_bytes + 15) / 16;            // 16 payload bytes = 32 wire bytes per item
  const uint64_t area = a.ll_off + (call & 1) * (uint64_t)c.world * kLLSrcStride;
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nitems) return;
#ifdef FT_BOUNDS
  // every word this thread writes or polls lies at the same offset of some rank's receive area
  if (!range_in_heap(c.heap_bytes, c.rank, c.world, area + (uint64_t)(c.world - 1) * kLLSrcStride + i * 32, 32)) {
    report(c.status, FT_ERR_BOUNDS, 105, c.rank, blockIdx.x);
    return;
  }
#endif
  const uint32_t valid = (uint32_t)(total_bytes - i * 16 < 16 ? total_bytes - i * 16 : 16);
  uint4 mine = make_uint4(0, 0, 0, 0);
  if (a.phase_mask & 1) {
    const unsigned char* src = (const unsigned char*)a.user_in + i * 16;
    mine = (valid == 16 && a.user_vec_ok) ? ld_stream(src) : ld_partial(src, valid, es);
    for (int k = 1; k < c.world; ++k) {
      const int p = (c.rank + k) % c.world;
      unsigned char* dst = c.heap[p] + area + (uint64_t)c.rank * kLLSrcStride + i * 32;
      st_ll(dst, mine.x, mine.y, tag);
      st_ll(dst + 16, mine.z, mine.w, tag);
    }
    if (!(a.phase_mask & 2)) {   // emulation: park the own contribution like a peer would
      unsigned char* dst = c.heap[c.rank] + area + (uint64_t)c.rank * kLLSrcStride + i * 32;
      st_ll(dst, mine.x, mine.y, tag);
      st_ll(dst + 16, mine.z, mine.w, tag);
    }
  }
  if (!(a.phase_mask & 2)) return;
  const bool own_from_mem = !(a.phase_mask & 1);
  typename P::Acc acc;
  const unsigned long long t0 = globaltimer_ns();
  for (int q = 0; q < c.world; ++q) {
    uint4 v;
    if (q == c.rank && !own_from_mem) {
      v = mine;
    } else {
      const unsigned char* src = c.heap[c.rank] + area + (uint64_t)q * kLLSrcStride + i * 32;
      uint4 lo, hi;
      int spins = 0;
      for (;;) {
        lo = ld_ll(src);
        hi = ld_ll(src + 16);
        if (lo.y == tag && lo.w == tag && hi.y == tag && hi.w == tag) break;
        if (++spins >= 64) {
          spins = 0;
          if (globaltimer_ns() - t0 > c.timeout_ns) {
            report(c.status, FT_ERR_TIMEOUT, 0, q, blockIdx.x);
            return;
          }
        }
      }
      v = make_uint4(lo.x, lo.z, hi.x, hi.z);
    }
    if (q == 0) P::init(acc, v);
    else P::add(acc, v);
  }
  const uint4 out = a.scale != 1.0f ? P::fins(acc, a.scale) : P::fin(acc);
  unsigned char* dst = (unsigned char*)a.user_out + i * 16;
  if (valid == 16 && a.user_vec_ok) st_vec(dst, out);
  else st_partial(dst, out, valid, es);
}

// ------------------------------------------------------------------------------- any plan, tagged words
// The staged kernel pays one cross-GPU rendezvous per stage, which at a few KB is all there is to pay.
// Here a plan (tree, lonely layout, ring) runs with the tagged-word protocol of ll_allreduce_kernel instead:
// at the start of a stage a rank pushes its current copy of every block some peer will fold in or take over
// into that peer's receive slot, then folds in (or takes over) what arrives in its own slots.  Nobody waits
// for a rendezvous; a tree level costs one one-way NVLink trip.  Thread i owns 16-byte item i of EVERY block
// from the first stage to the last and keeps the running values in the caller's output buffer, so stages need
// no CTA barrier either.  Pushing before the own pulls of a stage sends the value a block had when the stage
// began, which is what the pull plan means (check_hazards: nothing a peer reads in a stage is written in it).
// Two receive areas alternate with the call parity as in ll_allreduce_kernel.
template <int POL>
__global__ void __launch_bounds__(256) ll_tree_allreduce_kernel(const __grid_constant__ CommDev c, const __grid_constant__ LLTreeArgs a) {
  using P = typename PolById<POL>::type;
  __shared__ unsigned long long call_slot;
  // The plan's tables are walked entry after entry by every thread; from global memory that is a chain of a few
  // dozen dependent loads (~0.5 us each) on the critical path of a message that takes 20 us in all.  When they fit,
  // the CTA copies them into shared memory once, all loads in flight together.
  extern __shared__ __align__(16) unsigned char ll_tree_tables[];
  const DevStage* stages = a.plan->stages;
  const DevPull* pulls = a.pulls;
  const DevPush* pushes = a.pushes;
  if (a.table_bytes) {
    const uint32_t nst = a.table_counts[0], npl = a.table_counts[1], nps = a.table_counts[2];
    DevStage* s_st = (DevStage*)ll_tree_tables;
    DevPull* s_pl = (DevPull*)(s_st + nst);
    DevPush* s_ps = (DevPush*)(s_pl + npl);
    const uint16_t* g0 = (const uint16_t*)a.plan->stages;
    const uint16_t* g1 = (const uint16_t*)a.pulls;
    const uint16_t* g2 = (const uint16_t*)a.pushes;
    for (uint32_t k = threadIdx.x; k < nst * sizeof(DevStage) / 2; k += blockDim.x) ((uint16_t*)s_st)[k] = g0[k];
    for (uint32_t k = threadIdx.x; k < npl * sizeof(DevPull) / 2; k += blockDim.x) ((uint16_t*)s_pl)[k] = g1[k];
    for (uint32_t k = threadIdx.x; k < nps * sizeof(DevPush) / 2; k += blockDim.x) ((uint16_t*)s_ps)[k] = g2[k];
    stages = s_st; pulls = s_pl; pushes = s_ps;
  }
  unsigned long long call;
  if (a.use_call_counter) call = begin_call(c, &call_slot);   // (its barrier also publishes the tables to the CTA)
  else { call = a.emu_call; __syncthreads(); }
  const uint32_t tag = (uint32_t)(call + 1) | 0x80000000u;
  const uint32_t es = a.elem_size;
  const uint64_t block_bytes = a.block_elems * es, total_bytes = a.count * es;
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i * 16 >= block_bytes) return;
  const uint64_t area = a.ll_off + (call & 1) * (uint64_t)c.world * kLLSrcStride;
  const uint64_t slot_wire = 2 * block_bytes;
  unsigned char* out = (unsigned char*)a.user_out;
  auto valid_of = [&](int b) -> uint32_t {   // bytes of my item of block b that hold data
    const uint64_t off = (uint64_t)b * block_bytes + i * 16;
    return off >= total_bytes ? 0u : (uint32_t)(total_bytes - off < 16 ? total_bytes - off : 16);
  };
  auto load_mine = [&](const unsigned char* base, int b, uint32_t valid) -> uint4 {
    const unsigned char* p = base + (uint64_t)b * block_bytes + i * 16;
    return (valid == 16 && a.user_vec_ok) ? ld_stream(p) : ld_partial(p, valid, es);
  };
  auto store_mine = [&](int b, uint32_t valid, uint4 v) {
    unsigned char* p = out + (uint64_t)b * block_bytes + i * 16;
    if (valid == 16 && a.user_vec_ok) st_vec(p, v);
    else st_partial(p, v, valid, es);
  };
  if (a.stage_begin == 0 && (a.phase_mask & 1) && a.user_in != a.user_out)
    for (int b = 0; b < c.world; ++b) {
      const uint32_t valid = valid_of(b);
      if (valid) store_mine(b, valid, load_mine((const unsigned char*)a.user_in, b, valid));
    }
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t s = a.stage_begin; s < a.stage_end; ++s) {
    const DevStage st = stages[s];
    if (a.phase_mask & 1)
      for (uint32_t q = st.push_begin; q < st.push_end; ++q) {
        const DevPush ps = pushes[q];
        const uint32_t valid = valid_of(ps.block);
        if (!valid) continue;
        const uint4 v = load_mine(out, ps.block, valid);
        unsigned char* dst = c.heap[ps.dst] + area + (uint64_t)ps.slot * slot_wire + i * 32;
        st_ll(dst, v.x, v.y, tag);
        st_ll(dst + 16, v.z, v.w, tag);
      }
    if (!(a.phase_mask & 2)) continue;
    for (uint32_t q = st.pull_begin; q < st.pull_end; ++q) {
      const DevPull pl = pulls[q];
      const uint32_t valid = valid_of(pl.block);
      if (!valid) continue;
      typename P::Acc acc;
      if (pl.reduce) P::init(acc, load_mine(out, pl.block, valid));
      for (int k = 0; k < pl.nsrc; ++k) {
        const unsigned char* src = c.heap[c.rank] + area + (uint64_t)(pl.slot + k) * slot_wire + i * 32;
        uint4 lo, hi;
        int spins = 0;
        for (;;) {
          lo = ld_ll(src);
          hi = ld_ll(src + 16);
          if (lo.y == tag && lo.w == tag && hi.y == tag && hi.w == tag) break;
          if (++spins >= 64) {
            spins = 0;
            if (globaltimer_ns() - t0 > c.timeout_ns) {
              report(c.status, FT_ERR_TIMEOUT, (int)s, pl.src[k], blockIdx.x);
              return;
            }
          }
        }
        const uint4 v = make_uint4(lo.x, lo.z, hi.x, hi.z);
        if (pl.reduce) P::add(acc, v);
        else P::init(acc, v);
      }
      store_mine(pl.block, valid, (pl.reduce && st.last_rs && a.scale != 1.0f) ? P::fins(acc, a.scale) : P::fin(acc));
    }
  }
}

// ------------------------------------------------------------------------------- NVLS
// multimem.ld_reduce sums one 16-byte vector across every GPU bound to the multicast
// object inside the switch; multimem.st writes one to all of them.  WEAK selects the
// .weak form of both (no ordering of its own; the rendezvous around the pass orders them).
template <int POL, int WEAK> struct Nvls;
#define FT_NVLS_LD(POL_ID, SUFFIX)                                                                                  \
  template <> struct Nvls<POL_ID, 0> {                                                                              \
    __device__ static __forceinline__ uint4 ld(const void* p) {                                                     \
      uint4 v;                                                                                                      \
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add" SUFFIX " {%0,%1,%2,%3}, [%4];"                       \
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");                               \
      return v;                                                                                                     \
    }                                                                                                               \
  };                                                                                                                \
  template <> struct Nvls<POL_ID, 1> {                                                                              \
    __device__ static __forceinline__ uint4 ld(const void* p) {                                                     \
      uint4 v;                                                                                                      \
      asm volatile("multimem.ld_reduce.weak.global.add" SUFFIX " {%0,%1,%2,%3}, [%4];"                              \
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");                               \
      return v;                                                                                                     \
    }                                                                                                               \
  };
FT_NVLS_LD(POL_F32, ".v4.f32")
FT_NVLS_LD(POL_BF16, ".acc::f32.v4.bf16x2")
FT_NVLS_LD(POL_F16, ".acc::f32.v4.f16x2")
#undef FT_NVLS_LD
template <int WEAK>
__device__ __forceinline__ void multimem_st(void* p, uint4 v) {
  if (WEAK) asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  else asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// What one lane does with its `nvec` 16-byte vectors at multicast address `mc` (and the same
// range of this rank's own heap at `own`):
//   MODE 0  all-reduce: reduce inside the switch, broadcast the result to every rank;
//   MODE 1  reduce-scatter: reduce inside the switch, keep the result in the own buffer only;
//   MODE 2  all-gather: broadcast the own buffer's contents to every rank.
// KU vectors are in flight per thread: KU reductions (or loads), then their KU stores.
template <int POL, int MODE, int KU, int WEAK>
__device__ __forceinline__ void nvls_pass(unsigned char* mc, unsigned char* own, uint64_t nvec, float scale) {
  using P = typename PolById<POL>::type;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)blockDim.x * KU) {
    uint4 v[KU];
    uint64_t idx[KU];
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      idx[u] = base + (uint64_t)u * blockDim.x + threadIdx.x;
      if (idx[u] < nvec) v[u] = MODE == 2 ? ld_stream(own + idx[u] * 16) : Nvls<POL, WEAK>::ld(mc + idx[u] * 16);
      else v[u] = make_uint4(0, 0, 0, 0);
    }
    if (MODE != 2 && scale != 1.0f) {
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        typename P::Acc t;
        P::init(t, v[u]);
        v[u] = P::fins(t, scale);
      }
    }
#pragma unroll
    for (int u = 0; u < KU; ++u)
      if (idx[u] < nvec) {
        if (MODE == 1) st_vec(own + idx[u] * 16, v[u]);
        else multimem_st<WEAK>(mc + idx[u] * 16, v[u]);
      }
  }
}

// In place on the symmetric work buffer.  Rank r handles the parts of the message it owns, lane-sliced:
// with stripe_bytes == 0 that is block r (one contiguous 1/N of the message, the blocks of the plans);
// otherwise the message is cut into stripes of stripe_bytes dealt round-robin to the ranks, so that at
// any moment the N ranks work on neighbouring addresses.  Requires count*es to be a multiple of 16.
// Rendezvous before the pass (every rank's input is in place / nobody still reads what gets overwritten)
// and after it (every rank's stores have landed everywhere).
template <int POL, int MODE, int KU, int WEAK>
__global__ void __launch_bounds__(1024) nvls_kernel(const __grid_constant__ CommDev c, const __grid_constant__ NvlsArgs a) {
  __shared__ int abort_flag;
  __shared__ unsigned long long call_slot;
  const int lane = blockIdx.x, nlanes = gridDim.x;
  if (threadIdx.x == 0) abort_flag = 0;
  const unsigned long long call = begin_call(c, &call_slot);
  LaneSync sync{c.flags, c.flags[c.rank], c.rank, c.world, lane, FT_MAX_RANKS, c.timeout_ns, c.status, &abort_flag};
  const unsigned long long all = c.world >= 64 ? ~0ull : ((1ull << c.world) - 1);
  const uint32_t es = a.elem_size;
  const uint64_t total_bytes = a.count * es;

  lane_rendezvous(sync, all, call * kCallStride + 1, 0);
  if (abort_flag) return;
  if (a.stripe_bytes == 0) {
    const uint64_t block_bytes = a.block_elems * es;
    const uint64_t chunk = lane_chunk(block_bytes, nlanes);
    const uint64_t lo = (uint64_t)c.rank * block_bytes;
    const uint64_t len = lo >= total_bytes ? 0 : (total_bytes - lo < block_bytes ? total_bytes - lo : block_bytes);
    const LaneSlice sl = lane_slice(len, chunk, lane);
    const uint64_t off = a.work_off + lo + sl.off;
    bool inside = true;
    FT_CHECK_RANGE(c, c.rank, off, sl.bytes, 110, lane, inside = false)
    if (inside) nvls_pass<POL, MODE, KU, WEAK>(c.mc_heap + off, c.heap[c.rank] + off, sl.bytes / 16, a.scale);
  } else {
    // stripe s belongs to rank s % world; lanes deal this rank's stripes round-robin among themselves
    const uint64_t nstripes = (total_bytes + a.stripe_bytes - 1) / a.stripe_bytes;
    for (uint64_t s = (uint64_t)c.rank + (uint64_t)lane * c.world; s < nstripes; s += (uint64_t)nlanes * c.world) {
      const uint64_t lo = s * a.stripe_bytes;
      const uint64_t len = total_bytes - lo < a.stripe_bytes ? total_bytes - lo : a.stripe_bytes;
      FT_CHECK_RANGE(c, c.rank, a.work_off + lo, len, 111, lane, continue)
      nvls_pass<POL, MODE, KU, WEAK>(c.mc_heap + a.work_off + lo, c.heap[c.rank] + a.work_off + lo, len / 16, a.scale);
    }
  }
  // all my stores are ordered before my signal; after the rendezvous every rank's part has landed here too
  __threadfence_system();
  lane_rendezvous(sync, all, call * kCallStride + 2, 1);
}

// ------------------------------------------------------------------------------- one-shot through the switch
// The one-shot all-reduce with the N peer loads per vector replaced by ONE multimem.ld_reduce: every rank
// publishes its input in its staging slot (two slots by call parity, as in oneshot_allreduce_kernel), one
// rendezvous, then every rank reduces the WHOLE message inside the switch and stores it to its own output.
// One rendezvous instead of the two of the reduce + broadcast pass, at the price of N times the switch traffic:
// the choice for messages of tens of KB to a few MB.
template <int POL>
__global__ void __launch_bounds__(kThreads) nvls_oneshot_kernel(const __grid_constant__ CommDev c, const __grid_constant__ OneShotArgs a,
                                                                uint64_t slot_bytes) {
  using P = typename PolById<POL>::type;
  __shared__ int abort_flag;
  __shared__ unsigned long long call_slot;
  const int lane = blockIdx.x, nlanes = gridDim.x;
  if (threadIdx.x == 0) abort_flag = 0;
  const unsigned long long call = begin_call(c, &call_slot);
  const uint32_t es = a.elem_size;
  const uint64_t total_bytes = a.count * es;
  const uint64_t chunk = lane_chunk(total_bytes, nlanes);
  const LaneSlice sl = lane_slice(total_bytes, chunk, lane);
  const uint64_t slot = a.slot_off + (call & 1) * slot_bytes;
  bool inside = true;
  FT_CHECK_RANGE(c, c.rank, slot + sl.off, (sl.bytes + 15) / 16 * 16, 140, lane, inside = false)
  if (sl.bytes && inside)
    copy_range((const unsigned char*)a.user_in + sl.off, a.user_vec_ok, c.heap[c.rank] + slot + sl.off, true, sl.bytes, es);
  LaneSync sync{c.flags, c.flags[c.rank], c.rank, c.world, lane, FT_MAX_RANKS, c.timeout_ns, c.status, &abort_flag};
  const unsigned long long all = c.world >= 64 ? ~0ull : ((1ull << c.world) - 1);
  lane_rendezvous(sync, all, call * kCallStride + 1, 0);
  if (abort_flag || !sl.bytes || !inside) return;
  const unsigned char* mc = c.mc_heap + slot + sl.off;
  unsigned char* out = (unsigned char*)a.user_out + sl.off;
  const uint64_t nvec = (sl.bytes + 15) / 16;   // a ragged last vector reads slot bytes past the message; only the valid ones are stored
  constexpr int KU = 4;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)blockDim.x * KU) {
    uint4 v[KU];
    uint64_t idx[KU];
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      idx[u] = base + (uint64_t)u * blockDim.x + threadIdx.x;
      v[u] = idx[u] < nvec ? Nvls<POL, 0>::ld(mc + idx[u] * 16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      if (idx[u] >= nvec) continue;
      if (a.scale != 1.0f) {
        typename P::Acc t;
        P::init(t, v[u]);
        v[u] = P::fins(t, a.scale);
      }
      const uint64_t off = idx[u] * 16;
      const uint32_t valid = (uint32_t)(sl.bytes - off < 16 ? sl.bytes - off : 16);
      if (valid == 16 && a.user_vec_ok) st_vec(out + off, v[u]);
      else st_partial(out + off, v[u], valid, es);
    }
  }
}

// ------------------------------------------------------------------------------- hybrid NVLS + peer loads
// The in-switch reduction tops out well below the bandwidth of the GPU's links, and a
// two-shot all-reduce over plain peer loads uses the same links in a different way (no
// switch arithmetic).  This kernel runs both at once on disjoint parts of every block: the
// first `nvls_bytes` of each block go through multimem.ld_reduce / multimem.st on lanes
// [0, nvls_lanes), the remainder through a flat reduce-scatter + gather over peer loads on
// the other lanes.  The two lane groups never wait for each other.
template <int POL>
__global__ void __launch_bounds__(kThreads, 1) hybrid_allreduce_kernel(const __grid_constant__ CommDev c, const __grid_constant__ NvlsArgs a,
                                                                     uint32_t nvls_lanes, uint64_t nvls_bytes) {
  using P = typename PolById<POL>::type;
  __shared__ const unsigned char* ptrs[FT_MAX_RANKS];
  __shared__ CopyJob jobs[kMaxGroup];
  __shared__ int abort_flag;
  __shared__ unsigned long long call_slot;
  const int lane = blockIdx.x;
  if (threadIdx.x == 0) abort_flag = 0;
  const unsigned long long call = begin_call(c, &call_slot);
  LaneSync sync{c.flags, c.flags[c.rank], c.rank, c.world, lane, FT_MAX_RANKS, c.timeout_ns, c.status, &abort_flag};
  const unsigned long long all = c.world >= 64 ? ~0ull : ((1ull << c.world) - 1);
  const uint32_t es = a.elem_size;
  const uint64_t block_bytes = a.block_elems * es, total_bytes = a.count * es;
  auto block_len = [&](int b) -> uint64_t {
    const uint64_t lo = (uint64_t)b * block_bytes;
    return lo >= total_bytes ? 0 : (total_bytes - lo < block_bytes ? total_bytes - lo : block_bytes);
  };
  // part of block b handled by this lane group: [part_lo, part_hi) inside the block
  const bool is_nvls = (uint32_t)lane < nvls_lanes;
  const int group_lanes = is_nvls ? (int)nvls_lanes : (int)(gridDim.x - nvls_lanes);
  const int group_lane = is_nvls ? lane : lane - (int)nvls_lanes;
  const uint64_t region = is_nvls ? nvls_bytes : block_bytes - nvls_bytes;
  const uint64_t chunk = lane_chunk(region, group_lanes);
  auto my_slice = [&](int b) -> LaneSlice {   // offsets relative to the block start
    const uint64_t len = block_len(b);
    const uint64_t lo = is_nvls ? 0 : nvls_bytes, hi = is_nvls ? (len < nvls_bytes ? len : nvls_bytes) : len;
    LaneSlice sl{0, 0};
    if (hi <= lo) return sl;
    sl = lane_slice(hi - lo, chunk, group_lane);
    sl.off += lo;
    return sl;
  };

  lane_rendezvous(sync, all, call * kCallStride + 1, 0);
  if (abort_flag) return;
  if (is_nvls) {
    const LaneSlice sl = my_slice(c.rank);
    unsigned char* mc = c.mc_heap + a.work_off + (uint64_t)c.rank * block_bytes + sl.off;
    bool inside = true;
    FT_CHECK_RANGE(c, c.rank, a.work_off + (uint64_t)c.rank * block_bytes + sl.off, sl.bytes, 120, lane, inside = false)
    if (inside) nvls_pass<POL, 0, 4, 0>(mc, nullptr, sl.bytes / 16, a.scale);
    __threadfence_system();
    lane_rendezvous(sync, all, call * kCallStride + 2, 1);
    return;
  }
  // ---- peer-load group: flat reduce-scatter of my block's part, then gather of the others'
  unsigned char* my_work = c.heap[c.rank] + a.work_off;
  {
    const LaneSlice sl = my_slice(c.rank);
    if (sl.bytes) {
      const uint64_t off = (uint64_t)c.rank * block_bytes + sl.off;
      bool inside = true;
      FT_CHECK_RANGE(c, c.rank, a.work_off + off, sl.bytes, 121, lane, inside = false)   // same offset in every rank's equal-sized heap
      if ((int)threadIdx.x < c.world) ptrs[threadIdx.x] = c.heap[(c.rank + threadIdx.x) % c.world] + a.work_off + off;
      __syncthreads();
      if (inside) pull_range<P>(ptrs, c.world, my_work + off, nullptr, true, sl.bytes, es, a.scale != 1.0f, a.scale);
    }
  }
  lane_rendezvous(sync, all, call * kCallStride + 2, 1);
  if (abort_flag) return;
  {
    int ng = 0;
    uint64_t max_bytes = 0;
    for (int k = 1; k < c.world; ++k) {
      const int src = (c.rank + k) % c.world;
      const LaneSlice sl = my_slice(src);
      if (!sl.bytes) continue;
      const uint64_t off = (uint64_t)src * block_bytes + sl.off;
      FT_CHECK_RANGE(c, src, a.work_off + off, sl.bytes, 122, lane, continue)
      if (threadIdx.x == 0) {
        jobs[ng].src = c.heap[src] + a.work_off + off;
        jobs[ng].dst_work = my_work + off;
        jobs[ng].dst_user = nullptr;
        jobs[ng].bytes = sl.bytes;
      }
      max_bytes = sl.bytes > max_bytes ? sl.bytes : max_bytes;
      if (++ng == kMaxGroup) {
        __syncthreads();
        copy_group(jobs, ng, max_bytes, true, es);
        __syncthreads();
        ng = 0; max_bytes = 0;
      }
    }
    __syncthreads();
    if (ng) copy_group(jobs, ng, max_bytes, true, es);
  }
  lane_rendezvous(sync, all, call * kCallStride + 3, 2);
}

// ------------------------------------------------------------------------------- flat, reduce + push
// Flat two-shot in ONE pass for tensors in the symmetric heap: rank r pulls block r from every
// peer, sums it, and stores the result straight into every rank's buffer (its own and the
// N-1 peers').  The gather half therefore travels as posted writes instead of read requests
// and responses, and the kernel needs two rendezvous instead of three.  Only rank r ever
// writes block r anywhere, and it reads a peer's copy of a vector before overwriting it.
template <int POL>
__global__ void __launch_bounds__(kThreads, 1) push_allreduce_kernel(const __grid_constant__ CommDev c, const __grid_constant__ NvlsArgs a,
                                                                      uint32_t do_sync) {
  using P = typename PolById<POL>::type;
  __shared__ unsigned char* bufs[FT_MAX_RANKS];   // every rank's block r, lane-sliced, rotated so that bufs[0] is mine
  __shared__ int abort_flag;
  __shared__ unsigned long long call_slot;
  const int lane = blockIdx.x, nlanes = gridDim.x;
  if (threadIdx.x == 0) abort_flag = 0;
  unsigned long long call = 0;
  if (do_sync) call = begin_call(c, &call_slot);
  else __syncthreads();
  LaneSync sync{c.flags, c.flags[c.rank], c.rank, c.world, lane, FT_MAX_RANKS, c.timeout_ns, c.status, &abort_flag};
  const unsigned long long all = c.world >= 64 ? ~0ull : ((1ull << c.world) - 1);
  const uint32_t es = a.elem_size;
  const uint64_t block_bytes = a.block_elems * es, total_bytes = a.count * es;
  const uint64_t chunk = lane_chunk(block_bytes, nlanes);
  const uint64_t lo = (uint64_t)c.rank * block_bytes;
  const uint64_t len = lo >= total_bytes ? 0 : (total_bytes - lo < block_bytes ? total_bytes - lo : block_bytes);
  const LaneSlice sl = lane_slice(len, chunk, lane);
  if ((int)threadIdx.x < c.world) bufs[threadIdx.x] = c.heap[(c.rank + threadIdx.x) % c.world] + a.work_off + lo + sl.off;
  if (do_sync) {
    lane_rendezvous(sync, all, call * kCallStride + 1, 0);
    if (abort_flag) return;
  } else {
    __syncthreads();
  }
  // sources: mine first, then the peers in rotated order; destinations: mine (dst_work) and every peer's
  bool inside = true;
  FT_CHECK_RANGE(c, c.rank, a.work_off + lo + sl.off, sl.bytes, 130, lane, inside = false)   // same offset in every rank's equal-sized heap
  if (sl.bytes && inside)
    pull_range<P>((const unsigned char* const*)bufs, c.world, bufs[0], nullptr, true, sl.bytes, es, a.scale != 1.0f, a.scale,
                  bufs + 1, c.world - 1);
  if (do_sync) {
    __threadfence_system();   // my stores into the peers' buffers are ordered before my signal
    lane_rendezvous(sync, all, call * kCallStride + 2, 1);
  }
}

// ------------------------------------------------------------------------------- bounded-wait probe
// One CTA waits on one of its own flags for a rendezvous number that nobody will signal.
// With a short limit it must come back with FT_ERR_TIMEOUT in the status block.
__global__ void wait_probe_kernel(const __grid_constant__ CommDev c, int peer, unsigned long long timeout_ns) {
  if (threadIdx.x == 0) {
    const flag_t never = ~0ull - 1;
    if (!wait_flag(c.flags[c.rank] + (size_t)(kMaxLanes - 1) * FT_MAX_RANKS + peer, never, timeout_ns))
      report(c.status, FT_ERR_TIMEOUT, 0, peer, kMaxLanes - 1);
  }
}

// ------------------------------------------------------------------------------- launchers
template <int POL> static cudaError_t launch_staged_t(const CommDev& c, const StagedArgs& a, int lanes, cudaStream_t st) {
  staged_allreduce_kernel<POL><<<lanes, kThreads, 0, st>>>(c, a);
  return cudaGetLastError();
}
template <int POL> static cudaError_t launch_oneshot_t(const CommDev& c, const OneShotArgs& a, uint64_t slot_bytes, int lanes, cudaStream_t st) {
  oneshot_allreduce_kernel<POL><<<lanes, kThreads, 0, st>>>(c, a, slot_bytes);
  return cudaGetLastError();
}

#define FT_POL_SWITCH(pol, CALL)                        \
  switch (pol) {                                        \
    case POL_ADD8: return CALL(POL_ADD8);               \
    case POL_ADD16: return CALL(POL_ADD16);             \
    case POL_ADD32: return CALL(POL_ADD32);             \
    case POL_ADD64: return CALL(POL_ADD64);             \
    case POL_OR: return CALL(POL_OR);                   \
    case POL_AND: return CALL(POL_AND);                 \
    case POL_F32: return CALL(POL_F32);                 \
    case POL_F64: return CALL(POL_F64);                 \
    case POL_BF16: return CALL(POL_BF16);               \
    case POL_F16: return CALL(POL_F16);                 \
    default: return cudaErrorInvalidValue;              \
  }

cudaError_t launch_staged(int pol, const CommDev& c, const StagedArgs& a, int lanes, cudaStream_t st) {
  ft_count_launch(1);
#define CALL(P) launch_staged_t<P>(c, a, lanes, st)
  FT_POL_SWITCH(pol, CALL)
#undef CALL
}
cudaError_t launch_oneshot(int pol, const CommDev& c, const OneShotArgs& a, uint64_t slot_bytes, int lanes, cudaStream_t st) {
  ft_count_launch(1);
#define CALL(P) launch_oneshot_t<P>(c, a, slot_bytes, lanes, st)
  FT_POL_SWITCH(pol, CALL)
#undef CALL
}
// mode: 0 all-reduce, 1 reduce-scatter, 2 all-gather.  cfg: threads per CTA (128..1024, a multiple of 32), vectors in
// flight per thread (2, 4 or 8) and the .weak form of the multimem instructions.
template <int POL, int MODE, int KU>
static cudaError_t launch_nvls_w(const CommDev& c, const NvlsArgs& a, int lanes, const NvlsConfig& cfg, cudaStream_t st) {
  if (cfg.weak) nvls_kernel<POL, MODE, KU, 1><<<lanes, cfg.threads, 0, st>>>(c, a);
  else nvls_kernel<POL, MODE, KU, 0><<<lanes, cfg.threads, 0, st>>>(c, a);
  return cudaGetLastError();
}
template <int POL, int MODE>
static cudaError_t launch_nvls_u(const CommDev& c, const NvlsArgs& a, int lanes, const NvlsConfig& cfg, cudaStream_t st) {
  switch (cfg.unroll) {
    case 2: return launch_nvls_w<POL, MODE, 2>(c, a, lanes, cfg, st);
    case 4: return launch_nvls_w<POL, MODE, 4>(c, a, lanes, cfg, st);
    case 8: return launch_nvls_w<POL, MODE, 8>(c, a, lanes, cfg, st);
    default: return cudaErrorInvalidValue;
  }
}
template <int POL>
static cudaError_t launch_nvls_m(const CommDev& c, const NvlsArgs& a, int lanes, int mode, const NvlsConfig& cfg, cudaStream_t st) {
  switch (mode) {
    case 0: return launch_nvls_u<POL, 0>(c, a, lanes, cfg, st);
    case 1: return launch_nvls_u<POL, 1>(c, a, lanes, cfg, st);
    case 2: return launch_nvls_u<POL, 2>(c, a, lanes, cfg, st);
    default: return cudaErrorInvalidValue;
  }
}
cudaError_t launch_nvls(int pol, const CommDev& c, const NvlsArgs& a, int lanes, int mode, const NvlsConfig& cfg, cudaStream_t st) {
  if (cfg.threads < 128 || cfg.threads > 1024 || cfg.threads % 32) return cudaErrorInvalidValue;
  ft_count_launch(1);
  switch (pol) {
    case POL_F32: return launch_nvls_m<POL_F32>(c, a, lanes, mode, cfg, st);
    case POL_BF16: return launch_nvls_m<POL_BF16>(c, a, lanes, mode, cfg, st);
    case POL_F16: return launch_nvls_m<POL_F16>(c, a, lanes, mode, cfg, st);
    default: return cudaErrorInvalidValue;
  }
}
template <int POL> static cudaError_t launch_ll_t(const CommDev& c, const LLArgs& a, cudaStream_t st) {
  const uint64_t nitems = (a.count * a.elem_size + 15) / 16;
  const int threads = nitems < 128 ? 128 : (nitems < 256 ? 256 : kThreads);
  ll_allreduce_kernel<POL><<<(unsigned)((nitems + threads - 1) / threads), threads, 0, st>>>(c, a);
  return cudaGetLastError();
}
cudaError_t launch_ll(int pol, const CommDev& c, const LLArgs& a, cudaStream_t st) {
  ft_count_launch(1);
#define CALL(P) launch_ll_t<P>(c, a, st)
  FT_POL_SWITCH(pol, CALL)
#undef CALL
}
cudaError_t launch_nvls_oneshot(int pol, const CommDev& c, const OneShotArgs& a, uint64_t slot_bytes, int lanes, int threads, cudaStream_t st) {
  if (threads < 128 || threads > kThreads || threads % 32) return cudaErrorInvalidValue;
  ft_count_launch(1);
  switch (pol) {
    case POL_F32: nvls_oneshot_kernel<POL_F32><<<lanes, threads, 0, st>>>(c, a, slot_bytes); break;
    case POL_BF16: nvls_oneshot_kernel<POL_BF16><<<lanes, threads, 0, st>>>(c, a, slot_bytes); break;
    case POL_F16: nvls_oneshot_kernel<POL_F16><<<lanes, threads, 0, st>>>(c, a, slot_bytes); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
template <int POL> static cudaError_t launch_ll_tree_t(const CommDev& c, const LLTreeArgs& a, cudaStream_t st) {
  const uint64_t items = (a.block_elems * a.elem_size + 15) / 16;
  const int threads = items <= 32 ? 32 : (items <= 64 ? 64 : (items <= 128 ? 128 : 256));
  ll_tree_allreduce_kernel<POL><<<(unsigned)((items + threads - 1) / threads), threads, a.table_bytes, st>>>(c, a);
  return cudaGetLastError();
}
cudaError_t launch_ll_tree(int pol, const CommDev& c, const LLTreeArgs& a, cudaStream_t st) {
  ft_count_launch(1);
#define CALL(P) launch_ll_tree_t<P>(c, a, st)
  FT_POL_SWITCH(pol, CALL)
#undef CALL
}
cudaError_t launch_hybrid(int pol, const CommDev& c, const NvlsArgs& a, int lanes, int nvls_lanes, uint64_t nvls_bytes, cudaStream_t st) {
  ft_count_launch(1);
  switch (pol) {
    case POL_F32: hybrid_allreduce_kernel<POL_F32><<<lanes, kThreads, 0, st>>>(c, a, nvls_lanes, nvls_bytes); break;
    case POL_BF16: hybrid_allreduce_kernel<POL_BF16><<<lanes, kThreads, 0, st>>>(c, a, nvls_lanes, nvls_bytes); break;
    case POL_F16: hybrid_allreduce_kernel<POL_F16><<<lanes, kThreads, 0, st>>>(c, a, nvls_lanes, nvls_bytes); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
cudaError_t launch_push(int pol, const CommDev& c, const NvlsArgs& a, int lanes, bool do_sync, cudaStream_t st) {
  ft_count_launch(1);
#define CALL(P) (push_allreduce_kernel<P><<<lanes, kThreads, 0, st>>>(c, a, do_sync ? 1u : 0u), cudaGetLastError())
  FT_POL_SWITCH(pol, CALL)
#undef CALL
}
cudaError_t launch_wait_probe(const CommDev& c, int peer, unsigned long long timeout_ns, cudaStream_t st) {
  ft_count_launch(1);
  wait_probe_kernel<<<1, 32, 0, st>>>(c, peer, timeout_ns);
  return cudaGetLastError();
}

}  // namespace ftk
