// Host executors for FlexTree plans.
//
// (1) run_plan_snapshot(): all ranks in one thread, stage by stage, every stage reading
//     the state as it was before the stage.  This is the "fake backend" for planner
//     tests and the oracle for GPU results; a plan that has a read/write race inside a
//     stage gives a wrong answer here instead of passing by luck.
// (2) CpuWorld / cpu_allreduce(): ranks are threads of one process that pull blocks
//     straight out of each other's buffers and synchronise with per-pair epoch flags,
//     i.e. the same protocol the device kernels use (flag = monotonically increasing
//     rendezvous number, release on signal, acquire on wait, every wait bounded).
//     Fault injection lives here, on the host: a rank that never signals, signals a
//     wrong epoch, or leaves early makes its peers return FT_ERR_TIMEOUT /
//     FT_ERR_PROTOCOL instead of hanging.
//
// Role in the reference: tree_allreduce / ring_allreduce (allreduce_over_mpi/
// mpi_mod.hpp:1510-1671, :1673-1719), where the transport is MPI_Isend/Irecv into a
// staging buffer followed by handle_reduce (:1316-1415) and an MPI_Barrier per stage.
#pragma once
#include <atomic>
#include <chrono>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../runtime/dev_plan.hpp"
#include "cpu_reduce.hpp"
#include "plan.hpp"

namespace ft {

// In-place execution over bufs[rank] (each `count` elements of dtype).  A stage range runs one
// phase alone: [0, num_stages/2) is the reduce-scatter, [num_stages/2, num_stages) the all-gather
// (stage_end < 0: to the end).
inline ft_status run_plan_snapshot(const Plan& p, ft_op op, ft_dtype dt, void* const* bufs, uint64_t count,
                                   uint64_t block_elems = 0, int stage_begin = 0, int stage_end = -1) {
  if (!p.ok()) return FT_ERR_INVALID_TOPO;
  if (!ft_op_supported(op, dt)) return ((int)op < 0 || op >= FT_OP_COUNT) ? FT_ERR_UNSUPPORTED_OP : FT_ERR_UNSUPPORTED_TYPE;
  const size_t es = ft_dtype_size(dt);
  Blocks g(count, p.world, block_elems);
  struct Pending { int rank; uint64_t off; std::vector<char> bytes; };
  if (stage_end < 0 || stage_end > p.num_stages) stage_end = p.num_stages;
  for (int s = stage_begin < 0 ? 0 : stage_begin; s < stage_end; ++s) {
    std::vector<Pending> pend;
    for (int r = 0; r < p.world; ++r)
      for (const Pull& pl : p.stages[r][s].pulls) {
        const uint64_t off = g.offset(pl.block), len = g.length(pl.block);
        if (!len) continue;
        Pending w{r, off, std::vector<char>(len * es)};
        if (pl.reduce) {
          const void* src[FT_MAX_FANIN];
          int n = 0;
          src[n++] = (const char*)bufs[r] + off * es;
          for (int q : pl.srcs) src[n++] = (const char*)bufs[q] + off * es;
          ft_status st = reduce_nway_cpu_dispatch(op, dt, src, w.bytes.data(), n, len, 1);
          if (st != FT_OK) return st;
        } else {
          std::memcpy(w.bytes.data(), (const char*)bufs[pl.srcs[0]] + off * es, len * es);
        }
        pend.push_back(std::move(w));
      }
    for (auto& w : pend) std::memcpy((char*)bufs[w.rank] + w.off * es, w.bytes.data(), w.bytes.size());
  }
  return FT_OK;
}

enum class Fault { None, NeverSignal, WrongEpoch, LeaveEarly };
struct FaultSpec {
  Fault kind = Fault::None;
  int rank = -1;   // which rank misbehaves
  int stage = 0;   // at (NeverSignal: from) which rendezvous index; 0 = opening
};

struct RankStatus {
  ft_status code = FT_OK;
  int stage = -1;  // rendezvous index where the wait gave up
  int peer = -1;
};

// Shared state of a thread-per-rank world.
struct CpuWorld {
  int n;
  std::unique_ptr<std::atomic<uint32_t>[]> flags;  // flags[dst * n + src]
  std::unique_ptr<std::atomic<void*>[]> bufs;      // buffer each rank exposes for the current call
  std::vector<uint32_t> epoch;                     // per-rank local rendezvous counter
  std::vector<uint64_t> calls;                     // per-rank count of collective calls (slot parity, low-latency tag)
  double timeout_s = 5.0;
  // Host twins of the device's staging slots and low-latency receive area (allocated on first use):
  // slots[rank] = two slots of kSlotBytes; ll[((dst * 2 + parity) * n + src) * kLLWords + i] = {data32, tag32}.
  static constexpr size_t kSlotBytes = 1 << 18;
  static constexpr size_t kLLWords = 2048;
  std::vector<std::vector<char>> slots;
  std::unique_ptr<std::atomic<uint64_t>[]> ll;
  std::once_flag twins_once;
  void (*mid_call_hook)(int rank) = nullptr;       // tests: called by the twins between publishing and waiting
  explicit CpuWorld(int n_) : n(n_), flags(new std::atomic<uint32_t>[(size_t)n_ * n_]), bufs(new std::atomic<void*>[n_]), epoch(n_, 0), calls(n_, 0) {
    for (int i = 0; i < n * n; ++i) flags[i].store(0);
    for (int i = 0; i < n; ++i) bufs[i].store(nullptr);
  }
  void ensure_twins() {
    std::call_once(twins_once, [this] {
      slots.assign(n, std::vector<char>(2 * kSlotBytes));
      const size_t words = (size_t)n * 2 * n * kLLWords;
      ll.reset(new std::atomic<uint64_t>[words]);
      for (size_t i = 0; i < words; ++i) ll[i].store(0, std::memory_order_relaxed);
    });
  }
};

namespace detail {
// A peer may legitimately be ahead of `value`: it can already have signalled the next
// rendezvous the two ranks share, at most `max_ahead` numbers later (the opening one of
// the next call).  Anything beyond that is a protocol violation.
inline RankStatus rendezvous(CpuWorld& w, int rank, const std::vector<int>& peers, uint32_t value, int index,
                             int max_ahead, const FaultSpec* fault) {
  RankStatus st;
  uint32_t sig = value;
  bool skip = false;
  if (fault && fault->rank == rank) {
    // a silent rank stays silent: a later signal would heal the missed one (waits are ">=")
    if (fault->kind == Fault::NeverSignal && index >= fault->stage) skip = true;
    if (fault->kind == Fault::WrongEpoch && index == fault->stage) sig = value + 1000;
  }
  if (!skip)
    for (int q : peers) w.flags[(size_t)q * w.n + rank].store(sig, std::memory_order_release);
  const auto t0 = std::chrono::steady_clock::now();
  for (int q : peers) {
    for (;;) {
      const uint32_t f = w.flags[(size_t)rank * w.n + q].load(std::memory_order_acquire);
      const int32_t ahead = (int32_t)(f - value);
      if (ahead > max_ahead) { st = {FT_ERR_PROTOCOL, index, q}; return st; }
      if (ahead >= 0) break;
      if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > w.timeout_s) {
        st = {FT_ERR_TIMEOUT, index, q};
        return st;
      }
      std::this_thread::yield();
    }
  }
  return st;
}
}  // namespace detail

// One rank's part of an all-reduce; call from n threads with the same arguments
// (sendbuf == nullptr or == recvbuf means in place).  Returns the rank's status.
// `phase` runs one half of the plan as a call of its own, the way the device entry points
// ft_reduce_scatter / ft_all_gather do: 1 = stages [0, S/2), 2 = stages [S/2, S); each stage keeps
// its rendezvous number inside the call, and the call closes with a rendezvous of ALL ranks (the
// caller may rewrite any part of its buffer afterwards).
inline RankStatus cpu_allreduce(CpuWorld& w, int rank, const Plan& p, ft_op op, ft_dtype dt, const void* sendbuf,
                                void* recvbuf, uint64_t count, uint64_t block_elems = 0,
                                const FaultSpec* fault = nullptr, int threads = 1, int phase = 0) {
  RankStatus st;
  if (!p.ok() || p.world != w.n) { st.code = FT_ERR_INVALID_TOPO; return st; }
  if (!ft_op_supported(op, dt)) {
    st.code = ((int)op < 0 || op >= FT_OP_COUNT) ? FT_ERR_UNSUPPORTED_OP : FT_ERR_UNSUPPORTED_TYPE;
    return st;
  }
  const size_t es = ft_dtype_size(dt);
  if (sendbuf && sendbuf != recvbuf) std::memcpy(recvbuf, sendbuf, count * es);
  if (w.n == 1) return st;
  Blocks g(count, p.world, block_elems);
  const uint32_t base = w.epoch[rank];
  w.epoch[rank] = base + (uint32_t)p.num_stages + 1;
  ++w.calls[rank];
  w.bufs[rank].store(recvbuf, std::memory_order_release);
  const int first = phase == 2 ? p.num_stages / 2 : 0;
  const int last = phase == 1 ? p.num_stages / 2 : p.num_stages;   // one past the last stage that runs
  std::vector<int> everyone;
  if (phase)
    for (int q = 0; q < w.n; ++q)
      if (q != rank) everyone.push_back(q);
  for (int s = first; s <= last; ++s) {
    const bool closing = s == last;
    const int index = closing ? p.num_stages : s;
    if (fault && fault->rank == rank && fault->kind == Fault::LeaveEarly && fault->stage == index) return st;
    st = detail::rendezvous(w, rank, closing && phase ? everyone : p.sync[index][rank], base + (uint32_t)index + 1, index,
                            p.num_stages + 1, fault);
    if (st.code != FT_OK) return st;
    if (closing) break;
    if (w.mid_call_hook) w.mid_call_hook(rank);
    for (const Pull& pl : p.stages[rank][s].pulls) {
      const uint64_t off = g.offset(pl.block), len = g.length(pl.block);
      if (!len) continue;
      char* mine = (char*)recvbuf + off * es;
      if (pl.reduce) {
        const void* src[FT_MAX_FANIN];
        int n = 0;
        src[n++] = mine;
        for (int q : pl.srcs) src[n++] = (const char*)w.bufs[q].load(std::memory_order_acquire) + off * es;
        st.code = reduce_nway_cpu_dispatch(op, dt, src, mine, n, len, threads);
        if (st.code != FT_OK) return st;
      } else {
        std::memcpy(mine, (const char*)w.bufs[pl.srcs[0]].load(std::memory_order_acquire) + off * es, len * es);
      }
    }
  }
  return st;
}

// Staged plan through the staging slots: the device's path for tensors that do not live in the symmetric
// heap (staged_allreduce_kernel with user_in / user_out).  The input is copied into work slot (call mod 2),
// the stages run on the ranks' work slots, every finished block is written to recvbuf, the last stage
// skips the work slot, and there is NO closing rendezvous.
inline RankStatus cpu_allreduce_slots(CpuWorld& w, int rank, const Plan& p, ft_op op, ft_dtype dt, const void* sendbuf,
                                      void* recvbuf, uint64_t count) {
  RankStatus st;
  if (!p.ok() || p.world != w.n) { st.code = FT_ERR_INVALID_TOPO; return st; }
  if (!ft_op_supported(op, dt)) { st.code = FT_ERR_UNSUPPORTED_TYPE; return st; }
  const size_t es = ft_dtype_size(dt), bytes = count * es;
  if (bytes > CpuWorld::kSlotBytes) { st.code = FT_ERR_TOO_LARGE; return st; }
  const void* input = sendbuf ? sendbuf : recvbuf;
  if (w.n == 1 || count == 0) {
    if (input != recvbuf) std::memcpy(recvbuf, input, bytes);
    return st;
  }
  w.ensure_twins();
  Blocks g(count, p.world);
  const uint64_t call = w.calls[rank]++;
  const uint32_t base = w.epoch[rank];
  w.epoch[rank] = base + (uint32_t)p.num_stages + 1;
  auto work = [&](int q) { return w.slots[q].data() + (call & 1) * CpuWorld::kSlotBytes; };
  std::memcpy(work(rank), input, bytes);
  const int last_rs = p.num_stages / 2 - 1;
  for (int s = 0; s < p.num_stages; ++s) {
    st = detail::rendezvous(w, rank, p.sync[s][rank], base + (uint32_t)s + 1, s, 1 << 20, nullptr);
    if (st.code != FT_OK) return st;
    if (w.mid_call_hook) w.mid_call_hook(rank);
    const bool need_work = s + 1 != p.num_stages;
    for (const Pull& pl : p.stages[rank][s].pulls) {
      const uint64_t off = g.offset(pl.block), len = g.length(pl.block);
      if (!len) continue;
      char* mine = work(rank) + off * es;
      char* user = (char*)recvbuf + off * es;
      if (pl.reduce) {
        const void* src[FT_MAX_FANIN];
        int n = 0;
        src[n++] = mine;
        for (int q : pl.srcs) src[n++] = work(q) + off * es;
        char* dst = s == last_rs ? user : mine;     // a block's last reduction lands in the caller's tensor
        st.code = reduce_nway_cpu_dispatch(op, dt, src, dst, n, len, 1);
        if (st.code != FT_OK) return st;
        if (s == last_rs && need_work) std::memcpy(mine, user, len * es);
      } else {
        const char* from = work(pl.srcs[0]) + off * es;
        if (need_work) std::memcpy(mine, from, len * es);
        std::memcpy(user, from, len * es);
      }
    }
  }
  return st;
}

// ---- host twins of the two small-message protocols -------------------------------------------
// They exist to check the protocols' reuse rules under real concurrency (thread sanitizer, jittered
// ranks): neither closes with a rendezvous, so a slot or receive area is safe to rewrite only because
// of what finishing the call in between implies about the peers.

// One-shot: publish the input in staging slot (call mod 2), one rendezvous of all ranks, every rank sums
// all slots in rank order.  Device form: oneshot_allreduce_kernel.
inline RankStatus cpu_allreduce_oneshot(CpuWorld& w, int rank, ft_op op, ft_dtype dt, const void* sendbuf, void* recvbuf,
                                        uint64_t count) {
  RankStatus st;
  if (!ft_op_supported(op, dt)) { st.code = FT_ERR_UNSUPPORTED_TYPE; return st; }
  const size_t es = ft_dtype_size(dt), bytes = count * es;
  if (bytes > CpuWorld::kSlotBytes || w.n > FT_MAX_FANIN) { st.code = FT_ERR_TOO_LARGE; return st; }
  if (sendbuf && sendbuf != recvbuf) std::memcpy(recvbuf, sendbuf, bytes);
  if (w.n == 1 || count == 0) return st;
  w.ensure_twins();
  const uint64_t call = w.calls[rank]++;
  const uint32_t base = w.epoch[rank];
  w.epoch[rank] = base + 1;
  const size_t slot = (call & 1) * CpuWorld::kSlotBytes;
  std::memcpy(w.slots[rank].data() + slot, recvbuf, bytes);
  if (w.mid_call_hook) w.mid_call_hook(rank);
  std::vector<int> everyone;
  for (int q = 0; q < w.n; ++q)
    if (q != rank) everyone.push_back(q);
  st = detail::rendezvous(w, rank, everyone, base + 1, 0, 1 << 20, nullptr);
  if (st.code != FT_OK) return st;
  if (w.mid_call_hook) w.mid_call_hook(rank);
  const void* src[FT_MAX_FANIN];
  for (int q = 0; q < w.n; ++q) src[q] = w.slots[q].data() + slot;
  st.code = reduce_nway_cpu_dispatch(op, dt, src, recvbuf, w.n, count, 1);
  return st;
}

// Reduce + push (flat two-shot in one pass), in place on the ranks' own buffers: a rendezvous of all ranks
// (inputs are in place), then rank r sums block r over all ranks and writes the result into block r of EVERY
// rank's buffer, then a second rendezvous (results have landed, nobody reads inputs any more).  Device form:
// push_allreduce_kernel; the switch-reduced variant (nvls_allreduce_kernel) has the same two brackets.
inline RankStatus cpu_allreduce_push(CpuWorld& w, int rank, ft_op op, ft_dtype dt, void* buf, uint64_t count) {
  RankStatus st;
  if (!ft_op_supported(op, dt)) { st.code = FT_ERR_UNSUPPORTED_TYPE; return st; }
  if (w.n > FT_MAX_FANIN) { st.code = FT_ERR_TOO_LARGE; return st; }
  if (w.n == 1 || count == 0) return st;
  const size_t es = ft_dtype_size(dt);
  ++w.calls[rank];
  const uint32_t base = w.epoch[rank];
  w.epoch[rank] = base + 2;
  w.bufs[rank].store(buf, std::memory_order_release);
  std::vector<int> everyone;
  for (int q = 0; q < w.n; ++q)
    if (q != rank) everyone.push_back(q);
  st = detail::rendezvous(w, rank, everyone, base + 1, 0, 1 << 20, nullptr);
  if (st.code != FT_OK) return st;
  if (w.mid_call_hook) w.mid_call_hook(rank);
  Blocks g(count, w.n);
  const uint64_t off = g.offset(rank), len = g.length(rank);
  if (len) {
    const void* src[FT_MAX_FANIN];
    for (int q = 0; q < w.n; ++q) src[q] = (const char*)w.bufs[q].load(std::memory_order_acquire) + off * es;
    std::vector<char> sum(len * es);
    st.code = reduce_nway_cpu_dispatch(op, dt, src, sum.data(), w.n, len, 1);
    if (st.code != FT_OK) return st;
    for (int q = 0; q < w.n; ++q) std::memcpy((char*)w.bufs[q].load(std::memory_order_acquire) + off * es, sum.data(), len * es);
  }
  return detail::rendezvous(w, rank, everyone, base + 2, 1, 1 << 20, nullptr);
}

// Low-latency push: no rendezvous at all.  Every rank writes its input as 8-byte words {32 bits of data,
// 32-bit tag of the call} into receive area (call mod 2) of every rank, then polls its own area until
// every word carries the tag, and sums in rank order.  Device form: ll_allreduce_kernel.
inline RankStatus cpu_allreduce_ll(CpuWorld& w, int rank, ft_op op, ft_dtype dt, const void* sendbuf, void* recvbuf,
                                   uint64_t count) {
  RankStatus st;
  if (!ft_op_supported(op, dt)) { st.code = FT_ERR_UNSUPPORTED_TYPE; return st; }
  const size_t es = ft_dtype_size(dt), bytes = count * es, words = (bytes + 3) / 4;
  if (words > CpuWorld::kLLWords || w.n > FT_MAX_FANIN) { st.code = FT_ERR_TOO_LARGE; return st; }
  if (sendbuf && sendbuf != recvbuf) std::memcpy(recvbuf, sendbuf, bytes);
  if (w.n == 1 || count == 0) return st;
  w.ensure_twins();
  const uint64_t call = w.calls[rank]++;
  const uint32_t tag = (uint32_t)(call + 1);   // never 0, the value of untouched memory
  const size_t parity = call & 1;
  auto area = [&](int dst, int src) { return w.ll.get() + (((size_t)dst * 2 + parity) * w.n + src) * CpuWorld::kLLWords; };
  std::vector<uint32_t> mine(words, 0);
  std::memcpy(mine.data(), recvbuf, bytes);
  for (int dst = 0; dst < w.n; ++dst) {
    std::atomic<uint64_t>* a = area(dst, rank);
    // release / acquire on the words stands for the kernel boundaries of the device: a rank's earlier calls
    // have completed (their loads have returned) before this call's stores are issued, and its later calls
    // start only after this call's polls have returned
    for (size_t i = 0; i < words; ++i) a[i].store(((uint64_t)tag << 32) | mine[i], std::memory_order_release);
  }
  if (w.mid_call_hook) w.mid_call_hook(rank);
  std::vector<std::vector<uint32_t>> got(w.n, std::vector<uint32_t>(words));
  const auto t0 = std::chrono::steady_clock::now();
  for (int src = 0; src < w.n; ++src) {
    std::atomic<uint64_t>* a = area(rank, src);
    for (size_t i = 0; i < words; ++i) {
      for (;;) {
        const uint64_t v = a[i].load(std::memory_order_acquire);
        if ((uint32_t)(v >> 32) == tag) { got[src][i] = (uint32_t)v; break; }
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > w.timeout_s) {
          st = {FT_ERR_TIMEOUT, 0, src};
          return st;
        }
        std::this_thread::yield();
      }
    }
  }
  const void* src[FT_MAX_FANIN];
  for (int q = 0; q < w.n; ++q) src[q] = got[q].data();
  std::vector<uint32_t> out(words);
  st.code = reduce_nway_cpu_dispatch(op, dt, src, out.data(), w.n, count, 1);
  std::memcpy(recvbuf, out.data(), bytes);
  return st;
}

// A plan on tagged words: the host twin of ll_tree_allreduce_kernel.  At the start of a stage a rank pushes its current
// copy of every block some peer will fold in or take over into that peer's receive slot (slots numbered by
// build_dev_plan, the table the device uses), then folds in / takes over what arrives in its own slots.  No rendezvous;
// the two receive areas alternate with the call parity and are shared with cpu_allreduce_ll.
inline RankStatus cpu_allreduce_ll_tree(CpuWorld& w, int rank, const Plan& p, ft_op op, ft_dtype dt, const void* sendbuf,
                                        void* recvbuf, uint64_t count) {
  RankStatus st;
  if (!ft_op_supported(op, dt)) { st.code = FT_ERR_UNSUPPORTED_TYPE; return st; }
  if (!p.ok() || p.world != w.n) { st.code = FT_ERR_INVALID_TOPO; return st; }
  const size_t es = ft_dtype_size(dt), bytes = count * es;
  if (sendbuf && sendbuf != recvbuf) std::memcpy(recvbuf, sendbuf, bytes);
  if (w.n == 1 || count == 0) return st;
  const HostDevPlan hd = build_dev_plan(p, rank);
  const Blocks g(count, w.n);
  const size_t block_words = (g.block_elems * es + 3) / 4;
  if ((size_t)hd.plan.nslots * block_words > (size_t)w.n * CpuWorld::kLLWords) { st.code = FT_ERR_TOO_LARGE; return st; }
  w.ensure_twins();
  const uint64_t call = w.calls[rank]++;
  const uint32_t tag = (uint32_t)(call + 1);
  const size_t parity = call & 1;
  auto slot_of = [&](int dst, uint32_t slot) { return w.ll.get() + ((size_t)dst * 2 + parity) * w.n * CpuWorld::kLLWords + (size_t)slot * block_words; };
  char* out = (char*)recvbuf;
  const auto t0 = std::chrono::steady_clock::now();
  std::vector<uint32_t> tmp(block_words);
  for (uint32_t s = 0; s < hd.plan.nstages; ++s) {
    const ftk::DevStage& ds = hd.plan.stages[s];
    for (uint32_t q = ds.push_begin; q < ds.push_end; ++q) {
      const ftk::DevPush& ps = hd.pushes[q];
      const size_t len = g.length(ps.block) * es, words = (len + 3) / 4;
      if (!len) continue;
      std::fill(tmp.begin(), tmp.end(), 0u);
      std::memcpy(tmp.data(), out + g.offset(ps.block) * es, len);
      std::atomic<uint64_t>* a = slot_of(ps.dst, ps.slot);
      for (size_t i = 0; i < words; ++i) a[i].store(((uint64_t)tag << 32) | tmp[i], std::memory_order_release);
    }
    if (w.mid_call_hook) w.mid_call_hook(rank);
    for (uint32_t q = ds.pull_begin; q < ds.pull_end; ++q) {
      const ftk::DevPull& pl = hd.pulls[q];
      const size_t elems = g.length(pl.block), len = elems * es, words = (len + 3) / 4;
      if (!len) continue;
      std::vector<std::vector<uint32_t>> got(pl.nsrc, std::vector<uint32_t>(words));
      for (int k = 0; k < pl.nsrc; ++k) {
        std::atomic<uint64_t>* a = slot_of(rank, pl.slot + k);
        for (size_t i = 0; i < words; ++i)
          for (;;) {
            const uint64_t v = a[i].load(std::memory_order_acquire);
            if ((uint32_t)(v >> 32) == tag) { got[k][i] = (uint32_t)v; break; }
            if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > w.timeout_s) {
              st = {FT_ERR_TIMEOUT, (int)s, pl.src[k]};
              return st;
            }
            std::this_thread::yield();
          }
      }
      char* mine = out + g.offset(pl.block) * es;
      if (pl.reduce) {
        std::vector<uint32_t> own(words, 0), res(words, 0);
        std::memcpy(own.data(), mine, len);
        const void* src[FT_MAX_FANIN + 1];
        src[0] = own.data();
        for (int k = 0; k < pl.nsrc; ++k) src[k + 1] = got[k].data();
        st.code = reduce_nway_cpu_dispatch(op, dt, src, res.data(), pl.nsrc + 1, elems, 1);
        if (st.code != FT_OK) return st;
        std::memcpy(mine, res.data(), len);
      } else {
        std::memcpy(mine, got[0].data(), len);
      }
    }
  }
  return st;
}

}  // namespace ft
