// Process-per-rank world on one host: the FlexTree plan executed between ordinary processes, the way an
// MPI program is launched (one process per rank), without an MPI library.
//
// The ranks meet in a small POSIX shared-memory segment that holds only control state: process ids, the
// address of the buffer each rank exposes for the running call, and the per-pair rendezvous flags (the same
// protocol as the thread world and the device kernels: growing numbers, release on signal, acquire on wait,
// every wait bounded).  Large DATA never goes through the segment: a rank pulls a block straight out of the
// peer process's own buffer with process_vm_readv (cross-memory attach), one call per peer and stage, and adds
// it to its own copy.  That is one copy per pulled block, where a message-passing transport needs two (into
// and out of a shared ring) before the reduction can start.  Messages of up to 16 KiB run on working copies
// inside the segment instead, read by the peers with plain loads: no system call at all.
//
// Role in the reference: tree_allreduce / ring_allreduce over MPI_Isend / MPI_Irecv / MPI_Waitall /
// MPI_Barrier between processes (allreduce_over_mpi/mpi_mod.hpp:1510-1719).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/prctl.h>
#include <sys/stat.h>
#include <sys/uio.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../runtime/heap_alloc.hpp"
#include "cpu_executor.hpp"

namespace ft {

struct ProcShared {
  std::atomic<uint32_t> ready;      // set by rank 0 once the segment is initialised
  std::atomic<uint32_t> attached;   // ranks that have mapped the segment
  std::atomic<uint32_t> detached;   // ranks that have left (the last one unlinks the name)
  int32_t world;
  std::atomic<int32_t> pid[FT_MAX_RANKS];
  std::atomic<int32_t> ppid[FT_MAX_RANKS];   // each rank's parent: one common launcher lets the ranks open up to it alone
  std::atomic<uint32_t> opened;              // ranks that have declared who may read their memory
  std::atomic<uint64_t> buf[FT_MAX_RANKS];                      // address exposed for the running call
  std::atomic<uint32_t> flags[FT_MAX_RANKS * FT_MAX_RANKS];     // flags[dst * world + src]
  // Small messages skip the system calls: a rank's working copy lives here for the length of the call and the
  // peers read it with ordinary loads (pages of ranks that never send small messages are never touched).
  static constexpr size_t kEagerBytes = 16 << 10;
  alignas(64) unsigned char eager[FT_MAX_RANKS][kEagerBytes];
};

class ProcWorld {
 public:
  int rank = 0, n = 1;
  double timeout_s = 30.0;
  std::string error;

  // Collective over the `world` processes that pass the same session name.  False (with `error` set) when
  // the segment cannot be created or the others do not show up in time.
  bool join(const std::string& session, int rank_, int world, double timeout) {
    rank = rank_;
    n = world;
    timeout_s = timeout > 0 ? timeout : timeout_s;
    if (world < 1 || world > FT_MAX_RANKS || rank < 0 || rank >= world) { error = "rank or world out of range"; return false; }
    name_ = "/ftpw-" + session;
    const auto t0 = std::chrono::steady_clock::now();
    auto late = [&] { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s; };
    int fd = -1;
    if (rank == 0) {
      shm_unlink(name_.c_str());   // a stale segment of an earlier run with the same name
      fd = shm_open(name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
      if (fd < 0 || ftruncate(fd, sizeof(ProcShared)) != 0) { error = std::string("shm_open: ") + std::strerror(errno); if (fd >= 0) close(fd); return false; }
    } else {
      while ((fd = shm_open(name_.c_str(), O_RDWR, 0600)) < 0) {
        if (late()) { error = "rank 0 never created the session segment"; return false; }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      struct stat sb;
      while (fstat(fd, &sb) == 0 && (size_t)sb.st_size < sizeof(ProcShared)) {
        if (late()) { error = "session segment never reached its size"; close(fd); return false; }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
    }
    void* p = mmap(nullptr, sizeof(ProcShared), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) { error = std::string("mmap: ") + std::strerror(errno); return false; }
    sh_ = static_cast<ProcShared*>(p);
    if (rank == 0) {
      sh_->world = world;   // a fresh segment is zero-filled: flags, addresses and counters start at 0
      sh_->ready.store(1, std::memory_order_release);
    } else {
      while (sh_->ready.load(std::memory_order_acquire) == 0) {
        if (late()) { error = "rank 0 never initialised the session segment"; return false; }
        std::this_thread::yield();
      }
      if (sh_->world != world) { error = "ranks disagree on the world size"; return false; }
    }
    if (const char* kb = std::getenv("FT_PROC_TILE_KB"); kb && std::atoi(kb) >= 4) tile_bytes_ = (size_t)std::atoi(kb) << 10;
    sh_->pid[rank].store((int32_t)getpid(), std::memory_order_release);
    sh_->ppid[rank].store((int32_t)getppid(), std::memory_order_release);
    sh_->attached.fetch_add(1, std::memory_order_acq_rel);
    while ((int)sh_->attached.load(std::memory_order_acquire) < world) {
      if (late()) { error = "not every rank joined the session"; return false; }
      std::this_thread::yield();
    }
    // Let the sibling ranks read this process's memory (needed where ptrace is restricted to descendants).  The
    // kernel takes ONE process per caller, and its descendants count too: when every rank was started by the same
    // launcher, naming that launcher admits exactly the launcher and the sibling ranks.  Only ranks with different
    // parents (started by hand from several shells) fall back to admitting any process of the same user.
    bool same_parent = true;
    const int32_t parent = sh_->ppid[0].load(std::memory_order_acquire);
    for (int r = 1; r < world; ++r) same_parent = same_parent && sh_->ppid[r].load(std::memory_order_acquire) == parent;
    if (same_parent && parent > 1) prctl(PR_SET_PTRACER, (unsigned long)parent, 0, 0, 0);
    else prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0);
    sh_->opened.fetch_add(1, std::memory_order_acq_rel);
    while ((int)sh_->opened.load(std::memory_order_acquire) < world) {   // nobody reads a peer before it has opened up
      if (late()) { error = "not every rank joined the session"; return false; }
      std::this_thread::yield();
    }
    return true;
  }

  void leave() {
    if (!sh_) return;
    for (unsigned char* b : heap_base_)
      if (b) munmap(b, heap_size_);
    heap_base_.clear();
    heap_size_ = 0;
    const bool last = (int)sh_->detached.fetch_add(1, std::memory_order_acq_rel) + 1 == n;
    munmap(sh_, sizeof(ProcShared));
    sh_ = nullptr;
    if (last || rank == 0) shm_unlink(name_.c_str());
  }
  ~ProcWorld() { leave(); }

  // Rendezvous with `peers`: signal `value` into their flag rows, wait until each of them has signalled at
  // least `value` into this rank's row.
  RankStatus rendezvous(const std::vector<int>& peers, uint32_t value, int index) {
    RankStatus st;
    for (int q : peers) sh_->flags[(size_t)q * n + rank].store(value, std::memory_order_release);
    const auto t0 = std::chrono::steady_clock::now();
    for (int q : peers) {
      unsigned spins = 0;
      while ((int32_t)(sh_->flags[(size_t)rank * n + q].load(std::memory_order_acquire) - value) < 0) {
        if (++spins > 256) {
          spins = 0;
          if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) {
            st = {FT_ERR_TIMEOUT, index, q};
            return st;
          }
          std::this_thread::yield();
        }
      }
    }
    return st;
  }

  RankStatus barrier() {
    std::vector<int> everyone;
    for (int q = 0; q < n; ++q)
      if (q != rank) everyone.push_back(q);
    return n > 1 ? rendezvous(everyone, ++epoch_, 0) : RankStatus{};
  }

  // Rendezvous that opens step `s` of a call running stages [first, last): the stage's own set, or after the last
  // stage the plan's closing set (every rank when a half runs alone).  Returns true when the call is over.
  bool open_step(const Plan& p, int s, int last, int phase, uint32_t base, RankStatus* st) {
    const bool closing = s == last;
    const int index = closing ? p.num_stages : s;
    if (closing && phase) {
      std::vector<int> everyone;
      for (int q = 0; q < n; ++q)
        if (q != rank) everyone.push_back(q);
      *st = rendezvous(everyone, base + (uint32_t)index + 1, index);
    } else {
      *st = rendezvous(p.sync[index][rank], base + (uint32_t)index + 1, index);
    }
    return st->code != FT_OK || closing;
  }

  // `len` bytes at byte offset `off` of the buffer that `peer` exposes for the running call.
  bool read_peer(int peer, uint64_t off, void* dst, size_t len) {
    const uint64_t base = sh_->buf[peer].load(std::memory_order_acquire);
    const pid_t pid = (pid_t)sh_->pid[peer].load(std::memory_order_acquire);
    char* out = static_cast<char*>(dst);
    uint64_t addr = base + off;
    while (len) {
      struct iovec local{out, len}, remote{reinterpret_cast<void*>(addr), len};
      const ssize_t got = process_vm_readv(pid, &local, 1, &remote, 1, 0);
      if (got <= 0) { error = std::string("process_vm_readv from rank ") + std::to_string(peer) + ": " + std::strerror(errno); return false; }
      out += got; addr += (uint64_t)got; len -= (size_t)got;
    }
    return true;
  }

  // Several ranges of the peer's exposed buffer in ONE system call: ranges[i] = {byte offset, bytes} lands
  // at local[i].  Used so that a stage costs one call per peer however many blocks it pulls.
  bool read_peer_ranges(int peer, const std::vector<std::pair<uint64_t, size_t>>& ranges, const std::vector<void*>& local) {
    const uint64_t base = sh_->buf[peer].load(std::memory_order_acquire);
    const pid_t pid = (pid_t)sh_->pid[peer].load(std::memory_order_acquire);
    constexpr size_t kMaxVec = 512;   // below IOV_MAX
    for (size_t first = 0; first < ranges.size(); first += kMaxVec) {
      const size_t cnt = std::min(kMaxVec, ranges.size() - first);
      struct iovec lv[kMaxVec], rv[kMaxVec];
      size_t total = 0;
      for (size_t i = 0; i < cnt; ++i) {
        lv[i] = {local[first + i], ranges[first + i].second};
        rv[i] = {reinterpret_cast<void*>(base + ranges[first + i].first), ranges[first + i].second};
        total += ranges[first + i].second;
      }
      const ssize_t got = process_vm_readv(pid, lv, cnt, rv, cnt, 0);
      if (got == (ssize_t)total) continue;
      if (got < 0) { error = std::string("process_vm_readv from rank ") + std::to_string(peer) + ": " + std::strerror(errno); return false; }
      for (size_t i = 0; i < cnt; ++i)   // a short transfer: finish range by range
        if (!read_peer(peer, ranges[first + i].first, local[first + i], ranges[first + i].second)) return false;
    }
    return true;
  }

  // One rank's part of an all-reduce, in place on recvbuf (sendbuf null or == recvbuf) or out of place.
  // phase 0: the whole all-reduce; 1: the reduce-scatter half alone; 2: the all-gather half alone (each half keeps its
  // stages' rendezvous numbers and closes with a rendezvous of ALL ranks, like ft_reduce_scatter / ft_all_gather).
  RankStatus allreduce(const Plan& p, ft_op op, ft_dtype dt, const void* sendbuf, void* recvbuf, uint64_t count, int phase = 0) {
    RankStatus st;
    if (!sh_) { st.code = FT_ERR_INVALID_ARG; return st; }
    if (!p.ok() || p.world != n) { st.code = FT_ERR_INVALID_TOPO; return st; }
    if (!ft_op_supported(op, dt)) {
      st.code = ((int)op < 0 || op >= FT_OP_COUNT) ? FT_ERR_UNSUPPORTED_OP : FT_ERR_UNSUPPORTED_TYPE;
      return st;
    }
    const size_t es = ft_dtype_size(dt);
    if (sendbuf && sendbuf != recvbuf) std::memcpy(recvbuf, sendbuf, count * es);
    if (n == 1 || count == 0) return st;
    Blocks g(count, n);
    const uint32_t base = epoch_;
    epoch_ = base + (uint32_t)p.num_stages + 1;
    const int first = phase == 2 ? p.num_stages / 2 : 0;
    const int last = phase == 1 ? p.num_stages / 2 : p.num_stages;   // one past the last stage that runs
    // a tensor in the symmetric heap: every peer has it mapped at the same offset of that peer's heap
    if (heap_size_ && in_heap(recvbuf, count * es)) {
      const uint64_t off_in_heap = (uint64_t)(static_cast<unsigned char*>(recvbuf) - heap_base_[rank]);
      return run_direct(p, op, dt, g, base, es, [&](int q) { return heap_base_[q] + off_in_heap; }, first, last, phase);
    }
    if (count * es <= ProcShared::kEagerBytes && phase == 0) {   // a half alone leaves partial sums behind: not on a scratch copy
      // the whole call runs on working copies inside the control segment, exactly like the thread world
      std::memcpy(sh_->eager[rank], recvbuf, count * es);
      st = run_direct(p, op, dt, g, base, es, [&](int q) { return sh_->eager[q]; }, first, last, phase);
      if (st.code == FT_OK) std::memcpy(recvbuf, sh_->eager[rank], count * es);
      return st;
    }
    sh_->buf[rank].store((uint64_t)reinterpret_cast<uintptr_t>(recvbuf), std::memory_order_release);
    const size_t tile_elems = tile_bytes_ / es;
    int max_src = 1;
    for (int s = 0; s < p.num_stages; ++s)
      for (const Pull& pl : p.stages[rank][s].pulls) max_src = std::max<int>(max_src, (int)pl.srcs.size());
    if (tmp_.size() < (size_t)max_src * tile_bytes_) tmp_.resize((size_t)max_src * tile_bytes_);
    for (int s = first; s <= last; ++s) {
      if (open_step(p, s, last, phase, base, &st)) return st;
      const std::vector<Pull>& pulls = p.stages[rank][s].pulls;
      size_t i = 0;
      while (i < pulls.size()) {
        if (!pulls[i].reduce) {
          // a run of gathers: one call per source rank, every block straight into its place
          size_t j = i;
          std::vector<int> order;
          std::vector<std::vector<std::pair<uint64_t, size_t>>> ranges(n);
          std::vector<std::vector<void*>> local(n);
          for (; j < pulls.size() && !pulls[j].reduce; ++j) {
            const uint64_t off = g.offset(pulls[j].block), len = g.length(pulls[j].block);
            if (!len) continue;
            const int q = pulls[j].srcs[0];
            if (ranges[q].empty()) order.push_back(q);
            ranges[q].push_back({off * es, (size_t)(len * es)});
            local[q].push_back(static_cast<char*>(recvbuf) + off * es);
          }
          for (int q : order)
            if (!read_peer_ranges(q, ranges[q], local[q])) { st = {FT_ERR_PROTOCOL, s, q}; return st; }
          i = j;
          continue;
        }
        // reductions with the same sources whose blocks fit one tile together: one call per source for all of them
        size_t j = i, batch_bytes = 0;
        while (j < pulls.size() && pulls[j].reduce && pulls[j].srcs == pulls[i].srcs &&
               batch_bytes + g.length(pulls[j].block) * es <= tile_bytes_) {
          batch_bytes += g.length(pulls[j].block) * es;
          ++j;
        }
        if (j > i + 1) {
          std::vector<std::pair<uint64_t, size_t>> ranges;
          std::vector<size_t> at;   // where each block of the batch sits inside a source's tile
          size_t pos = 0;
          for (size_t b = i; b < j; ++b) {
            const size_t bytes = g.length(pulls[b].block) * es;
            at.push_back(pos);
            if (bytes) ranges.push_back({g.offset(pulls[b].block) * es, bytes});
            pos += bytes;
          }
          int k = 0;
          for (int q : pulls[i].srcs) {
            std::vector<void*> local;
            for (size_t b = i; b < j; ++b)
              if (g.length(pulls[b].block)) local.push_back(tmp_.data() + (size_t)k * tile_bytes_ + at[b - i]);
            if (!ranges.empty() && !read_peer_ranges(q, ranges, local)) { st = {FT_ERR_PROTOCOL, s, q}; return st; }
            ++k;
          }
          for (size_t b = i; b < j; ++b) {
            const uint64_t len = g.length(pulls[b].block);
            if (!len) continue;
            char* mine = static_cast<char*>(recvbuf) + g.offset(pulls[b].block) * es;
            const void* src[FT_MAX_FANIN];
            int m = 0;
            src[m++] = mine;
            for (size_t q = 0; q < pulls[i].srcs.size(); ++q) src[m++] = tmp_.data() + q * tile_bytes_ + at[b - i];
            st.code = reduce_nway_cpu_dispatch(op, dt, src, mine, m, len, 1);
            if (st.code != FT_OK) return st;
          }
          i = j;
          continue;
        }
        const Pull& pl = pulls[i++];
        const uint64_t off = g.offset(pl.block), len = g.length(pl.block);
        for (uint64_t t = 0; t < len; t += tile_elems) {
          const uint64_t m = std::min<uint64_t>(tile_elems, len - t);
          char* mine = static_cast<char*>(recvbuf) + (off + t) * es;
          const void* src[FT_MAX_FANIN];
          int k = 0;
          src[k++] = mine;
          for (int q : pl.srcs) {
            char* slot = tmp_.data() + (size_t)(k - 1) * tile_bytes_;
            if (!read_peer(q, (off + t) * es, slot, m * es)) { st = {FT_ERR_PROTOCOL, s, q}; return st; }
            src[k++] = slot;
          }
          st.code = reduce_nway_cpu_dispatch(op, dt, src, mine, k, m, 1);
          if (st.code != FT_OK) return st;
        }
      }
    }
    return st;
  }

  // ---- symmetric heap: memory that every rank can address directly -------------------------------------
  // Each rank owns one shared segment of `bytes` and maps everybody else's.  A tensor allocated from it is
  // reduced in place with plain loads from the peers' mappings (no system call, no copy), provided every rank
  // allocates in the same order so that the tensor sits at the same offset everywhere: the design of the GPU
  // communicator's symmetric heap, on the host.  Collective; call once.
  bool heap_create(size_t bytes) {
    if (!sh_ || heap_size_) { error = "heap_create: not joined, or a heap exists already"; return false; }
    bytes = (bytes + 4095) / 4096 * 4096;
    auto seg = [&](int q) { return name_ + "-h" + std::to_string(q); };
    auto map_seg = [&](int q, bool create) -> unsigned char* {
      const int fd = shm_open(seg(q).c_str(), create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
      if (fd < 0 || (create && ftruncate(fd, (off_t)bytes) != 0)) { error = "heap segment: " + std::string(std::strerror(errno)); if (fd >= 0) close(fd); return nullptr; }
      void* m = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
      close(fd);
      if (m == MAP_FAILED) { error = "heap mmap: " + std::string(std::strerror(errno)); return nullptr; }
      return static_cast<unsigned char*>(m);
    };
    shm_unlink(seg(rank).c_str());
    heap_base_.assign(n, nullptr);
    bool ok = (heap_base_[rank] = map_seg(rank, true)) != nullptr;
    if (barrier().code != FT_OK) return false;          // every segment exists (or its owner failed)
    for (int q = 0; q < n && ok; ++q)
      if (q != rank) ok = (heap_base_[q] = map_seg(q, false)) != nullptr;
    const bool all_here = barrier().code == FT_OK;      // everybody has mapped everything: the names can go
    shm_unlink(seg(rank).c_str());
    if (!ok || !all_here) return false;
    heap_size_ = bytes;
    heap_alloc_.reset(bytes);
    return true;
  }
  void* heap_alloc(size_t bytes) {
    if (!heap_size_) return nullptr;
    const size_t off = heap_alloc_.alloc(bytes);
    return off == HeapAllocator::kNone ? nullptr : heap_base_[rank] + off;
  }
  bool heap_free(void* ptr) {
    return heap_size_ && in_heap(ptr, 1) && heap_alloc_.free((size_t)(static_cast<unsigned char*>(ptr) - heap_base_[rank]));
  }
  // Collective debugging aid: true when `ptr` sits at the same heap offset on every rank (ranks that allocate
  // in different orders would otherwise reduce unrelated memory without any error).
  bool heap_symmetric(const void* ptr) {
    if (!heap_size_ || !in_heap(ptr, 1)) return false;
    const uint64_t mine = (uint64_t)(static_cast<const unsigned char*>(ptr) - heap_base_[rank]);
    sh_->buf[rank].store(mine, std::memory_order_release);
    if (barrier().code != FT_OK) return false;
    bool same = true;
    for (int q = 0; q < n; ++q) same = same && sh_->buf[q].load(std::memory_order_acquire) == mine;
    return barrier().code == FT_OK && same;
  }
  bool in_heap(const void* ptr, size_t bytes) const {
    const unsigned char* q = static_cast<const unsigned char*>(ptr);
    return heap_size_ && q >= heap_base_[rank] && q + bytes <= heap_base_[rank] + heap_size_;
  }

 private:
  // The plan on working copies that every rank can address: base_of(q) is rank q's copy as mapped here.
  template <class BaseOf>
  RankStatus run_direct(const Plan& p, ft_op op, ft_dtype dt, const Blocks& g, uint32_t base, size_t es, BaseOf base_of, int first,
                        int last, int phase) {
    RankStatus st;
    unsigned char* work = base_of(rank);
    for (int s = first; s <= last; ++s) {
      if (open_step(p, s, last, phase, base, &st)) return st;
      for (const Pull& pl : p.stages[rank][s].pulls) {
        const uint64_t off = g.offset(pl.block), len = g.length(pl.block);
        if (!len) continue;
        unsigned char* mine = work + off * es;
        if (pl.reduce) {
          const void* src[FT_MAX_FANIN];
          int k = 0;
          src[k++] = mine;
          for (int q : pl.srcs) src[k++] = base_of(q) + off * es;
          st.code = reduce_nway_cpu_dispatch(op, dt, src, mine, k, len, 1);
          if (st.code != FT_OK) return st;
        } else {
          std::memcpy(mine, base_of(pl.srcs[0]) + off * es, len * es);
        }
      }
    }
    return st;
  }

  size_t tile_bytes_ = 256 << 10;   // pulled tiles stay in the cache until they are added (FT_PROC_TILE_KB overrides)
  ProcShared* sh_ = nullptr;
  std::string name_;
  uint32_t epoch_ = 0;
  std::vector<char> tmp_;
  std::vector<unsigned char*> heap_base_;   // heap_base_[q] = rank q's heap segment as mapped in this process
  size_t heap_size_ = 0;
  HeapAllocator heap_alloc_;
};

}  // namespace ft
