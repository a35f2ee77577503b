// Shared-memory implementation of the MPI subset declared in mpi.h (see there for scope).
//
// Layout of the shared segment:  Header | barrier slots | split table | N*N rings.
// ring(src,dst) is a single-producer single-consumer byte queue; Isend/Irecv only record a
// request, MPI_Waitall moves bytes for all of its requests until they are complete, keeping
// per-pair FIFO order.  Barriers are generation counters, one slot per communicator.
#include "mpi.h"

#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr int kMaxRanks = 64;
constexpr int kBarrierSlots = 4096;
constexpr size_t kRingBytes = 4u << 20;

struct Ring {
  alignas(64) std::atomic<unsigned long long> head;  // bytes consumed
  alignas(64) std::atomic<unsigned long long> tail;  // bytes produced
  alignas(64) unsigned char data[kRingBytes];
};
struct BarrierSlot {
  alignas(64) std::atomic<int> count;
  std::atomic<int> gen;
};
struct Header {
  std::atomic<int> attached;
  std::atomic<int> ready;
  int world;
  BarrierSlot barriers[kBarrierSlots];
  int split_color[kMaxRanks];
  int split_key[kMaxRanks];
};

struct CommInfo {
  std::vector<int> members;  // world ranks, ordered by key
  int my_index = 0;
  int barrier_slot = 0;
};

struct Req {
  bool send = false, done = true;
  unsigned char* buf = nullptr;
  size_t bytes = 0, moved = 0;
  int peer = 0;
};

Header* g_hdr = nullptr;
Ring* g_rings = nullptr;
size_t g_seg_bytes = 0;
std::string g_name;
int g_rank = 0, g_world = 1;
std::vector<CommInfo> g_comms;
std::vector<Req> g_reqs;
std::vector<int> g_active;  // open request slots in posting order
int g_split_seq = 0;

Ring& ring(int src, int dst) { return g_rings[(size_t)src * g_world + dst]; }

size_t type_size(MPI_Datatype t) {
  switch (t) {
    case MPI_UINT8_T: case MPI_INT8_T: case MPI_C_BOOL: return 1;
    case MPI_UINT16_T: case MPI_INT16_T: return 2;
    case MPI_INT32_T: case MPI_FLOAT: return 4;
    case MPI_INT64_T: case MPI_DOUBLE: case MPI_LONG_LONG_INT: case MPI_LONG_LONG: return 8;
    default: return 0;
  }
}

void barrier_on(const CommInfo& c) {
  const int n = (int)c.members.size();
  if (n <= 1) return;
  BarrierSlot& b = g_hdr->barriers[c.barrier_slot];
  const int gen = b.gen.load(std::memory_order_acquire);
  if (b.count.fetch_add(1, std::memory_order_acq_rel) == n - 1) {
    b.count.store(0, std::memory_order_relaxed);
    b.gen.fetch_add(1, std::memory_order_release);
  } else {
    int spins = 0;
    while (b.gen.load(std::memory_order_acquire) == gen)
      if (++spins > 200) { sched_yield(); spins = 0; }
  }
}

// Move what can be moved for one request; returns true when it made progress.
bool progress(Req& r) {
  if (r.done) return false;
  if (r.bytes == r.moved) { r.done = true; return true; }
  if (r.send) {
    Ring& q = ring(g_rank, r.peer);
    const unsigned long long head = q.head.load(std::memory_order_acquire), tail = q.tail.load(std::memory_order_relaxed);
    size_t room = kRingBytes - (size_t)(tail - head), n = r.bytes - r.moved;
    if (n > room) n = room;
    if (!n) return false;
    const size_t pos = (size_t)(tail % kRingBytes), first = n < kRingBytes - pos ? n : kRingBytes - pos;
    std::memcpy(q.data + pos, r.buf + r.moved, first);
    if (n > first) std::memcpy(q.data, r.buf + r.moved + first, n - first);
    q.tail.store(tail + n, std::memory_order_release);
    r.moved += n;
  } else {
    Ring& q = ring(r.peer, g_rank);
    const unsigned long long tail = q.tail.load(std::memory_order_acquire), head = q.head.load(std::memory_order_relaxed);
    size_t avail = (size_t)(tail - head), n = r.bytes - r.moved;
    if (n > avail) n = avail;
    if (!n) return false;
    const size_t pos = (size_t)(head % kRingBytes), first = n < kRingBytes - pos ? n : kRingBytes - pos;
    std::memcpy(r.buf + r.moved, q.data + pos, first);
    if (n > first) std::memcpy(r.buf + r.moved + first, q.data, n - first);
    q.head.store(head + n, std::memory_order_release);
    r.moved += n;
  }
  if (r.moved == r.bytes) r.done = true;
  return true;
}

int new_req(bool send, void* buf, size_t bytes, int peer, MPI_Request* out) {
  int slot = -1;
  for (size_t i = 0; i < g_reqs.size(); ++i)
    if (g_reqs[i].done && g_reqs[i].buf == nullptr && !g_reqs[i].bytes) { slot = (int)i; break; }
  if (slot < 0) { g_reqs.emplace_back(); slot = (int)g_reqs.size() - 1; }
  Req& r = g_reqs[slot];
  r.send = send; r.done = false; r.buf = (unsigned char*)buf; r.bytes = bytes; r.moved = 0; r.peer = peer;
  out->slot = slot;
  g_active.push_back(slot);
  return MPI_SUCCESS;
}

}  // namespace

extern "C" {

int MPI_Init_thread(int*, char***, int required, int* provided) {
  const char* r = getenv("FTSHIM_RANK") ? getenv("FTSHIM_RANK") : getenv("RANK");
  const char* w = getenv("FTSHIM_SIZE") ? getenv("FTSHIM_SIZE") : getenv("WORLD_SIZE");
  const char* s = getenv("FTSHIM_SESSION") ? getenv("FTSHIM_SESSION") : getenv("MASTER_PORT");
  g_rank = r ? atoi(r) : 0;
  g_world = w ? atoi(w) : 1;
  if (g_world < 1 || g_world > kMaxRanks || g_rank < 0 || g_rank >= g_world) {
    fprintf(stderr, "mpi shim: bad RANK/WORLD_SIZE\n");
    exit(2);
  }
  g_name = std::string("/ftshim-") + (s ? s : "default");
  g_seg_bytes = sizeof(Header) + sizeof(Ring) * (size_t)g_world * g_world + 4096;
  int fd = shm_open(g_name.c_str(), O_CREAT | O_RDWR, 0600);
  if (fd < 0 || ftruncate(fd, (off_t)g_seg_bytes) != 0) { perror("mpi shim: shm"); exit(2); }
  void* p = mmap(nullptr, g_seg_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) { perror("mpi shim: mmap"); exit(2); }
  g_hdr = (Header*)p;                       // a fresh segment is all zeroes: every counter starts at 0
  g_rings = (Ring*)(((uintptr_t)p + sizeof(Header) + 4095) & ~(uintptr_t)4095);
  g_hdr->world = g_world;
  CommInfo world;
  for (int i = 0; i < g_world; ++i) world.members.push_back(i);
  world.my_index = g_rank;
  world.barrier_slot = 0;
  g_comms.push_back(world);
  g_hdr->attached.fetch_add(1);
  while (g_hdr->attached.load() < g_world) sched_yield();
  barrier_on(g_comms[0]);
  if (provided) *provided = required;
  return MPI_SUCCESS;
}

int MPI_Finalize(void) {
  barrier_on(g_comms[0]);
  if (g_hdr->ready.fetch_add(1) == g_world - 1) shm_unlink(g_name.c_str());  // last one out removes the name
  munmap((void*)g_hdr, g_seg_bytes);
  g_hdr = nullptr;
  return MPI_SUCCESS;
}

int MPI_Comm_size(MPI_Comm comm, int* size) { *size = (int)g_comms[comm].members.size(); return MPI_SUCCESS; }
int MPI_Comm_rank(MPI_Comm comm, int* rank) { *rank = g_comms[comm].my_index; return MPI_SUCCESS; }

int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm) {
  const CommInfo parent = g_comms[comm];
  g_hdr->split_color[g_rank] = color;
  g_hdr->split_key[g_rank] = key;
  barrier_on(parent);  // everyone has published (color, key)
  CommInfo c;
  std::vector<std::pair<int, int>> mine;  // (key, world rank)
  for (int r : parent.members)
    if (g_hdr->split_color[r] == color) mine.push_back({g_hdr->split_key[r], r});
  for (size_t i = 0; i < mine.size(); ++i)
    for (size_t j = i + 1; j < mine.size(); ++j)
      if (mine[j] < mine[i]) std::swap(mine[i], mine[j]);
  for (size_t i = 0; i < mine.size(); ++i) {
    c.members.push_back(mine[i].second);
    if (mine[i].second == g_rank) c.my_index = (int)i;
  }
  // every rank performs the same sequence of splits, so (sequence number, colour) names the
  // new communicator consistently; colours beyond 0/1 share slots modulo 8
  ++g_split_seq;
  c.barrier_slot = 1 + ((g_split_seq * 8 + (color & 7)) % (kBarrierSlots - 1));
  barrier_on(parent);  // the table may be reused by the next split
  g_comms.push_back(c);
  *newcomm = (MPI_Comm)g_comms.size() - 1;
  return MPI_SUCCESS;
}

int MPI_Type_size(MPI_Datatype t, int* size) { *size = (int)type_size(t); return MPI_SUCCESS; }
int MPI_Type_get_name(MPI_Datatype t, char* name, int* len) {
  snprintf(name, 20, "MPI_TYPE_%d", t);
  *len = (int)strlen(name);
  return MPI_SUCCESS;
}

int MPI_Isend(const void* buf, int count, MPI_Datatype t, int dest, int, MPI_Comm comm, MPI_Request* req) {
  return new_req(true, (void*)buf, (size_t)count * type_size(t), g_comms[comm].members[dest], req);
}
int MPI_Irecv(void* buf, int count, MPI_Datatype t, int source, int, MPI_Comm comm, MPI_Request* req) {
  return new_req(false, buf, (size_t)count * type_size(t), g_comms[comm].members[source], req);
}

int MPI_Waitall(int count, MPI_Request reqs[], MPI_Status[]) {
  // Like a real MPI, waiting drives EVERY outstanding request of this process, not only the
  // ones waited for (the reference waits for its receives before its sends).  Per peer and
  // direction, bytes move in posting order.
  for (;;) {
    bool moved = false;
    bool blocked[2][kMaxRanks] = {};
    for (int slot : g_active) {
      Req& r = g_reqs[slot];
      if (r.done) continue;
      if (!blocked[r.send][r.peer]) moved = progress(r) || moved;
      if (!r.done) blocked[r.send][r.peer] = true;
    }
    bool all_done = true;
    for (int i = 0; i < count; ++i) all_done = all_done && g_reqs[reqs[i].slot].done;
    if (all_done) break;
    if (!moved) sched_yield();
  }
  for (int i = 0; i < count; ++i) {
    const int slot = reqs[i].slot;
    g_reqs[slot].buf = nullptr;  // slot free for reuse
    g_reqs[slot].bytes = 0;
    for (size_t k = 0; k < g_active.size(); ++k)
      if (g_active[k] == slot) { g_active.erase(g_active.begin() + k); break; }
  }
  return MPI_SUCCESS;
}

int MPI_Barrier(MPI_Comm comm) { barrier_on(g_comms[comm]); return MPI_SUCCESS; }

// The library's own all-reduce (the reference benchmark's "--comm-type mpi" arm): gather to
// every rank through the rings and add locally.  Only what that arm uses: SUM on float/double/int32/int64.
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype t, MPI_Op op, MPI_Comm comm) {
  const CommInfo& c = g_comms[comm];
  const size_t es = type_size(t), bytes = (size_t)count * es;
  if (op != MPI_SUM || !es) return 1;
  std::vector<unsigned char> mine(bytes), tmp(bytes);
  std::memcpy(mine.data(), sendbuf == MPI_IN_PLACE ? recvbuf : sendbuf, bytes);
  std::memcpy(recvbuf, mine.data(), bytes);
  const int n = (int)c.members.size();
  for (int step = 1; step < n; ++step) {
    const int to = (c.my_index + step) % n, from = (c.my_index - step + n) % n;
    MPI_Request rq[2];
    MPI_Isend(mine.data(), count, t, to, 0, comm, &rq[0]);
    MPI_Irecv(tmp.data(), count, t, from, 0, comm, &rq[1]);
    MPI_Waitall(2, rq, nullptr);
    for (int i = 0; i < count; ++i) {
      switch (t) {
        case MPI_FLOAT: ((float*)recvbuf)[i] += ((float*)tmp.data())[i]; break;
        case MPI_DOUBLE: ((double*)recvbuf)[i] += ((double*)tmp.data())[i]; break;
        case MPI_INT32_T: ((int*)recvbuf)[i] += ((int*)tmp.data())[i]; break;
        default: ((long long*)recvbuf)[i] += ((long long*)tmp.data())[i]; break;
      }
    }
  }
  return MPI_SUCCESS;
}

double MPI_Wtime(void) {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

}  // extern "C"
