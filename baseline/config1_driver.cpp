// CPU all-reduce comparison on one workload, one source, two builds:
//
//   -DCONFIG1_REFERENCE   the unmodified reference (allreduce_over_mpi/mpi_mod.hpp, MPI_Allreduce_FT)
//                         over baseline/mpi_shim; ranks are processes (FTSHIM_RANK / FTSHIM_SIZE)
//   (default)             this repository's MPI-compatible entry (csrc/api/flextree_mpi.h) over the
//                         thread world of libflextree.so; ranks are threads of this process
//   -DCONFIG1_PROCS       the same entry over the process world: ranks are processes (FT_RANK / FT_WORLD /
//                         FT_SESSION), exactly like the reference arm, with no MPI library underneath
//
//   config1_driver <world> <count> <repeat> [warmup]         (world is ignored by the reference build)
//
// Workload: every rank holds `count` floats drawn uniform[-1,1) from std::mt19937 seeded with its
// rank; the result of the in-place SUM all-reduce is compared on every rank with a double-precision
// sum of the same N streams.  Each repeat starts from the original input (restored outside the
// timed span).  A repeat's time runs from a barrier to the moment every rank has returned (call +
// barrier), read on rank 0.  Tree shape comes from FT_TOPO / FT_LONELY in both builds.
// Rank 0 prints one JSON line.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#ifdef CONFIG1_REFERENCE
#include <mpi.h>
#include <glog/logging.h>
#define STANDALONE_TEST
#include "mpi_mod.hpp"
#else
#include <atomic>
#include <chrono>
#include <thread>
#include "api/flextree_mpi.h"
#endif

namespace {

void fill(std::vector<float>& v, int seed) {
  std::mt19937 rng((unsigned)seed);
  std::uniform_real_distribution<float> u(-1.f, 1.f);
  for (auto& x : v) x = u(rng);
}

std::vector<double> oracle(int world, size_t count) {
  std::vector<double> sum(count, 0.0);
  std::vector<float> v(count);
  for (int r = 0; r < world; ++r) {
    fill(v, r);
    for (size_t i = 0; i < count; ++i) sum[i] += v[i];
  }
  return sum;
}

double max_err(const std::vector<float>& got, const std::vector<double>& want) {
  double e = 0;
  for (size_t i = 0; i < got.size(); ++i) e = std::max(e, std::fabs((double)got[i] - want[i]));
  return e;
}

void report(const char* impl, int world, size_t count, int repeat, const std::vector<double>& sec, double err) {
  double mn = 1e30, sum = 0;
  for (double s : sec) { mn = std::min(mn, s); sum += s; }
  const double avg = sum / sec.size(), bytes = (double)count * sizeof(float);
  const char* topo = getenv("FT_TOPO");
  const char* lonely = getenv("FT_LONELY");
  // fp32 sums of N values in [-1,1): a few ulp of N is the most any summation order can be off
  const bool ok = err <= 4e-7 * world * 4;
  printf("{\"impl\": \"%s\", \"world\": %d, \"count\": %zu, \"repeat\": %d, \"FT_TOPO\": \"%s\", \"FT_LONELY\": \"%s\", "
         "\"ms_min\": %.4f, \"ms_avg\": %.4f, \"busbw_gbs_at_min\": %.3f, \"max_abs_err_vs_fp64\": %.3g, \"check\": \"%s\"}\n",
         impl, world, count, repeat, topo ? topo : "", lonely ? lonely : "0", mn * 1e3, avg * 1e3,
         bytes / mn * 1e-9 * 2.0 * (world - 1) / world, err, ok ? "passed" : "FAILED");
}

}  // namespace

#ifdef CONFIG1_REFERENCE

int main(int argc, char** argv) {
  if (argc < 4) { fprintf(stderr, "usage: %s <world> <count> <repeat> [warmup]\n", argv[0]); return 2; }
  const size_t count = strtoull(argv[2], nullptr, 10);
  const int repeat = atoi(argv[3]), warmup = argc > 4 ? atoi(argv[4]) : 1;
  int tmp = 0, world = 0, rank = 0;
  MPI_Init_thread(&argc, &argv, MPI_THREAD_MULTIPLE, &tmp);
  MPI_Comm_size(MPI_COMM_WORLD, &world);
  MPI_Comm_rank(MPI_COMM_WORLD, &rank);
  std::vector<float> input(count), work(count);
  fill(input, rank);
  std::vector<double> sec;
  for (int i = 0; i < warmup + repeat; ++i) {
    work = input;
    MPI_Barrier(MPI_COMM_WORLD);
    const double t0 = MPI_Wtime();
    MPI_Allreduce_FT(MPI_IN_PLACE, work.data(), count, MPI_FLOAT, MPI_SUM, MPI_COMM_WORLD);
    MPI_Barrier(MPI_COMM_WORLD);
    const double t1 = MPI_Wtime();
    if (i >= warmup) sec.push_back(t1 - t0);
  }
  const double err = max_err(work, oracle(world, count));
  // every rank's verdict reaches rank 0 as a sum of 0/1 flags
  float bad = err > 4e-7 * world * 4 ? 1.f : 0.f, bad_all = 0.f;
  MPI_Allreduce(&bad, &bad_all, 1, MPI_FLOAT, MPI_SUM, MPI_COMM_WORLD);
  if (rank == 0) report("reference", world, count, repeat, sec, bad_all > 0 ? 1.0 : err);
  MPI_Finalize();
  return bad_all > 0 ? 1 : 0;
}

#elif defined(CONFIG1_PROCS)

int main(int argc, char** argv) {
  if (argc < 4) { fprintf(stderr, "usage: %s <world> <count> <repeat> [warmup]\n", argv[0]); return 2; }
  const size_t count = strtoull(argv[2], nullptr, 10);
  const int repeat = atoi(argv[3]), warmup = argc > 4 ? atoi(argv[4]) : 1;
  FT_Comm comm = ft_mpi_proc_init_env(60.0);
  if (!comm) { fprintf(stderr, "%s\n", ft_mpi_last_error()); return 2; }
  int world = 0, rank = 0;
  FT_Comm_size(comm, &world);
  FT_Comm_rank(comm, &rank);
  std::vector<float> input(count), private_work(count);
  fill(input, rank);
  // CONFIG1_HEAP=1: the tensor lives in the process world's symmetric heap (shared mappings, reduced in place
  // with plain loads); otherwise in ordinary private memory (pulled with process_vm_readv)
  const bool heap = getenv("CONFIG1_HEAP") && getenv("CONFIG1_HEAP")[0] == '1';
  float* work = private_work.data();
  int rc = 0;
  if (heap) {
    ft_proc_world* w = ft_mpi_proc_world(comm);
    rc |= ft_proc_heap_create(w, count * sizeof(float) + (1 << 20));
    work = rc ? nullptr : (float*)ft_proc_alloc(w, count * sizeof(float));
    if (!work || !ft_proc_heap_symmetric(w, work)) { fprintf(stderr, "rank %d: no symmetric heap (%s)\n", rank, ft_proc_last_error(w)); return 2; }
  }
  std::vector<double> sec;
  for (int i = 0; i < warmup + repeat; ++i) {
    memcpy(work, input.data(), count * sizeof(float));
    FT_Barrier(comm);
    const auto t0 = std::chrono::steady_clock::now();
    rc |= MPI_Allreduce_FT(FT_IN_PLACE, work, (int)count, FT_FLOAT, FT_OP_SUM, comm);
    FT_Barrier(comm);
    const auto t1 = std::chrono::steady_clock::now();
    if (i >= warmup) sec.push_back(std::chrono::duration<double>(t1 - t0).count());
  }
  const double err = max_err(std::vector<float>(work, work + count), oracle(world, count));
  float bad = (rc != 0 || err > 4e-7 * world * 4) ? 1.f : 0.f;
  MPI_Allreduce_FT(FT_IN_PLACE, &bad, 1, FT_FLOAT, FT_OP_SUM, comm);   // every rank's verdict reaches rank 0
  if (rank == 0) report(heap ? "flextree-procs-heap" : "flextree-procs", world, count, repeat, sec, bad > 0 ? 1.0 : err);
  ft_mpi_proc_finalize(comm);
  return bad > 0 ? 1 : 0;
}

#else

namespace {
// sense-reversing barrier for the rank threads (the timed span must not include thread start-up)
struct Barrier {
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    const int gen = gen_.load(std::memory_order_acquire);
    if (count_.fetch_add(1, std::memory_order_acq_rel) + 1 == n_) {
      count_.store(0, std::memory_order_relaxed);
      gen_.store(gen + 1, std::memory_order_release);
    } else {
      while (gen_.load(std::memory_order_acquire) == gen) std::this_thread::yield();
    }
  }
  const int n_;
  std::atomic<int> count_{0}, gen_{0};
};
}  // namespace

int main(int argc, char** argv) {
  if (argc < 4) { fprintf(stderr, "usage: %s <world> <count> <repeat> [warmup]\n", argv[0]); return 2; }
  const int world = atoi(argv[1]);
  const size_t count = strtoull(argv[2], nullptr, 10);
  const int repeat = atoi(argv[3]), warmup = argc > 4 ? atoi(argv[4]) : 1;
  if (world < 1 || world > FT_MAX_RANKS) { fprintf(stderr, "world must be in [1, %d]\n", FT_MAX_RANKS); return 2; }
  ft_cpu_world* w = ft_cpu_world_create(world, 60.0);
  Barrier bar(world);
  std::vector<double> sec;
  std::vector<double> errs(world, 0.0);
  std::vector<int> rcs(world, 0);
  const std::vector<double> want = oracle(world, count);
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r)
    ranks.emplace_back([&, r] {
      FT_Comm comm = ft_mpi_thread_rank(w, r);
      std::vector<float> input(count), work(count);
      fill(input, r);
      for (int i = 0; i < warmup + repeat; ++i) {
        work = input;
        bar.wait();
        const auto t0 = std::chrono::steady_clock::now();
        const int rc = MPI_Allreduce_FT(FT_IN_PLACE, work.data(), (int)count, FT_FLOAT, FT_OP_SUM, comm);
        bar.wait();
        const auto t1 = std::chrono::steady_clock::now();
        if (rc != 0) rcs[r] = rc;
        if (r == 0 && i >= warmup) sec.push_back(std::chrono::duration<double>(t1 - t0).count());
      }
      errs[r] = max_err(work, want);
      ft_mpi_comm_free(comm);
    });
  for (auto& t : ranks) t.join();
  ft_cpu_world_destroy(w);
  int bad = 0;
  double err = 0;
  for (int r = 0; r < world; ++r) {
    if (rcs[r]) { fprintf(stderr, "rank %d: MPI_Allreduce_FT returned %d (%s)\n", r, rcs[r], ft_mpi_last_error()); bad = 1; }
    err = std::max(err, errs[r]);
  }
  if (bad) return 1;
  report("flextree-threads", world, count, repeat, sec, err);
  return err <= 4e-7 * world * 4 ? 0 : 1;
}

#endif
