// Standalone all-reduce benchmark with the reference driver's command line
// (allreduce_over_mpi/benchmark.cpp:69-122):
//
//     ft_bench [--size N] [--repeat R] [--to-file] [--comm-type flextree|threads|procs|nccl] [--tag T]
//              [--version] [--check] [--gpus G | --ranks G] [--dtype float|bf16] [--phases]
//
//   --size       elements per rank (default 35, like the reference)
//   --repeat     number of timed all-reduces (data is NOT re-initialised between repeats)
//   --comm-type  flextree = GPU ranks over NVLink peer memory, one host thread per GPU in this
//                process; threads = CPU ranks (thread world, host memory); procs = this process is one CPU
//                rank of a process world, started once per rank like an MPI job (FT_RANK / FT_WORLD /
//                FT_SESSION in the environment); nccl = the vendor
//                library's own all-reduce on the same GPUs (the comparison arm, like the reference's
//                "--comm-type mpi", which is accepted as another name for it); libnccl is opened at run
//                time, nothing links against it
//   --to-file    write one time per line to "<tag.>N.len.<w0-w1-+L>.ar_test.<epoch>.txt"
//   --check      closed-form check: data[i] = i*0.1 on every rank, so after R in-place sums every
//                rank must hold i*0.1*N^R (two-sided, relative tolerance)
//   --phases     (flextree, threads) every all-reduce is issued as its two halves, reduce-scatter then
//                all-gather (ft_reduce_scatter / ft_all_gather on GPUs, ft_cpu_phase on threads); with --check everything a rank does not own is overwritten with NaN
//                bit patterns between the two, so the gather has to rebuild it from the owners
// The tree shape comes from FT_TOPO / FT_LONELY exactly as for the library entry point.
// GPU times are CUDA-event intervals, reported as the maximum over ranks; CPU times are
// steady-clock intervals on rank 0 like the reference's MPI_Wtime.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <fstream>
#include <string>
#include <thread>
#include <vector>

#include "../api/flextree_mpi.h"
#include "../planner/config.hpp"
#include "timer.hpp"

namespace {
struct Opts {
  size_t size = 35;
  int repeat = 1, ranks = 0;
  bool to_file = false, check = false, bf16 = false, phases = false;
  std::string comm = "flextree", tag;
};

struct SpinBarrier {
  std::atomic<int> count{0}, gen{0};
  int n;
  explicit SpinBarrier(int n_) : n(n_) {}
  void wait() {
    const int g = gen.load();
    if (count.fetch_add(1) == n - 1) { count.store(0); gen.fetch_add(1); }
    else while (gen.load() == g) std::this_thread::yield();
  }
};

// The five NCCL entry points the comparison arm needs, resolved from libnccl.so.2 at run time.
struct Nccl {
  typedef void* comm_t;
  int (*CommInitAll)(comm_t*, int, const int*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*CommDestroy)(comm_t) = nullptr;
  bool load() {
    void* h = nullptr;
    for (const char* name : {"libnccl.so.2", "libnccl.so"})
      if ((h = dlopen(name, RTLD_NOW | RTLD_GLOBAL))) break;
    if (!h) return false;
    CommInitAll = (decltype(CommInitAll))dlsym(h, "ncclCommInitAll");
    AllReduce = (decltype(AllReduce))dlsym(h, "ncclAllReduce");
    GroupStart = (decltype(GroupStart))dlsym(h, "ncclGroupStart");
    GroupEnd = (decltype(GroupEnd))dlsym(h, "ncclGroupEnd");
    CommDestroy = (decltype(CommDestroy))dlsym(h, "ncclCommDestroy");
    return CommInitAll && AllReduce && GroupStart && GroupEnd && CommDestroy;
  }
};
constexpr int kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0;   // ncclDataType_t / ncclRedOp_t values

unsigned short f2bf(float f) {
  unsigned u;
  memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (unsigned short)(u >> 16);
}
float bf2f(unsigned short h) {
  unsigned u = (unsigned)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
}  // namespace

// --comm-type procs: this process is ONE rank; start as many copies as there are ranks, the way the reference's
// benchmark is started by mpirun, with FT_RANK / FT_WORLD / FT_SESSION (or RANK / WORLD_SIZE / MASTER_PORT) set.
// Host buffers, the process world underneath (no MPI library); rank 0 prints the summary and writes the file.
static int run_as_process_rank(const Opts& o) {
  FT_Comm comm = ft_mpi_proc_init_env(60.0);
  if (!comm) { fprintf(stderr, "%s\n", ft_mpi_last_error()); return 1; }
  int world = 1, rank = 0;
  FT_Comm_size(comm, &world);
  FT_Comm_rank(comm, &rank);
  ft::ShapeConfig cfg = ft::shape_from_env(world);
  if (!cfg.ok()) { if (rank == 0) fprintf(stderr, "%s\n", cfg.error.c_str()); ft_mpi_proc_finalize(comm); return 1; }
  if (rank == 0) {
    FT_enabled();
    printf("configuration:\n  - total_peers: %d\n  - data_size: %zu\n  - repeat: %d\n  - to_file: %s\n  - check_validity: %s\n"
           "  - communication method: procs\n  - And FlexTree topo is %s\n",
           world, o.size, o.repeat, o.to_file ? "true" : "false", o.check ? "true" : "false",
           cfg.is_auto ? "auto" : cfg.shape.str().c_str());
  }
  std::vector<float> data(o.size);
  for (size_t i = 0; i < o.size; ++i) data[i] = (float)i * 0.1f;
  std::vector<double> times;
  int bad = 0;
  for (int i = 0; i < o.repeat; ++i) {
    FT_Barrier(comm);
    ft::Timer t;
    t.Start();
    if (MPI_Allreduce_FT_c(FT_IN_PLACE, data.data(), o.size, FT_FLOAT, FT_OP_SUM, comm) != 0) bad = 2;
    t.Stop();
    times.push_back(t.seconds());
  }
  if (o.check && !bad) {
    const double scale = std::pow((double)world, o.repeat);
    for (size_t i = 0; i < o.size; ++i) {
      const double want = (double)((float)i * 0.1f) * scale;
      if (!(std::fabs(data[i] - want) <= 1e-5 * o.repeat * std::fabs(want) + 1e-6)) {
        bad = 1;
        fprintf(stderr, "node %d says the result seems not right at %zu: %g vs %g\n", rank, i, (double)data[i], want);
        break;
      }
    }
  }
  float failed = bad ? 1.f : 0.f;   // every rank's verdict reaches rank 0
  MPI_Allreduce_FT_c(FT_IN_PLACE, &failed, 1, FT_FLOAT, FT_OP_SUM, comm);
  if (rank == 0) {
    double sum = 0, mn = 1e30;
    for (double t : times) { sum += t; mn = std::min(mn, t); }
    if (o.check) printf("%s\n", failed > 0 ? "CHECK failed" : "CHECK (test passed)");
    if (o.to_file) {
      std::string name;
      if (!o.tag.empty()) name += o.tag + ".";
      name += std::to_string(world) + "." + std::to_string(o.size) + ".";
      if (cfg.shape.ring) name += "ring";
      else for (int w : cfg.shape.widths) name += std::to_string(w) + "-";
      name += "+" + std::to_string(cfg.shape.lonely) + ".ar_test." + std::to_string((long long)time(nullptr)) + ".txt";
      std::ofstream f(name);
      for (double t : times) f << t << std::endl;
      printf("times written to %s\n", name.c_str());
    }
    printf("DONE, average time: %g, min time: %g  (busbw at min: %.2f GB/s)\n", sum / o.repeat, mn,
           (double)o.size * 4 / mn / 1e9 * 2.0 * (world - 1) / world);
  }
  ft_mpi_proc_finalize(comm);
  return failed > 0 ? 2 : 0;
}

int main(int argc, char** argv) {
  setvbuf(stdout, nullptr, _IOLBF, 0);   // a reader on a pipe sees every finished line, whatever happens later
  Opts o;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--size") o.size = strtoull(next(), nullptr, 10);
    else if (a == "--repeat") o.repeat = atoi(next());
    else if (a == "--to-file") o.to_file = true;
    else if (a == "--comm-type") o.comm = next();
    else if (a == "--tag") o.tag = next();
    else if (a == "--check") o.check = true;
    else if (a == "--gpus" || a == "--ranks") o.ranks = atoi(next());
    else if (a == "--dtype") o.bf16 = std::string(next()) == "bf16";
    else if (a == "--phases") o.phases = true;
    else if (a == "--version") { printf("FlexTree Standalone Benchmark\nversion: %s\n", ft_version()); return 0; }
    else { fprintf(stderr, "unknown parameter: %s\n", a.c_str()); return 1; }
  }
  if (o.comm == "procs") return run_as_process_rank(o);
  if (o.comm == "mpi") o.comm = "nccl";   // the reference's name for "the library's own all-reduce"
  const bool use_nccl = o.comm == "nccl";
  const bool gpu = o.comm == "flextree" || use_nccl;
  if (!gpu && o.comm != "threads") { fprintf(stderr, "unknown comm type: %s\n", o.comm.c_str()); return 1; }
  Nccl nccl;
  if (use_nccl && !nccl.load()) { fprintf(stderr, "libnccl.so.2 not found or incomplete\n"); return 1; }
  int world = o.ranks;
  if (gpu) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { fprintf(stderr, "no CUDA device; use --comm-type threads\n"); return 1; }
    if (world <= 0 || world > ndev) world = ndev;
  } else if (world <= 0) {
    world = 4;
  }
  ft::ShapeConfig cfg = ft::shape_from_env(world);
  if (!cfg.ok()) { fprintf(stderr, "%s\n", cfg.error.c_str()); return 1; }
  FT_enabled();
  printf("configuration:\n  - total_peers: %d\n  - data_size: %zu\n  - repeat: %d\n  - to_file: %s\n  - check_validity: %s\n"
         "  - communication method: %s\n  - And FlexTree topo is %s\n",
         world, o.size, o.repeat, o.to_file ? "true" : "false", o.check ? "true" : "false", o.comm.c_str(),
         cfg.is_auto ? "auto" : cfg.shape.str().c_str());

  const size_t es = o.bf16 ? 2 : 4;
  const int dtype = o.bf16 ? FT_BFLOAT16 : FT_FLOAT;
  std::vector<std::vector<double>> times(world, std::vector<double>(o.repeat, 0.0));
  std::vector<int> bad(world, 0);
  SpinBarrier bar(world);
  std::vector<ft_comm*> comms(world, nullptr);
  ft_cpu_world* cpu_world = nullptr;
  std::vector<Nccl::comm_t> ncomms(world, nullptr);
  if (use_nccl) {
    std::vector<int> devs(world);
    for (int r = 0; r < world; ++r) devs[r] = r;
    if (nccl.CommInitAll(ncomms.data(), world, devs.data()) != 0) { fprintf(stderr, "ncclCommInitAll failed\n"); return 1; }
  } else if (gpu) {
    // heaps from the virtual-memory API where the driver offers it (that is what NVLS multicast binds to),
    // else plain cudaMalloc + peer access
    const size_t heap = ((o.size * es + (1 << 20)) + 255) / 256 * 256;
    bool up = false;
    for (int kind : {FT_MEM_VMM, FT_MEM_IPC}) {
      bool ok = true;
      for (int r = 0; r < world && ok; ++r) {
        cudaSetDevice(r);
        ok = ft_comm_create(r, world, r, heap, 1 << 20, kind, &comms[r]) == FT_OK;
        if (!ok && kind == FT_MEM_IPC) fprintf(stderr, "rank %d: %s\n", r, ft_comm_last_error(comms[r]));
      }
      if (ok && ft_comm_connect_local(comms.data(), world) == FT_OK) { up = true; break; }
      if (kind == FT_MEM_IPC && ok) fprintf(stderr, "connect: %s\n", ft_comm_last_error(comms[0]));
      for (auto*& c : comms) { if (c) ft_comm_destroy(c); c = nullptr; }
    }
    if (!up) return 1;
    printf("  - symmetric memory: %s, nvls %s\n", ft_comm_mem_kind(comms[0]) == FT_MEM_VMM ? "vmm" : "ipc",
           ft_comm_has_nvls(comms[0]) ? "on" : "off");
  } else {
    cpu_world = ft_cpu_world_create(world, 60.0);
  }

  std::vector<uint64_t> holders(world, 0);
  if (o.phases) {
    if (use_nccl) { fprintf(stderr, "--phases needs --comm-type flextree or threads\n"); return 1; }
    const ft::Shape& sh = cfg.shape;
    if (ft_plan_rs_holders(world, sh.widths.data(), (int)sh.widths.size(), sh.lonely, sh.ring, holders.data()) != FT_OK) {
      fprintf(stderr, "no plan for %s\n", sh.str().c_str());
      return 1;
    }
  }

  auto rank_main = [&](int r) {
    std::vector<float> host(o.size);
    for (size_t i = 0; i < o.size; ++i) host[i] = (float)i * 0.1f;
    std::vector<unsigned short> host16;
    if (o.bf16) { host16.resize(o.size); for (size_t i = 0; i < o.size; ++i) host16[i] = f2bf(host[i]); }
    void* hostp = o.bf16 ? (void*)host16.data() : (void*)host.data();
    if (gpu) {
      cudaSetDevice(r);
      cudaStream_t st;
      cudaStreamCreate(&st);
      void* dev = nullptr;
      if (use_nccl) cudaMalloc(&dev, o.size * es);
      else dev = ft_comm_alloc(comms[r], o.size * es);
      cudaMemcpy(dev, hostp, o.size * es, cudaMemcpyHostToDevice);
      FT_Comm mc = use_nccl ? nullptr : ft_mpi_from_comm(comms[r], st);
      cudaEvent_t a, b;
      cudaEventCreate(&a); cudaEventCreate(&b);
      for (int i = 0; i < o.repeat; ++i) {
        bar.wait();
        cudaEventRecord(a, st);
        if (use_nccl) {
          if (nccl.AllReduce(dev, dev, o.size, o.bf16 ? kNcclBfloat16 : kNcclFloat32, kNcclSum, ncomms[r], st) != 0) bad[r] = 2;
        } else if (o.phases) {
          // the two halves as calls of their own; with --check everything this rank does not own is
          // overwritten with NaN bit patterns in between, so the gather must rebuild it from the owners
          const ft::Shape& sh = cfg.shape;
          const int nw = (int)sh.widths.size();
          if (ft_reduce_scatter(comms[r], dev, o.size, dtype, FT_SUM, sh.widths.data(), nw, sh.lonely, sh.ring, 1.0f, st) != FT_OK) bad[r] = 2;
          if (o.check && world > 1) {
            const uint64_t B = ft_comm_block_elems(comms[r], o.size, dtype);
            uint64_t lo = o.size, hi = o.size;
            for (int blk = 0; blk < world; ++blk)
              if (holders[blk] >> r & 1) { lo = std::min<uint64_t>(o.size, blk * B); hi = std::min<uint64_t>(o.size, (blk + 1) * B); }
            if (lo) cudaMemsetAsync(dev, 0xFF, lo * es, st);
            if (hi < o.size) cudaMemsetAsync((char*)dev + hi * es, 0xFF, (o.size - hi) * es, st);
          }
          if (ft_all_gather(comms[r], dev, o.size, dtype, sh.widths.data(), nw, sh.lonely, sh.ring, st) != FT_OK) bad[r] = 2;
        } else if (MPI_Allreduce_FT_c(FT_IN_PLACE, dev, o.size, dtype, FT_OP_SUM, mc) != 0) {
          bad[r] = 2;
        }
        cudaEventRecord(b, st);
        cudaEventSynchronize(b);
        float ms = 0;
        cudaEventElapsedTime(&ms, a, b);
        times[r][i] = ms * 1e-3;
      }
      int status[5];
      if (!use_nccl && ft_comm_status(comms[r], status) != FT_OK) bad[r] = 3;
      cudaMemcpy(hostp, dev, o.size * es, cudaMemcpyDeviceToHost);
      if (use_nccl) cudaFree(dev);
      else ft_mpi_comm_free(mc);
      cudaStreamDestroy(st);
    } else {
      FT_Comm mc = ft_mpi_thread_rank(cpu_world, r);
      for (int i = 0; i < o.repeat; ++i) {
        bar.wait();
        ft::Timer t;
        t.Start();
        if (o.phases) {
          const ft::Shape& sh = cfg.shape;
          const int nw = (int)sh.widths.size();
          int st3[3];
          if (ft_cpu_phase(cpu_world, r, sh.widths.data(), nw, sh.lonely, sh.ring, FT_SUM, dtype, hostp, o.size, 0, 1, st3) != FT_OK) bad[r] = 2;
          if (o.check && world > 1) {   // wipe what this rank does not own (host blocks are ceil(size / world) elements)
            const uint64_t B = (o.size + world - 1) / world;
            for (int b = 0; b < world; ++b)
              if (!(holders[b] >> r & 1)) {
                const uint64_t lo = std::min<uint64_t>(o.size, b * B), hi = std::min<uint64_t>(o.size, (b + 1) * B);
                std::memset((char*)hostp + lo * es, 0xFF, (hi - lo) * es);
              }
          }
          if (ft_cpu_phase(cpu_world, r, sh.widths.data(), nw, sh.lonely, sh.ring, FT_SUM, dtype, hostp, o.size, 0, 2, st3) != FT_OK) bad[r] = 2;
        } else if (MPI_Allreduce_FT_c(FT_IN_PLACE, hostp, o.size, dtype, FT_OP_SUM, mc) != 0) {
          bad[r] = 2;
        }
        t.Stop();
        times[r][i] = t.seconds();
      }
      ft_mpi_comm_free(mc);
    }
    if (o.check && !bad[r]) {
      const double scale = std::pow((double)world, o.repeat);
      for (size_t i = 0; i < o.size; ++i) {
        const double got = o.bf16 ? bf2f(host16[i]) : host[i];
        const double want = (o.bf16 ? (double)bf2f(f2bf((float)i * 0.1f)) : (double)((float)i * 0.1f)) * scale;
        const double tol = (o.bf16 ? 2e-2 * o.repeat : 1e-5 * o.repeat) * std::fabs(want) + 1e-6;
        if (!(std::fabs(got - want) <= tol)) { bad[r] = 1; fprintf(stderr, "node %d says the result seems not right at %zu: %g vs %g\n", r, i, got, want); break; }
      }
    }
    bar.wait();
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(rank_main, r);
  for (auto& t : th) t.join();

  std::vector<double> per_repeat(o.repeat, 0.0);
  double sum = 0, mn = 1e30;
  for (int i = 0; i < o.repeat; ++i) {
    for (int r = 0; r < world; ++r) per_repeat[i] = std::max(per_repeat[i], gpu ? times[r][i] : times[0][i]);
    sum += per_repeat[i];
    mn = std::min(mn, per_repeat[i]);
  }
  int failed = 0;
  for (int r = 0; r < world; ++r) failed |= bad[r];
  if (o.check) printf("%s\n", failed ? "CHECK failed" : "CHECK (test passed)");
  if (o.to_file) {
    std::string name;
    if (!o.tag.empty()) name += o.tag + ".";
    name += std::to_string(world) + "." + std::to_string(o.size) + ".";
    if (cfg.shape.ring) name += "ring";
    else for (int w : cfg.shape.widths) name += std::to_string(w) + "-";
    name += "+" + std::to_string(cfg.shape.lonely) + ".ar_test." + std::to_string((long long)time(nullptr)) + ".txt";
    std::ofstream f(name);
    for (double t : per_repeat) f << t << std::endl;
    printf("times written to %s\n", name.c_str());
  }
  const double bytes = (double)o.size * es;
  printf("DONE, average time: %g, min time: %g  (busbw at min: %.2f GB/s)\n", sum / o.repeat, mn,
         bytes / mn / 1e9 * 2.0 * (world - 1) / world);
  for (auto c : ncomms) if (c) nccl.CommDestroy(c);
  for (auto* c : comms) if (c) ft_comm_destroy(c);
  if (cpu_world) ft_cpu_world_destroy(cpu_world);
  return failed ? 2 : 0;
}
