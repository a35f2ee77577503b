// reduce_bench: n-way reduce-sum on the GPU against the multi-threaded CPU reduction.
//
//     reduce_bench [--elements E] [--rounds R] [--max-width W] [--min-width w] [--variant 0|1|2]
//                  [--cpu-threads T] [--cpu-only] [--json]
//
// For every fan-in n in [min-width, max-width] it fills n vectors of E floats with uniform
// [0,1) values, sums them element-wise on the device (ft_reduce_nway) and on the host
// (ft_cpu_reduce), compares the two results and accumulates both times over R rounds.
// It ends like the program it stands in for (vector_add/vector_add.cu:50-204): one line of
// average GPU milliseconds per fan-in, one line of average CPU milliseconds.  Differences:
// the device time is taken with CUDA events after a warm-up launch instead of a host
// stopwatch around the first launch, bandwidth is printed beside it, the element count is
// a flag (the reference hard-codes 150e6, 10 rounds, widths 1..16), and without a CUDA
// device (or with --cpu-only) only the host side runs.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "api/flextree.h"
#include "tools/timer.hpp"

namespace {

struct Opts {
  size_t elements = 16u << 20;
  int rounds = 3, max_width = 16, min_width = 1, variant = 0, cpu_threads = 0;
  bool cpu_only = false, json = false;
};

#define CUDA_OK(call)                                                                      \
  do {                                                                                     \
    cudaError_t e_ = (call);                                                               \
    if (e_ != cudaSuccess) {                                                               \
      fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_));                   \
      return 1;                                                                            \
    }                                                                                      \
  } while (0)

void usage() {
  fprintf(stderr,
          "usage: reduce_bench [--elements E] [--rounds R] [--max-width W] [--min-width w]\n"
          "                    [--variant 0|1|2] [--cpu-threads T] [--cpu-only] [--json]\n");
}

}  // namespace

int main(int argc, char** argv) {
  Opts o;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> const char* {
      if (i + 1 >= argc) { usage(); exit(2); }
      return argv[++i];
    };
    if (a == "--elements") o.elements = (size_t)strtod(next(), nullptr);
    else if (a == "--rounds") o.rounds = atoi(next());
    else if (a == "--max-width") o.max_width = atoi(next());
    else if (a == "--min-width") o.min_width = atoi(next());
    else if (a == "--variant") o.variant = atoi(next());
    else if (a == "--cpu-threads") o.cpu_threads = atoi(next());
    else if (a == "--cpu-only") o.cpu_only = true;
    else if (a == "--json") o.json = true;
    else { usage(); return 2; }
  }
  if (o.elements == 0 || o.rounds < 1 || o.min_width < 1 || o.max_width < o.min_width || o.max_width > FT_MAX_FANIN) {
    fprintf(stderr, "need elements > 0, rounds >= 1, 1 <= min-width <= max-width <= %d\n", FT_MAX_FANIN);
    return 2;
  }
  bool gpu = !o.cpu_only;
  if (gpu) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
      fprintf(stderr, "no CUDA device: timing the host reduction only\n");
      gpu = false;
    }
  }
  const size_t E = o.elements, bytes = E * sizeof(float);
  const int W = o.max_width;

  // one set of inputs, filled once; fan-in n uses the first n vectors
  std::vector<std::vector<float>> h(W, std::vector<float>(E));
  {
    std::mt19937 rng(12345);
    std::uniform_real_distribution<float> u(0.f, 1.f);
    for (int j = 0; j < W; ++j)
      for (size_t i = 0; i < E; ++i) h[j][i] = u(rng);
  }
  std::vector<float> h_cpu(E), h_gpu(E);
  std::vector<const void*> hp(W);
  for (int j = 0; j < W; ++j) hp[j] = h[j].data();

  std::vector<void*> d(W, nullptr);
  void* d_out = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (gpu) {
    for (int j = 0; j < W; ++j) {
      CUDA_OK(cudaMalloc(&d[j], bytes));
      CUDA_OK(cudaMemcpy(d[j], h[j].data(), bytes, cudaMemcpyHostToDevice));
    }
    CUDA_OK(cudaMalloc(&d_out, bytes));
    CUDA_OK(cudaEventCreate(&e0));
    CUDA_OK(cudaEventCreate(&e1));
  }

  std::vector<double> gpu_ms(W + 1, 0.0), cpu_ms(W + 1, 0.0);
  for (int r = 0; r < o.rounds; ++r) {
    for (int n = o.min_width; n <= W; ++n) {
      if (gpu) {
        std::vector<const void*> dp(d.begin(), d.begin() + n);
        int st = ft_reduce_nway(FT_SUM, FT_F32, dp.data(), d_out, n, E, o.variant, nullptr);  // warm-up
        if (st != FT_OK) { fprintf(stderr, "ft_reduce_nway: status %d (%s)\n", st, ft_last_cuda_error()); return 1; }
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaEventRecord(e0));
        st = ft_reduce_nway(FT_SUM, FT_F32, dp.data(), d_out, n, E, o.variant, nullptr);
        CUDA_OK(cudaEventRecord(e1));
        CUDA_OK(cudaEventSynchronize(e1));
        if (st != FT_OK) { fprintf(stderr, "ft_reduce_nway: status %d (%s)\n", st, ft_last_cuda_error()); return 1; }
        float ms = 0;
        CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
        gpu_ms[n] += ms;
      }
      {
        ft::Timer t;
        t.Start();
        int st = ft_cpu_reduce(FT_SUM, FT_F32, hp.data(), h_cpu.data(), n, E, o.cpu_threads);
        t.Stop();
        if (st != FT_OK) { fprintf(stderr, "ft_cpu_reduce: status %d\n", st); return 1; }
        cpu_ms[n] += t.seconds() * 1e3;
      }
      if (gpu) {
        CUDA_OK(cudaMemcpy(h_gpu.data(), d_out, bytes, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < E; ++i) {
          const float tol = 1e-5f * std::fmax(1.f, std::fabs(h_cpu[i]));
          if (std::fabs(h_cpu[i] - h_gpu[i]) > tol) {
            fprintf(stderr, "Result verification failed at element %zu (fan-in %d)\nCPU: %g, GPU: %g\n", i, n,
                    h_cpu[i], h_gpu[i]);
            return 1;
          }
        }
      }
    }
  }
  for (int n = o.min_width; n <= W; ++n) {
    gpu_ms[n] /= o.rounds;
    cpu_ms[n] /= o.rounds;
    const double moved = (double)(n + 1) * bytes;
    if (o.json) {
      printf("{\"bench\": \"reduce_nway\", \"n\": %d, \"elements\": %zu, \"dtype\": \"float32\", \"cpu_ms\": %.4f, "
             "\"cpu_gbs\": %.2f",
             n, E, cpu_ms[n], moved / cpu_ms[n] * 1e-6);
      if (gpu) printf(", \"gpu_ms\": %.4f, \"gpu_gbs\": %.1f", gpu_ms[n], moved / gpu_ms[n] * 1e-6);
      printf("}\n");
    } else {
      printf("n=%2d  %zu floats", n, E);
      if (gpu) printf("  GPU %9.4f ms %8.1f GB/s", gpu_ms[n], moved / gpu_ms[n] * 1e-6);
      printf("  CPU %9.3f ms %7.2f GB/s\n", cpu_ms[n], moved / cpu_ms[n] * 1e-6);
    }
  }
  if (gpu) printf("Test PASSED\n");
  if (!o.json) {
    // the closing two lines of the original program: average milliseconds per fan-in, GPU then CPU
    if (gpu) {
      for (int n = o.min_width; n <= W; ++n) printf("%.3f ", gpu_ms[n]);
      printf("\n");
    }
    for (int n = o.min_width; n <= W; ++n) printf("%.3f ", cpu_ms[n]);
    printf("\n");
  }
  if (gpu) {
    for (int j = 0; j < W; ++j) cudaFree(d[j]);
    cudaFree(d_out);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  return 0;
}
