// Times the reference's own GPU launcher reduce_sum_gpu<float>() (vector_add/reduce_sum_gpu.h,
// included unmodified from the copy under baseline/_ref/src) on this repository's n-way
// benchmark configuration: n in {2,3,4,8} vectors of `elems` floats, launch shape exactly as
// the reference's benchmark uses it (256 threads per block, one element per thread;
// vector_add/vector_add.cu:102-103).  CUDA-event timing, one JSON object on stdout.
#include <cuda_runtime.h>
#include <glog/logging.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "reduce_sum_gpu.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)

int main(int argc, char** argv) {
  const size_t elems = argc > 1 ? strtoull(argv[1], nullptr, 10) : (64ull << 20);
  const int steps = argc > 2 ? atoi(argv[2]) : 10, warmup = argc > 3 ? atoi(argv[3]) : 3;
  const int fanins[4] = {2, 3, 4, 8};
  const int threads = 256;
  const int blocks = (int)((elems + threads - 1) / threads);
  std::vector<float*> dev(8);
  float* host = (float*)malloc(elems * sizeof(float));
  srand(2024);
  for (int k = 0; k < 8; ++k) {
    for (size_t i = 0; i < elems; ++i) host[i] = (float)rand() / RAND_MAX * 2.f - 1.f;
    CK(cudaMalloc(&dev[k], elems * sizeof(float)));
    CK(cudaMemcpy(dev[k], host, elems * sizeof(float), cudaMemcpyHostToDevice));
  }
  float** d_vectors;   // the launcher takes a host array of device pointers
  d_vectors = dev.data();
  float* out[4];
  for (int j = 0; j < 4; ++j) CK(cudaMalloc(&out[j], elems * sizeof(float)));
  auto step = [&]() { for (int j = 0; j < 4; ++j) reduce_sum_gpu<float>((const float**)d_vectors, out[j], fanins[j], elems, blocks, threads); };
  for (int i = 0; i < warmup; ++i) step();
  CK(cudaDeviceSynchronize());
  cudaEvent_t a, b;
  cudaEventCreate(&a); cudaEventCreate(&b);
  cudaEventRecord(a);
  for (int i = 0; i < steps; ++i) step();
  cudaEventRecord(b);
  CK(cudaEventSynchronize(b));
  float ms = 0;
  cudaEventElapsedTime(&ms, a, b);
  double per_fanin[4];
  for (int j = 0; j < 4; ++j) {
    cudaEventRecord(a);
    reduce_sum_gpu<float>((const float**)d_vectors, out[j], fanins[j], elems, blocks, threads);
    cudaEventRecord(b);
    cudaEventSynchronize(b);
    float t; cudaEventElapsedTime(&t, a, b);
    per_fanin[j] = t;
  }
  // End to end, the sequence of the reference's own benchmark (vector_add/vector_add.cu:81-99 copy the inputs in,
  // :113 launch, :136 copy the result out), per step: the 8 inputs from pinned host memory to the device, the four
  // launches, the four results back to pinned host memory.  Pinned memory and asynchronous copies on the
  // launcher's (default) stream are kinder to the reference than its pageable cudaMemcpy calls.
  const int e2e_steps = steps < 2 ? 2 : (steps > 4 ? 4 : steps);
  double e2e_ms = -1;
  {
    std::vector<float*> hin(8, nullptr), hout(4, nullptr);
    bool ok = true;
    for (int k = 0; k < 8 && ok; ++k) ok = cudaHostAlloc(&hin[k], elems * sizeof(float), cudaHostAllocDefault) == cudaSuccess;
    for (int j = 0; j < 4 && ok; ++j) ok = cudaHostAlloc(&hout[j], elems * sizeof(float), cudaHostAllocDefault) == cudaSuccess;
    if (ok) {
      for (int k = 0; k < 8; ++k) CK(cudaMemcpy(hin[k], dev[k], elems * sizeof(float), cudaMemcpyDeviceToHost));
      auto e2e_step = [&]() {
        for (int k = 0; k < 8; ++k) cudaMemcpyAsync(dev[k], hin[k], elems * sizeof(float), cudaMemcpyHostToDevice, 0);
        step();
        for (int j = 0; j < 4; ++j) cudaMemcpyAsync(hout[j], out[j], elems * sizeof(float), cudaMemcpyDeviceToHost, 0);
      };
      e2e_step();
      CK(cudaDeviceSynchronize());
      cudaEventRecord(a);
      for (int i = 0; i < e2e_steps; ++i) e2e_step();
      cudaEventRecord(b);
      CK(cudaEventSynchronize(b));
      float t = 0;
      cudaEventElapsedTime(&t, a, b);
      e2e_ms = t / e2e_steps;
    } else {
      cudaGetLastError();
    }
    for (float* p : hin) if (p) cudaFreeHost(p);
    for (float* p : hout) if (p) cudaFreeHost(p);
  }
  // spot check of n = 4 against the host
  std::vector<float> res(1024), v(1024);
  CK(cudaMemcpy(res.data(), out[2], 1024 * sizeof(float), cudaMemcpyDeviceToHost));
  std::vector<float> acc(1024, 0.f);
  for (int k = 0; k < 4; ++k) { CK(cudaMemcpy(v.data(), dev[k], 1024 * sizeof(float), cudaMemcpyDeviceToHost)); for (int i = 0; i < 1024; ++i) acc[i] += v[i]; }
  double err = 0;
  for (int i = 0; i < 1024; ++i) { double d = res[i] - acc[i]; if (d < 0) d = -d; if (d > err) err = d; }
  printf("{\"ms_per_step\": %.5f, \"per_fanin_ms\": [%.5f, %.5f, %.5f, %.5f], \"max_abs_err\": %.3g, \"elems\": %zu, \"steps\": %d, "
         "\"e2e_ms_per_step\": %.4f, \"e2e_steps\": %d, \"e2e_h2d_bytes\": %zu, \"e2e_d2h_bytes\": %zu}\n",
         ms / steps, per_fanin[0], per_fanin[1], per_fanin[2], per_fanin[3], err, elems, steps, e2e_ms, e2e_steps,
         8 * elems * sizeof(float), 4 * elems * sizeof(float));
  return err < 1e-4 ? 0 : 3;
}
