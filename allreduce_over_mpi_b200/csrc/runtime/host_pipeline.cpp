// n-way reductions whose operands and results live in host memory, streamed through one GPU.
//
// The reference's GPU experiment does this in three serial steps: copy every input to the device,
// run the kernel, copy the result back (vector_add/vector_add.cu:81-99, :113, :136).  On a PCIe
// link that carries traffic in both directions at once, that leaves half of the link idle at any
// time.  Here the vectors are cut into chunks that rotate through a small ring of device buffers on
// three streams: while chunk k is being reduced, chunk k+1 arrives and the results of chunk k-1
// leave, so a step costs about max(bytes in, bytes out) / link rate instead of their sum.
#include <cuda_runtime.h>

#include <cstring>
#include <string>
#include <vector>

#include "../api/flextree.h"

struct ft_host_pipe {
  static constexpr int kDepth = 3;
  int device = 0, max_in = 0, max_out = 0;
  size_t chunk_bytes = 0;
  cudaStream_t in = nullptr, run = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, in_done[kDepth] = {}, run_done[kDepth] = {}, out_done[kDepth] = {};
  bool used[kDepth] = {};
  unsigned char* mem = nullptr;   // kDepth x (max_in + max_out) chunks
  std::string err;
  unsigned char* in_buf(int slot, int k) const { return mem + ((size_t)slot * (max_in + max_out) + k) * chunk_bytes; }
  unsigned char* out_buf(int slot, int j) const { return mem + ((size_t)slot * (max_in + max_out) + max_in + j) * chunk_bytes; }
};

namespace {
int fail(ft_host_pipe* p, int code, const std::string& what) {
  if (p) p->err = what;
  return code;
}
#define HP_CUDA(p, call)                                                                              \
  do {                                                                                                \
    cudaError_t e_ = (call);                                                                          \
    if (e_ != cudaSuccess) return fail(p, FT_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
  } while (0)
}  // namespace

extern "C" {

int ft_host_pipe_create(int device, size_t chunk_bytes, int max_in, int max_out, ft_host_pipe** out) {
  if (!out || max_in < 1 || max_in > FT_MAX_FANIN || max_out < 1 || max_out > FT_MAX_FANIN || chunk_bytes < 4096) return FT_ERR_INVALID_ARG;
  ft_host_pipe* p = new ft_host_pipe;
  *out = p;
  p->device = device;
  p->max_in = max_in;
  p->max_out = max_out;
  p->chunk_bytes = chunk_bytes / 4096 * 4096;
  HP_CUDA(p, cudaSetDevice(device));
  HP_CUDA(p, cudaMalloc(&p->mem, (size_t)ft_host_pipe::kDepth * (max_in + max_out) * p->chunk_bytes));
  HP_CUDA(p, cudaStreamCreateWithFlags(&p->in, cudaStreamNonBlocking));
  HP_CUDA(p, cudaStreamCreateWithFlags(&p->run, cudaStreamNonBlocking));
  HP_CUDA(p, cudaStreamCreateWithFlags(&p->out, cudaStreamNonBlocking));
  HP_CUDA(p, cudaEventCreateWithFlags(&p->start, cudaEventDisableTiming));
  for (int k = 0; k < ft_host_pipe::kDepth; ++k) {
    HP_CUDA(p, cudaEventCreateWithFlags(&p->in_done[k], cudaEventDisableTiming));
    HP_CUDA(p, cudaEventCreateWithFlags(&p->run_done[k], cudaEventDisableTiming));
    HP_CUDA(p, cudaEventCreateWithFlags(&p->out_done[k], cudaEventDisableTiming));
  }
  return FT_OK;
}

void ft_host_pipe_destroy(ft_host_pipe* p) {
  if (!p) return;
  cudaSetDevice(p->device);
  if (p->out) cudaStreamSynchronize(p->out);
  if (p->in) cudaStreamDestroy(p->in);
  if (p->run) cudaStreamDestroy(p->run);
  if (p->out) cudaStreamDestroy(p->out);
  if (p->start) cudaEventDestroy(p->start);
  for (int k = 0; k < ft_host_pipe::kDepth; ++k) {
    if (p->in_done[k]) cudaEventDestroy(p->in_done[k]);
    if (p->run_done[k]) cudaEventDestroy(p->run_done[k]);
    if (p->out_done[k]) cudaEventDestroy(p->out_done[k]);
  }
  cudaFree(p->mem);
  delete p;
}

const char* ft_host_pipe_last_error(ft_host_pipe* p) { return p ? p->err.c_str() : "null pipeline"; }

int ft_host_pipe_reduce(ft_host_pipe* p, int op, int dtype, const void* const* host_src, int n_in, const int* fanin,
                        void* const* host_dst, int n_out, size_t len, void* stream) {
  if (!p || !host_src || !host_dst || !fanin) return FT_ERR_INVALID_ARG;
  if (n_in < 1 || n_in > p->max_in || n_out < 1 || n_out > p->max_out) return fail(p, FT_ERR_INVALID_ARG, "more vectors than the pipeline was built for");
  const size_t es = ft_dtype_size((ft_dtype)dtype);
  if (!es) return fail(p, FT_ERR_UNSUPPORTED_TYPE, "unknown element type");
  for (int j = 0; j < n_out; ++j)
    if (fanin[j] < 1 || fanin[j] > n_in) return fail(p, FT_ERR_INVALID_ARG, "fan-in outside 1..n_in");
  if (len == 0) return FT_OK;
  HP_CUDA(p, cudaSetDevice(p->device));
  constexpr int D = ft_host_pipe::kDepth;
  const size_t per = p->chunk_bytes / es;
  cudaStream_t user = (cudaStream_t)stream;
  HP_CUDA(p, cudaEventRecord(p->start, user));
  HP_CUDA(p, cudaStreamWaitEvent(p->in, p->start, 0));
  int s = 0;
  for (size_t lo = 0; lo < len; lo += per, s = (s + 1) % D) {
    const size_t n = len - lo < per ? len - lo : per;
    // the slot's inputs are free once its previous reductions ran; its outputs once they were copied out
    if (p->used[s]) HP_CUDA(p, cudaStreamWaitEvent(p->in, p->run_done[s], 0));
    for (int k = 0; k < n_in; ++k)
      HP_CUDA(p, cudaMemcpyAsync(p->in_buf(s, k), (const unsigned char*)host_src[k] + lo * es, n * es, cudaMemcpyHostToDevice, p->in));
    HP_CUDA(p, cudaEventRecord(p->in_done[s], p->in));
    HP_CUDA(p, cudaStreamWaitEvent(p->run, p->in_done[s], 0));
    if (p->used[s]) HP_CUDA(p, cudaStreamWaitEvent(p->run, p->out_done[s], 0));
    const void* src[FT_MAX_FANIN];
    for (int k = 0; k < n_in; ++k) src[k] = p->in_buf(s, k);
    for (int j = 0; j < n_out; ++j) {
      const int rc = ft_reduce_nway(op, dtype, src, p->out_buf(s, j), fanin[j], n, 0, p->run);
      if (rc != FT_OK) return fail(p, rc, ft_last_cuda_error());
    }
    HP_CUDA(p, cudaEventRecord(p->run_done[s], p->run));
    HP_CUDA(p, cudaStreamWaitEvent(p->out, p->run_done[s], 0));
    for (int j = 0; j < n_out; ++j)
      HP_CUDA(p, cudaMemcpyAsync((unsigned char*)host_dst[j] + lo * es, p->out_buf(s, j), n * es, cudaMemcpyDeviceToHost, p->out));
    HP_CUDA(p, cudaEventRecord(p->out_done[s], p->out));
    p->used[s] = true;
  }
  for (int k = 0; k < D; ++k)
    if (p->used[k]) HP_CUDA(p, cudaStreamWaitEvent(user, p->out_done[k], 0));
  return FT_OK;
}

}  // extern "C"
