// ft_local_allreduce_noalloc(): the one-shot all-reduce kernel run over a staging area that is a
// file-scope device array instead of communicator heap memory.  See no_alloc_entry.h for who
// needs this and for the rules; nothing like it exists in the reference project.
//
// The array's name is only a stand-in on the host: its device address is fetched once per
// device with cudaGetSymbolAddress (while that device is current) and that pointer is what the
// kernels get.
#include "no_alloc_entry.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "comm_dev.h"
#include "pol_ids.h"

namespace ftk {
cudaError_t launch_oneshot(int pol, const CommDev& c, const OneShotArgs& a, uint64_t slot_bytes, int lanes, cudaStream_t st);
}

namespace {

// Staging space shared by every call on this device (and kept by the device until exit).
static __device__ __align__(256) unsigned char g_noalloc_scratch[FT_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {};
thread_local std::string g_err;

int fail(int code, const std::string& what) {
  g_err = what;
  return code;
}

// Device address of the array on the current device; resolved on the first call per device.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0) return fail(FT_ERR_CUDA, "no current CUDA device");
  if (dev >= kMaxDevices)
    return fail(FT_ERR_TOO_LARGE, "device ordinal " + std::to_string(dev) + " is beyond the " + std::to_string(kMaxDevices) +
                                      " devices this entry point keeps an address for");
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return fail(FT_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = (unsigned char*)p;
  }
  *out = g_scratch_addr[dev];
  return FT_OK;
}

}  // namespace

extern "C" {

const char* ft_noalloc_last_error(void) { return g_err.c_str(); }

int ft_local_allreduce_noalloc(void* const* bufs, int n, size_t count, int dtype, int op, float scale, void* stream) {
  if (op < 0 || op >= FT_OP_COUNT) return fail(FT_ERR_UNSUPPORTED_OP, "Unsupported op " + std::to_string(op));
  const int pol = ftk::policy_id(op, dtype);
  if (pol < 0) return fail(FT_ERR_UNSUPPORTED_TYPE, std::string("Type ") + ft_dtype_name((ft_dtype)dtype) + " is not supported");
  if (!bufs || n < 1 || n > FT_MAX_RANKS) return fail(FT_ERR_INVALID_ARG, "need 1.." + std::to_string(FT_MAX_RANKS) + " buffers");
  if (count == 0) return FT_OK;
  for (int r = 0; r < n; ++r)
    if (!bufs[r]) return fail(FT_ERR_INVALID_ARG, "null buffer");
  const size_t es = ft_dtype_size((ft_dtype)dtype);
  const size_t bytes = count * es;
  const size_t per_rank = (bytes + 255) / 256 * 256;
  if (count > FT_NOALLOC_SCRATCH_BYTES / es || per_rank * (size_t)n > FT_NOALLOC_SCRATCH_BYTES)
    return fail(FT_ERR_TOO_LARGE, "ft_local_allreduce_noalloc: " + std::to_string(n) + " buffers of " + std::to_string(bytes) +
                                      " bytes need " + std::to_string(per_rank * (size_t)n) + " bytes of staging, the built-in area holds " +
                                      std::to_string((size_t)FT_NOALLOC_SCRATCH_BYTES));
  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != FT_OK) return rc;

  cudaStream_t st = (cudaStream_t)stream;
  uint64_t lanes = bytes / 4096;
  if (lanes < 1) lanes = 1;
  if (lanes > 64) lanes = 64;
  // phase 1: every buffer is copied into its own part of the staging area (this overwrites
  // whatever the previous call left there); phase 4: every buffer becomes the sum of all parts.
  // Stream order separates the phases, so the kernels never wait on one another.
  for (int phase : {1, 4}) {
    for (int r = 0; r < n; ++r) {
      ftk::CommDev c{};
      for (int q = 0; q < n; ++q) c.heap[q] = scratch + (size_t)q * per_rank;
      c.rank = r;
      c.world = n;
      ftk::OneShotArgs a{};
      a.slot_off = 0;
      a.emu_call = 0;
      a.user_in = bufs[r];
      a.user_out = bufs[r];
      a.count = count;
      a.elem_size = (uint32_t)es;
      a.phase_mask = (uint32_t)phase;
      a.user_vec_ok = ((uintptr_t)bufs[r] & 15) == 0;
      a.scale = scale;
      cudaError_t e = ftk::launch_oneshot(pol, c, a, 0, (int)lanes, st);
      if (e != cudaSuccess) return fail(FT_ERR_CUDA, std::string("launch: ") + cudaGetErrorString(e));
    }
  }
  return FT_OK;
}

}  // extern "C"
