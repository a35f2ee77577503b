// Argument block of the single-GPU n-way reduction kernels (reduce_nway.cu, reduce_nway_wide.cu).
#pragma once
#include <cuda_runtime.h>

#include "../api/ft_types.h"

namespace ftk {

struct NwayArgs {
  const void* src[FT_MAX_FANIN];
  void* dst;
  unsigned long long nvec;   // 16-byte vectors
  unsigned long long nunit;  // scalar units (see ScalarOp) for the scalar kernel
  int n;
};

// 32-byte-per-access kernels (reduce_nway_wide.cu).  `code` selects a configuration (0: the default;
// see launch_cfg there); returns cudaErrorInvalidValue when (policy, fan-in, code) has no
// instantiation, in which case the caller falls back to the 16-byte kernels.
cudaError_t launch_wide(int pol, const NwayArgs& a, unsigned long long n32, int code, int sms, cudaStream_t st);

}  // namespace ftk
