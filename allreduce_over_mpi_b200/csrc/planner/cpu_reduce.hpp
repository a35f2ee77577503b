// Host n-way element-wise reductions: dst[i] = src[0][i] (op) src[1][i] (op) ... .
//
// These are the oracle for the GPU kernels and the timed CPU baseline.  They cover
// the reference's CPU kernels reduce_sum<T> / reduce_band<T>
// (allreduce_over_mpi/mpi_mod.hpp:812-1031, :1033-1251; vector_add/reduce_sum.h) and
// its (op, datatype) dispatcher handle_reduce (mpi_mod.hpp:1363-1412).
//
// Differences by design: the fan-in is a run-time loop over a cache-sized tile rather
// than twenty hand-unrolled cases; 16-bit floats are accumulated in fp32 and rounded
// once; bool SUM saturates to true (what `bool + bool` converted back to bool gives).
// Native types are added left to right in their own type, like the reference.
#pragma once
#include <cstdint>
#include <cstring>

#include "../api/ft_types.h"

namespace ft {

struct bf16_t { uint16_t bits; };
struct f16_t { uint16_t bits; };

inline float bf16_to_float(bf16_t h) {
  uint32_t u = (uint32_t)h.bits << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline bf16_t float_to_bf16(float f) {  // round to nearest even, NaN preserved
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return bf16_t{(uint16_t)((u >> 16) | 0x40)};
  u += 0x7fffu + ((u >> 16) & 1u);
  return bf16_t{(uint16_t)(u >> 16)};
}
inline float f16_to_float(f16_t h) {
  _Float16 x;
  std::memcpy(&x, &h.bits, 2);
  return (float)x;
}
inline f16_t float_to_f16(float f) {
  _Float16 x = (_Float16)f;
  f16_t h;
  std::memcpy(&h.bits, &x, 2);
  return h;
}

template <typename T> struct Acc { using type = T; static T load(T v) { return v; } static T store(T v) { return v; } };
template <> struct Acc<bf16_t> { using type = float; static float load(bf16_t v) { return bf16_to_float(v); } static bf16_t store(float v) { return float_to_bf16(v); } };
template <> struct Acc<f16_t> { using type = float; static float load(f16_t v) { return f16_to_float(v); } static f16_t store(float v) { return float_to_f16(v); } };

struct OpSum { template <typename A> static A apply(A a, A b) { return (A)(a + b); } };
struct OpBand { template <typename A> static A apply(A a, A b) { return (A)(a & b); } };
template <> inline bool OpSum::apply<bool>(bool a, bool b) { return a || b; }

// n = 0 leaves dst untouched; n = 1 is a copy.  `threads` <= 0 keeps the OpenMP default.
template <typename T, typename Op>
void reduce_nway_cpu(const T* const* src, T* dst, int n, size_t len, int threads = 0) {
  if (n <= 0 || len == 0) return;
  using A = typename Acc<T>::type;
  constexpr size_t kTile = 2048;
  const long ntiles = (long)((len + kTile - 1) / kTile);
  (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) if (len > (1u << 16)) num_threads(threads > 0 ? threads : 14)
#endif
  for (long t = 0; t < ntiles; ++t) {
    const size_t lo = (size_t)t * kTile;
    const size_t m = (len - lo < kTile) ? len - lo : kTile;
    A acc[kTile];
    const T* s0 = src[0] + lo;
    for (size_t i = 0; i < m; ++i) acc[i] = Acc<T>::load(s0[i]);
    for (int k = 1; k < n; ++k) {
      const T* sk = src[k] + lo;
      for (size_t i = 0; i < m; ++i) acc[i] = Op::template apply<A>(acc[i], Acc<T>::load(sk[i]));
    }
    T* d = dst + lo;
    for (size_t i = 0; i < m; ++i) d[i] = Acc<T>::store(acc[i]);
  }
}

// Type-erased entry.  Returns FT_ERR_UNSUPPORTED_TYPE / _OP for pairs without a kernel
// (the reference prints "Type ... is not supported" / "Unsupported op" and exits).
inline ft_status reduce_nway_cpu_dispatch(ft_op op, ft_dtype t, const void* const* src, void* dst, int n,
                                          size_t len, int threads = 0) {
  if ((int)op < 0 || op >= FT_OP_COUNT) return FT_ERR_UNSUPPORTED_OP;
  if (!ft_op_supported(op, t)) return FT_ERR_UNSUPPORTED_TYPE;
  if (n > FT_MAX_FANIN) return FT_ERR_TOO_LARGE;
#define FT_CASE(E, T)                                                                              \
  case E:                                                                                          \
    if (op == FT_SUM) reduce_nway_cpu<T, OpSum>((const T* const*)src, (T*)dst, n, len, threads);   \
    else reduce_nway_cpu<T, OpBand>((const T* const*)src, (T*)dst, n, len, threads);               \
    return FT_OK;
#define FT_CASE_SUM(E, T)                                                                          \
  case E:                                                                                          \
    reduce_nway_cpu<T, OpSum>((const T* const*)src, (T*)dst, n, len, threads);                     \
    return FT_OK;
  switch (t) {
    FT_CASE(FT_U8, uint8_t) FT_CASE(FT_I8, int8_t) FT_CASE(FT_U16, uint16_t) FT_CASE(FT_I16, int16_t)
    FT_CASE(FT_I32, int32_t) FT_CASE(FT_I64, int64_t) FT_CASE(FT_U32, uint32_t) FT_CASE(FT_U64, uint64_t)
    FT_CASE_SUM(FT_F32, float) FT_CASE_SUM(FT_F64, double) FT_CASE_SUM(FT_BOOL, bool)
    FT_CASE_SUM(FT_BF16, bf16_t) FT_CASE_SUM(FT_F16, f16_t)
    default: return FT_ERR_UNSUPPORTED_TYPE;
  }
#undef FT_CASE
#undef FT_CASE_SUM
}

}  // namespace ft
