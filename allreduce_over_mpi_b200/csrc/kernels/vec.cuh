// 16-byte vector primitives and per-type reduction policies shared by the single-GPU
// n-way reduction and the multi-GPU pull-reduce kernels (sm_100a).
//
// All data loads go through inline PTX so that the compiler never turns a load of
// memory that another GPU (or an earlier stage of the same kernel) writes into a
// non-coherent `ld.global.nc`.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api/ft_types.h"
#include "pol_ids.h"

namespace ftk {

// ---- loads / stores -----------------------------------------------------------------
// Read-only input streamed once from local HBM (single-GPU kernels).
__device__ __forceinline__ uint4 ld_nc(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Coherent streaming load: local or peer memory that is rewritten between rendezvous.
// Not cached in L1, so a later stage can never see a stale line.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_vec(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_vec_cs(void* p, uint4 v) {  // evict-first: written once, not re-read by this kernel
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Store the first `nbytes` (< 16, a multiple of `es`) bytes of v with element-sized stores.
__device__ __forceinline__ void st_partial(void* p, uint4 v, uint32_t nbytes, uint32_t es) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  unsigned char* d = (unsigned char*)p;
  for (uint32_t b = 0; b < nbytes; b += es) {
    if (es == 8) { ((volatile uint32_t*)(d + b))[0] = w[b / 4]; ((volatile uint32_t*)(d + b))[1] = w[b / 4 + 1]; }
    else if (es == 4) *(volatile uint32_t*)(d + b) = w[b / 4];
    else if (es == 2) *(volatile uint16_t*)(d + b) = (uint16_t)(w[b / 4] >> ((b & 2) * 8));
    else *(volatile uint8_t*)(d + b) = (uint8_t)(w[b / 4] >> ((b & 3) * 8));
  }
}
// Gather `nbytes` (<= 16) from an address that is only element-aligned.
__device__ __forceinline__ uint4 ld_partial(const void* p, uint32_t nbytes, uint32_t es) {
  uint32_t w[4] = {0, 0, 0, 0};
  const unsigned char* s = (const unsigned char*)p;
  for (uint32_t b = 0; b < nbytes; b += es) {
    if (es == 8) { w[b / 4] = ((const volatile uint32_t*)(s + b))[0]; w[b / 4 + 1] = ((const volatile uint32_t*)(s + b))[1]; }
    else if (es == 4) w[b / 4] = *(const volatile uint32_t*)(s + b);
    else if (es == 2) w[b / 4] |= (uint32_t)(*(const volatile uint16_t*)(s + b)) << ((b & 2) * 8);
    else w[b / 4] |= (uint32_t)(*(const volatile uint8_t*)(s + b)) << ((b & 3) * 8);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- element types --------------------------------------------------------------------
template <int DT> struct ElemOf;
template <> struct ElemOf<FT_U8> { using type = uint8_t; };
template <> struct ElemOf<FT_I8> { using type = int8_t; };
template <> struct ElemOf<FT_U16> { using type = uint16_t; };
template <> struct ElemOf<FT_I16> { using type = int16_t; };
template <> struct ElemOf<FT_I32> { using type = int32_t; };
template <> struct ElemOf<FT_I64> { using type = long long; };
template <> struct ElemOf<FT_F32> { using type = float; };
template <> struct ElemOf<FT_F64> { using type = double; };
template <> struct ElemOf<FT_BOOL> { using type = uint8_t; };
template <> struct ElemOf<FT_U32> { using type = uint32_t; };
template <> struct ElemOf<FT_U64> { using type = unsigned long long; };
template <> struct ElemOf<FT_BF16> { using type = __nv_bfloat16; };
template <> struct ElemOf<FT_F16> { using type = __half; };

// ---- vector policies ------------------------------------------------------------------
// A policy reduces 16-byte vectors: Acc holds the running value of one vector,
// init() starts it from the first source, add() folds another source in, fin() packs
// the result.  Floating 16-bit types widen to fp32 in Acc and round once in fin().

struct PolWordsBase {
  struct Acc { uint4 v; };
  __device__ static __forceinline__ void init(Acc& a, uint4 v) { a.v = v; }
  __device__ static __forceinline__ uint4 fin(const Acc& a) { return a.v; }
  // integer / bitwise results are never scaled
  __device__ static __forceinline__ uint4 fins(const Acc& a, float) { return a.v; }
};
#define FT_WORD_POLICY(NAME, EXPR)                                              \
  struct NAME : PolWordsBase {                                                  \
    __device__ static __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return EXPR; } \
    __device__ static __forceinline__ void add(Acc& a, uint4 v) {               \
      a.v.x = f(a.v.x, v.x); a.v.y = f(a.v.y, v.y); a.v.z = f(a.v.z, v.z); a.v.w = f(a.v.w, v.w); \
    }                                                                           \
  };
FT_WORD_POLICY(PolAdd32, a + b)
FT_WORD_POLICY(PolAdd16, __vadd2(a, b))
FT_WORD_POLICY(PolAdd8, __vadd4(a, b))
FT_WORD_POLICY(PolOr, a | b)
FT_WORD_POLICY(PolAnd, a & b)
#undef FT_WORD_POLICY

struct PolAdd64 : PolWordsBase {
  __device__ static __forceinline__ void add(Acc& a, uint4 v) {
    unsigned long long lo = ((unsigned long long)a.v.y << 32 | a.v.x) + ((unsigned long long)v.y << 32 | v.x);
    unsigned long long hi = ((unsigned long long)a.v.w << 32 | a.v.z) + ((unsigned long long)v.w << 32 | v.z);
    a.v.x = (uint32_t)lo; a.v.y = (uint32_t)(lo >> 32); a.v.z = (uint32_t)hi; a.v.w = (uint32_t)(hi >> 32);
  }
};
struct PolF64 {
  struct Acc { double a, b; };
  __device__ static __forceinline__ void init(Acc& s, uint4 v) {
    s.a = __hiloint2double((int)v.y, (int)v.x); s.b = __hiloint2double((int)v.w, (int)v.z);
  }
  __device__ static __forceinline__ void add(Acc& s, uint4 v) {
    s.a += __hiloint2double((int)v.y, (int)v.x); s.b += __hiloint2double((int)v.w, (int)v.z);
  }
  __device__ static __forceinline__ uint4 fin(const Acc& s) {
    return make_uint4((uint32_t)__double2loint(s.a), (uint32_t)__double2hiint(s.a), (uint32_t)__double2loint(s.b), (uint32_t)__double2hiint(s.b));
  }
  __device__ static __forceinline__ uint4 fins(const Acc& s, float k) { Acc t{s.a * (double)k, s.b * (double)k}; return fin(t); }
};
struct PolF32 {
  struct Acc { float f[4]; };
  __device__ static __forceinline__ void init(Acc& s, uint4 v) {
    s.f[0] = __uint_as_float(v.x); s.f[1] = __uint_as_float(v.y); s.f[2] = __uint_as_float(v.z); s.f[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ void add(Acc& s, uint4 v) {
    s.f[0] += __uint_as_float(v.x); s.f[1] += __uint_as_float(v.y); s.f[2] += __uint_as_float(v.z); s.f[3] += __uint_as_float(v.w);
  }
  __device__ static __forceinline__ uint4 fin(const Acc& s) {
    return make_uint4(__float_as_uint(s.f[0]), __float_as_uint(s.f[1]), __float_as_uint(s.f[2]), __float_as_uint(s.f[3]));
  }
  __device__ static __forceinline__ uint4 fins(const Acc& s, float k) {
    return make_uint4(__float_as_uint(s.f[0] * k), __float_as_uint(s.f[1] * k), __float_as_uint(s.f[2] * k), __float_as_uint(s.f[3] * k));
  }
};
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
struct PolBF16 {
  struct Acc { float f[8]; };
  __device__ static __forceinline__ void init(Acc& s, uint4 v) {
    s.f[0] = bf_lo(v.x); s.f[1] = bf_hi(v.x); s.f[2] = bf_lo(v.y); s.f[3] = bf_hi(v.y);
    s.f[4] = bf_lo(v.z); s.f[5] = bf_hi(v.z); s.f[6] = bf_lo(v.w); s.f[7] = bf_hi(v.w);
  }
  __device__ static __forceinline__ void add(Acc& s, uint4 v) {
    s.f[0] += bf_lo(v.x); s.f[1] += bf_hi(v.x); s.f[2] += bf_lo(v.y); s.f[3] += bf_hi(v.y);
    s.f[4] += bf_lo(v.z); s.f[5] += bf_hi(v.z); s.f[6] += bf_lo(v.w); s.f[7] += bf_hi(v.w);
  }
  __device__ static __forceinline__ uint4 fin(const Acc& s) {
    return make_uint4(pack_bf16x2(s.f[0], s.f[1]), pack_bf16x2(s.f[2], s.f[3]), pack_bf16x2(s.f[4], s.f[5]), pack_bf16x2(s.f[6], s.f[7]));
  }
  __device__ static __forceinline__ uint4 fins(const Acc& s, float k) {
    return make_uint4(pack_bf16x2(s.f[0] * k, s.f[1] * k), pack_bf16x2(s.f[2] * k, s.f[3] * k), pack_bf16x2(s.f[4] * k, s.f[5] * k), pack_bf16x2(s.f[6] * k, s.f[7] * k));
  }
};
__device__ __forceinline__ float2 h2f(uint32_t w) {
  __half2 h;
  *reinterpret_cast<uint32_t*>(&h) = w;
  return __half22float2(h);
}
__device__ __forceinline__ uint32_t f2h(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
struct PolF16 {
  struct Acc { float f[8]; };
  __device__ static __forceinline__ void init(Acc& s, uint4 v) {
    float2 a = h2f(v.x), b = h2f(v.y), c = h2f(v.z), d = h2f(v.w);
    s.f[0] = a.x; s.f[1] = a.y; s.f[2] = b.x; s.f[3] = b.y; s.f[4] = c.x; s.f[5] = c.y; s.f[6] = d.x; s.f[7] = d.y;
  }
  __device__ static __forceinline__ void add(Acc& s, uint4 v) {
    float2 a = h2f(v.x), b = h2f(v.y), c = h2f(v.z), d = h2f(v.w);
    s.f[0] += a.x; s.f[1] += a.y; s.f[2] += b.x; s.f[3] += b.y; s.f[4] += c.x; s.f[5] += c.y; s.f[6] += d.x; s.f[7] += d.y;
  }
  __device__ static __forceinline__ uint4 fin(const Acc& s) {
    return make_uint4(f2h(s.f[0], s.f[1]), f2h(s.f[2], s.f[3]), f2h(s.f[4], s.f[5]), f2h(s.f[6], s.f[7]));
  }
  __device__ static __forceinline__ uint4 fins(const Acc& s, float k) {
    return make_uint4(f2h(s.f[0] * k, s.f[1] * k), f2h(s.f[2] * k, s.f[3] * k), f2h(s.f[4] * k, s.f[5] * k), f2h(s.f[6] * k, s.f[7] * k));
  }
};

template <int DT, int OP> struct Policy;
#define FT_POL(DT, OP, P) template <> struct Policy<DT, OP> { using type = P; };
FT_POL(FT_U8, FT_SUM, PolAdd8) FT_POL(FT_I8, FT_SUM, PolAdd8) FT_POL(FT_U16, FT_SUM, PolAdd16) FT_POL(FT_I16, FT_SUM, PolAdd16)
FT_POL(FT_I32, FT_SUM, PolAdd32) FT_POL(FT_U32, FT_SUM, PolAdd32) FT_POL(FT_I64, FT_SUM, PolAdd64) FT_POL(FT_U64, FT_SUM, PolAdd64)
FT_POL(FT_F32, FT_SUM, PolF32) FT_POL(FT_F64, FT_SUM, PolF64) FT_POL(FT_BOOL, FT_SUM, PolOr)
FT_POL(FT_BF16, FT_SUM, PolBF16) FT_POL(FT_F16, FT_SUM, PolF16)
FT_POL(FT_U8, FT_BAND, PolAnd) FT_POL(FT_I8, FT_BAND, PolAnd) FT_POL(FT_U16, FT_BAND, PolAnd) FT_POL(FT_I16, FT_BAND, PolAnd)
FT_POL(FT_I32, FT_BAND, PolAnd) FT_POL(FT_U32, FT_BAND, PolAnd) FT_POL(FT_I64, FT_BAND, PolAnd) FT_POL(FT_U64, FT_BAND, PolAnd)
#undef FT_POL

// Policy ids used by the type-erased kernels: many (dtype, op) pairs share one policy,
// so kernels are instantiated per policy, not per pair.
template <int ID> struct PolById;
template <> struct PolById<POL_ADD8> { using type = PolAdd8; };
template <> struct PolById<POL_ADD16> { using type = PolAdd16; };
template <> struct PolById<POL_ADD32> { using type = PolAdd32; };
template <> struct PolById<POL_ADD64> { using type = PolAdd64; };
template <> struct PolById<POL_OR> { using type = PolOr; };
template <> struct PolById<POL_AND> { using type = PolAnd; };
template <> struct PolById<POL_F32> { using type = PolF32; };
template <> struct PolById<POL_F64> { using type = PolF64; };
template <> struct PolById<POL_BF16> { using type = PolBF16; };
template <> struct PolById<POL_F16> { using type = PolF16; };

// ---- scalar fallbacks (unaligned bases, ragged tails) ------------------------------------
// One element at a time, same arithmetic as the vector policies.
template <int ID> struct ScalarOp;
#define FT_SC(ID, T, A, LOAD, EXPR, STORE)                                         \
  template <> struct ScalarOp<ID> {                                                \
    using elem = T; using acc = A;                                                 \
    __device__ static __forceinline__ A load(T v) { return LOAD; }                 \
    __device__ static __forceinline__ A comb(A a, A b) { return EXPR; }            \
    __device__ static __forceinline__ T store(A a) { return STORE; }               \
  };
FT_SC(POL_ADD8, uint8_t, uint8_t, v, (uint8_t)(a + b), a)
FT_SC(POL_ADD16, uint16_t, uint16_t, v, (uint16_t)(a + b), a)
FT_SC(POL_ADD32, uint32_t, uint32_t, v, a + b, a)
FT_SC(POL_ADD64, unsigned long long, unsigned long long, v, a + b, a)
FT_SC(POL_OR, uint8_t, uint8_t, v, (uint8_t)(a | b), a)
FT_SC(POL_F32, float, float, v, a + b, a)
FT_SC(POL_F64, double, double, v, a + b, a)
FT_SC(POL_BF16, __nv_bfloat16, float, __bfloat162float(v), a + b, __float2bfloat16_rn(a))
FT_SC(POL_F16, __half, float, __half2float(v), a + b, __float2half_rn(a))
#undef FT_SC
// BAND works on bytes whatever the element width.
template <> struct ScalarOp<POL_AND> {
  using elem = uint8_t; using acc = uint8_t;
  __device__ static __forceinline__ uint8_t load(uint8_t v) { return v; }
  __device__ static __forceinline__ uint8_t comb(uint8_t a, uint8_t b) { return a & b; }
  __device__ static __forceinline__ uint8_t store(uint8_t a) { return a; }
};

}  // namespace ftk
