// Single-GPU n-way reduction with 256-bit global accesses (sm_100a).
//
// Blackwell adds 32-byte vector loads and stores (ld/st.global.v8.b32) and, on them only,
// the per-instruction L2 eviction priority.  For a pure streaming sum that halves the
// number of memory instructions per byte against the 16-byte kernels of reduce_nway.cu
// and lets both the inputs (read once) and the result (written once) leave L2 first.
// The fan-in is a template parameter for the common cases, so every load of a step is
// issued before the first add and nothing is indexed at run time.
//
// Same job as the reference's reduce_sum_2 .. reduce_sum_8 kernels
// (vector_add/reduce_sum_gpu.h:13-69), which move 4 bytes per thread.
#include "reduce_nway.cuh"
#include "vec.cuh"

namespace ftk {

// LD: 0 = L1::no_allocate, 1 = L1::no_allocate + L2::evict_first, 2 = non-coherent + L2::evict_first
template <int LD>
__device__ __forceinline__ void ld32(const void* p, uint4& a, uint4& b) {
  if (LD == 0)
    asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p) : "memory");
  else if (LD == 1)
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p) : "memory");
  else
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
}
// ST: 0 = default (write-back), 1 = L2::evict_first, 2 = L1::no_allocate only
template <int ST>
__device__ __forceinline__ void st32(void* p, const uint4& a, const uint4& b) {
  if (ST == 0)
    asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
  else if (ST == 1)
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
  else
    asm volatile("st.global.L1::no_allocate.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}

// One thread handles UNROLL 32-byte units per step, THREADS apart (every warp access is one
// contiguous 1 KiB run).  The grid either covers the vector once (one step per thread) or is
// capped and strides over it.  NSRC > 0: the fan-in is known at compile time; NSRC == 0: it is
// a.n (any value up to FT_MAX_FANIN), taken four sources at a time.
template <int POL, int NSRC, int UNROLL, int LD, int ST, int THREADS>
__global__ void __launch_bounds__(THREADS) reduce_nway_wide_kernel(const __grid_constant__ NwayArgs a, unsigned long long n32) {
  using P = typename PolById<POL>::type;
  const int nsrc = NSRC > 0 ? NSRC : a.n;
  const unsigned long long stride = (unsigned long long)gridDim.x * THREADS * UNROLL;
  for (unsigned long long base = (unsigned long long)blockIdx.x * THREADS * UNROLL; base < n32; base += stride) {
    unsigned long long idx[UNROLL];
    bool ok[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      idx[u] = base + (unsigned long long)u * THREADS + threadIdx.x;
      ok[u] = idx[u] < n32;
    }
    // sources are taken four at a time: all loads of a group are issued before its first add
    constexpr int G = (NSRC > 0 && NSRC < 4) ? NSRC : 4;
    typename P::Acc al[UNROLL], ah[UNROLL];
#pragma unroll
    for (int g0 = 0; g0 < (NSRC > 0 ? NSRC : FT_MAX_FANIN); g0 += G) {
      if (NSRC == 0 && g0 >= nsrc) break;
      uint4 lo[G][UNROLL], hi[G][UNROLL];
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          if (ok[u] && g0 + g < nsrc) ld32<LD>((const unsigned char*)a.src[g0 + g] + idx[u] * 32, lo[g][u], hi[g][u]);
          else lo[g][u] = hi[g][u] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          if (g0 + g == 0) { P::init(al[u], lo[g][u]); P::init(ah[u], hi[g][u]); }
          else if (g0 + g < nsrc) { P::add(al[u], lo[g][u]); P::add(ah[u], hi[g][u]); }
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (ok[u]) st32<ST>((unsigned char*)a.dst + idx[u] * 32, P::fin(al[u]), P::fin(ah[u]));
  }
}

// code = U*1000 + LD*100 + ST*10 + T, with U units per thread per step, LD/ST as above,
// T: 0 = 256 threads and one step per thread (the grid covers the vector), 1 = 512 threads likewise,
//    3 = 512 threads x 4 CTAs per SM striding over the vector.
// Measured on B200 over fan-in 2/3/4/8, fp32 and bf16, 64 Mi elements, launches back to back: 1011 is within
// 1 % of the best configuration in every case (6.5-7.2 TB/s) and is the default; the others stay selectable.
constexpr int kWideDefault = 1011;

template <int POL, int NSRC, int UNROLL, int LD, int ST>
static cudaError_t launch_t(const NwayArgs& a, unsigned long long n32, int t, int sms, cudaStream_t st) {
  const int threads = t == 0 ? 256 : 512;
  const unsigned long long per_cta = (unsigned long long)threads * UNROLL;
  unsigned long long grid = (n32 + per_cta - 1) / per_cta;
  if (t == 3 && grid > (unsigned long long)sms * 4) grid = (unsigned long long)sms * 4;
  if (grid > 0x7fffffffull) return cudaErrorInvalidValue;
  if (grid < 1) grid = 1;
  if (threads == 256) reduce_nway_wide_kernel<POL, NSRC, UNROLL, LD, ST, 256><<<(unsigned)grid, 256, 0, st>>>(a, n32);
  else reduce_nway_wide_kernel<POL, NSRC, UNROLL, LD, ST, 512><<<(unsigned)grid, 512, 0, st>>>(a, n32);
  return cudaGetLastError();
}

template <int POL, int NSRC, bool TUNING>
static cudaError_t launch_cfg(const NwayArgs& a, unsigned long long n32, int code, int sms, cudaStream_t st) {
  const int t = code % 10;
  if (t != 0 && t != 1 && t != 3) return cudaErrorInvalidValue;
  if (code / 10 == kWideDefault / 10) return launch_t<POL, NSRC, 1, 0, 1>(a, n32, t, sms, st);
  if constexpr (TUNING) {
    switch (code / 10) {
      case 100: return launch_t<POL, NSRC, 1, 0, 0>(a, n32, t, sms, st);
      case 111: return launch_t<POL, NSRC, 1, 1, 1>(a, n32, t, sms, st);
      case 200: return launch_t<POL, NSRC, 2, 0, 0>(a, n32, t, sms, st);
      case 201: return launch_t<POL, NSRC, 2, 0, 1>(a, n32, t, sms, st);
      case 211: return launch_t<POL, NSRC, 2, 1, 1>(a, n32, t, sms, st);
      default: break;
    }
  }
  return cudaErrorInvalidValue;
}

template <int POL, bool TUNING>
static cudaError_t launch_n(const NwayArgs& a, unsigned long long n32, int code, int sms, cudaStream_t st) {
  switch (a.n) {
    case 1: return launch_cfg<POL, 1, false>(a, n32, code, sms, st);
    case 2: return launch_cfg<POL, 2, TUNING>(a, n32, code, sms, st);
    case 3: return launch_cfg<POL, 3, TUNING>(a, n32, code, sms, st);
    case 4: return launch_cfg<POL, 4, TUNING>(a, n32, code, sms, st);
    case 5: return launch_cfg<POL, 5, false>(a, n32, code, sms, st);
    case 6: return launch_cfg<POL, 6, false>(a, n32, code, sms, st);
    case 7: return launch_cfg<POL, 7, false>(a, n32, code, sms, st);
    case 8: return launch_cfg<POL, 8, TUNING>(a, n32, code, sms, st);
    default: return launch_cfg<POL, 0, false>(a, n32, code, sms, st);
  }
}

cudaError_t launch_wide(int pol, const NwayArgs& a, unsigned long long n32, int code, int sms, cudaStream_t st) {
  if (code <= 0) code = kWideDefault;
  switch (pol) {
    case POL_ADD8: return launch_n<POL_ADD8, false>(a, n32, code, sms, st);
    case POL_ADD16: return launch_n<POL_ADD16, false>(a, n32, code, sms, st);
    case POL_ADD32: return launch_n<POL_ADD32, false>(a, n32, code, sms, st);
    case POL_ADD64: return launch_n<POL_ADD64, false>(a, n32, code, sms, st);
    case POL_OR: return launch_n<POL_OR, false>(a, n32, code, sms, st);
    case POL_AND: return launch_n<POL_AND, false>(a, n32, code, sms, st);
    case POL_F32: return launch_n<POL_F32, true>(a, n32, code, sms, st);
    case POL_F64: return launch_n<POL_F64, false>(a, n32, code, sms, st);
    case POL_BF16: return launch_n<POL_BF16, true>(a, n32, code, sms, st);
    case POL_F16: return launch_n<POL_F16, false>(a, n32, code, sms, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ftk
