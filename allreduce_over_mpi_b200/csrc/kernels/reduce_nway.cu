// Single-GPU n-way element-wise reduction for sm_100a:  dst[i] = src[0][i] (op) ... (op) src[n-1][i].
//
// Replaces the reference's twenty one-element-per-thread kernels reduce_sum_1..20 and
// their switch launcher (vector_add/reduce_sum_gpu.h:4-203, :205-316) and gives the CPU
// kernels reduce_sum / reduce_band (allreduce_over_mpi/mpi_mod.hpp:812-1251) a device
// form.  One kernel template covers every fan-in 1..FT_MAX_FANIN: the source pointers
// travel in a __grid_constant__ parameter block and the fan-in loop is unrolled in
// groups so that GROUP x UNROLL independent 16-byte loads are in flight per thread.
//
// Data paths:
//   * 32-byte path (reduce_nway_wide.cu): the default whenever every pointer sits on a 32-byte boundary;
//   * vector path: persistent grid-stride loop of 16-byte non-allocating loads;
//   * TMA path: per-CTA ring of shared-memory stages filled by 1-D bulk async copies
//     (cp.async.bulk, completion on an mbarrier) and drained by all threads.
// Unaligned pointers and the sub-16-byte tail take a scalar path with the same arithmetic.
//
// 16-bit floats accumulate in fp32; 64-bit indexing throughout.
#include <atomic>
#include <cstdio>
#include <mutex>

#include "../api/flextree.h"
#include "reduce_nway.cuh"
#include "vec.cuh"

namespace ftk {

static std::atomic<uint64_t> g_launches{0};


// ---------------------------------------------------------------------------- vector path
template <int POL, int UNROLL, int GROUP>
__global__ void __launch_bounds__(512) reduce_nway_vec_kernel(const __grid_constant__ NwayArgs a) {
  using P = typename PolById<POL>::type;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x * UNROLL;
  for (unsigned long long base = (unsigned long long)blockIdx.x * blockDim.x * UNROLL; base < a.nvec; base += stride) {
    unsigned long long idx[UNROLL];
    bool ok[UNROLL];
    typename P::Acc acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      idx[u] = base + (unsigned long long)u * blockDim.x + threadIdx.x;
      ok[u] = idx[u] < a.nvec;
    }
    // sources are consumed GROUP at a time: all GROUP x UNROLL loads of a group are issued
    // before the first add, whatever the fan-in (the bounds test is uniform across the grid)
    {
      uint4 v[GROUP][UNROLL];
#pragma unroll
      for (int g = 0; g < GROUP; ++g)
        if (g < a.n) {
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) v[g][u] = ok[u] ? ld_stream((const uint4*)a.src[g] + idx[u]) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) P::init(acc[u], v[0][u]);
#pragma unroll
      for (int g = 1; g < GROUP; ++g)
        if (g < a.n) {
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) P::add(acc[u], v[g][u]);
        }
    }
    for (int k = GROUP; k < a.n; k += GROUP) {
      uint4 v[GROUP][UNROLL];
#pragma unroll
      for (int g = 0; g < GROUP; ++g)
        if (k + g < a.n) {
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) v[g][u] = ok[u] ? ld_stream((const uint4*)a.src[k + g] + idx[u]) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int g = 0; g < GROUP; ++g)
        if (k + g < a.n) {
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) P::add(acc[u], v[g][u]);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (ok[u]) st_vec_cs((uint4*)a.dst + idx[u], P::fin(acc[u]));
  }
}

// ---------------------------------------------------------------------------- narrow-word path
// One 4- or 8-byte word per thread, one CTA per tile, every source's load issued before the
// first add: the access pattern of a one-element-per-thread kernel (many more warps in
// flight, 128-byte requests per warp) with this file's per-type arithmetic.  At high fan-in
// this keeps HBM busier than 16-byte vectors do.
template <int POL, int WORDS>   // WORDS = 1 (4 bytes) or 2 (8 bytes) per thread
__global__ void __launch_bounds__(256) reduce_nway_narrow_kernel(const __grid_constant__ NwayArgs a, unsigned long long nwords) {
  using P = typename PolById<POL>::type;
  const unsigned long long i = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) * WORDS;
  if (i >= nwords) return;
  typename P::Acc acc;
  constexpr int G = 8;
  for (int k = 0; k < a.n; k += G) {
    uint32_t w[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g)
      if (k + g < a.n) {
        const uint32_t* p = (const uint32_t*)a.src[k + g] + i;
        if (WORDS == 2) asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(w[g][0]), "=r"(w[g][1]) : "l"(p) : "memory");
        else { asm volatile("ld.global.L1::no_allocate.u32 %0, [%1];" : "=r"(w[g][0]) : "l"(p) : "memory"); w[g][1] = 0; }
      }
#pragma unroll
    for (int g = 0; g < G; ++g)
      if (k + g < a.n) {
        const uint4 v = make_uint4(w[g][0], w[g][1], 0, 0);
        if (k + g == 0) P::init(acc, v);
        else P::add(acc, v);
      }
  }
  const uint4 out = P::fin(acc);
  uint32_t* d = (uint32_t*)a.dst + i;
  if (WORDS == 2) asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(d), "r"(out.x), "r"(out.y) : "memory");
  else asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(d), "r"(out.x) : "memory");
}

template <int POL, int WORDS>
static cudaError_t launch_narrow(const NwayArgs& a, cudaStream_t st) {
  const unsigned long long nwords = a.nvec * 4;   // the aligned part, in 4-byte words (a multiple of 4)
  const unsigned long long threads = nwords / WORDS;
  reduce_nway_narrow_kernel<POL, WORDS><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(a, nwords);
  g_launches++;
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------- scalar path
template <int POL>
__global__ void __launch_bounds__(256) reduce_nway_scalar_kernel(const __grid_constant__ NwayArgs a, unsigned long long first_unit) {
  using S = ScalarOp<POL>;
  using T = typename S::elem;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = first_unit + (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.nunit; i += stride) {
    typename S::acc acc = S::load(((const T*)a.src[0])[i]);
    for (int k = 1; k < a.n; ++k) acc = S::comb(acc, S::load(((const T*)a.src[k])[i]));
    ((T*)a.dst)[i] = S::store(acc);
  }
}

// ---------------------------------------------------------------------------- TMA path
// Each CTA owns a ring of STAGES shared-memory stages; a stage holds one TILE-byte tile
// of each of the n sources.  Thread 0 is the producer: it waits for the stage to be
// free, arms the stage's "full" mbarrier with the byte count and issues n bulk copies.
// All threads consume: wait "full", sum the n tiles from shared memory, store 16-byte
// vectors to global, then arrive on the stage's "empty" mbarrier.  Copies are plain
// (no cluster multicast), source and destination 16-byte aligned, sizes multiples of 16.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: gives up after `limit` polls and reports failure so the kernel can leave.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = 1u << 20) {
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int POL, int STAGES>
__global__ void __launch_bounds__(256) reduce_nway_tma_kernel(const __grid_constant__ NwayArgs a, int tile_vecs, int* error_flag) {
  using P = typename PolById<POL>::type;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[STAGES], empty[STAGES];
  __shared__ int failed;
  const int n = a.n;
  const unsigned long long ntiles = (a.nvec + tile_vecs - 1) / tile_vecs;
  const uint32_t stage_bytes = (uint32_t)n * tile_vecs * 16u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], blockDim.x); }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](unsigned long long tile, int stage) {
    const unsigned long long v0 = tile * tile_vecs;
    const uint32_t vecs = (uint32_t)min((unsigned long long)tile_vecs, a.nvec - v0);
    mbar_expect_tx(&full[stage], vecs * 16u * n);
    unsigned char* sbase = smem + (size_t)stage * stage_bytes;
    for (int k = 0; k < n; ++k)
      bulk_g2s(sbase + (size_t)k * tile_vecs * 16u, (const uint4*)a.src[k] + v0, vecs * 16u, &full[stage]);
  };

  // prologue: fill the ring
  unsigned long long next = blockIdx.x;
  if (threadIdx.x == 0)
    for (int s = 0; s < STAGES && next < ntiles; ++s, next += gridDim.x) issue(next, s);

  int stage = 0;
  uint32_t phase = 0;
  for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    if (!mbar_wait(&full[stage], phase)) failed = 1;
    if (failed) break;
    const unsigned long long v0 = tile * tile_vecs;
    const uint32_t vecs = (uint32_t)min((unsigned long long)tile_vecs, a.nvec - v0);
    const uint4* sbase = (const uint4*)(smem + (size_t)stage * stage_bytes);
    for (uint32_t i = threadIdx.x; i < vecs; i += blockDim.x) {
      typename P::Acc acc;
      P::init(acc, sbase[i]);
      for (int k = 1; k < n; ++k) P::add(acc, sbase[(size_t)k * tile_vecs + i]);
      st_vec_cs((uint4*)a.dst + v0 + i, P::fin(acc));
    }
    mbar_arrive(&empty[stage]);
    if (threadIdx.x == 0) {
      const unsigned long long refill = tile + (unsigned long long)STAGES * gridDim.x;
      if (refill < ntiles) {
        if (mbar_wait(&empty[stage], phase)) issue(refill, stage);
        else failed = 1;
      }
    }
    if (++stage == STAGES) { stage = 0; phase ^= 1; }
  }
  __syncthreads();
  if (threadIdx.x == 0 && failed) {
    // give copies that are still in flight a bounded chance to land before the CTA's
    // shared memory is released, then report
    for (int s = 0; s < STAGES; ++s) mbar_wait(&full[s], 0, 1u << 12);
    if (error_flag) atomicExch(error_flag, 1);
  }
}

// ---------------------------------------------------------------------------- host side
static thread_local char g_cuda_err[256] = "";

static int cuda_fail(cudaError_t e, const char* where) {
  snprintf(g_cuda_err, sizeof g_cuda_err, "%s: %s", where, cudaGetErrorString(e));
  return FT_ERR_CUDA;
}

struct DevInfo { int sms = 0; };
static DevInfo dev_info() {
  static std::mutex mu;
  static DevInfo info[64];
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  if (dev >= 0 && dev < 64 && info[dev].sms == 0) {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    info[dev].sms = sms;
  }
  return info[dev < 64 && dev >= 0 ? dev : 0];
}

template <int POL, int UNROLL, int GROUP>
static cudaError_t launch_vec(const NwayArgs& a, int threads, int ctas_per_sm, cudaStream_t st) {
  const unsigned long long per_cta = (unsigned long long)threads * UNROLL;
  unsigned long long want = (a.nvec + per_cta - 1) / per_cta;
  unsigned long long cap = ctas_per_sm > 0 ? (unsigned long long)dev_info().sms * ctas_per_sm : 0x7fffffffull;
  int grid = (int)(want < cap ? want : cap);
  if (grid < 1) grid = 1;
  reduce_nway_vec_kernel<POL, UNROLL, GROUP><<<grid, threads, 0, st>>>(a);
  g_launches++;
  return cudaGetLastError();
}

template <int POL>
static cudaError_t launch_scalar(const NwayArgs& a, unsigned long long first_unit, cudaStream_t st) {
  if (first_unit >= a.nunit) return cudaSuccess;
  unsigned long long want = (a.nunit - first_unit + 255) / 256;
  unsigned long long cap = (unsigned long long)dev_info().sms * 8;
  reduce_nway_scalar_kernel<POL><<<(int)(want < cap ? want : cap), 256, 0, st>>>(a, first_unit);
  g_launches++;
  return cudaGetLastError();
}

static int* tma_error_flag() {
  static std::mutex mu;
  static int* flag[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  if (!flag[dev]) {
    if (cudaMalloc(&flag[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(flag[dev], 0, sizeof(int));
  }
  return flag[dev];
}

template <int POL>
static cudaError_t launch_tma(const NwayArgs& a, cudaStream_t st) {
  constexpr int STAGES = 4;
  // stage = n tiles; keep the ring within ~176 KB of shared memory
  int tile_vecs = 512;  // 8 KB per source
  while ((size_t)a.n * tile_vecs * 16 * STAGES > 176 * 1024 && tile_vecs > 16) tile_vecs >>= 1;
  const size_t smem = (size_t)a.n * tile_vecs * 16 * STAGES;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  std::call_once(once[dev], [] {
    cudaFuncSetAttribute(reduce_nway_tma_kernel<POL, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  });
  const unsigned long long ntiles = (a.nvec + tile_vecs - 1) / tile_vecs;
  unsigned long long cap = dev_info().sms;  // one CTA per SM: the ring already fills shared memory
  int grid = (int)(ntiles < cap ? ntiles : cap);
  if (grid < 1) grid = 1;
  reduce_nway_tma_kernel<POL, STAGES><<<grid, 256, smem, st>>>(a, tile_vecs, tma_error_flag());
  g_launches++;
  return cudaGetLastError();
}

template <int POL>
static int run_policy(NwayArgs& a, size_t bytes, int variant, cudaStream_t st) {
  bool aligned = ((uintptr_t)a.dst & 15) == 0;
  for (int k = 0; k < a.n; ++k) aligned = aligned && (((uintptr_t)a.src[k] & 15) == 0);
  const size_t unit = sizeof(typename ScalarOp<POL>::elem);
  a.nunit = bytes / unit;
  a.nvec = aligned ? bytes / 16 : 0;
  cudaError_t e = cudaSuccess;
  // 32-byte accesses (reduce_nway_wide.cu) when every pointer sits on a 32-byte boundary
  if (a.nvec >= 2 && (variant >= 1000 || variant == 0)) {
    bool a32 = ((uintptr_t)a.dst & 31) == 0;
    for (int k = 0; k < a.n; ++k) a32 = a32 && (((uintptr_t)a.src[k] & 31) == 0);
    if (a32) {
      const unsigned long long n32 = bytes / 32;
      e = launch_wide(POL, a, n32, variant >= 1000 ? variant : 0, dev_info().sms, st);
      if (e == cudaSuccess) {
        g_launches++;
        e = launch_scalar<POL>(a, n32 * 32 / unit, st);
        if (e != cudaSuccess) return cuda_fail(e, "reduce_nway scalar launch");
        return FT_OK;
      }
      if (e != cudaErrorInvalidValue) return cuda_fail(e, "reduce_nway wide launch");
      cudaGetLastError();
      e = cudaSuccess;   // no such instantiation: the 16-byte kernels take it
    }
  }
  if (a.nvec) {
    bool done = false;
    if (variant == 2) { e = launch_tma<POL>(a, st); done = true; }
    if constexpr (POL == POL_F32 || POL == POL_BF16) {
      // tuning variants (unroll, fan-in group, threads, CTAs per SM); 0/1 pick the default
      switch (variant) {
        case 11: e = launch_vec<POL, 2, 2>(a, 512, 4, st); done = true; break;
        case 12: e = launch_vec<POL, 2, 4>(a, 512, 4, st); done = true; break;
        case 13: e = launch_vec<POL, 4, 2>(a, 512, 2, st); done = true; break;
        case 14: e = launch_vec<POL, 4, 2>(a, 512, 4, st); done = true; break;
        case 15: e = launch_vec<POL, 4, 2>(a, 256, 8, st); done = true; break;
        case 16: e = launch_vec<POL, 2, 8>(a, 256, 4, st); done = true; break;
        case 17: e = launch_vec<POL, 1, 8>(a, 256, 0, st); done = true; break;
        case 18: e = launch_vec<POL, 2, 4>(a, 256, 0, st); done = true; break;
        case 19: e = launch_vec<POL, 4, 4>(a, 256, 0, st); done = true; break;
        case 20: e = launch_vec<POL, 1, 4>(a, 512, 0, st); done = true; break;
        case 21: e = launch_vec<POL, 2, 8>(a, 256, 8, st); done = true; break;
        case 22: e = launch_vec<POL, 1, 8>(a, 512, 4, st); done = true; break;
        case 23: e = launch_narrow<POL, 1>(a, st); done = true; break;
        case 24: e = launch_narrow<POL, 2>(a, st); done = true; break;
        default: break;
      }
    }
    // defaults picked from a B200 sweep (fp32 and bf16, 64 Mi elements): low fan-in runs a
    // persistent grid of 2 CTAs x 512 threads per SM with 4 vectors x 2 sources in flight; from
    // fan-in 6 up one CTA per tile with 1 vector x 4 sources in flight does better;
    // fp32 with three or more sources: 8 bytes per thread, one CTA per tile, all loads up front
    if (!done) {
      if (POL == POL_F32 && a.n >= 3) e = launch_narrow<POL, 2>(a, st);
      else e = a.n >= 6 ? launch_vec<POL, 1, 4>(a, 512, 0, st) : launch_vec<POL, 4, 2>(a, 512, 2, st);
    }
    if (e != cudaSuccess) return cuda_fail(e, "reduce_nway vector launch");
  }
  e = launch_scalar<POL>(a, a.nvec * 16 / unit, st);
  if (e != cudaSuccess) return cuda_fail(e, "reduce_nway scalar launch");
  return FT_OK;
}

// ---------------------------------------------------------------------------- scaled / cast variant
// out = scale * sum_k src[k], fp32 accumulation; IN/OUT in {fp32, bf16}.
template <bool IN_BF16, bool OUT_BF16>
__global__ void __launch_bounds__(512) reduce_nway_scaled_kernel(const __grid_constant__ NwayArgs a, unsigned long long len, float scale, bool vec_ok) {
  // work in groups of 8 elements: 8 bf16 = 16 B, 8 fp32 = 32 B
  const unsigned long long ngroups = vec_ok ? len / 8 : 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long g = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += stride) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k = 0; k < a.n; ++k) {
      if (IN_BF16) {
        uint4 v = ld_stream((const uint4*)a.src[k] + g);
        acc[0] += bf_lo(v.x); acc[1] += bf_hi(v.x); acc[2] += bf_lo(v.y); acc[3] += bf_hi(v.y);
        acc[4] += bf_lo(v.z); acc[5] += bf_hi(v.z); acc[6] += bf_lo(v.w); acc[7] += bf_hi(v.w);
      } else {
        uint4 v = ld_stream((const uint4*)a.src[k] + 2 * g), w = ld_stream((const uint4*)a.src[k] + 2 * g + 1);
        acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y); acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
        acc[4] += __uint_as_float(w.x); acc[5] += __uint_as_float(w.y); acc[6] += __uint_as_float(w.z); acc[7] += __uint_as_float(w.w);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= scale;
    if (OUT_BF16) {
      st_vec((uint4*)a.dst + g, make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7])));
    } else {
      st_vec((uint4*)a.dst + 2 * g, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])));
      st_vec((uint4*)a.dst + 2 * g + 1, make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]), __float_as_uint(acc[6]), __float_as_uint(acc[7])));
    }
  }
  // ragged tail / unaligned: scalar
  for (unsigned long long i = ngroups * 8 + (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
    float acc = 0.f;
    for (int k = 0; k < a.n; ++k)
      acc += IN_BF16 ? __bfloat162float(((const __nv_bfloat16*)a.src[k])[i]) : ((const float*)a.src[k])[i];
    acc *= scale;
    if (OUT_BF16) ((__nv_bfloat16*)a.dst)[i] = __float2bfloat16_rn(acc);
    else ((float*)a.dst)[i] = acc;
  }
}

// ---------------------------------------------------------------------------- scale in place
// buf[i] *= scale for every floating type, with the policies' arithmetic (16-bit floats through fp32,
// one rounding): what a one-rank "average" all-reduce has to do.
template <int POL>
__global__ void __launch_bounds__(256) scale_inplace_kernel(void* buf, unsigned long long nvec, unsigned long long nunit, float scale) {
  using P = typename PolById<POL>::type;
  using S = ScalarOp<POL>;
  using T = typename S::elem;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (unsigned long long i = tid; i < nvec; i += stride) {
    typename P::Acc acc;
    P::init(acc, ld_stream((const uint4*)buf + i));
    st_vec((uint4*)buf + i, P::fins(acc, scale));
  }
  for (unsigned long long i = nvec * (16 / sizeof(T)) + tid; i < nunit; i += stride)
    ((T*)buf)[i] = S::store(S::load(((const T*)buf)[i]) * (typename S::acc)scale);
}

}  // namespace ftk

extern "C" {

int ft_scale_inplace(int dtype, void* buf, size_t len, float scale, void* stream) {
  using namespace ftk;
  const int pol = policy_id(FT_SUM, dtype);
  if (pol != POL_F32 && pol != POL_F64 && pol != POL_BF16 && pol != POL_F16) return FT_ERR_UNSUPPORTED_TYPE;
  if (len == 0 || scale == 1.0f) return FT_OK;
  if (!buf) return FT_ERR_INVALID_ARG;
  const size_t es = ft_dtype_size((ft_dtype)dtype);
  const unsigned long long nvec = ((uintptr_t)buf & 15) == 0 ? (unsigned long long)len * es / 16 : 0;
  unsigned long long want = ((nvec ? nvec : len) + 255) / 256, cap = (unsigned long long)dev_info().sms * 8;
  const int grid = (int)(want < cap ? (want ? want : 1) : cap);
  cudaStream_t st = (cudaStream_t)stream;
  switch (pol) {
    case POL_F32: scale_inplace_kernel<POL_F32><<<grid, 256, 0, st>>>(buf, nvec, len, scale); break;
    case POL_F64: scale_inplace_kernel<POL_F64><<<grid, 256, 0, st>>>(buf, nvec, len, scale); break;
    case POL_BF16: scale_inplace_kernel<POL_BF16><<<grid, 256, 0, st>>>(buf, nvec, len, scale); break;
    default: scale_inplace_kernel<POL_F16><<<grid, 256, 0, st>>>(buf, nvec, len, scale); break;
  }
  g_launches++;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FT_OK : cuda_fail(e, "scale launch");
}

int ft_reduce_nway(int op, int dtype, const void* const* src, void* dst, int n, size_t len, int variant, void* stream) {
  using namespace ftk;
  if (op < 0 || op >= FT_OP_COUNT) return FT_ERR_UNSUPPORTED_OP;
  const int pol = policy_id(op, dtype);
  if (pol < 0) return FT_ERR_UNSUPPORTED_TYPE;
  if (n < 1 || n > FT_MAX_FANIN) return n > FT_MAX_FANIN ? FT_ERR_TOO_LARGE : FT_ERR_INVALID_ARG;
  if (len == 0) return FT_OK;
  if (!src || !dst) return FT_ERR_INVALID_ARG;
  NwayArgs a{};
  for (int k = 0; k < n; ++k) {
    if (!src[k]) return FT_ERR_INVALID_ARG;
    a.src[k] = src[k];
  }
  a.dst = dst;
  a.n = n;
  const size_t bytes = len * ft_dtype_size((ft_dtype)dtype);
  cudaStream_t st = (cudaStream_t)stream;
  switch (pol) {
    case POL_ADD8: return run_policy<POL_ADD8>(a, bytes, variant, st);
    case POL_ADD16: return run_policy<POL_ADD16>(a, bytes, variant, st);
    case POL_ADD32: return run_policy<POL_ADD32>(a, bytes, variant, st);
    case POL_ADD64: return run_policy<POL_ADD64>(a, bytes, variant, st);
    case POL_OR: return run_policy<POL_OR>(a, bytes, variant, st);
    case POL_AND: return run_policy<POL_AND>(a, bytes, variant, st);
    case POL_F32: return run_policy<POL_F32>(a, bytes, variant, st);
    case POL_F64: return run_policy<POL_F64>(a, bytes, variant, st);
    case POL_BF16: return run_policy<POL_BF16>(a, bytes, variant, st);
    case POL_F16: return run_policy<POL_F16>(a, bytes, variant, st);
  }
  return FT_ERR_UNSUPPORTED_TYPE;
}

int ft_reduce_nway_scaled(int in_dtype, int out_dtype, const void* const* src, void* dst, int n, size_t len, float scale, void* stream) {
  using namespace ftk;
  if ((in_dtype != FT_F32 && in_dtype != FT_BF16) || (out_dtype != FT_F32 && out_dtype != FT_BF16)) return FT_ERR_UNSUPPORTED_TYPE;
  if (n < 1 || n > FT_MAX_FANIN) return FT_ERR_INVALID_ARG;
  if (len == 0) return FT_OK;
  if (!src || !dst) return FT_ERR_INVALID_ARG;
  NwayArgs a{};
  bool aligned = ((uintptr_t)dst & 15) == 0;
  for (int k = 0; k < n; ++k) {
    if (!src[k]) return FT_ERR_INVALID_ARG;
    a.src[k] = src[k];
    aligned = aligned && (((uintptr_t)src[k] & 15) == 0);
  }
  a.dst = dst;
  a.n = n;
  unsigned long long want = (len / 8 + 511) / 512 + 1, cap = (unsigned long long)dev_info().sms * 4;
  const int grid = (int)(want < cap ? want : cap);
  cudaStream_t st = (cudaStream_t)stream;
  const bool ib = in_dtype == FT_BF16, ob = out_dtype == FT_BF16;
  if (ib && ob) reduce_nway_scaled_kernel<true, true><<<grid, 512, 0, st>>>(a, len, scale, aligned);
  else if (ib) reduce_nway_scaled_kernel<true, false><<<grid, 512, 0, st>>>(a, len, scale, aligned);
  else if (ob) reduce_nway_scaled_kernel<false, true><<<grid, 512, 0, st>>>(a, len, scale, aligned);
  else reduce_nway_scaled_kernel<false, false><<<grid, 512, 0, st>>>(a, len, scale, aligned);
  g_launches++;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FT_OK : cuda_fail(e, "reduce_nway_scaled launch");
}

const char* ft_last_cuda_error(void) { return ftk::g_cuda_err; }
uint64_t ft_launch_count(void) { return ftk::g_launches.load(); }
void ft_count_launch(uint64_t n) { ftk::g_launches += n; }

}  // extern "C"
