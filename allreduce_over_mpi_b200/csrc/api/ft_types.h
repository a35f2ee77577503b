/* Element types, reduction operators and status codes shared by host code, device
 * code and the C API.  Plain C so that ctypes / C callers can include it.
 *
 * The SUM / BAND type coverage is a superset of the reference dispatcher
 * (allreduce_over_mpi/mpi_mod.hpp:1363-1412): its eleven MPI datatypes map onto
 * FT_U8..FT_BOOL (MPI_LONG_LONG and MPI_LONG_LONG_INT are both FT_I64); FT_U32, FT_U64,
 * FT_BF16 and FT_F16 are additions.  The 16-bit floats accumulate in fp32. */
#ifndef FLEXTREE_TYPES_H_
#define FLEXTREE_TYPES_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ft_dtype {
  FT_U8 = 0,
  FT_I8 = 1,
  FT_U16 = 2,
  FT_I16 = 3,
  FT_I32 = 4,
  FT_I64 = 5,
  FT_F32 = 6,
  FT_F64 = 7,
  FT_BOOL = 8,
  FT_U32 = 9,
  FT_U64 = 10,
  FT_BF16 = 11,
  FT_F16 = 12,
  FT_DTYPE_COUNT = 13
} ft_dtype;

typedef enum ft_op { FT_SUM = 0, FT_BAND = 1, FT_OP_COUNT = 2 } ft_op;

typedef enum ft_status {
  FT_OK = 0,
  FT_ERR_INVALID_ARG = 1,
  FT_ERR_UNSUPPORTED_TYPE = 2, /* "Type ... is not supported" */
  FT_ERR_UNSUPPORTED_OP = 3,   /* "Unsupported op ..." */
  FT_ERR_INVALID_TOPO = 4,     /* "invalid FT_TOPO ..." */
  FT_ERR_TIMEOUT = 5,          /* a bounded wait on a peer ran out */
  FT_ERR_CUDA = 6,
  FT_ERR_TOO_LARGE = 7,
  FT_ERR_PROTOCOL = 8, /* a peer signalled an unexpected epoch */
  FT_ERR_NOT_AVAILABLE = 9,
  FT_ERR_BOUNDS = 10 /* debugging build (-DFT_BOUNDS): a kernel was about to leave the symmetric heap and skipped the access */
} ft_status;

/* All-reduce algorithms of the GPU communicator (flextree_comm.h); AUTO asks the selection policy. */
enum { FT_ALGO_AUTO = 0, FT_ALGO_STAGED = 1, FT_ALGO_ONESHOT = 2, FT_ALGO_NVLS = 3, FT_ALGO_HYBRID = 4, FT_ALGO_LL = 5, FT_ALGO_PUSH = 6,
       FT_ALGO_NVLS1 = 9 /* one-shot through the switch; 7 and 8 number the reduce-scatter / all-gather calls in the usage counters */ };

/* Maximum number of sources of one n-way reduction (own copy included).  The
 * reference stops at 20 (MAX_NUM_BLOCKS, mpi_mod.hpp:811). */
#define FT_MAX_FANIN 32
/* Largest world the device-side plan tables are sized for. */
#define FT_MAX_RANKS 64

static inline size_t ft_dtype_size(ft_dtype t) {
  switch (t) {
    case FT_U8: case FT_I8: case FT_BOOL: return 1;
    case FT_U16: case FT_I16: case FT_BF16: case FT_F16: return 2;
    case FT_I32: case FT_U32: case FT_F32: return 4;
    case FT_I64: case FT_U64: case FT_F64: return 8;
    default: return 0;
  }
}

static inline const char* ft_dtype_name(ft_dtype t) {
  switch (t) {
    case FT_U8: return "uint8"; case FT_I8: return "int8"; case FT_U16: return "uint16";
    case FT_I16: return "int16"; case FT_I32: return "int32"; case FT_I64: return "int64";
    case FT_F32: return "float32"; case FT_F64: return "float64"; case FT_BOOL: return "bool";
    case FT_U32: return "uint32"; case FT_U64: return "uint64"; case FT_BF16: return "bfloat16";
    case FT_F16: return "float16"; default: return "unknown";
  }
}

/* 1 when (op, dtype) has a reduction kernel.  BAND exists for integers only. */
static inline int ft_op_supported(ft_op op, ft_dtype t) {
  if ((int)t < 0 || t >= FT_DTYPE_COUNT) return 0;
  if (op == FT_SUM) return 1;
  if (op == FT_BAND)
    return t == FT_U8 || t == FT_I8 || t == FT_U16 || t == FT_I16 || t == FT_I32 || t == FT_I64 ||
           t == FT_U32 || t == FT_U64;
  return 0;
}

static inline const char* ft_status_name(ft_status s) {
  switch (s) {
    case FT_OK: return "ok"; case FT_ERR_INVALID_ARG: return "invalid argument";
    case FT_ERR_UNSUPPORTED_TYPE: return "unsupported type"; case FT_ERR_UNSUPPORTED_OP: return "unsupported op";
    case FT_ERR_INVALID_TOPO: return "invalid topology"; case FT_ERR_TIMEOUT: return "timeout waiting for a peer";
    case FT_ERR_CUDA: return "CUDA error"; case FT_ERR_TOO_LARGE: return "size exceeds limit";
    case FT_ERR_PROTOCOL: return "protocol error"; case FT_ERR_NOT_AVAILABLE: return "not available";
    case FT_ERR_BOUNDS: return "address outside the symmetric heap (access skipped)";
    default: return "unknown";
  }
}

#ifdef __cplusplus
}
#endif
#endif /* FLEXTREE_TYPES_H_ */
