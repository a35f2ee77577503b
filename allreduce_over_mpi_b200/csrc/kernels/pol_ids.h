// Reduction-policy ids: many (dtype, op) pairs share one kernel instantiation (e.g. every
// bitwise AND is the same kernel whatever the integer width).  Host-safe header.
#pragma once
#include "../api/ft_types.h"

namespace ftk {

enum PolId { POL_ADD8 = 0, POL_ADD16, POL_ADD32, POL_ADD64, POL_OR, POL_AND, POL_F32, POL_F64, POL_BF16, POL_F16, POL_COUNT };

// -1 when (op, dtype) has no kernel.
inline int policy_id(int op, int dt) {
  if (op == FT_BAND) {
    switch (dt) {
      case FT_U8: case FT_I8: case FT_U16: case FT_I16: case FT_I32: case FT_U32: case FT_I64: case FT_U64: return POL_AND;
      default: return -1;
    }
  }
  if (op != FT_SUM) return -1;
  switch (dt) {
    case FT_U8: case FT_I8: return POL_ADD8;
    case FT_U16: case FT_I16: return POL_ADD16;
    case FT_I32: case FT_U32: return POL_ADD32;
    case FT_I64: case FT_U64: return POL_ADD64;
    case FT_BOOL: return POL_OR;
    case FT_F32: return POL_F32;
    case FT_F64: return POL_F64;
    case FT_BF16: return POL_BF16;
    case FT_F16: return POL_F16;
    default: return -1;
  }
}

}  // namespace ftk
