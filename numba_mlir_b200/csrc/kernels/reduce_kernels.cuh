// Instantiation macros for the reduction kernels: every (op, dtype) pair gets
// an extern "C" entry named nmb_reduce_<kind>_<op>_<dtype>.
#pragma once

#include "../gpu_common.h"
#include "reduce_ws.cuh"

#define NMB_RED_TYPES(X, kind, op, RT)                                                         \
  X(kind, op, f32, RT<float>)                                                                  \
  X(kind, op, f64, RT<double>)                                                                 \
  X(kind, op, i32, RT<int32_t>)                                                                \
  X(kind, op, i64, RT<int64_t>)

namespace nmb {
namespace red {
template <typename T> using ArgMinR = ArgR<T, true>;
template <typename T> using ArgMaxR = ArgR<T, false>;
} // namespace red
} // namespace nmb

#define NMB_RED_ALL_OPS(X, kind)                                                               \
  NMB_RED_TYPES(X, kind, sum, nmb::red::SumR)                                                  \
  NMB_RED_TYPES(X, kind, prod, nmb::red::ProdR)                                                \
  NMB_RED_TYPES(X, kind, min, nmb::red::MinR)                                                  \
  NMB_RED_TYPES(X, kind, max, nmb::red::MaxR)                                                  \
  NMB_RED_TYPES(X, kind, argmin, nmb::red::ArgMinR)                                            \
  NMB_RED_TYPES(X, kind, argmax, nmb::red::ArgMaxR)
