// Hand-written fused elementwise chains linked into the runtime as builtin
// kernels.  They have exactly the shape the front-end generates for a fused
// ufunc chain (one Chain struct driven by nmb::eltwise_tile), and serve the
// C-ABI-only callers that have no NVRTC.
//
//   nmb_bcast_add_f32     out[i,j] = a[i,j] + b[0,j]      (eltwise + broadcast,
//                         numba_mlir/mlir/linalg_builder.py:297-325)
//   nmb_black_scholes_f32 the Black-Scholes chain of
//                         numba_mlir/mlir/tests/test_numpy.py:2827-2852 with
//                         float32 constants (one loop, no temporaries).
//
// Compiled with -fmad=false: the reference contracts a*b+c only under
// fastmath (mlir/lib/Conversion/GpuToGpuRuntime.cpp:2598-2631).

#include "../gpu_common.h"
#include "nmb_device.cuh"

namespace {

constexpr int kBlock = 256;

struct BcastAddChain {
  const float *a;
  const float *b;
  float *out;
  int64_t inner; // length of the broadcast row

  template <int V> struct In {
    nmb::Vec<float, V> a, b;
  };
  template <int V> struct Out {
    nmb::Vec<float, V> r;
  };
  template <int V> __device__ __forceinline__ void load(int64_t i, In<V> &in) const {
    in.a = nmb::load_stream<float, V>(a + i);
    in.b = nmb::load_reuse<float, V>(b + (i % inner));
  }
  template <int V>
  __device__ __forceinline__ void compute(const In<V> &in, Out<V> &out_) const {
#pragma unroll
    for (int l = 0; l < V; ++l)
      out_.r.v[l] = in.a.v[l] + in.b.v[l];
  }
  template <int V> __device__ __forceinline__ void store(int64_t i, const Out<V> &o) const {
    nmb::store_stream<float, V>(out + i, o.r);
  }
};

struct BlackScholesChain {
  const float *price;
  const float *strike;
  const float *t;
  float rate;
  float volatility;
  float *call;
  float *put;

  template <int V> struct In {
    nmb::Vec<float, V> p, s, t;
  };
  template <int V> struct Out {
    nmb::Vec<float, V> call, put;
  };
  template <int V> __device__ __forceinline__ void load(int64_t i, In<V> &in) const {
    in.p = nmb::load_stream<float, V>(price + i);
    in.s = nmb::load_stream<float, V>(strike + i);
    in.t = nmb::load_stream<float, V>(t + i);
  }
  template <int V>
  __device__ __forceinline__ void compute(const In<V> &in, Out<V> &o) const {
    const float mr = -rate;
    const float sig_sig_two = volatility * volatility * 2.0f;
#pragma unroll
    for (int l = 0; l < V; ++l) {
      const float P = in.p.v[l], S = in.s.v[l], T = in.t.v[l];
      const float a = nmb::f_log(nmb::f_div(P, S));
      const float b = T * mr;
      const float z = T * sig_sig_two;
      const float c = 0.25f * z;
      const float y = nmb::f_div(1.0f, nmb::f_sqrt(z));
      const float w1 = (a - b + c) * y;
      const float w2 = (a - b - c) * y;
      const float d1 = 0.5f + 0.5f * nmb::f_erf(w1);
      const float d2 = 0.5f + 0.5f * nmb::f_erf(w2);
      const float Se = nmb::f_exp(b) * S;
      const float r = P * d1 - Se * d2;
      o.call.v[l] = r;
      o.put.v[l] = r - P + Se;
    }
  }
  template <int V> __device__ __forceinline__ void store(int64_t i, const Out<V> &o) const {
    nmb::store_stream<float, V>(call + i, o.call);
    nmb::store_stream<float, V>(put + i, o.put);
  }
};

} // namespace

// Launch: grid.x = eltwise_grid(n, 256, 4, 4), block.x = 256.
// Requires 16-byte aligned a/out, 16-byte aligned b and inner % 4 == 0.
extern "C" __global__ void __launch_bounds__(kBlock)
    nmb_bcast_add_f32(const float *a, const float *b, float *out, int64_t n,
                      int64_t inner) {
  BcastAddChain chain{a, b, out, inner};
  nmb::eltwise_tile<kBlock, 4, 4>(chain, n);
}

// Same chain for unaligned pointers or inner % 4 != 0: one element per step.
extern "C" __global__ void __launch_bounds__(kBlock)
    nmb_bcast_add_f32_v1(const float *a, const float *b, float *out, int64_t n,
                         int64_t inner) {
  BcastAddChain chain{a, b, out, inner};
  nmb::eltwise_tile<kBlock, 1, 4>(chain, n);
}

// Launch: grid.x = eltwise_grid(n, 256, 4, 2), block.x = 256; all five arrays
// 16-byte aligned.
extern "C" __global__ void __launch_bounds__(kBlock)
    nmb_black_scholes_f32(const float *price, const float *strike,
                          const float *t, float rate, float volatility,
                          float *call, float *put, int64_t n) {
  BlackScholesChain chain{price, strike, t, rate, volatility, call, put};
  nmb::eltwise_tile<kBlock, 4, 2>(chain, n);
}

extern "C" __global__ void __launch_bounds__(kBlock)
    nmb_black_scholes_f32_v1(const float *price, const float *strike,
                             const float *t, float rate, float volatility,
                             float *call, float *put, int64_t n) {
  BlackScholesChain chain{price, strike, t, rate, volatility, call, put};
  nmb::eltwise_tile<kBlock, 1, 2>(chain, n);
}

NMB_REGISTER_KERNEL(nmb_bcast_add_f32, 0);
NMB_REGISTER_KERNEL(nmb_bcast_add_f32_v1, 0);
NMB_REGISTER_KERNEL(nmb_black_scholes_f32, 0);
NMB_REGISTER_KERNEL(nmb_black_scholes_f32_v1, 0);
