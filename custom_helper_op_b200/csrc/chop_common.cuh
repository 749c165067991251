// Shared device helpers for the cost-volume kernels: unfused IEEE arithmetic, vector loads/stores of
// a lane's channel slice, vector reductions into global memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace chop {

// ---------------------------------------------------------------------------------------------
// Unfused arithmetic.  The compiler never contracts these intrinsics into fused multiply-adds, so a
// chain written with them is the same sequence of correctly rounded IEEE operations as the scalar
// C++ of the reference compiled without contraction.  Everything that decides a sample's validity
// or its texel (the homography projection) goes through these, which is what makes the validity
// count and the MIN arg-indices exact.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float xmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float xadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float xsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float xdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double xmul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double xadd(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double xsub(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ double xdiv(double a, double b) { return __ddiv_rn(a, b); }

__device__ __forceinline__ float xfma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double xfma(double a, double b, double c) { return fma(a, b, c); }

template <typename R> struct Lim;
template <> struct Lim<float> {
  __device__ static float max() { return 3.402823466e+38f; }
  __device__ static float min_pos() { return 1.175494351e-38f; }
};
template <> struct Lim<double> {
  __device__ static double max() { return 1.7976931348623157e+308; }
  __device__ static double min_pos() { return 2.2250738585072014e-308; }
};

// ---------------------------------------------------------------------------------------------
// A lane owns CPL consecutive channels.  load_vec reads them as one 4/8/16-byte access (the host
// guarantees C % CPL == 0 and pointer alignment) and widens to the compute type R.
// ---------------------------------------------------------------------------------------------
template <typename T, typename R, int CPL>
struct Vec;

template <> struct Vec<float, float, 1> {
  static __device__ __forceinline__ void load(const float* p, float* o) { o[0] = __ldg(p); }
};
template <> struct Vec<float, float, 2> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    float2 v = __ldg(reinterpret_cast<const float2*>(p)); o[0] = v.x; o[1] = v.y;
  }
};
template <> struct Vec<float, float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    float4 v = __ldg(reinterpret_cast<const float4*>(p)); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec<double, double, 1> {
  static __device__ __forceinline__ void load(const double* p, double* o) { o[0] = __ldg(p); }
};
template <> struct Vec<double, double, 2> {
  static __device__ __forceinline__ void load(const double* p, double* o) {
    double2 v = __ldg(reinterpret_cast<const double2*>(p)); o[0] = v.x; o[1] = v.y;
  }
};
template <> struct Vec<__nv_bfloat16, float, 1> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    unsigned short u = __ldg(reinterpret_cast<const unsigned short*>(p));
    o[0] = __uint_as_float(((unsigned)u) << 16);
  }
};
template <> struct Vec<__nv_bfloat16, float, 2> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    unsigned u = __ldg(reinterpret_cast<const unsigned*>(p));
    o[0] = __uint_as_float(u << 16); o[1] = __uint_as_float(u & 0xffff0000u);
  }
};
template <> struct Vec<__nv_bfloat16, float, 4> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u);
    o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
  }
};
template <> struct Vec<__nv_bfloat16, float, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u);
    o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
    o[4] = __uint_as_float(u.z << 16); o[5] = __uint_as_float(u.z & 0xffff0000u);
    o[6] = __uint_as_float(u.w << 16); o[7] = __uint_as_float(u.w & 0xffff0000u);
  }
};

// Streaming (evict-first) store of K consecutive values of R / int32: the cost volume is written once
// and never re-read by this kernel, so it should not displace the feature maps from L2.
template <typename R, int K>
__device__ __forceinline__ void store_stream(R* p, const R* v) {
  if constexpr (sizeof(R) == 4 && K % 4 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 4)
      __stcs(reinterpret_cast<float4*>(p + i),
             make_float4(__int_as_float(*(const int*)&v[i]), __int_as_float(*(const int*)&v[i + 1]),
                         __int_as_float(*(const int*)&v[i + 2]), __int_as_float(*(const int*)&v[i + 3])));
  } else if constexpr (sizeof(R) == 4 && K % 2 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 2)
      __stcs(reinterpret_cast<float2*>(p + i),
             make_float2(__int_as_float(*(const int*)&v[i]), __int_as_float(*(const int*)&v[i + 1])));
  } else if constexpr (sizeof(R) == 8 && K % 2 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 2)
      __stcs(reinterpret_cast<double2*>(p + i),
             make_double2(__longlong_as_double(*(const long long*)&v[i]),
                          __longlong_as_double(*(const long long*)&v[i + 1])));
  } else {
#pragma unroll
    for (int i = 0; i < K; ++i) __stcs(p + i, v[i]);
  }
}

// Streaming load of K consecutive R values that are read exactly once (upstream gradient).
template <typename R, int K>
__device__ __forceinline__ void load_stream(const R* p, R* v) {
  if constexpr (sizeof(R) == 4 && K % 4 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 4) {
      float4 t = __ldcs(reinterpret_cast<const float4*>(p + i));
      v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
    }
  } else if constexpr (sizeof(R) == 4 && K % 2 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 2) {
      float2 t = __ldcs(reinterpret_cast<const float2*>(p + i));
      v[i] = t.x; v[i + 1] = t.y;
    }
  } else if constexpr (sizeof(R) == 8 && K % 2 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 2) {
      double2 t = __ldcs(reinterpret_cast<const double2*>(p + i));
      v[i] = t.x; v[i + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < K; ++i) v[i] = __ldcs(p + i);
  }
}

// Sum K consecutive values into global memory without returning the old value.  float uses the
// 16-byte vector reduction of sm_90+ where the slice allows it; double falls back to scalar atomics.
template <typename R, int K>
__device__ __forceinline__ void red_add(R* p, const R* v) {
  if constexpr (sizeof(R) == 4 && K % 4 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 4)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + i), "f"(v[i]), "f"(v[i + 1]),
                   "f"(v[i + 2]), "f"(v[i + 3])
                   : "memory");
  } else if constexpr (sizeof(R) == 4 && K % 2 == 0) {
#pragma unroll
    for (int i = 0; i < K; i += 2)
      asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p + i), "f"(v[i]), "f"(v[i + 1]) : "memory");
  } else {
#pragma unroll
    for (int i = 0; i < K; ++i) atomicAdd(p + i, v[i]);
  }
}

// Arguments shared by the forward and backward cost-volume kernels (device pointers, validated and
// narrowed on the host).
struct CvArgs {
  const void* ref;
  const void* src;
  const void* depth;    // base_plane [B,H,W] or depth_grid [B,H,W,D]
  const void* offsets;  // [B,D] or null
  const void* Rs;
  const void* Ts;
  void* cost;
  int* mask;
  const void* cost_grad;
  void* ref_grad;
  void* src_grad;
  void* depth_grad;
  int B, H, W, C, D, N, Hs, Ws, G;
  int d_begin, d_end;
  int half_centor;
  int lg_log2;     // log2(lanes that share one pixel)
  int chunk;       // depth planes per warp work item
  int nchunks;
  int npb;         // pixel blocks = ceil(B*H*W / pixels per warp)
  long long npix;  // B*H*W
};

}  // namespace chop
