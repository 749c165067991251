// TEST INFRASTRUCTURE ONLY.  Host-side stand-ins for the handful of TensorFlow GPU helpers the
// reference's kernel bodies use, so that those bodies (read from the reference checkout at build
// time, never stored in this repository) compile as ordinary C++ and run on CPU cores.
//
//   __global__               -> nothing (a plain function template)
//   GpuGridRangeX<I>(count)  -> the half-open index range [ref_shim::lo, ref_shim::hi) of the
//                               calling host thread, clipped to count (one "virtual thread" sweep)
//   GpuAtomicAdd(p, v)       -> an OpenMP atomic update
//   __ldg / ldg              -> a plain load
//
// Nothing in the shipped library includes this header.
#pragma once
#include <algorithm>
#include <cstdint>
#include <limits>

#define __global__
#define __restrict__

typedef int32_t int32;
typedef int64_t int64;

namespace ref_shim {
extern thread_local int64 lo;
extern thread_local int64 hi;

template <typename I>
struct Range {
  I b, e;
  struct It {
    I i;
    I operator*() const { return i; }
    It& operator++() { ++i; return *this; }
    bool operator!=(const It& o) const { return i != o.i; }
  };
  It begin() const { return It{b}; }
  It end() const { return It{e}; }
};
}  // namespace ref_shim

template <typename I>
inline ref_shim::Range<I> GpuGridRangeX(I count) {
  int64 b = std::min<int64>(ref_shim::lo, (int64)count);
  int64 e = std::min<int64>(ref_shim::hi, (int64)count);
  return ref_shim::Range<I>{(I)b, (I)e};
}

template <typename T>
inline void GpuAtomicAdd(T* p, T v) {
#pragma omp atomic
  *p += v;
}

template <typename T>
inline T __ldg(const T* p) { return *p; }
template <typename T>
inline T ldg(const T* p) { return *p; }
