// Generic manifold-convolution kernels (any filter size, stride, dilation; float32, float64, bfloat16
// storage with float32 accumulation).  They are the complete, shape-agnostic implementation of
// SparseConv3DFast / SparseConv3DFastGrad; the tensor-core kernel in sc_umma.cu takes over for the
// bf16 3x3x3 stride-1 case.
//
// forward / image gradient: one thread per (voxel, output channel); the 32 threads of a warp share
//   voxels, so image values are broadcast loads and filter rows are coalesced.
// filter gradient: every CTA takes a contiguous slice of the output voxels and accumulates a private
//   [K = taps*Cin, Cout] partial product in registers (thread <-> k, 16 output channels at a time);
//   partials go to a workspace and a second kernel sums them in a fixed order (deterministic, no atomics).
#include "sc_common.cuh"
#include "sc_entry.h"

#include <mutex>

namespace chop {
namespace {

// Scratch for chop_sparse_conv3d_bwd_noalloc: the per-CTA partial filter gradients live in this
// file-scope device array instead of caller memory.  Every GPU that loads the library holds these
// 4 MiB until the process exits.  In host code the name below is only a host-side stand-in for the
// symbol - it is NOT a device address; the address a kernel may use comes from cudaGetSymbolAddress.
constexpr size_t kStaticScratchBytes = (size_t)4 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

template <typename T, typename ACC>
__global__ void __launch_bounds__(256) sc_fwd_simt(const ScArgs a) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.nvox_out * a.Cout) return;
  const int oc = (int)(idx % a.Cout);
  long long v = idx / a.Cout;
  const int dz = (int)(v % a.oD); v /= a.oD;
  const int co = (int)(v % a.oW); v /= a.oW;
  const int ro = (int)(v % a.oH);
  const int b = (int)(v / a.oH);
  const T* img = static_cast<const T*>(a.images);
  const T* flt = static_cast<const T*>(a.filters);
  const ACC defv = (ACC)ScIo<T>::ld(static_cast<const T*>(a.default_value));
  ACC acc = 0;
  for (int fr = 0; fr < a.fh; ++fr)
    for (int fc = 0; fc < a.fw; ++fc)
      for (int fz = 0; fz < a.fd; ++fz) {
        const long long at = sc_tap(a, b, ro, co, dz, fr, fc, fz);
        const T* w = flt + ((long long)(fr * a.fw + fc) * a.fd + fz) * a.Cin * a.Cout + oc;
        if (at < 0) {
          for (int ci = 0; ci < a.Cin; ++ci) acc += (ACC)ScIo<T>::ld(w + (long long)ci * a.Cout) * defv;
        } else {
          const T* x = img + at * a.Cin;
          for (int ci = 0; ci < a.Cin; ++ci)
            acc += (ACC)ScIo<T>::ld(w + (long long)ci * a.Cout) * (ACC)ScIo<T>::ld(x + ci);
        }
      }
  ScIo<T>::st(static_cast<T*>(a.output) + idx, acc);
}

// images_grad in gather form: the forward run over out_grad with the flipped, channel-swapped filter,
// zero padding value and right padding (custom_helper_op/cc/kernels/sparse_conv3d_fast_op.cc:298-323).
template <typename T, typename ACC>
__global__ void __launch_bounds__(256) sc_dgrad_simt(const ScArgs a) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.nvox_in * a.Cin) return;
  const int ci = (int)(idx % a.Cin);
  long long v = idx / a.Cin;
  const int dz = (int)(v % a.D); v /= a.D;
  const int c = (int)(v % a.W); v /= a.W;
  const int r = (int)(v % a.H);
  const int b = (int)(v / a.H);
  const T* og = static_cast<const T*>(a.out_grad);
  const T* flt = static_cast<const T*>(a.filters);
  const int qr = (a.fh - 1) * a.dr - a.pr, qc = (a.fw - 1) * a.dc - a.pc, qd = (a.fd - 1) * a.dd - a.pd;
  const int depth = dz + __ldg(a.base_plane + (b * a.H + r) * a.W + c);
  ACC acc = 0;
  for (int fr = 0; fr < a.fh; ++fr)
    for (int fc = 0; fc < a.fw; ++fc)
      for (int fz = 0; fz < a.fd; ++fz) {
        const int orow = r - qr + fr * a.dr, ocol = c - qc + fc * a.dc;
        if (oob(orow, a.H) || oob(ocol, a.W)) continue;
        int od = depth - qd + fz * a.dd;
        if ((orow % a.sr) != 0 || (ocol % a.sc) != 0 || (od % a.sd) != 0) continue;
        od = od / a.sd - (__ldg(a.base_plane + (b * a.H + orow) * a.W + ocol) + a.sd - 1) / a.sd;
        if (oob(od, a.oD)) continue;
        const T* g = og + ((((long long)b * a.oH + orow / a.sr) * a.oW + ocol / a.sc) * a.oD + od) * a.Cout;
        const T* w = flt + (((long long)(a.fh - 1 - fr) * a.fw + (a.fw - 1 - fc)) * a.fd + (a.fd - 1 - fz)) * a.Cin * a.Cout +
                     (long long)ci * a.Cout;
        for (int o = 0; o < a.Cout; ++o) acc += (ACC)ScIo<T>::ld(w + o) * (ACC)ScIo<T>::ld(g + o);
      }
  ScIo<T>::st(static_cast<T*>(a.images_grad) + idx, acc);
}

constexpr int WG_THREADS = 256;
constexpr int WG_TM = 32;   // voxels staged per step
constexpr int WG_NC = 16;   // output channels per sweep
constexpr int WG_KPT = 4;   // k values per thread -> K <= 1024

// partial[cta][k][n] (+ partial default gradient at the end of every CTA's slab)
template <typename T, typename ACC>
__global__ void __launch_bounds__(WG_THREADS) sc_wgrad_partial(const ScArgs a, const int vox_per_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int taps = a.fh * a.fw * a.fd;
  const int K = taps * a.Cin;
  long long* tapidx = reinterpret_cast<long long*>(smem_raw);             // [WG_TM][taps]
  ACC* gt = reinterpret_cast<ACC*>(tapidx + (size_t)WG_TM * taps);         // [WG_TM][WG_NC]
  ACC* red = gt + WG_TM * WG_NC;                                           // [WG_THREADS]
  const T* img = static_cast<const T*>(a.images);
  const T* flt = static_cast<const T*>(a.filters);
  const T* og = static_cast<const T*>(a.out_grad);
  const ACC defv = (ACC)ScIo<T>::ld(static_cast<const T*>(a.default_value));
  const long long v0 = (long long)blockIdx.x * vox_per_cta;
  const long long v1 = min(a.nvox_out, v0 + vox_per_cta);
  ACC* part = static_cast<ACC*>(a.workspace) + (size_t)blockIdx.x * ((size_t)K * a.Cout + 1);
  ACC dacc = 0;

  for (int n0 = 0; n0 < a.Cout; n0 += WG_NC) {
    const int nn = min(WG_NC, a.Cout - n0);
    ACC acc[WG_KPT][WG_NC];
#pragma unroll
    for (int i = 0; i < WG_KPT; ++i)
#pragma unroll
      for (int n = 0; n < WG_NC; ++n) acc[i][n] = 0;

    for (long long vt = v0; vt < v1; vt += WG_TM) {
      const int tm = (int)min((long long)WG_TM, v1 - vt);
      __syncthreads();
      for (int e = threadIdx.x; e < tm * taps; e += WG_THREADS) {
        const int m = e / taps, t = e - m * taps;
        long long v = vt + m;
        const int dz = (int)(v % a.oD); v /= a.oD;
        const int co = (int)(v % a.oW); v /= a.oW;
        const int ro = (int)(v % a.oH);
        const int b = (int)(v / a.oH);
        const int fz = t % a.fd, fc = (t / a.fd) % a.fw, fr = t / a.fd / a.fw;
        tapidx[m * taps + t] = sc_tap(a, b, ro, co, dz, fr, fc, fz);
      }
      for (int e = threadIdx.x; e < tm * WG_NC; e += WG_THREADS) {
        const int m = e / WG_NC, n = e - m * WG_NC;
        gt[e] = n < nn ? (ACC)ScIo<T>::ld(og + (vt + m) * a.Cout + n0 + n) : (ACC)0;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < WG_KPT; ++i) {
        const int k = threadIdx.x + i * WG_THREADS;
        if (k >= K) break;
        const int t = k / a.Cin, ci = k - t * a.Cin;
        for (int m = 0; m < tm; ++m) {
          const long long at = tapidx[m * taps + t];
          const ACC x = at < 0 ? defv : (ACC)ScIo<T>::ld(img + at * a.Cin + ci);
          const ACC* g = gt + m * WG_NC;
#pragma unroll
          for (int n = 0; n < WG_NC; ++n) acc[i][n] += x * g[n];
          if (at < 0 && a.dynamic_default) {
            // fixed_param_op_gpu.cu.cc:273-277: d(default) collects filter*out_grad over the padded taps
            const T* w = flt + (long long)k * a.Cout + n0;
            for (int n = 0; n < nn; ++n) dacc += (ACC)ScIo<T>::ld(w + n) * g[n];
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < WG_KPT; ++i) {
      const int k = threadIdx.x + i * WG_THREADS;
      if (k >= K) break;
#pragma unroll
      for (int n = 0; n < WG_NC; ++n)
        if (n < nn) part[(size_t)k * a.Cout + n0 + n] = acc[i][n];
    }
  }
  // block sum of the default-value gradient
  __syncthreads();
  red[threadIdx.x] = dacc;
  __syncthreads();
  for (int o = WG_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) part[(size_t)K * a.Cout] = red[0];
}

// filter_grad[e] = sum over CTAs of partial[cta][e]; element K*Cout is the default-value gradient.
template <typename ACC, typename OUT>
__global__ void sc_wgrad_reduce(const ACC* part, int nparts, long long n_el, OUT* filter_grad, OUT* default_grad) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e > n_el) return;
  ACC s = 0;
  for (int p = 0; p < nparts; ++p) s += part[(size_t)p * (n_el + 1) + e];
  if (e < n_el) filter_grad[e] = (OUT)s;
  else *default_grad = (OUT)s;
}

template <typename T, typename ACC>
int fwd_t(const ScArgs& a, cudaStream_t st) {
  const long long n = a.nvox_out * a.Cout;
  sc_fwd_simt<T, ACC><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}
template <typename T, typename ACC>
int dgrad_t(const ScArgs& a, cudaStream_t st) {
  const long long n = a.nvox_in * a.Cin;
  sc_dgrad_simt<T, ACC><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}
template <typename T, typename ACC, typename OUT>
int wgrad_t(const ScArgs& a, int nparts, cudaStream_t st) {
  const int taps = a.fh * a.fw * a.fd;
  const long long n_el = (long long)taps * a.Cin * a.Cout;
  const int vox_per_cta = (int)((a.nvox_out + nparts - 1) / nparts);
  const size_t smem = (size_t)WG_TM * taps * sizeof(long long) + (size_t)(WG_TM * WG_NC + WG_THREADS) * sizeof(ACC);
  auto k = sc_wgrad_partial<T, ACC>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  k<<<nparts, WG_THREADS, smem, st>>>(a, vox_per_cta);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  sc_wgrad_reduce<ACC, OUT><<<(unsigned)((n_el + 1 + 255) / 256), 256, 0, st>>>(
      static_cast<const ACC*>(a.workspace), nparts, n_el, static_cast<OUT*>(a.filter_grad),
      static_cast<OUT*>(a.default_grad));
  return (int)cudaGetLastError();
}

}  // namespace

// Device address of g_static_scratch for the CURRENT device, looked up once per device (first call on
// that device, with that device current) and cached.  Returns a cudaError_t value.
int sc_static_scratch(void** ptr, size_t* bytes) {
  constexpr int kMaxDevices = 64;
  static void* cached[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    cached[dev] = p;
  }
  *ptr = cached[dev];
  *bytes = kStaticScratchBytes;
  return 0;
}

// Filter gradient with a caller-chosen number of partial slabs (the workspace holds nparts slabs).
int sc_wgrad_simt_launch_parts(int dtype, const ScArgs& a, int nparts, cudaStream_t st) {
  switch (dtype) {
    case 0: return wgrad_t<float, float, float>(a, nparts, st);
    case 1: return wgrad_t<double, double, double>(a, nparts, st);
    default: return wgrad_t<__nv_bfloat16, float, float>(a, nparts, st);
  }
}

int sc_wgrad_parts(long long nvox_out) {
  long long p = (nvox_out + 511) / 512;  // at least 512 voxels per CTA
  if (p > 148 * 4) p = 148 * 4;
  if (p < 1) p = 1;
  return (int)p;
}

size_t sc_wgrad_workspace_bytes(int dtype, int taps, int Cin, int Cout, long long nvox_out) {
  const size_t acc = dtype == 1 ? 8 : 4;
  return (size_t)sc_wgrad_parts(nvox_out) * ((size_t)taps * Cin * Cout + 1) * acc;
}

int sc_fwd_simt_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  switch (dtype) {
    case 0: return fwd_t<float, float>(a, st);
    case 1: return fwd_t<double, double>(a, st);
    default: return fwd_t<__nv_bfloat16, float>(a, st);
  }
}
int sc_dgrad_simt_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  switch (dtype) {
    case 0: return dgrad_t<float, float>(a, st);
    case 1: return dgrad_t<double, double>(a, st);
    default: return dgrad_t<__nv_bfloat16, float>(a, st);
  }
}
int sc_wgrad_simt_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  const int nparts = sc_wgrad_parts(a.nvox_out);
  switch (dtype) {
    case 0: return wgrad_t<float, float, float>(a, nparts, st);
    case 1: return wgrad_t<double, double, double>(a, nparts, st);
    default: return wgrad_t<__nv_bfloat16, float, float>(a, nparts, st);
  }
}

}  // namespace chop
