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
#include "smem_grant.h"

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
  const ACC defv = a.pad_zero ? (ACC)0 : (ACC)ScIo<T>::ld(static_cast<const T*>(a.default_value));
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

// Gather form: every voxel of the fine grid [B,H,W,D] sums, over the taps of the flipped, channel-swapped
// filter, the coarse voxel under the tap.  Two users:
//   * images_grad of the convolution: coarse tensor = out_grad, padded taps contribute nothing
//     (custom_helper_op/cc/kernels/sparse_conv3d_fast_op.cc:298-323);
//   * the transposed convolution itself: coarse tensor = its input, padded taps contribute default_value
//     (sparse_conv3d_fast_op.cc:383-407) - PADDED: per-(tap, channel) sums of the filter over the coarse
//     channels are formed once per CTA in shared memory, a padded tap then costs one add.
template <typename T, typename ACC, bool PADDED>
__global__ void __launch_bounds__(256) sc_dgrad_simt(const ScArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ACC* wsum = reinterpret_cast<ACC*>(smem_raw);   // [taps][Cin], PADDED only
  const T* flt = static_cast<const T*>(a.filters);
  const int taps = a.fh * a.fw * a.fd;
  if (PADDED) {
    for (int e = threadIdx.x; e < taps * a.Cin; e += blockDim.x) {
      const int t = e / a.Cin, ci = e - t * a.Cin;
      const T* w = flt + ((long long)(taps - 1 - t) * a.Cin + ci) * a.Cout;   // flipped in all three dimensions
      ACC sum = 0;
      for (int o = 0; o < a.Cout; ++o) sum += (ACC)ScIo<T>::ld(w + o);
      wsum[e] = sum;
    }
    __syncthreads();
  }
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.nvox_in * a.Cin) return;
  const int ci = (int)(idx % a.Cin);
  long long v = idx / a.Cin;
  const int dz = (int)(v % a.D); v /= a.D;
  const int c = (int)(v % a.W); v /= a.W;
  const int r = (int)(v % a.H);
  const int b = (int)(v / a.H);
  const T* og = static_cast<const T*>(a.out_grad);
  ACC acc = 0, pad = 0;
  int t = 0;
  for (int fr = 0; fr < a.fh; ++fr)
    for (int fc = 0; fc < a.fw; ++fc)
      for (int fz = 0; fz < a.fd; ++fz, ++t) {
        const long long at = sc_tap_t(a, b, r, c, dz, fr, fc, fz);
        if (at < 0) {
          if (PADDED) pad += wsum[t * a.Cin + ci];
          continue;
        }
        const T* g = og + at * a.Cout;
        const T* w = flt + ((long long)(taps - 1 - t) * a.Cin + ci) * a.Cout;
        for (int o = 0; o < a.Cout; ++o) acc += (ACC)ScIo<T>::ld(w + o) * (ACC)ScIo<T>::ld(g + o);
      }
  if (PADDED) acc += pad * (ACC)ScIo<T>::ld(static_cast<const T*>(a.default_value));
  ScIo<T>::st(static_cast<T*>(a.images_grad) + idx, acc);
}

constexpr int WG_THREADS = 256;
constexpr int WG_TM = 32;   // voxels staged per step
constexpr int WG_NC = 16;   // output channels per sweep
constexpr int WG_KPT = 4;   // k values per thread and sweep

// partial[cta][k][n] (+ partial default gradient at the end of every CTA's slab).
// TR = false: filter gradient of the convolution; the CTA's voxels are output voxels, k = (tap, input
//   channel) of the gathered image value, n = output channel of out_grad.
// TR = true: filter gradient of the TRANSPOSED convolution (sparse_conv3d_fast_op.cc:477-488); the CTA's
//   voxels are voxels of the fine grid, k = (tap, coarse channel) of the gathered coarse input (default_value
//   where the tap is padding), n = fine channel of out_grad; the reduce kernel moves element [tap][co][ci]
//   to filter_grad[flipped tap][ci][co].
template <typename T, typename ACC, bool TR>
__global__ void __launch_bounds__(WG_THREADS) sc_wgrad_partial(const ScArgs a, const int vox_per_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int taps = a.fh * a.fw * a.fd;
  const int KC = TR ? a.Cout : a.Cin;   // channels of the gathered tensor
  const int NC = TR ? a.Cin : a.Cout;   // channels of the upstream gradient
  const int K = taps * KC;
  const long long nvox = TR ? a.nvox_in : a.nvox_out;
  const int d1 = TR ? a.D : a.oD, d2 = TR ? a.W : a.oW, d3 = TR ? a.H : a.oH;
  long long* tapidx = reinterpret_cast<long long*>(smem_raw);             // [WG_TM][taps]
  ACC* gt = reinterpret_cast<ACC*>(tapidx + (size_t)WG_TM * taps);         // [WG_TM][WG_NC]
  ACC* red = gt + WG_TM * WG_NC;                                           // [WG_THREADS]
  __shared__ int4 vox[WG_TM];                                              // b, row, column, depth of a staged voxel
  const T* img = static_cast<const T*>(a.images);
  const T* flt = static_cast<const T*>(a.filters);
  const T* og = static_cast<const T*>(a.out_grad);
  const ACC defv = (ACC)ScIo<T>::ld(static_cast<const T*>(a.default_value));
  const long long v0 = (long long)blockIdx.x * vox_per_cta;
  const long long v1 = min(nvox, v0 + vox_per_cta);
  ACC* part = static_cast<ACC*>(a.workspace) + (size_t)blockIdx.x * ((size_t)K * NC + 1);
  ACC dacc = 0;

  // K = taps * channels is swept in blocks of WG_THREADS * WG_KPT accumulator rows (one block for K <= 1024)
  for (int n0 = 0; n0 < NC; n0 += WG_NC)
  for (int k0 = 0; k0 < K; k0 += WG_THREADS * WG_KPT) {
    const int nn = min(WG_NC, NC - n0);
    ACC acc[WG_KPT][WG_NC];
#pragma unroll
    for (int i = 0; i < WG_KPT; ++i)
#pragma unroll
      for (int n = 0; n < WG_NC; ++n) acc[i][n] = 0;

    for (long long vt = v0; vt < v1; vt += WG_TM) {
      const int tm = (int)min((long long)WG_TM, v1 - vt);
      __syncthreads();
      // voxel coordinates once per voxel (64-bit divisions), then the tap table with 32-bit arithmetic
      if (threadIdx.x < tm) {
        long long v = vt + threadIdx.x;
        const int dz = (int)(v % d1); v /= d1;
        const int co = (int)(v % d2); v /= d2;
        vox[threadIdx.x] = make_int4((int)(v / d3), (int)(v % d3), co, dz);
      }
      for (int e = threadIdx.x; e < tm * WG_NC; e += WG_THREADS) {
        const int m = e / WG_NC, n = e - m * WG_NC;
        gt[e] = n < nn ? (ACC)ScIo<T>::ld(og + (vt + m) * NC + n0 + n) : (ACC)0;
      }
      __syncthreads();
      for (int e = threadIdx.x; e < tm * taps; e += WG_THREADS) {
        const int m = e / taps, t = e - m * taps;
        const int4 c4 = vox[m];
        const int fz = t % a.fd, fc = (t / a.fd) % a.fw, fr = t / a.fd / a.fw;
        tapidx[e] = TR ? sc_tap_t(a, c4.x, c4.y, c4.z, c4.w, fr, fc, fz) : sc_tap(a, c4.x, c4.y, c4.z, c4.w, fr, fc, fz);
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < WG_KPT; ++i) {
        const int k = k0 + threadIdx.x + i * WG_THREADS;
        if (k >= K) break;
        const int t = k / KC, ci = k - t * KC;
        for (int m = 0; m < tm; ++m) {
          const long long at = tapidx[m * taps + t];
          const ACC x = at < 0 ? defv : (ACC)ScIo<T>::ld(img + at * KC + ci);
          const ACC* g = gt + m * WG_NC;
#pragma unroll
          for (int n = 0; n < WG_NC; ++n) acc[i][n] += x * g[n];
          if (!TR && at < 0 && a.dynamic_default) {
            // fixed_param_op_gpu.cu.cc:273-277: d(default) collects filter*out_grad over the padded taps
            const T* w = flt + (long long)k * a.Cout + n0;
            for (int n = 0; n < nn; ++n) dacc += (ACC)ScIo<T>::ld(w + n) * g[n];
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < WG_KPT; ++i) {
      const int k = k0 + threadIdx.x + i * WG_THREADS;
      if (k >= K) break;
#pragma unroll
      for (int n = 0; n < WG_NC; ++n)
        if (n < nn) part[(size_t)k * NC + n0 + n] = acc[i][n];
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
  if (threadIdx.x == 0) part[(size_t)K * NC] = red[0];
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

// Transposed convolution: partial element [tap][co][ci] -> filter_grad[taps-1-tap][ci][co].
template <typename ACC, typename OUT>
__global__ void sc_wgrad_reduce_t(const ACC* part, int nparts, int taps, int Cin, int Cout, OUT* filter_grad) {
  const long long n_el = (long long)taps * Cin * Cout;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_el) return;
  ACC s = 0;
  for (int p = 0; p < nparts; ++p) s += part[(size_t)p * (n_el + 1) + e];
  const int ci = (int)(e % Cin), co = (int)((e / Cin) % Cout), t = (int)(e / ((long long)Cin * Cout));
  filter_grad[((long long)(taps - 1 - t) * Cin + ci) * Cout + co] = (OUT)s;
}

// SparsePad (custom_helper_op/cc/kernels/sparse_pad_kernels_gpu.cu.cc:36-64): the coarse band [B,h,w,d,C]
// placed into the fine band [B,h*sr,w*sc,d*sd,C] whose first plane per pixel is base_plane; a fine voxel
// receives a coarse value iff its row, column and absolute depth are multiples of the strides, else zero.
// One thread per 16-byte piece of a fine voxel's channel vector (E elements).
// I: index type of the flattened thread index - unsigned where the element count allows it (64-bit divisions cost
// several times the copy itself)
template <typename T, int E, typename I>
__global__ void __launch_bounds__(256) sc_pad_fwd(const T* img, const int* bp, T* out, int B, int h, int w, int d, int C,
                                                   int sr, int sc, int sd) {
  const int cv = C / E;
  const I idx = (I)blockIdx.x * blockDim.x + threadIdx.x;
  const int oh = h * sr, ow = w * sc, od = d * sd;
  if ((long long)idx >= (long long)B * oh * ow * od * cv) return;
  const int q = (int)(idx % cv);
  I v = idx / cv;
  int z = (int)(v % od);
  const I pos = v / od;
  const int x = (int)(pos % ow), y = (int)((pos / ow) % oh), b = (int)(pos / ow / oh);
  const int p0 = __ldg(bp + pos);
  z = z + p0 - ((p0 + sd - 1) / sd) * sd;
  struct alignas(sizeof(T) * E) Vec { T e[E]; };
  Vec val;
#pragma unroll
  for (int i = 0; i < E; ++i) val.e[i] = T(0);
  if ((y % sr) == 0 && (x % sc) == 0 && (z % sd) == 0)   // z > -sd, so a negative z is never a multiple
    val = *reinterpret_cast<const Vec*>(img + ((((long long)b * h + y / sr) * w + x / sc) * d + z / sd) * C + q * E);
  *reinterpret_cast<Vec*>(out + (long long)v * C + q * E) = val;
}

// SparsePadGrad: every coarse voxel reads the fine voxel it was copied to - pixel (y*sr, x*sc), plane
// z*sd + ceil(bp/sd)*sd - bp.  (The reference kernel, :82-104, forms the fine pixel index from the coarse
// row and column before scaling them and so reads another pixel when sr or sc exceeds 1.)
template <typename T, int E, typename I>
__global__ void __launch_bounds__(256) sc_pad_bwd(const T* og, const int* bp, T* igrad, int B, int h, int w, int d, int C,
                                                   int sr, int sc, int sd) {
  const int cv = C / E;
  const I idx = (I)blockIdx.x * blockDim.x + threadIdx.x;
  if ((long long)idx >= (long long)B * h * w * d * cv) return;
  const int q = (int)(idx % cv);
  I v = idx / cv;
  const int z = (int)(v % d);
  const I pc = v / d;
  const int x = (int)(pc % w), y = (int)((pc / w) % h), b = (int)(pc / w / h);
  const long long pos = ((long long)b * h * sr + (long long)y * sr) * ((long long)w * sc) + (long long)x * sc;
  const int p0 = __ldg(bp + pos);
  const int zf = z * sd + ((p0 + sd - 1) / sd) * sd - p0;
  struct alignas(sizeof(T) * E) Vec { T e[E]; };
  *reinterpret_cast<Vec*>(igrad + (long long)v * C + q * E) =
      *reinterpret_cast<const Vec*>(og + (pos * ((long long)d * sd) + zf) * C + q * E);
}

template <typename T>
int pad_t(bool grad, const void* src, const int* bp, void* dst, int B, int h, int w, int d, int C, int sr, int sc, int sd,
          cudaStream_t st) {
  constexpr int EV = 16 / (int)sizeof(T);
  const bool vec = (C % EV) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  const long long nv = grad ? (long long)B * h * w * d : (long long)B * h * sr * w * sc * d * sd;
  const long long n = nv * (vec ? C / EV : C);
  const unsigned grid = (unsigned)((n + 255) / 256);
  const T* s = static_cast<const T*>(src);
  T* o = static_cast<T*>(dst);
  const bool small = n + 256 < 0xffffffffLL;   // the thread index (rounded up to the grid) fits 32 bits
#define CHOP_PAD_GO(K, EE)                                                                              \
  do {                                                                                                  \
    if (small) K<T, EE, unsigned><<<grid, 256, 0, st>>>(s, bp, o, B, h, w, d, C, sr, sc, sd);           \
    else K<T, EE, long long><<<grid, 256, 0, st>>>(s, bp, o, B, h, w, d, C, sr, sc, sd);                \
  } while (0)
  if (grad) {
    if (vec) CHOP_PAD_GO(sc_pad_bwd, EV); else CHOP_PAD_GO(sc_pad_bwd, 1);
  } else {
    if (vec) CHOP_PAD_GO(sc_pad_fwd, EV); else CHOP_PAD_GO(sc_pad_fwd, 1);
  }
#undef CHOP_PAD_GO
  return (int)cudaGetLastError();
}

template <typename T, typename ACC>
int fwd_t(const ScArgs& a, cudaStream_t st) {
  const long long n = a.nvox_out * a.Cout;
  sc_fwd_simt<T, ACC><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}
template <typename T, typename ACC>
int dgrad_t(const ScArgs& a, bool padded, cudaStream_t st) {
  const long long n = a.nvox_in * a.Cin;
  if (padded) {
    const size_t smem = (size_t)a.fh * a.fw * a.fd * a.Cin * sizeof(ACC);
    sc_dgrad_simt<T, ACC, true><<<(unsigned)((n + 255) / 256), 256, smem, st>>>(a);
  } else {
    sc_dgrad_simt<T, ACC, false><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a);
  }
  return (int)cudaGetLastError();
}
template <typename T, typename ACC, typename OUT, bool TR>
int wgrad_t(const ScArgs& a, int nparts, cudaStream_t st) {
  const int taps = a.fh * a.fw * a.fd;
  const long long n_el = (long long)taps * a.Cin * a.Cout;
  const long long nvox = TR ? a.nvox_in : a.nvox_out;
  const int vox_per_cta = (int)((nvox + nparts - 1) / nparts);
  const size_t smem = (size_t)WG_TM * taps * sizeof(long long) + (size_t)(WG_TM * WG_NC + WG_THREADS) * sizeof(ACC);
  auto k = sc_wgrad_partial<T, ACC, TR>;
  if (int e = grant_smem(k, smem)) return e;
  k<<<nparts, WG_THREADS, smem, st>>>(a, vox_per_cta);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (TR)
    sc_wgrad_reduce_t<ACC, OUT><<<(unsigned)((n_el + 255) / 256), 256, 0, st>>>(
        static_cast<const ACC*>(a.workspace), nparts, taps, a.Cin, a.Cout, static_cast<OUT*>(a.filter_grad));
  else
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
    case 0: return wgrad_t<float, float, float, false>(a, nparts, st);
    case 1: return wgrad_t<double, double, double, false>(a, nparts, st);
    default: return wgrad_t<__nv_bfloat16, float, float, false>(a, nparts, st);
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
    case 0: return dgrad_t<float, float>(a, false, st);
    case 1: return dgrad_t<double, double>(a, false, st);
    default: return dgrad_t<__nv_bfloat16, float>(a, false, st);
  }
}
// Transposed convolution forward: a.out_grad = the coarse input, a.images_grad = the fine output.
int sc_tconv_simt_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  switch (dtype) {
    case 0: return dgrad_t<float, float>(a, true, st);
    case 1: return dgrad_t<double, double>(a, true, st);
    default: return dgrad_t<__nv_bfloat16, float>(a, true, st);
  }
}
// Filter gradient of the transposed convolution: a.images = the coarse input, a.out_grad = the fine gradient.
int sc_twgrad_simt_launch(int dtype, const ScArgs& a, int nparts, cudaStream_t st) {
  switch (dtype) {
    case 0: return wgrad_t<float, float, float, true>(a, nparts, st);
    case 1: return wgrad_t<double, double, double, true>(a, nparts, st);
    default: return wgrad_t<__nv_bfloat16, float, float, true>(a, nparts, st);
  }
}
int sc_wgrad_simt_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  const int nparts = sc_wgrad_parts(a.nvox_out);
  switch (dtype) {
    case 0: return wgrad_t<float, float, float, false>(a, nparts, st);
    case 1: return wgrad_t<double, double, double, false>(a, nparts, st);
    default: return wgrad_t<__nv_bfloat16, float, float, false>(a, nparts, st);
  }
}

int sc_pad_launch(int dtype, bool grad, const void* src, const int* base_plane, void* dst, int B, int h, int w, int d,
                  int C, int sr, int sc, int sd, cudaStream_t st) {
  switch (dtype) {
    case 0: return pad_t<float>(grad, src, base_plane, dst, B, h, w, d, C, sr, sc, sd, st);
    case 1: return pad_t<double>(grad, src, base_plane, dst, B, h, w, d, C, sr, sc, sd, st);
    default: return pad_t<unsigned short>(grad, src, base_plane, dst, B, h, w, d, C, sr, sc, sd, st);
  }
}

}  // namespace chop
