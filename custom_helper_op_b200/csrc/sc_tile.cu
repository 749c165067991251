// Register-tiled CUDA-core manifold convolution for float32 data (the reference's own dtype) and for bfloat16 storage
// with float32 accumulation where the tensor-core kernels do not apply (8 channels, other filter sizes, dilation):
// forward, gather-form image gradient, transposed forward and filter gradient, any filter size / stride / dilation,
// 8, 16 or 32 channels on either side.
//
// One thread owns four consecutive voxels (two for 32 output channels) and all output channels: per tap it loads
// their gathered channel vectors once (16-byte loads) and multiplies them with the tap's [gathered x produced] weight block, which the CTA
// keeps in shared memory and reads with warp-uniform 16-byte loads (every weight load feeds 16 FMAs).
// Padded taps add default_value times a per-(tap, produced channel) weight sum that is formed once per CTA.
// The shape-agnostic one-thread-per-output-element kernels of sc_simt.cu remain the fallback (other channel counts,
// float64, filters whose weights do not fit in shared memory).
#include "sc_common.cuh"
#include "sc_entry.h"
#include "smem_grant.h"

namespace chop {
namespace {

// Storage type T: float, or bfloat16 widened to float on load and rounded on store (float32 accumulation).
template <typename T> struct TileIo;
template <> struct TileIo<float> {
  static __device__ __forceinline__ float ld1(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ float4 ld4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ void st4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  }
};
template <> struct TileIo<__nv_bfloat16> {
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return ScIo<__nv_bfloat16>::ld(p); }
  static __device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
  }
  static __device__ __forceinline__ void st4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
  }
};

// FORM 0: forward - voxels of the output grid gather the input grid (sc_tap); weights w[t][ci][co].
// FORM 1: gather form - voxels of the fine grid gather the coarse grid (sc_tap_t); the gathered tensor has Cout
//         channels, the produced one Cin, weights flipped: w'[t][co][ci] = filter[taps-1-t][ci][co].
// A thread owns VPT consecutive voxels (in linear order - the weights are shared by all voxels, so any grouping
// works) and all NCH produced channels: every 16-byte weight load from shared memory feeds 4*VPT FMAs.
template <int NCH>
struct TileVpt { static constexpr int v = NCH <= 16 ? 4 : 2; };   // 4*NCH accumulators beyond 16 channels would spill

template <typename T, int KCH, int NCH, int FORM>
__global__ void __launch_bounds__(128, 3) sc_tile_kernel(const ScArgs a, const long long nvox) {
  constexpr int VPT = TileVpt<NCH>::v;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int taps = a.fh * a.fw * a.fd;
  float* ws = reinterpret_cast<float*>(smem_raw);          // [taps][KCH][NCH]
  float* wsum = ws + (size_t)taps * KCH * NCH;              // [taps][NCH]
  const T* flt = static_cast<const T*>(a.filters);
  for (int e = threadIdx.x; e < taps * KCH * NCH; e += blockDim.x) {
    const int n = e % NCH, k = (e / NCH) % KCH, t = e / (NCH * KCH);
    ws[e] = FORM == 0 ? TileIo<T>::ld1(flt + e) : TileIo<T>::ld1(flt + ((size_t)(taps - 1 - t) * NCH + n) * KCH + k);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < taps * NCH; e += blockDim.x) {
    const int n = e % NCH, t = e / NCH;
    float s = 0.f;
    for (int k = 0; k < KCH; ++k) s += ws[((size_t)t * KCH + k) * NCH + n];
    wsum[e] = s;
  }
  __syncthreads();

  const T* src = static_cast<const T*>(FORM == 0 ? a.images : a.out_grad);
  T* dst = static_cast<T*>(FORM == 0 ? a.output : a.images_grad);
  const float pad = a.pad_zero ? 0.f : TileIo<T>::ld1(static_cast<const T*>(a.default_value));
  const int d1 = FORM == 0 ? a.oD : a.D, d2 = FORM == 0 ? a.oW : a.W, d3 = FORM == 0 ? a.oH : a.H;
  const long long ngroups = (nvox + VPT - 1) / VPT;

  for (long long grp = (long long)blockIdx.x * blockDim.x + threadIdx.x; grp < ngroups; grp += (long long)gridDim.x * blockDim.x) {
    const long long vbase = grp * VPT;
    int cb[VPT], cr[VPT], cc[VPT], cz[VPT];
    bool live[VPT];
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      long long v = vbase + u;
      live[u] = v < nvox;
      if (!live[u]) v = nvox - 1;
      cz[u] = (int)(v % d1); v /= d1;
      cc[u] = (int)(v % d2); v /= d2;
      cr[u] = (int)(v % d3);
      cb[u] = (int)(v / d3);
    }
    float acc[VPT][NCH];
#pragma unroll
    for (int u = 0; u < VPT; ++u)
#pragma unroll
      for (int n = 0; n < NCH; ++n) acc[u][n] = 0.f;

    int t = 0;
    for (int fr = 0; fr < a.fh; ++fr)
      for (int fc = 0; fc < a.fw; ++fc)
        for (int fz = 0; fz < a.fd; ++fz, ++t) {
          long long at[VPT];
          bool any = false, anypad = false;
#pragma unroll
          for (int u = 0; u < VPT; ++u) {
            at[u] = FORM == 0 ? sc_tap(a, cb[u], cr[u], cc[u], cz[u], fr, fc, fz) : sc_tap_t(a, cb[u], cr[u], cc[u], cz[u], fr, fc, fz);
            any |= at[u] >= 0;
            anypad |= at[u] < 0;
          }
          if (anypad) {
            const float* wsn = wsum + t * NCH;
#pragma unroll
            for (int n = 0; n < NCH; ++n) {
              const float p = pad * wsn[n];
#pragma unroll
              for (int u = 0; u < VPT; ++u)
                if (at[u] < 0) acc[u][n] += p;
            }
          }
          if (!any) continue;
          const float* wt = ws + (size_t)t * KCH * NCH;
#pragma unroll
          for (int k4 = 0; k4 < KCH / 4; ++k4) {
            float xs[VPT][4];
#pragma unroll
            for (int u = 0; u < VPT; ++u) {
              // a voxel whose tap is padding got its share above: it adds zero here
              float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
              if (at[u] >= 0) x = TileIo<T>::ld4(src + at[u] * KCH + k4 * 4);
              xs[u][0] = x.x; xs[u][1] = x.y; xs[u][2] = x.z; xs[u][3] = x.w;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const float4* wrow = reinterpret_cast<const float4*>(wt + (k4 * 4 + kk) * NCH);
#pragma unroll
              for (int n4 = 0; n4 < NCH / 4; ++n4) {
                const float4 w = wrow[n4];
#pragma unroll
                for (int u = 0; u < VPT; ++u) {
                  acc[u][n4 * 4 + 0] = fmaf(xs[u][kk], w.x, acc[u][n4 * 4 + 0]);
                  acc[u][n4 * 4 + 1] = fmaf(xs[u][kk], w.y, acc[u][n4 * 4 + 1]);
                  acc[u][n4 * 4 + 2] = fmaf(xs[u][kk], w.z, acc[u][n4 * 4 + 2]);
                  acc[u][n4 * 4 + 3] = fmaf(xs[u][kk], w.w, acc[u][n4 * 4 + 3]);
                }
              }
            }
          }
        }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (!live[u]) continue;
      T* o = dst + (vbase + u) * NCH;
#pragma unroll
      for (int n4 = 0; n4 < NCH / 4; ++n4)
        TileIo<T>::st4(o + n4 * 4, acc[u][n4 * 4], acc[u][n4 * 4 + 1], acc[u][n4 * 4 + 2], acc[u][n4 * 4 + 3]);
    }
  }
}

// Filter gradient, float32: dW[tap][k][n] = sum over voxels of gathered(voxel, tap)[k] * upstream(voxel)[n].
// A CTA owns a contiguous slice of the voxels and the whole [taps*KCH][NCH] result: thread q holds four consecutive
// gathered channels of one tap times NT upstream channels in registers (4*NT accumulators), so a voxel costs one
// 16-byte load of the gathered values, NT/4 warp-uniform 16-byte loads of the upstream row from shared memory and
// 4*NT FMAs.  Tap indices and upstream rows of WT voxels are staged per step.  Per-CTA slabs are summed in a fixed
// order by wgrad_tile_reduce (deterministic).  TR = transposed convolution: the voxels are those of the fine grid,
// the gathered tensor is the coarse input (Cout channels), the upstream one has Cin channels, and the reduction
// writes element [tap][co][ci] to filter_grad[taps-1-tap][ci][co].
constexpr int WT = 32;   // voxels per staging step

template <typename T, int KCH, int NCH, bool TR>
__global__ void __launch_bounds__(256) sc_wgrad_tile_kernel(const ScArgs a, const int vox_per_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int NT = NCH < 16 ? NCH : 16;                   // upstream channels per sweep
  const int taps = a.fh * a.fw * a.fd;
  const int K4 = taps * KCH / 4;                            // threads with work
  long long* tapidx = reinterpret_cast<long long*>(smem_raw);            // [WT][taps]
  float* gt = reinterpret_cast<float*>(tapidx + (size_t)WT * taps);       // [WT][NCH]
  float* wsum = gt + WT * NCH;                                            // [taps][NCH], dynamic_default only
  float* red = wsum + (size_t)taps * NCH;                                 // [blockDim]
  int4* vox = reinterpret_cast<int4*>(red + blockDim.x);                  // [WT]: b, row, column, depth of a staged voxel
  int3* tapf = reinterpret_cast<int3*>(vox + WT);                         // [taps]: fr, fc, fz
  for (int t = threadIdx.x; t < taps; t += blockDim.x) tapf[t] = make_int3(t / a.fd / a.fw, (t / a.fd) % a.fw, t % a.fd);
  const T* img = static_cast<const T*>(a.images);
  const T* og = static_cast<const T*>(a.out_grad);
  const bool dyn = !TR && a.dynamic_default;
  if (dyn) {
    const T* flt = static_cast<const T*>(a.filters);
    for (int e = threadIdx.x; e < taps * NCH; e += blockDim.x) {
      const int n = e % NCH, t = e / NCH;
      float s = 0.f;
      for (int k = 0; k < KCH; ++k) s += TileIo<T>::ld1(flt + ((size_t)t * KCH + k) * NCH + n);
      wsum[e] = s;
    }
  }
  const float defv = TileIo<T>::ld1(static_cast<const T*>(a.default_value));
  const float4 pad4 = make_float4(defv, defv, defv, defv);
  const long long nvox = TR ? a.nvox_in : a.nvox_out;
  const int d1 = TR ? a.D : a.oD, d2 = TR ? a.W : a.oW, d3 = TR ? a.H : a.oH;
  const long long v0 = (long long)blockIdx.x * vox_per_cta;
  const long long v1 = min(nvox, v0 + vox_per_cta);
  const int q = threadIdx.x;
  const bool active = q < K4;
  const int my_tap = active ? (q * 4) / KCH : 0;
  const int my_k = active ? (q * 4) % KCH : 0;
  const size_t slab = (size_t)taps * KCH * NCH + 1;
  float* part = static_cast<float*>(a.workspace) + (size_t)blockIdx.x * slab;
  float dacc = 0.f;

  for (int n0 = 0; n0 < NCH; n0 += NT) {
    float acc[4][NT];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int n = 0; n < NT; ++n) acc[i][n] = 0.f;
    for (long long vt = v0; vt < v1; vt += WT) {
      const int tm = (int)min((long long)WT, v1 - vt);
      __syncthreads();
      // voxel coordinates once per voxel (the 64-bit divisions are the expensive part), then the tap table
      if (threadIdx.x < tm) {
        long long v = vt + threadIdx.x;
        const int dz = (int)(v % d1); v /= d1;
        const int cc = (int)(v % d2); v /= d2;
        vox[threadIdx.x] = make_int4((int)(v / d3), (int)(v % d3), cc, dz);
      }
      for (int e = threadIdx.x; e < tm * NCH; e += blockDim.x) gt[e] = TileIo<T>::ld1(og + vt * NCH + e);
      __syncthreads();
      for (int e = threadIdx.x; e < tm * taps; e += blockDim.x) {
        const int m = e / taps, t = e - m * taps;
        const int4 c4 = vox[m];
        const int3 f = tapf[t];
        tapidx[e] = TR ? sc_tap_t(a, c4.x, c4.y, c4.z, c4.w, f.x, f.y, f.z) : sc_tap(a, c4.x, c4.y, c4.z, c4.w, f.x, f.y, f.z);
      }
      __syncthreads();
      if (active) {
        // four voxels per step: their gathered loads are issued together, then 4 x 4 x NT FMAs
        for (int m0 = 0; m0 < tm; m0 += 4) {
          long long at[4];
          float4 x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) at[u] = m0 + u < tm ? tapidx[(m0 + u) * taps + my_tap] : -2;   // -2: no voxel
#pragma unroll
          for (int u = 0; u < 4; ++u)
            x[u] = at[u] >= 0 ? TileIo<T>::ld4(img + at[u] * KCH + my_k)
                              : (at[u] == -1 ? pad4 : make_float4(0.f, 0.f, 0.f, 0.f));
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (m0 + u >= tm) break;
            const float4* g4 = reinterpret_cast<const float4*>(gt + (m0 + u) * NCH + n0);
            const float xs[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
            for (int n4 = 0; n4 < NT / 4; ++n4) {
              const float4 g = g4[n4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                acc[i][n4 * 4 + 0] = fmaf(xs[i], g.x, acc[i][n4 * 4 + 0]);
                acc[i][n4 * 4 + 1] = fmaf(xs[i], g.y, acc[i][n4 * 4 + 1]);
                acc[i][n4 * 4 + 2] = fmaf(xs[i], g.z, acc[i][n4 * 4 + 2]);
                acc[i][n4 * 4 + 3] = fmaf(xs[i], g.w, acc[i][n4 * 4 + 3]);
              }
            }
            if (dyn && at[u] == -1 && my_k == 0) {
              // d(default) collects (sum over input channels of the filter) . out_grad over the padded taps
              // (sparse_conv3d_fast_fixed_param_op_gpu.cu.cc:273-277); one thread per tap does it
              const float* ws = wsum + my_tap * NCH + n0;
              const float* gr = gt + (m0 + u) * NCH + n0;
#pragma unroll
              for (int n = 0; n < NT; ++n) dacc = fmaf(ws[n], gr[n], dacc);
            }
          }
        }
      }
    }
    if (active) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float* o = part + ((size_t)my_tap * KCH + my_k + i) * NCH + n0;
#pragma unroll
        for (int n = 0; n < NT; ++n) o[n] = acc[i][n];
      }
    }
  }
  __syncthreads();
  red[threadIdx.x] = dacc;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) part[slab - 1] = red[0];
}

// filter_grad = sum of the slabs in a fixed order, four loads in flight; the last slab element is d(default_value).
template <bool TR>
__global__ void __launch_bounds__(256) wgrad_tile_reduce(const float* part, int nparts, int taps, int KCH, int NCH,
                                                         float* filter_grad, float* default_grad) {
  const long long n_el = (long long)taps * KCH * NCH;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e > n_el || (TR && e == n_el)) return;
  const float* col = part + e;
  const size_t stride = (size_t)n_el + 1;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int p = 0;
  for (; p + 3 < nparts; p += 4) {
    const float a0 = col[(size_t)p * stride], a1 = col[(size_t)(p + 1) * stride], a2 = col[(size_t)(p + 2) * stride],
                a3 = col[(size_t)(p + 3) * stride];
    s0 += a0; s1 += a1; s2 += a2; s3 += a3;
  }
  for (; p < nparts; ++p) s0 += col[(size_t)p * stride];
  const float s = (s0 + s1) + (s2 + s3);
  if (e == n_el) { *default_grad = s; return; }
  if (!TR) { filter_grad[e] = s; return; }
  const int n = (int)(e % NCH), k = (int)((e / NCH) % KCH), t = (int)(e / ((long long)NCH * KCH));
  filter_grad[((long long)(taps - 1 - t) * NCH + n) * KCH + k] = s;
}

template <typename T, int KCH, int NCH, bool TR>
int launch_wgrad(const ScArgs& a, int nparts, cudaStream_t st) {
  const int taps = a.fh * a.fw * a.fd;
  const int K4 = taps * KCH / 4;
  int threads = 64;   // a power of two (the block sum of the default-value gradient halves the block repeatedly)
  while (threads < K4) threads <<= 1;
  if (threads > 256) return -4;
  const long long nvox = TR ? a.nvox_in : a.nvox_out;
  if (nparts > (nvox + WT - 1) / WT) nparts = (int)((nvox + WT - 1) / WT);
  const int vox_per_cta = (int)((nvox + nparts - 1) / nparts);
  nparts = (int)((nvox + vox_per_cta - 1) / vox_per_cta);   // every launched CTA owns at least one voxel and writes its slab
  const size_t smem = (size_t)WT * taps * sizeof(long long) + ((size_t)WT * NCH + (size_t)taps * NCH + threads) * sizeof(float) +
                      WT * sizeof(int4) + (size_t)taps * sizeof(int3);
  auto k = sc_wgrad_tile_kernel<T, KCH, NCH, TR>;
  if (int e = grant_smem(k, smem)) return e;
  k<<<nparts, threads, smem, st>>>(a, vox_per_cta);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const long long n_el = (long long)taps * KCH * NCH;
  wgrad_tile_reduce<TR><<<(unsigned)((n_el + 1 + 255) / 256), 256, 0, st>>>(static_cast<const float*>(a.workspace), nparts, taps,
                                                                             KCH, NCH, static_cast<float*>(a.filter_grad),
                                                                             static_cast<float*>(a.default_grad));
  return (int)cudaGetLastError();
}

template <typename T, bool TR>
int dispatch_wgrad(const ScArgs& a, int nparts, cudaStream_t st) {
  const int kch = TR ? a.Cout : a.Cin, nch = TR ? a.Cin : a.Cout;
#define CHOP_TILE_CASE(K, N) \
  if (kch == K && nch == N) return launch_wgrad<T, K, N, TR>(a, nparts, st);
  CHOP_TILE_CASE(8, 8) CHOP_TILE_CASE(8, 16) CHOP_TILE_CASE(16, 8) CHOP_TILE_CASE(16, 16) CHOP_TILE_CASE(16, 32)
  CHOP_TILE_CASE(32, 16) CHOP_TILE_CASE(32, 32)
#undef CHOP_TILE_CASE
  return -4;
}

template <typename T, int KCH, int NCH, int FORM>
int launch(const ScArgs& a, cudaStream_t st) {
  const int taps = a.fh * a.fw * a.fd;
  const size_t smem = ((size_t)taps * KCH * NCH + (size_t)taps * NCH) * sizeof(float);
  auto k = sc_tile_kernel<T, KCH, NCH, FORM>;
  if (int e = grant_smem(k, smem)) return e;
  const long long nvox = FORM == 0 ? a.nvox_out : a.nvox_in;
  const long long ngroups = (nvox + TileVpt<NCH>::v - 1) / TileVpt<NCH>::v;
  long long blocks = (ngroups + 127) / 128;
  const long long cap = 148LL * 16;   // weights are staged per CTA: a bounded, persistent grid
  if (blocks > cap) blocks = cap;
  k<<<(unsigned)blocks, 128, smem, st>>>(a, nvox);
  return (int)cudaGetLastError();
}

template <typename T, int FORM>
int dispatch(const ScArgs& a, cudaStream_t st) {
  const int kch = FORM == 0 ? a.Cin : a.Cout, nch = FORM == 0 ? a.Cout : a.Cin;
#define CHOP_TILE_CASE(K, N) \
  if (kch == K && nch == N) return launch<T, K, N, FORM>(a, st);
  CHOP_TILE_CASE(8, 8) CHOP_TILE_CASE(8, 16) CHOP_TILE_CASE(16, 8) CHOP_TILE_CASE(16, 16) CHOP_TILE_CASE(16, 32)
  CHOP_TILE_CASE(32, 16) CHOP_TILE_CASE(32, 32)
#undef CHOP_TILE_CASE
  return -4;
}

}  // namespace

// float32 or bfloat16 data, both channel counts in {8,16,32} (one of the instantiated pairs), weights + sums within
// 160 KB of shared memory, 16-byte aligned tensors (checked by the caller)
bool sc_tile_supported(int dtype, const ScArgs& a) {
  if (dtype != 0 && dtype != 2) return false;
  const int taps = a.fh * a.fw * a.fd;
  if (((size_t)taps * a.Cin * a.Cout + (size_t)taps * (a.Cin > a.Cout ? a.Cin : a.Cout)) * 4 > 160 * 1024) return false;
  const int c[2] = {a.Cin, a.Cout};
  for (int v : c)
    if (v != 8 && v != 16 && v != 32) return false;
  return !(a.Cin == 8 && a.Cout == 32) && !(a.Cin == 32 && a.Cout == 8);
}

// the filter gradient additionally needs taps * (gathered channels) / 4 <= 256 threads
bool sc_tile_wgrad_supported(int dtype, const ScArgs& a, bool transposed) {
  if (!sc_tile_supported(dtype, a)) return false;
  return (long long)a.fh * a.fw * a.fd * (transposed ? a.Cout : a.Cin) / 4 <= 256;
}
int sc_tile_wgrad_launch(int dtype, const ScArgs& a, int nparts, cudaStream_t st) {
  return dtype == 0 ? dispatch_wgrad<float, false>(a, nparts, st) : dispatch_wgrad<__nv_bfloat16, false>(a, nparts, st);
}
int sc_tile_twgrad_launch(int dtype, const ScArgs& a, int nparts, cudaStream_t st) {
  return dtype == 0 ? dispatch_wgrad<float, true>(a, nparts, st) : dispatch_wgrad<__nv_bfloat16, true>(a, nparts, st);
}

int sc_tile_fwd_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  return dtype == 0 ? dispatch<float, 0>(a, st) : dispatch<__nv_bfloat16, 0>(a, st);
}
// gather form: a.out_grad = the coarse tensor (Cout channels), a.images_grad = the fine result (Cin channels);
// a.pad_zero selects the image gradient (1) or the transposed forward (0)
int sc_tile_gather_launch(int dtype, const ScArgs& a, cudaStream_t st) {
  return dtype == 0 ? dispatch<float, 1>(a, st) : dispatch<__nv_bfloat16, 1>(a, st);
}

}  // namespace chop
