// Register-tiled CUDA-core manifold convolution for float32 data (the reference's own dtype): forward, gather-form
// image gradient and transposed forward, any filter size / stride / dilation, 8, 16 or 32 channels on either side.
//
// One thread owns two depth-adjacent voxels of a pixel and all output channels: per tap it loads the two gathered
// channel vectors once (16-byte loads) and multiplies them with the tap's [gathered x produced] weight block, which
// the CTA keeps in shared memory and reads with warp-uniform 16-byte loads (every weight load feeds 8 FMAs).
// Padded taps add default_value times a per-(tap, produced channel) weight sum that is formed once per CTA.
// The shape-agnostic one-thread-per-output-element kernels of sc_simt.cu remain the fallback (other channel counts,
// float64, filters whose weights do not fit in shared memory).
#include "sc_common.cuh"
#include "sc_entry.h"

namespace chop {
namespace {

// FORM 0: forward - voxels of the output grid gather the input grid (sc_tap); weights w[t][ci][co].
// FORM 1: gather form - voxels of the fine grid gather the coarse grid (sc_tap_t); the gathered tensor has Cout
//         channels, the produced one Cin, weights flipped: w'[t][co][ci] = filter[taps-1-t][ci][co].
template <int KCH, int NCH, int FORM>
__global__ void __launch_bounds__(128) sc_tile_kernel(const ScArgs a, const long long npairs) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int taps = a.fh * a.fw * a.fd;
  float* ws = reinterpret_cast<float*>(smem_raw);          // [taps][KCH][NCH]
  float* wsum = ws + (size_t)taps * KCH * NCH;              // [taps][NCH]
  const float* flt = static_cast<const float*>(a.filters);
  for (int e = threadIdx.x; e < taps * KCH * NCH; e += blockDim.x) {
    const int n = e % NCH, k = (e / NCH) % KCH, t = e / (NCH * KCH);
    ws[e] = FORM == 0 ? __ldg(flt + e) : __ldg(flt + ((size_t)(taps - 1 - t) * NCH + n) * KCH + k);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < taps * NCH; e += blockDim.x) {
    const int n = e % NCH, t = e / NCH;
    float s = 0.f;
    for (int k = 0; k < KCH; ++k) s += ws[((size_t)t * KCH + k) * NCH + n];
    wsum[e] = s;
  }
  __syncthreads();

  const float* src = static_cast<const float*>(FORM == 0 ? a.images : a.out_grad);
  float* dst = static_cast<float*>(FORM == 0 ? a.output : a.images_grad);
  const float pad = a.pad_zero ? 0.f : __ldg(static_cast<const float*>(a.default_value));
  const int d1 = FORM == 0 ? a.oD : a.D, d2 = FORM == 0 ? a.oW : a.W, d3 = FORM == 0 ? a.oH : a.H;
  const int dp = (d1 + 1) >> 1;   // voxel pairs per pixel

  for (long long pr = (long long)blockIdx.x * blockDim.x + threadIdx.x; pr < npairs; pr += (long long)gridDim.x * blockDim.x) {
    long long v = pr;
    const int z0 = (int)(v % dp) * 2; v /= dp;
    const int cc = (int)(v % d2); v /= d2;
    const int rr = (int)(v % d3);
    const int b = (int)(v / d3);
    const bool two = z0 + 1 < d1;
    float acc0[NCH], acc1[NCH];
#pragma unroll
    for (int n = 0; n < NCH; ++n) acc0[n] = acc1[n] = 0.f;

    int t = 0;
    for (int fr = 0; fr < a.fh; ++fr)
      for (int fc = 0; fc < a.fw; ++fc)
        for (int fz = 0; fz < a.fd; ++fz, ++t) {
          long long at0, at1 = -1;
          if (FORM == 0) {
            at0 = sc_tap(a, b, rr, cc, z0, fr, fc, fz);
            if (two) at1 = sc_tap(a, b, rr, cc, z0 + 1, fr, fc, fz);
          } else {
            at0 = sc_tap_t(a, b, rr, cc, z0, fr, fc, fz);
            if (two) at1 = sc_tap_t(a, b, rr, cc, z0 + 1, fr, fc, fz);
          }
          const float* wt = ws + (size_t)t * KCH * NCH;
          if (at0 < 0 || at1 < 0) {
            const float* wsn = wsum + t * NCH;
#pragma unroll
            for (int n = 0; n < NCH; ++n) {
              const float p = pad * wsn[n];
              if (at0 < 0) acc0[n] += p;
              if (at1 < 0 && two) acc1[n] += p;
            }
          }
          if (at0 < 0 && at1 < 0) continue;
          const float4* x0 = reinterpret_cast<const float4*>(src + (at0 >= 0 ? at0 : at1) * KCH);
          const float4* x1 = reinterpret_cast<const float4*>(src + (at1 >= 0 ? at1 : at0) * KCH);
          const bool v0 = at0 >= 0, v1 = at1 >= 0;   // a voxel whose tap is padding got its share above: it adds zero here
#pragma unroll
          for (int k4 = 0; k4 < KCH / 4; ++k4) {
            float4 a0 = __ldg(x0 + k4), a1 = __ldg(x1 + k4);
            const float xa[4] = {v0 ? a0.x : 0.f, v0 ? a0.y : 0.f, v0 ? a0.z : 0.f, v0 ? a0.w : 0.f};
            const float xb[4] = {v1 ? a1.x : 0.f, v1 ? a1.y : 0.f, v1 ? a1.z : 0.f, v1 ? a1.w : 0.f};
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const float4* wrow = reinterpret_cast<const float4*>(wt + (k4 * 4 + kk) * NCH);
#pragma unroll
              for (int n4 = 0; n4 < NCH / 4; ++n4) {
                const float4 w = wrow[n4];
                acc0[n4 * 4 + 0] = fmaf(xa[kk], w.x, acc0[n4 * 4 + 0]);
                acc0[n4 * 4 + 1] = fmaf(xa[kk], w.y, acc0[n4 * 4 + 1]);
                acc0[n4 * 4 + 2] = fmaf(xa[kk], w.z, acc0[n4 * 4 + 2]);
                acc0[n4 * 4 + 3] = fmaf(xa[kk], w.w, acc0[n4 * 4 + 3]);
                acc1[n4 * 4 + 0] = fmaf(xb[kk], w.x, acc1[n4 * 4 + 0]);
                acc1[n4 * 4 + 1] = fmaf(xb[kk], w.y, acc1[n4 * 4 + 1]);
                acc1[n4 * 4 + 2] = fmaf(xb[kk], w.z, acc1[n4 * 4 + 2]);
                acc1[n4 * 4 + 3] = fmaf(xb[kk], w.w, acc1[n4 * 4 + 3]);
              }
            }
          }
        }
    const long long vox0 = (((long long)b * d3 + rr) * d2 + cc) * d1 + z0;
    float4* o0 = reinterpret_cast<float4*>(dst + vox0 * NCH);
#pragma unroll
    for (int n4 = 0; n4 < NCH / 4; ++n4) o0[n4] = make_float4(acc0[n4 * 4], acc0[n4 * 4 + 1], acc0[n4 * 4 + 2], acc0[n4 * 4 + 3]);
    if (two) {
      float4* o1 = o0 + NCH / 4;
#pragma unroll
      for (int n4 = 0; n4 < NCH / 4; ++n4) o1[n4] = make_float4(acc1[n4 * 4], acc1[n4 * 4 + 1], acc1[n4 * 4 + 2], acc1[n4 * 4 + 3]);
    }
  }
}

template <int KCH, int NCH, int FORM>
int launch(const ScArgs& a, cudaStream_t st) {
  const int taps = a.fh * a.fw * a.fd;
  const size_t smem = ((size_t)taps * KCH * NCH + (size_t)taps * NCH) * sizeof(float);
  auto k = sc_tile_kernel<KCH, NCH, FORM>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int d1 = FORM == 0 ? a.oD : a.D;
  const long long nvox = FORM == 0 ? a.nvox_out : a.nvox_in;
  const long long npairs = nvox / d1 * ((d1 + 1) / 2);
  long long blocks = (npairs + 127) / 128;
  const long long cap = 148LL * 16;   // weights are staged per CTA: a bounded, persistent grid
  if (blocks > cap) blocks = cap;
  k<<<(unsigned)blocks, 128, smem, st>>>(a, npairs);
  return (int)cudaGetLastError();
}

template <int FORM>
int dispatch(const ScArgs& a, cudaStream_t st) {
  const int kch = FORM == 0 ? a.Cin : a.Cout, nch = FORM == 0 ? a.Cout : a.Cin;
#define CHOP_TILE_CASE(K, N) \
  if (kch == K && nch == N) return launch<K, N, FORM>(a, st);
  CHOP_TILE_CASE(8, 8) CHOP_TILE_CASE(8, 16) CHOP_TILE_CASE(16, 8) CHOP_TILE_CASE(16, 16) CHOP_TILE_CASE(16, 32)
  CHOP_TILE_CASE(32, 16) CHOP_TILE_CASE(32, 32)
#undef CHOP_TILE_CASE
  return -4;
}

}  // namespace

// float32 data, both channel counts in {8,16,32} (one of the instantiated pairs), weights + sums within 160 KB of
// shared memory, 16-byte aligned tensors (checked by the caller)
bool sc_tile_supported(int dtype, const ScArgs& a) {
  if (dtype != 0) return false;
  const int taps = a.fh * a.fw * a.fd;
  if (((size_t)taps * a.Cin * a.Cout + (size_t)taps * (a.Cin > a.Cout ? a.Cin : a.Cout)) * 4 > 160 * 1024) return false;
  const int c[2] = {a.Cin, a.Cout};
  for (int v : c)
    if (v != 8 && v != 16 && v != 32) return false;
  return !(a.Cin == 8 && a.Cout == 32) && !(a.Cin == 32 && a.Cout == 8);
}

int sc_tile_fwd_launch(const ScArgs& a, cudaStream_t st) { return dispatch<0>(a, st); }
// gather form: a.out_grad = the coarse tensor (Cout channels), a.images_grad = the fine result (Cin channels);
// a.pad_zero selects the image gradient (1) or the transposed forward (0)
int sc_tile_gather_launch(const ScArgs& a, cudaStream_t st) { return dispatch<1>(a, st); }

}  // namespace chop
