// Manifold ("sparse") 3-D convolution: shared argument block and index helpers.
//
// images [B,H,W,D,Cin] holds, for every pixel, a band of D depth planes starting at absolute plane
// base_plane[b,h,w]; the convolution runs in absolute depth, so a filter tap that lands in a neighbour
// pixel has to be shifted by the difference of the two base planes.  Taps outside the image plane or
// outside the neighbour's band read default_value (reference:
// custom_helper_op/cc/kernels/sparse_conv3d_fast_fixed_param_op_gpu.cu.cc:78-113).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace chop {

struct ScArgs {
  const void* images;
  const void* filters;        // [fh,fw,fd,Cin,Cout]
  const void* default_value;  // device scalar
  const int* base_plane;      // [B,H,W]
  const void* out_grad;       // [B,oH,oW,oD,Cout]
  void* output;               // [B,oH,oW,oD,Cout]
  void* images_grad;          // [B,H,W,D,Cin]
  void* filter_grad;          // [fh,fw,fd,Cin,Cout]
  void* default_grad;         // scalar
  void* workspace;
  int B, H, W, D, Cin, Cout;
  int fh, fw, fd, sr, sc, sd, dr, dc, dd;
  int oH, oW, oD, pr, pc, pd;
  int dynamic_default;
  int pad_zero;               // gathered taps that are padding read 0 instead of *default_value
  int ls_r, ls_c, ls_d;       // log2 of the strides when all three are powers of two, else -1
  long long nvox_in, nvox_out;
};

__device__ __forceinline__ bool oob(int a, int b) { return (unsigned)a >= (unsigned)b; }

template <typename T> struct ScIo;
template <> struct ScIo<float> {
  static __device__ __forceinline__ float ld(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct ScIo<double> {
  static __device__ __forceinline__ double ld(const double* p) { return __ldg(p); }
  static __device__ __forceinline__ void st(double* p, double v) { *p = v; }
};
template <> struct ScIo<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) {
    return __uint_as_float(((unsigned)__ldg(reinterpret_cast<const unsigned short*>(p))) << 16);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// Element offset (in units of Cin) of the input voxel that tap (fr,fc,fz) of output voxel (b,ro,co,dz)
// reads, or -1 when the tap is padding.
__device__ __forceinline__ long long sc_tap(const ScArgs& a, int b, int ro, int co, int dz, int fr, int fc, int fz) {
  const int row = ro * a.sr, col = co * a.sc;
  const int depth = (dz + (__ldg(a.base_plane + (b * a.H + row) * a.W + col) + a.sd - 1) / a.sd) * a.sd;
  const int orow = row - a.pr + fr * a.dr, ocol = col - a.pc + fc * a.dc;
  if (oob(orow, a.H) || oob(ocol, a.W)) return -1;
  const int pix = (b * a.H + orow) * a.W + ocol;
  const int ind = depth - a.pd + fz * a.dd - __ldg(a.base_plane + pix);
  if (oob(ind, a.D)) return -1;
  return (long long)pix * a.D + ind;
}

// Gather form used by the image gradient and by the transposed convolution: index (in voxels of the
// COARSE grid [B,oH,oW,oD]) of the voxel that lies exactly under tap (fr,fc,fz) of FINE voxel (b,r,c,dz),
// or -1 when the tap is padding - outside the image plane, not aligned with the strides, or outside the
// coarse band (custom_helper_op/cc/kernels/sparse_conv3d_fast_op_gpu.cu.cc:201,233-247, with the right
// padding of sparse_conv3d_fast_op.cc:314-316 / :395-397).
__device__ __forceinline__ long long sc_tap_t(const ScArgs& a, int b, int r, int c, int dz, int fr, int fc, int fz) {
  const int qr = (a.fh - 1) * a.dr - a.pr, qc = (a.fw - 1) * a.dc - a.pc, qd = (a.fd - 1) * a.dd - a.pd;
  const int orow = r - qr + fr * a.dr, ocol = c - qc + fc * a.dc;
  if (oob(orow, a.H) || oob(ocol, a.W)) return -1;
  int od = dz + __ldg(a.base_plane + (b * a.H + r) * a.W + c) - qd + fz * a.dd;
  if ((orow % a.sr) != 0 || (ocol % a.sc) != 0 || (od % a.sd) != 0) return -1;
  od = od / a.sd - (__ldg(a.base_plane + (b * a.H + orow) * a.W + ocol) + a.sd - 1) / a.sd;
  if (oob(od, a.oD)) return -1;
  return (((long long)b * a.oH + orow / a.sr) * a.oW + ocol / a.sc) * a.oD + od;
}

}  // namespace chop
