// Homography projection shared by the forward and backward cost-volume kernels.
//
// Work decomposition (both directions): a warp owns 32/LG neighbouring reference pixels, LG lanes
// per pixel, each lane holding CPL consecutive channels.  It walks a chunk of depth planes in blocks
// of LG planes.  For every block it runs two phases:
//   A. lane (pixel g, plane j) projects its own voxel into every source view - one projection per
//      lane instead of one per channel lane - and leaves {texel index, dh, dw, ...} in shared memory;
//   B. for each plane of the block all LG lanes of the pixel read that record (one broadcast shared
//      load) and do the channel work with 16-byte loads of the four bilinear corners.
// Per-(pixel, view) row products R*(x,y,1) are hoisted once per work item (Coef).
#pragma once
#include "chop_common.cuh"

namespace chop {

// R rows applied to the pixel, translation, and the first texel row of view n of batch b.
template <typename R>
struct alignas(16) Coef {
  R zc, wc, hc, t0, t1, t2;
  int row0;
  int pad;
};

// Phase-A record, forward.
template <typename R>
struct alignas(16) ProjF {
  int texel;  // index of the top-left texel in [B*N*Hs*Ws), or -1 when the view does not see the voxel
  R dh, dw;
  R aux;      // in the record of view 0: 1/(number of views that see the voxel), 0 if none
};

// Phase-A record, backward: also the factors of d(sample row)/d(depth) and d(sample col)/d(depth).
template <typename R>
struct alignas(16) ProjB {
  int texel;  // -1 also when the whole voxel is skipped (no view counted in the forward pass)
  R dh, dw;
  R gh, gw;
  R aux;      // in the record of the pass's first view: constant factor of d(cost)/d(sample)
  R pad1, pad2;
};

// Row products for (pixel, view) pairs of one warp: entry [n*G + gg] for pixel pix0+gg.
// Reference arithmetic: custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:65-70,83,88,91.
template <typename R>
__device__ __forceinline__ void stage_coefs(const CvArgs& a, Coef<R>* coef, int lane, int G, long long pix0) {
  const R* Rs = static_cast<const R*>(a.Rs);
  const R* Ts = static_cast<const R*>(a.Ts);
  for (int idx = lane; idx < a.N * G; idx += 32) {
    const int n = idx / G;
    const int gg = idx - n * G;
    long long pix = pix0 + gg;
    if (pix >= a.npix) pix = a.npix - 1;
    const int w = (int)(pix % a.W);
    const long long t = pix / a.W;
    const int h = (int)(t % a.H);
    const int b = (int)(t / a.H);
    R x = (R)w, y = (R)h;
    if (a.half_centor) {
      x = xadd(x, (R)0.5);
      y = xadd(y, (R)0.5);
    }
    const R* Rm = Rs + (size_t)(b * a.N + n) * 9;
    const R* tv = Ts + (size_t)(b * a.N + n) * 3;
    Coef<R> c;
    c.zc = xadd(xadd(xmul(Rm[6], x), xmul(Rm[7], y)), Rm[8]);
    c.wc = xadd(xadd(xmul(Rm[0], x), xmul(Rm[1], y)), Rm[2]);
    c.hc = xadd(xadd(xmul(Rm[3], x), xmul(Rm[4], y)), Rm[5]);
    c.t0 = tv[0];
    c.t1 = tv[1];
    c.t2 = tv[2];
    c.row0 = a.Hs * (n + a.N * b);
    c.pad = 0;
    coef[idx] = c;
  }
}

// One voxel into one view (cost_volume_kernels_gpu.cu.cc:84-104).  Returns the texel index or -1.
template <typename R, bool BWD>
__device__ __forceinline__ int project(const Coef<R>& c, R depth, int half_centor, int Hs, int Ws, R& dh,
                                       R& dw, R& gh, R& gw) {
  const R z = xadd(xmul(c.zc, depth), c.t2);
  if (!(z > (R)0)) return -1;
  const R w3 = xadd(xmul(c.wc, depth), c.t0);
  R sw = xdiv(w3, z);
  const R h3 = xadd(xmul(c.hc, depth), c.t1);
  R sh = xdiv(h3, z);
  if (half_centor) {
    sw = xsub(sw, (R)0.5);
    sh = xsub(sh, (R)0.5);
  }
  if (sh > (R)0 && sw > (R)0 && sh < (R)(Hs - 1) && sw < (R)(Ws - 1)) {
    const int fh = (int)sh;
    const int fw = (int)sw;
    dh = xsub(sh, (R)fh);
    dw = xsub(sw, (R)fw);
    if (BWD) {
      // :451  ((hc*z - zc*h3d)*h_grad + (wc*z - zc*w3d)*w_grad)/(z*z), factored per term
      // one reciprocal serves both factors (gradient tolerance, not the bit-exact part of the projection)
      const R izz = (R)1 / (z * z);
      gh = (c.hc * z - c.zc * h3) * izz;
      gw = (c.wc * z - c.zc * w3) * izz;
    }
    return fw + Ws * (fh + c.row0);
  }
  return -1;
}

// Bilinear weights, reference naming in brackets (:105-108): w00 [coef_cc] for texel (fh,fw), w01
// [coef_cf] for (fh,fw+1), w11 [coef_ff] for (fh+1,fw+1), w10 [coef_fc] for (fh+1,fw).
// The same weights with 4 operations instead of 6 (differs from the reference in the last bit; used
// where the result only has to meet a floating tolerance).
template <typename R>
__device__ __forceinline__ void bilinear_weights_fast(R dh, R dw, R& w00, R& w01, R& w11, R& w10) {
  w11 = dh * dw;
  w10 = dh - w11;
  w01 = dw - w11;
  w00 = ((R)1 - dh) - w01;
}

template <typename R>
__device__ __forceinline__ void bilinear_weights(R dh, R dw, R& w00, R& w01, R& w11, R& w10) {
  const R omh = xsub((R)1, dh);
  const R omw = xsub((R)1, dw);
  w11 = xmul(dh, dw);
  w10 = xmul(dh, omw);
  w00 = xmul(omh, omw);
  w01 = xmul(omh, dw);
}

}  // namespace chop
