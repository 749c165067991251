// Gradient of the plane-sweep cost volume with respect to the reference features, the source
// features and the depth input (custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:342-577,
// cost_volume_kernels_gpu_v2.cu.cc:349-601, cost_aggregate_kernels_gpu.cu.cc:339-568).
//
// Same warp decomposition as the forward kernel (LG lanes per pixel, CPL channels per lane, phase A
// projection / phase B channel work).  What the reference does with 5*C*N+1 scalar atomics per voxel
// is restructured so that almost nothing reaches memory:
//   * a pixel stays on the same lanes for the whole depth chunk, so d(ref) and d(base_plane) are
//     plain register sums, written once per work item;
//   * as the depth advances a view's sample slides along its epipolar line and usually stays inside
//     the same 2x2 texel footprint for several planes; the four corner gradients are accumulated in
//     registers and flushed with 16-byte vector reductions only when the footprint changes;
//   * NV source views are tracked at a time (NV*4*CPL accumulator registers); more views are handled
//     in further passes over the depth chunk.
// The forward sample is recomputed (the op saves nothing but the validity mask, as in the reference).
#pragma once
#include "cv_project.cuh"

namespace chop {

struct BwdCfg {
  int sub;    // channels per group (KIND 2)
  int warps;  // warps per block
  size_t smem_per_warp;
};

template <typename R>
__host__ __device__ inline size_t bwd_smem_per_warp(int N, int G, int NV) {
  size_t s = (size_t)N * G * sizeof(Coef<R>) + (size_t)NV * 32 * sizeof(ProjB<R>);
  return (s + 15) & ~(size_t)15;
}

template <typename T, typename R, int CPL, int KIND, bool RMIN, int NV>
__global__ void __launch_bounds__(256) cv_bwd_kernel(const CvArgs a, const BwdCfg cfg) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int lgl = a.lg_log2;
  const int LG = 1 << lgl;
  const int G = 32 >> lgl;
  const int li = lane & (LG - 1);
  const int g = lane >> lgl;

  const long long item = (long long)blockIdx.x * cfg.warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const long long pix = pix0 + g;
  const bool pvalid = pix < a.npix;
  const int dlo = a.d_begin + chunk_id * a.chunk;
  const int dhi = min(a.d_end, dlo + a.chunk);

  unsigned char* mine = smem_raw + (size_t)wib * cfg.smem_per_warp;
  Coef<R>* coef = reinterpret_cast<Coef<R>*>(mine);
  ProjB<R>* proj = reinterpret_cast<ProjB<R>*>(coef + a.N * G);

  stage_coefs<R>(a, coef, lane, G, pix0);
  __syncwarp();

  const int C = a.C;
  const int Ws = a.Ws;
  const bool lane_on = pvalid && (li * CPL < C);
  const T* src = static_cast<const T*>(a.src);
  R* src_grad = static_cast<R*>(a.src_grad);
  const R* cgp = static_cast<const R*>(a.cost_grad);
  const int CO = KIND == 1 ? C : (KIND == 2 ? a.G : 1);
  const int MC = RMIN ? CO : 1;

  R refv[CPL], rg[CPL];
#pragma unroll
  for (int k = 0; k < CPL; ++k) { refv[k] = (R)0; rg[k] = (R)0; }
  if (lane_on) Vec<T, R, CPL>::load(static_cast<const T*>(a.ref) + pix * C + li * CPL, refv);
  const int b = pvalid ? (int)(pix / ((long long)a.H * a.W)) : 0;
  R base = (R)0;
  if (KIND != 2 && pvalid) base = static_cast<const R*>(a.depth)[pix];
  R dsum = (R)0;  // KIND 1/3: this lane's share of d(base_plane) for the pixel

  for (int n0 = 0; n0 < a.N; n0 += NV) {
    R acc[NV][4][CPL];
    int cur[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      cur[v] = -1;
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int k = 0; k < CPL; ++k) acc[v][q][k] = (R)0;
    }

    for (int dblk = dlo; dblk < dhi; dblk += LG) {
      // ---- phase A --------------------------------------------------------------------------------
      const int dA = dblk + li;
      const bool dv = pvalid && dA < dhi;
      {
        R depth = (R)0;
        R scale = (R)0;
        bool live = false;  // the voxel contributes at all
        if (dv) {
          if (KIND == 2) depth = static_cast<const R*>(a.depth)[pix * a.D + dA];
          else depth = xadd(base, static_cast<const R*>(a.offsets)[(long long)b * a.D + dA]);
          const int m0 = __ldg(a.mask + (pix * a.D + dA) * MC);
          // :367 (MEAN: no view saw the voxel) and :484 (MIN: first channel has no winner)
          live = RMIN ? (m0 >= 0) : (m0 > 0);
          // constant factors of d(cost)/d(sample), folded into the upstream gradient in phase B
          if (live) {
            if (KIND == 1) scale = RMIN ? (R)2 : (R)2 / (R)m0;          // :439, :560
            else if (KIND == 2) scale = RMIN ? (R)1 : (R)1 / (R)m0;     // v2:461, v2:583
            else scale = RMIN ? (R)2 / (R)C : (R)2 / (R)(m0 * C);       // aggregate :385, :500
          }
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          ProjB<R> pr;
          pr.texel = -1;
          pr.dh = pr.dw = pr.gh = pr.gw = pr.pad1 = pr.pad2 = (R)0;
          pr.aux = scale;
          const int n = n0 + v;
          if (live && n < a.N)
            pr.texel = project<R, true>(coef[n * G + g], depth, a.half_centor, a.Hs, Ws, pr.dh, pr.dw, pr.gh, pr.gw);
          proj[v * 32 + lane] = pr;
        }
      }
      __syncwarp();

      // ---- phase B --------------------------------------------------------------------------------
      R dkeep = (R)0;  // KIND 2: gradient of depth plane dblk+li of this pixel
      const int jn = min(LG, dhi - dblk);
      for (int j = 0; j < jn; ++j) {
        const long long vox = pix * a.D + dblk + j;
        const ProjB<R>* rec = proj + (g << lgl) + j;
        bool any = false;
#pragma unroll
        for (int v = 0; v < NV; ++v) any |= rec[v * 32].texel >= 0;
        R dvox = (R)0;
        if (any && lane_on) {
          R cgv[CPL];
          int mk[CPL];
          if (KIND == 1) {
            load_stream<R, CPL>(cgp + vox * C + li * CPL, cgv);
#pragma unroll
            for (int k = 0; k < CPL; ++k) mk[k] = RMIN ? __ldg(a.mask + vox * C + li * CPL + k) : 0;
          } else if (KIND == 2) {
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              const int gi = (li * CPL + k) / cfg.sub;
              cgv[k] = __ldg(cgp + vox * CO + gi);
              mk[k] = RMIN ? __ldg(a.mask + vox * CO + gi) : 0;
            }
          } else {
            const R c0 = __ldg(cgp + vox);
            const int m0 = RMIN ? __ldg(a.mask + vox) : 0;
#pragma unroll
            for (int k = 0; k < CPL; ++k) { cgv[k] = c0; mk[k] = m0; }
          }
          const R scale = rec->aux;
#pragma unroll
          for (int k = 0; k < CPL; ++k) cgv[k] *= scale;

#pragma unroll
          for (int v = 0; v < NV; ++v) {
            const int n = n0 + v;
            const ProjB<R> pr = rec[v * 32];
            if (pr.texel < 0) continue;
            if (pr.texel != cur[v]) {
              // footprint changed: flush the four corner sums of the old one
              if (cur[v] >= 0) {
                R* gp = src_grad + (size_t)cur[v] * C + li * CPL;
                red_add<R, CPL>(gp, acc[v][0]);
                red_add<R, CPL>(gp + C, acc[v][1]);
                red_add<R, CPL>(gp + (size_t)Ws * C + C, acc[v][2]);
                red_add<R, CPL>(gp + (size_t)Ws * C, acc[v][3]);
              }
              cur[v] = pr.texel;
#pragma unroll
              for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int k = 0; k < CPL; ++k) acc[v][q][k] = (R)0;
            }
            R w00, w01, w11, w10;
            bilinear_weights_fast(pr.dh, pr.dw, w00, w01, w11, w10);
            const T* p00 = src + (size_t)pr.texel * C + li * CPL;
            R t00[CPL], t01[CPL], t10[CPL], t11[CPL];
            Vec<T, R, CPL>::load(p00, t00);
            Vec<T, R, CPL>::load(p00 + C, t01);
            Vec<T, R, CPL>::load(p00 + (size_t)Ws * C, t10);
            Vec<T, R, CPL>::load(p00 + (size_t)Ws * C + C, t11);
            R hg = (R)0, wg = (R)0;
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              if (RMIN && mk[k] != n) continue;  // :553 only the winning view of this channel/group
              const R s = xfma(w10, t10[k], xfma(w11, t11[k], xfma(w01, t01[k], w00 * t00[k])));
              R gs;  // d(loss)/d(sample)
              if (KIND == 2) {
                rg[k] = xfma(cgv[k], s, rg[k]);  // v2:462
                gs = cgv[k] * refv[k];
              } else {
                gs = (s - refv[k]) * cgv[k];
                rg[k] -= gs;  // :440
              }
              acc[v][0][k] = xfma(gs, w00, acc[v][0][k]);  // :441-444
              acc[v][1][k] = xfma(gs, w01, acc[v][1][k]);
              acc[v][2][k] = xfma(gs, w11, acc[v][2][k]);
              acc[v][3][k] = xfma(gs, w10, acc[v][3][k]);
              const R t1 = t11[k] - t10[k] - t01[k] + t00[k];  // :447-449
              hg = xfma(gs, xfma(t1, pr.dw, t10[k] - t00[k]), hg);
              wg = xfma(gs, xfma(t1, pr.dh, t01[k] - t00[k]), wg);
            }
            dvox = xfma(pr.gh, hg, xfma(pr.gw, wg, dvox));  // :451
          }
        }
        if (KIND == 2) {
          for (int o = LG >> 1; o > 0; o >>= 1) dvox += __shfl_xor_sync(0xffffffffu, dvox, o);
          if (li == j) dkeep = dvox;
        } else {
          dsum += dvox;
        }
      }
      if (KIND == 2 && dv) {
        // v2:375-378,477: a plain store per voxel (zero where no view saw it); later passes add
        R* dg = static_cast<R*>(a.depth_grad) + pix * a.D + dA;
        if (n0 == 0) *dg = dkeep;
        else *dg += dkeep;
      }
      __syncwarp();
    }

    if (lane_on) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if (cur[v] >= 0) {
          R* gp = src_grad + (size_t)cur[v] * C + li * CPL;
          red_add<R, CPL>(gp, acc[v][0]);
          red_add<R, CPL>(gp + C, acc[v][1]);
          red_add<R, CPL>(gp + (size_t)Ws * C + C, acc[v][2]);
          red_add<R, CPL>(gp + (size_t)Ws * C, acc[v][3]);
        }
      }
    }
  }

  if (lane_on) red_add<R, CPL>(static_cast<R*>(a.ref_grad) + pix * C + li * CPL, rg);
  if (KIND != 2) {
    for (int o = LG >> 1; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
    if (pvalid && li == 0) atomicAdd(static_cast<R*>(a.depth_grad) + pix, dsum);  // :454
  }
}

}  // namespace chop
