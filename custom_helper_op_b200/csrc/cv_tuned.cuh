// Tuned CostVolume (KIND 1, MEAN, fused arithmetic) kernels for compile-time channel counts.
//
// Same decomposition as the generic kernels in cv_fwd.cuh / cv_bwd.cuh - LG = C/CPL lanes per pixel,
// phase A projects one voxel per lane, phase B does the channel work - with the per-channel-lane
// overhead stripped out of phase B:
//   * phase A leaves a ready texel POINTER and the four bilinear weights in the record, so the
//     redundant per-lane index arithmetic disappears (C is a template constant: the +C neighbour is an
//     immediate offset of the load);
//   * views that do not see the voxel get zero weights and a zero validity factor instead of a branch,
//     so phase B of the forward kernel has uniform control flow and the depth loop is fully unrolled
//     (record and output addresses become immediates);
//   * the number of valid views and its reciprocal are produced once per voxel in phase A.
// Results: mask bit-exact (projection stays unfused), cost / gradients within the float tolerances.
#pragma once
#include "cv_project.cuh"

namespace chop {

template <typename T>
struct alignas(16) RecB {
  const T* p;
  float dh, dw, gh, gw;
  float scale;  // record of the pass's first view only: 2/(valid views), 0 when the voxel is skipped
  int texel;    // -1: nothing to do for this view
};

template <typename T>
__host__ __device__ inline size_t tuned_fwd_smem_per_warp(int N, int G) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)N * 32 * sizeof(ProjF<float>);
}
template <typename T>
__host__ __device__ inline size_t tuned_bwd_smem_per_warp(int N, int G, int NV) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)NV * 32 * sizeof(RecB<T>);
}

// ---------------------------------------------------------------------------------------------------
// forward
//
// The four texel loads per (voxel, view) are what saturates the L1 data path in a straightforward
// kernel: 512 B gathered for every 128 B written.  Consecutive depth planes of one pixel project onto
// almost the same spot of a source view (a fraction of a pixel apart), so the loop nest here is
//     depth block (LG planes) -> view -> plane
// with the 2x2 texel footprint cached in registers along the innermost loop and reloaded only when the
// footprint moves.  On a reload the corners are turned into differences against the reference pixel
// (a0 = t00 - ref, u = t10 - t00, v = t01 - t00, t1 = t11 - t01 - u), after which a plane costs four
// fused operations per channel:  df = a0 + dw*v + dh*(u + dw*t1),  acc += df*df.
// ---------------------------------------------------------------------------------------------------
template <typename T, int C, int CPL>
__global__ void __launch_bounds__(256) cv_fwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  static_assert(LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 32, "C/CPL must be a power of two <= 32");
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1);
  const int g = lane / LG;

  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk;
  const int dhi = min(a.d_end, dlo + a.chunk);
  const int N = a.N;
  const int D = a.D;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<float>* coef = reinterpret_cast<Coef<float>*>(mine);
  ProjF<float>* proj = reinterpret_cast<ProjF<float>*>(coef + N * G);

  stage_coefs<float>(a, coef, lane, G, pix0);
  __syncwarp();

  const T* src_lane = static_cast<const T*>(a.src) + li * CPL;
  float refv[CPL];
  Vec<T, float, CPL>::load(static_cast<const T*>(a.ref) + pix * C + li * CPL, refv);
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const size_t row = (size_t)a.Ws * C;
  const ProjF<float>* myrec = proj + g * LG;
  float* out = static_cast<float*>(a.cost) + (pix * D + dlo) * C + li * CPL;

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG * C) {
    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
    float inv_mine;
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = dv ? xadd(base, offs[d]) : 0.0f;
      int used = 0;
      for (int n = 0; n < N; ++n) {
        ProjF<float> r;
        r.texel = -1;
        r.dh = r.dw = r.aux = 0.0f;
        if (dv) {
          float gh, gw;
          r.texel = project<float, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, gh, gw);
          used += r.texel >= 0;
        }
        proj[n * 32 + lane] = r;
      }
      if (dv) __stcs(a.mask + pix * D + d, used);
      inv_mine = used > 0 ? 1.0f / (float)used : 0.0f;
    }
    __syncwarp();

    // ---- phase B ---------------------------------------------------------------------------------------
    float acc[LG][CPL];
#pragma unroll
    for (int j = 0; j < LG; ++j)
#pragma unroll
      for (int k = 0; k < CPL; ++k) acc[j][k] = 0.0f;

    for (int n = 0; n < N; ++n) {
      const ProjF<float>* r = myrec + n * 32;
      int cur = -1;
      float a0[CPL], u[CPL], v[CPL], t1[CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) a0[k] = u[k] = v[k] = t1[k] = 0.0f;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = r[j];
        if (rc.texel >= 0) {
          if (rc.texel != cur) {
            cur = rc.texel;
            const T* p00 = src_lane + (size_t)rc.texel * C;
            const T* p10 = p00 + row;
            float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
            Vec<T, float, CPL>::load(p00, t00);
            Vec<T, float, CPL>::load(p00 + C, t01);
            Vec<T, float, CPL>::load(p10, t10);
            Vec<T, float, CPL>::load(p10 + C, t11);
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              a0[k] = t00[k] - refv[k];
              u[k] = t10[k] - t00[k];
              v[k] = t01[k] - t00[k];
              t1[k] = (t11[k] - t01[k]) - u[k];
            }
          }
#pragma unroll
          for (int k = 0; k < CPL; ++k) {
            const float X = fmaf(t1[k], rc.dw, u[k]);
            const float df = fmaf(rc.dh, X, fmaf(rc.dw, v[k], a0[k]));
            acc[j][k] = fmaf(df, df, acc[j][k]);
          }
        }
      }
    }

#pragma unroll
    for (int j = 0; j < LG; ++j) {
      const float inv = __shfl_sync(0xffffffffu, inv_mine, g * LG + j);
#pragma unroll
      for (int k = 0; k < CPL; ++k) acc[j][k] *= inv;
      if (pvalid && dblk + j < dhi) store_stream<float, CPL>(out + j * C, acc[j]);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------
template <typename T, int C, int CPL, int NV>
__global__ void __launch_bounds__(256) cv_bwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  static_assert(LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 32, "C/CPL must be a power of two <= 32");
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1);
  const int g = lane / LG;

  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk;
  const int dhi = min(a.d_end, dlo + a.chunk);
  const int N = a.N;
  const int D = a.D;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<float>* coef = reinterpret_cast<Coef<float>*>(mine);
  RecB<T>* proj = reinterpret_cast<RecB<T>*>(coef + N * G);

  stage_coefs<float>(a, coef, lane, G, pix0);
  __syncwarp();

  const T* src = static_cast<const T*>(a.src);
  float* src_grad = static_cast<float*>(a.src_grad);
  float refv[CPL], rg[CPL];
  Vec<T, float, CPL>::load(static_cast<const T*>(a.ref) + pix * C + li * CPL, refv);
#pragma unroll
  for (int k = 0; k < CPL; ++k) rg[k] = 0.0f;
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const size_t row = (size_t)a.Ws * C;
  const RecB<T>* myrec = proj + g * LG;
  float dsum = 0.0f;

  for (int n0 = 0; n0 < N; n0 += NV) {
    float acc[NV][4][CPL];
    int cur[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      cur[v] = -1;
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int k = 0; k < CPL; ++k) acc[v][q][k] = 0.0f;
    }
    const float* cgb = static_cast<const float*>(a.cost_grad) + (pix * D + dlo) * C + li * CPL;

    for (int dblk = dlo; dblk < dhi; dblk += LG, cgb += LG * C) {
      // the upstream gradient of the block's first plane is requested before the projection math
      float cgn[CPL];
      load_stream<float, CPL>(cgb, cgn);

      // ---- phase A ---------------------------------------------------------------------------------
      {
        const int d = dblk + li;
        const bool dv = pvalid && d < dhi;
        float depth = 0.0f, scale = 0.0f;
        bool live = false;
        if (dv) {
          depth = xadd(base, offs[d]);
          const int m0 = __ldg(a.mask + pix * D + d);
          live = m0 > 0;                          // cost_volume_kernels_gpu.cu.cc:367
          if (live) scale = 2.0f / (float)m0;     // :439
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          RecB<T> r;
          r.p = src;
          r.dh = r.dw = r.gh = r.gw = 0.0f;
          r.scale = scale;
          r.texel = -1;
          const int n = n0 + v;
          if (live && n < N) {
            r.texel = project<float, true>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, r.gh, r.gw);
            if (r.texel >= 0) r.p = src + (size_t)r.texel * C;
          }
          proj[v * 32 + lane] = r;
        }
      }
      __syncwarp();

      // ---- phase B ---------------------------------------------------------------------------------
      const int jn = dhi - dblk;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        if (j < jn) {
          float cgv[CPL];
#pragma unroll
          for (int k = 0; k < CPL; ++k) cgv[k] = cgn[k];
          if (j + 1 < LG && j + 1 < jn) load_stream<float, CPL>(cgb + (j + 1) * C, cgn);
          const RecB<T>* r = myrec + j;
          const float scale = r->scale;
#pragma unroll
          for (int k = 0; k < CPL; ++k) cgv[k] *= scale;
          float dvox = 0.0f;
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            const RecB<T> rc = r[v * 32];
            if (rc.texel < 0) continue;
            if (rc.texel != cur[v]) {
              if (cur[v] >= 0) {
                float* gp = src_grad + (size_t)cur[v] * C + li * CPL;
                red_add<float, CPL>(gp, acc[v][0]);
                red_add<float, CPL>(gp + C, acc[v][1]);
                red_add<float, CPL>(gp + row, acc[v][2]);
                red_add<float, CPL>(gp + row + C, acc[v][3]);
              }
              cur[v] = rc.texel;
#pragma unroll
              for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int k = 0; k < CPL; ++k) acc[v][q][k] = 0.0f;
            }
            float w00, w01, w11, w10;
            bilinear_weights_fast(rc.dh, rc.dw, w00, w01, w11, w10);
            const T* p00 = rc.p + li * CPL;
            const T* p10 = p00 + row;
            float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
            Vec<T, float, CPL>::load(p00, t00);
            Vec<T, float, CPL>::load(p00 + C, t01);
            Vec<T, float, CPL>::load(p10, t10);
            Vec<T, float, CPL>::load(p10 + C, t11);
            float hg = 0.0f, wg = 0.0f;
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              // bilinear sample and its two spatial derivatives share the corner differences
              const float u = t10[k] - t00[k];             // d/dh at dw = 0
              const float vv = t01[k] - t00[k];            // d/dw at dh = 0
              const float t1 = (t11[k] - t01[k]) - u;      // :447
              const float X = fmaf(t1, rc.dw, u);          // d(sample)/dh
              const float Y = fmaf(t1, rc.dh, vv);         // d(sample)/dw
              const float s = fmaf(rc.dh, X, fmaf(rc.dw, vv, t00[k]));
              const float gs = (s - refv[k]) * cgv[k];     // :439
              rg[k] -= gs;                                 // :440
              acc[v][0][k] = fmaf(gs, w00, acc[v][0][k]);  // :441-444 (acc[2] is corner (fh+1,fw))
              acc[v][1][k] = fmaf(gs, w01, acc[v][1][k]);
              acc[v][2][k] = fmaf(gs, w10, acc[v][2][k]);
              acc[v][3][k] = fmaf(gs, w11, acc[v][3][k]);
              hg = fmaf(gs, X, hg);                        // :448
              wg = fmaf(gs, Y, wg);                        // :449
            }
            dvox = fmaf(rc.gh, hg, fmaf(rc.gw, wg, dvox));  // :451
          }
          dsum += dvox;
        }
      }
      __syncwarp();
    }

#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (cur[v] >= 0) {
        float* gp = src_grad + (size_t)cur[v] * C + li * CPL;
        red_add<float, CPL>(gp, acc[v][0]);
        red_add<float, CPL>(gp + C, acc[v][1]);
        red_add<float, CPL>(gp + row, acc[v][2]);
        red_add<float, CPL>(gp + row + C, acc[v][3]);
      }
    }
  }

  if (pvalid) red_add<float, CPL>(static_cast<float*>(a.ref_grad) + pix * C + li * CPL, rg);
#pragma unroll
  for (int o = LG >> 1; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
  if (pvalid && li == 0) atomicAdd(static_cast<float*>(a.depth_grad) + pix, dsum);  // :454
}

}  // namespace chop
