// Tuned CostVolume (KIND 1, MEAN, fused arithmetic) kernels for compile-time channel counts.
//
// Same warp decomposition as the generic kernels in cv_fwd.cuh / cv_bwd.cuh - LG = C/CPL lanes per
// pixel, phase A projects one voxel per lane into every view, phase B does the channel work - but the
// loop nest of phase B is  depth block -> view -> plane  and the 2x2 texel footprint of a view is kept
// in registers while consecutive planes keep hitting it.  Results: mask bit-exact (the projection stays
// unfused), cost and gradients within the float tolerances.
#pragma once
#include "cv_project.cuh"

namespace chop {

template <typename T>
__host__ __device__ inline size_t tuned_fwd_smem_per_warp(int N, int G) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)N * 32 * sizeof(ProjF<float>);
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
// three 256-thread CTAs per SM (<= 85 registers) measured fastest: 4 still fits, 5 and up spill
#ifndef CHOP_FWD_MIN_BLOCKS
#define CHOP_FWD_MIN_BLOCKS 3
#endif
// AGG = true is CostAggregate: the same sum of squared differences added over the channels and divided
// by views*C (cost_aggregate_kernels_gpu.cu.cc:34-127); cost is one float per voxel, written coalesced
// after a reduce-scatter over the pixel's lanes.
template <typename T, int C, int CPL, bool AGG = false>
__global__ void __launch_bounds__(256, CHOP_FWD_MIN_BLOCKS) cv_fwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
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
  float* out = AGG ? static_cast<float*>(a.cost) + pix * D + dlo + li
                   : static_cast<float*>(a.cost) + (pix * D + dlo) * C + li * CPL;

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += AGG ? LG : LG * C) {
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
      // A view that does not see a plane is the "empty footprint" (-1): all differences zero, so the
      // plane contributes exactly zero and the arithmetic below needs no validity branch.
      int cur = -1;
      float a0[CPL], u[CPL], v[CPL], t1[CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) a0[k] = u[k] = v[k] = t1[k] = 0.0f;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = r[j];
        if (rc.texel != cur) {
          cur = rc.texel;
          if (rc.texel >= 0) {
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
          } else {
#pragma unroll
            for (int k = 0; k < CPL; ++k) a0[k] = u[k] = v[k] = t1[k] = 0.0f;
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

    if constexpr (AGG) {
      // channel sum per plane, then lane li collects plane li (reduce-scatter over the pixel's lanes)
      float tot[LG];
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        tot[j] = acc[j][0];
#pragma unroll
        for (int k = 1; k < CPL; ++k) tot[j] += acc[j][k];
      }
#pragma unroll
      for (int s = LG / 2; s >= 1; s >>= 1) {
#pragma unroll
        for (int i = 0; i < s; ++i) {
          const bool hi = (li & s) != 0;
          const float keep = hi ? tot[i + s] : tot[i];
          const float send = hi ? tot[i] : tot[i + s];
          tot[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
      }
      if (pvalid && dblk + li < dhi) __stcs(out, tot[0] * inv_mine * (1.0f / (float)C));
    } else {
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const float inv = __shfl_sync(0xffffffffu, inv_mine, g * LG + j);
#pragma unroll
        for (int k = 0; k < CPL; ++k) acc[j][k] *= inv;
        if (pvalid && dblk + j < dhi) store_stream<float, CPL>(out + j * C, acc[j]);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------------
// forward, MIN (cost_volume_kernels_gpu.cu.cc:133-228): per channel the smallest squared difference over
// the views and the view that gave it (-1 and the largest float where no view sees the voxel).  Same
// loop nest and register-cached footprint as the MEAN kernel, but the RAW corners are kept and every
// operation is unfused and in the reference's order, so cost and arg index are bit-exact.  The arg
// indices of a lane's four channels ride in one register per plane (a byte each, 0xFF = -1): at most
// 254 source views (the host falls back to the generic kernel beyond that).
// ---------------------------------------------------------------------------------------------------
template <typename T, int C, int CPL>
__global__ void __launch_bounds__(256, 2) cv_fwd_min_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  static_assert(CPL == 4 && LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 8, "four channels per lane, at most 8 lanes per pixel");
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
  int* outm = a.mask + (pix * D + dlo) * C + li * CPL;

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG * C, outm += LG * C) {
    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = dv ? xadd(base, offs[d]) : 0.0f;
      for (int n = 0; n < N; ++n) {
        ProjF<float> r;
        r.texel = -1;
        r.dh = r.dw = r.aux = 0.0f;
        if (dv) {
          float gh, gw;
          r.texel = project<float, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, gh, gw);
        }
        proj[n * 32 + lane] = r;
      }
    }
    __syncwarp();

    // ---- phase B ---------------------------------------------------------------------------------------
    float acc[LG][CPL];
    unsigned argp[LG];
#pragma unroll
    for (int j = 0; j < LG; ++j) {
      argp[j] = 0xFFFFFFFFu;
#pragma unroll
      for (int k = 0; k < CPL; ++k) acc[j][k] = 3.402823466e+38f;   // :174-177
    }

    for (int n = 0; n < N; ++n) {
      const ProjF<float>* r = myrec + n * 32;
      int cur = -1;
      float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) t00[k] = t01[k] = t10[k] = t11[k] = 0.0f;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = r[j];
        if (rc.texel < 0) continue;            // the view does not see this plane (:194-197)
        if (rc.texel != cur) {
          cur = rc.texel;
          const T* p00 = src_lane + (size_t)rc.texel * C;
          const T* p10 = p00 + row;
          Vec<T, float, CPL>::load(p00, t00);
          Vec<T, float, CPL>::load(p00 + C, t01);
          Vec<T, float, CPL>::load(p10, t10);
          Vec<T, float, CPL>::load(p10 + C, t11);
        }
        float w00, w01, w11, w10;
        bilinear_weights(rc.dh, rc.dw, w00, w01, w11, w10);
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
          const float s = xadd(xadd(xadd(xmul(w00, t00[k]), xmul(w01, t01[k])), xmul(w11, t11[k])), xmul(w10, t10[k]));
          const float df = xsub(s, refv[k]);
          const float sq = xmul(df, df);
          if (acc[j][k] > sq) {                 // :214-217 strictly smaller: the first view wins a tie
            acc[j][k] = sq;
            argp[j] = (argp[j] & ~(0xFFu << (8 * k))) | ((unsigned)n << (8 * k));
          }
        }
      }
    }

#pragma unroll
    for (int j = 0; j < LG; ++j) {
      if (pvalid && dblk + j < dhi) {
        store_stream<float, CPL>(out + j * C, acc[j]);
        int arg[CPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k) arg[k] = (int)(signed char)((argp[j] >> (8 * k)) & 0xFFu);
        store_stream<int, CPL>(outm + j * C, arg);
      }
    }
    __syncwarp();
  }
}

// CostAggregate MIN forward (cost_aggregate_kernels_gpu.cu.cc:129-227): the view with the smallest channel SUM of
// squared differences wins the voxel.  The reference adds the C values one by one, so the sum is formed in that
// order by one lane per plane after a transpose through shared memory (rows of C + 4 floats: conflict-free 16-byte
// reads); the corners stay cached in registers along the planes as in the kernels above.
template <typename T, int C, int CPL>
__global__ void __launch_bounds__(256, 2) cv_agg_min_fwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  static_assert(CPL == 4 && LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 8, "four channels per lane, at most 8 lanes per pixel");
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
  constexpr int RS = C + 4;                                            // row stride of the transpose scratch (floats)
  float* rows = reinterpret_cast<float*>(proj + N * 32) + (g * LG) * RS;   // this pixel's LG rows

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
  float* out = static_cast<float*>(a.cost) + pix * D + dlo + li;
  int* outm = a.mask + pix * D + dlo + li;

  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG, outm += LG) {
    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = dv ? xadd(base, offs[d]) : 0.0f;
      for (int n = 0; n < N; ++n) {
        ProjF<float> r;
        r.texel = -1;
        r.dh = r.dw = r.aux = 0.0f;
        if (dv) {
          float gh, gw;
          r.texel = project<float, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, gh, gw);
        }
        proj[n * 32 + lane] = r;
      }
    }
    __syncwarp();

    // ---- phase B: per view, every lane computes its four squared differences for the LG planes (footprint cached
    // along the planes), the slices meet in shared memory and lane li adds plane li's C values in channel order -----
    float tot = 3.402823466e+38f;
    int targ = -1;
    for (int n = 0; n < N; ++n) {
      const ProjF<float>* r = myrec + n * 32;
      int cur = -1;
      float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) t00[k] = t01[k] = t10[k] = t11[k] = 0.0f;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = r[j];
        if (rc.texel < 0) continue;            // the view does not see this plane: its row is not read either
        if (rc.texel != cur) {
          cur = rc.texel;
          const T* p00 = src_lane + (size_t)rc.texel * C;
          const T* p10 = p00 + row;
          Vec<T, float, CPL>::load(p00, t00);
          Vec<T, float, CPL>::load(p00 + C, t01);
          Vec<T, float, CPL>::load(p10, t10);
          Vec<T, float, CPL>::load(p10 + C, t11);
        }
        float w00, w01, w11, w10;
        bilinear_weights(rc.dh, rc.dw, w00, w01, w11, w10);
        float sq[CPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
          const float s = xadd(xadd(xadd(xmul(w00, t00[k]), xmul(w01, t01[k])), xmul(w11, t11[k])), xmul(w10, t10[k]));
          const float df = xsub(s, refv[k]);
          sq[k] = xmul(df, df);
        }
        store_slice<float, CPL>(rows + j * RS + li * CPL, sq);
      }
      __syncwarp();
      if (r[li].texel >= 0) {                  // cost_aggregate_kernels_gpu.cu.cc:190-223
        const float s = row_sum_ordered<float>(rows + li * RS, C, true, 0.0f);
        if (tot > s) { tot = s; targ = n; }
      }
      __syncwarp();
    }
    if (pvalid && dblk + li < dhi) {
      __stcs(out, targ >= 0 ? xdiv(tot, (float)C) : 0.0f);
      __stcs(outm, targ);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------------
// backward
//
// Loop nest as in the forward kernel: depth block (LG planes) -> view -> plane, with the footprint's
// corner differences (a0, u, v, t1) AND the four corner gradient sums in registers along the innermost
// loop.  A footprint change (or the end of the block) flushes the sums with four 16-byte vector
// reductions and reloads the corners.  Register use does not depend on the number of views, and the
// upstream gradient is read from HBM exactly once: each block's slice of cost_grad (LG planes x C
// floats per pixel, contiguous) is staged in shared memory with cp.async one block ahead of its use, so
// its latency hides behind the previous block's arithmetic and every view reads it from shared memory.
// d(ref) and d(base_plane) are register sums written once per work item.
// ---------------------------------------------------------------------------------------------------
// six 128-thread CTAs per SM with a single staging buffer measured fastest (271 us at c1 against 288 us
// with two buffers and five CTAs: the extra shared memory costs more L1 and occupancy than the deeper
// prefetch gains)
#ifndef CHOP_BWD_MIN_BLOCKS
#define CHOP_BWD_MIN_BLOCKS 6
#endif
#ifndef CHOP_BWD_CG_BUFS
#define CHOP_BWD_CG_BUFS 1
#endif
constexpr int CG_BUFS = CHOP_BWD_CG_BUFS;  // 2: copy a block ahead into the other buffer; 1: copy after use

struct alignas(8) RecG {
  float gh, gw;  // d(sample row)/d(depth), d(sample column)/d(depth)
};

// `staged` = per-channel tensors copied into shared memory ahead of use: cost_grad, and for MIN also
// the arg-index tensor; each buffer holds G*LG*C values = 128*C bytes.
template <int C>
__host__ __device__ inline size_t tuned_bwd_smem_per_warp(int N, int G, int staged = 1) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)N * 32 * (sizeof(ProjF<float>) + sizeof(RecG)) +
         (size_t)staged * CG_BUFS * 128 * C;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// AGG = true is CostAggregateGrad: one upstream value per voxel, d(cost)/d(sample) = 2*diff*cost_grad/(views*C)
// (cost_aggregate_kernels_gpu.cu.cc:385,431); the upstream value rides in the phase-A record, nothing is staged.
// Moments of the per-plane sample gradients over one 2x2 footprint -> the four corner gradients, added to
// src_grad with vector reductions; the first moment is also what d(ref) loses.
//   m0 = sum g, m1 = sum g*dw, m2 = sum g*dh, m3 = sum g*dh*dw
//   corner (0,0): m0 - m1 - m2 + m3   (0,1): m1 - m3   (1,0): m2 - m3   (1,1): m3
template <int CPL>
__device__ __forceinline__ void flush_corners(float* gp, size_t row, int C, float (&m)[4][CPL], float (&rg)[CPL]) {
  float c00[CPL], c01[CPL], c10[CPL];
#pragma unroll
  for (int k = 0; k < CPL; ++k) {
    rg[k] -= m[0][k];
    c01[k] = m[1][k] - m[3][k];
    c10[k] = m[2][k] - m[3][k];
    c00[k] = (m[0][k] - m[1][k]) - c10[k];
  }
  red_add<float, CPL>(gp, c00);
  red_add<float, CPL>(gp + C, c01);
  red_add<float, CPL>(gp + row, c10);
  red_add<float, CPL>(gp + row + C, m[3]);
}

// RMIN = true is the MIN reduction: `mask` holds the winning view per (voxel, channel) (per voxel for
// AGG) and only that view receives the gradient (cost_volume_kernels_gpu.cu.cc:472-577,
// cost_aggregate_kernels_gpu.cu.cc:462-568); a voxel whose first channel has no winner is skipped (:484).
template <typename T, int C, int CPL, bool AGG = false, bool RMIN = false>
__global__ void __launch_bounds__(128, CHOP_BWD_MIN_BLOCKS) cv_bwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  static_assert(CPL == 4, "the cost_grad staging copies 16 bytes per lane and plane");
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
  ProjF<float>* recA = reinterpret_cast<ProjF<float>*>(coef + N * G);  // aux = 2/(valid views)
  RecG* recG = reinterpret_cast<RecG*>(recA + N * 32);
  float* cgbuf = reinterpret_cast<float*>(recG + N * 32);             // [2][G][LG][C]
  float* cg_mine = cgbuf + (g * LG) * C + li * CPL;                    // + buf*32*C + j*C
  constexpr bool STAGE_MASK = RMIN && !AGG;
  constexpr int MK_OFF = CG_BUFS * 32 * C;                             // arg indices behind the cost_grad buffers

  stage_coefs<float>(a, coef, lane, G, pix0);

  const T* src_lane = static_cast<const T*>(a.src) + li * CPL;
  float* sg_lane = static_cast<float*>(a.src_grad) + li * CPL;
  float refv[CPL], rg[CPL];
  Vec<T, float, CPL>::load(static_cast<const T*>(a.ref) + pix * C + li * CPL, refv);
#pragma unroll
  for (int k = 0; k < CPL; ++k) rg[k] = 0.0f;
  const int b = (int)(pix / ((long long)a.H * a.W));
  const float base = static_cast<const float*>(a.depth)[pix];
  const float* offs = static_cast<const float*>(a.offsets) + (long long)b * D;
  const size_t row = (size_t)a.Ws * C;
  float dsum = 0.0f;
  const float* cg_src = static_cast<const float*>(a.cost_grad) + (pix * D + dlo) * C + li * CPL;
  const int* mk_src = a.mask + (pix * D + dlo) * C + li * CPL;  // + (plane - dlo) * C; read for MIN only

  // stage the first block's upstream gradient
  if constexpr (!AGG) {
#pragma unroll
    for (int j = 0; j < LG; ++j) {
      if (dlo + j < dhi) {
        cp_async16(cg_mine + j * C, cg_src + j * C);
        if (STAGE_MASK) cp_async16(cg_mine + MK_OFF + j * C, mk_src + j * C);
      } else {
        *reinterpret_cast<float4*>(cg_mine + j * C) = make_float4(0.f, 0.f, 0.f, 0.f);  // never left uninitialised
        if (STAGE_MASK) *reinterpret_cast<int4*>(cg_mine + MK_OFF + j * C) = make_int4(-1, -1, -1, -1);
      }
    }
    cp_async_commit();
  }
  __syncwarp();

  // The lane's validity count / winning view of plane dblk+li streams in from HBM: it is requested one block ahead,
  // so phase A does not start with an exposed DRAM round trip.
  const int mk_stride = (RMIN && !AGG) ? C : 1;
  int m_next = 0;
  float ag_next = 0.0f;   // aggregate: the voxel's single upstream value, requested a block ahead as well
  if (pvalid && dlo + li < dhi) {
    m_next = __ldg(a.mask + (pix * D + dlo + li) * mk_stride);
    if (AGG) ag_next = __ldg(static_cast<const float*>(a.cost_grad) + pix * D + dlo + li);
  }
  int buf = 0;
  for (int dblk = dlo; dblk < dhi; dblk += LG, cg_src += LG * C, buf ^= (CG_BUFS - 1)) {
    if (!AGG && CG_BUFS == 2) {
      cp_async_wait_all();  // this block's slice has landed (each lane reads back only what it copied)
      __syncwarp();         // and every lane is done with the other buffer and with the records
      const int nxt = dblk + LG;
      float* dst = cg_mine + (buf ^ 1) * 32 * C;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        if (nxt + j < dhi) {
          cp_async16(dst + j * C, cg_src + (LG + j) * C);
          if (STAGE_MASK) cp_async16(dst + MK_OFF + j * C, mk_src + (nxt - dlo + j) * C);
        } else {
          *reinterpret_cast<float4*>(dst + j * C) = make_float4(0.f, 0.f, 0.f, 0.f);
          if (STAGE_MASK) *reinterpret_cast<int4*>(dst + MK_OFF + j * C) = make_int4(-1, -1, -1, -1);
        }
      }
      cp_async_commit();
    } else {
      __syncwarp();
    }

    // ---- phase A: lane (g, li) projects plane dblk+li of pixel g into every view ---------------------
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      float depth = 0.0f, scale = 0.0f;
      bool live = false;
      const int m0 = m_next;
      const float ag0 = ag_next;
      if (pvalid && d + LG < dhi) {
        m_next = __ldg(a.mask + (pix * D + d + LG) * mk_stride);
        if (AGG) ag_next = __ldg(static_cast<const float*>(a.cost_grad) + pix * D + d + LG);
      }
      if (dv) {
        depth = xadd(base, offs[d]);
        if constexpr (RMIN) {
          live = m0 >= 0;                    // :484, aggregate :476
          scale = 2.0f;                      // :560
          if (AGG && live)                   // aggregate :500
            scale = 2.0f * ag0 / (float)C;
        } else {
          live = m0 > 0;                       // cost_volume_kernels_gpu.cu.cc:367
          if (live) scale = 2.0f / (float)m0;  // :439
          if (AGG && live)                     // one upstream value per voxel, divided by views*C
            scale = 2.0f * ag0 / (float)(m0 * C);
        }
      }
      for (int n = 0; n < N; ++n) {
        ProjF<float> r;
        RecG q;
        r.texel = -1;
        r.dh = r.dw = 0.0f;
        r.aux = scale;
        q.gh = q.gw = 0.0f;
        // aggregate MIN: only the winning view of the voxel is differentiated
        if (live && (!(RMIN && AGG) || m0 == n))
          r.texel = project<float, true>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, q.gh, q.gw);
        recA[n * 32 + lane] = r;
        recG[n * 32 + lane] = q;
      }
    }
    if (!AGG && CG_BUFS == 1) cp_async_wait_all();  // the slice requested at the end of the previous block
    __syncwarp();

    // ---- phase B ---------------------------------------------------------------------------------------
    const float* cgb = cg_mine + buf * 32 * C;
    for (int n = 0; n < N; ++n) {
      const ProjF<float>* rA = recA + n * 32 + g * LG;
      const RecG* rGp = recG + n * 32 + g * LG;
      int cur = -1;
      float a0[CPL], u[CPL], v[CPL], t1[CPL], acc[4][CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) {
        a0[k] = u[k] = v[k] = t1[k] = 0.0f;
        acc[0][k] = acc[1][k] = acc[2][k] = acc[3][k] = 0.0f;
      }
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = rA[j];
        if (rc.texel >= 0) {
          if (rc.texel != cur) {
            if (cur >= 0) flush_corners<CPL>(sg_lane + (size_t)cur * C, row, C, acc, rg);
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
              t1[k] = (t11[k] - t01[k]) - u[k];  // :447
              acc[0][k] = acc[1][k] = acc[2][k] = acc[3][k] = 0.0f;
            }
          }
          const RecG rq = rGp[j];
          float cgs[4];
          if constexpr (AGG) {
            cgs[0] = cgs[1] = cgs[2] = cgs[3] = rc.aux;
          } else {
            const float4 cg4 = *reinterpret_cast<const float4*>(cgb + j * C);
            cgs[0] = cg4.x * rc.aux; cgs[1] = cg4.y * rc.aux; cgs[2] = cg4.z * rc.aux; cgs[3] = cg4.w * rc.aux;
            if constexpr (RMIN) {  // :553 a channel's gradient goes to its winning view only
              const int4 mk = *reinterpret_cast<const int4*>(cgb + MK_OFF + j * C);
              if (mk.x != n) cgs[0] = 0.0f;
              if (mk.y != n) cgs[1] = 0.0f;
              if (mk.z != n) cgs[2] = 0.0f;
              if (mk.w != n) cgs[3] = 0.0f;
            }
          }
          // Per channel: gs = d(cost)/d(sample) (:439).  The four corner sums (:441-444) are kept as moments
          // sum gs, sum gs*dw, sum gs*dh, sum gs*dh*dw and turned into corner values when the footprint is
          // flushed; d(ref) (:440) is taken from the first moment at the same time.  The two coordinate
          // derivatives (:448-449) are dw*P + Q and dh*P + R with P = sum gs*t1, Q = sum gs*u, R = sum gs*v.
          const float hw = rc.dh * rc.dw;
          float P = 0.0f, Q = 0.0f, R = 0.0f;
#pragma unroll
          for (int k = 0; k < CPL; ++k) {
            const float X = fmaf(t1[k], rc.dw, u[k]);
            const float df = fmaf(rc.dh, X, fmaf(rc.dw, v[k], a0[k]));  // sample - ref
            const float gs = df * cgs[k];
            acc[0][k] += gs;
            acc[1][k] = fmaf(gs, rc.dw, acc[1][k]);
            acc[2][k] = fmaf(gs, rc.dh, acc[2][k]);
            acc[3][k] = fmaf(gs, hw, acc[3][k]);
            P = fmaf(gs, t1[k], P);
            Q = fmaf(gs, u[k], Q);
            R = fmaf(gs, v[k], R);
          }
          dsum = fmaf(rq.gh, fmaf(rc.dw, P, Q), fmaf(rq.gw, fmaf(rc.dh, P, R), dsum));  // :451
        }
      }
      if (cur >= 0) flush_corners<CPL>(sg_lane + (size_t)cur * C, row, C, acc, rg);
    }
    if (!AGG && CG_BUFS == 1) {
      // single buffer: each lane has finished reading its own slots, request the next block's slice now
      const int nxt = dblk + LG;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        if (nxt + j < dhi) {
          cp_async16(cg_mine + j * C, cg_src + (LG + j) * C);
          if (STAGE_MASK) cp_async16(cg_mine + MK_OFF + j * C, mk_src + (nxt - dlo + j) * C);
        } else {
          *reinterpret_cast<float4*>(cg_mine + j * C) = make_float4(0.f, 0.f, 0.f, 0.f);
          if (STAGE_MASK) *reinterpret_cast<int4*>(cg_mine + MK_OFF + j * C) = make_int4(-1, -1, -1, -1);
        }
      }
      cp_async_commit();
    }
  }
  cp_async_wait_all();

  if (pvalid) red_add<float, CPL>(static_cast<float*>(a.ref_grad) + pix * C + li * CPL, rg);
#pragma unroll
  for (int o = LG >> 1; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
  if (pvalid && li == 0) atomicAdd(static_cast<float*>(a.depth_grad) + pix, dsum);  // :454
}

// ---------------------------------------------------------------------------------------------------
// CostVolumeV2 (group-wise correlation, per-pixel depth hypotheses), MEAN, compile-time C and channels
// per group SUB in {1,2,4} (a lane's four channels cover whole groups).  Same loop nest and footprint
// caching as above.  Reference: cost_volume_kernels_gpu_v2.cu.cc:33-135 (forward), :349-479 (gradient).
// ---------------------------------------------------------------------------------------------------
template <typename T>
__host__ __device__ inline size_t tuned2_bwd_smem_per_warp(int N, int G) {
  return (size_t)N * G * sizeof(Coef<float>) + (size_t)N * 32 * (sizeof(ProjF<float>) + sizeof(RecG));
}

// Forward: on a reload the corner differences are multiplied by the reference pixel and summed over each
// group's channels, so a plane costs  acc += a0' + dw*v' + dh*(u' + dw*t1')  per GROUP (not per channel):
// the group's correlation  sum_c sample_c*ref_c  is bilinear in (dh, dw) with those four sums as coefficients.
template <typename T, int C, int SUB>
__global__ void __launch_bounds__(256, 3) cv2_fwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CPL = 4;
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  constexpr int NG = CPL / SUB;   // groups per lane
  constexpr int GR = C / SUB;     // groups per voxel
  static_assert(LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 32 && NG * SUB == CPL, "unsupported C / SUB");
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
  const float* dgrid = static_cast<const float*>(a.depth) + pix * D;
  const size_t row = (size_t)a.Ws * C;
  const ProjF<float>* myrec = proj + g * LG;
  float* out = static_cast<float*>(a.cost) + (pix * D + dlo) * GR + li * NG;

  // the lane's depth hypothesis of plane dblk+li streams in from HBM: requested one block ahead
  float depth_next = (pvalid && dlo + li < dhi) ? __ldg(dgrid + dlo + li) : 0.0f;
  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG * GR) {
    float inv_mine;
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = depth_next;
      if (pvalid && d + LG < dhi) depth_next = __ldg(dgrid + d + LG);
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

    float acc[LG][NG];
#pragma unroll
    for (int j = 0; j < LG; ++j)
#pragma unroll
      for (int q = 0; q < NG; ++q) acc[j][q] = 0.0f;

    for (int n = 0; n < N; ++n) {
      const ProjF<float>* r = myrec + n * 32;
      int cur = -1;  // the empty footprint: all terms zero
      float a0[NG], u[NG], v[NG], t1[NG];
#pragma unroll
      for (int q = 0; q < NG; ++q) a0[q] = u[q] = v[q] = t1[q] = 0.0f;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = r[j];
        if (rc.texel != cur) {
          cur = rc.texel;
#pragma unroll
          for (int q = 0; q < NG; ++q) a0[q] = u[q] = v[q] = t1[q] = 0.0f;
          if (rc.texel >= 0) {
            const T* p00 = src_lane + (size_t)rc.texel * C;
            const T* p10 = p00 + row;
            float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
            Vec<T, float, CPL>::load(p00, t00);
            Vec<T, float, CPL>::load(p00 + C, t01);
            Vec<T, float, CPL>::load(p10, t10);
            Vec<T, float, CPL>::load(p10 + C, t11);
            // The correlation is linear in the sample, so the reference pixel is applied to the four CORNERS first
            // (one dot product per corner and group) and the bilinear differences are formed on the group sums:
            // 4 multiply-adds per channel + 4 subtractions per group instead of 8 operations per channel.
            float d00[NG], d01[NG], d10[NG], d11[NG];
#pragma unroll
            for (int q = 0; q < NG; ++q) d00[q] = d01[q] = d10[q] = d11[q] = 0.0f;
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              const int q = k / SUB;
              d00[q] = fmaf(t00[k], refv[k], d00[q]);
              d01[q] = fmaf(t01[k], refv[k], d01[q]);
              d10[q] = fmaf(t10[k], refv[k], d10[q]);
              d11[q] = fmaf(t11[k], refv[k], d11[q]);
            }
#pragma unroll
            for (int q = 0; q < NG; ++q) {
              a0[q] = d00[q];
              u[q] = d10[q] - d00[q];
              v[q] = d01[q] - d00[q];
              t1[q] = (d11[q] - d01[q]) - u[q];
            }
          }
        }
#pragma unroll
        for (int q = 0; q < NG; ++q) {
          const float X = fmaf(t1[q], rc.dw, u[q]);
          acc[j][q] = fmaf(rc.dh, X, fmaf(rc.dw, v[q], acc[j][q] + a0[q]));   // += sum_c sample*ref  (v2:118-120)
        }
      }
    }

#pragma unroll
    for (int j = 0; j < LG; ++j) {
      const float inv = __shfl_sync(0xffffffffu, inv_mine, g * LG + j);
      float o[NG];
#pragma unroll
      for (int q = 0; q < NG; ++q) o[q] = acc[j][q] * inv;   // v2:128-133
      if (pvalid && dblk + j < dhi) store_stream<float, NG>(out + j * GR, o);
    }
    __syncwarp();
  }
}

// CostVolumeV2 "MIN" forward (cost_volume_kernels_gpu_v2.cu.cc:137-235; it keeps the LARGEST group correlation and the
// view that gave it): the nest and the register-cached RAW corners of the kernels above, every operation unfused and in
// the reference's order (cost and arg index bit-exact), arg indices a byte per group.
template <typename T, int C, int SUB>
__global__ void __launch_bounds__(256, 2) cv2_fwd_min_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CPL = 4;
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  constexpr int NG = CPL / SUB;   // groups per lane
  constexpr int GR = C / SUB;     // groups per voxel
  static_assert(LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 32 && NG * SUB == CPL, "unsupported C / SUB");
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
  const float* dgrid = static_cast<const float*>(a.depth) + pix * D;
  const size_t row = (size_t)a.Ws * C;
  const ProjF<float>* myrec = proj + g * LG;
  float* out = static_cast<float*>(a.cost) + (pix * D + dlo) * GR + li * NG;
  int* outm = a.mask + (pix * D + dlo) * GR + li * NG;

  // the lane's depth hypothesis of plane dblk+li streams in from HBM: requested one block ahead
  float depth_next = (pvalid && dlo + li < dhi) ? __ldg(dgrid + dlo + li) : 0.0f;
  for (int dblk = dlo; dblk < dhi; dblk += LG, out += LG * GR, outm += LG * GR) {
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const float depth = depth_next;
      if (pvalid && d + LG < dhi) depth_next = __ldg(dgrid + d + LG);
      for (int n = 0; n < N; ++n) {
        ProjF<float> r;
        r.texel = -1;
        r.dh = r.dw = r.aux = 0.0f;
        if (dv) {
          float gh, gw;
          r.texel = project<float, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, gh, gw);
        }
        proj[n * 32 + lane] = r;
      }
    }
    __syncwarp();

    float acc[LG][NG];
    unsigned argp[LG];   // winning view per group, a byte each (0xFF = -1)
#pragma unroll
    for (int j = 0; j < LG; ++j) {
      argp[j] = 0xFFFFFFFFu;
#pragma unroll
      for (int q = 0; q < NG; ++q) acc[j][q] = 1.175494351e-38f;   // v2:179-180: numeric_limits<T>::min()
    }

    for (int n = 0; n < N; ++n) {
      const ProjF<float>* r = myrec + n * 32;
      int cur = -1;
      float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) t00[k] = t01[k] = t10[k] = t11[k] = 0.0f;
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = r[j];
        if (rc.texel < 0) continue;            // the view does not see this plane
        if (rc.texel != cur) {
          cur = rc.texel;
          const T* p00 = src_lane + (size_t)rc.texel * C;
          const T* p10 = p00 + row;
          Vec<T, float, CPL>::load(p00, t00);
          Vec<T, float, CPL>::load(p00 + C, t01);
          Vec<T, float, CPL>::load(p10, t10);
          Vec<T, float, CPL>::load(p10 + C, t11);
        }
        float w00, w01, w11, w10;
        bilinear_weights(rc.dh, rc.dw, w00, w01, w11, w10);
        float val[CPL], gs[NG];
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
          const float sm = xadd(xadd(xadd(xmul(w00, t00[k]), xmul(w01, t01[k])), xmul(w11, t11[k])), xmul(w10, t10[k]));
          val[k] = xmul(sm, refv[k]);          // v2:213-216
        }
        in_lane_groups_t<float, CPL, SUB, true>(val, gs);
#pragma unroll
        for (int q = 0; q < NG; ++q) {
          if (acc[j][q] < gs[q]) {             // v2:221-224: the LARGEST group correlation wins, first view on ties
            acc[j][q] = gs[q];
            argp[j] = (argp[j] & ~(0xFFu << (8 * q))) | ((unsigned)n << (8 * q));
          }
        }
      }
    }

#pragma unroll
    for (int j = 0; j < LG; ++j) {
      if (pvalid && dblk + j < dhi) {
        store_stream<float, NG>(out + j * GR, acc[j]);
        int arg[NG];
#pragma unroll
        for (int q = 0; q < NG; ++q) arg[q] = (int)(signed char)((argp[j] >> (8 * q)) & 0xFFu);
        store_stream<int, NG>(outm + j * GR, arg);
      }
    }
    __syncwarp();
  }
}

// Gradient.  With bg = cost_grad[group]/views (v2:461) everything a plane contributes is linear in bg times
// a function of (dh, dw), so per (plane, view, group) only the bilinear moments
//   m0 += bg, m1 += bg*dw, m2 += bg*dh, m3 += bg*dh*dw
// are accumulated while the 2x2 footprint stays; on a flush they give, per channel,
//   d(ref)  += m0*p00 + m1*(p01-p00) + m2*(p10-p00) + m3*t1                    (v2:462)
//   d(src corners) += ref * (m0-m1-m2+m3, m1-m3, m2-m3, m3)                     (v2:463-467)
// The coordinate derivatives (v2:470-472) use per-group sums over channels of ref*t1, ref*(p10-p00),
// ref*(p01-p00), formed once per footprint.  The depth-hypothesis gradient is per voxel: every lane keeps
// one partial per plane of the block, the partials are reduce-scattered over the pixel's lanes (lane li
// ends up with plane li) and stored coalesced (zero where no view saw the voxel, v2:375-378).
// five 128-thread CTAs per SM measured fastest (four: 4-5 % slower at the c2 stages)
#ifndef CHOP_V2_BWD_MIN_BLOCKS
#define CHOP_V2_BWD_MIN_BLOCKS 5
#endif
// RMIN = true: `mask` holds the winning view per (voxel, group); only that view is differentiated, with
// no division by the view count (v2:483-601); a voxel whose first group has no winner is skipped.
template <typename T, int C, int SUB, bool RMIN = false>
__global__ void __launch_bounds__(128, CHOP_V2_BWD_MIN_BLOCKS) cv2_bwd_tuned(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CPL = 4;
  constexpr int LG = C / CPL;
  constexpr int G = 32 / LG;
  constexpr int NG = CPL / SUB;
  constexpr int GR = C / SUB;
  static_assert(LG * CPL == C && (LG & (LG - 1)) == 0 && LG <= 32 && NG * SUB == CPL, "unsupported C / SUB");
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
  ProjF<float>* recA = reinterpret_cast<ProjF<float>*>(coef + N * G);  // aux = 1/(valid views)
  RecG* recG = reinterpret_cast<RecG*>(recA + N * 32);

  stage_coefs<float>(a, coef, lane, G, pix0);
  __syncwarp();

  const T* src_lane = static_cast<const T*>(a.src) + li * CPL;
  float* sg_lane = static_cast<float*>(a.src_grad) + li * CPL;
  float refv[CPL], rg[CPL];
  Vec<T, float, CPL>::load(static_cast<const T*>(a.ref) + pix * C + li * CPL, refv);
#pragma unroll
  for (int k = 0; k < CPL; ++k) rg[k] = 0.0f;
  const float* dgrid = static_cast<const float*>(a.depth) + pix * D;
  float* dgrad = static_cast<float*>(a.depth_grad) + pix * D;
  const size_t row = (size_t)a.Ws * C;
  const float* cg_lane = static_cast<const float*>(a.cost_grad) + (pix * D + dlo) * GR + li * NG;
  const int* mk_lane = a.mask + (pix * D + dlo) * GR + li * NG;  // read for MIN only

  // The lane's depth hypothesis and validity count / winner of plane dblk+li stream in from HBM: they are requested
  // one block ahead, so phase A does not start with an exposed DRAM round trip.
  const int mk_stride = RMIN ? GR : 1;
  float depth_next = 0.0f;
  int m_next = 0;
  if (pvalid && dlo + li < dhi) {
    depth_next = __ldg(dgrid + dlo + li);
    m_next = __ldg(a.mask + (pix * D + dlo + li) * mk_stride);
  }
  for (int dblk = dlo; dblk < dhi; dblk += LG, cg_lane += LG * GR, mk_lane += LG * GR) {
    __syncwarp();
    // the block's upstream gradient (and winners): one request per plane, all in flight together and shared by the
    // views, instead of a dependent load per (plane, view); requested before phase A, whose projections cover the latency
    float cgall[LG][NG];
    int mkall[RMIN ? LG : 1][NG];
#pragma unroll
    for (int j = 0; j < LG; ++j) {
#pragma unroll
      for (int q = 0; q < NG; ++q) {
        cgall[j][q] = 0.0f;
        if (RMIN) mkall[j][q] = -1;
      }
      if (dblk + j < dhi) {
        Vec<float, float, NG>::load(cg_lane + j * GR, cgall[j]);
        if constexpr (RMIN) {
          float mk[NG];
          Vec<float, float, NG>::load(reinterpret_cast<const float*>(mk_lane) + j * GR, mk);
#pragma unroll
          for (int q = 0; q < NG; ++q) mkall[j][q] = __float_as_int(mk[q]);
        }
      }
    }
    // ---- phase A -----------------------------------------------------------------------------------------
    const int dA = dblk + li;
    const bool dvA = pvalid && dA < dhi;
    {
      float depth = 0.0f, scale = 0.0f;
      bool live = false;
      const int m0 = m_next;
      depth = depth_next;
      if (pvalid && dA + LG < dhi) {
        depth_next = __ldg(dgrid + dA + LG);
        m_next = __ldg(a.mask + (pix * D + dA + LG) * mk_stride);
      }
      if (dvA) {
        if constexpr (RMIN) {
          live = m0 >= 0;                      // v2:495
          scale = 1.0f;                        // v2:583
        } else {
          live = m0 > 0;                       // v2:375
          if (live) scale = 1.0f / (float)m0;  // v2:461
        }
      }
      for (int n = 0; n < N; ++n) {
        ProjF<float> r;
        RecG q;
        r.texel = -1;
        r.dh = r.dw = 0.0f;
        r.aux = scale;
        q.gh = q.gw = 0.0f;
        if (live) r.texel = project<float, true>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, q.gh, q.gw);
        recA[n * 32 + lane] = r;
        recG[n * 32 + lane] = q;
      }
    }
    __syncwarp();

    // ---- phase B -----------------------------------------------------------------------------------------
    float dv[LG];
#pragma unroll
    for (int j = 0; j < LG; ++j) dv[j] = 0.0f;
    for (int n = 0; n < N; ++n) {
      const ProjF<float>* rA = recA + n * 32 + g * LG;
      const RecG* rGp = recG + n * 32 + g * LG;
      int cur = -1;
      float a0[CPL], u[CPL], v[CPL], t1[CPL];   // p00 and the corner differences of the footprint
      float T1R[NG], UR[NG], VR[NG], m[4][NG];
#pragma unroll
      for (int k = 0; k < CPL; ++k) a0[k] = u[k] = v[k] = t1[k] = 0.0f;
#pragma unroll
      for (int q = 0; q < NG; ++q) T1R[q] = UR[q] = VR[q] = m[0][q] = m[1][q] = m[2][q] = m[3][q] = 0.0f;
      auto flush = [&]() {
        float c00[CPL], c01[CPL], c10[CPL], c11[CPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
          const int q = k / SUB;
          rg[k] = fmaf(m[3][q], t1[k], fmaf(m[2][q], u[k], fmaf(m[1][q], v[k], fmaf(m[0][q], a0[k], rg[k]))));
          const float w01 = m[1][q] - m[3][q], w10 = m[2][q] - m[3][q];
          c00[k] = ((m[0][q] - m[1][q]) - w10) * refv[k];
          c01[k] = w01 * refv[k];
          c10[k] = w10 * refv[k];
          c11[k] = m[3][q] * refv[k];
        }
        float* gp = sg_lane + (size_t)cur * C;
        red_add<float, CPL>(gp, c00);
        red_add<float, CPL>(gp + C, c01);
        red_add<float, CPL>(gp + row, c10);
        red_add<float, CPL>(gp + row + C, c11);
      };
#pragma unroll
      for (int j = 0; j < LG; ++j) {
        const ProjF<float> rc = rA[j];
        if (rc.texel >= 0) {
          if (rc.texel != cur) {
            if (cur >= 0) flush();
            cur = rc.texel;
            float t00[CPL], t01[CPL], t10[CPL], t11[CPL];
            const T* p00 = src_lane + (size_t)rc.texel * C;
            const T* p10 = p00 + row;
            Vec<T, float, CPL>::load(p00, t00);
            Vec<T, float, CPL>::load(p00 + C, t01);
            Vec<T, float, CPL>::load(p10, t10);
            Vec<T, float, CPL>::load(p10 + C, t11);
#pragma unroll
            for (int q = 0; q < NG; ++q) T1R[q] = UR[q] = VR[q] = m[0][q] = m[1][q] = m[2][q] = m[3][q] = 0.0f;
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              const int q = k / SUB;
              a0[k] = t00[k];
              u[k] = t10[k] - t00[k];
              v[k] = t01[k] - t00[k];
              t1[k] = (t11[k] - t01[k]) - u[k];
              T1R[q] = fmaf(t1[k], refv[k], T1R[q]);
              UR[q] = fmaf(u[k], refv[k], UR[q]);
              VR[q] = fmaf(v[k], refv[k], VR[q]);
            }
          }
          const RecG rq = rGp[j];
          float cgv[NG];
#pragma unroll
          for (int q = 0; q < NG; ++q) cgv[q] = cgall[j][q];
          if constexpr (RMIN) {  // v2:575 a group's gradient goes to its winning view only
#pragma unroll
            for (int q = 0; q < NG; ++q)
              if (mkall[j][q] != n) cgv[q] = 0.0f;
          }
          const float hw = rc.dh * rc.dw;
          float P = 0.0f, Q = 0.0f, R = 0.0f;
#pragma unroll
          for (int q = 0; q < NG; ++q) {
            const float bg = cgv[q] * rc.aux;                                // v2:461
            m[0][q] += bg;
            m[1][q] = fmaf(bg, rc.dw, m[1][q]);
            m[2][q] = fmaf(bg, rc.dh, m[2][q]);
            m[3][q] = fmaf(bg, hw, m[3][q]);
            P = fmaf(bg, T1R[q], P);
            Q = fmaf(bg, UR[q], Q);
            R = fmaf(bg, VR[q], R);
          }
          // d(sample)/dh summed = dw*P + Q, d(sample)/dw summed = dh*P + R           (v2:470-474)
          dv[j] = fmaf(rq.gh, fmaf(rc.dw, P, Q), fmaf(rq.gw, fmaf(rc.dh, P, R), dv[j]));
        }
      }
      if (cur >= 0) flush();
    }
    // reduce-scatter the per-plane partials over the pixel's LG lanes: lane li keeps plane li
#pragma unroll
    for (int s = LG / 2; s >= 1; s >>= 1) {
#pragma unroll
      for (int i = 0; i < s; ++i) {
        const bool hi = (li & s) != 0;
        const float keep = hi ? dv[i + s] : dv[i];
        const float send = hi ? dv[i] : dv[i + s];
        dv[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
      }
    }
    if (dvA) dgrad[dA] = dv[0];   // v2:477 (plain store; zero for a voxel no view saw)
  }

  if (pvalid) red_add<float, CPL>(static_cast<float*>(a.ref_grad) + pix * C + li * CPL, rg);
}

}  // namespace chop
