// Forward plane-sweep cost volume: homography projection, bilinear gather and view aggregation fused
// in one pass; no warped source volume is ever written.
//
// KIND 1  CostVolume     cost[vox,c]  = mean/min over views of (sample_c - ref_c)^2
//         (custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:33-228)
// KIND 2  CostVolumeV2   cost[vox,g]  = mean/"min" over views of sum_{c in g} sample_c*ref_c
//         (cost_volume_kernels_gpu_v2.cu.cc:33-235; its MIN keeps the largest value)
// KIND 3  CostAggregate  cost[vox]    = KIND 1 summed over channels / (views * C)
//         (cost_aggregate_kernels_gpu.cu.cc:34-227)
// MODE 0  MEAN, fused multiply-adds in the channel arithmetic (projection stays unfused, so the
//         validity count `mask` is exact)
// MODE 1  MEAN, every operation unfused and in reference order: cost reproducible bit for bit
// MODE 2  MIN, unfused (the arg-index output must be exact)
#pragma once
#include "cv_project.cuh"

namespace chop {

// How the lanes of a pixel combine per-channel values into per-group sums (KIND 2 and 3).
enum GroupMode {
  GROUP_IN_LANE = 0,  // every group lies inside one lane's channel slice (CPL % (C/G) == 0)
  GROUP_XOR = 1,      // a group spans a power-of-two run of lanes: butterfly shuffle
  GROUP_SMEM = 2,     // anything else, and the unfused grouped modes: sequential sum through shared memory
  GROUP_ROWS = 3      // unfused KIND 3: per-channel values of a block of depth planes are transposed
                      // through shared memory, then every lane sums ONE plane's channels in order
};

struct FwdCfg {
  int group_mode;
  int sub;       // channels per group (KIND 2), C for KIND 3
  int run;       // lanes per group for GROUP_XOR
  int warps;     // warps per block
  size_t smem_per_warp;
};

// Row stride (in values) of the GROUP_ROWS scratch: LG*CPL channel slots plus 16 bytes, so that the
// 16-byte reads of lanes that own consecutive rows fall into different banks.
template <typename R>
__host__ __device__ inline int rows_stride(int LG, int CPL) { return LG * CPL + 16 / (int)sizeof(R); }

template <typename R>
__host__ __device__ inline size_t fwd_smem_per_warp(int N, int G, int LG, int CPL, int group_mode) {
  size_t s = (size_t)N * G * sizeof(Coef<R>) + (size_t)N * 32 * sizeof(ProjF<R>);
  if (group_mode == GROUP_SMEM) s += (size_t)32 * CPL * sizeof(R);
  if (group_mode == GROUP_ROWS) s += (size_t)32 * rows_stride<R>(LG, CPL) * sizeof(R);
  return (s + 15) & ~(size_t)15;
}

// s + row[0] + row[1] + ... + row[n-1], added one by one in ascending order (unfused).  `vec` says
// that row is 16-byte aligned and n a multiple of the 16-byte vector length.
template <typename R>
__device__ __forceinline__ R row_sum_ordered(const R* row, int n, bool vec, R s) {
  if (vec) {
    if constexpr (sizeof(R) == 4) {
      for (int c = 0; c < n; c += 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + c);
        s = xadd(xadd(xadd(xadd(s, v.x), v.y), v.z), v.w);
      }
    } else {
      for (int c = 0; c < n; c += 2) {
        const double2 v = *reinterpret_cast<const double2*>(row + c);
        s = xadd(xadd(s, v.x), v.y);
      }
    }
  } else {
    for (int c = 0; c < n; ++c) s = xadd(s, row[c]);
  }
  return s;
}

// CPL consecutive values to shared memory, as 16-byte stores where the slice allows it.
template <typename R, int CPL>
__device__ __forceinline__ void store_slice(R* p, const R* v) {
  if constexpr (sizeof(R) == 4 && CPL % 4 == 0) {
#pragma unroll
    for (int i = 0; i < CPL; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else if constexpr (sizeof(R) == 8 && CPL % 2 == 0) {
#pragma unroll
    for (int i = 0; i < CPL; i += 2) *reinterpret_cast<double2*>(p + i) = make_double2(v[i], v[i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < CPL; ++i) p[i] = v[i];
  }
}


// out[q] = sum of the q-th run of SUB consecutive values of val, added in ascending order.
template <typename R, int CPL, int SUB, bool STRICT>
__device__ __forceinline__ void in_lane_groups_t(const R* val, R* out) {
#pragma unroll
  for (int q = 0; q < CPL / SUB; ++q) {
    // the reference starts every group sum from zero (0 + x also turns -0 into +0)
    R s = STRICT ? xadd((R)0, val[q * SUB]) : val[q * SUB];
#pragma unroll
    for (int k = 1; k < SUB; ++k) s = STRICT ? xadd(s, val[q * SUB + k]) : s + val[q * SUB + k];
    out[q] = s;
  }
}

template <typename R, int CPL, bool STRICT>
__device__ __forceinline__ void in_lane_groups(const R* val, int sub, R* out) {
  if (sub == 1) in_lane_groups_t<R, CPL, 1, STRICT>(val, out);
  if constexpr (CPL >= 2) { if (sub == 2) in_lane_groups_t<R, CPL, 2, STRICT>(val, out); }
  if constexpr (CPL >= 4) { if (sub == 4) in_lane_groups_t<R, CPL, 4, STRICT>(val, out); }
  if constexpr (CPL >= 8) { if (sub == 8) in_lane_groups_t<R, CPL, 8, STRICT>(val, out); }
}

// Per-channel values of one pixel (val, CPL per lane) -> per-group sums in the owning lanes' out[].
// Must be called by all 32 lanes.  STRICT sums channel by channel in ascending order, starting from
// `init` (zero, or the running total where the reference keeps one sum across views).
template <typename R, int CPL, bool STRICT>
__device__ __forceinline__ void group_sums(const R* val, const FwdCfg& cfg, R* scratch, int lane, int li,
                                           int gbase, int ngroups, R init, R* out) {
  if (cfg.group_mode == GROUP_IN_LANE) {
    in_lane_groups<R, CPL, STRICT>(val, cfg.sub, out);
  } else if (!STRICT && cfg.group_mode == GROUP_XOR) {
    R s = val[0];
#pragma unroll
    for (int k = 1; k < CPL; ++k) s += val[k];
    for (int o = cfg.run >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    out[0] = s;
  } else {
#pragma unroll
    for (int k = 0; k < CPL; ++k) scratch[lane * CPL + k] = val[k];
    __syncwarp();
    R s = (R)0;
    if (li < ngroups) {
      const R* row = scratch + gbase * CPL + li * cfg.sub;
      s = init;
      for (int k = 0; k < cfg.sub; ++k) s = STRICT ? xadd(s, row[k]) : s + row[k];
    }
    __syncwarp();
    out[0] = s;
  }
}

template <typename T, typename R, int CPL, int KIND, int MODE>
__global__ void __launch_bounds__(256) cv_fwd_kernel(const CvArgs a, const FwdCfg cfg) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr bool STRICT = MODE != 0;
  constexpr bool RMIN = MODE == 2;
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
  ProjF<R>* proj = reinterpret_cast<ProjF<R>*>(coef + a.N * G);
  R* scratch = reinterpret_cast<R*>(proj + a.N * 32);  // [32 lanes][CPL], GROUP_SMEM only

  stage_coefs<R>(a, coef, lane, G, pix0);
  __syncwarp();

  const int C = a.C;
  const bool lane_on = pvalid && (li * CPL < C);
  const T* src = static_cast<const T*>(a.src);
  R refv[CPL];
#pragma unroll
  for (int k = 0; k < CPL; ++k) refv[k] = (R)0;
  if (lane_on) Vec<T, R, CPL>::load(static_cast<const T*>(a.ref) + pix * C + li * CPL, refv);
  const int b = pvalid ? (int)(pix / ((long long)a.H * a.W)) : 0;
  R base = (R)0;
  if (KIND != 2 && pvalid) base = static_cast<const R*>(a.depth)[pix];

  const int CO = KIND == 1 ? C : (KIND == 2 ? a.G : 1);  // cost channels per voxel
  R* cost = static_cast<R*>(a.cost);
  const int Ws = a.Ws;

  // grouped kinds: which output slots (groups) this lane writes
  const int ngroups = KIND == 2 ? a.G : 1;
  int nslots = 0, first = 0;
  if (KIND != 1) {
    if (cfg.group_mode == GROUP_IN_LANE) { nslots = CPL / cfg.sub; first = li * nslots; }
    else if (MODE == 0 && cfg.group_mode == GROUP_XOR) { nslots = (li & (cfg.run - 1)) == 0; first = li / cfg.run; }
    else { nslots = li < ngroups; first = li; }
    if (!pvalid || first >= CO) nslots = 0;
  }

  for (int dblk = dlo; dblk < dhi; dblk += LG) {
    // ---- phase A: one projection per lane and view -------------------------------------------
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      R depth = (R)0;
      if (dv) {
        if (KIND == 2) depth = static_cast<const R*>(a.depth)[pix * a.D + d];
        else depth = xadd(base, static_cast<const R*>(a.offsets)[(long long)b * a.D + d]);
      }
      int used = 0;
      for (int n = 0; n < a.N; ++n) {
        ProjF<R> pr;
        pr.texel = -1;
        pr.dh = pr.dw = pr.aux = (R)0;
        if (dv) {
          R gh, gw;
          pr.texel = project<R, false>(coef[n * G + g], depth, a.half_centor, a.Hs, Ws, pr.dh, pr.dw, gh, gw);
          used += pr.texel >= 0;
        }
        proj[n * 32 + lane] = pr;
      }
      if (!RMIN && dv) __stcs(a.mask + pix * a.D + d, used);
      if (KIND == 1 && MODE == 0) proj[lane].aux = used > 0 ? (R)1 / (R)used : (R)0;
    }
    __syncwarp();

    if constexpr (KIND == 1 && MODE == 0) {
      // ---- phase B, tuned path: per-channel mean of squared differences, fused arithmetic ---------
      const int jn = min(LG, dhi - dblk);
      const T* src_lane = src + li * CPL;
      const size_t row = (size_t)Ws * C;
      if (lane_on) {
        R* out = cost + (pix * a.D + dblk) * C + li * CPL;
        for (int j = 0; j < jn; ++j, out += C) {
          R acc[CPL];
#pragma unroll
          for (int k = 0; k < CPL; ++k) acc[k] = (R)0;
          const ProjF<R>* rec = proj + (g << lgl) + j;
          const R inv = rec->aux;
          for (int n = 0; n < a.N; ++n) {
            const ProjF<R> pr = rec[n * 32];
            if (pr.texel < 0) continue;
            R w00, w01, w11, w10;
            bilinear_weights_fast(pr.dh, pr.dw, w00, w01, w11, w10);
            const T* p00 = src_lane + (size_t)pr.texel * C;
            R t00[CPL], t01[CPL], t10[CPL], t11[CPL];
            Vec<T, R, CPL>::load(p00, t00);
            Vec<T, R, CPL>::load(p00 + C, t01);
            Vec<T, R, CPL>::load(p00 + row, t10);
            Vec<T, R, CPL>::load(p00 + row + C, t11);
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              const R s = xfma(w10, t10[k], xfma(w11, t11[k], xfma(w01, t01[k], w00 * t00[k])));
              const R df = s - refv[k];
              acc[k] = xfma(df, df, acc[k]);
            }
          }
#pragma unroll
          for (int k = 0; k < CPL; ++k) acc[k] *= inv;
          store_stream<R, CPL>(out, acc);
        }
      }
      __syncwarp();
      continue;
    }

    if constexpr (KIND == 3 && MODE != 0) {
      // ---- phase B, unfused aggregate: the reference adds the C squared differences of a (voxel,
      // view) one by one (cost_aggregate_kernels_gpu.cu.cc:100-126, 190-223).  All lanes compute
      // their channel slice for every plane of the block (coalesced gathers), the slices meet in
      // shared memory, and lane li then owns plane dblk+li and runs that chain in order.
      if (cfg.group_mode == GROUP_ROWS) {
        const int jn = min(LG, dhi - dblk);
        const int RS = rows_stride<R>(LG, CPL);
        R* rows = scratch + (size_t)(g << lgl) * RS;
        const bool vec = ((RS * (int)sizeof(R)) & 15) == 0 && (C % (16 / (int)sizeof(R))) == 0;
        const ProjF<R>* rec = proj + (g << lgl);
        R tot = RMIN ? Lim<R>::max() : (R)0;
        int targ = -1, tused = 0;
        for (int n = 0; n < a.N; ++n) {
          for (int j = 0; j < jn; ++j) {
            const ProjF<R> pr = rec[n * 32 + j];
            R val[CPL];
#pragma unroll
            for (int k = 0; k < CPL; ++k) val[k] = (R)0;
            if (pr.texel >= 0 && lane_on) {
              R w00, w01, w11, w10;
              bilinear_weights(pr.dh, pr.dw, w00, w01, w11, w10);
              const T* p00 = src + (size_t)pr.texel * C + li * CPL;
              R t00[CPL], t01[CPL], t10[CPL], t11[CPL];
              Vec<T, R, CPL>::load(p00, t00);
              Vec<T, R, CPL>::load(p00 + C, t01);
              Vec<T, R, CPL>::load(p00 + (size_t)Ws * C, t10);
              Vec<T, R, CPL>::load(p00 + (size_t)Ws * C + C, t11);
#pragma unroll
              for (int k = 0; k < CPL; ++k) {
                const R s = xadd(xadd(xadd(xmul(w00, t00[k]), xmul(w01, t01[k])), xmul(w11, t11[k])), xmul(w10, t10[k]));
                const R df = xsub(s, refv[k]);
                val[k] = xmul(df, df);
              }
            }
            store_slice<R, CPL>(rows + j * RS + li * CPL, val);
          }
          __syncwarp();
          if (li < jn && rec[n * 32 + li].texel >= 0) {
            const R s = row_sum_ordered<R>(rows + li * RS, C, vec, MODE == 1 ? tot : (R)0);
            if (MODE == 1) { tot = s; ++tused; }
            else if (tot > s) { tot = s; targ = n; }
          }
          __syncwarp();
        }
        if (pvalid && li < jn) {
          const long long vox = pix * a.D + dblk + li;
          R v;
          if (MODE == 2) v = targ >= 0 ? xdiv(tot, (R)C) : (R)0;
          else v = tused > 0 ? xdiv(tot, (R)(tused * C)) : (R)0;
          __stcs(cost + vox, v);
          if (RMIN) __stcs(a.mask + vox, targ);
        }
        continue;
      }
    }

    // ---- phase B: channel work, one depth plane at a time -----------------------------------------
    const int jn = min(LG, dhi - dblk);
    for (int j = 0; j < jn; ++j) {
      const long long vox = pix * a.D + dblk + j;
      R acc[CPL];
      int arg[CPL];
#pragma unroll
      for (int k = 0; k < CPL; ++k) {
        acc[k] = RMIN ? (KIND == 2 ? Lim<R>::min_pos() : Lim<R>::max()) : (R)0;
        arg[k] = -1;
      }
      int used = 0;
      for (int n = 0; n < a.N; ++n) {
        const ProjF<R> pr = proj[n * 32 + (g << lgl) + j];
        const bool valid = pr.texel >= 0;
        if (KIND == 1 && !valid) continue;
        used += valid;
        R val[CPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k) val[k] = (R)0;
        if (valid && lane_on) {
          R w00, w01, w11, w10;
          bilinear_weights(pr.dh, pr.dw, w00, w01, w11, w10);
          const T* p00 = src + (size_t)pr.texel * C + li * CPL;
          R t00[CPL], t01[CPL], t10[CPL], t11[CPL];
          Vec<T, R, CPL>::load(p00, t00);
          Vec<T, R, CPL>::load(p00 + C, t01);
          Vec<T, R, CPL>::load(p00 + (size_t)Ws * C, t10);
          Vec<T, R, CPL>::load(p00 + (size_t)Ws * C + C, t11);
#pragma unroll
          for (int k = 0; k < CPL; ++k) {
            R s;
            if (STRICT) {
              s = xadd(xadd(xadd(xmul(w00, t00[k]), xmul(w01, t01[k])), xmul(w11, t11[k])), xmul(w10, t10[k]));
            } else {
              s = xfma(w10, t10[k], xfma(w11, t11[k], xfma(w01, t01[k], w00 * t00[k])));
            }
            if (KIND == 2) {
              val[k] = STRICT ? xmul(s, refv[k]) : s * refv[k];
            } else {
              const R df = STRICT ? xsub(s, refv[k]) : s - refv[k];
              if (KIND == 1) {
                if (MODE == 0) acc[k] = xfma(df, df, acc[k]);
                else if (MODE == 1) acc[k] = xadd(acc[k], xmul(df, df));
                else {
                  const R sq = xmul(df, df);
                  if (acc[k] > sq) { acc[k] = sq; arg[k] = n; }
                }
              } else {
                val[k] = STRICT ? xmul(df, df) : df * df;
              }
            }
          }
        }
        if (KIND != 1) {
          if (MODE == 0) {
            // fast MEAN: keep per-channel partial sums over the views, reduce once per voxel below
#pragma unroll
            for (int k = 0; k < CPL; ++k) acc[k] += val[k];
          } else {
            // unfused: this view's group values, then the reference's update rule per group
            // (the aggregate MEAN kernel keeps ONE running sum over channels and views,
            // cost_aggregate_kernels_gpu.cu.cc:114, so its chain starts from the total so far)
            R gv[CPL];
            const bool chain = KIND == 3 && MODE == 1;
            group_sums<R, CPL, true>(val, cfg, scratch, lane, li, g << lgl, ngroups, chain ? acc[0] : (R)0, gv);
            if (valid) {
#pragma unroll
              for (int q = 0; q < CPL; ++q) {
                if (q < nslots) {
                  if (chain) acc[q] = gv[q];
                  else if (MODE == 1) acc[q] = xadd(acc[q], gv[q]);
                  else if (KIND == 2) { if (acc[q] < gv[q]) { acc[q] = gv[q]; arg[q] = n; } }
                  else { if (acc[q] > gv[q]) { acc[q] = gv[q]; arg[q] = n; } }
                }
              }
            }
          }
        }
      }

      // ---- finalise and store ------------------------------------------------------------
      if (KIND == 1) {
        if (!lane_on) continue;
        if (MODE == 0) {
          if (used > 0) {
            const R inv = (R)1 / (R)used;
#pragma unroll
            for (int k = 0; k < CPL; ++k) acc[k] *= inv;
          }
        } else if (MODE == 1) {
          if (used > 0) {
#pragma unroll
            for (int k = 0; k < CPL; ++k) acc[k] = xdiv(acc[k], (R)used);
          }
        }
        store_stream<R, CPL>(cost + vox * C + li * CPL, acc);
        if (RMIN) store_stream<int, CPL>(a.mask + vox * C + li * CPL, arg);
      } else {
        if (MODE == 0) {
          R gv[CPL];
          group_sums<R, CPL, false>(acc, cfg, scratch, lane, li, g << lgl, ngroups, (R)0, gv);
#pragma unroll
          for (int k = 0; k < CPL; ++k) acc[k] = gv[k];
        }
#pragma unroll
        for (int q = 0; q < CPL; ++q) {
          if (q < nslots) {
            R v = acc[q];
            if (KIND == 2) {
              if (MODE == 0) { if (used > 0) v *= (R)1 / (R)used; }
              else if (MODE == 1) { if (used > 0) v = xdiv(v, (R)used); }
            } else {  // KIND 3: cost_aggregate_kernels_gpu.cu.cc:121-126,218-223
              if (MODE == 2) v = arg[q] >= 0 ? xdiv(v, (R)C) : (R)0;
              else if (MODE == 1) v = used > 0 ? xdiv(v, (R)(used * C)) : (R)0;
              else v = used > 0 ? v / (R)(used * C) : (R)0;
            }
            __stcs(cost + vox * CO + first + q, v);
            if (RMIN) __stcs(a.mask + vox * CO + first + q, arg[q]);
          }
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace chop
