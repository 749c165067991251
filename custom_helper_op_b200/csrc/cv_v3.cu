// CostVolumeV3 / CostVolumeGradV3 (reference: custom_helper_op/cc/kernels/cost_volume_kernels_gpu_v3.cu.cc:
// forward MEAN :33-143, MIN :145-260; gradient MEAN :376-520, MIN :522-639).
//
// Per voxel and source view the cost is the largest dot product between any group of the bilinearly
// sampled source feature and any group of the reference feature (groups = contiguous blocks of
// sub = C/groups <= 8 channels).  MEAN averages the per-view maxima, MIN keeps the largest over the views
// together with (view, reference group, source group) of the winner.
//
// Decomposition: a warp owns 32/LG neighbouring pixels, LG = groups rounded up to a power of two lanes per
// pixel; lane gs holds source group gs.  Depth planes are walked in blocks of LG:
//   phase A - lane (pixel, j) projects plane j of its pixel into every view (shared-memory records);
//   phase B - for each plane all lanes of the pixel sample their own group once and take its dot product
//             with every reference group (reference pixel in shared memory, broadcast reads); the winner
//             over the pixel's lanes is found with xor-shuffles.
// The running maximum of the reference is sequential over (source group, reference group) with a strict
// "<": the winner is the largest value and, among equal values, the smallest source group, then the
// smallest reference group.  The shuffle reduction applies exactly that order, and sample and dot product
// are evaluated with unfused operations in the reference's order, so cost, mask and winner indices are
// bit-identical to the reference compiled without contraction.
#include "cv_project.cuh"
#include "cv_v3_entry.h"
#include "smem_grant.h"

namespace chop {
namespace {

constexpr int V3_MAX_SUB = 8;  // MAX_SUBCHANNELS_SIZE, cost_volume_v3.h:35

template <typename T, typename R>
__device__ __forceinline__ R ld1(const T* p) {
  R o[1];
  Vec<T, R, 1>::load(p, o);
  return o[0];
}


// Sample group gs at the four corners (unfused, the reference's operand order :114-115) and take the dot
// product with every reference group (:118-126).  Returns the lane's best value above `start`.
// SUBT = 4 or 8 (float arithmetic only): channels per group known at compile time - 16-byte loads of the
// corners and of the reference groups (shared memory), fully unrolled dot products.  SUBT = 0: any sub <= 8.
template <typename T, typename R, int SUBT>
__device__ __forceinline__ R lane_best(const T* t00, int C, size_t row, const R* refp, int groups, int sub, int gs,
                                       R dh, R dw, R start, int& best_gi, R* smp) {
  R w00, w01, w11, w10;
  bilinear_weights(dh, dw, w00, w01, w11, w10);
  R cur = start;
  best_gi = -1;
  if constexpr (SUBT > 0) {
    const T* p = t00 + gs * SUBT;
    R a[SUBT], b[SUBT], c[SUBT], d[SUBT];
#pragma unroll
    for (int q = 0; q < SUBT; q += 4) {
      Vec<T, R, 4>::load(p + q, a + q);
      Vec<T, R, 4>::load(p + C + q, b + q);
      Vec<T, R, 4>::load(p + row + C + q, c + q);
      Vec<T, R, 4>::load(p + row + q, d + q);
    }
#pragma unroll
    for (int k = 0; k < SUBT; ++k)
      smp[k] = xadd(xadd(xadd(xmul(w00, a[k]), xmul(w01, b[k])), xmul(w11, c[k])), xmul(w10, d[k]));
    for (int gi = 0; gi < groups; ++gi) {
      R rv[SUBT];
#pragma unroll
      for (int q = 0; q < SUBT; q += 4) {
        const float4 t = *reinterpret_cast<const float4*>(refp + gi * SUBT + q);
        rv[q] = t.x; rv[q + 1] = t.y; rv[q + 2] = t.z; rv[q + 3] = t.w;
      }
      R tmp = (R)0;
#pragma unroll
      for (int k = 0; k < SUBT; ++k) tmp = xadd(tmp, xmul(smp[k], rv[k]));
      if (cur < tmp) {
        cur = tmp;
        best_gi = gi;
      }
    }
  } else {
    const T* p = t00 + gs * sub;
#pragma unroll
    for (int k = 0; k < V3_MAX_SUB; ++k) {
      if (k < sub) {
        const R a = ld1<T, R>(p + k), b = ld1<T, R>(p + C + k), c = ld1<T, R>(p + row + C + k), d = ld1<T, R>(p + row + k);
        smp[k] = xadd(xadd(xadd(xmul(w00, a), xmul(w01, b)), xmul(w11, c)), xmul(w10, d));
      }
    }
    for (int gi = 0; gi < groups; ++gi) {
      R tmp = (R)0;
#pragma unroll
      for (int k = 0; k < V3_MAX_SUB; ++k)
        if (k < sub) tmp = xadd(tmp, xmul(smp[k], refp[gi * sub + k]));
      if (cur < tmp) {
        cur = tmp;
        best_gi = gi;
      }
    }
  }
  return cur;
}

// Winner over the LG lanes of a pixel: largest value; among equal values the lane that found a winner at
// all, then the smaller source group.
template <typename R>
__device__ __forceinline__ void group_best(R& cur, int& gi, int& gs, int LG) {
  for (int o = LG >> 1; o > 0; o >>= 1) {
    const R oc = __shfl_xor_sync(0xffffffffu, cur, o);
    const int ogi = __shfl_xor_sync(0xffffffffu, gi, o);
    const int ogs = __shfl_xor_sync(0xffffffffu, gs, o);
    const bool take = (ogi >= 0) && (gi < 0 || oc > cur || (oc == cur && ogs < gs));
    if (take) {
      cur = oc;
      gi = ogi;
      gs = ogs;
    }
  }
}

template <typename R>
struct alignas(16) RecB3 {
  int texel;   // -1: nothing to do for this (voxel, view)
  R dh, dw, gh, gw, cg;
  int gi, gs;  // MIN: the winner recorded by the forward pass
};

template <typename R>
size_t v3_smem_per_warp(int N, int G, int C, bool bwd) {
  size_t s = (size_t)N * G * sizeof(Coef<R>) + (size_t)G * C * sizeof(R);
  s += (size_t)N * 32 * (bwd ? sizeof(RecB3<R>) : sizeof(ProjF<R>));
  if (bwd) s += (size_t)G * C * sizeof(R);
  return (s + 15) & ~(size_t)15;
}

template <typename T, typename R, bool RMIN, int SUBT>
__global__ void __launch_bounds__(256) cv3_fwd_kernel(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int LG = 1 << a.lg_log2;
  const int G = 32 / LG;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1), g = lane >> a.lg_log2;
  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk, dhi = min(a.d_end, dlo + a.chunk);
  const int N = a.N, D = a.D, C = a.C, groups = a.G, sub = C / groups;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<R>* coef = reinterpret_cast<Coef<R>*>(mine);
  R* refs = reinterpret_cast<R*>(coef + N * G);                        // [G][C]
  ProjF<R>* rec = reinterpret_cast<ProjF<R>*>(refs + G * C);           // [N][32]

  stage_coefs<R>(a, coef, lane, G, pix0);
  for (int e = lane; e < G * C; e += 32) {
    long long p = pix0 + e / C;
    if (p >= a.npix) p = a.npix - 1;
    refs[e] = ld1<T, R>(static_cast<const T*>(a.ref) + p * C + (e % C));
  }
  __syncwarp();

  const int b = (int)(pix / ((long long)a.H * a.W));
  const R base = static_cast<const R*>(a.depth)[pix];
  const R* offs = static_cast<const R*>(a.offsets) + (long long)b * D;
  const T* src = static_cast<const T*>(a.src);
  const size_t row = (size_t)a.Ws * C;
  const R* refp = refs + g * C;
  const bool lane_on = li < groups;

  for (int dblk = dlo; dblk < dhi; dblk += LG) {
    __syncwarp();
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const R depth = dv ? xadd(base, offs[d]) : (R)0;
      for (int n = 0; n < N; ++n) {
        ProjF<R> r;
        r.texel = -1;
        r.dh = r.dw = r.aux = (R)0;
        R gh, gw;
        if (dv) r.texel = project<R, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, gh, gw);
        rec[n * 32 + lane] = r;
      }
    }
    __syncwarp();

    R out_cost = (R)0;
    int out_m0 = RMIN ? -1 : 0, out_m1 = -1, out_m2 = -1;
    for (int j = 0; j < LG; ++j) {
      R acc = RMIN ? Lim<R>::min_pos() : (R)0;   // :73 / :193
      int used = 0, wn = -1, wgi = -1, wgs = -1;
      for (int n = 0; n < N; ++n) {
        const ProjF<R> r = rec[n * 32 + g * LG + j];
        const bool valid = r.texel >= 0;
        const R start = RMIN ? acc : Lim<R>::min_pos();   // :110 per view / :193 over all views
        R cur = start;
        int gi = -1, gs = li;
        if (valid && lane_on) {
          R smp[V3_MAX_SUB];
          cur = lane_best<T, R, SUBT>(src + (size_t)r.texel * C, C, row, refp, groups, sub, li, r.dh, r.dw, start, gi, smp);
        }
        group_best<R>(cur, gi, gs, LG);
        if (valid) {
          if (RMIN) {
            if (gi >= 0) { acc = cur; wn = n; wgi = gi; wgs = gs; }   // :237-242
          } else {
            acc = xadd(acc, cur);                                     // :130
            used += 1;
          }
        }
      }
      if (li == j) {
        if (RMIN) {
          out_cost = wn >= 0 ? acc : (R)0;                           // :253-257
          out_m0 = wn; out_m1 = wgi; out_m2 = wgs;
        } else {
          out_cost = used > 0 ? xdiv(acc, (R)used) : (R)0;           // :136-141
          out_m0 = used;
        }
      }
    }
    const int d = dblk + li;
    if (pvalid && d < dhi) {
      const long long vox = pix * D + d;
      static_cast<R*>(a.cost)[vox] = out_cost;
      if (RMIN) {
        a.mask[vox * 3] = out_m0; a.mask[vox * 3 + 1] = out_m1; a.mask[vox * 3 + 2] = out_m2;
      } else {
        a.mask[vox] = out_m0;
      }
    }
  }
}

template <typename T, typename R, bool RMIN, int SUBT>
__global__ void __launch_bounds__(256) cv3_bwd_kernel(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int LG = 1 << a.lg_log2;
  const int G = 32 / LG;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1), g = lane >> a.lg_log2;
  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk, dhi = min(a.d_end, dlo + a.chunk);
  const int N = a.N, D = a.D, C = a.C, groups = a.G, sub = C / groups;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<R>* coef = reinterpret_cast<Coef<R>*>(mine);
  R* refs = reinterpret_cast<R*>(coef + N * G);                        // [G][C]
  R* rgacc = refs + G * C;                                             // [G][C] d(ref) of this work item
  RecB3<R>* rec = reinterpret_cast<RecB3<R>*>(rgacc + G * C);          // [N][32]

  stage_coefs<R>(a, coef, lane, G, pix0);
  for (int e = lane; e < G * C; e += 32) {
    long long p = pix0 + e / C;
    if (p >= a.npix) p = a.npix - 1;
    refs[e] = ld1<T, R>(static_cast<const T*>(a.ref) + p * C + (e % C));
    rgacc[e] = (R)0;
  }
  __syncwarp();

  const int b = (int)(pix / ((long long)a.H * a.W));
  const R base = static_cast<const R*>(a.depth)[pix];
  const R* offs = static_cast<const R*>(a.offsets) + (long long)b * D;
  const T* src = static_cast<const T*>(a.src);
  R* sgrad = static_cast<R*>(a.src_grad);
  const size_t row = (size_t)a.Ws * C;
  const R* refp = refs + g * C;
  R* rgp = rgacc + g * C;
  const bool lane_on = li < groups;
  R dsum = (R)0;

  // The lane's mask entry and upstream value of plane dblk+li stream in from HBM: both are requested together and
  // one block ahead (the upstream value whether or not the voxel turns out to be live), so phase A neither starts
  // with a DRAM round trip nor chains two of them.
  int nm0 = -1, nm1 = -1, nm2 = -1;
  R ncg = (R)0;
  auto request = [&](int d) {
    if (pvalid && d < dhi) {
      const long long vox = pix * D + d;
      if (RMIN) {
        nm0 = __ldg(a.mask + vox * 3); nm1 = __ldg(a.mask + vox * 3 + 1); nm2 = __ldg(a.mask + vox * 3 + 2);
      } else {
        nm0 = __ldg(a.mask + vox);
      }
      ncg = __ldg(static_cast<const R*>(a.cost_grad) + vox);
    }
  };
  request(dlo + li);
  for (int dblk = dlo; dblk < dhi; dblk += LG) {
    __syncwarp();
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      R depth = (R)0, cg = (R)0;
      int m0 = nm0, m1 = nm1, m2 = nm2;
      const R cg_raw = ncg;
      request(d + LG);
      bool live = false;
      if (dv) {
        depth = xadd(base, offs[d]);
        if (RMIN) {
          live = m0 >= 0 && m0 < N && m1 >= 0 && m1 < groups && m2 >= 0 && m2 < groups;   // :541
          if (live) cg = cg_raw;
        } else {
          live = m0 > 0;                                                                  // :393
          if (live) cg = cg_raw / (R)m0;                                                  // :426
        }
      } else {
        m0 = m1 = m2 = -1;
      }
      for (int n = 0; n < N; ++n) {
        RecB3<R> r;
        r.texel = -1;
        r.dh = r.dw = r.gh = r.gw = (R)0;
        r.cg = cg;
        r.gi = m1; r.gs = m2;
        if (live && (!RMIN || n == m0))
          r.texel = project<R, true>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, r.gh, r.gw);
        rec[n * 32 + lane] = r;
      }
    }
    __syncwarp();

    for (int j = 0; j < LG; ++j) {
      for (int n = 0; n < N; ++n) {
        const RecB3<R> r = rec[n * 32 + g * LG + j];
        const bool valid = r.texel >= 0;
        if (RMIN && !__any_sync(0xffffffffu, valid)) continue;
        int gi = -1, gs = li;
        R smp[V3_MAX_SUB];
        const T* t00 = src + (size_t)(valid ? r.texel : 0) * C;
        if (RMIN) {
          gi = r.gi; gs = r.gs;      // the winner the forward pass recorded (:548-549)
        } else {
          // recompute this view's winner exactly as the forward pass did (:470-489)
          R cur = Lim<R>::min_pos();
          if (valid && lane_on) cur = lane_best<T, R, SUBT>(t00, C, row, refp, groups, sub, li, r.dh, r.dw, cur, gi, smp);
          group_best<R>(cur, gi, gs, LG);
        }
        // the lane that holds the winning source group scatters the gradient of its `sub` channels; a view
        // without a winner (no dot product above the start value) contributes nothing
        if (valid && gi >= 0 && li == gs) {
          R w00, w01, w11, w10;
          bilinear_weights(r.dh, r.dw, w00, w01, w11, w10);
          R hg = (R)0, wg = (R)0;
          R* g00 = sgrad + (size_t)r.texel * C + gs * sub;
          const T* p = t00 + gs * sub;
          if constexpr (SUBT > 0) {
            // whole group at once: 16-byte corner loads, 16-byte vector reductions into src_grad
            R v00[SUBT], v01[SUBT], v11[SUBT], v10[SUBT], c00[SUBT], c01[SUBT], c11[SUBT], c10[SUBT];
#pragma unroll
            for (int q = 0; q < SUBT; q += 4) {
              Vec<T, R, 4>::load(p + q, v00 + q);
              Vec<T, R, 4>::load(p + C + q, v01 + q);
              Vec<T, R, 4>::load(p + row + C + q, v11 + q);
              Vec<T, R, 4>::load(p + row + q, v10 + q);
            }
#pragma unroll
            for (int k = 0; k < SUBT; ++k) {
              const R s = w00 * v00[k] + w01 * v01[k] + w11 * v11[k] + w10 * v10[k];
              const int rc = gi * SUBT + k;
              rgp[rc] += r.cg * s;                        // :490 (one lane per pixel is here at a time)
              const R bg = r.cg * refp[rc];               // :491
              c00[k] = bg * w00; c01[k] = bg * w01; c11[k] = bg * w11; c10[k] = bg * w10;   // :492-495
              const R t1 = v11[k] - v10[k] - v01[k] + v00[k];   // :498
              hg += bg * (t1 * r.dw + v10[k] - v00[k]);
              wg += bg * (t1 * r.dh + v01[k] - v00[k]);
            }
            red_add<R, SUBT>(g00, c00);
            red_add<R, SUBT>(g00 + C, c01);
            red_add<R, SUBT>(g00 + row + C, c11);
            red_add<R, SUBT>(g00 + row, c10);
          } else {
            for (int k = 0; k < sub; ++k) {
              const R v00 = ld1<T, R>(p + k), v01 = ld1<T, R>(p + C + k), v11 = ld1<T, R>(p + row + C + k),
                      v10 = ld1<T, R>(p + row + k);
              const R s = w00 * v00 + w01 * v01 + w11 * v11 + w10 * v10;
              const int rc = gi * sub + k;
              rgp[rc] += r.cg * s;                          // :490 (one lane per pixel is here at a time)
              const R bg = r.cg * refp[rc];                 // :491
              atomicAdd(g00 + k, bg * w00);                 // :492-495
              atomicAdd(g00 + C + k, bg * w01);
              atomicAdd(g00 + row + C + k, bg * w11);
              atomicAdd(g00 + row + k, bg * w10);
              const R t1 = v11 - v10 - v01 + v00;           // :498
              hg += bg * (t1 * r.dw + v10 - v00);
              wg += bg * (t1 * r.dh + v01 - v00);
            }
          }
          dsum += r.gh * hg + r.gw * wg;                  // :502
        }
        __syncwarp();   // orders this lane's d(ref) updates before another lane of the pixel touches them
      }
    }
  }
  __syncwarp();
  if (pvalid)
    for (int c = li; c < C; c += LG) {
      const R v = rgp[c];
      if (v != (R)0) atomicAdd(static_cast<R*>(a.ref_grad) + pix * C + c, v);
    }
  for (int o = LG >> 1; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
  if (pvalid && li == 0) atomicAdd(static_cast<R*>(a.depth_grad) + pix, dsum);   // :505
}

template <typename T, typename R, bool BWD, bool RMIN, int SUBT>
int launch_sub(const CvArgs& a, cudaStream_t st) {
  const int LG = 1 << a.lg_log2, G = 32 / LG;
  const size_t spw = v3_smem_per_warp<R>(a.N, G, a.C, BWD);
  int warps = 8;
  while (warps > 1 && spw * warps > 200 * 1024) warps >>= 1;
  if (spw * warps > 200 * 1024) return -4;  // CHOP_ERR_UNSUPPORTED
  const size_t smem = spw * warps;
  const long long items = (long long)a.npb * a.nchunks;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -2;     // CHOP_ERR_SHAPE
  auto k = BWD ? cv3_bwd_kernel<T, R, RMIN, SUBT> : cv3_fwd_kernel<T, R, RMIN, SUBT>;
  if (int e = grant_smem(k, smem)) return e;
  k<<<(unsigned)blocks, warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <typename T, typename R, bool BWD, bool RMIN>
int launch(const CvArgs& a, cudaStream_t st) {
  if constexpr (sizeof(R) == 4) {
    const int sub = a.C / a.G;
    if (sub == 4) return launch_sub<T, R, BWD, RMIN, 4>(a, st);
    if (sub == 8) return launch_sub<T, R, BWD, RMIN, 8>(a, st);
  }
  return launch_sub<T, R, BWD, RMIN, 0>(a, st);
}

template <bool BWD>
int dispatch(int dtype, bool rmin, const CvArgs& a, cudaStream_t st) {
  switch (dtype) {
    case 0: return rmin ? launch<float, float, BWD, true>(a, st) : launch<float, float, BWD, false>(a, st);
    case 1: return rmin ? launch<double, double, BWD, true>(a, st) : launch<double, double, BWD, false>(a, st);
    default: return rmin ? launch<__nv_bfloat16, float, BWD, true>(a, st) : launch<__nv_bfloat16, float, BWD, false>(a, st);
  }
}

}  // namespace

int cv3_fwd_launch(int dtype, bool rmin, const CvArgs& a, cudaStream_t st) { return dispatch<false>(dtype, rmin, a, st); }
int cv3_bwd_launch(int dtype, bool rmin, const CvArgs& a, cudaStream_t st) { return dispatch<true>(dtype, rmin, a, st); }

}  // namespace chop
