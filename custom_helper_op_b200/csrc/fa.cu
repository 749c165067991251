// FeatureAggregate / FeatureAggregateGrad (reference: custom_helper_op/cc/kernels/
// feature_aggregate_kernels_gpu.cu.cc:33-121, 219-317) and IndexInitializer (index_initializer_kernels_gpu.cu.cc:21-29).
//
// FeatureAggregate is the plane-sweep warp without a reduction: mapped_feature [B,H,W,D,N,C] receives the bilinear
// sample of every source view at every voxel (zeros where the view does not see it), mapped_mask [B,H,W,D,N,1]
// the validity.  It writes N times the bytes of a cost volume and is bound by that write stream; the gradient is
// bound by reading mapped_feature_grad once.
//
// Same decomposition as the cost-volume kernels (cv_project.cuh): a warp owns 32/LG pixels, LG lanes per pixel, CPL
// channels per lane, depth planes in blocks of LG; phase A projects (one lane per plane and pixel), phase B does
// the channel work with the 2x2 texel footprint cached in registers along the plane loop.  The sample is evaluated
// with unfused operations in the reference's order, so the forward output is bit-identical to the reference
// compiled without contraction.  The gradient keeps the corner sums of a footprint as bilinear moments and flushes
// them with vector reductions when the footprint changes.
#include <atomic>

#include "cv_project.cuh"
#include "fa_entry.h"
#include "smem_grant.h"

namespace chop {
std::atomic<int> g_fa_stage{1};   // tuning knob "fa_stage": 0 = the gradient reads its upstream tensor plane by plane
namespace {

template <typename R>
struct alignas(8) RecGF {
  R gh, gw;
};

// `stage_planes` > 0 (gradient only): two buffers for the upstream gradient of that many planes of ONE view, 16 bytes
// per lane and plane.
template <typename R>
size_t fa_smem_per_warp(int N, int G, bool bwd, int stage_planes = 0) {
  size_t bytes = (size_t)N * G * sizeof(Coef<R>) + (size_t)N * 32 * (sizeof(ProjF<R>) + (bwd ? sizeof(RecGF<R>) : 0));
  if (stage_planes > 0) bytes = ((bytes + 15) & ~(size_t)15) + (size_t)2 * stage_planes * 512;   // 16-byte aligned slices
  return bytes;
}

__device__ __forceinline__ void fa_cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}

template <typename T, typename R, int CPL>
__global__ void __launch_bounds__(256) fa_fwd_kernel(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int LG = 1 << a.lg_log2, G = 32 / LG;
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
  const int N = a.N, D = a.D, C = a.C;
  const bool lane_on = li * CPL < C;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<R>* coef = reinterpret_cast<Coef<R>*>(mine);
  ProjF<R>* rec = reinterpret_cast<ProjF<R>*>(coef + N * G);

  stage_coefs<R>(a, coef, lane, G, pix0);
  __syncwarp();

  const int b = (int)(pix / ((long long)a.H * a.W));
  const R base = static_cast<const R*>(a.depth)[pix];
  const R* offs = static_cast<const R*>(a.offsets) + (long long)b * D;
  const T* src_lane = static_cast<const T*>(a.src) + li * CPL;
  const size_t row = (size_t)a.Ws * C;
  R* mapped = static_cast<R*>(a.cost);

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
        if (dv) {
          r.texel = project<R, false>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, gh, gw);
          __stcs(a.mask + (pix * D + d) * N + n, r.texel >= 0 ? 1 : 0);   // :108 / :118
        }
        rec[n * 32 + lane] = r;
      }
    }
    __syncwarp();
    if (!lane_on || !pvalid) continue;

    for (int n = 0; n < N; ++n) {
      const ProjF<R>* r = rec + n * 32 + g * LG;
      int cur = -1;
      R t00[CPL], t01[CPL], t10[CPL], t11[CPL];
      const int jn = min(LG, dhi - dblk);
      for (int j = 0; j < jn; ++j) {
        const ProjF<R> rc = r[j];
        R s[CPL];
        if (rc.texel >= 0) {
          if (rc.texel != cur) {
            cur = rc.texel;
            const T* p00 = src_lane + (size_t)rc.texel * C;
            Vec<T, R, CPL>::load(p00, t00);
            Vec<T, R, CPL>::load(p00 + C, t01);
            Vec<T, R, CPL>::load(p00 + row, t10);
            Vec<T, R, CPL>::load(p00 + row + C, t11);
          }
          R w00, w01, w11, w10;
          bilinear_weights(rc.dh, rc.dw, w00, w01, w11, w10);
#pragma unroll
          for (int k = 0; k < CPL; ++k)   // :104-105, operand order of the reference
            s[k] = xadd(xadd(xadd(xmul(w00, t00[k]), xmul(w01, t01[k])), xmul(w11, t11[k])), xmul(w10, t10[k]));
        } else {
#pragma unroll
          for (int k = 0; k < CPL; ++k) s[k] = (R)0;   // :113-117
        }
        store_stream<R, CPL>(mapped + ((pix * D + dblk + j) * N + n) * C + li * CPL, s);
      }
    }
  }
}

// Moments of the upstream gradient over one footprint -> the four corner gradients.
template <typename R, int CPL>
__device__ __forceinline__ void fa_flush(R* gp, size_t row, int C, R (&m)[4][CPL]) {
  R c00[CPL], c01[CPL], c10[CPL];
#pragma unroll
  for (int k = 0; k < CPL; ++k) {
    c01[k] = m[1][k] - m[3][k];
    c10[k] = m[2][k] - m[3][k];
    c00[k] = (m[0][k] - m[1][k]) - c10[k];
  }
  red_add<R, CPL>(gp, c00);
  red_add<R, CPL>(gp + C, c01);
  red_add<R, CPL>(gp + row, c10);
  red_add<R, CPL>(gp + row + C, m[3]);
}

// STAGED (16-byte channel slices, every lane carries channels): the upstream gradient of one view over a whole block
// of planes is copied into one of two shared-memory buffers with cp.async while the previous (block, view) is
// processed - each lane copies exactly the 16-byte slices it will read itself, so no barrier is involved.  The tensor is
// read once and nothing else hides its latency: with one plane requested ahead per warp the kernel ran at what
// 24 warps x 512 bytes in flight give (2.1 TB/s at c1 shapes).
// LGC > 0 (STAGED only): the lanes per pixel - hence the channel count LGC*CPL and the planes per block - are
// compile-time constants; the plane loops unroll and the index arithmetic folds (a third of the generic kernel's
// instructions were integer address and loop work).  LGC = 0 keeps them run-time values.
template <typename T, typename R, int CPL, bool STAGED, int LGC = 0>
__global__ void __launch_bounds__(256) fa_bwd_kernel(const CvArgs a, const int warps, const size_t smem_per_warp) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int LG = LGC > 0 ? LGC : 1 << a.lg_log2, G = 32 / LG;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int li = lane & (LG - 1), g = LGC > 0 ? lane / LGC : lane >> a.lg_log2;
  const long long item = (long long)blockIdx.x * warps + wib;
  if (item >= (long long)a.npb * a.nchunks) return;
  const int chunk_id = (int)(item / a.npb);
  const int pb = (int)(item - (long long)chunk_id * a.npb);
  const long long pix0 = (long long)pb * G;
  const bool pvalid = pix0 + g < a.npix;
  const long long pix = pvalid ? pix0 + g : a.npix - 1;
  const int dlo = a.d_begin + chunk_id * a.chunk, dhi = min(a.d_end, dlo + a.chunk);
  const int N = a.N, D = a.D, C = LGC > 0 ? LGC * CPL : a.C;
  const bool lane_on = li * CPL < C;

  unsigned char* mine = smem_raw + (size_t)wib * smem_per_warp;
  Coef<R>* coef = reinterpret_cast<Coef<R>*>(mine);
  ProjF<R>* rec = reinterpret_cast<ProjF<R>*>(coef + N * G);
  RecGF<R>* recg = reinterpret_cast<RecGF<R>*>(rec + N * 32);
  // [buffer][plane of the block][lane] 16-byte slices (STAGED), behind the records at the next 16-byte boundary
  R* stage = reinterpret_cast<R*>(mine + (((size_t)(reinterpret_cast<unsigned char*>(recg + N * 32) - mine) + 15) & ~(size_t)15));

  stage_coefs<R>(a, coef, lane, G, pix0);
  __syncwarp();

  const int b = (int)(pix / ((long long)a.H * a.W));
  const R base = static_cast<const R*>(a.depth)[pix];
  const R* offs = static_cast<const R*>(a.offsets) + (long long)b * D;
  const T* src_lane = static_cast<const T*>(a.src) + li * CPL;
  R* sg_lane = static_cast<R*>(a.src_grad) + li * CPL;
  const R* mg = static_cast<const R*>(a.cost_grad);
  const size_t row = (size_t)a.Ws * C;
  R dsum = (R)0;

  // the lane's slices of view n over the block of planes that starts at d0, into buffer `buf`
  auto request = [&](int buf, int n, int d0) {
    if constexpr (STAGED) {
      if constexpr (LGC > 0) {
#pragma unroll
        for (int j = 0; j < LGC; ++j)
          if (d0 + j < dhi)
            fa_cp_async16(stage + ((size_t)(buf * LG + j) * 32 + lane) * CPL, mg + ((pix * D + d0 + j) * N + n) * C + li * CPL);
      } else
      for (int j = 0; j < LG && d0 + j < dhi; ++j)
        fa_cp_async16(stage + ((size_t)(buf * LG + j) * 32 + lane) * CPL, mg + ((pix * D + d0 + j) * N + n) * C + li * CPL);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  };
  int sbuf = 0;   // the buffer of the (block, view) processed next
  if (STAGED && pvalid) request(0, 0, dlo);
  for (int dblk = dlo; dblk < dhi; dblk += LG) {
    __syncwarp();
    {
      const int d = dblk + li;
      const bool dv = pvalid && d < dhi;
      const R depth = dv ? xadd(base, offs[d]) : (R)0;
      for (int n = 0; n < N; ++n) {
        ProjF<R> r;
        RecGF<R> q;
        r.texel = -1;
        r.dh = r.dw = r.aux = (R)0;
        q.gh = q.gw = (R)0;
        if (dv && __ldg(a.mask + (pix * D + d) * N + n) != 0)   // :262-264
          r.texel = project<R, true>(coef[n * G + g], depth, a.half_centor, a.Hs, a.Ws, r.dh, r.dw, q.gh, q.gw);
        rec[n * 32 + lane] = r;
        recg[n * 32 + lane] = q;
      }
    }
    __syncwarp();
    if (!lane_on || !pvalid) continue;

    for (int n = 0; n < N; ++n) {
      const ProjF<R>* r = rec + n * 32 + g * LG;
      const RecGF<R>* rq = recg + n * 32 + g * LG;
      int cur = -1;
      R t00[CPL], u[CPL], v[CPL], t1[CPL], m[4][CPL];
      const int jn = min(LG, dhi - dblk);
      // the upstream gradient of plane j+1 is requested before plane j is processed (each value is read once, so
      // nothing else hides its latency)
      const R* mgp = mg + ((pix * D + dblk) * N + n) * C + li * CPL;
      const size_t mstep = (size_t)N * C;
      R gnext[CPL];
      if constexpr (STAGED) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");   // this (block, view) has landed: own slices only
        // the other buffer was read a view ago: fill it with the next view of this block, or the next block's first
        if (n + 1 < N) request(sbuf ^ 1, n + 1, dblk);
        else if (dblk + LG < dhi) request(sbuf ^ 1, 0, dblk + LG);
      } else {
        load_stream<R, CPL>(mgp, gnext);
      }
#pragma unroll
      for (int j = 0; j < (LGC > 0 ? LGC : jn); ++j) {
        if (LGC > 0 && j >= jn) break;
        R gv[CPL];
        if constexpr (STAGED) {
          const uint4 w = *reinterpret_cast<const uint4*>(stage + ((size_t)(sbuf * LG + j) * 32 + lane) * CPL);
          *reinterpret_cast<uint4*>(gv) = w;
        } else {
#pragma unroll
          for (int k = 0; k < CPL; ++k) gv[k] = gnext[k];
          if (j + 1 < jn) load_stream<R, CPL>(mgp + (size_t)(j + 1) * mstep, gnext);
        }
        const ProjF<R> rc = r[j];
        if (rc.texel < 0) continue;
        if (rc.texel != cur) {
          if (cur >= 0) fa_flush<R, CPL>(sg_lane + (size_t)cur * C, row, C, m);
          cur = rc.texel;
          const T* p00 = src_lane + (size_t)rc.texel * C;
          R t01[CPL], t10[CPL], t11[CPL];
          Vec<T, R, CPL>::load(p00, t00);
          Vec<T, R, CPL>::load(p00 + C, t01);
          Vec<T, R, CPL>::load(p00 + row, t10);
          Vec<T, R, CPL>::load(p00 + row + C, t11);
#pragma unroll
          for (int k = 0; k < CPL; ++k) {
            u[k] = t10[k] - t00[k];
            v[k] = t01[k] - t00[k];
            t1[k] = (t11[k] - t01[k]) - u[k];   // :308
            m[0][k] = m[1][k] = m[2][k] = m[3][k] = (R)0;
          }
        }
        const R hw = rc.dh * rc.dw;
        R P = (R)0, Q = (R)0, S = (R)0;
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
          m[0][k] += gv[k];                       // corner sums :303-306 as moments
          m[1][k] = xfma(gv[k], rc.dw, m[1][k]);
          m[2][k] = xfma(gv[k], rc.dh, m[2][k]);
          m[3][k] = xfma(gv[k], hw, m[3][k]);
          P = xfma(gv[k], t1[k], P);              // :309-310: h_grad = dw*P + Q, w_grad = dh*P + S
          Q = xfma(gv[k], u[k], Q);
          S = xfma(gv[k], v[k], S);
        }
        const RecGF<R> q = rq[j];
        dsum = xfma(q.gh, xfma(rc.dw, P, Q), xfma(q.gw, xfma(rc.dh, P, S), dsum));   // :312
      }
      if (cur >= 0) fa_flush<R, CPL>(sg_lane + (size_t)cur * C, row, C, m);
      sbuf ^= 1;
    }
  }
  if constexpr (STAGED) asm volatile("cp.async.wait_group 0;" ::: "memory");
  for (int o = LG >> 1; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
  if (pvalid && li == 0) atomicAdd(static_cast<R*>(a.depth_grad) + pix, dsum);   // :315
}

template <typename T, typename R, int CPL, bool BWD>
int launch(const CvArgs& a, cudaStream_t st) {
  const int LG = 1 << a.lg_log2, G = 32 / LG;
  // the gradient stages the upstream tensor when a lane's slice is 16 bytes and every lane carries channels
  const bool staged = BWD && g_fa_stage.load() != 0 && CPL * sizeof(R) == 16 && LG * CPL == a.C;
  const size_t spw = fa_smem_per_warp<R>(a.N, G, BWD, staged ? LG : 0);
  int warps = 8;
  while (warps > 1 && spw * warps > (staged ? 56 : 200) * 1024) warps >>= 1;   // staged: four CTAs per SM
  if (spw * warps > 200 * 1024) return -4;  // CHOP_ERR_UNSUPPORTED
  const size_t smem = spw * warps;
  const long long items = (long long)a.npb * a.nchunks;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -2;     // CHOP_ERR_SHAPE
  void (*k)(const CvArgs, const int, const size_t);
  if constexpr (!BWD) {
    k = fa_fwd_kernel<T, R, CPL>;
  } else if constexpr (CPL * sizeof(R) == 16) {
    k = fa_bwd_kernel<T, R, CPL, false>;
    if (staged) {
      switch (LG) {   // 8 / 16 / 32 float channels (4 / 8 / 16 doubles): compile-time loops; 16 lanes and more ran faster without
        case 2: k = fa_bwd_kernel<T, R, CPL, true, 2>; break;
        case 4: k = fa_bwd_kernel<T, R, CPL, true, 4>; break;
        case 8: k = fa_bwd_kernel<T, R, CPL, true, 8>; break;
        default: k = fa_bwd_kernel<T, R, CPL, true>; break;
      }
    }
  } else {
    k = fa_bwd_kernel<T, R, CPL, false>;
  }
  if (int e = grant_smem(k, smem)) return e;
  k<<<(unsigned)blocks, warps * 32, smem, st>>>(a, warps, spw);
  return (int)cudaGetLastError();
}

template <bool BWD>
int dispatch(int dtype, int cpl, const CvArgs& a, cudaStream_t st) {
  if (dtype == 0) return cpl == 4 ? launch<float, float, 4, BWD>(a, st) : launch<float, float, 1, BWD>(a, st);
  if (dtype == 1) return cpl == 2 ? launch<double, double, 2, BWD>(a, st) : launch<double, double, 1, BWD>(a, st);
  return cpl == 4 ? launch<__nv_bfloat16, float, 4, BWD>(a, st) : launch<__nv_bfloat16, float, 1, BWD>(a, st);
}

// IndexInitializer: out [H,W,3] = (column, row, 1), the first two plus 0.5 when half_centor.
template <typename R>
__global__ void index_init_kernel(R* out, int n, int W, R half) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[(size_t)i * 3] = (R)(i % W) + half;
  out[(size_t)i * 3 + 1] = (R)(i / W) + half;
  out[(size_t)i * 3 + 2] = (R)1;
}

}  // namespace

int fa_fwd_launch(int dtype, int cpl, const CvArgs& a, cudaStream_t st) { return dispatch<false>(dtype, cpl, a, st); }
int fa_bwd_launch(int dtype, int cpl, const CvArgs& a, cudaStream_t st) { return dispatch<true>(dtype, cpl, a, st); }

int index_init_launch(int dtype, int half_centor, int H, int W, void* out, cudaStream_t st) {
  const int n = H * W;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == 1) index_init_kernel<double><<<grid, 256, 0, st>>>(static_cast<double*>(out), n, W, half_centor ? 0.5 : 0.0);
  else index_init_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(out), n, W, half_centor ? 0.5f : 0.0f);
  return (int)cudaGetLastError();
}

}  // namespace chop
