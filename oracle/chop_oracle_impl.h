/* TEST INFRASTRUCTURE ONLY - included by chop_oracle.c once per floating type.
 *
 * CPU restatement of the reference's plane-sweep cost-volume arithmetic.  REAL is float or double,
 * FN(x) appends the type suffix.  Every floating operation below is written as its own statement
 * or parenthesised so that, compiled with -ffp-contract=off, it is the same sequence of correctly
 * rounded IEEE operations as the reference source (file:line cited at each step; paths are
 * relative to custom_helper_op/cc/kernels/ of the reference).
 */

typedef struct {
  int valid;
  int64_t fh, fw;          /* top-left texel of the bilinear footprint */
  REAL dh, dw;             /* fractional offsets inside the footprint */
  REAL zc, wc, hc;         /* R rows applied to (x, y, 1) */
  REAL z, w3d, h3d;        /* projected homogeneous coordinates */
} FN(proj);

/* cost_volume_kernels_gpu.cu.cc:80-104 (identical in the v2 and aggregate files). */
static void FN(project)(REAL x, REAL y, REAL depth, const REAL *R, const REAL *t, int half_centor,
                        int64_t Hs, int64_t Ws, FN(proj) * p) {
  p->valid = 0;
  p->zc = R[6] * x + R[7] * y + R[8];
  p->z = p->zc * depth + t[2];
  if (p->z <= (REAL)0) return;
  p->wc = R[0] * x + R[1] * y + R[2];
  p->w3d = p->wc * depth + t[0];
  REAL sw = p->w3d / p->z;
  p->hc = R[3] * x + R[4] * y + R[5];
  p->h3d = p->hc * depth + t[1];
  REAL sh = p->h3d / p->z;
  if (half_centor) {
    sw = sw - (REAL)0.5;
    sh = sh - (REAL)0.5;
  }
  if (sh > (REAL)0 && sw > (REAL)0 && sh < (REAL)(Hs - 1) && sw < (REAL)(Ws - 1)) {
    p->fh = (int64_t)sh;
    p->fw = (int64_t)sw;
    p->dh = sh - (REAL)p->fh;
    p->dw = sw - (REAL)p->fw;
    p->valid = 1;
  }
}

/* Bilinear weights in the reference's naming (cost_volume_kernels_gpu.cu.cc:105-108):
 * w[0] multiplies texel (fh,fw), w[1] (fh,fw+1), w[2] (fh+1,fw+1), w[3] (fh+1,fw). */
static void FN(weights)(REAL dh, REAL dw, REAL w[4]) {
  w[2] = dh * dw;
  w[3] = dh * ((REAL)1 - dw);
  w[0] = ((REAL)1 - dh) * ((REAL)1 - dw);
  w[1] = ((REAL)1 - dh) * dw;
}

/* kind 1 = CostVolume  (cost [B,H,W,D,C];  depth = base_plane[b,h,w] + offsets[b,d])
 * kind 2 = CostVolumeV2 (cost [B,H,W,D,G]; depth = depth_grid[b,h,w,d]; per-group dot product)
 * kind 3 = CostAggregate (cost [B,H,W,D];  kind 1 summed over channels, divided by used*C)
 * reduce_min 0 = MEAN, 1 = MIN (for kind 2 "MIN" keeps the largest correlation, as the
 * reference does: cost_volume_kernels_gpu_v2.cu.cc:179,227-230). */
static void FN(cost_fwd)(int kind, int reduce_min, int half_centor, const int64_t *dims, int groups,
                         const REAL *ref, const REAL *src, const REAL *depth_in,
                         const REAL *offsets, const REAL *Rs, const REAL *Ts, REAL *cost,
                         int32_t *mask, int nthreads) {
  const int64_t B = dims[0], H = dims[1], W = dims[2], C = dims[3], D = dims[4], N = dims[5],
                Hs = dims[6], Ws = dims[7];
  const int64_t CO = kind == 1 ? C : (kind == 2 ? groups : 1);   /* cost channels per voxel */
  const int64_t MC = reduce_min ? CO : 1;                        /* mask channels per voxel */
  const int64_t sub = kind == 2 ? C / groups : 1;
  const int64_t npix = B * H * W;
#pragma omp parallel for schedule(dynamic, 16) num_threads(nthreads > 0 ? nthreads : 1)
  for (int64_t pix = 0; pix < npix; ++pix) {
    const int64_t b = pix / (H * W), h = (pix / W) % H, w = pix % W;
    REAL x = (REAL)w, y = (REAL)h;
    if (half_centor) { x = x + (REAL)0.5; y = y + (REAL)0.5; }
    const REAL *rc = ref + pix * C;
    for (int64_t d = 0; d < D; ++d) {
      const int64_t vox = pix * D + d;
      const REAL depth = kind == 2 ? depth_in[vox] : depth_in[pix] + offsets[b * D + d];
      REAL *co = cost + vox * CO;
      int32_t *mo = mask + vox * MC;
      if (reduce_min) {
        /* :174-177 (v1: numeric max), v2:177-180 (smallest positive normal) */
        for (int64_t k = 0; k < CO; ++k) { co[k] = kind == 2 ? REAL_MIN_POS : REAL_MAX; mo[k] = -1; }
      } else {
        for (int64_t k = 0; k < CO; ++k) co[k] = (REAL)0;
      }
      int32_t used = 0;
      for (int64_t n = 0; n < N; ++n) {
        FN(proj) p;
        FN(project)(x, y, depth, Rs + (b * N + n) * 9, Ts + (b * N + n) * 3, half_centor, Hs, Ws, &p);
        if (!p.valid) continue;
        REAL wt[4];
        FN(weights)(p.dh, p.dw, wt);
        const REAL *t00 = src + C * (p.fw + Ws * (p.fh + Hs * (n + N * b)));
        const REAL *t01 = t00 + C, *t10 = t00 + Ws * C, *t11 = t10 + C;
        if (kind == 2) {
          for (int64_t g = 0; g < groups; ++g) {
            REAL acc = (REAL)0;
            for (int64_t c = g * sub; c < (g + 1) * sub; ++c) {
              REAL s = wt[0] * t00[c] + wt[1] * t01[c] + wt[2] * t11[c] + wt[3] * t10[c];
              acc += s * rc[c];
            }
            if (reduce_min) { if (co[g] < acc) { co[g] = acc; mo[g] = (int32_t)n; } }
            else co[g] += acc;
          }
        } else {
          REAL total = (REAL)0;   /* kind 3 MIN: this view's channel sum */
          for (int64_t c = 0; c < C; ++c) {
            REAL s = wt[0] * t00[c] + wt[1] * t01[c] + wt[2] * t11[c] + wt[3] * t10[c];
            REAL df = s - rc[c];
            REAL sq = df * df;
            if (kind == 3) { if (reduce_min) total += sq; else co[0] += sq; }
            else if (reduce_min) { if (co[c] > sq) { co[c] = sq; mo[c] = (int32_t)n; } }
            else co[c] += sq;
          }
          if (kind == 3) {
            /* cost_aggregate_kernels_gpu.cu.cc:114 MEAN keeps one running sum over channels and
             * views; :207-215 MIN keeps the smallest per-view channel sum */
            if (reduce_min) { if (co[0] > total) { co[0] = total; mo[0] = (int32_t)n; } }
          }
        }
        used += 1;
      }
      if (!reduce_min) {
        mo[0] = used;
        if (kind == 3) {
          co[0] = used > 0 ? co[0] / (REAL)(used * (int32_t)C) : (REAL)0;
        } else if (used > 0) {
          for (int64_t k = 0; k < CO; ++k) co[k] = co[k] / (REAL)used;
        }
      } else if (kind == 3) {
        /* the aggregate MIN kernel divides the winning view's sum by C */
        co[0] = mo[0] >= 0 ? co[0] / (REAL)C : (REAL)0;
      }
    }
  }
}

/* Gradient (cost_volume_kernels_gpu.cu.cc:342-577, v2:349-601).  Outputs are zero-filled here as
 * the reference launcher does (:637-642).  Sums are accumulated voxel by voxel in ascending
 * linear index with views and channels innermost - the order a single reference thread uses -
 * so that with nthreads <= 1 the result is reproducible bit for bit. */
#ifndef SCATTER_ADD
#define SCATTER_ADD(p, v)                 \
  do {                                    \
    if (par) {                            \
      _Pragma("omp atomic") *(p) += (v);  \
    } else {                              \
      *(p) += (v);                        \
    }                                     \
  } while (0)
#endif

static void FN(cost_bwd)(int kind, int reduce_min, int half_centor, const int64_t *dims, int groups,
                         const REAL *ref, const REAL *src, const REAL *depth_in,
                         const REAL *offsets, const REAL *Rs, const REAL *Ts, const REAL *cost_grad,
                         const int32_t *mask, REAL *ref_grad, REAL *src_grad, REAL *depth_grad,
                         int nthreads) {
  const int64_t B = dims[0], H = dims[1], W = dims[2], C = dims[3], D = dims[4], N = dims[5],
                Hs = dims[6], Ws = dims[7];
  const int64_t CO = kind == 1 ? C : (kind == 2 ? groups : 1);
  const int64_t MC = reduce_min ? CO : 1;
  const int64_t sub = kind == 2 ? C / groups : 1;
  const int64_t npix = B * H * W;
  memset(ref_grad, 0, sizeof(REAL) * (size_t)(npix * C));
  memset(src_grad, 0, sizeof(REAL) * (size_t)(B * N * Hs * Ws * C));
  if (kind != 2) memset(depth_grad, 0, sizeof(REAL) * (size_t)npix);
  /* nthreads > 1: pixels are spread over threads and the source-gradient scatter becomes an atomic
   * update (what the reference does on the GPU); the sums then depend on the thread schedule. */
  const int par = nthreads > 1;
#pragma omp parallel for schedule(dynamic, 16) num_threads(par ? nthreads : 1) if (par)
  for (int64_t pix = 0; pix < npix; ++pix) {
    const int64_t b = pix / (H * W), h = (pix / W) % H, w = pix % W;
    REAL x = (REAL)w, y = (REAL)h;
    if (half_centor) { x = x + (REAL)0.5; y = y + (REAL)0.5; }
    const REAL *rc = ref + pix * C;
    REAL *rg = ref_grad + pix * C;
    for (int64_t d = 0; d < D; ++d) {
      const int64_t vox = pix * D + d;
      const int32_t *mo = mask + vox * MC;
      if (reduce_min ? (mo[0] < 0) : (mo[0] <= 0)) {
        if (kind == 2) depth_grad[vox] = (REAL)0;
        continue;
      }
      const REAL depth = kind == 2 ? depth_in[vox] : depth_in[pix] + offsets[b * D + d];
      const REAL *cg = cost_grad + vox * CO;
      REAL dsum = (REAL)0;
      for (int64_t n = 0; n < N; ++n) {
        FN(proj) p;
        FN(project)(x, y, depth, Rs + (b * N + n) * 9, Ts + (b * N + n) * 3, half_centor, Hs, Ws, &p);
        if (!p.valid) continue;
        REAL wt[4];
        FN(weights)(p.dh, p.dw, wt);
        const int64_t off = C * (p.fw + Ws * (p.fh + Hs * (n + N * b)));
        const REAL *t00 = src + off, *t01 = t00 + C, *t10 = t00 + Ws * C, *t11 = t10 + C;
        REAL *g00 = src_grad + off, *g01 = g00 + C, *g10 = g00 + Ws * C, *g11 = g10 + C;
        REAL hg = (REAL)0, wg = (REAL)0;
        REAL agg_scale = (REAL)0;
        if (kind == 3)
          agg_scale = reduce_min ? cg[0] / (REAL)(int32_t)C
                                 : cg[0] / (REAL)(mo[0] * (int32_t)C);
        for (int64_t c = 0; c < C; ++c) {
          const int64_t k = kind == 1 ? c : (kind == 2 ? c / sub : 0);
          if (reduce_min && mo[k] != (int32_t)n) continue;
          REAL s = wt[0] * t00[c] + wt[1] * t01[c] + wt[2] * t11[c] + wt[3] * t10[c];
          REAL gsrc;   /* d(loss)/d(sample) */
          if (kind == 2) {
            REAL bg = reduce_min ? cg[k] : cg[k] / (REAL)mo[0];
            rg[c] += bg * s;                                 /* v2:462 */
            gsrc = bg * rc[c];
          } else {
            REAL df = s - rc[c];
            if (kind == 3) gsrc = (REAL)2 * df * agg_scale;
            else gsrc = reduce_min ? (REAL)2 * df * cg[k] : (REAL)2 * df * cg[k] / (REAL)mo[0];
            rg[c] += -gsrc;                                  /* :440 */
          }
          SCATTER_ADD(&g00[c], gsrc * wt[0]);
          SCATTER_ADD(&g01[c], gsrc * wt[1]);
          SCATTER_ADD(&g11[c], gsrc * wt[2]);
          SCATTER_ADD(&g10[c], gsrc * wt[3]);
          REAL t1 = t11[c] - t10[c] - t01[c] + t00[c];       /* :447 */
          hg += gsrc * (t1 * p.dw + t10[c] - t00[c]);
          wg += gsrc * (t1 * p.dh + t01[c] - t00[c]);
        }
        dsum += ((p.hc * p.z - p.zc * p.h3d) * hg + (p.wc * p.z - p.zc * p.w3d) * wg) / (p.z * p.z);
      }
      if (kind == 2) depth_grad[vox] = dsum;
      else depth_grad[pix] += dsum;
    }
  }
}

/* ---- kind 4 = CostVolumeV3 (cost_volume_kernels_gpu_v3.cu.cc) ---------------------------------------
 * cost [B,H,W,D,1]; depth = base_plane + offsets as in kind 1.  Per view the cost is the LARGEST dot
 * product between any group of the sampled source feature and any group of the reference feature
 * (groups are contiguous blocks of sub = C/groups <= 8 channels, :111-128); the running maximum starts
 * at the smallest positive normal number, so a view whose dot products are all <= that contributes that
 * number.  MEAN averages the per-view maxima over the valid views, mask = number of valid views
 * (:130-141).  MIN keeps the maximum over views too, mask [..,3] = (view, reference group, source group)
 * of the winner or -1,-1,-1 and cost 0 when nothing exceeded the start value (:190-193,237-257). */
static REAL FN(v3_best)(const REAL *rc, const REAL *t00, const REAL *t01, const REAL *t10, const REAL *t11,
                        const REAL wt[4], int64_t groups, int64_t sub, REAL start, int *best_gi, int *best_gs) {
  REAL cur = start;
  REAL buf[64];
  for (int64_t gs = 0; gs < groups; ++gs) {
    for (int64_t k = 0; k < sub; ++k) {
      const int64_t c = gs * sub + k;
      buf[k] = wt[0] * t00[c] + wt[1] * t01[c] + wt[2] * t11[c] + wt[3] * t10[c];   /* :114-115 */
    }
    for (int64_t gi = 0; gi < groups; ++gi) {
      REAL tmp = (REAL)0;
      for (int64_t k = 0; k < sub; ++k) tmp += buf[k] * rc[gi * sub + k];            /* :119-122 */
      if (cur < tmp) { cur = tmp; *best_gi = (int)gi; *best_gs = (int)gs; }          /* :123-125 */
    }
  }
  return cur;
}

static void FN(cost3_fwd)(int reduce_min, int half_centor, const int64_t *dims, int groups, const REAL *ref,
                          const REAL *src, const REAL *base, const REAL *offsets, const REAL *Rs,
                          const REAL *Ts, REAL *cost, int32_t *mask, int nthreads) {
  const int64_t B = dims[0], H = dims[1], W = dims[2], C = dims[3], D = dims[4], N = dims[5],
                Hs = dims[6], Ws = dims[7];
  const int64_t sub = C / groups, npix = B * H * W;
#pragma omp parallel for schedule(dynamic, 16) num_threads(nthreads > 0 ? nthreads : 1)
  for (int64_t pix = 0; pix < npix; ++pix) {
    const int64_t b = pix / (H * W), h = (pix / W) % H, w = pix % W;
    REAL x = (REAL)w, y = (REAL)h;
    if (half_centor) { x = x + (REAL)0.5; y = y + (REAL)0.5; }
    const REAL *rc = ref + pix * C;
    for (int64_t d = 0; d < D; ++d) {
      const int64_t vox = pix * D + d;
      const REAL depth = base[pix] + offsets[b * D + d];
      int32_t used = 0;
      int32_t win[3] = {-1, -1, -1};
      REAL acc = reduce_min ? REAL_MIN_POS : (REAL)0;
      for (int64_t n = 0; n < N; ++n) {
        FN(proj) p;
        FN(project)(x, y, depth, Rs + (b * N + n) * 9, Ts + (b * N + n) * 3, half_centor, Hs, Ws, &p);
        if (!p.valid) continue;
        REAL wt[4];
        FN(weights)(p.dh, p.dw, wt);
        const REAL *t00 = src + C * (p.fw + Ws * (p.fh + Hs * (n + N * b)));
        const REAL *t01 = t00 + C, *t10 = t00 + Ws * C, *t11 = t10 + C;
        int gi = -1, gs = -1;
        if (reduce_min) {
          const REAL best = FN(v3_best)(rc, t00, t01, t10, t11, wt, groups, sub, acc, &gi, &gs);
          if (gi >= 0) { acc = best; win[0] = (int32_t)n; win[1] = gi; win[2] = gs; }
        } else {
          acc += FN(v3_best)(rc, t00, t01, t10, t11, wt, groups, sub, REAL_MIN_POS, &gi, &gs);  /* :130 */
          used += 1;
        }
      }
      if (reduce_min) {
        mask[vox * 3] = win[0]; mask[vox * 3 + 1] = win[1]; mask[vox * 3 + 2] = win[2];
        cost[vox] = win[0] >= 0 ? acc : (REAL)0;
      } else {
        mask[vox] = used;
        cost[vox] = used > 0 ? acc / (REAL)used : (REAL)0;
      }
    }
  }
}

/* Gradient (:376-520 MEAN, :522-639 MIN): only the winning pair of groups of each view receives a
 * gradient.  MEAN recomputes the winner per view; a view in which no dot product exceeded the start
 * value has no winner - the reference then indexes group -1 (out of bounds); here that view contributes
 * nothing.  MIN reads the winner from the mask and does not re-test the sample position. */
static void FN(cost3_bwd)(int reduce_min, int half_centor, const int64_t *dims, int groups, const REAL *ref,
                          const REAL *src, const REAL *base, const REAL *offsets, const REAL *Rs,
                          const REAL *Ts, const REAL *cost_grad, const int32_t *mask, REAL *ref_grad,
                          REAL *src_grad, REAL *depth_grad, int nthreads) {
  const int64_t B = dims[0], H = dims[1], W = dims[2], C = dims[3], D = dims[4], N = dims[5],
                Hs = dims[6], Ws = dims[7];
  const int64_t sub = C / groups, npix = B * H * W;
  memset(ref_grad, 0, sizeof(REAL) * (size_t)(npix * C));
  memset(src_grad, 0, sizeof(REAL) * (size_t)(B * N * Hs * Ws * C));
  memset(depth_grad, 0, sizeof(REAL) * (size_t)npix);
  const int par = nthreads > 1;
#pragma omp parallel for schedule(dynamic, 16) num_threads(par ? nthreads : 1) if (par)
  for (int64_t pix = 0; pix < npix; ++pix) {
    const int64_t b = pix / (H * W), h = (pix / W) % H, w = pix % W;
    REAL x = (REAL)w, y = (REAL)h;
    if (half_centor) { x = x + (REAL)0.5; y = y + (REAL)0.5; }
    const REAL *rc = ref + pix * C;
    REAL *rg = ref_grad + pix * C;
    for (int64_t d = 0; d < D; ++d) {
      const int64_t vox = pix * D + d;
      const int32_t *mo = mask + vox * (reduce_min ? 3 : 1);
      if (reduce_min ? (mo[0] < 0) : (mo[0] <= 0)) continue;                       /* :393, :541 */
      const REAL depth = base[pix] + offsets[b * D + d];
      const REAL cg = reduce_min ? cost_grad[vox] : cost_grad[vox] / (REAL)mo[0];   /* :426 */
      REAL dsum = (REAL)0;
      for (int64_t n = reduce_min ? mo[0] : 0; n < (reduce_min ? mo[0] + 1 : N); ++n) {
        FN(proj) p;
        FN(project)(x, y, depth, Rs + (b * N + n) * 9, Ts + (b * N + n) * 3, half_centor, Hs, Ws, &p);
        if (!p.valid) continue;
        REAL wt[4];
        FN(weights)(p.dh, p.dw, wt);
        const int64_t off = C * (p.fw + Ws * (p.fh + Hs * (n + N * b)));
        const REAL *t00 = src + off, *t01 = t00 + C, *t10 = t00 + Ws * C, *t11 = t10 + C;
        REAL *g00 = src_grad + off, *g01 = g00 + C, *g10 = g00 + Ws * C, *g11 = g10 + C;
        int gi = -1, gs = -1;
        if (reduce_min) { gi = mo[1]; gs = mo[2]; }
        else FN(v3_best)(rc, t00, t01, t10, t11, wt, groups, sub, REAL_MIN_POS, &gi, &gs);
        if (gi < 0) continue;
        REAL hg = (REAL)0, wg = (REAL)0;
        for (int64_t k = 0; k < sub; ++k) {
          const int64_t r = gi * sub + k, c = gs * sub + k;
          REAL s = wt[0] * t00[c] + wt[1] * t01[c] + wt[2] * t11[c] + wt[3] * t10[c];
          rg[r] += cg * s;                                                           /* :490 */
          REAL bg = cg * rc[r];
          SCATTER_ADD(&g00[c], bg * wt[0]);
          SCATTER_ADD(&g01[c], bg * wt[1]);
          SCATTER_ADD(&g11[c], bg * wt[2]);
          SCATTER_ADD(&g10[c], bg * wt[3]);
          REAL t1 = t11[c] - t10[c] - t01[c] + t00[c];                               /* :498 */
          hg += bg * (t1 * p.dw + t10[c] - t00[c]);
          wg += bg * (t1 * p.dh + t01[c] - t00[c]);
        }
        dsum += ((p.hc * p.z - p.zc * p.h3d) * hg + (p.wc * p.z - p.zc * p.w3d) * wg) / (p.z * p.z);
      }
      depth_grad[pix] += dsum;
    }
  }
}

/* ---- FeatureAggregate (feature_aggregate_kernels_gpu.cu.cc:33-121, gradient :219-317) -----------------
 * The plane-sweep warp without a reduction: mapped [B,H,W,D,N,C] holds the bilinear sample of every source
 * view at every voxel (zeros where the view does not see it), mask [B,H,W,D,N,1] is 1/0.  (H,W) is the
 * output grid (that of base_plane) and may differ from the source size (Hs,Ws). */
static void FN(fa_fwd)(int half_centor, const int64_t *dims, const REAL *src, const REAL *base,
                       const REAL *offsets, const REAL *Rs, const REAL *Ts, REAL *mapped, int32_t *mask,
                       int nthreads) {
  const int64_t B = dims[0], H = dims[1], W = dims[2], C = dims[3], D = dims[4], N = dims[5],
                Hs = dims[6], Ws = dims[7];
  const int64_t npix = B * H * W;
#pragma omp parallel for schedule(dynamic, 16) num_threads(nthreads > 0 ? nthreads : 1)
  for (int64_t pix = 0; pix < npix; ++pix) {
    const int64_t b = pix / (H * W), h = (pix / W) % H, w = pix % W;
    REAL x = (REAL)w, y = (REAL)h;
    if (half_centor) { x = x + (REAL)0.5; y = y + (REAL)0.5; }
    for (int64_t d = 0; d < D; ++d) {
      const int64_t vox = pix * D + d;
      const REAL depth = base[pix] + offsets[b * D + d];
      for (int64_t n = 0; n < N; ++n) {
        REAL *out = mapped + (vox * N + n) * C;
        FN(proj) p;
        FN(project)(x, y, depth, Rs + (b * N + n) * 9, Ts + (b * N + n) * 3, half_centor, Hs, Ws, &p);
        mask[vox * N + n] = p.valid;
        if (!p.valid) {
          for (int64_t c = 0; c < C; ++c) out[c] = (REAL)0;   /* :113-117 */
          continue;
        }
        REAL wt[4];
        FN(weights)(p.dh, p.dw, wt);
        const REAL *t00 = src + C * (p.fw + Ws * (p.fh + Hs * (n + N * b)));
        const REAL *t01 = t00 + C, *t10 = t00 + Ws * C, *t11 = t10 + C;
        for (int64_t c = 0; c < C; ++c)
          out[c] = wt[0] * t00[c] + wt[1] * t01[c] + wt[2] * t11[c] + wt[3] * t10[c];   /* :104-105 */
      }
    }
  }
}

static void FN(fa_bwd)(int half_centor, const int64_t *dims, const REAL *src, const REAL *base,
                       const REAL *offsets, const REAL *Rs, const REAL *Ts, const REAL *mapped_grad,
                       const int32_t *mask, REAL *src_grad, REAL *base_grad, int nthreads) {
  const int64_t B = dims[0], H = dims[1], W = dims[2], C = dims[3], D = dims[4], N = dims[5],
                Hs = dims[6], Ws = dims[7];
  const int64_t npix = B * H * W;
  memset(src_grad, 0, sizeof(REAL) * (size_t)(B * N * Hs * Ws * C));
  memset(base_grad, 0, sizeof(REAL) * (size_t)npix);
  const int par = nthreads > 1;
#pragma omp parallel for schedule(dynamic, 16) num_threads(par ? nthreads : 1) if (par)
  for (int64_t pix = 0; pix < npix; ++pix) {
    const int64_t b = pix / (H * W), h = (pix / W) % H, w = pix % W;
    REAL x = (REAL)w, y = (REAL)h;
    if (half_centor) { x = x + (REAL)0.5; y = y + (REAL)0.5; }
    for (int64_t d = 0; d < D; ++d) {
      const int64_t vox = pix * D + d;
      const REAL depth = base[pix] + offsets[b * D + d];
      REAL dsum = (REAL)0;
      for (int64_t n = 0; n < N; ++n) {
        if (mask[vox * N + n] == 0) continue;   /* :262-264; the position is not re-tested */
        FN(proj) p;
        FN(project)(x, y, depth, Rs + (b * N + n) * 9, Ts + (b * N + n) * 3, half_centor, Hs, Ws, &p);
        if (!p.valid) continue;                 /* (a mask that did not come from the forward pass) */
        REAL wt[4];
        FN(weights)(p.dh, p.dw, wt);
        const int64_t off = C * (p.fw + Ws * (p.fh + Hs * (n + N * b)));
        const REAL *t00 = src + off, *t01 = t00 + C, *t10 = t00 + Ws * C, *t11 = t10 + C;
        REAL *g00 = src_grad + off, *g01 = g00 + C, *g10 = g00 + Ws * C, *g11 = g10 + C;
        const REAL *g = mapped_grad + (vox * N + n) * C;
        REAL hg = (REAL)0, wg = (REAL)0;
        for (int64_t c = 0; c < C; ++c) {
          SCATTER_ADD(&g00[c], g[c] * wt[0]);   /* :303-306 */
          SCATTER_ADD(&g01[c], g[c] * wt[1]);
          SCATTER_ADD(&g11[c], g[c] * wt[2]);
          SCATTER_ADD(&g10[c], g[c] * wt[3]);
          REAL t1 = t11[c] - t10[c] - t01[c] + t00[c];
          hg += g[c] * (t1 * p.dw + t10[c] - t00[c]);
          wg += g[c] * (t1 * p.dh + t01[c] - t00[c]);
        }
        dsum += ((p.hc * p.z - p.zc * p.h3d) * hg + (p.wc * p.z - p.zc * p.w3d) * wg) / (p.z * p.z);
      }
      if (par) {
#pragma omp atomic
        base_grad[pix] += dsum;
      } else {
        base_grad[pix] += dsum;
      }
    }
  }
}
