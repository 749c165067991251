/* TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's manifold ("sparse") 3-D convolution
 * SparseConv3DFast and its gradient (paths relative to custom_helper_op/cc/kernels/ of the reference):
 *   forward        sparse_conv3d_fast_op_gpu.cu.cc:174-278 / sparse_conv3d_fast_fixed_param_op_gpu.cu.cc:56-160
 *   filter grad    sparse_conv3d_fast_op_gpu.cu.cc:455-576 / ..._fixed_param_op_gpu.cu.cc:206-327
 *   image grad     the forward run "strideOnOutput=false" over out_grad with the flipped, channel-swapped
 *                  filter, zero default and right padding (sparse_conv3d_fast_op.cc:298-323)
 * The reference kernels are warp/block cooperative (shuffles, shared-memory trees) and cannot be compiled
 * for the host, so this file restates them; products are accumulated in double and rounded once, which is
 * the "truth" the CUDA kernels are compared with under a floating tolerance.  The restatement itself is
 * checked against a dense convolution (the reference tests' own method) and, for the forward pass,
 * against the reference's older thread-per-voxel kernel compiled as host code.
 *
 * A voxel images[b,r,c,d,:] sits at absolute depth base_plane[b,r,c] + d.  Neighbours outside the image
 * plane or outside their own band contribute default_value.
 *
 * Transposed convolution SparseConv3DTransposeFast (sparse_conv3d_fast_op.cc:346-411) and its gradient
 * (:427-505): the geometry p is that of the forward convolution whose transpose is taken - (H,W,D) is the
 * FINE grid (the transposed op's output, which base_plane describes), (oH,oW,oD) the COARSE grid (its
 * input, with Cout channels); the output has Cin channels.  The op gathers: every fine voxel sums, over
 * the taps of the flipped filter, the coarse voxel that lies exactly on the tap (stride-aligned in all
 * three dimensions and inside its band), else default_value.
 *
 * SparsePad / SparsePadGrad (sparse_pad_kernels_gpu.cu.cc:36-64, 82-104): zero insertion from the coarse
 * band into the fine band.
 *
 * p = {B, H, W, D, Cin, Cout, fh, fw, fd, sr, sc, sd, dr, dc, dd}
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  int B, H, W, D, Cin, Cout, fh, fw, fd, sr, sc, sd, dr, dc, dd;
  int oH, oW, oD, pr, pc, pd;
} sp_t;

static sp_t unpack(const int *p) {
  sp_t s = {p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7], p[8], p[9], p[10], p[11], p[12], p[13], p[14]};
  s.oH = (s.H + s.sr - 1) / s.sr;  /* sparse_conv3d_fast_op.cc:104-106 */
  s.oW = (s.W + s.sc - 1) / s.sc;
  s.oD = (s.D + s.sd - 1) / s.sd;
  s.pr = s.fh / 2 * s.dr;          /* :107-109 */
  s.pc = s.fw / 2 * s.dc;
  s.pd = s.fd / 2 * s.dd;
  return s;
}

#define OOB(a, b) ((unsigned)(a) >= (unsigned)(b)) /* CHECK_PADDING, fixed_param_op_gpu.cu.cc:20 */

#define DEFINE(REAL, SUF)                                                                                   \
  /* Band-local input depth of tap (fr,fc,fz) for output voxel (b,ro,co,dz); -1 if padded. */               \
  static int64_t tap_index_##SUF(const sp_t *s, const int32_t *bp, int b, int ro, int co, int dz, int fr,   \
                                 int fc, int fz) {                                                           \
    const int row = ro * s->sr, col = co * s->sc;                                                            \
    const int depth = (dz + (bp[(b * s->H + row) * s->W + col] + s->sd - 1) / s->sd) * s->sd; /* :80 */      \
    const int orow = row - s->pr + fr * s->dr, ocol = col - s->pc + fc * s->dc;                              \
    if (OOB(orow, s->H) || OOB(ocol, s->W)) return -1;                                                       \
    const int pix = (b * s->H + orow) * s->W + ocol;                                                         \
    const int ind = depth - s->pd + fz * s->dd - bp[pix]; /* :106 */                                         \
    if (OOB(ind, s->D)) return -1;                                                                           \
    return ((int64_t)pix * s->D + ind) * s->Cin;                                                             \
  }                                                                                                          \
                                                                                                             \
  static void fwd_##SUF(const int *p, const REAL *img, const REAL *flt, REAL defv, const int32_t *bp,       \
                        REAL *out, int nthreads) {                                                           \
    const sp_t s = unpack(p);                                                                                \
    const int64_t nvox = (int64_t)s.B * s.oH * s.oW * s.oD;                                                  \
    _Pragma("omp parallel for schedule(static) num_threads(nthreads > 0 ? nthreads : 1)")                    \
    for (int64_t v = 0; v < nvox; ++v) {                                                                     \
      const int dz = (int)(v % s.oD), co = (int)(v / s.oD % s.oW), ro = (int)(v / s.oD / s.oW % s.oH),      \
                b = (int)(v / s.oD / s.oW / s.oH);                                                           \
      double acc[512];                                                                                       \
      for (int o = 0; o < s.Cout; ++o) acc[o] = 0.0;                                                         \
      for (int fr = 0; fr < s.fh; ++fr)                                                                      \
        for (int fc = 0; fc < s.fw; ++fc)                                                                    \
          for (int fz = 0; fz < s.fd; ++fz) {                                                                \
            const int64_t at = tap_index_##SUF(&s, bp, b, ro, co, dz, fr, fc, fz);                           \
            const REAL *w = flt + (((int64_t)fr * s.fw + fc) * s.fd + fz) * s.Cin * s.Cout;                  \
            for (int ci = 0; ci < s.Cin; ++ci) {                                                             \
              const double x = at < 0 ? (double)defv : (double)img[at + ci];                                 \
              for (int o = 0; o < s.Cout; ++o) acc[o] += (double)w[ci * s.Cout + o] * x;                     \
            }                                                                                                \
          }                                                                                                  \
      for (int o = 0; o < s.Cout; ++o) out[v * s.Cout + o] = (REAL)acc[o];                                   \
    }                                                                                                        \
  }                                                                                                          \
                                                                                                             \
  /* filter_grad [fh,fw,fd,Cin,Cout] and default_value_grad (scalar, only if dynamic_default). */           \
  static void wgrad_##SUF(const int *p, const REAL *img, const REAL *flt, REAL defv, const int32_t *bp,     \
                          const REAL *og, int dynamic_default, REAL *fgrad, REAL *dgrad) {                   \
    const sp_t s = unpack(p);                                                                                \
    const int64_t nvox = (int64_t)s.B * s.oH * s.oW * s.oD;                                                  \
    const int64_t nf = (int64_t)s.fh * s.fw * s.fd * s.Cin * s.Cout;                                         \
    double *acc = (double *)calloc((size_t)nf, sizeof(double));                                              \
    double dacc = 0.0;                                                                                       \
    for (int64_t v = 0; v < nvox; ++v) {                                                                     \
      const int dz = (int)(v % s.oD), co = (int)(v / s.oD % s.oW), ro = (int)(v / s.oD / s.oW % s.oH),      \
                b = (int)(v / s.oD / s.oW / s.oH);                                                           \
      const REAL *g = og + v * s.Cout;                                                                       \
      for (int fr = 0; fr < s.fh; ++fr)                                                                      \
        for (int fc = 0; fc < s.fw; ++fc)                                                                    \
          for (int fz = 0; fz < s.fd; ++fz) {                                                                \
            const int64_t at = tap_index_##SUF(&s, bp, b, ro, co, dz, fr, fc, fz);                           \
            const int64_t wo = (((int64_t)fr * s.fw + fc) * s.fd + fz) * s.Cin * s.Cout;                     \
            for (int ci = 0; ci < s.Cin; ++ci) {                                                             \
              const double x = at < 0 ? (double)defv : (double)img[at + ci]; /* fixed :279-281 */            \
              for (int o = 0; o < s.Cout; ++o) {                                                             \
                acc[wo + ci * s.Cout + o] += x * (double)g[o];                                               \
                if (at < 0 && dynamic_default) dacc += (double)flt[wo + ci * s.Cout + o] * (double)g[o];     \
              }                                                                                              \
            }                                                                                                \
          }                                                                                                  \
    }                                                                                                        \
    for (int64_t i = 0; i < nf; ++i) fgrad[i] = (REAL)acc[i];                                                \
    *dgrad = (REAL)dacc; /* zero unless dynamic_default (sparse_conv3d_fast_op.cc:269) */                    \
    free(acc);                                                                                               \
  }                                                                                                          \
                                                                                                             \
  /* images_grad, gather form: for every INPUT voxel, sum over the taps of the flipped filter. */           \
  static void dgrad_##SUF(const int *p, const REAL *flt, const int32_t *bp, const REAL *og, REAL *igrad,    \
                          int nthreads) {                                                                    \
    const sp_t s = unpack(p);                                                                                \
    /* right padding of the swapped problem (sparse_conv3d_fast_op.cc:314-316) */                            \
    const int qr = (s.fh - 1) * s.dr - s.pr, qc = (s.fw - 1) * s.dc - s.pc, qd = (s.fd - 1) * s.dd - s.pd;   \
    const int64_t nvox = (int64_t)s.B * s.H * s.W * s.D;                                                     \
    _Pragma("omp parallel for schedule(static) num_threads(nthreads > 0 ? nthreads : 1)")                    \
    for (int64_t v = 0; v < nvox; ++v) {                                                                     \
      const int dz = (int)(v % s.D), c = (int)(v / s.D % s.W), r = (int)(v / s.D / s.W % s.H),              \
                b = (int)(v / s.D / s.W / s.H);                                                              \
      double acc[512];                                                                                       \
      for (int ci = 0; ci < s.Cin; ++ci) acc[ci] = 0.0;                                                      \
      const int depth = dz + bp[(b * s.H + r) * s.W + c]; /* fixed :82 */                                    \
      for (int fr = 0; fr < s.fh; ++fr)                                                                      \
        for (int fc = 0; fc < s.fw; ++fc)                                                                    \
          for (int fz = 0; fz < s.fd; ++fz) {                                                                \
            const int orow = r - qr + fr * s.dr, ocol = c - qc + fc * s.dc; /* fixed :114-131 */             \
            if (OOB(orow, s.H) || OOB(ocol, s.W)) continue;                                                  \
            int od = depth - qd + fz * s.dd;                                                                 \
            if ((orow % s.sr) != 0 || (ocol % s.sc) != 0 || (od % s.sd) != 0) continue;                      \
            od = od / s.sd - (bp[(b * s.H + orow) * s.W + ocol] + s.sd - 1) / s.sd;                          \
            if (OOB(od, s.oD)) continue;                                                                     \
            const int64_t at = ((((int64_t)b * s.oH + orow / s.sr) * s.oW + ocol / s.sc) * s.oD + od) * s.Cout; \
            /* flipped in all three filter dimensions, Cin/Cout swapped (:304-305) */                        \
            const REAL *w = flt + (((int64_t)(s.fh - 1 - fr) * s.fw + (s.fw - 1 - fc)) * s.fd + (s.fd - 1 - fz)) * \
                                      s.Cin * s.Cout;                                                        \
            for (int ci = 0; ci < s.Cin; ++ci)                                                               \
              for (int o = 0; o < s.Cout; ++o) acc[ci] += (double)w[ci * s.Cout + o] * (double)og[at + o];   \
          }                                                                                                  \
      for (int ci = 0; ci < s.Cin; ++ci) igrad[v * s.Cin + ci] = (REAL)acc[ci];                              \
    }                                                                                                        \
  }                                                                                                          \
                                                                                                             \
  /* Offset (in units of Cout) of the coarse voxel under tap (fr,fc,fz) of FINE voxel (b,r,c,dz), gather    \
   * form with right padding (sparse_conv3d_fast_op.cc:395-397; kernel branch strideOnOutput=false,          \
   * sparse_conv3d_fast_op_gpu.cu.cc:201,233-247); -1 if the tap is padding. */                              \
  static int64_t ttap_index_##SUF(const sp_t *s, const int32_t *bp, int b, int r, int c, int dz, int fr,    \
                                  int fc, int fz) {                                                          \
    const int qr = (s->fh - 1) * s->dr - s->pr, qc = (s->fw - 1) * s->dc - s->pc,                            \
              qd = (s->fd - 1) * s->dd - s->pd;                                                              \
    const int depth = dz + bp[(b * s->H + r) * s->W + c];                                                    \
    const int orow = r - qr + fr * s->dr, ocol = c - qc + fc * s->dc;                                        \
    if (OOB(orow, s->H) || OOB(ocol, s->W)) return -1;                                                       \
    int od = depth - qd + fz * s->dd;                                                                        \
    if ((orow % s->sr) != 0 || (ocol % s->sc) != 0 || (od % s->sd) != 0) return -1;                          \
    od = od / s->sd - (bp[(b * s->H + orow) * s->W + ocol] + s->sd - 1) / s->sd;                             \
    if (OOB(od, s->oD)) return -1;                                                                           \
    return (((int64_t)b * s->oH + orow / s->sr) * s->oW + ocol / s->sc) * s->oD + od;                        \
  }                                                                                                          \
                                                                                                             \
  /* out [B,H,W,D,Cin] from images [B,oH,oW,oD,Cout]. */                                                    \
  static void tfwd_##SUF(const int *p, const REAL *img, const REAL *flt, REAL defv, const int32_t *bp,      \
                         REAL *out, int nthreads) {                                                          \
    const sp_t s = unpack(p);                                                                                \
    const int64_t nvox = (int64_t)s.B * s.H * s.W * s.D;                                                     \
    _Pragma("omp parallel for schedule(static) num_threads(nthreads > 0 ? nthreads : 1)")                    \
    for (int64_t v = 0; v < nvox; ++v) {                                                                     \
      const int dz = (int)(v % s.D), c = (int)(v / s.D % s.W), r = (int)(v / s.D / s.W % s.H),              \
                b = (int)(v / s.D / s.W / s.H);                                                              \
      double acc[512];                                                                                       \
      for (int ci = 0; ci < s.Cin; ++ci) acc[ci] = 0.0;                                                      \
      for (int fr = 0; fr < s.fh; ++fr)                                                                      \
        for (int fc = 0; fc < s.fw; ++fc)                                                                    \
          for (int fz = 0; fz < s.fd; ++fz) {                                                                \
            const int64_t at = ttap_index_##SUF(&s, bp, b, r, c, dz, fr, fc, fz);                            \
            /* filter flipped in the three spatial dimensions (sparse_conv3d_fast_op.cc:383-384) */          \
            const REAL *w = flt + (((int64_t)(s.fh - 1 - fr) * s.fw + (s.fw - 1 - fc)) * s.fd + (s.fd - 1 - fz)) * \
                                      s.Cin * s.Cout;                                                        \
            for (int ci = 0; ci < s.Cin; ++ci)                                                               \
              for (int o = 0; o < s.Cout; ++o)                                                               \
                acc[ci] += (double)w[ci * s.Cout + o] * (at < 0 ? (double)defv : (double)img[at * s.Cout + o]); \
          }                                                                                                  \
      for (int ci = 0; ci < s.Cin; ++ci) out[v * s.Cin + ci] = (REAL)acc[ci];                                \
    }                                                                                                        \
  }                                                                                                          \
                                                                                                             \
  /* Filter gradient of the transposed op: fgrad[flip(tap)][ci][co] = sum over fine voxels of                \
   * value(tap, co) * out_grad[voxel][ci], value = coarse voxel or default_value                             \
   * (sparse_conv3d_fast_op.cc:477-488 with the kernel of sparse_conv3d_fast_op_gpu.cu.cc:455-546).          \
   * The reference leaves the two channel axes of its result in the order [.., Cout, Cin] inside a buffer   \
   * declared [.., Cin, Cout] (the kernel writes [tap][in_ch][out_ch] of the swapped problem and :487-488    \
   * only reverses the spatial axes); ref_layout != 0 reproduces that buffer, 0 gives d(out)/d(filter). */   \
  static void twgrad_##SUF(const int *p, const REAL *img, REAL defv, const int32_t *bp, const REAL *og,     \
                           int ref_layout, REAL *fgrad) {                                                    \
    const sp_t s = unpack(p);                                                                                \
    const int64_t nvox = (int64_t)s.B * s.H * s.W * s.D;                                                     \
    const int64_t nf = (int64_t)s.fh * s.fw * s.fd * s.Cin * s.Cout;                                         \
    double *acc = (double *)calloc((size_t)nf, sizeof(double));                                              \
    for (int64_t v = 0; v < nvox; ++v) {                                                                     \
      const int dz = (int)(v % s.D), c = (int)(v / s.D % s.W), r = (int)(v / s.D / s.W % s.H),              \
                b = (int)(v / s.D / s.W / s.H);                                                              \
      const REAL *g = og + v * s.Cin;                                                                        \
      for (int fr = 0; fr < s.fh; ++fr)                                                                      \
        for (int fc = 0; fc < s.fw; ++fc)                                                                    \
          for (int fz = 0; fz < s.fd; ++fz) {                                                                \
            const int64_t at = ttap_index_##SUF(&s, bp, b, r, c, dz, fr, fc, fz);                            \
            const int64_t wo = (((int64_t)(s.fh - 1 - fr) * s.fw + (s.fw - 1 - fc)) * s.fd + (s.fd - 1 - fz)) * \
                               s.Cin * s.Cout;                                                               \
            for (int o = 0; o < s.Cout; ++o) {                                                               \
              const double x = at < 0 ? (double)defv : (double)img[at * s.Cout + o];                         \
              for (int ci = 0; ci < s.Cin; ++ci)                                                             \
                acc[wo + (ref_layout ? o * s.Cin + ci : ci * s.Cout + o)] += x * (double)g[ci];              \
            }                                                                                                \
          }                                                                                                  \
    }                                                                                                        \
    for (int64_t i = 0; i < nf; ++i) fgrad[i] = (REAL)acc[i];                                                \
    free(acc);                                                                                               \
  }                                                                                                          \
                                                                                                             \
  /* SparsePad: out [B,H,W,D,C] (H = oH*sr ...) from images [B,oH,oW,oD,C]; p[4] = C. */                    \
  static void pad_fwd_##SUF(const int *p, const REAL *img, const int32_t *bp, REAL *out) {                   \
    const int sr = p[9], sc = p[10], sd = p[11], C = p[4];                                                   \
    const int ih = p[1], iw = p[2], id = p[3], oh = ih * sr, ow = iw * sc, od = id * sd;                     \
    const int64_t n = (int64_t)p[0] * oh * ow * od;                                                          \
    for (int64_t i = 0; i < n; ++i) {                                                                        \
      int d = (int)(i % od);                                                                                 \
      const int64_t pos = i / od;                                                                            \
      const int w = (int)(pos % ow), h = (int)(pos / ow % oh), b = (int)(pos / ow / oh);                     \
      d = d + bp[pos] - ((bp[pos] + sd - 1) / sd) * sd; /* sparse_pad_kernels_gpu.cu.cc:50 */                \
      if ((h % sr) == 0 && (w % sc) == 0 && (d % sd) == 0) {                                                 \
        const REAL *x = img + ((((int64_t)b * ih + h / sr) * iw + w / sc) * id + d / sd) * C;                \
        for (int c = 0; c < C; ++c) out[i * C + c] = x[c];                                                   \
      } else {                                                                                               \
        for (int c = 0; c < C; ++c) out[i * C + c] = (REAL)0;                                                \
      }                                                                                                      \
    }                                                                                                        \
  }                                                                                                          \
  /* SparsePadGrad: the adjoint gather.  The reference kernel (:82-104) forms the fine pixel index from      \
   * the COARSE (h, w) before scaling them by the strides, so for row/column strides > 1 it reads the wrong  \
   * pixel; ref_quirk != 0 reproduces that, 0 reads pixel (h*sr, w*sc). */                                   \
  static void pad_bwd_##SUF(const int *p, const int32_t *bp, const REAL *og, int ref_quirk, REAL *igrad) {   \
    const int sr = p[9], sc = p[10], sd = p[11], C = p[4];                                                   \
    const int ih = p[1], iw = p[2], id = p[3], oh = ih * sr, ow = iw * sc, od = id * sd;                     \
    const int64_t n = (int64_t)p[0] * ih * iw * id;                                                          \
    for (int64_t i = 0; i < n; ++i) {                                                                        \
      int d = (int)(i % id);                                                                                 \
      const int64_t q = i / id;                                                                              \
      const int w = (int)(q % iw), h = (int)(q / iw % ih), b = (int)(q / iw / ih);                           \
      const int64_t pos = ref_quirk ? ((int64_t)b * oh + h) * ow + w : ((int64_t)b * oh + h * sr) * ow + w * sc; \
      d = d * sd + ((bp[pos] + sd - 1) / sd) * sd - bp[pos];                                                 \
      for (int c = 0; c < C; ++c) igrad[i * C + c] = og[(pos * od + d) * C + c];                             \
    }                                                                                                        \
  }

DEFINE(float, f32)
DEFINE(double, f64)

int oracle_sparse_conv3d_fwd(int dtype, const int *p, const void *img, const void *flt, const void *defv,
                             const int32_t *bp, void *out, int nthreads) {
  if (p[4] > 512 || p[5] > 512) return -1;
  if (dtype == 0) fwd_f32(p, img, flt, *(const float *)defv, bp, out, nthreads);
  else fwd_f64(p, img, flt, *(const double *)defv, bp, out, nthreads);
  return 0;
}

int oracle_sparse_conv3d_bwd(int dtype, const int *p, const void *img, const void *flt, const void *defv,
                             const int32_t *bp, const void *og, int dynamic_default, void *igrad, void *fgrad,
                             void *dgrad, int nthreads) {
  if (p[4] > 512 || p[5] > 512) return -1;
  if (dtype == 0) {
    wgrad_f32(p, img, flt, *(const float *)defv, bp, og, dynamic_default, fgrad, dgrad);
    dgrad_f32(p, flt, bp, og, igrad, nthreads);
  } else {
    wgrad_f64(p, img, flt, *(const double *)defv, bp, og, dynamic_default, fgrad, dgrad);
    dgrad_f64(p, flt, bp, og, igrad, nthreads);
  }
  return 0;
}

/* Transposed convolution.  reference_quirks = 0: the derivatives (images_grad with zero padding,
 * filter_grad laid out [fh,fw,fd,Cin,Cout]).  reference_quirks = 1: what the reference's grad op writes -
 * images_grad with default_value at padded taps (sparse_conv3d_fast_op.cc:495-500) and filter_grad with
 * its channel axes in the order [Cout, Cin] (see twgrad above). */
int oracle_sparse_conv3d_transpose_fwd(int dtype, const int *p, const void *img, const void *flt, const void *defv,
                                       const int32_t *bp, void *out, int nthreads) {
  if (p[4] > 512 || p[5] > 512) return -1;
  if (dtype == 0) tfwd_f32(p, img, flt, *(const float *)defv, bp, out, nthreads);
  else tfwd_f64(p, img, flt, *(const double *)defv, bp, out, nthreads);
  return 0;
}

int oracle_sparse_conv3d_transpose_bwd(int dtype, const int *p, const void *img, const void *flt, const void *defv,
                                       const int32_t *bp, const void *og, int reference_quirks, void *igrad,
                                       void *fgrad, int nthreads) {
  if (p[4] > 512 || p[5] > 512) return -1;
  if (dtype == 0) {
    const float pad = reference_quirks ? *(const float *)defv : 0.0f;
    fwd_f32(p, og, flt, pad, bp, igrad, nthreads);
    twgrad_f32(p, img, *(const float *)defv, bp, og, reference_quirks, fgrad);
  } else {
    const double pad = reference_quirks ? *(const double *)defv : 0.0;
    fwd_f64(p, og, flt, pad, bp, igrad, nthreads);
    twgrad_f64(p, img, *(const double *)defv, bp, og, reference_quirks, fgrad);
  }
  return 0;
}

/* p = {B, coarse H, W, D, C, -, -, -, -, sr, sc, sd, ...}; base_plane is [B, H*sr, W*sc]. */
int oracle_sparse_pad_fwd(int dtype, const int *p, const void *img, const int32_t *bp, void *out) {
  if (dtype == 0) pad_fwd_f32(p, img, bp, out);
  else pad_fwd_f64(p, img, bp, out);
  return 0;
}
int oracle_sparse_pad_bwd(int dtype, const int *p, const int32_t *bp, const void *og, int reference_quirk, void *igrad) {
  if (dtype == 0) pad_bwd_f32(p, bp, og, reference_quirk, igrad);
  else pad_bwd_f64(p, bp, og, reference_quirk, igrad);
  return 0;
}
