/* TEST INFRASTRUCTURE ONLY.  CPU oracle for the cost-volume path: a plain-C restatement of the
 * reference's arithmetic (see chop_oracle_impl.h), instantiated for float and double.  Used by
 * tests/, by the smoke check and by the cpu_baseline leg of bench.py; the shipped library never
 * links, loads or calls it.
 *
 * Parity of this restatement is pinned two ways: against the reference's own kernel bodies
 * compiled as host code (oracle/_ref, built by build_ref.py wherever the reference checkout is
 * present) and against the fixtures under tests/golden/ that those bodies produced.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off -fPIC -shared chop_oracle.c -o libchop_oracle.so -lm
 */
#include <float.h>
#include <stdint.h>
#include <string.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define REAL_MAX FLT_MAX
#define REAL_MIN_POS FLT_MIN
#define FN(x) CAT(x, _f32)
#include "chop_oracle_impl.h"
#undef REAL
#undef REAL_MAX
#undef REAL_MIN_POS
#undef FN

#define REAL double
#define REAL_MAX DBL_MAX
#define REAL_MIN_POS DBL_MIN
#define FN(x) CAT(x, _f64)
#include "chop_oracle_impl.h"
#undef REAL
#undef REAL_MAX
#undef REAL_MIN_POS
#undef FN

/* dtype: 0 = float32, 1 = float64; dims = {B,H,W,C,D,N,Hs,Ws}. */
int oracle_cost_fwd(int kind, int dtype, int reduce_min, int half_centor, const int64_t *dims,
                    int groups, const void *ref, const void *src, const void *depth,
                    const void *offsets, const void *Rs, const void *Ts, void *cost,
                    int32_t *mask, int nthreads) {
  if (kind == 4) {
    if (dtype == 0) cost3_fwd_f32(reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost, mask, nthreads);
    else cost3_fwd_f64(reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost, mask, nthreads);
    return 0;
  }
  if (dtype == 0)
    cost_fwd_f32(kind, reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost, mask, nthreads);
  else
    cost_fwd_f64(kind, reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost, mask, nthreads);
  return 0;
}

int oracle_cost_bwd(int kind, int dtype, int reduce_min, int half_centor, const int64_t *dims,
                    int groups, const void *ref, const void *src, const void *depth,
                    const void *offsets, const void *Rs, const void *Ts, const void *cost_grad,
                    const int32_t *mask, void *ref_grad, void *src_grad, void *depth_grad,
                    int nthreads) {
  if (kind == 4) {
    if (dtype == 0) cost3_bwd_f32(reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, ref_grad, src_grad, depth_grad, nthreads);
    else cost3_bwd_f64(reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, ref_grad, src_grad, depth_grad, nthreads);
    return 0;
  }
  if (dtype == 0)
    cost_bwd_f32(kind, reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, ref_grad, src_grad, depth_grad, nthreads);
  else
    cost_bwd_f64(kind, reduce_min, half_centor, dims, groups, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, ref_grad, src_grad, depth_grad, nthreads);
  return 0;
}

/* dims = {B, H, W, C, D, N, Hs, Ws}: (H, W) the output grid, (Hs, Ws) the source images. */
int oracle_feature_aggregate_fwd(int dtype, int half_centor, const int64_t *dims, const void *src, const void *base,
                                 const void *offsets, const void *Rs, const void *Ts, void *mapped, int32_t *mask,
                                 int nthreads) {
  if (dtype == 0) fa_fwd_f32(half_centor, dims, src, base, offsets, Rs, Ts, mapped, mask, nthreads);
  else fa_fwd_f64(half_centor, dims, src, base, offsets, Rs, Ts, mapped, mask, nthreads);
  return 0;
}

int oracle_feature_aggregate_bwd(int dtype, int half_centor, const int64_t *dims, const void *src, const void *base,
                                 const void *offsets, const void *Rs, const void *Ts, const void *mapped_grad,
                                 const int32_t *mask, void *src_grad, void *base_grad, int nthreads) {
  if (dtype == 0) fa_bwd_f32(half_centor, dims, src, base, offsets, Rs, Ts, mapped_grad, mask, src_grad, base_grad, nthreads);
  else fa_bwd_f64(half_centor, dims, src, base, offsets, Rs, Ts, mapped_grad, mask, src_grad, base_grad, nthreads);
  return 0;
}
