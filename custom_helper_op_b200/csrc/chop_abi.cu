// extern "C" surface of libchop_b200.so for the cost-volume ops: argument validation (what the
// reference's OpKernel::Compute checks with OP_REQUIRES, custom_helper_op/cc/kernels/
// cost_volume_kernels.cc:91-106), launch planning, the zero fill of the gradient outputs, dispatch.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "../../include/chop.h"
#include "cv_entry.h"
#include "cv_launch.cuh"
#include "cv_v3_entry.h"
#include "fa_entry.h"

namespace chop {
extern std::atomic<int> g_use_umma;
extern std::atomic<int> g_use_tile;
void sc_umma_set_rows(int on);
extern std::atomic<int> g_fa_stage;
int sc_umma_note_timeout_for_test(int on);
}

namespace {

using chop::CvArgs;
using chop::CvPlan;

std::atomic<int> g_fwd_chunk{0}, g_bwd_chunk{0}, g_bwd_views{0}, g_tuned{1}, g_packed{1};

inline int pow2ceil_log2(int x) {
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}
inline bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

struct Typed {
  size_t feat_size;  // bytes per ref/src element
  size_t real_size;  // bytes per depth/camera/cost element
};

int typed_of(int dtype, Typed* t) {
  switch (dtype) {
    case CHOP_F32: *t = {4, 4}; return 0;
    case CHOP_F64: *t = {8, 8}; return 0;
    case CHOP_BF16: *t = {2, 4}; return 0;
    default: return CHOP_ERR_ATTR;
  }
}

// Shape / attribute checks shared by forward and backward.  Fills the narrowed CvArgs dims.
int validate(const chop_cv_desc* d, CvArgs* a, Typed* ty) {
  if (!d) return CHOP_ERR_NULL;
  if (d->kind < CHOP_COST_VOLUME || d->kind > CHOP_COST_VOLUME_V3) return CHOP_ERR_ATTR;
  if (d->reduce != CHOP_REDUCE_MEAN && d->reduce != CHOP_REDUCE_MIN) return CHOP_ERR_ATTR;
  if (int e = typed_of(d->dtype, ty)) return e;
  if (d->flags & ~(CHOP_FLAG_STRICT | CHOP_FLAG_ACCUMULATE)) return CHOP_ERR_ATTR;  // a bit this build does not know
  const int64_t dims[] = {d->B, d->H, d->W, d->C, d->D, d->N, d->Hs, d->Ws};
  for (int64_t v : dims)
    if (v < 1 || v > INT32_MAX) return CHOP_ERR_SHAPE;
  // the reference's host op requires source and reference images of one size
  // (cost_volume_kernels.cc:93-95)
  if (d->Hs != d->H || d->Ws != d->W) return CHOP_ERR_SHAPE;
  if (d->Hs < 2 || d->Ws < 2) return CHOP_ERR_SHAPE;
  int G = 1;
  if (d->kind == CHOP_COST_VOLUME_V2) {
    if (d->groups < 1 || d->C % d->groups != 0) return CHOP_ERR_ATTR;  // cost_volume_kernels_v2.cc:107-108
    G = d->groups;
  }
  if (d->kind == CHOP_COST_VOLUME_V3) {
    // cost_volume_kernels_v3.cc:107-111: groups divides C, at most 8 channels per group
    if (d->groups < 1 || d->C % d->groups != 0) return CHOP_ERR_ATTR;
    if (d->C / d->groups > 8) return CHOP_ERR_ATTR;
    if (d->groups > 32) return CHOP_ERR_UNSUPPORTED;  // one lane per group
    G = d->groups;
  }
  // texel and pixel indices are 32-bit inside the kernels; voxel and element offsets are 64-bit
  if (d->B * d->N * d->Hs * d->Ws > INT32_MAX) return CHOP_ERR_SHAPE;
  if (d->B * d->H * d->W > INT32_MAX) return CHOP_ERR_SHAPE;
  if (d->B * d->D > INT32_MAX) return CHOP_ERR_SHAPE;
  const int64_t d_end = d->d_end == 0 ? d->D : d->d_end;
  if (d->d_begin < 0 || d_end > d->D || d->d_begin > d_end) return CHOP_ERR_RANGE;
  a->B = (int)d->B; a->H = (int)d->H; a->W = (int)d->W; a->C = (int)d->C; a->D = (int)d->D;
  a->N = (int)d->N; a->Hs = (int)d->Hs; a->Ws = (int)d->Ws; a->G = G;
  a->d_begin = (int)d->d_begin;
  a->d_end = (int)d_end;
  a->half_centor = d->half_centor ? 1 : 0;
  a->npix = d->B * d->H * d->W;
  return 0;
}

// CostVolume MEAN (fused arithmetic) with a common channel count runs the compile-time-C kernels of
// cv_tuned.cuh, which use four channels per lane for float32 and bfloat16 features alike.
bool tuned_eligible(const chop_cv_desc* d, const CvArgs& a, bool backward) {
  if (!g_tuned.load() || !(d->dtype == CHOP_F32 || d->dtype == CHOP_BF16)) return false;
  // MIN: every gradient kernel, and the CostVolume / CostAggregate forward for up to 32 channels (254 views)
  const bool min_ok = backward || (d->kind == CHOP_COST_VOLUME && a.C <= 32 && a.N <= 254) ||
                      (d->kind == CHOP_COST_AGGREGATE && a.C <= 32) || (d->kind == CHOP_COST_VOLUME_V2 && a.N <= 254);
  if (d->reduce != CHOP_REDUCE_MEAN && !min_ok) return false;
  if (d->kind == CHOP_COST_VOLUME || d->kind == CHOP_COST_AGGREGATE) return a.C == 8 || a.C == 16 || a.C == 32 || a.C == 64;
  if (d->kind == CHOP_COST_VOLUME_V2) {
    const int sub = a.C / a.G;  // channels per group: a lane's four channels must cover whole groups
    return (a.C == 8 || a.C == 16 || a.C == 32) && (sub == 1 || sub == 2 || sub == 4);
  }
  return false;
}

// Channel slice per lane and lanes per pixel.
int plan_lanes(const chop_cv_desc* d, const CvArgs& a, int* cpl, int* lgl, bool strict, bool backward) {
  int c = 1;
  if (d->dtype == CHOP_F32 && a.C % 4 == 0) c = 4;
  if (d->dtype == CHOP_F64 && a.C % 2 == 0) c = 2;
  if (d->dtype == CHOP_BF16 && a.C % 8 == 0) c = 8;
  if (!strict && tuned_eligible(d, a, backward)) c = 4;
  const int lanes = (a.C + c - 1) / c;
  if (lanes > 32) return CHOP_ERR_UNSUPPORTED;
  *cpl = c;
  *lgl = pow2ceil_log2(lanes);
  return 0;
}

void plan_chunks(CvArgs* a, int LG, int wanted_warps, int min_chunk, int forced) {
  const int G = 32 / LG;
  a->npb = (int)((a->npix + G - 1) / G);
  const int drange = a->d_end - a->d_begin;
  int chunk;
  if (forced > 0) {
    chunk = forced;
  } else {
    if (min_chunk < LG) min_chunk = LG;
    const int by_warps = (wanted_warps + a->npb - 1) / a->npb;
    int nchunks;
    for (;;) {
      const int by_depth = (drange + min_chunk - 1) / min_chunk;
      nchunks = by_depth < by_warps ? by_depth : by_warps;
      if (nchunks < 1) nchunks = 1;
      // a small problem (fewer than eight warps per SM): shorter chunks, down to one block of planes, so that the
      // kernel is not one long serial walk per warp on a mostly idle GPU
      if ((long long)a->npb * nchunks >= 148 * 8 || min_chunk <= LG) break;
      min_chunk = min_chunk / 2 > LG ? min_chunk / 2 : LG;
    }
    chunk = (drange + nchunks - 1) / nchunks;
  }
  chunk = (chunk + LG - 1) / LG * LG;
  if (chunk < LG) chunk = LG;
  a->chunk = chunk;
  a->nchunks = (drange + chunk - 1) / chunk;
}

int pick_warps(size_t smem_per_warp) {
  int w = 8;
  while (w > 1 && smem_per_warp * w > 200 * 1024) w >>= 1;
  return smem_per_warp * w > 200 * 1024 ? 0 : w;
}

int dispatch_fwd(int dtype, const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  switch (dtype) {
    case CHOP_F32: return chop::cv_fwd_f32(a, p, st);
    case CHOP_F64: return chop::cv_fwd_f64(a, p, st);
    default: return chop::cv_fwd_bf16(a, p, st);
  }
}
int dispatch_bwd(int dtype, const CvArgs& a, const CvPlan& p, cudaStream_t st) {
  switch (dtype) {
    case CHOP_F32: return chop::cv_bwd_f32(a, p, st);
    case CHOP_F64: return chop::cv_bwd_f64(a, p, st);
    default: return chop::cv_bwd_bf16(a, p, st);
  }
}

// Zero fill of up to three gradient outputs in ONE launch (the reference launcher issues three,
// cost_volume_kernels_gpu.cu.cc:637-642).  Sizes in bytes, multiples of 4; 16-byte stores where a buffer's
// base allows it.
struct ZeroJob {
  void* p[3];
  unsigned long long bytes[3];
};
__global__ void __launch_bounds__(256) zero_fill_kernel(const ZeroJob z) {
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned long long nth = (unsigned long long)gridDim.x * blockDim.x;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    if (!z.p[i]) continue;
    unsigned char* base = static_cast<unsigned char*>(z.p[i]);
    const unsigned long long n = z.bytes[i];
    if ((reinterpret_cast<uintptr_t>(base) & 15) == 0) {
      const unsigned long long n16 = n / 16;
      for (unsigned long long k = tid; k < n16; k += nth) reinterpret_cast<uint4*>(base)[k] = make_uint4(0u, 0u, 0u, 0u);
      for (unsigned long long k = n16 * 4 + tid; k < n / 4; k += nth) reinterpret_cast<unsigned*>(base)[k] = 0u;
    } else {
      for (unsigned long long k = tid; k < n / 4; k += nth) reinterpret_cast<unsigned*>(base)[k] = 0u;
    }
  }
}
int zero_fill(void* p0, size_t b0, void* p1, size_t b1, void* p2, size_t b2, cudaStream_t st) {
  ZeroJob z;
  z.p[0] = p0; z.bytes[0] = b0;
  z.p[1] = p1; z.bytes[1] = b1;
  z.p[2] = p2; z.bytes[2] = b2;
  const size_t most = (b0 > b1 ? (b0 > b2 ? b0 : b2) : (b1 > b2 ? b1 : b2));
  size_t blocks = (most / 16 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  zero_fill_kernel<<<(unsigned)blocks, 256, 0, st>>>(z);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int chop_cost_volume_fwd(const chop_cv_desc* d, const void* ref, const void* src, const void* depth,
                         const void* offsets, const void* Rs, const void* Ts, void* cost, int32_t* mask,
                         void* stream) {
  CvArgs a;
  std::memset(&a, 0, sizeof(a));
  Typed ty;
  if (int e = validate(d, &a, &ty)) return e;
  if (!ref || !src || !depth || !Rs || !Ts || !cost || !mask) return CHOP_ERR_NULL;
  if (d->kind != CHOP_COST_VOLUME_V2 && !offsets) return CHOP_ERR_NULL;
  if (a.d_begin == a.d_end) return CHOP_OK;
  if (d->kind == CHOP_COST_VOLUME_V3) {
    // groups of 4 or 8 channels are fetched with vector loads
    const size_t fa = ((a.C / a.G) % 4 == 0 ? 4 : 1) * ty.feat_size;
    if (!aligned(ref, ty.feat_size) || !aligned(src, fa) || !aligned(depth, ty.real_size) ||
        !aligned(cost, ty.real_size) || !aligned(mask, 4))
      return CHOP_ERR_ALIGN;
    a.lg_log2 = pow2ceil_log2(a.G);
    plan_chunks(&a, 1 << a.lg_log2, 148 * 64, 16, g_fwd_chunk.load());
    a.ref = ref; a.src = src; a.depth = depth; a.offsets = offsets; a.Rs = Rs; a.Ts = Ts;
    a.cost = cost; a.mask = mask;
    return chop::cv3_fwd_launch(d->dtype, d->reduce == CHOP_REDUCE_MIN, a, static_cast<cudaStream_t>(stream));
  }
  int cpl, lgl;
  if (int e = plan_lanes(d, a, &cpl, &lgl, (d->flags & CHOP_FLAG_STRICT) != 0, false)) return e;
  const int mode = d->reduce == CHOP_REDUCE_MIN ? 2 : ((d->flags & CHOP_FLAG_STRICT) ? 1 : 0);

  CvPlan p;
  std::memset(&p, 0, sizeof(p));
  p.kind = d->kind;
  p.mode = mode;
  p.use_tuned = g_tuned.load();
  p.use_packed = g_packed.load();
  // how lanes combine channels into groups (kinds 2 and 3)
  p.fwd.group_mode = chop::GROUP_IN_LANE;
  p.fwd.sub = 1;
  p.fwd.run = 1;
  if (d->kind != CHOP_COST_VOLUME) {
    for (int attempt = 0; attempt < 2; ++attempt) {
      const int LG = 1 << lgl;
      const int sub = d->kind == CHOP_COST_VOLUME_V2 ? a.C / a.G : a.C;
      p.fwd.sub = sub;
      bool ok = true;
      if (d->kind == CHOP_COST_VOLUME_V2 && cpl % sub == 0) {
        p.fwd.group_mode = chop::GROUP_IN_LANE;
      } else if (mode == 0 && d->kind == CHOP_COST_AGGREGATE) {
        p.fwd.group_mode = chop::GROUP_XOR;
        p.fwd.run = LG;
      } else if (d->kind == CHOP_COST_AGGREGATE) {
        p.fwd.group_mode = chop::GROUP_ROWS;
      } else if (mode == 0 && sub % cpl == 0 && is_pow2(sub / cpl)) {
        p.fwd.group_mode = chop::GROUP_XOR;
        p.fwd.run = sub / cpl;
      } else {
        p.fwd.group_mode = chop::GROUP_SMEM;
        const int ngroups = d->kind == CHOP_COST_VOLUME_V2 ? a.G : 1;
        ok = ngroups <= LG;
      }
      if (ok) break;
      if (attempt == 1 || cpl == 1) return CHOP_ERR_UNSUPPORTED;
      // one channel per lane always has at least as many lanes as groups
      cpl = 1;
      if (a.C > 32) return CHOP_ERR_UNSUPPORTED;
      lgl = pow2ceil_log2(a.C);
    }
  }
  p.cpl = cpl;
  a.lg_log2 = lgl;
  const int LG = 1 << lgl;
  if (!aligned(ref, cpl * ty.feat_size) || !aligned(src, cpl * ty.feat_size) || !aligned(depth, ty.real_size) ||
      !aligned(cost, (d->kind == CHOP_COST_VOLUME ? cpl : 1) * ty.real_size) || !aligned(mask, 4))
    return CHOP_ERR_ALIGN;
  if (d->kind == CHOP_COST_VOLUME && d->reduce == CHOP_REDUCE_MIN && !aligned(mask, cpl * 4)) return CHOP_ERR_ALIGN;
  if (d->kind == CHOP_COST_VOLUME_V2 && cpl == 4 && tuned_eligible(d, a, false)) {
    // the compile-time-C kernels store the 4/(C/G) groups of a lane's four channels as one vector
    const size_t ga = (size_t)(4 / (a.C / a.G)) * 4;
    if (!aligned(cost, ga) || (d->reduce == CHOP_REDUCE_MIN && !aligned(mask, ga))) return CHOP_ERR_ALIGN;
  }

  plan_chunks(&a, LG, 148 * 128, 16, g_fwd_chunk.load());
  p.fwd.smem_per_warp = ty.real_size == 8
      ? chop::fwd_smem_per_warp<double>(a.N, 32 / LG, LG, cpl, p.fwd.group_mode)
      : chop::fwd_smem_per_warp<float>(a.N, 32 / LG, LG, cpl, p.fwd.group_mode);
  p.fwd.warps = pick_warps(p.fwd.smem_per_warp);
  if (p.fwd.warps == 0) return CHOP_ERR_UNSUPPORTED;
  const long long items = (long long)a.npb * a.nchunks;
  const long long blocks = (items + p.fwd.warps - 1) / p.fwd.warps;
  if (blocks > INT32_MAX) return CHOP_ERR_SHAPE;
  p.blocks = (int)blocks;

  a.ref = ref; a.src = src; a.depth = depth; a.offsets = offsets; a.Rs = Rs; a.Ts = Ts;
  a.cost = cost; a.mask = mask;
  return dispatch_fwd(d->dtype, a, p, static_cast<cudaStream_t>(stream));
}

int chop_cost_volume_bwd(const chop_cv_desc* d, const void* ref, const void* src, const void* depth,
                         const void* offsets, const void* Rs, const void* Ts, const void* cost_grad,
                         const int32_t* mask, void* ref_grad, void* src_grad, void* depth_grad, void* stream) {
  CvArgs a;
  std::memset(&a, 0, sizeof(a));
  Typed ty;
  if (int e = validate(d, &a, &ty)) return e;
  if (!ref || !src || !depth || !Rs || !Ts || !cost_grad || !mask || !ref_grad || !src_grad || !depth_grad)
    return CHOP_ERR_NULL;
  if (d->kind != CHOP_COST_VOLUME_V2 && !offsets) return CHOP_ERR_NULL;
  if (d->kind == CHOP_COST_VOLUME_V3) {
    const size_t fa = ((a.C / a.G) % 4 == 0 ? 4 : 1) * ty.feat_size;
    if (!aligned(ref, ty.feat_size) || !aligned(src, fa) || !aligned(depth, ty.real_size) ||
        !aligned(cost_grad, ty.real_size) || !aligned(mask, 4) || !aligned(ref_grad, ty.real_size) ||
        !aligned(src_grad, ((a.C / a.G) % 4 == 0 ? 4 : 1) * ty.real_size) || !aligned(depth_grad, ty.real_size))
      return CHOP_ERR_ALIGN;
    cudaStream_t st3 = static_cast<cudaStream_t>(stream);
    if (!(d->flags & CHOP_FLAG_ACCUMULATE)) {   // zero fill: cost_volume_kernels_gpu_v3.cu.cc:667-672
      if (int e = zero_fill(ref_grad, (size_t)a.npix * a.C * ty.real_size, src_grad,
                            (size_t)a.B * a.N * a.Hs * a.Ws * a.C * ty.real_size, depth_grad, (size_t)a.npix * ty.real_size, st3))
        return e;
    }
    if (a.d_begin == a.d_end) return CHOP_OK;
    a.lg_log2 = pow2ceil_log2(a.G);
    plan_chunks(&a, 1 << a.lg_log2, 148 * 64, 16, g_bwd_chunk.load());
    a.ref = ref; a.src = src; a.depth = depth; a.offsets = offsets; a.Rs = Rs; a.Ts = Ts;
    a.cost_grad = cost_grad; a.mask = const_cast<int32_t*>(mask);
    a.ref_grad = ref_grad; a.src_grad = src_grad; a.depth_grad = depth_grad;
    return chop::cv3_bwd_launch(d->dtype, d->reduce == CHOP_REDUCE_MIN, a, st3);
  }
  int cpl, lgl;
  if (int e = plan_lanes(d, a, &cpl, &lgl, false, true)) return e;
  a.lg_log2 = lgl;
  const int LG = 1 << lgl;
  if (!aligned(ref, cpl * ty.feat_size) || !aligned(src, cpl * ty.feat_size) || !aligned(depth, ty.real_size) ||
      !aligned(cost_grad, (d->kind == CHOP_COST_VOLUME ? cpl : 1) * ty.real_size) || !aligned(mask, 4) ||
      !aligned(ref_grad, cpl * ty.real_size) || !aligned(src_grad, cpl * ty.real_size) ||
      !aligned(depth_grad, ty.real_size))
    return CHOP_ERR_ALIGN;
  // the compile-time-C MIN kernel copies a lane's four arg indices as one 16-byte vector
  if (d->kind == CHOP_COST_VOLUME && d->reduce == CHOP_REDUCE_MIN && cpl == 4 && !aligned(mask, 16)) return CHOP_ERR_ALIGN;
  if (d->kind == CHOP_COST_VOLUME_V2 && tuned_eligible(d, a, true)) {
    // a lane reads the 4/(C/G) groups of its four channels as one vector
    const size_t ga = (size_t)(4 / (a.C / a.G)) * 4;
    if (!aligned(cost_grad, ga) || !aligned(mask, ga)) return CHOP_ERR_ALIGN;
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!(d->flags & CHOP_FLAG_ACCUMULATE)) {
    // the reference launcher zero-fills the three outputs (cost_volume_kernels_gpu.cu.cc:637-642);
    // the v2 depth gradient is a per-voxel store and needs no fill
    if (int e = zero_fill(ref_grad, (size_t)a.npix * a.C * ty.real_size, src_grad,
                          (size_t)a.B * a.N * a.Hs * a.Ws * a.C * ty.real_size,
                          d->kind != CHOP_COST_VOLUME_V2 ? depth_grad : nullptr, (size_t)a.npix * ty.real_size, st))
      return e;
  }
  if (a.d_begin == a.d_end) return CHOP_OK;

  CvPlan p;
  std::memset(&p, 0, sizeof(p));
  p.kind = d->kind;
  p.cpl = cpl;
  p.use_tuned = g_tuned.load();
  p.use_packed = g_packed.load();
  p.rmin = d->reduce == CHOP_REDUCE_MIN;
  int nv = g_bwd_views.load();
  if (nv <= 0) {
    // accumulator registers grow with views per pass x channels per lane; keep the product modest
    const int cap = cpl >= 8 ? 2 : 4;
    const int passes = (a.N + cap - 1) / cap;
    nv = (a.N + passes - 1) / passes;
  }
  if (nv > 4) nv = 4;
  if (nv > a.N) nv = a.N;
  if (p.rmin) nv = 2;
  p.nv = nv;
  p.bwd.sub = d->kind == CHOP_COST_VOLUME_V2 ? a.C / a.G : 1;
  plan_chunks(&a, LG, 148 * 128, 32, g_bwd_chunk.load());
  p.bwd.smem_per_warp = ty.real_size == 8 ? chop::bwd_smem_per_warp<double>(a.N, 32 / LG, nv)
                                         : chop::bwd_smem_per_warp<float>(a.N, 32 / LG, nv);
  p.bwd.warps = pick_warps(p.bwd.smem_per_warp);
  if (p.bwd.warps == 0) return CHOP_ERR_UNSUPPORTED;
  const long long items = (long long)a.npb * a.nchunks;
  const long long blocks = (items + p.bwd.warps - 1) / p.bwd.warps;
  if (blocks > INT32_MAX) return CHOP_ERR_SHAPE;
  p.blocks = (int)blocks;

  a.ref = ref; a.src = src; a.depth = depth; a.offsets = offsets; a.Rs = Rs; a.Ts = Ts;
  a.cost_grad = cost_grad; a.mask = const_cast<int32_t*>(mask);
  a.ref_grad = ref_grad; a.src_grad = src_grad; a.depth_grad = depth_grad;
  return dispatch_bwd(d->dtype, a, p, st);
}

namespace {
// Shared checks of the two FeatureAggregate entry points; fills the kernel arguments and the lane split.
int fa_prepare(const chop_cv_desc* d, CvArgs* a, Typed* ty, int* cpl) {
  if (!d) return CHOP_ERR_NULL;
  if (int e = typed_of(d->dtype, ty)) return e;
  // FeatureAggregate has no kind / reduce_method / groups: the fields must be left at zero (groups: 0 or 1)
  if (d->kind != 0 || d->reduce != 0 || d->groups < 0 || d->groups > 1) return CHOP_ERR_ATTR;
  if (d->flags & ~CHOP_FLAG_ACCUMULATE) return CHOP_ERR_ATTR;
  const int64_t dims[] = {d->B, d->H, d->W, d->C, d->D, d->N, d->Hs, d->Ws};
  for (int64_t v : dims)
    if (v < 1 || v > INT32_MAX) return CHOP_ERR_SHAPE;
  if (d->Hs < 2 || d->Ws < 2) return CHOP_ERR_SHAPE;
  if (d->B * d->N * d->Hs * d->Ws > INT32_MAX || d->B * d->H * d->W > INT32_MAX || d->B * d->D > INT32_MAX)
    return CHOP_ERR_SHAPE;
  const int64_t d_end = d->d_end == 0 ? d->D : d->d_end;
  if (d->d_begin < 0 || d_end > d->D || d->d_begin > d_end) return CHOP_ERR_RANGE;
  std::memset(a, 0, sizeof(*a));
  a->B = (int)d->B; a->H = (int)d->H; a->W = (int)d->W; a->C = (int)d->C; a->D = (int)d->D;
  a->N = (int)d->N; a->Hs = (int)d->Hs; a->Ws = (int)d->Ws; a->G = 1;
  a->d_begin = (int)d->d_begin; a->d_end = (int)d_end;
  a->half_centor = d->half_centor ? 1 : 0;
  a->npix = d->B * d->H * d->W;
  int c = 1;
  if (d->dtype == CHOP_F64) { if (a->C % 2 == 0) c = 2; }
  else if (a->C % 4 == 0) c = 4;
  const int lanes = (a->C + c - 1) / c;
  if (lanes > 32) return CHOP_ERR_UNSUPPORTED;
  *cpl = c;
  a->lg_log2 = pow2ceil_log2(lanes);
  return 0;
}
}  // namespace

int chop_feature_aggregate_fwd(const chop_cv_desc* d, const void* src, const void* base_plane, const void* offsets,
                               const void* Rs, const void* Ts, void* mapped_feature, int32_t* mapped_mask, void* stream) {
  CvArgs a;
  Typed ty;
  int cpl;
  if (int e = fa_prepare(d, &a, &ty, &cpl)) return e;
  if (!src || !base_plane || !offsets || !Rs || !Ts || !mapped_feature || !mapped_mask) return CHOP_ERR_NULL;
  if (!aligned(src, cpl * ty.feat_size) || !aligned(base_plane, ty.real_size) || !aligned(mapped_feature, cpl * ty.real_size) ||
      !aligned(mapped_mask, 4))
    return CHOP_ERR_ALIGN;
  if (a.d_begin == a.d_end) return CHOP_OK;
  plan_chunks(&a, 1 << a.lg_log2, 148 * 128, 16, g_fwd_chunk.load());
  a.src = src; a.depth = base_plane; a.offsets = offsets; a.Rs = Rs; a.Ts = Ts;
  a.cost = mapped_feature; a.mask = mapped_mask;
  return chop::fa_fwd_launch(d->dtype, cpl, a, static_cast<cudaStream_t>(stream));
}

int chop_feature_aggregate_bwd(const chop_cv_desc* d, const void* src, const void* base_plane, const void* offsets,
                               const void* Rs, const void* Ts, const void* mapped_feature_grad, const int32_t* mapped_mask,
                               void* src_grad, void* base_plane_grad, void* stream) {
  CvArgs a;
  Typed ty;
  int cpl;
  if (int e = fa_prepare(d, &a, &ty, &cpl)) return e;
  if (!src || !base_plane || !offsets || !Rs || !Ts || !mapped_feature_grad || !mapped_mask || !src_grad || !base_plane_grad)
    return CHOP_ERR_NULL;
  if (!aligned(src, cpl * ty.feat_size) || !aligned(base_plane, ty.real_size) ||
      !aligned(mapped_feature_grad, cpl * ty.real_size) || !aligned(mapped_mask, 4) || !aligned(src_grad, cpl * ty.real_size) ||
      !aligned(base_plane_grad, ty.real_size))
    return CHOP_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!(d->flags & CHOP_FLAG_ACCUMULATE)) {
    if (int e = zero_fill(src_grad, (size_t)a.B * a.N * a.Hs * a.Ws * a.C * ty.real_size, base_plane_grad,
                          (size_t)a.npix * ty.real_size, nullptr, 0, st))
      return e;
  }
  if (a.d_begin == a.d_end) return CHOP_OK;
  plan_chunks(&a, 1 << a.lg_log2, 148 * 128, 16, g_bwd_chunk.load());
  a.src = src; a.depth = base_plane; a.offsets = offsets; a.Rs = Rs; a.Ts = Ts;
  a.cost_grad = mapped_feature_grad; a.mask = const_cast<int32_t*>(mapped_mask);
  a.src_grad = src_grad; a.depth_grad = base_plane_grad;
  return chop::fa_bwd_launch(d->dtype, cpl, a, st);
}

int chop_index_initializer(int32_t dtype, int32_t half_centor, int64_t H, int64_t W, void* out, void* stream) {
  if (dtype != CHOP_F32 && dtype != CHOP_F64) return CHOP_ERR_ATTR;
  if (H < 1 || W < 1 || H * W > INT32_MAX / 3) return CHOP_ERR_SHAPE;
  if (!out) return CHOP_ERR_NULL;
  return chop::index_init_launch(dtype, half_centor ? 1 : 0, (int)H, (int)W, out, static_cast<cudaStream_t>(stream));
}

int chop_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                       void* stream) {
  if (!dst || !src) return CHOP_ERR_NULL;
  if (width_bytes == 0 || rows == 0) return CHOP_OK;
  if (dst_pitch < width_bytes || src_pitch < width_bytes) return CHOP_ERR_SHAPE;
  return (int)cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                                static_cast<cudaStream_t>(stream));
}

const char* chop_status_string(int status) {
  switch (status) {
    case CHOP_OK: return "ok";
    case CHOP_ERR_NULL: return "a required pointer is NULL";
    case CHOP_ERR_SHAPE: return "invalid or inconsistent shape";
    case CHOP_ERR_ATTR: return "invalid attribute (kind, dtype, reduce_method or groups)";
    case CHOP_ERR_UNSUPPORTED: return "configuration not supported by this build";
    case CHOP_ERR_ALIGN: return "pointer not aligned for its element type";
    case CHOP_ERR_WORKSPACE: return "workspace missing or too small";
    case CHOP_ERR_RANGE: return "depth range outside [0, D]";
    case CHOP_ERR_FORMAT: return "malformed or unsupported file contents";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown status";
}

int chop_version(void) { return 100; }

int chop_set_tuning(const char* name, int value) {
  if (!name) return CHOP_ERR_NULL;
  // the knobs are process-wide: a test / benchmark facility, refused unless the process opted in
  static const bool enabled = [] { const char* e = std::getenv("CHOP_ENABLE_TUNING"); return e && e[0] == '1'; }();
  if (!enabled) return CHOP_ERR_UNSUPPORTED;
  if (!std::strcmp(name, "fwd_chunk")) { g_fwd_chunk = value; return CHOP_OK; }
  if (!std::strcmp(name, "bwd_chunk")) { g_bwd_chunk = value; return CHOP_OK; }
  if (!std::strcmp(name, "bwd_views")) { g_bwd_views = value; return CHOP_OK; }
  if (!std::strcmp(name, "tuned")) { g_tuned = value; return CHOP_OK; }
  if (!std::strcmp(name, "packed")) { g_packed = value; return CHOP_OK; }
  if (!std::strcmp(name, "umma")) { chop::g_use_umma = value; return CHOP_OK; }
  if (!std::strcmp(name, "umma_rows")) { chop::sc_umma_set_rows(value); return CHOP_OK; }
  if (!std::strcmp(name, "tile")) { chop::g_use_tile = value; return CHOP_OK; }
  if (!std::strcmp(name, "fa_stage")) { chop::g_fa_stage = value; return CHOP_OK; }
  if (!std::strcmp(name, "note_timeout")) return chop::sc_umma_note_timeout_for_test(value);
  return CHOP_ERR_ATTR;
}

}  // extern "C"
