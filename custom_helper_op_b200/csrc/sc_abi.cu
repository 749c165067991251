// extern "C" surface for the manifold 3-D convolution: validation (the checks of
// SparseConv3DFastOpBase::Compute, custom_helper_op/cc/kernels/sparse_conv3d_fast_op.cc:54-146),
// derived extents and padding, kernel selection.
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/chop.h"
#include "sc_common.cuh"
#include "sc_entry.h"

#include <atomic>

namespace chop {
std::atomic<int> g_use_umma{1};  // tuning knob "umma": 0 forces the generic kernels
std::atomic<int> g_use_tile{1};  // tuning knob "tile": 0 = never the register-tiled float32 kernels
}

namespace {

using chop::ScArgs;

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The tensor-core and register-tiled kernels move channel vectors as 16-byte words; a tensor that is not 16-byte
// aligned takes the scalar kernels instead.
int run_fwd(int dtype, const ScArgs& a, cudaStream_t st) {
  if (chop::g_use_umma.load() && chop::sc_umma_supported(dtype, a) && al16(a.images) && al16(a.output) && al16(a.filters))
    return chop::sc_umma_fwd_launch(a, st);
  if (chop::g_use_tile.load() && chop::sc_tile_supported(dtype, a) && al16(a.images) && al16(a.output) && al16(a.filters))
    return chop::sc_tile_fwd_launch(dtype, a, st);
  return chop::sc_fwd_simt_launch(dtype, a, st);
}
int run_wgrad(int dtype, const ScArgs& a, int nparts, cudaStream_t st) {
  if (chop::g_use_umma.load() && chop::sc_umma_supported(dtype, a) && al16(a.images) && al16(a.out_grad) && al16(a.workspace)) {
    // a persistent CTA per partial slab; more CTAs than 128-voxel tiles would leave slabs unwritten
    const long long ntiles = (a.nvox_out + 127) / 128;
    if (nparts > ntiles) nparts = (int)ntiles;
    return chop::sc_umma_wgrad_launch(a, nparts, st);
  }
  if (chop::g_use_tile.load() && chop::sc_tile_wgrad_supported(dtype, a, false) && al16(a.images) && al16(a.out_grad) &&
      al16(a.workspace))
    return chop::sc_tile_wgrad_launch(dtype, a, nparts, st);
  return chop::sc_wgrad_simt_launch_parts(dtype, a, nparts, st);
}
int run_dgrad(int dtype, const ScArgs& in, cudaStream_t st) {
  ScArgs a = in;
  a.pad_zero = 1;  // a padded tap contributes nothing to the image gradient (sparse_conv3d_fast_op.cc:306,321)
  if (chop::g_use_umma.load() && chop::sc_umma_supported(dtype, a) && al16(a.out_grad) && al16(a.images_grad) && al16(a.filters))
    return chop::sc_umma_dgrad_launch(a, st);
  if (chop::g_use_tile.load() && chop::sc_tile_supported(dtype, a) && al16(a.out_grad) && al16(a.images_grad) && al16(a.filters))
    return chop::sc_tile_gather_launch(dtype, a, st);
  return chop::sc_dgrad_simt_launch(dtype, a, st);
}

int fill(const chop_sc_desc* d, ScArgs* a) {
  if (!d) return CHOP_ERR_NULL;
  if (d->dtype < CHOP_F32 || d->dtype > CHOP_BF16) return CHOP_ERR_ATTR;
  const int64_t dims[] = {d->B, d->H, d->W, d->D, d->Cin, d->Cout};
  for (int64_t v : dims)
    if (v < 1 || v > INT32_MAX) return CHOP_ERR_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (d->filter[i] < 1 || d->strides[i] < 1 || d->dilations[i] < 1) return CHOP_ERR_ATTR;
  std::memset(a, 0, sizeof(*a));
  a->B = (int)d->B; a->H = (int)d->H; a->W = (int)d->W; a->D = (int)d->D;
  a->Cin = (int)d->Cin; a->Cout = (int)d->Cout;
  a->fh = d->filter[0]; a->fw = d->filter[1]; a->fd = d->filter[2];
  a->sr = d->strides[0]; a->sc = d->strides[1]; a->sd = d->strides[2];
  a->dr = d->dilations[0]; a->dc = d->dilations[1]; a->dd = d->dilations[2];
  a->oH = (a->H + a->sr - 1) / a->sr;
  a->oW = (a->W + a->sc - 1) / a->sc;
  a->oD = (a->D + a->sd - 1) / a->sd;
  a->pr = a->fh / 2 * a->dr;
  a->pc = a->fw / 2 * a->dc;
  a->pd = a->fd / 2 * a->dd;
  a->dynamic_default = d->dynamic_default ? 1 : 0;
  {
    auto lg = [](int v) { int l = 0; while ((1 << l) < v) ++l; return (1 << l) == v ? l : -1; };
    a->ls_r = lg(a->sr); a->ls_c = lg(a->sc); a->ls_d = lg(a->sd);
    if (a->ls_r < 0 || a->ls_c < 0 || a->ls_d < 0) a->ls_r = a->ls_c = a->ls_d = -1;
  }
  a->nvox_in = d->B * d->H * d->W * d->D;
  a->nvox_out = (long long)a->B * a->oH * a->oW * a->oD;
  // the reference indexes these tensors with int32 (fixed_param_op_gpu.cu.cc:171-174); pixel indices here
  // are int32 too, element offsets 64-bit
  if (d->B * d->H * d->W > INT32_MAX) return CHOP_ERR_SHAPE;
  // rows of the filter matrix (taps x channels) are counted in 32 bits
  if ((int64_t)a->fh * a->fw * a->fd * (a->Cin > a->Cout ? a->Cin : a->Cout) > (1 << 24)) return CHOP_ERR_UNSUPPORTED;
  return 0;
}

// The transposed op's filter gradient gathers the coarse tensor: taps * Cout accumulator rows.
int fill_transpose(const chop_sc_desc* d, ScArgs* a) {
  if (int e = fill(d, a)) return e;
  a->dynamic_default = 0;
  return 0;
}

}  // namespace

extern "C" {

size_t chop_sparse_conv3d_bwd_workspace_size(const chop_sc_desc* d) {
  ScArgs a;
  if (fill(d, &a)) return 0;
  return chop::sc_wgrad_workspace_bytes(d->dtype, a.fh * a.fw * a.fd, a.Cin, a.Cout, a.nvox_out);
}

int chop_sparse_conv3d_fwd(const chop_sc_desc* d, const void* images, const void* filters, const void* default_value,
                           const int32_t* base_plane, void* output, void* stream) {
  ScArgs a;
  if (int e = fill(d, &a)) return e;
  if (!images || !filters || !default_value || !base_plane || !output) return CHOP_ERR_NULL;
  a.images = images; a.filters = filters; a.default_value = default_value; a.base_plane = base_plane;
  a.output = output;
  return run_fwd(d->dtype, a, static_cast<cudaStream_t>(stream));
}

int chop_sparse_conv3d_bwd(const chop_sc_desc* d, const void* images, const void* filters, const void* default_value,
                           const int32_t* base_plane, const void* out_grad, void* images_grad, void* filter_grad,
                           void* default_value_grad, void* workspace, size_t workspace_bytes, void* stream) {
  ScArgs a;
  if (int e = fill(d, &a)) return e;
  if (!images || !filters || !default_value || !base_plane || !out_grad || !images_grad || !filter_grad ||
      !default_value_grad)
    return CHOP_ERR_NULL;
  const size_t need = chop::sc_wgrad_workspace_bytes(d->dtype, a.fh * a.fw * a.fd, a.Cin, a.Cout, a.nvox_out);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return CHOP_ERR_WORKSPACE;
  a.images = images; a.filters = filters; a.default_value = default_value; a.base_plane = base_plane;
  a.out_grad = out_grad; a.images_grad = images_grad; a.filter_grad = filter_grad;
  a.default_grad = default_value_grad; a.workspace = workspace;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int e = run_wgrad(d->dtype, a, chop::sc_wgrad_parts(a.nvox_out), st)) return e;
  return run_dgrad(d->dtype, a, st);
}

// Same gradient as chop_sparse_conv3d_bwd, but the partial filter gradients go to a fixed 4 MiB array
// inside the library instead of a caller workspace, so the call allocates nothing and asks the caller
// for no scratch.  It serves hosts that must not touch the CUDA allocator while they run: a framework
// whose device memory is owned by its own pool (a raw cudaMalloc there fragments the pool's address
// space and synchronises the whole device), or a latency-critical loop with a fixed memory budget.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
//     that first call during set-up, before any stream capture begins.
//   * The number of partial slabs shrinks to what fits; a problem whose single slab
//     ((fh*fw*fd*Cin*Cout + 1) accumulators) exceeds 4 MiB is rejected with CHOP_ERR_WORKSPACE.
//   * All calls on a device share the array.  Nothing in it needs clearing - every slab element that is
//     read was written by the same call - but two calls that overlap on the GPU (different streams)
//     race on it; serialise them.
int chop_sparse_conv3d_bwd_noalloc(const chop_sc_desc* d, const void* images, const void* filters,
                                   const void* default_value, const int32_t* base_plane, const void* out_grad,
                                   void* images_grad, void* filter_grad, void* default_value_grad, void* stream) {
  ScArgs a;
  if (int e = fill(d, &a)) return e;
  if (!images || !filters || !default_value || !base_plane || !out_grad || !images_grad || !filter_grad ||
      !default_value_grad)
    return CHOP_ERR_NULL;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  if (int e = chop::sc_static_scratch(&scratch, &scratch_bytes)) return e;
  const size_t slab = ((size_t)a.fh * a.fw * a.fd * a.Cin * a.Cout + 1) * (d->dtype == CHOP_F64 ? 8 : 4);
  if (slab > scratch_bytes) return CHOP_ERR_WORKSPACE;  // larger than the built-in scratch: use chop_sparse_conv3d_bwd
  int nparts = chop::sc_wgrad_parts(a.nvox_out);
  if ((size_t)nparts * slab > scratch_bytes) nparts = (int)(scratch_bytes / slab);
  a.images = images; a.filters = filters; a.default_value = default_value; a.base_plane = base_plane;
  a.out_grad = out_grad; a.images_grad = images_grad; a.filter_grad = filter_grad;
  a.default_grad = default_value_grad; a.workspace = scratch;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int e = run_wgrad(d->dtype, a, nparts, st)) return e;
  return run_dgrad(d->dtype, a, st);
}

int chop_sparse_conv3d_transpose_fwd(const chop_sc_desc* d, const void* images, const void* filters,
                                     const void* default_value, const int32_t* base_plane, void* output, void* stream) {
  ScArgs a;
  if (int e = fill_transpose(d, &a)) return e;
  if (!images || !filters || !default_value || !base_plane || !output) return CHOP_ERR_NULL;
  // the gather-form kernels name their coarse tensor out_grad and their fine result images_grad
  a.out_grad = images; a.images_grad = output;
  a.filters = filters; a.default_value = default_value; a.base_plane = base_plane;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (chop::g_use_umma.load() && chop::sc_umma_supported(d->dtype, a) && al16(a.out_grad) && al16(a.images_grad) && al16(a.filters))
    return chop::sc_umma_dgrad_launch(a, st);
  if (chop::g_use_tile.load() && chop::sc_tile_supported(d->dtype, a) && al16(a.out_grad) && al16(a.images_grad) && al16(a.filters))
    return chop::sc_tile_gather_launch(d->dtype, a, st);
  return chop::sc_tconv_simt_launch(d->dtype, a, st);
}

size_t chop_sparse_conv3d_transpose_bwd_workspace_size(const chop_sc_desc* d) {
  ScArgs a;
  if (fill_transpose(d, &a)) return 0;
  return chop::sc_wgrad_workspace_bytes(d->dtype, a.fh * a.fw * a.fd, a.Cin, a.Cout, a.nvox_in);
}

int chop_sparse_conv3d_transpose_bwd(const chop_sc_desc* d, const void* images, const void* filters,
                                     const void* default_value, const int32_t* base_plane, const void* out_grad,
                                     void* images_grad, void* filter_grad, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  ScArgs a;
  if (int e = fill_transpose(d, &a)) return e;
  if (!images || !filters || !default_value || !base_plane || !out_grad || !images_grad || !filter_grad)
    return CHOP_ERR_NULL;
  const size_t need = chop::sc_wgrad_workspace_bytes(d->dtype, a.fh * a.fw * a.fd, a.Cin, a.Cout, a.nvox_in);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return CHOP_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  a.filters = filters; a.default_value = default_value; a.base_plane = base_plane;
  // filter gradient: gathers the coarse input under every tap of every fine voxel
  a.images = images; a.out_grad = out_grad; a.filter_grad = filter_grad; a.workspace = workspace;
  const int nparts = chop::sc_wgrad_parts(a.nvox_in);
  if (chop::g_use_umma.load() && chop::sc_umma_supported(d->dtype, a) && al16(a.images) && al16(a.out_grad) && al16(a.workspace)) {
    if (int e = chop::sc_umma_twgrad_launch(a, nparts, st)) return e;
  } else if (chop::g_use_tile.load() && chop::sc_tile_wgrad_supported(d->dtype, a, true) && al16(a.images) && al16(a.out_grad) &&
             al16(a.workspace)) {
    if (int e = chop::sc_tile_twgrad_launch(d->dtype, a, nparts, st)) return e;
  } else {
    if (int e = chop::sc_twgrad_simt_launch(d->dtype, a, nparts, st)) return e;
  }
  // image gradient: the forward convolution of out_grad (fine, Cin channels) with the same filter, a padded tap
  // contributing nothing
  a.images = out_grad; a.output = images_grad; a.out_grad = nullptr; a.pad_zero = 1;
  return run_fwd(d->dtype, a, st);
}

namespace {
int pad_check(int32_t dtype, int64_t B, int64_t h, int64_t w, int64_t d, int64_t C, const int32_t* s) {
  if (dtype < CHOP_F32 || dtype > CHOP_BF16) return CHOP_ERR_ATTR;
  if (!s) return CHOP_ERR_NULL;
  if (s[0] < 1 || s[1] < 1 || s[2] < 1) return CHOP_ERR_ATTR;
  if (B < 1 || h < 1 || w < 1 || d < 1 || C < 1) return CHOP_ERR_SHAPE;
  if (B * h * s[0] * w * s[1] > INT32_MAX || d * s[2] > INT32_MAX || C > INT32_MAX) return CHOP_ERR_SHAPE;
  return 0;
}
}  // namespace

int chop_sparse_pad_fwd(int32_t dtype, int64_t B, int64_t h, int64_t w, int64_t d, int64_t C, const int32_t strides[3],
                        const void* images, const int32_t* base_plane, void* output, void* stream) {
  if (int e = pad_check(dtype, B, h, w, d, C, strides)) return e;
  if (!images || !base_plane || !output) return CHOP_ERR_NULL;
  return chop::sc_pad_launch(dtype, false, images, base_plane, output, (int)B, (int)h, (int)w, (int)d, (int)C, strides[0],
                             strides[1], strides[2], static_cast<cudaStream_t>(stream));
}

int chop_sparse_pad_bwd(int32_t dtype, int64_t B, int64_t h, int64_t w, int64_t d, int64_t C, const int32_t strides[3],
                        const int32_t* base_plane, const void* out_grad, void* images_grad, void* stream) {
  if (int e = pad_check(dtype, B, h, w, d, C, strides)) return e;
  if (!out_grad || !base_plane || !images_grad) return CHOP_ERR_NULL;
  return chop::sc_pad_launch(dtype, true, out_grad, base_plane, images_grad, (int)B, (int)h, (int)w, (int)d, (int)C,
                             strides[0], strides[1], strides[2], static_cast<cudaStream_t>(stream));
}

int chop_umma_timeouts(void) { return chop::sc_umma_timeouts(); }
int chop_umma_watch(void) { return chop::sc_umma_watch(); }

}  // extern "C"
