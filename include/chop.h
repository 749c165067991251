/* chop.h - C ABI of libchop_b200.so: plane-sweep cost volume (+ gradient) and manifold 3-D
 * convolution for NVIDIA B200 (sm_100a).
 *
 * The entry points sit exactly where the reference project's TensorFlow OpKernels call their
 * device functors: the caller (an OpKernel, a torch wrapper, a cgo/ctypes stub ...) validates
 * nothing, owns every buffer, and passes raw DEVICE pointers plus a CUDA stream.  The library
 *   - allocates nothing (device or host memory) and keeps no state between calls, with these exceptions,
 *     all process-wide and none of them visible in results:
 *       . a table of which kernels have been granted more than 48 KB of dynamic shared memory on which
 *         device (the opt-in attribute is set the first time a launch needs it, not on every call);
 *       . chop_umma_timeouts(): a device-side counter of bounded waits that gave up (see below), and - only
 *         after a call of chop_umma_watch() - one int of pinned host memory that mirrors it;
 *       . the 4 MiB device array behind chop_sparse_conv3d_bwd_noalloc and its per-device address;
 *       . the test / benchmark knobs of chop_set_tuning, inert unless the process sets
 *         CHOP_ENABLE_TUNING=1 in its environment before the first call,
 *   - enqueues all work on the given stream and never synchronises,
 *   - returns 0 on success, a negative chop_status for an invalid argument detected on the host
 *     before any launch, or a positive cudaError_t value if a launch failed,
 *   - never aborts and never throws across the boundary; it is re-entrant and thread-safe.
 * There is no CPU fallback: without a CUDA device every compute entry point fails.
 *
 * Tensor layouts are the reference's (row-major, channels last):
 *   ref [B,H,W,C]   src [B,N,Hs,Ws,C]   Rs [B,N,3,3]   Ts [B,N,3]
 *   CostVolume   : base_plane [B,H,W,1], offsets [B,D]   -> cost [B,H,W,D,C], mask [B,H,W,D,1|C]
 *   CostVolumeV2 : depth_grid [B,H,W,D]                  -> cost [B,H,W,D,G], mask [B,H,W,D,1|G]
 *   CostAggregate: base_plane, offsets                   -> cost [B,H,W,D],   mask [B,H,W,D]
 *   CostVolumeV3 : base_plane, offsets                   -> cost [B,H,W,D,1], mask [B,H,W,D,1|3]
 * (mask is int32; its last dimension is 1 for MEAN and C|G for MIN; for CostVolumeV3 MIN it holds the
 * winning (view, reference group, source group)).
 */
#ifndef CHOP_H_
#define CHOP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CHOP_API __attribute__((visibility("default")))
#else
#define CHOP_API
#endif

typedef enum chop_status {
  CHOP_OK = 0,
  CHOP_ERR_NULL = -1,         /* a required pointer is NULL */
  CHOP_ERR_SHAPE = -2,        /* a dimension is < 1, inconsistent, or too large for 32-bit texel indices */
  CHOP_ERR_ATTR = -3,         /* unknown kind / dtype / reduce method, groups does not divide C ... */
  CHOP_ERR_UNSUPPORTED = -4,  /* valid for the reference but not implemented here */
  CHOP_ERR_ALIGN = -5,        /* a pointer is not aligned for the element type */
  CHOP_ERR_WORKSPACE = -6,    /* workspace missing or too small */
  CHOP_ERR_RANGE = -7,        /* depth range outside [0, D] */
  CHOP_ERR_FORMAT = -8        /* chop_decode_pfm: malformed or unsupported file contents */
} chop_status;

typedef enum chop_dtype {
  CHOP_F32 = 0,  /* everything float32 (reference dtype) */
  CHOP_F64 = 1,  /* everything float64 (reference dtype) */
  CHOP_BF16 = 2  /* ref/src (cost volume) or images/filters (conv) in bfloat16; depths, cameras,
                    cost, upstream gradients and all gradient outputs float32 (superset of the
                    reference, which accepts float32/float64 only) */
} chop_dtype;

typedef enum chop_kind {
  CHOP_COST_VOLUME = 1,    /* op CostVolume / CostVolumeGrad */
  CHOP_COST_VOLUME_V2 = 2, /* op CostVolumeV2 / CostVolumeGradV2 */
  CHOP_COST_AGGREGATE = 3, /* op CostAggregate / CostAggregateGrad */
  CHOP_COST_VOLUME_V3 = 4  /* op CostVolumeV3 / CostVolumeGradV3 (cost_volume_kernels_v3.cc:57-150,
                              cost_volume_kernels_gpu_v3.cu.cc): largest group-pair correlation; needs
                              C % groups == 0 and C / groups <= 8.  Depth-range fields are honoured;
                              CHOP_FLAG_STRICT is implied (the arithmetic is always the unfused one). */
} chop_kind;

typedef enum chop_reduce { CHOP_REDUCE_MEAN = 0, CHOP_REDUCE_MIN = 1 } chop_reduce;

/* flags */
#define CHOP_FLAG_STRICT 1u     /* forward: every floating operation is the single correctly rounded IEEE
                                   operation of the reference source, in source order (no fused
                                   multiply-add), so cost is reproducible bit for bit.  MIN always runs
                                   this way because its arg-indices must be exact. */
#define CHOP_FLAG_ACCUMULATE 2u /* backward: add into ref_grad/src_grad/base_plane_grad instead of
                                   zero-filling them first (used when a batch item is split by depth
                                   range over several calls). */
/* Any other bit set in chop_cv_desc.flags is rejected with CHOP_ERR_ATTR. */

/* Describes one cost-volume call.  Replaces the scalar argument list of the reference functors
 * CostVolumeFunctor / CostVolumeGradFunctor (custom_helper_op/cc/kernels/cost_volume.h:37-132) and
 * their v2 / aggregate twins (cost_volume_v2.h, cost_aggregate.h). */
typedef struct chop_cv_desc {
  int32_t kind;        /* chop_kind */
  int32_t dtype;       /* chop_dtype */
  int32_t reduce;      /* chop_reduce; attr reduce_method */
  int32_t half_centor; /* attr half_centor (pixel centres at +0.5) */
  int32_t groups;      /* attr groups (CostVolumeV2 / CostVolumeV3; must divide C) */
  uint32_t flags;
  int64_t B, H, W, C;  /* ref image */
  int64_t D;           /* depth hypotheses = extent of every D-indexed tensor passed in */
  int64_t N, Hs, Ws;   /* source views */
  int64_t d_begin;     /* process depth planes [d_begin, d_end) only; d_end == 0 means D.  Planes */
  int64_t d_end;       /* outside the range are neither read nor written.                         */
} chop_cv_desc;

/* Forward.  Replaces CostVolumeFunctor<GPUDevice,T,half_centor>::operator()
 * (custom_helper_op/cc/kernels/cost_volume_kernels_gpu.cu.cc:289-335), CostVolumeV2Functor
 * (cost_volume_kernels_gpu_v2.cu.cc:296-342) and CostAggregateFunctor.
 * depth = base_plane (kinds 1,3) or depth_grid (kind 2); offsets is NULL for kind 2. */
CHOP_API int chop_cost_volume_fwd(const chop_cv_desc *desc, const void *ref, const void *src, const void *depth,
                         const void *offsets, const void *Rs, const void *Ts, void *cost, int32_t *mask,
                         void *stream);

/* Gradient.  Replaces CostVolumeGradFunctor::operator() including its zero fill of the outputs
 * (cost_volume_kernels_gpu.cu.cc:590-655; v2 :614-679).  depth_grad has the shape of `depth`.
 * There is no gradient for offsets, Rs, Ts (custom_helper_op/python/ops/custom_helper_ops.py:61). */
CHOP_API int chop_cost_volume_bwd(const chop_cv_desc *desc, const void *ref, const void *src, const void *depth,
                         const void *offsets, const void *Rs, const void *Ts, const void *cost_grad,
                         const int32_t *mask, void *ref_grad, void *src_grad, void *depth_grad,
                         void *stream);

/* Describes one manifold ("sparse") 3-D convolution call.  Replaces the reference's SparseConv3DFastParams
 * (custom_helper_op/cc/kernels/sparse_conv3d_fast_op.h:26-49); output extents are ceil(input/stride) and
 * the left padding is (filter/2)*dilation as in sparse_conv3d_fast_op.cc:104-109.
 *   images [B,H,W,D,Cin]  filters [fh,fw,fd,Cin,Cout]  default_value: DEVICE scalar  base_plane int32 [B,H,W,1]
 *   output / out_grad [B,ceil(H/sr),ceil(W/sc),ceil(D/sd),Cout]
 * dtype CHOP_BF16: images, filters, default_value, output, out_grad and images_grad are bfloat16;
 * filter_grad and default_value_grad are float32. */
typedef struct chop_sc_desc {
  int32_t dtype;           /* chop_dtype */
  int32_t dynamic_default; /* attr dynamic_default: also produce d(default_value) */
  int64_t B, H, W, D, Cin, Cout;
  int32_t filter[3];       /* fh, fw, fd */
  int32_t strides[3];      /* attr strides */
  int32_t dilations[3];    /* attr dilations */
  int32_t reserved;
} chop_sc_desc;

/* Scratch bytes the backward call needs (per-CTA partial filter gradients, summed in a fixed order so
 * the result is deterministic).  The forward call needs none. */
CHOP_API size_t chop_sparse_conv3d_bwd_workspace_size(const chop_sc_desc *desc);

/* Forward.  Replaces SparseConv3DFastFunctor<GPUDevice,T,true>::operator() together with the filter
 * transpose the reference launches before it (sparse_conv3d_fast_op.cc:186-201). */
CHOP_API int chop_sparse_conv3d_fwd(const chop_sc_desc *desc, const void *images, const void *filters,
                                    const void *default_value, const int32_t *base_plane, void *output,
                                    void *stream);

/* Gradient.  Replaces SparseConv3DFastGradOp::Compute's device work (sparse_conv3d_fast_op.cc:232-325):
 * filter gradient, default-value gradient (zero unless dynamic_default) and image gradient.  workspace:
 * caller-owned device memory of at least chop_sparse_conv3d_bwd_workspace_size() bytes, 16-byte aligned. */
CHOP_API int chop_sparse_conv3d_bwd(const chop_sc_desc *desc, const void *images, const void *filters,
                                    const void *default_value, const int32_t *base_plane, const void *out_grad,
                                    void *images_grad, void *filter_grad, void *default_value_grad,
                                    void *workspace, size_t workspace_bytes, void *stream);

/* No counterpart in the reference.  chop_sparse_conv3d_bwd without the workspace argument: the partial
 * filter gradients are kept in a fixed 4 MiB device array inside the library, so the call allocates
 * nothing and needs no scratch from the caller.  For hosts that may not call the CUDA allocator where
 * this runs - their device memory belongs to a framework pool, or the loop has a fixed memory budget and
 * cannot afford the device-wide synchronisation of cudaMalloc.  Limits: one partial slab
 * ((fh*fw*fd*Cin*Cout + 1) accumulators of 4 bytes, 8 for float64) must fit in 4 MiB, else
 * CHOP_ERR_WORKSPACE; the first call on a device resolves the array's address and should happen during
 * set-up, before any stream capture; calls that overlap on one GPU race on the shared array. */
CHOP_API int chop_sparse_conv3d_bwd_noalloc(const chop_sc_desc *desc, const void *images, const void *filters,
                                            const void *default_value, const int32_t *base_plane,
                                            const void *out_grad, void *images_grad, void *filter_grad,
                                            void *default_value_grad, void *stream);

/* ---- transposed manifold convolution -------------------------------------------------------------------
 * SparseConv3DTransposeFast / SparseConv3DTransposeFastGrad (custom_helper_op/cc/kernels/
 * sparse_conv3d_fast_op.cc:346-411, 427-505; schema cc/ops/custom_helper_ops.cc:644-715).  desc describes the
 * forward convolution whose transpose is taken, exactly as the reference derives it from its inputs
 * (sparse_conv3d_fast_op.cc:78-146): (H,W,D) = the op's output_size, the FINE grid that base_plane
 * [B,H,W,1] describes; the op's input `images` is the COARSE grid [B,ceil(H/sr),ceil(W/sc),ceil(D/sd),Cout];
 * filters [fh,fw,fd,Cin,Cout]; output [B,H,W,D,Cin].  Every fine voxel sums, over the taps of the flipped
 * filter, the coarse voxel lying exactly under the tap, or default_value where there is none.
 * desc->dynamic_default is ignored (the reference produces no default-value gradient for this op). */
CHOP_API int chop_sparse_conv3d_transpose_fwd(const chop_sc_desc *desc, const void *images, const void *filters,
                                              const void *default_value, const int32_t *base_plane, void *output,
                                              void *stream);

CHOP_API size_t chop_sparse_conv3d_transpose_bwd_workspace_size(const chop_sc_desc *desc);

/* Gradient of the transposed convolution: images_grad [B,oH,oW,oD,Cout], filter_grad [fh,fw,fd,Cin,Cout]
 * (float32 for bfloat16 data).  Both are the derivatives of the forward entry point.  The reference's grad
 * op differs from them in two places, neither reachable from its own layer (which fixes default_value to a
 * non-trainable 0 and Cin/Cout by construction): it adds default_value times the filter at padded taps to
 * images_grad (sparse_conv3d_fast_op.cc:495-500), and it leaves the two channel axes of filter_grad in the
 * order [Cout, Cin] (:477-488 only reverses the spatial axes of the swapped problem's result). */
CHOP_API int chop_sparse_conv3d_transpose_bwd(const chop_sc_desc *desc, const void *images, const void *filters,
                                              const void *default_value, const int32_t *base_plane,
                                              const void *out_grad, void *images_grad, void *filter_grad,
                                              void *workspace, size_t workspace_bytes, void *stream);

/* SparsePad / SparsePadGrad (custom_helper_op/cc/kernels/sparse_pad_kernels.cc:76-130, 150-210; kernels
 * sparse_pad_kernels_gpu.cu.cc:36-64, 82-104).  images [B,h,w,d,C] (coarse band) -> output
 * [B,h*sr,w*sc,d*sd,C]; base_plane [B,h*sr,w*sc,1] is the fine band's first plane per pixel.  The gradient
 * entry reads, for every coarse voxel, the fine voxel the forward wrote it to (the reference's kernel
 * addresses the fine pixel by the unscaled coarse row/column and is only right for sr = sc = 1). */
CHOP_API int chop_sparse_pad_fwd(int32_t dtype, int64_t B, int64_t h, int64_t w, int64_t d, int64_t C,
                                 const int32_t strides[3], const void *images, const int32_t *base_plane,
                                 void *output, void *stream);
CHOP_API int chop_sparse_pad_bwd(int32_t dtype, int64_t B, int64_t h, int64_t w, int64_t d, int64_t C,
                                 const int32_t strides[3], const int32_t *base_plane, const void *out_grad,
                                 void *images_grad, void *stream);

/* ---- FeatureAggregate / IndexInitializer / DecodePfm -----------------------------------------------------
 * FeatureAggregate(Grad) (custom_helper_op/cc/kernels/feature_aggregate_kernels.cc:60-130,170-250; kernels
 * feature_aggregate_kernels_gpu.cu.cc:33-121,219-317): the plane-sweep warp without a reduction.
 *   src [B,N,Hs,Ws,C], base_plane [B,H,W,1], offsets [B,D], Rs, Ts ->
 *   mapped_feature [B,H,W,D,N,C] (zeros where a view does not see the voxel), mapped_mask int32 [B,H,W,D,N,1].
 * desc: kind and reduce must be 0 and groups 0 or 1 (the op has none of these attributes; anything else is
 * CHOP_ERR_ATTR); (H,W) is the output grid and may differ from (Hs,Ws); the depth range fields and
 * CHOP_FLAG_ACCUMULATE (gradient) are honoured, any other flag bit is CHOP_ERR_ATTR.  Gradient outputs: src_grad like src,
 * base_plane_grad like base_plane, zero-filled first as the reference functor does (:337-383). */
CHOP_API int chop_feature_aggregate_fwd(const chop_cv_desc *desc, const void *src, const void *base_plane,
                                        const void *offsets, const void *Rs, const void *Ts, void *mapped_feature,
                                        int32_t *mapped_mask, void *stream);
CHOP_API int chop_feature_aggregate_bwd(const chop_cv_desc *desc, const void *src, const void *base_plane,
                                        const void *offsets, const void *Rs, const void *Ts,
                                        const void *mapped_feature_grad, const int32_t *mapped_mask, void *src_grad,
                                        void *base_plane_grad, void *stream);

/* IndexInitializer (index_initializer_kernels.cc:60-100, index_initializer_kernels_gpu.cu.cc:21-29):
 * out [H,W,3] = (column, row, 1), the first two plus 0.5 when half_centor.  dtype CHOP_F32 or CHOP_F64. */
CHOP_API int chop_index_initializer(int32_t dtype, int32_t half_centor, int64_t H, int64_t W, void *out, void *stream);

/* DecodePfm (pfm_decoder_kernels.cc:38-116), a HOST function: parses the header of a PFM file held in memory and,
 * when image != NULL, copies the single-channel little-endian payload into image [height,width,1] (host memory,
 * image_capacity floats) with the rows flipped.  Call once with image == NULL to learn the shape.  Errors are those
 * of the reference (magic other than Pf/PF, missing field, big-endian scale, colour format "PF" not implemented,
 * too little data, a comment line after the magic): CHOP_ERR_FORMAT with the reference's message in msg. */
CHOP_API int chop_decode_pfm(const void *contents, size_t size, int64_t *height, int64_t *width, int64_t *channels,
                             float *image, size_t image_capacity, char *msg, size_t msg_capacity);

/* Diagnostic: how many times a tensor-core convolution kernel gave up waiting for its MMAs since the
 * library was loaded (0 in a healthy run; the affected call's output is then incomplete).  Copies one
 * int from the device, so it synchronises with the current device; -1 if that copy fails. */
CHOP_API int chop_umma_timeouts(void);

/* The same count without touching the device, for hosts that must not synchronise (a framework op, a serving loop):
 * the kernels also bump a mapped, pinned host int once this function has published it to the current device.  The
 * first call in a process allocates that int (4 bytes, cudaHostAlloc) and the first call per device copies its address
 * to the device - those calls synchronise; every later call only reads host memory.  Give-ups on a device before its
 * first call are not in the count, and a bump becomes visible when the kernel that made it has written it through,
 * at the latest when that kernel ends: a caller polls before its NEXT call, or after its own synchronisation point.
 * No compute entry point calls this by itself (they allocate nothing).  -1 if the mirror cannot be set up. */
CHOP_API int chop_umma_watch(void);

/* Strided host<->device copy of a depth range: `rows` rows of `width_bytes` bytes, row pitches given
 * (cudaMemcpy2DAsync with cudaMemcpyDefault).  A [d0,d1) slice of a [...,D,C] tensor is rows = B*H*W,
 * width = (d1-d0)*C*elem, pitch = D*C*elem.  Used by hosts that stream cost / cost_grad between pinned
 * host memory and the device chunk by chunk while the kernels run on another stream. */
CHOP_API int chop_copy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes,
                                size_t rows, void *stream);

/* Text for a status returned by any entry point (negative: chop_status, positive: CUDA). */
CHOP_API const char *chop_status_string(int status);

/* Library version as major*10000 + minor*100 + patch. */
CHOP_API int chop_version(void);

/* Tuning knobs for experiments: "fwd_chunk", "bwd_chunk" (depth planes per warp work item, 0 =
 * heuristic), "bwd_views" (source views per backward pass, 0 = heuristic), "tuned" (1 = use the compile-time-C
 * kernels where one exists, 0 = always the generic kernels), "umma" (1 = tensor-core manifold convolution
 * where supported, 0 = always the generic kernels), "umma_rows" (1 = the stride-1 tensor-core forward / image
 * gradient stages one copy per neighbour pixel, 0 = one per tap), "tile" (1 = register-tiled float32 manifold
 * convolution kernels where supported, 0 = the one-thread-per-element kernels), "packed" (1 = the packed-pair CostVolume
 * MEAN kernels where one exists, 0 = the previous compile-time-C kernels), "fa_stage" (1 = FeatureAggregateGrad copies
 * its upstream tensor into shared memory a block of planes ahead where the channel count allows, 0 = never), "note_timeout" (1 = launch a one-thread
 * kernel that performs the bookkeeping of an abandoned tensor-core wait, without any wait; 0 = clear the counter of
 * the current device and its host mirror).  Returns CHOP_ERR_ATTR for an unknown name.
 * Process-wide, hence a facility for tests and benchmarks only: every call returns CHOP_ERR_UNSUPPORTED unless the
 * process has CHOP_ENABLE_TUNING=1 in its environment (read once, at the first call); a production host never sets it
 * and always gets the default kernel selection.  Not part of the reference surface. */
CHOP_API int chop_set_tuning(const char *name, int value);

#ifdef __cplusplus
}
#endif
#endif /* CHOP_H_ */
