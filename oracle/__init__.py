"""TEST INFRASTRUCTURE ONLY - the CPU oracle for the cost-volume / manifold-conv path.

Two implementations sit behind the same numpy interface:

* ``impl="port"``: ``libchop_oracle.so``, the plain-C restatement in ``chop_oracle.c`` (always
  available; built on first use with gcc).
* ``impl="ref"``: ``_ref/libchop_ref.so``, the reference's own kernel bodies compiled as host
  C++ by ``build_ref.py`` (available wherever that script ran with the reference checkout present;
  the built library is carried along, the reference sources are not).

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this package.
The shipped library (``custom_helper_op_b200``) never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = os.path.join(_HERE, "libchop_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libchop_ref.so")

KIND_V1, KIND_V2, KIND_AGG, KIND_V3 = 1, 2, 3, 4
_libs = {}


def build_port(force=False):
    """Compile the plain-C restatement (a couple of seconds)."""
    srcs = [os.path.join(_HERE, f) for f in ("chop_oracle.c", "chop_oracle_impl.h", "sparse_oracle.c")]
    srcs = [s for s in srcs if os.path.exists(s)]
    if not force and os.path.exists(_PORT) and all(
            os.path.getmtime(_PORT) >= os.path.getmtime(s) for s in srcs):
        return _PORT
    cs = [s for s in srcs if s.endswith(".c")]
    cmd = ["gcc", "-O3", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-Wall",
           "-Wno-unused-function"] + cs + ["-o", _PORT, "-lm"]
    subprocess.check_call(cmd)
    return _PORT


def have_ref():
    return os.path.exists(_REF)


def _lib(impl):
    if impl not in _libs:
        if impl == "port":
            _libs[impl] = ctypes.CDLL(build_port())
        elif impl == "ref":
            if not have_ref():
                raise FileNotFoundError("oracle/_ref/libchop_ref.so not built (run oracle/build_ref.py "
                                        "where the reference checkout is present)")
            _libs[impl] = ctypes.CDLL(_REF)
        else:
            raise ValueError(impl)
    return _libs[impl]


def max_threads():
    return os.cpu_count() or 1


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _prep(dtype, *arrs):
    return [None if a is None else np.ascontiguousarray(a, dtype=dtype) for a in arrs]


def _dims(ref, src, D):
    B, H, W, C = ref.shape
    N, Hs, Ws = src.shape[1], src.shape[2], src.shape[3]
    return (ctypes.c_int64 * 8)(B, H, W, C, D, N, Hs, Ws)


def cost_fwd(kind, ref, src, depth, offsets, Rs, Ts, reduce_method="MEAN", groups=1, half_centor=True,
             dtype=np.float32, impl="port", nthreads=None):
    """Forward of CostVolume (kind 1), CostVolumeV2 (kind 2), CostAggregate (kind 3) or CostVolumeV3
    (kind 4: cost [B,H,W,D,1]; mask [B,H,W,D,1] for MEAN, [B,H,W,D,3] = (view, ref group, src group) for MIN).

    ``depth`` is base_plane [B,H,W,1] for kinds 1/3 and depth_grid [B,H,W,D] for kind 2 (offsets
    None).  Returns (cost, mask) shaped like the reference op's outputs."""
    dtype = np.dtype(dtype)
    ref, src, depth, offsets, Rs, Ts = _prep(dtype, ref, src, depth, offsets, Rs, Ts)
    B, H, W, C = ref.shape
    D = depth.shape[3] if kind == KIND_V2 else offsets.shape[1]
    rmin = int(reduce_method == "MIN")
    CO = C if kind == KIND_V1 else (groups if kind == KIND_V2 else 1)
    cost = np.empty((B, H, W, D, CO), dtype)
    mask = np.empty((B, H, W, D, (3 if kind == KIND_V3 else CO) if rmin else 1), np.int32)
    nt = nthreads if nthreads is not None else max_threads()
    fn = _lib(impl).oracle_cost_fwd if impl == "port" else _lib(impl).ref_cost_fwd
    fn(ctypes.c_int(kind), ctypes.c_int(0 if dtype == np.float32 else 1), ctypes.c_int(rmin),
       ctypes.c_int(int(half_centor)), _dims(ref, src, D), ctypes.c_int(int(groups)), _p(ref), _p(src),
       _p(depth), _p(offsets), _p(Rs), _p(Ts), _p(cost), _p(mask), ctypes.c_int(nt))
    if kind == KIND_AGG:
        cost = cost.reshape(B, H, W, D)
        mask = mask.reshape(B, H, W, D)
    return cost, mask


def cost_bwd(kind, ref, src, depth, offsets, Rs, Ts, cost_grad, mask, reduce_method="MEAN", groups=1,
             half_centor=True, dtype=np.float32, impl="port", nthreads=1):
    """Gradient op.  Returns (ref_grad, src_grad, depth_grad) where depth_grad has the shape of
    base_plane (kinds 1/3) or depth_grid (kind 2).  nthreads=1 gives reproducible sums."""
    dtype = np.dtype(dtype)
    ref, src, depth, offsets, Rs, Ts, cost_grad = _prep(dtype, ref, src, depth, offsets, Rs, Ts, cost_grad)
    mask = np.ascontiguousarray(mask, np.int32)
    D = depth.shape[3] if kind == KIND_V2 else offsets.shape[1]
    rmin = int(reduce_method == "MIN")
    ref_grad = np.empty_like(ref)
    src_grad = np.empty_like(src)
    depth_grad = np.empty_like(depth)
    fn = _lib(impl).oracle_cost_bwd if impl == "port" else _lib(impl).ref_cost_bwd
    fn(ctypes.c_int(kind), ctypes.c_int(0 if dtype == np.float32 else 1), ctypes.c_int(rmin),
       ctypes.c_int(int(half_centor)), _dims(ref, src, D), ctypes.c_int(int(groups)), _p(ref), _p(src),
       _p(depth), _p(offsets), _p(Rs), _p(Ts), _p(cost_grad), _p(mask), _p(ref_grad), _p(src_grad),
       _p(depth_grad), ctypes.c_int(nthreads))
    return ref_grad, src_grad, depth_grad


# ---- manifold 3-D convolution -------------------------------------------------------------------------
def _sc_params(images, filters, strides, dilations):
    B, H, W, D, Cin = images.shape
    fh, fw, fd, Cin2, Cout = filters.shape
    assert Cin == Cin2
    p = (ctypes.c_int * 15)(B, H, W, D, Cin, Cout, fh, fw, fd, *[int(x) for x in strides], *[int(x) for x in dilations])
    out_shape = (B, (H + strides[0] - 1) // strides[0], (W + strides[1] - 1) // strides[1],
                 (D + strides[2] - 1) // strides[2], Cout)
    return p, out_shape


def sparse_conv3d_fwd(images, filters, default_value, base_plane, strides=(1, 1, 1), dilations=(1, 1, 1),
                      dtype=np.float32, impl="port", nthreads=None):
    """SparseConv3DFast forward.  impl="ref" runs the reference's older thread-per-voxel kernel compiled as
    host code (same semantics for the forward pass)."""
    dtype = np.dtype(dtype)
    images, filters = _prep(dtype, images, filters)
    base_plane = np.ascontiguousarray(base_plane, np.int32)
    defv = np.asarray(default_value, dtype).reshape(1)
    p, out_shape = _sc_params(images, filters, strides, dilations)
    out = np.empty(out_shape, dtype)
    nt = nthreads if nthreads is not None else max_threads()
    if impl == "port":
        rc = _lib("port").oracle_sparse_conv3d_fwd(ctypes.c_int(0 if dtype == np.float32 else 1), p, _p(images),
                                                   _p(filters), _p(defv), _p(base_plane), _p(out), ctypes.c_int(nt))
        assert rc == 0
    else:
        B, H, W, D, Cin = images.shape
        fh, fw, fd, _, Cout = filters.shape
        q = (ctypes.c_int * 18)(*[int(x) for x in strides], *[int(x) for x in dilations], fh, fw, fd, B, H, W, D, Cin,
                                out_shape[1], out_shape[2], out_shape[3], Cout)
        _lib("ref").ref_sparse_conv3d_fwd(ctypes.c_int(0 if dtype == np.float32 else 1), q, _p(images), _p(filters),
                                          _p(defv), _p(base_plane), _p(out), ctypes.c_int(nt))
    return out


def sparse_conv3d_bwd(images, filters, default_value, base_plane, out_grad, strides=(1, 1, 1), dilations=(1, 1, 1),
                      dynamic_default=False, dtype=np.float32, nthreads=None):
    """SparseConv3DFastGrad: returns (images_grad, filter_grad, default_value_grad)."""
    dtype = np.dtype(dtype)
    images, filters, out_grad = _prep(dtype, images, filters, out_grad)
    base_plane = np.ascontiguousarray(base_plane, np.int32)
    defv = np.asarray(default_value, dtype).reshape(1)
    p, out_shape = _sc_params(images, filters, strides, dilations)
    assert tuple(out_grad.shape) == out_shape
    igrad = np.empty_like(images)
    fgrad = np.empty_like(filters)
    dgrad = np.zeros(1, dtype)
    nt = nthreads if nthreads is not None else max_threads()
    rc = _lib("port").oracle_sparse_conv3d_bwd(ctypes.c_int(0 if dtype == np.float32 else 1), p, _p(images), _p(filters),
                                               _p(defv), _p(base_plane), _p(out_grad), ctypes.c_int(int(dynamic_default)),
                                               _p(igrad), _p(fgrad), _p(dgrad), ctypes.c_int(nt))
    assert rc == 0
    return igrad, fgrad, dgrad.reshape(())


def sparse_conv3d_transpose_fwd(images, filters, default_value, base_plane, output_size, strides=(1, 1, 1),
                                dilations=(1, 1, 1), dtype=np.float32, nthreads=None):
    """SparseConv3DTransposeFast forward: images [B,oH,oW,oD,Cout] (coarse), filters [fh,fw,fd,Cin,Cout],
    base_plane [B,H,W,1] and output_size = (H,W,D) of the fine grid -> [B,H,W,D,Cin]."""
    dtype = np.dtype(dtype)
    images, filters = _prep(dtype, images, filters)
    base_plane = np.ascontiguousarray(base_plane, np.int32)
    defv = np.asarray(default_value, dtype).reshape(1)
    B = images.shape[0]
    H, W, D = [int(x) for x in output_size]
    fh, fw, fd, Cin, Cout = filters.shape
    p = (ctypes.c_int * 15)(B, H, W, D, Cin, Cout, fh, fw, fd, *[int(x) for x in strides], *[int(x) for x in dilations])
    coarse = tuple((n + s - 1) // s for n, s in zip((H, W, D), strides))
    assert tuple(images.shape) == (B, *coarse, Cout), (images.shape, coarse)
    assert tuple(base_plane.shape[:3]) == (B, H, W)
    out = np.empty((B, H, W, D, Cin), dtype)
    nt = nthreads if nthreads is not None else max_threads()
    rc = _lib("port").oracle_sparse_conv3d_transpose_fwd(ctypes.c_int(0 if dtype == np.float32 else 1), p, _p(images),
                                                         _p(filters), _p(defv), _p(base_plane), _p(out), ctypes.c_int(nt))
    assert rc == 0
    return out


def sparse_conv3d_transpose_bwd(images, filters, default_value, base_plane, output_size, out_grad, strides=(1, 1, 1),
                                dilations=(1, 1, 1), reference_quirks=False, dtype=np.float32, nthreads=None):
    """SparseConv3DTransposeFastGrad: returns (images_grad, filter_grad).  reference_quirks=True reproduces the
    buffers the reference's grad op writes (see sparse_oracle.c); False gives the derivatives."""
    dtype = np.dtype(dtype)
    images, filters, out_grad = _prep(dtype, images, filters, out_grad)
    base_plane = np.ascontiguousarray(base_plane, np.int32)
    defv = np.asarray(default_value, dtype).reshape(1)
    B = images.shape[0]
    H, W, D = [int(x) for x in output_size]
    fh, fw, fd, Cin, Cout = filters.shape
    p = (ctypes.c_int * 15)(B, H, W, D, Cin, Cout, fh, fw, fd, *[int(x) for x in strides], *[int(x) for x in dilations])
    assert tuple(out_grad.shape) == (B, H, W, D, Cin)
    igrad = np.empty_like(images)
    fgrad = np.empty_like(filters)
    nt = nthreads if nthreads is not None else max_threads()
    rc = _lib("port").oracle_sparse_conv3d_transpose_bwd(ctypes.c_int(0 if dtype == np.float32 else 1), p, _p(images),
                                                         _p(filters), _p(defv), _p(base_plane), _p(out_grad),
                                                         ctypes.c_int(int(reference_quirks)), _p(igrad), _p(fgrad),
                                                         ctypes.c_int(nt))
    assert rc == 0
    return igrad, fgrad


def _pad_params(images, strides):
    B, h, w, d, C = images.shape
    sr, sc, sd = [int(x) for x in strides]
    p = (ctypes.c_int * 15)(B, h, w, d, C, 0, 0, 0, 0, sr, sc, sd, 1, 1, 1)
    q = (ctypes.c_int * 11)(sr, sc, sd, B, h, w, d, C, h * sr, w * sc, d * sd)
    return p, q, (B, h * sr, w * sc, d * sd, C)


def sparse_pad_fwd(images, base_plane, strides, dtype=np.float32, impl="port"):
    """SparsePad: images [B,h,w,d,C] (coarse band) -> [B,h*sr,w*sc,d*sd,C] with zeros between; base_plane
    [B,h*sr,w*sc,1] is the fine band's first plane."""
    dtype = np.dtype(dtype)
    images, = _prep(dtype, images)
    base_plane = np.ascontiguousarray(base_plane, np.int32)
    p, q, oshape = _pad_params(images, strides)
    assert tuple(base_plane.shape[:3]) == oshape[:3]
    out = np.empty(oshape, dtype)
    dt = ctypes.c_int(0 if dtype == np.float32 else 1)
    if impl == "port":
        _lib("port").oracle_sparse_pad_fwd(dt, p, _p(images), _p(base_plane), _p(out))
    else:
        _lib("ref").ref_sparse_pad_fwd(dt, q, _p(images), _p(base_plane), _p(out))
    return out


def sparse_pad_bwd(images, base_plane, out_grad, strides, reference_quirk=False, dtype=np.float32, impl="port"):
    """SparsePadGrad.  impl="ref" runs the reference kernel, which reads the wrong pixel when a row/column
    stride exceeds 1 (see sparse_oracle.c); impl="port" with reference_quirk=True reproduces that."""
    dtype = np.dtype(dtype)
    images, out_grad = _prep(dtype, images, out_grad)
    base_plane = np.ascontiguousarray(base_plane, np.int32)
    p, q, oshape = _pad_params(images, strides)
    assert tuple(out_grad.shape) == oshape
    igrad = np.empty_like(images)
    dt = ctypes.c_int(0 if dtype == np.float32 else 1)
    if impl == "port":
        _lib("port").oracle_sparse_pad_bwd(dt, p, _p(base_plane), _p(out_grad), ctypes.c_int(int(reference_quirk)), _p(igrad))
    else:
        _lib("ref").ref_sparse_pad_bwd(dt, q, _p(images), _p(base_plane), _p(out_grad), _p(igrad))
    return igrad


# ---- FeatureAggregate, IndexInitializer, DecodePfm ----------------------------------------------------
def feature_aggregate_fwd(src, base_plane, offsets, Rs, Ts, half_centor=True, dtype=np.float32, impl="port",
                          nthreads=None):
    """FeatureAggregate: src [B,N,Hs,Ws,C], base_plane [B,H,W,1], offsets [B,D] ->
    (mapped_feature [B,H,W,D,N,C], mapped_mask int32 [B,H,W,D,N,1])."""
    dtype = np.dtype(dtype)
    src, base_plane, offsets, Rs, Ts = _prep(dtype, src, base_plane, offsets, Rs, Ts)
    B, N, Hs, Ws, C = src.shape
    H, W, D = base_plane.shape[1], base_plane.shape[2], offsets.shape[1]
    dims = (ctypes.c_int64 * 8)(B, H, W, C, D, N, Hs, Ws)
    mapped = np.empty((B, H, W, D, N, C), dtype)
    mask = np.empty((B, H, W, D, N, 1), np.int32)
    nt = nthreads if nthreads is not None else max_threads()
    fn = _lib("port").oracle_feature_aggregate_fwd if impl == "port" else _lib("ref").ref_feature_aggregate_fwd
    fn(ctypes.c_int(0 if dtype == np.float32 else 1), ctypes.c_int(int(half_centor)), dims, _p(src), _p(base_plane),
       _p(offsets), _p(Rs), _p(Ts), _p(mapped), _p(mask), ctypes.c_int(nt))
    return mapped, mask


def feature_aggregate_bwd(src, base_plane, offsets, Rs, Ts, mapped_grad, mask, half_centor=True, dtype=np.float32,
                          impl="port", nthreads=1):
    """FeatureAggregateGrad: returns (src_grad, base_plane_grad)."""
    dtype = np.dtype(dtype)
    src, base_plane, offsets, Rs, Ts, mapped_grad = _prep(dtype, src, base_plane, offsets, Rs, Ts, mapped_grad)
    mask = np.ascontiguousarray(mask, np.int32)
    B, N, Hs, Ws, C = src.shape
    H, W, D = base_plane.shape[1], base_plane.shape[2], offsets.shape[1]
    dims = (ctypes.c_int64 * 8)(B, H, W, C, D, N, Hs, Ws)
    src_grad = np.empty_like(src)
    base_grad = np.empty_like(base_plane)
    fn = _lib("port").oracle_feature_aggregate_bwd if impl == "port" else _lib("ref").ref_feature_aggregate_bwd
    fn(ctypes.c_int(0 if dtype == np.float32 else 1), ctypes.c_int(int(half_centor)), dims, _p(src), _p(base_plane),
       _p(offsets), _p(Rs), _p(Ts), _p(mapped_grad), _p(mask), _p(src_grad), _p(base_grad), ctypes.c_int(nthreads))
    return src_grad, base_grad


def index_initializer(H, W, half_centor=True, dtype=np.float32, impl="port"):
    """IndexInitializer: [H,W,3] = (column, row, 1), +0.5 on the first two when half_centor
    (index_initializer_kernels_gpu.cu.cc:21-29)."""
    dtype = np.dtype(dtype)
    if impl == "ref":
        out = np.empty((H, W, 3), dtype)
        _lib("ref").ref_index_initializer(ctypes.c_int(0 if dtype == np.float32 else 1), ctypes.c_int(int(half_centor)),
                                          ctypes.c_int(H), ctypes.c_int(W), _p(out))
        return out
    out = np.ones((H, W, 3), dtype)
    out[..., 0] = np.arange(W, dtype=dtype)[None, :] + (0.5 if half_centor else 0.0)
    out[..., 1] = np.arange(H, dtype=dtype)[:, None] + (0.5 if half_centor else 0.0)
    return out


def decode_pfm(contents):
    """DecodePfm (pfm_decoder_kernels.cc:38-116), statement by statement: a little-endian single-channel "Pf"
    image -> float32 [H,W,1] with the rows flipped (PFM stores the bottom row first).  Raises ValueError where the
    reference reports InvalidArgument: a magic other than Pf/PF, a missing field, a positive (big-endian) scale on
    a little-endian host, the unimplemented colour format "PF", too little data - and a comment line after the
    magic, which the reference skips up to (not past) its newline and then fails to parse as the width."""
    ws = b" \t\r\n"
    n = len(contents)

    def first_of(pos):
        while pos < n and contents[pos] not in ws:
            pos += 1
        return pos if pos < n else -1

    def first_not_of(pos):
        while pos < n and contents[pos] in ws:
            pos += 1
        return pos if pos < n else -1

    def number(tok, conv, what):
        try:
            return conv(tok.decode("ascii"))
        except (ValueError, UnicodeDecodeError):
            raise ValueError("unable to parse %s: %r" % (what, tok))

    off = first_of(0)
    if off < 0:
        raise ValueError("no magic")
    magic = contents[:off]
    if magic not in (b"Pf", b"PF"):
        raise ValueError("invalid format: %r" % magic)
    off = first_not_of(off)
    if off < 0:
        raise ValueError("no width")
    if contents[off:off + 1] == b"#":
        while off < n and contents[off:off + 1] != b"\n":
            off += 1
    pos = off
    off = first_of(pos)
    if off < 0:
        raise ValueError("no width")
    width = number(contents[pos:off], int, "width")
    fields = []
    for what, conv in (("height", int), ("scaling_factor", float)):
        off = first_not_of(off)
        if off < 0:
            raise ValueError("no " + what)
        pos = off
        off = first_of(pos)
        if off < 0:
            raise ValueError("no " + what)
        fields.append(number(contents[pos:off], conv, what))
    height, scale = fields
    if scale > 0.0:     # big-endian data on a little-endian host
        raise ValueError("invalid scaling_factor value: mismatched endian type")
    off += 1
    if magic != b"Pf":
        raise ValueError("no implement")
    if off + 4 * width * height > n:
        raise ValueError("not enough data")
    img = np.frombuffer(contents, dtype="<f4", count=width * height, offset=off).reshape(height, width)
    return np.ascontiguousarray(img[::-1])[..., None]
