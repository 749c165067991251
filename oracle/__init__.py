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

KIND_V1, KIND_V2, KIND_AGG = 1, 2, 3
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
    """Forward of CostVolume (kind 1), CostVolumeV2 (kind 2) or CostAggregate (kind 3).

    ``depth`` is base_plane [B,H,W,1] for kinds 1/3 and depth_grid [B,H,W,D] for kind 2 (offsets
    None).  Returns (cost, mask) shaped like the reference op's outputs."""
    dtype = np.dtype(dtype)
    ref, src, depth, offsets, Rs, Ts = _prep(dtype, ref, src, depth, offsets, Rs, Ts)
    B, H, W, C = ref.shape
    D = depth.shape[3] if kind == KIND_V2 else offsets.shape[1]
    rmin = int(reduce_method == "MIN")
    CO = C if kind == KIND_V1 else (groups if kind == KIND_V2 else 1)
    cost = np.empty((B, H, W, D, CO), dtype)
    mask = np.empty((B, H, W, D, CO if rmin else 1), np.int32)
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
