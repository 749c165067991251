"""ctypes binding of libchop_b200.so - the same C ABI a TensorFlow OpKernel, a cgo stub or any other
host would bind (include/chop.h).  There is no fallback: if the library is missing or a call fails,
the caller gets an exception."""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libchop_b200.so")

F32, F64, BF16 = 0, 1, 2
KIND_V1, KIND_V2, KIND_AGG, KIND_V3 = 1, 2, 3, 4
REDUCE_MEAN, REDUCE_MIN = 0, 1
FLAG_STRICT, FLAG_ACCUMULATE = 1, 2
ERR_FORMAT = -8


class CvDesc(ctypes.Structure):
    """struct chop_cv_desc (include/chop.h)."""
    _fields_ = [("kind", ctypes.c_int32), ("dtype", ctypes.c_int32), ("reduce", ctypes.c_int32),
                ("half_centor", ctypes.c_int32), ("groups", ctypes.c_int32), ("flags", ctypes.c_uint32),
                ("B", ctypes.c_int64), ("H", ctypes.c_int64), ("W", ctypes.c_int64), ("C", ctypes.c_int64),
                ("D", ctypes.c_int64), ("N", ctypes.c_int64), ("Hs", ctypes.c_int64), ("Ws", ctypes.c_int64),
                ("d_begin", ctypes.c_int64), ("d_end", ctypes.c_int64)]


class ScDesc(ctypes.Structure):
    """struct chop_sc_desc (include/chop.h)."""
    _fields_ = [("dtype", ctypes.c_int32), ("dynamic_default", ctypes.c_int32),
                ("B", ctypes.c_int64), ("H", ctypes.c_int64), ("W", ctypes.c_int64), ("D", ctypes.c_int64),
                ("Cin", ctypes.c_int64), ("Cout", ctypes.c_int64),
                ("filter", ctypes.c_int32 * 3), ("strides", ctypes.c_int32 * 3), ("dilations", ctypes.c_int32 * 3),
                ("reserved", ctypes.c_int32)]


class ChopError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__("%s failed with status %d: %s" % (what, status, status_string(status)))


_lib = None


def lib():
    """Load the shared library once.  Raises if it has not been built (python -m
    custom_helper_op_b200.build) - there is deliberately no CPU or PyTorch fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libchop_b200.so not found at %s; build it with "
                              "`python -m custom_helper_op_b200.build`" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp = ctypes.c_void_p
        L.chop_cost_volume_fwd.restype = ctypes.c_int
        L.chop_cost_volume_fwd.argtypes = [ctypes.POINTER(CvDesc)] + [vp] * 9
        L.chop_cost_volume_bwd.restype = ctypes.c_int
        L.chop_cost_volume_bwd.argtypes = [ctypes.POINTER(CvDesc)] + [vp] * 12
        L.chop_sparse_conv3d_bwd_workspace_size.restype = ctypes.c_size_t
        L.chop_sparse_conv3d_bwd_workspace_size.argtypes = [ctypes.POINTER(ScDesc)]
        L.chop_sparse_conv3d_fwd.restype = ctypes.c_int
        L.chop_sparse_conv3d_fwd.argtypes = [ctypes.POINTER(ScDesc)] + [vp] * 6
        L.chop_sparse_conv3d_bwd.restype = ctypes.c_int
        L.chop_sparse_conv3d_bwd.argtypes = [ctypes.POINTER(ScDesc)] + [vp] * 9 + [ctypes.c_size_t, vp]
        L.chop_sparse_conv3d_bwd_noalloc.restype = ctypes.c_int
        L.chop_sparse_conv3d_bwd_noalloc.argtypes = [ctypes.POINTER(ScDesc)] + [vp] * 9
        L.chop_sparse_conv3d_transpose_fwd.restype = ctypes.c_int
        L.chop_sparse_conv3d_transpose_fwd.argtypes = [ctypes.POINTER(ScDesc)] + [vp] * 6
        L.chop_sparse_conv3d_transpose_bwd_workspace_size.restype = ctypes.c_size_t
        L.chop_sparse_conv3d_transpose_bwd_workspace_size.argtypes = [ctypes.POINTER(ScDesc)]
        L.chop_sparse_conv3d_transpose_bwd.restype = ctypes.c_int
        L.chop_sparse_conv3d_transpose_bwd.argtypes = [ctypes.POINTER(ScDesc)] + [vp] * 8 + [ctypes.c_size_t, vp]
        i64, i3 = ctypes.c_int64, ctypes.POINTER(ctypes.c_int32)
        L.chop_sparse_pad_fwd.restype = ctypes.c_int
        L.chop_sparse_pad_fwd.argtypes = [ctypes.c_int32, i64, i64, i64, i64, i64, i3, vp, vp, vp, vp]
        L.chop_sparse_pad_bwd.restype = ctypes.c_int
        L.chop_sparse_pad_bwd.argtypes = [ctypes.c_int32, i64, i64, i64, i64, i64, i3, vp, vp, vp, vp]
        L.chop_feature_aggregate_fwd.restype = ctypes.c_int
        L.chop_feature_aggregate_fwd.argtypes = [ctypes.POINTER(CvDesc)] + [vp] * 8
        L.chop_feature_aggregate_bwd.restype = ctypes.c_int
        L.chop_feature_aggregate_bwd.argtypes = [ctypes.POINTER(CvDesc)] + [vp] * 10
        L.chop_index_initializer.restype = ctypes.c_int
        L.chop_index_initializer.argtypes = [ctypes.c_int32, ctypes.c_int32, i64, i64, vp, vp]
        L.chop_decode_pfm.restype = ctypes.c_int
        L.chop_decode_pfm.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(i64), ctypes.POINTER(i64),
                                      ctypes.POINTER(i64), vp, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t]
        L.chop_copy_2d_async.restype = ctypes.c_int
        L.chop_copy_2d_async.argtypes = [vp, ctypes.c_size_t, vp, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, vp]
        L.chop_umma_timeouts.restype = ctypes.c_int
        L.chop_umma_watch.restype = ctypes.c_int
        L.chop_status_string.restype = ctypes.c_char_p
        L.chop_status_string.argtypes = [ctypes.c_int]
        L.chop_version.restype = ctypes.c_int
        L.chop_set_tuning.restype = ctypes.c_int
        L.chop_set_tuning.argtypes = [ctypes.c_char_p, ctypes.c_int]
        _lib = L
    return _lib


def status_string(status):
    return lib().chop_status_string(int(status)).decode()


def check(status, what):
    if status != 0:
        raise ChopError(status, what)


def set_tuning(name, value):
    check(lib().chop_set_tuning(name.encode(), int(value)), "chop_set_tuning")
