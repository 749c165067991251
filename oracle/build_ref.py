#!/usr/bin/env python3
"""TEST INFRASTRUCTURE ONLY.  Build ``oracle/_ref/libchop_ref.so``: the reference's own CUDA kernel
bodies for the cost-volume / manifold-conv path, compiled unmodified as host C++.

The reference registers GPU kernels only, so there is no CPU build of it to call.  Its kernel
*bodies*, however, are ordinary C++ apart from ``__global__``, ``GpuGridRangeX``, ``GpuAtomicAdd``
and ``__ldg``.  This script reads the kernel templates out of the reference checkout (brace
matching on the ``__global__`` definitions, plus the ``#define`` blocks they depend on), writes
them to a temporary directory, and compiles them together with ``ref_shim.h`` and
``ref_driver.cc``.  Only the shared library is kept; no reference text is stored in this
repository and the temporary directory is removed.

Floating-point contract: ``-ffp-contract=off`` - every ``*``, ``+``, ``/`` in the reference source
is one correctly-rounded IEEE operation, evaluated in source order.  That is the arithmetic the
CUDA kernels reproduce bit-for-bit for the projection (and, in strict mode, for everything).

Usage: python oracle/build_ref.py [--reference PATH_OF_THE_REFERENCE_CHECKOUT] [--quiet]
Exit code 0 with the library built, 3 if the reference checkout is absent (nothing to do).
"""
import argparse
import os
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
KDIR = "custom_helper_op/cc/kernels"

# (file, [kernel names], [macro names], output include name)
EXTRACTS = [
    ("cost_volume_kernels_gpu.cu.cc",
     ["CostMeanVolumeKernel", "CostMinVolumeKernel", "CostMeanVolumeGradKernel", "CostMinVolumeGradKernel"],
     [], "ref_cost_volume_v1.inc"),
    ("cost_volume_kernels_gpu_v2.cu.cc",
     ["CostMeanVolumeV2Kernel", "CostMinVolumeV2Kernel", "CostMeanVolumeGradV2Kernel", "CostMinVolumeGradV2Kernel"],
     [], "ref_cost_volume_v2.inc"),
    ("cost_aggregate_kernels_gpu.cu.cc",
     ["CostMeanAggregateKernel", "CostMinAggregateKernel", "CostMeanAggregateGradKernel", "CostMinAggregateGradKernel"],
     [], "ref_cost_aggregate.inc"),
    ("sparse_conv3d_kernels_gpu.cu.cc",
     ["SparseConv3DKernel"],
     ["SPARSE_CONV3D_KERNEL_BASE_ARG_DEF_LIST", "CHECK_PADDING"], "ref_sparse_conv3d.inc"),
    ("sparse_conv.h", [], ["SPARSE_CONV3D_FIX_PARAMETOR_DEF_LIST"], "ref_sparse_conv_macros.inc"),
    ("cost_volume_v3.h", [], ["MAX_SUBCHANNELS_SIZE"], "ref_cost_volume_v3_macros.inc"),
    ("cost_volume_kernels_gpu_v3.cu.cc",
     ["CostMeanVolumeV3Kernel", "CostMinVolumeV3Kernel", "CostMeanVolumeGradV3Kernel", "CostMinVolumeGradV3Kernel"],
     [], "ref_cost_volume_v3.inc"),
    ("feature_aggregate_kernels_gpu.cu.cc", ["FeatureAggregateKernel", "FeatureAggregateGradKernel"], [],
     "ref_feature_aggregate.inc"),
    ("index_initializer_kernels_gpu.cu.cc", ["SetToIndex"], [], "ref_index_initializer.inc"),
    ("sparse_pad.h", [], ["SPARSE_PAD_BASE_ARG_DEF_LIST"], "ref_sparse_pad_macros.inc"),
    ("sparse_pad_kernels_gpu.cu.cc", ["SparsePadKernel", "SparsePadGradKernel"], [], "ref_sparse_pad.inc"),
]


def extract_macro(text, name):
    m = re.search(r"^#define\s+" + re.escape(name) + r"\b", text, re.M)
    if not m:
        raise RuntimeError("macro %s not found" % name)
    lines = text[m.start():].split("\n")
    out = []
    for ln in lines:
        out.append(ln)
        if not ln.rstrip().endswith("\\"):
            break
    return "\n".join(out) + "\n"


def extract_kernel(text, name):
    m = re.search(r"__global__\s+void\s+" + re.escape(name) + r"\s*\(", text)
    if not m:
        raise RuntimeError("kernel %s not found" % name)
    # the template header sits on the line(s) just before __global__
    start = text.rfind("template", 0, m.start())
    if start < 0:
        raise RuntimeError("template header of %s not found" % name)
    i = text.index("{", m.end())
    depth = 0
    n = len(text)
    while i < n:
        c = text[i]
        if text.startswith("//", i):          # braces inside comments do not count
            i = text.index("\n", i)
            continue
        if text.startswith("/*", i):
            i = text.index("*/", i) + 2
            continue
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                break
        i += 1
    return text[start:i + 1] + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CHOP_REFERENCE_DIR", ""),
                    help="checkout of zhuimeng999/custom_helper_op (or set CHOP_REFERENCE_DIR)")
    ap.add_argument("--quiet", action="store_true")
    args = ap.parse_args()
    src_dir = os.path.join(args.reference, KDIR) if args.reference else ""
    if not src_dir or not os.path.isdir(src_dir):
        if not args.quiet:
            print("no reference checkout given (--reference DIR or CHOP_REFERENCE_DIR): keeping any prebuilt oracle/_ref")
        return 3
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    tmp = tempfile.mkdtemp(prefix="chop_ref_")
    try:
        for fname, kernels, macros, inc in EXTRACTS:
            with open(os.path.join(src_dir, fname)) as f:
                text = f.read()
            parts = [extract_macro(text, m) for m in macros] + [extract_kernel(text, k) for k in kernels]
            with open(os.path.join(tmp, inc), "w") as f:
                f.write("\n".join(parts))
        out = os.path.join(out_dir, "libchop_ref.so")
        cmd = ["g++", "-std=c++17", "-O3", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
               "-fno-fast-math", "-I", tmp, "-I", HERE, os.path.join(HERE, "ref_driver.cc"), "-o", out]
        if not args.quiet:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    if not args.quiet:
        print("built", out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
