#!/usr/bin/env python
"""Build the reference's own CUDA extension (kvhq_gemv) and stage the reference modules that call it.

    python baseline/build_ref.py [--reference /path/to/HqeKV]      (default: $HQKV_REFERENCE)

The reference tree is read-only and its extension builds in place, so ``quant/`` is copied to a temporary
directory, built there with the reference's own ``setup.py`` (torch.utils.cpp_extension, nvcc; only the
architecture list is set: TORCH_CUDA_ARCH_LIST=10.0 for B200) and the result - the extension's shared object
and the reference's Python modules of the decode path, unmodified - is placed in ``baseline/_ref/``, which is
ignored by git (nothing of the reference enters the history) but travels to the GPU box.  ``bench.py --impl
reference-cuda`` and the cross-check test import from there when it exists.
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PY_MODULES = ["quant/pack_unpack.py", "quant/matmul.py", "quant/hqe_matmul.py", "quant/hqe.py", "quant/hqe_1.py",
              "quant/hqe_2.py", "model/public_func.py"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("HQKV_REFERENCE", ""))
    args = ap.parse_args()
    ref = args.reference
    if not ref or not os.path.isdir(os.path.join(ref, "quant", "csrc")):
        sys.exit("pass --reference <checkout of skywclouds/HqeKV> (or set HQKV_REFERENCE)")
    tmp = tempfile.mkdtemp(prefix="hqkv_ref_build_")
    try:
        work = os.path.join(tmp, "quant")
        shutil.copytree(os.path.join(ref, "quant"), work)
        env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0", MAX_JOBS=str(os.cpu_count() or 4))
        subprocess.check_call([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=work, env=env)
        built = glob.glob(os.path.join(work, "kvhq_gemv*.so"))
        if not built:
            sys.exit("the build produced no kvhq_gemv shared object")
        if os.path.isdir(DEST):
            shutil.rmtree(DEST)
        os.makedirs(os.path.join(DEST, "quant"))
        os.makedirs(os.path.join(DEST, "model"))
        shutil.copy(built[0], os.path.join(DEST, "quant", os.path.basename(built[0])))
        for rel in PY_MODULES:
            shutil.copy(os.path.join(ref, rel), os.path.join(DEST, rel))
        print("built", os.path.join(DEST, "quant", os.path.basename(built[0])))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()
