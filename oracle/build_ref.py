#!/usr/bin/env python
"""Stage the reference's own Python modules of the hot path for the CPU baseline.

    python oracle/build_ref.py [--reference /path/to/HqeKV]      (default: $HQEKV_REFERENCE_ROOT)

The reference is Python on this path (its C++/CUDA part is the GPU extension, built by baseline/build_ref.py), so
"building" it means copying the modules, unmodified, into ``oracle/_ref/`` - a directory git ignores, so nothing of
the reference enters the history, but which travels to the GPU box, where no checkout of the reference exists.
``bench.py --impl reference`` then times the reference's own ``KV_cache_reconstruct_hqe`` (quant/hqe_2.py:967-1084)
+ fp32 attention on the host cores through ``oracle/ref_shim.py``; without the staged copy it times the numpy
restatement instead and says so (``cpu_baseline.kind``: "reference" / "port").
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
MODULES = ["quant/pack_unpack.py", "quant/hqe_2.py", "model/public_func.py"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("HQEKV_REFERENCE_ROOT", ""))
    args = ap.parse_args()
    ref = args.reference
    if not ref or not os.path.isfile(os.path.join(ref, "quant", "hqe_2.py")):
        sys.exit("pass --reference <checkout of skywclouds/HqeKV> (or set HQEKV_REFERENCE_ROOT)")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    for rel in MODULES:
        os.makedirs(os.path.dirname(os.path.join(DEST, rel)), exist_ok=True)
        shutil.copy(os.path.join(ref, rel), os.path.join(DEST, rel))
    print("staged", ", ".join(MODULES), "in", DEST)


if __name__ == "__main__":
    main()
