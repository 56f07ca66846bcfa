"""Build libhqkv.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m hqekv_b200.build          # rebuild if a source is newer than the library
    python -m hqekv_b200.build --force

No --use_fast_math: the codec relies on IEEE division and explicit roundings.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_PATH = os.path.join(HERE, "libhqkv.so")
SOURCES = ["codec.cu", "decode.cu", "gemv.cu", "policy.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "hqkv.h")]
    return any(os.path.getmtime(d) > built for d in deps)


CHECKED_LIB_PATH = os.path.join(HERE, "libhqkv_checked.so")


def build(force=False, verbose=False, checks=False):
    """Compile every .cu into objects and link the shared library.  Returns its path.
    ``checks``: the bounds-check build (-DHQKV_CHECKS) into libhqkv_checked.so; load it with HQKV_LIB=<path>."""
    if os.environ.get("HQKV_LIB") and not checks:
        return os.environ["HQKV_LIB"]  # the caller points at a library it built itself
    if checks:
        return _compile(CHECKED_LIB_PATH, os.path.join(HERE, "build", "checked"), ["-DHQKV_CHECKS"], verbose)
    if not force and not needs_build():
        return LIB_PATH
    return _compile(LIB_PATH, os.path.join(HERE, "build"), [], verbose)


def _compile(lib_path, objdir, extra, verbose):
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", INCLUDE, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
        objs.append(obj)
    link = [nvcc, "-shared", "-o", lib_path, *objs, "-Xcompiler", "-fPIC"]  # static cudart (nvcc default)
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, checks="--checks" in sys.argv)
    print(path)
