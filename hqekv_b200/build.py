"""Build libhqkv.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m hqekv_b200.build          # rebuild if the library was not compiled from the sources present
    python -m hqekv_b200.build --force
    python -m hqekv_b200.build --checks # the bounds-check build, libhqkv_checked.so

Every build is stamped with a hash of its sources (hqkv_build_id()).

No --use_fast_math: the codec relies on IEEE division and explicit roundings.
"""
import hashlib
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


def source_id():
    """First 16 hex digits of the SHA-256 over the library's sources (csrc sorted by name, then the header)."""
    h = hashlib.sha256()
    for path in sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)) + [os.path.join(INCLUDE, "hqkv.h")]:
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read())
    return h.hexdigest()[:16]


def library_id(path=LIB_PATH):
    """The stamp inside a built library, read from the file without loading it (None if there is none)."""
    marker = b"HQKV_BUILD_ID="
    try:
        with open(path, "rb") as f:
            blob = f.read()
    except OSError:
        return None
    at = blob.find(marker)
    if at < 0:
        return None
    end = blob.find(b"\0", at)
    return blob[at + len(marker):end].decode(errors="replace")


def needs_build():
    """True when the library is missing or was compiled from other sources than the ones present."""
    return not os.path.exists(LIB_PATH) or library_id(LIB_PATH) != source_id()


CHECKED_LIB_PATH = os.path.join(HERE, "libhqkv_checked.so")


def build(force=False, verbose=False, checks=False):
    """Compile every .cu into objects and link the shared library.  Returns its path.
    ``checks``: the bounds-check build (-DHQKV_CHECKS) into libhqkv_checked.so; load it with HQKV_LIB=<path>."""
    if os.environ.get("HQKV_LIB") and not checks:
        return os.environ["HQKV_LIB"]  # the caller points at a library it built itself
    if checks:
        if not force and os.path.exists(CHECKED_LIB_PATH) and library_id(CHECKED_LIB_PATH) == source_id():
            return CHECKED_LIB_PATH
        return _compile(CHECKED_LIB_PATH, os.path.join(HERE, "build", "checked"), ["-DHQKV_CHECKS"], verbose)
    if not force and not needs_build():
        return LIB_PATH
    return _compile(LIB_PATH, os.path.join(HERE, "build"), [], verbose)


def _compile(lib_path, objdir, extra, verbose):
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    extra = [*extra, f'-DHQKV_BUILD_ID="{source_id()}"']
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
