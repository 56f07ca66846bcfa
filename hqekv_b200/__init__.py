"""hqekv_b200 — sm_100a implementation of the hybrid mixed-precision KV-cache decode path.

Layout
  csrc/ + ../include/hqkv.h   CUDA kernels and the C ABI (libhqkv.so, built by ``hqekv_b200.build``)
  _lib.py                     ctypes binding of the C ABI
  quant/, model/              host-side mirror of the reference's operator modules for this path
                              (quant/pack_unpack.py, matmul.py, hqe_2.py, hqe_matmul.py, model/public_func.py)

``install_reference_names()`` registers those modules under the import names the reference's model
files use (``quant.hqe``, ``quant.hqe_2``, ``quant.hqe_matmul``, ``model.public_func``, flat ``pack_unpack``,
``hqe``, ``hqe_1`` ...), so that the project imports of ``model/llama_hqe.py`` / ``model/qwen3_hqe.py``
(lines 21-25 of either file) resolve to this implementation.
"""
import importlib
import sys

__version__ = "0.1.0"

_REFERENCE_NAMES = {
    "pack_unpack": "hqekv_b200.quant.pack_unpack",
    "matmul": "hqekv_b200.quant.matmul",
    "hqe": "hqekv_b200.quant.hqe",
    "hqe_1": "hqekv_b200.quant.hqe_1",
    "hqe_2": "hqekv_b200.quant.hqe_2",
    "hqe_matmul": "hqekv_b200.quant.hqe_matmul",
    "hybrid_quant": "hqekv_b200.quant.hybrid_quant",
    "quant_matmul_hq": "hqekv_b200.quant.quant_matmul_hq",
    "kvhq_gemv": "hqekv_b200.quant.kvhq_gemv",
    "quant.pack_unpack": "hqekv_b200.quant.pack_unpack",
    "quant.matmul": "hqekv_b200.quant.matmul",
    "quant.hqe": "hqekv_b200.quant.hqe",
    "quant.hqe_1": "hqekv_b200.quant.hqe_1",
    "quant.hqe_2": "hqekv_b200.quant.hqe_2",
    "quant.hqe_matmul": "hqekv_b200.quant.hqe_matmul",
    "quant.hybrid_quant": "hqekv_b200.quant.hybrid_quant",
    "quant.quant_matmul_hq": "hqekv_b200.quant.quant_matmul_hq",
    "quant.kvhq_gemv": "hqekv_b200.quant.kvhq_gemv",
    "model.public_func": "hqekv_b200.model.public_func",
}


def install_reference_names(overwrite: bool = False):
    """Make ``import quant.hqe_2`` etc. resolve to this package (the reference has the repository
    root and ``quant/`` on sys.path, so both the flat and the dotted names exist there)."""
    installed = []
    for alias, target in _REFERENCE_NAMES.items():
        if alias in sys.modules and not overwrite:
            continue
        sys.modules[alias] = importlib.import_module(target)
        installed.append(alias)
    if "quant" not in sys.modules or overwrite:
        sys.modules["quant"] = importlib.import_module("hqekv_b200.quant")
    return installed
