"""Names of the reference's quant/hqe.py that its model files import.

model/llama_hqe.py:23 and model/qwen3_hqe.py:23 do ``from quant.hqe import KV_cache_hqe`` and never call
it: their flush goes through quant.hqe_2.KV_cache_hqe_2 (model/llama_hqe.py:230).  quant/hqe.py is the
earlier, token-granular flush (no 32-token blocks, ``torch.isin`` ladders, quant/hqe.py:143-541); it is
not on the decode path this package rebuilds, so its two builders exist here under their names and raise
when called.  The dense reconstruction works on the same 42-slot tuple as quant/hqe_2.py's and is shared.
"""
from .hqe_2 import KV_cache_reconstruct_hqe  # noqa: F401  (quant/hqe.py:544-660, same tuple layout)


def _not_built(name, where):
    def f(*args, **kwargs):
        raise NotImplementedError(f"{name} ({where}): the token-granular flush of the reference is not built in "
                                  "hqekv_b200; the models flush through quant.hqe_2.KV_cache_hqe_2")
    f.__name__ = name
    return f


KV_cache_hqe = _not_built("KV_cache_hqe", "quant/hqe.py:143")
KV_cache_fake_hqe = _not_built("KV_cache_fake_hqe", "quant/hqe.py:77")
