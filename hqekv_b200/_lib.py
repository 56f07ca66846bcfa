"""ctypes binding of libhqkv.so (declarations in include/hqkv.h).

The library is the only compute path of this package: if it cannot be loaded the import of any
operator module raises — there is no PyTorch or CPU fallback.
"""
import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HQKV_LIB") or os.path.join(HERE, "libhqkv.so")  # HQKV_LIB: another build of the same library

NUM_TIERS = 5
TIER_BITS = (16, 8, 4, 2, 1)
WS_HEADER_BYTES = 12288
CODEC_UNIFORM, CODEC_NORMAL = 0, 1


class HqkvError(RuntimeError):
    """A libhqkv entry point returned a negative status."""

    def __init__(self, code, message):
        super().__init__(f"libhqkv error {code}: {message}")
        self.code = code


class Tier(C.Structure):
    _fields_ = [("bits", C.c_int32), ("n_k", C.c_int32), ("n_v", C.c_int32), ("codec", C.c_int32),
                ("k_data", C.c_void_p), ("k_scale", C.c_void_p), ("k_zero", C.c_void_p), ("k_idx", C.c_void_p),
                ("v_data", C.c_void_p), ("v_scale", C.c_void_p), ("v_zero", C.c_void_p), ("v_idx", C.c_void_p)]


class CacheDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("nh_q", C.c_int32), ("D", C.c_int32),
                ("group_k", C.c_int32), ("group_v", C.c_int32), ("n_new", C.c_int32), ("softmax_scale", C.c_float),
                ("new_k", C.c_void_p), ("new_v", C.c_void_p), ("tier", Tier * NUM_TIERS)]


class FlushSrc(C.Structure):
    _fields_ = [("data", C.c_void_p * NUM_TIERS), ("scale", C.c_void_p * NUM_TIERS), ("zero", C.c_void_p * NUM_TIERS),
                ("n", C.c_int32 * NUM_TIERS), ("low_codec", C.c_int32), ("residual", C.c_void_p),
                ("residual_b_stride", C.c_int64), ("residual_h_stride", C.c_int64)]


_SIGNATURES = {
    "hqkv_last_error": (C.c_char_p, []),
    "hqkv_version": (C.c_int, []),
    "hqkv_build_id": (C.c_char_p, []),
    "hqkv_checks_enabled": (C.c_int, []),
    "hqkv_check_failures": (C.c_int, [C.c_int, C.POINTER(C.c_uint)]),
    "hqkv_quantize_pack": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                     C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hqkv_normal1_quantize_pack": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                             C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hqkv_normal1_dequantize_unpack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int,
                                                 C.c_void_p, C.c_void_p]),
    "hqkv_dequantize_unpack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int,
                                         C.c_void_p, C.c_void_p]),
    "hqkv_pack": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "hqkv_unpack": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "hqkv_decode_workspace_bytes": (C.c_size_t, [C.POINTER(CacheDesc)]),
    "hqkv_decode_workspace_zero_bytes": (C.c_size_t, [C.POINTER(CacheDesc)]),
    "hqkv_decode_attention_headsum": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_size_t, C.c_void_p]),
    "hqkv_decode_logits": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "hqkv_decode_weighted_sum": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                           C.c_void_p]),
    "hqkv_decode_attention_masked": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p,
                                               C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "hqkv_decode_attention": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_size_t, C.c_void_p]),
    "hqkv_decode_attention_phases": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_size_t, C.c_int, C.c_void_p]),
    "hqkv_decode_static_scratch_bytes": (C.c_size_t, []),
    "hqkv_decode_attention_gather": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_size_t, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.c_int,
                                               C.c_int, C.c_void_p, C.c_longlong, C.c_void_p]),
    "hqkv_decode_attention_gather_flagged": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                       C.c_size_t, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p]),
    "hqkv_peer_unpack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p]),
    "hqkv_peer_barrier": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p]),
    "hqkv_decode_attention_static": (C.c_int, [C.POINTER(CacheDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hqkv_gemv_uniform_group": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hqkv_gemv_normal_group": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hqkv_head_sum": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "hqkv_token_importance": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "hqkv_token_range": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_int64,
                                   C.c_void_p, C.c_void_p]),
    "hqkv_block_rank": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hqkv_flush_plan_workspace_bytes": (C.c_size_t, [C.c_int64]),
    "hqkv_flush_plan": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int64, C.c_int64, C.c_void_p,
                                  C.POINTER(C.c_int64), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_size_t, C.c_void_p]),
    "hqkv_flush_build_k": (C.c_int, [C.POINTER(FlushSrc), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hqkv_flush_build_v": (C.c_int, [C.POINTER(FlushSrc), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "hqkv_gather_columns_f16": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int64, C.c_void_p,
                                          C.c_int64, C.c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m hqekv_b200.build` (needs nvcc); "
            "this package has no fallback path")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc):
    if rc != 0:
        raise HqkvError(rc, lib.hqkv_last_error().decode())


def ptr(t):
    """Device pointer of a tensor (or None)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device):
    """Handle of the current stream of `device` (the direct binding when torch has it: this sits on
    the per-layer decode path, where a microsecond of host time is a tenth of the GPU time)."""
    if _raw_stream is not None:
        idx = device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("hqekv_b200 operators run on CUDA tensors only (no CPU path)")


# ---- scratch for the decode call: one buffer per (device, stream).  The library wants it zeroed once (arrival
#      counters, status word, output accumulators); every call that completes leaves it zero again.  Calls on
#      different streams get different buffers, so they cannot race on the counters.  A buffer that was handed
#      out is never released while the process lives: a CUDA graph captured earlier still holds its address.
_decode_ws = {}
_decode_ws_retired = []


def decode_workspace(device, nbytes, stream=None):
    if stream is None:
        stream = stream_ptr(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device(), stream)
    buf = _decode_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _decode_ws_retired.append(buf)
        grow = max(nbytes, 1 << 20)
        buf = torch.zeros(grow, dtype=torch.uint8, device=device)
        _decode_ws[key] = buf
    return buf
