"""Group quantise + bit-pack codec on the GPU — same names and argument meaning as the reference's
quant/pack_unpack.py, backed by libhqkv (hqekv_b200/csrc/codec.cu) instead of torch elementwise
passes plus Triton pack/unpack kernels.

Differences a caller can observe:
  * the input of the quantisers is left untouched (the reference overwrites it with intermediate
    values through ``sub_``/``div_`` when ``reshape`` returns a view, quant/pack_unpack.py:171-173);
  * only CUDA tensors are accepted.
"""
import torch
from scipy.stats import norm

from .._lib import check, lib, ptr, require_cuda, stream_ptr

n_bits_range = [8, 4, 2, 1]
# Gaussian-quantile codebooks of the "normal" codec (quant/pack_unpack.py:6-14); kept because other
# modules import them by name.
normal_quantiles_upper_bound = {
    n: torch.tensor(norm.ppf(torch.arange(0, 1, 1 / (2 ** n)) + 1 / (2 ** n)), dtype=torch.float32)
    for n in n_bits_range
}
normal_quantiles_center = {
    n: torch.tensor(norm.ppf(torch.arange(0, 1, 1 / (2 ** n)) + 0.5 / (2 ** n)), dtype=torch.float32)
    for n in n_bits_range
}


def _check_bits(bit):
    if bit not in (8, 4, 2, 1):
        raise ValueError(f"bit must be 8, 4, 2 or 1 (got {bit})")


def uniform_group_quantize_pack_last_dim(data: torch.Tensor, group_size: int, bit: int):
    """quant/pack_unpack.py:156-193.  data fp16 [B, nh, D, T] (any strides; a ``transpose(2, 3)``
    view of token-major K is read in place) -> (code int32 [B,nh,D,T*bit/32], scale fp16
    [B,nh,D,T/group], mn fp16 [B,nh,D,T/group])."""
    _check_bits(bit)
    require_cuda(data)
    if data.dtype != torch.float16 or data.dim() != 4:
        raise ValueError("data must be a 4-D float16 tensor")
    B, nh, D, T = data.shape
    if T % group_size:
        raise ValueError("last dimension must be a multiple of group_size")
    sb, sh, sd, st = data.stride()
    collapsible = B == 1 or sb == nh * sh
    if not (collapsible and (st == 1 or sd == 1)) or D == 1 or T == 1:
        data = data.contiguous()
        sb, sh, sd, st = data.stride()
    code = torch.empty(B, nh, D, T * bit // 32, dtype=torch.int32, device=data.device)
    scale = torch.empty(B, nh, D, T // group_size, dtype=torch.float16, device=data.device)
    mn = torch.empty_like(scale)
    with torch.cuda.device(data.device):
        check(lib.hqkv_quantize_pack(ptr(data), B * nh * D, T, D, sh, sd, st, group_size, bit, ptr(code), ptr(scale),
                                     ptr(mn), stream_ptr(data.device)))
    return code, scale, mn


def uniform_group_dequantize_unpack_last_dim(code: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor,
                                             group_size: int, bit: int):
    """quant/pack_unpack.py:316-333: x = half(half(code*scale) + mn) as fp16 [B, nh, D, T]."""
    _check_bits(bit)
    require_cuda(code, scale, mn)
    B, nh, D, T_d = code.shape
    T = T_d * (32 // bit)
    code, scale, mn = code.contiguous(), scale.contiguous(), mn.contiguous()
    out = torch.empty(B, nh, D, T, dtype=torch.float16, device=code.device)
    with torch.cuda.device(code.device):
        check(lib.hqkv_dequantize_unpack(ptr(code), ptr(scale), ptr(mn), B * nh * D, T, group_size, bit, ptr(out),
                                         stream_ptr(code.device)))
    return out


def uniform_group_fake_quant(data: torch.Tensor, group_size: int, bit: int):
    """quant/pack_unpack.py:134-154: quantise then dequantise (both roundings of the dequantiser)."""
    if bit == 0:
        return 0
    code, scale, mn = uniform_group_quantize_pack_last_dim(data, group_size, bit)
    return uniform_group_dequantize_unpack_last_dim(code, scale, mn, group_size, bit)


def pack_along_last_dim(data: torch.Tensor, bit: int):
    """quant/pack_unpack.py:53-70: int32 codes [B,nh,D,T] -> int32 words [B,nh,D,T*bit/32]."""
    _check_bits(bit)
    require_cuda(data)
    B, nh, D, T = data.shape
    data = data.to(torch.int32).contiguous()
    words = torch.empty(B, nh, D, T * bit // 32, dtype=torch.int32, device=data.device)
    with torch.cuda.device(data.device):
        check(lib.hqkv_pack(ptr(data), B * nh * D, T, bit, ptr(words), stream_ptr(data.device)))
    return words


def unpack_along_last_dim(code: torch.Tensor, bit: int):
    """quant/pack_unpack.py:281-297: int32 words [B,nh,D,W] -> fp16 integers [B,nh,D,W*32/bit]."""
    _check_bits(bit)
    require_cuda(code)
    B, nh, D, W = code.shape
    code = code.contiguous()
    out = torch.empty(B, nh, D, W * (32 // bit), dtype=torch.float16, device=code.device)
    with torch.cuda.device(code.device):
        check(lib.hqkv_unpack(ptr(code), B * nh * D, W, bit, ptr(out), stream_ptr(code.device)))
    return out


def _not_built(name):
    def f(*args, **kwargs):
        raise NotImplementedError(
            f"{name}: the Gaussian-quantile ('normal') and un-grouped codecs are not built in hqekv_b200; "
            "use quant_strategy='uniform_group'")
    f.__name__ = name
    return f


normal_quantize_pack_last_dim = _not_built("normal_quantize_pack_last_dim")
normal_dequantize_unpack_last_dim = _not_built("normal_dequantize_unpack_last_dim")


def normal_group_quantize_pack_last_dim(data: torch.Tensor, group_size: int, bit: int):
    """quant/pack_unpack.py:218-253 at bit = 1 (the only width the live strategy
    'high_uniform_group_low_normal_group' uses it at): data fp16 [B, nh, D, T] (any strides) ->
    (code int32 [B,nh,D,T/32], std fp16 [B,nh,D,T/group], mean fp16 [B,nh,D,T/group]).
    The source is not modified (the reference overwrites it with the normalised values)."""
    if bit != 1:
        raise NotImplementedError("normal_group_quantize_pack_last_dim: only bit = 1 is built in hqekv_b200")
    require_cuda(data)
    if data.dtype != torch.float16 or data.dim() != 4:
        raise ValueError("data must be a 4-D float16 tensor")
    B, nh, D, T = data.shape
    if T % group_size:
        raise ValueError("last dimension must be a multiple of group_size")
    sb, sh, sd, st = data.stride()
    if not (B == 1 or sb == nh * sh):
        data = data.contiguous()
        sb, sh, sd, st = data.stride()
    code = torch.empty(B, nh, D, T // 32, dtype=torch.int32, device=data.device)
    std = torch.empty(B, nh, D, T // group_size, dtype=torch.float16, device=data.device)
    mean = torch.empty_like(std)
    with torch.cuda.device(data.device):
        check(lib.hqkv_normal1_quantize_pack(ptr(data), B * nh * D, T, D, sh, sd, st, group_size, ptr(code), ptr(std),
                                             ptr(mean), stream_ptr(data.device)))
    return code, std, mean


def normal_group_dequantize_unpack_last_dim(code: torch.Tensor, std: torch.Tensor, mean: torch.Tensor,
                                            group_size: int, bit: int):
    """quant/pack_unpack.py:356-376 at bit = 1: x = half(half(center[code] * std) + mean), fp16 [B, nh, D, T]."""
    if bit != 1:
        raise NotImplementedError("normal_group_dequantize_unpack_last_dim: only bit = 1 is built in hqekv_b200")
    require_cuda(code, std, mean)
    B, nh, D, T_d = code.shape
    T = T_d * 32
    code, std, mean = code.contiguous(), std.contiguous(), mean.contiguous()
    out = torch.empty(B, nh, D, T, dtype=torch.float16, device=code.device)
    with torch.cuda.device(code.device):
        check(lib.hqkv_normal1_dequantize_unpack(ptr(code), ptr(std), ptr(mean), B * nh * D, T, group_size, ptr(out),
                                                 stream_ptr(code.device)))
    return out


def normal_group_fake_quant(data: torch.Tensor, group_size: int, bit: int):
    """quant/pack_unpack.py:195-216: quantise then dequantise with the Gaussian codebook (bit = 1 only)."""
    if bit == 0:
        return 0
    code, std, mean = normal_group_quantize_pack_last_dim(data, group_size, bit)
    return normal_group_dequantize_unpack_last_dim(code, std, mean, group_size, bit)


uniform_quantize_pack_last_dim = _not_built("uniform_quantize_pack_last_dim")
uniform_dequantize_unpack_last_dim = _not_built("uniform_dequantize_unpack_last_dim")
