"""Name-compatible stand-in for the reference's ``kvhq_gemv`` extension module
(quant/csrc/pybind.cpp:5-27) for the one export the decode path of the models reaches.

The reference's native entry takes operands that quant/matmul.py has already transposed into
[B*nh_kv, N/feat_per_int, K] (codes) and [B*nh_kv, N/group, K] (scale, zero).  libhqkv reads the
cache's own layout, so this shim transposes back (a copy) before calling it; callers that hold the
cache layout should call quant.matmul.cuda_bmm_fA_qB_uniform_group directly, which copies nothing.
"""
from .matmul import cuda_bmm_fA_qB_uniform_group


def gemv_forward_cuda_uniform_group(in_feats, kernel, scaling_factors, zeros, bit, group_size, nh_q, nh_kv):
    """quant/csrc/gemv_cuda_uniform.cu:1533-1599.  in_feats [B*nh_q, 1, K] fp16; kernel
    [B*nh_kv, N/fpi, K] int32; scaling_factors / zeros [B*nh_kv, N/group, K] fp16.
    Returns [B*nh_q, 1, N] fp16."""
    BSq, M, K = in_feats.shape
    B = BSq // nh_q
    fA = in_feats.reshape(B, nh_q, M, K)
    qB = kernel.transpose(1, 2).reshape(B, nh_kv, K, kernel.shape[1])
    sc = scaling_factors.transpose(1, 2).reshape(B, nh_kv, K, scaling_factors.shape[1])
    zp = zeros.transpose(1, 2).reshape(B, nh_kv, K, zeros.shape[1])
    out = cuda_bmm_fA_qB_uniform_group(group_size, fA, qB, sc, zp, bit)
    return out.reshape(BSq, M, -1)


def __getattr__(name):
    if name.startswith("gemv_forward_cuda"):
        def f(*args, **kwargs):
            raise NotImplementedError(f"kvhq_gemv.{name} is not built in hqekv_b200")
        return f
    raise AttributeError(name)
