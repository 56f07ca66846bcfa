"""Name-compatible stand-in for the reference's ``kvhq_gemv`` extension module
(quant/csrc/pybind.cpp:5-27): the six exports the uniform-group / Gaussian-codebook decode paths reach.

The reference's native entries take operands that quant/matmul.py has already flattened over (batch, head)
and transposed: codes [B*nh_kv, N/feat_per_int, K], scales / zeros [B*nh_kv, N/group, K], activations
[B*nh_q, 1, K]; the fp16 residual K arrives as [B*nh_kv, r, D], the residual V transposed to [B*nh_kv, D, r]
(quant/matmul.py:400-421, :554-569).  libhqkv reads the cache's own layout, so these shims transpose back
(a copy) before calling it; callers that hold the cache layout should call the functions of quant.matmul
directly, which copy nothing.  Outlier, un-grouped and token-major exports raise NotImplementedError.
"""
from . import matmul as _mm


def _back(x, B):
    """[B*nh_kv, a, b] -> [B, nh_kv, b, a] (None passes through)."""
    if x is None:
        return None
    return x.transpose(1, 2).reshape(B, x.shape[0] // B, x.shape[2], x.shape[1])


def gemv_forward_cuda_uniform_group(in_feats, kernel, scaling_factors, zeros, bit, group_size, nh_q, nh_kv):
    """quant/csrc/gemv_cuda_uniform.cu:1533-1599 (prototype gemv_cuda.h:46-54).  Returns [B*nh_q, 1, N] fp16."""
    BSq, M, K = in_feats.shape
    B = BSq // nh_q
    out = _mm.cuda_bmm_fA_qB_uniform_group(group_size, in_feats.reshape(B, nh_q, M, K), _back(kernel, B),
                                           _back(scaling_factors, B), _back(zeros, B), bit)
    return out.reshape(BSq, M, -1)


def gemv_forward_cuda_normalize_group(in_feats, kernel, scaling_factors, zeros, normal_quantiles_center, bit,
                                      group_size, nh_q, nh_kv):
    """quant/csrc/gemv_cuda_normal.cu (prototype gemv_cuda.h:257-266) at bit = 1: scaling_factors = std, zeros = mean;
    the centre table is the library's own constant (+-0.67448974), the argument is accepted and not read."""
    BSq, M, K = in_feats.shape
    B = BSq // nh_q
    out = _mm.cuda_bmm_fA_qB_normal_group(group_size, in_feats.reshape(B, nh_q, M, K), _back(kernel, B),
                                          _back(scaling_factors, B), _back(zeros, B), bit)
    return out.reshape(BSq, M, -1)


def _qk(in_feats, tiers, kernel_new, group_size, nh_q, nh_kv, sequential):
    BSq, M, K = in_feats.shape
    B = BSq // nh_q
    q = in_feats.reshape(B, nh_q, M, K)
    new_K = None if kernel_new is None else kernel_new.reshape(B, nh_kv, kernel_new.shape[1], kernel_new.shape[2])
    tiers = [(bits, _back(d, B), idx, _back(s, B), _back(z, B)) for bits, d, idx, s, z in tiers]
    return _mm._qk_group_hq(group_size, nh_kv, q, tiers, new_K, sequential).reshape(BSq, M, -1)


def _wv(in_feats, tiers, kernel_new, group_size, nh_q, nh_kv, sequential):
    BSq, M, L = in_feats.shape
    B = BSq // nh_q
    w = in_feats.reshape(B, nh_q, M, L)
    new_V = _back(kernel_new, B)   # [B*nh_kv, D, r] -> [B, nh_kv, r, D]
    tiers = [(bits, _back(d, B), idx, _back(s, B), _back(z, B)) for bits, d, idx, s, z in tiers]
    return _mm._wv_group_hq(group_size, nh_kv, w, tiers, new_V, sequential).reshape(BSq, M, -1)


def gemv_forward_cuda_qk_group_hq(in_feats, kernel_16, kernel_16_idx, kernel_8, kernel_8_idx, scaling_factors_8, zeros_8,
                                  kernel_4, kernel_4_idx, scaling_factors_4, zeros_4, kernel_2, kernel_2_idx,
                                  scaling_factors_2, zeros_2, kernel_1, kernel_1_idx, std_1, means_1,
                                  normal_quantiles_center, kernel_new, num_out_channels, num_16, num_8, num_4, num_2, num_1,
                                  new_len, group_size, nh_q, nh_kv):
    """Prototype gemv_cuda.h:78-109.  The counts are re-derived from the tensors."""
    tiers = [(16, kernel_16, kernel_16_idx, None, None), (8, kernel_8, kernel_8_idx, scaling_factors_8, zeros_8),
             (4, kernel_4, kernel_4_idx, scaling_factors_4, zeros_4), (2, kernel_2, kernel_2_idx, scaling_factors_2, zeros_2),
             (1, kernel_1, kernel_1_idx, std_1, means_1)]
    return _qk(in_feats, tiers, kernel_new, group_size, nh_q, nh_kv, False)


def gemv_forward_cuda_qk_group_hq_seq(in_feats, kernel_16, kernel_8, scaling_factors_8, zeros_8, kernel_4, scaling_factors_4,
                                      zeros_4, kernel_2, scaling_factors_2, zeros_2, kernel_1, std_1, means_1,
                                      normal_quantiles_center, kernel_new, num_out_channels, num_16, num_8, num_4, num_2,
                                      num_1, new_len, group_size, nh_q, nh_kv):
    """Prototype gemv_cuda.h:111-137."""
    tiers = [(16, kernel_16, None, None, None), (8, kernel_8, None, scaling_factors_8, zeros_8),
             (4, kernel_4, None, scaling_factors_4, zeros_4), (2, kernel_2, None, scaling_factors_2, zeros_2),
             (1, kernel_1, None, std_1, means_1)]
    return _qk(in_feats, tiers, kernel_new, group_size, nh_q, nh_kv, True)


def gemv_forward_cuda_wv_group_hq(in_feats, kernel_16, kernel_16_idx, kernel_8, kernel_8_idx, scaling_factors_8, zeros_8,
                                  kernel_4, kernel_4_idx, scaling_factors_4, zeros_4, kernel_2, kernel_2_idx,
                                  scaling_factors_2, zeros_2, kernel_1, kernel_1_idx, std_1, means_1,
                                  normal_quantiles_center, kernel_new, num_out_channels, num_16, num_8, num_4, num_2, num_1,
                                  new_len, group_size, nh_q, nh_kv):
    """Prototype gemv_cuda.h:139-170."""
    tiers = [(16, kernel_16, kernel_16_idx, None, None), (8, kernel_8, kernel_8_idx, scaling_factors_8, zeros_8),
             (4, kernel_4, kernel_4_idx, scaling_factors_4, zeros_4), (2, kernel_2, kernel_2_idx, scaling_factors_2, zeros_2),
             (1, kernel_1, kernel_1_idx, std_1, means_1)]
    return _wv(in_feats, tiers, kernel_new, group_size, nh_q, nh_kv, False)


def gemv_forward_cuda_wv_group_hq_seq(in_feats, kernel_16, kernel_8, scaling_factors_8, zeros_8, kernel_4, scaling_factors_4,
                                      zeros_4, kernel_2, scaling_factors_2, zeros_2, kernel_1, std_1, means_1,
                                      normal_quantiles_center, kernel_new, num_out_channels, num_16, num_8, num_4, num_2,
                                      num_1, new_len, group_size, nh_q, nh_kv):
    """Prototype gemv_cuda.h:172-198."""
    tiers = [(16, kernel_16, None, None, None), (8, kernel_8, None, scaling_factors_8, zeros_8),
             (4, kernel_4, None, scaling_factors_4, zeros_4), (2, kernel_2, None, scaling_factors_2, zeros_2),
             (1, kernel_1, None, std_1, means_1)]
    return _wv(in_feats, tiers, kernel_new, group_size, nh_q, nh_kv, True)


def __getattr__(name):
    if name.startswith("gemv_forward_cuda"):
        def f(*args, **kwargs):
            raise NotImplementedError(f"kvhq_gemv.{name} is not built in hqekv_b200 (outlier, un-grouped and token-major paths)")
        return f
    raise AttributeError(name)
