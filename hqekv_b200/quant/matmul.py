"""Batched GEMV of fp16 activations with one packed tier — same names and argument meaning as
cuda_bmm_fA_qB_uniform_group / cuda_bmm_fA_qB_normal_group in the reference's quant/matmul.py:263-299,
72-95, backed by hqkv_gemv_uniform_group / hqkv_gemv_normal_group (hqekv_b200/csrc/gemv.cu).

The reference flattens (B, nh) and makes transposed contiguous copies of the codes, scales and
zeros on every call before entering its extension; here the operands are read in the layout the
cache stores them in.
"""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_ptr


def _gemv(entry, widths, group_size, fA, qB, scales, zeros, bits):
    """C = fA x dequant(qB) with fp32 accumulation.

    fA     (B, nh_q, 1, K) float16
    qB     (B, nh_kv, K, N // feat_per_int) int32
    scales (B, nh_kv, K, N // group_size) float16
    zeros  (B, nh_kv, K, N // group_size) float16
    Returns C (B, nh_q, 1, N) float16.
    """
    require_cuda(fA, qB, scales, zeros)
    if fA.dim() != 4 or qB.dim() != 4:
        raise ValueError("invalid matrix.")
    B, nh_q, M, K = fA.shape
    if M != 1:
        raise ValueError("invalid matrix.")  # decode only: one query row, as in the reference's kernels
    nh_kv = qB.shape[1]
    if qB.shape[2] != K or bits not in widths:
        raise ValueError("invalid matrix.")
    N = qB.shape[3] * (32 // bits)
    fA, qB, scales, zeros = fA.contiguous(), qB.contiguous(), scales.contiguous(), zeros.contiguous()
    out = torch.empty(B, nh_q, 1, N, dtype=torch.float16, device=fA.device)
    with torch.cuda.device(fA.device):
        check(entry(ptr(fA), ptr(qB), ptr(scales), ptr(zeros), B, nh_q, nh_kv, K, N, group_size, bits, ptr(out),
                    stream_ptr(fA.device)))
    return out


def cuda_bmm_fA_qB_uniform_group(group_size: int, fA: torch.Tensor, qB: torch.Tensor, scales: torch.Tensor,
                                 zeros: torch.Tensor, bits: int) -> torch.Tensor:
    """quant/matmul.py:263-299; shapes as in :func:`_gemv`, bits 8, 4, 2 or 1."""
    return _gemv(lib.hqkv_gemv_uniform_group, (8, 4, 2, 1), group_size, fA, qB, scales, zeros, bits)


def cuda_bmm_fA_qB_normal_group(group_size: int, fA: torch.Tensor, qB: torch.Tensor, stds: torch.Tensor,
                                means: torch.Tensor, bits: int) -> torch.Tensor:
    """quant/matmul.py:72-95 at bits = 1 (Gaussian codebook: std * (+-0.67448974) + mean); wider
    codebooks raise NotImplementedError."""
    if bits != 1:
        raise NotImplementedError("cuda_bmm_fA_qB_normal_group: only bits = 1 is built in hqekv_b200")
    return _gemv(lib.hqkv_gemv_normal_group, (1,), group_size, fA, qB, stds, means, bits)


def _side_desc(side, group_size, nh_kv, nh_q, tiers, residual, sequential):
    """CacheDesc holding one side of a cache.  tiers: [(bits, data, idx, scale, zero)] in tier order."""
    from .._lib import CODEC_NORMAL, CacheDesc
    desc = CacheDesc()
    keep = []
    B = D = dev = None
    at = 0
    for t, (bits, data, idx, scale, zero) in enumerate(tiers):
        tier = desc.tier[t]
        tier.bits = bits
        if data is None:
            continue
        data = data.contiguous()
        B, dev = data.shape[0], data.device
        fpi = 1 if bits == 16 else 32 // bits
        if side == "K":
            D, n = data.shape[2], data.shape[3] * fpi
        else:
            D, n = data.shape[3] * fpi, data.shape[2]
        if sequential:
            idx = torch.arange(at, at + n, dtype=torch.int64, device=dev)
        elif idx is None or idx.numel() != n or idx.dtype != torch.int64:
            raise ValueError("invalid matrix.")
        at += n
        scale = None if scale is None else scale.contiguous()
        zero = None if zero is None else zero.contiguous()
        idx = idx.contiguous()
        keep += [data, idx, scale, zero]
        tier.codec = CODEC_NORMAL if bits == 1 else 0
        if side == "K":
            tier.n_k, tier.k_data, tier.k_idx, tier.k_scale, tier.k_zero = n, ptr(data), ptr(idx), ptr(scale), ptr(zero)
        else:
            tier.n_v, tier.v_data, tier.v_idx, tier.v_scale, tier.v_zero = n, ptr(data), ptr(idx), ptr(scale), ptr(zero)
    r = 0
    if residual is not None:
        residual = residual.contiguous()
        B, _, r, D = residual.shape
        dev = residual.device
        keep.append(residual)
        if side == "K":
            desc.new_k = ptr(residual)
        else:
            desc.new_v = ptr(residual)
    if B is None:
        raise ValueError("invalid matrix.")
    desc.B, desc.H, desc.nh_q, desc.D, desc.n_new = B, nh_kv, nh_q, D, r
    desc.group_k = desc.group_v = group_size
    desc.softmax_scale = 1.0
    return desc, keep, at + r, dev


def _qk_group_hq(group_size, nh_kv, in_vector, tiers, new_K, sequential):
    from .._lib import decode_workspace
    require_cuda(in_vector)
    if in_vector.dim() != 4 or in_vector.shape[2] != 1:
        raise ValueError("invalid matrix.")
    desc, keep, L, dev = _side_desc("K", group_size, nh_kv, in_vector.shape[1], tiers, new_K, sequential)
    q = in_vector.contiguous()
    out = torch.empty(q.shape[0], q.shape[1], 1, L, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        st = stream_ptr(dev)
        ws = decode_workspace(dev, lib.hqkv_decode_workspace_bytes(desc), st)
        check(lib.hqkv_decode_logits(desc, ptr(q), ptr(out), ptr(ws), ws.numel(), st))
    return out


def _wv_group_hq(group_size, nh_kv, in_vector, tiers, new_V, sequential):
    from .._lib import decode_workspace
    require_cuda(in_vector)
    if in_vector.dim() != 4 or in_vector.shape[2] != 1:
        raise ValueError("invalid matrix.")
    desc, keep, L, dev = _side_desc("V", group_size, nh_kv, in_vector.shape[1], tiers, new_V, sequential)
    if in_vector.shape[3] != L:
        raise ValueError("invalid matrix.")
    w = in_vector.contiguous()
    out = torch.empty(w.shape[0], w.shape[1], 1, desc.D, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        st = stream_ptr(dev)
        ws = decode_workspace(dev, lib.hqkv_decode_workspace_bytes(desc), st)
        check(lib.hqkv_decode_weighted_sum(desc, ptr(w), ptr(out), ptr(ws), ws.numel(), st))
    return out


def cuda_bmm_forward_qk_group_hq(group_size, nh_kv, in_vector, matrix_16, matrix_16_idx, matrix_8, matrix_8_idx, scales_8,
                                 zeros_8, matrix_4, matrix_4_idx, scales_4, zeros_4, matrix_2, matrix_2_idx, scales_2,
                                 zeros_2, matrix_1, matrix_1_idx, std_1, means_1, new_K):
    """quant/matmul.py:351-434: raw q.K^T over every K tier (uniform-group 8 / 4 / 2 bit, Gaussian-codebook 1 bit,
    fp16 tier) and the residual window, each token's product written at its logical position; one K pass.
    in_vector [B, nh_q, 1, D] fp16; tiers in the cache layout ([B, nh_kv, D, n * bits / 32]); returns
    [B, nh_q, 1, L] fp16 (not yet divided by sqrt(head_dim), as in the reference)."""
    tiers = [(16, matrix_16, matrix_16_idx, None, None), (8, matrix_8, matrix_8_idx, scales_8, zeros_8),
             (4, matrix_4, matrix_4_idx, scales_4, zeros_4), (2, matrix_2, matrix_2_idx, scales_2, zeros_2),
             (1, matrix_1, matrix_1_idx, std_1, means_1)]
    return _qk_group_hq(group_size, nh_kv, in_vector, tiers, new_K, False)


def cuda_bmm_forward_qk_group_hq_seq(group_size, nh_kv, in_vector, matrix_16, matrix_8, scales_8, zeros_8, matrix_4,
                                     scales_4, zeros_4, matrix_2, scales_2, zeros_2, matrix_1, std_1, means_1, new_K):
    """quant/matmul.py:436-505: the same over the sequential layout (no index lists: tier order, then the residual)."""
    tiers = [(16, matrix_16, None, None, None), (8, matrix_8, None, scales_8, zeros_8), (4, matrix_4, None, scales_4, zeros_4),
             (2, matrix_2, None, scales_2, zeros_2), (1, matrix_1, None, std_1, means_1)]
    return _qk_group_hq(group_size, nh_kv, in_vector, tiers, new_K, True)


def cuda_bmm_forward_wv_group_hq(group_size, nh_kv, in_vector, matrix_16, matrix_16_idx, matrix_8, matrix_8_idx, scales_8,
                                 zeros_8, matrix_4, matrix_4_idx, scales_4, zeros_4, matrix_2, matrix_2_idx, scales_2,
                                 zeros_2, matrix_1, matrix_1_idx, std_1, means_1, new_V):
    """quant/matmul.py:507-579: sum over all cached tokens of weight x dequantised V row, the weight of a token
    read at its logical position; one V pass.  in_vector [B, nh_q, 1, L] fp16; V tiers in the cache layout
    ([B, nh_kv, n, D * bits / 32]); returns [B, nh_q, 1, D] fp16."""
    tiers = [(16, matrix_16, matrix_16_idx, None, None), (8, matrix_8, matrix_8_idx, scales_8, zeros_8),
             (4, matrix_4, matrix_4_idx, scales_4, zeros_4), (2, matrix_2, matrix_2_idx, scales_2, zeros_2),
             (1, matrix_1, matrix_1_idx, std_1, means_1)]
    return _wv_group_hq(group_size, nh_kv, in_vector, tiers, new_V, False)


def cuda_bmm_forward_wv_group_hq_seq(group_size, nh_kv, in_vector, matrix_16, matrix_8, scales_8, zeros_8, matrix_4,
                                     scales_4, zeros_4, matrix_2, scales_2, zeros_2, matrix_1, std_1, means_1, new_V):
    """quant/matmul.py:581-649: the same over the sequential layout."""
    tiers = [(16, matrix_16, None, None, None), (8, matrix_8, None, scales_8, zeros_8), (4, matrix_4, None, scales_4, zeros_4),
             (2, matrix_2, None, scales_2, zeros_2), (1, matrix_1, None, std_1, means_1)]
    return _wv_group_hq(group_size, nh_kv, in_vector, tiers, new_V, True)


def _not_built(name):
    def f(*args, **kwargs):
        raise NotImplementedError(f"{name}: this variant of the reference's GEMV wrappers is not built in hqekv_b200 "
                                  "(outlier, un-grouped and token-major paths)")
    f.__name__ = name
    return f


cuda_bmm_fA_qB_normal = _not_built("cuda_bmm_fA_qB_normal")
cuda_bmm_fA_qB_uniform = _not_built("cuda_bmm_fA_qB_uniform")
# names quant/hqe_matmul.py:10-24 of the reference imports next to the ones above: outlier and token-major paths
cuda_bmm_forward_qk_uniform_group_token = _not_built("cuda_bmm_forward_qk_uniform_group_token")
cuda_bmm_forward_qk_normal_group_token = _not_built("cuda_bmm_forward_qk_normal_group_token")
cuda_bmm_forward_wv_group_outlier_hq = _not_built("cuda_bmm_forward_wv_group_outlier_hq")
cuda_bmm_fA_qB_uniform_group_outlier = _not_built("cuda_bmm_fA_qB_uniform_group_outlier")
cuda_bmm_fA_qB_wv_uniform_group = _not_built("cuda_bmm_fA_qB_wv_uniform_group")
cuda_bmm_fA_qB_wv_uniform_group_outlier = _not_built("cuda_bmm_fA_qB_wv_uniform_group_outlier")
cuda_bmm_fA_qB_normal_group_outlier = _not_built("cuda_bmm_fA_qB_normal_group_outlier")
cuda_bmm_fA_qB_wv_normal_group = _not_built("cuda_bmm_fA_qB_wv_normal_group")
cuda_bmm_fA_qB_wv_normal_group_outlier = _not_built("cuda_bmm_fA_qB_wv_normal_group_outlier")
cuda_bmm_fA_qB_normal_outlier = _not_built("cuda_bmm_fA_qB_normal_outlier")
cuda_bmm_fA_qB_uniform_outlier = _not_built("cuda_bmm_fA_qB_uniform_outlier")
