"""Importance bookkeeping and block ranking on the GPU — same names and argument meaning as the
hot-path part of the reference's model/public_func.py (lines 58-106 and 208-268), backed by libhqkv
(hqekv_b200/csrc/policy.cu).

The offline helpers of that file (memory-budget ratio solvers, Hadamard weight folding) are not part
of the decode path and are not provided.
"""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_ptr


def calculate_new_token_range(new_cache: torch.Tensor):
    """Per-token (max - min over head_dim) summed over batch and heads, fp16 with a rounding after
    each step (model/public_func.py:75-83).  new_cache fp16 [B, H, T, D] -> fp16 [T]."""
    if new_cache is None:
        return None
    require_cuda(new_cache)
    if new_cache.dtype != torch.float16 or new_cache.dim() != 4:
        raise ValueError("new_cache must be a 4-D float16 tensor")
    B, H, T, D = new_cache.shape
    if new_cache.stride(3) != 1 or new_cache.stride(2) != D:
        new_cache = new_cache.contiguous()
    out = torch.empty(T, dtype=torch.float16, device=new_cache.device)
    with torch.cuda.device(new_cache.device):
        check(lib.hqkv_token_range(ptr(new_cache), B, H, T, D, new_cache.stride(0), new_cache.stride(1), ptr(out),
                                   stream_ptr(new_cache.device)))
    return out


def calculate_token_range(new_cache: torch.Tensor, token_range: torch.Tensor):
    """model/public_func.py:58-73: append the range of the new tokens to ``token_range``."""
    if new_cache is None:
        return None
    new_range = calculate_new_token_range(new_cache)
    return new_range if token_range is None else torch.cat((token_range, new_range), dim=-1)


def get_block_token_idx(block_size: int, block_num: int, importance: torch.Tensor, _range: torch.Tensor = None):
    """model/public_func.py:92-106.  ``importance`` (fp16, block_num*block_size entries, contiguous) is
    divided by the block length IN PLACE, as the reference does to its argument; blocks are ordered by
    descending fp16 key, equal keys by ascending block id (the reference's default torch.sort leaves
    ties unspecified).  Returns the int64 token ids, block by block."""
    require_cuda(importance)
    if importance.dtype != torch.float16 or not importance.is_contiguous():
        raise ValueError("importance must be a contiguous float16 tensor")
    if importance.numel() != block_num * block_size:
        raise ValueError("importance must hold block_num * block_size entries")
    ids = torch.empty(block_num * block_size, dtype=torch.int64, device=importance.device)
    with torch.cuda.device(importance.device):
        check(lib.hqkv_block_rank(ptr(importance), ptr(_range), block_size, block_num, ptr(ids),
                                  stream_ptr(importance.device)))
    return ids


def get_block_importance(block_size: int, block_num: int, importance: torch.Tensor):
    raise NotImplementedError("get_block_importance is not on the decode path; use get_block_token_idx")


def make_sum_equal(array: torch.Tensor, array_sum: int, start_idx: int = 4):
    """Take the rounding surplus off the lowest tiers first (model/public_func.py:259-268).  Host-side
    integer bookkeeping on a 6-entry CPU tensor, as in the reference's model code."""
    sub = array.sum() - array_sum
    for i in range(start_idx, -1, -1):
        if array[i] - sub < 0:
            sub -= array[i]
            array[i] = 0
        else:
            array[i] -= sub
            break
    return array


class last_attn_weights:
    """Rolling buffer of the last ``last_length`` head-summed probability rows and the token importance
    derived from it (model/public_func.py:208-257)."""

    def __init__(self, last_length: int = 20):
        self.last_length = last_length
        self.max_length = 0
        self.kv_seq_len = 0
        self.next_line = 0
        self.weights = None

    def calculate_token_importance(self):
        L = self.kv_seq_len
        out = torch.empty(L, dtype=torch.float16, device=self.weights.device)
        with torch.cuda.device(self.weights.device):
            check(lib.hqkv_token_importance(ptr(self.weights), self.last_length, self.weights.stride(0), L, ptr(out),
                                            stream_ptr(self.weights.device)))
        return out

    def clear(self):
        self.next_line = 0
        self.weights.zero_()

    def eviction(self, reserve_idx):
        """Move the columns of the surviving tokens to the front (:228-231)."""
        if self.weights is None:
            return
        n = reserve_idx.numel()
        kept = torch.empty(self.last_length, n, dtype=self.weights.dtype, device=self.weights.device)
        with torch.cuda.device(self.weights.device):
            check(lib.hqkv_gather_columns_f16(ptr(self.weights), self.weights.stride(0), self.last_length,
                                              ptr(reserve_idx), n, ptr(kept), n, stream_ptr(self.weights.device)))
        self.weights[:, :n] = kept

    def reset(self):
        self.max_length = 0
        self.kv_seq_len = 0
        self.next_line = 0
        self.weights = None

    def set_max_length(self, max_length: int):
        self.max_length = max_length

    def decode_row(self, device) -> torch.Tensor:
        """The ring row that the head sum of the next decode step belongs in, for a decode call that writes it
        itself (``qkv_matmul_hqe_2(..., head_sum_out=row)``, which refuses a row shorter than the cache); follow
        it with ``advance(L)``.  The pair does what ``update`` does on a decode step (:253-255) without a pass of
        its own over the probabilities."""
        if self.weights is None:
            self.weights = torch.zeros(self.last_length, self.max_length, dtype=torch.float16, device=device)
        return self.weights[self.next_line]

    def advance(self, L: int):
        self.kv_seq_len = L
        self.next_line = (self.next_line + 1) % self.last_length

    def update(self, attn_weights: torch.Tensor):
        cap = self.max_length if self.weights is None else self.weights.shape[1]
        if attn_weights.shape[-1] > cap:
            # the reference fails here too (shape mismatch of the row assignment, model/public_func.py:247-255);
            # the kernels below write L halfs into a ring row and must never be handed a shorter one
            raise ValueError(f"attn_weights holds {attn_weights.shape[-1]} positions but the ring is sized for {cap} "
                             "(call set_max_length with the longest sequence before the first update)")
        require_cuda(attn_weights)
        if self.weights is None:
            self.weights = torch.zeros(self.last_length, self.max_length, dtype=attn_weights.dtype,
                                       device=attn_weights.device)
        B, nh, q_len, L = attn_weights.shape
        w = attn_weights if attn_weights.is_contiguous() else attn_weights.contiguous()
        if w.dtype != torch.float16:
            raise ValueError("attn_weights must be float16")
        st = stream_ptr(w.device)
        with torch.cuda.device(w.device):
            if q_len > 1:
                # prefill seeding (:247-252): the last rows of the block fill ring rows 0..rows-1
                rows = min(q_len, self.last_length)
                for r in range(rows):
                    src = w.data_ptr() + (q_len - rows + r) * L * w.element_size()
                    check(lib.hqkv_head_sum(src, B, nh, L, q_len * L, ptr(self.weights[r]), st))
            else:
                # one decode step (:253-255): fixed-order head sum straight into the ring row
                check(lib.hqkv_head_sum(ptr(w), B, nh, L, L, ptr(self.weights[self.next_line]), st))
                rows = 1
        self.kv_seq_len = L
        self.next_line = (self.next_line + rows) % self.last_length
