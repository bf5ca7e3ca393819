"""Operator functions with the reference's names, argument meaning and assertions, running the
sm_100a kernels of libdejavu_b200.so on the current CUDA stream.

Mirrors Dejavu/src/ops/triton/gather_gemv.py (gather_gemv :198-254, gather_transposed_gemv :572-644,
mlp_sparse :647-657) and Dejavu/src/ops/triton/attention_proj_sparse.py (qkv_proj_sparse :110-194,
out_proj_sparse :274-338, v_cache_copy_sparse :396-456, k_cache_copy_sparse :525-590).
Outputs are allocated by the callee with torch.empty, inputs are borrowed, exactly as there.
There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import contextlib
import os

from typing import Optional

import torch

from . import _lib
from ._lib import call

_ACTIVATIONS = ["id", "relu", "gelu", "gelu_approx", "squared_relu"]

_scratch_cache: dict = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("dejavu_b200 operators run on CUDA tensors only (there is no CPU path)")


def _scratch(nbytes: int, device: torch.device) -> torch.Tensor:
    """Zero-initialised per-(device, stream) workspace; the kernels leave their counters zeroed."""
    key = (device.index, _stream())
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(nbytes, 1 << 20)
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _scratch_cache[key] = buf
    return buf


def _idx_args(idx: torch.Tensor):
    assert idx.dtype in (torch.int32, torch.int64), f"idx must be int32 or int64, got {idx.dtype}"
    return idx.contiguous(), 1 if idx.dtype == torch.int64 else 0


def gather_gemv(
    x: torch.Tensor,
    weight: torch.Tensor,
    idx: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    activation: str = "id",
) -> torch.Tensor:
    """y = activation(x @ weight[idx, :].T + bias[idx]);  x (batch, N), weight (Z, N), idx (M,),
    bias (Z,) -> (batch, M) in x.dtype. Indices are not validated (as in the reference)."""
    assert activation in _ACTIVATIONS
    Z, N = weight.shape
    batch, _ = x.shape
    assert x.shape == (batch, N)
    assert 1 <= batch <= _lib.MAX_BATCH, f"batch must be in [1, {_lib.MAX_BATCH}]"
    (M,) = idx.shape
    _require_cuda(x, weight, idx, bias)
    x = x.contiguous()
    if weight.stride(1) > 1:
        weight = weight.contiguous()
    assert x.dtype == weight.dtype, f"Input and weight must have the same dtype, got {x.dtype} and {weight.dtype}"
    assert x.dtype == torch.float16, "only fp16 is implemented"
    if bias is not None:
        bias = bias.contiguous()
        assert bias.shape == (Z,), "Incompatible dimensions in between weight and bias"
        assert x.dtype == bias.dtype, f"Input and bias must have the same dtype, got {x.dtype} and {bias.dtype}"
    idx, idx64 = _idx_args(idx)
    output = torch.empty(batch, M, device=x.device, dtype=x.dtype)
    call("djv_gather_gemv", output.data_ptr(), weight.data_ptr(), x.data_ptr(), idx.data_ptr(), _ptr(bias),
         batch, N, M, weight.stride(0), idx64, _lib.ACT[activation], _stream())
    return output


def dense_gemv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
               activation: str = "id") -> torch.Tensor:
    """y = activation(x @ weight.T + bias) with the same kernel (identity index list)."""
    Z, N = weight.shape
    batch, _ = x.shape
    assert x.shape == (batch, N) and 1 <= batch <= _lib.MAX_BATCH
    _require_cuda(x, weight, bias)
    x = x.contiguous()
    if weight.stride(1) > 1:
        weight = weight.contiguous()
    assert x.dtype == weight.dtype == torch.float16
    output = torch.empty(batch, Z, device=x.device, dtype=x.dtype)
    call("djv_gather_gemv", output.data_ptr(), weight.data_ptr(), x.data_ptr(), None, _ptr(bias),
         batch, N, Z, weight.stride(0), 0, _lib.ACT[activation], _stream())
    return output


def gather_transposed_gemv(
    x: torch.Tensor,
    weight: torch.Tensor,
    idx: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    push_comm=None,
) -> torch.Tensor:
    """y = weight[idx, :]^T @ x + bias;  x (batch, M), weight (Z, N), idx (M,), bias (N,) -> (batch, N).
    Deterministic (fixed summation order), unlike the reference's atomic-add kernel.
    With `push_comm` (a TensorParallelComm) the result is not written to the returned tensor but sent into
    every rank's receive buffer of the exchange; the returned tensor is a placeholder that
    push_comm.allreduce_add_layernorm recognises."""
    Z, N = weight.shape
    (M,) = idx.shape
    batch, _ = x.shape
    assert x.shape == (batch, M)
    assert 1 <= batch <= _lib.MAX_BATCH, f"batch must be in [1, {_lib.MAX_BATCH}]"
    _require_cuda(x, weight, idx, bias)
    x = x.contiguous()
    if weight.stride(1) > 1:
        weight = weight.contiguous()
    assert x.dtype == weight.dtype, f"Input and weight must have the same dtype, got {x.dtype} and {weight.dtype}"
    assert x.dtype == torch.float16, "only fp16 is implemented"
    if bias is not None:
        bias = bias.contiguous()
        assert bias.shape == (N,), "Incompatible dimensions in between weight and bias"
        assert x.dtype == bias.dtype, f"Input and bias must have the same dtype, got {x.dtype} and {bias.dtype}"
    idx, idx64 = _idx_args(idx)
    output = torch.empty(batch, N, device=x.device, dtype=x.dtype)
    lib = _lib.load()
    need = max(lib.djv_gather_transposed_gemv_scratch_bytes(batch, N, M),
               lib.djv_mlp_sparse_fused_scratch_bytes(batch, N, M) if batch <= 4 else 0)
    scratch = _scratch(need, x.device)
    if push_comm is not None and M >= 1 and batch <= 4:
        seq = push_comm.next_seq()
        call("djv_gather_transposed_gemv_push", push_comm.handle, seq, weight.data_ptr(), x.data_ptr(),
             idx.data_ptr(), _ptr(bias), batch, N, M, weight.stride(0), idx64, scratch.data_ptr(), scratch.numel(),
             _stream())
        push_comm.note_pushed(output, seq)
        return output
    call("djv_gather_transposed_gemv", output.data_ptr(), weight.data_ptr(), x.data_ptr(), idx.data_ptr(),
         _ptr(bias), batch, N, M, weight.stride(0), idx64, scratch.data_ptr(), scratch.numel(), _stream())
    return output


def dense_transposed_gemv(x: torch.Tensor, weight_t: torch.Tensor, bias: Optional[torch.Tensor] = None,
                          push_comm=None):
    """y = x @ weight_t + bias with weight_t (M, N) contiguous (a transposed Linear weight), same kernel
    as gather_transposed_gemv with the identity index list."""
    M, N = weight_t.shape
    batch, _ = x.shape
    assert x.shape == (batch, M) and 1 <= batch <= _lib.MAX_BATCH
    _require_cuda(x, weight_t, bias)
    assert weight_t.stride(1) == 1 and x.dtype == weight_t.dtype == torch.float16
    x = x.contiguous()
    output = torch.empty(batch, N, device=x.device, dtype=x.dtype)
    need = _lib.load().djv_gather_transposed_gemv_scratch_bytes(batch, N, M)
    scratch = _scratch(need, x.device)
    if push_comm is not None and batch <= 4:
        seq = push_comm.next_seq()
        call("djv_gather_transposed_gemv_push", push_comm.handle, seq, weight_t.data_ptr(), x.data_ptr(), None,
             _ptr(bias), batch, N, M, weight_t.stride(0), 0, scratch.data_ptr(), scratch.numel(), _stream())
        push_comm.note_pushed(output, seq)
        return output
    call("djv_gather_transposed_gemv", output.data_ptr(), weight_t.data_ptr(), x.data_ptr(), None, _ptr(bias),
         batch, N, M, weight_t.stride(0), 0, scratch.data_ptr(), scratch.numel(), _stream())
    return output


def mlp_sparse(x, W1, W2t, idx, bias1=None, bias2=None, push_comm=None, fused=False):
    """x (batch, d); W1 (4d, d); W2t (4d, d) = W2 transposed, contiguous; bias1 (4d); bias2 (d).
    gather_gemv followed by gather_transposed_gemv, as in the reference; with fused=True one kernel and one pass
    over the gathered rows (batch <= 4, d % 64 == 0; see mlp_sparse_fused_supported). Measured on a B200 the two
    kernels are the faster form when the call stands alone; the one-pass kernel is for the decode step of a
    tensor-parallel shard, where it also takes in the exchange in front of it (mlp_sparse_after_exchange)."""
    batch, N = x.shape
    (M,) = idx.shape
    if fused:
        assert push_comm is None and mlp_sparse_fused_supported(batch, N, M)
        assert x.dtype == W1.dtype == W2t.dtype == torch.float16 and W1.stride(1) == 1 and W2t.stride(1) == 1
        assert W1.shape[1] == N and W2t.shape[1] == N
    if not fused:
        x = gather_gemv(x, W1, idx, bias1, activation="relu")
        return gather_transposed_gemv(x, W2t, idx, bias2, push_comm=push_comm)
    _require_cuda(x, W1, W2t, idx, bias1, bias2)
    x = x.contiguous()
    idx, idx64 = _idx_args(idx)
    if bias1 is not None:
        bias1 = bias1.contiguous()
        assert bias1.shape == (W1.shape[0],) and bias1.dtype == x.dtype
    if bias2 is not None:
        bias2 = bias2.contiguous()
        assert bias2.shape == (N,) and bias2.dtype == x.dtype
    output = torch.empty(batch, N, device=x.device, dtype=x.dtype)
    need = _lib.load().djv_mlp_sparse_fused_scratch_bytes(batch, N, M)
    scratch = _scratch(need, x.device)
    call("djv_mlp_sparse_fused", output.data_ptr(), W1.data_ptr(), W2t.data_ptr(), x.data_ptr(), idx.data_ptr(),
         _ptr(bias1), _ptr(bias2), batch, N, M, W1.shape[0], W1.stride(0), W2t.stride(0), idx64,
         scratch.data_ptr(), scratch.numel(), _stream())
    return output


def mlp_sparse_fused_supported(batch: int, N: int, M: int) -> bool:
    return bool(_lib.load().djv_mlp_sparse_fused_supported(batch, N, M))


def mlp_sparse_after_exchange(comm, partial, residual, norm_weight, norm_bias, eps, W1, W2t, idx, bias1=None,
                              bias2=None, push=True):
    """The second half of a decoder block in one launch:
        r = sum over ranks(partial) + residual;  x = LayerNorm(r);  out = mlp_sparse(x, W1, W2t, idx, bias1, bias2)
    `partial` (batch, d) is a placeholder whose content its producer sent as an exchange of `comm`. With
    `push` the result is sent as the next exchange (the returned `out` is then a placeholder for it), otherwise
    it is stored. Returns (out, r)."""
    batch, N = partial.shape
    (M,) = idx.shape
    seq_in = comm.take_pushed(partial)
    assert seq_in is not None, "partial must have been sent by its producer"
    _require_cuda(partial, residual, W1, W2t, idx, bias1, bias2)
    idx, idx64 = _idx_args(idx)
    out = torch.empty(batch, N, device=partial.device, dtype=partial.dtype)
    r = torch.empty(batch, N, device=partial.device, dtype=partial.dtype)
    need = _lib.load().djv_mlp_sparse_fused_scratch_bytes(batch, N, M)
    scratch = _scratch(need, partial.device)
    seq_out = comm.next_seq() if push else -1
    call("djv_mlp_sparse_fused_exchange", comm.handle, seq_in, _lib.EXCHANGE_REFILL, seq_out,
         None if push else out.data_ptr(), r.data_ptr(), _ptr(None if residual is None else residual.contiguous()),
         norm_weight.data_ptr(), norm_bias.data_ptr(), float(eps), W1.data_ptr(), W2t.data_ptr(), idx.data_ptr(),
         _ptr(bias1), _ptr(bias2), batch, N, M, W1.shape[0], W1.stride(0), W2t.stride(0), idx64,
         scratch.data_ptr(), scratch.numel(), _stream())
    if push:
        comm.note_pushed(out, seq_out)
    return out, r


def qkv_proj_sparse(
    x: torch.Tensor,
    weight: torch.Tensor,
    head_idx: torch.Tensor,
    batch_idx: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """y = einsum("bm,thdm->bthd", x, weight) + bias for the heads in head_idx and the rows named by the
    non-negative entries of batch_idx; every other entry of y is uninitialised (torch.empty)."""
    three, nheads, head_dim, hidden_dim = weight.shape
    assert three == 3
    assert head_dim in [32, 64, 128]
    assert hidden_dim % 128 == 0
    batch_size, _ = x.shape
    assert batch_size <= 16
    assert x.shape == (batch_size, hidden_dim)
    n_active = head_idx.shape[0]
    assert n_active <= nheads
    assert head_idx.shape == (n_active,)
    assert head_idx.dtype == torch.int32
    assert batch_idx.shape == (n_active, batch_size)
    assert batch_idx.dtype == torch.int32
    _require_cuda(x, weight, head_idx, batch_idx, bias)
    x = x.contiguous()
    weight = weight.contiguous()
    head_idx = head_idx.contiguous()
    batch_idx = batch_idx.contiguous()
    assert x.dtype == weight.dtype, f"Input and weight must have the same dtype, got {x.dtype} and {weight.dtype}"
    assert x.dtype == torch.float16, "only fp16 is implemented"
    if bias is not None:
        bias = bias.contiguous()
        assert bias.shape == (3, nheads, head_dim), "Incompatible dimensions in between weight and bias"
        assert x.dtype == bias.dtype, f"Input and bias must have the same dtype, got {x.dtype} and {bias.dtype}"
    output = torch.empty(batch_size, 3, nheads, head_dim, device=x.device, dtype=x.dtype)
    call("djv_qkv_proj_sparse", output.data_ptr(), weight.data_ptr(), x.data_ptr(), head_idx.data_ptr(),
         batch_idx.data_ptr(), _ptr(bias), batch_size, hidden_dim, nheads, head_dim, n_active, _stream())
    return output


def out_proj_sparse(
    x: torch.Tensor,
    weight: torch.Tensor,
    head_idx: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """y = einsum("bhd,nhd->bn", x, weight) + bias over the heads in head_idx only.
    x (batch, nheads, head_dim), weight (hidden_dim, nheads, head_dim) -> (batch, hidden_dim)."""
    hidden_dim, nheads, head_dim = weight.shape
    assert head_dim in [32, 64, 128]
    assert hidden_dim % 128 == 0
    batch, _, _ = x.shape
    assert x.shape == (batch, nheads, head_dim)
    n_active = head_idx.shape[0]
    assert head_idx.shape == (n_active,)
    assert head_idx.dtype == torch.int32
    assert batch <= 16
    _require_cuda(x, weight, head_idx, bias)
    x = x.contiguous()
    weight = weight.contiguous()
    head_idx = head_idx.contiguous()
    assert x.dtype == weight.dtype, f"Input and weight must have the same dtype, got {x.dtype} and {weight.dtype}"
    assert x.dtype == torch.float16, "only fp16 is implemented"
    if bias is not None:
        bias = bias.contiguous()
        assert bias.shape == (hidden_dim,), "Incompatible dimensions in between weight and bias"
        assert x.dtype == bias.dtype, f"Input and bias must have the same dtype, got {x.dtype} and {bias.dtype}"
    output = torch.empty(batch, hidden_dim, device=x.device, dtype=x.dtype)
    call("djv_out_proj_sparse", output.data_ptr(), weight.data_ptr(), x.data_ptr(), head_idx.data_ptr(), None,
         _ptr(bias), batch, hidden_dim, nheads, head_dim, n_active, _stream())
    return output


def _cache_copy(fn, src, cache, head_idx, seqlen_idx, padding, S, head_dim):
    nnz_seqlen, nheads, _ = src.shape
    n_active = head_idx.shape[0]
    assert head_dim in [32, 64, 128]
    assert nnz_seqlen <= 16
    assert n_active <= nheads
    assert head_idx.shape == (n_active,)
    assert head_idx.dtype == torch.int32
    assert seqlen_idx.shape == (n_active, nnz_seqlen)
    assert seqlen_idx.dtype == torch.int32
    assert src.dtype == cache.dtype, f"k/v and cache must have the same dtype, got {src.dtype} and {cache.dtype}"
    assert src.dtype == torch.float16, "only fp16 is implemented"
    assert src.stride(-1) == 1 and cache.is_contiguous()
    _require_cuda(src, cache, head_idx, seqlen_idx, padding)
    if padding is not None:
        assert padding.shape == (1,)
        assert padding.dtype == torch.int32
    head_idx = head_idx.contiguous()
    seqlen_idx = seqlen_idx.contiguous()
    call(fn, src.data_ptr(), cache.data_ptr(), head_idx.data_ptr(), seqlen_idx.data_ptr(), _ptr(padding),
         nnz_seqlen, nheads, head_dim, S, n_active, src.stride(0), src.stride(1), _stream())


def v_cache_copy_sparse(v, v_cache, head_idx, seqlen_idx, padding=None) -> None:
    """v (nnz_seqlen, nheads, head_dim) -> v_cache (1, nheads, seqlen, head_dim) at the positions
    seqlen_idx[i, t] + padding for head head_idx[i]; negative positions are skipped."""
    nnz_seqlen, nheads, head_dim = v.shape
    _, _, seqlen, _ = v_cache.shape
    assert v_cache.shape == (1, nheads, seqlen, head_dim)
    _cache_copy("djv_v_cache_copy_sparse", v, v_cache, head_idx, seqlen_idx, padding, seqlen, head_dim)


def k_cache_copy_sparse(k, k_cache, head_idx, seqlen_idx, padding=None) -> None:
    """k (nnz_seqlen, nheads, head_dim) -> k_cache (1, nheads, head_dim/8, seqlen, 8), same rules."""
    nnz_seqlen, nheads, head_dim = k.shape
    _, _, _, seqlen, _ = k_cache.shape
    assert k_cache.shape == (1, nheads, head_dim // 8, seqlen, 8)
    _cache_copy("djv_k_cache_copy_sparse", k, k_cache, head_idx, seqlen_idx, padding, seqlen, head_dim)


# ---- L2 warm-up (hints; no counterpart in the reference) ---------------------------------------------

def prefetch_rows_l2(idx: torch.Tensor, *weights: torch.Tensor, rows_per_index: int = 1):
    """Ask for rows idx[m] of up to three (Z, N) matrices to be brought into L2. With rows_per_index = r an index
    names r consecutive rows (a head's slab of a (heads * r, N) matrix)."""
    assert 1 <= len(weights) <= 3
    w0 = weights[0]
    _require_cuda(idx, *weights)
    for w in weights:
        assert w.dtype == torch.float16 and w.stride(1) == 1 and w.shape == w0.shape and w.stride(0) == w0.stride(0)
    assert rows_per_index == 1 or w0.stride(0) == w0.shape[1], "a slab of several rows must be contiguous"
    idx, idx64 = _idx_args(idx)
    ptrs = [w.data_ptr() for w in weights] + [None] * (3 - len(weights))
    call("djv_prefetch_rows_l2", ptrs[0], ptrs[1], ptrs[2], idx.data_ptr(), idx64, idx.numel(),
         w0.shape[0] // rows_per_index, w0.stride(0) * 2 * rows_per_index, w0.shape[1] * 2 * rows_per_index,
         _stream())


def prefetch_head_columns_l2(head_idx: torch.Tensor, weight: torch.Tensor, head_dim: int):
    """Ask for the columns of a (rows, heads * head_dim) matrix that belong to the listed heads (int32)."""
    _require_cuda(head_idx, weight)
    assert head_idx.dtype == torch.int32 and weight.dtype == torch.float16 and weight.stride(1) == 1
    assert (head_dim * 2) % 128 == 0
    call("djv_prefetch_segments_l2", weight.data_ptr(), head_idx.contiguous().data_ptr(), head_idx.numel(),
         weight.shape[1] // head_dim, weight.shape[0], weight.stride(0) * 2, head_dim * 2, _stream())


# ---- operators the reference obtains from torch / third-party extensions -------------------------

def topk_indices(scores: torch.Tensor, k: int, dtype: torch.dtype = torch.int64) -> torch.Tensor:
    """Indices of the k largest entries of a 1-D fp16/fp32 score vector, ascending index order, ties on
    the k-th value resolved towards the lowest index. Stands in for `scores.topk(k, sorted=False)[1]`
    (Dejavu/src/models/modules/mha_dejavu.py:1069, 1369, 1506)."""
    assert scores.dim() == 1 and scores.dtype in (torch.float16, torch.float32)
    assert dtype in (torch.int32, torch.int64)
    n = scores.shape[0]
    assert 0 <= k <= n
    _require_cuda(scores)
    scores = scores.contiguous()
    out = torch.empty(k, dtype=dtype, device=scores.device)
    a32, a64 = (out.data_ptr(), None) if dtype == torch.int32 else (None, out.data_ptr())
    call("djv_topk", a32, a64, scores.data_ptr(), n, k, 1 if scores.dtype == torch.float32 else 0, _stream())
    return out


def batch_sum(x: torch.Tensor) -> torch.Tensor:
    """(B, N) fp16 -> (1, N): the rows added in fp32, rounded once (djv_batch_sum)."""
    assert x.is_cuda and x.dtype == torch.float16 and x.dim() == 2
    x = x.contiguous()
    y = torch.empty(1, x.size(1), dtype=x.dtype, device=x.device)
    call("djv_batch_sum", y.data_ptr(), x.data_ptr(), x.size(0), x.size(1), _stream())
    return y


@contextlib.contextmanager
def indices_ready(ready: bool = True):
    """Inside this block the caller promises that the index lists / attention state passed to the operators
    are complete before the kernels can start (produced on another stream and joined with an event): the
    kernels then prefetch their weight rows while the kernel launched before them is still running
    (see djv_set_early_weight_prefetch)."""
    lib = _lib.load()
    if ready:
        lib.djv_set_early_weight_prefetch(1)
    try:
        yield
    finally:
        if ready:
            lib.djv_set_early_weight_prefetch(0)


def topk_indices_open_step(scores: torch.Tensor, k: int, state: torch.Tensor, cache_len: int) -> torch.Tensor:
    """topk_indices(scores, k, int32) over one score per head, fused with the head-selection half of the
    decode step of the attention layer the selection is for: `state` is that layer's lazy-K/V state
    (see djv_topk_attn_prep). The layer then runs its step with step_is_open = 1."""
    assert scores.dim() == 1 and scores.dtype in (torch.float16, torch.float32)
    n = scores.shape[0]
    assert 1 <= k <= n <= 1024 and state.dtype == torch.int32
    _require_cuda(scores, state)
    scores = scores.contiguous()
    out = torch.empty(k, dtype=torch.int32, device=scores.device)
    call("djv_topk_attn_prep", out.data_ptr(), scores.data_ptr(), n, k, 1 if scores.dtype == torch.float32 else 0,
         state.data_ptr(), cache_len, _stream())
    return out


def add_layernorm(x, residual, weight, bias, eps: float, xbias=None):
    """r = x + residual (+ xbias); y = LayerNorm(r). Returns (y, r). x, residual (batch, d) fp16.
    Stands in for `residual = dropped + residual; hidden = norm(residual)`
    (Dejavu/src/models/modules/block_dejavu.py:575-584, 625-636)."""
    batch, d = x.shape
    _require_cuda(x, residual, weight, bias, xbias)
    assert x.dtype == torch.float16 and weight.dtype == torch.float16 and bias.dtype == torch.float16
    x = x.contiguous()
    if residual is not None:
        assert residual.shape == x.shape and residual.dtype == x.dtype
        residual = residual.contiguous()
    y = torch.empty_like(x)
    r = torch.empty_like(x)
    call("djv_add_layernorm", y.data_ptr(), r.data_ptr(), x.data_ptr(), _ptr(residual), _ptr(xbias),
         weight.data_ptr(), bias.data_ptr(), batch, d, float(eps), _stream())
    return y, r


def decode_attention(q, k_cache, v_cache, head_idx, length: int, softmax_scale: float):
    """ctx[b,h] = softmax(scale * q[b,h] . K[b,h,:length]) V[b,h,:length] for h in head_idx (or all heads
    when head_idx is None); rows of other heads are uninitialised. q (B, nheads, hd);
    k_cache (B, nheads, hd/8, S, 8); v_cache (B, nheads, S, hd). Stands in for
    ft_attention.single_query_attention at Dejavu/src/models/modules/mha_dejavu.py:1439-1446."""
    B, nheads, hd = q.shape
    S = v_cache.shape[2]
    assert v_cache.shape == (B, nheads, S, hd) and k_cache.shape == (B, nheads, hd // 8, S, 8)
    assert q.dtype == k_cache.dtype == v_cache.dtype == torch.float16
    assert 0 <= length <= S
    _require_cuda(q, k_cache, v_cache, head_idx)
    q = q.contiguous()
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    nnz = nheads
    if head_idx is not None:
        assert head_idx.dtype == torch.int32 and head_idx.dim() == 1
        head_idx = head_idx.contiguous()
        nnz = head_idx.shape[0]
    ctx = torch.empty_like(q)
    need = _lib.load().djv_decode_attn_scratch_bytes(max(nnz, 1), B, hd, S)
    scratch = _scratch(need, q.device)
    call("djv_decode_attn", ctx.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _ptr(head_idx),
         nnz, B, nheads, hd, S, length, float(softmax_scale), scratch.data_ptr(), scratch.numel(), _stream())
    return ctx
