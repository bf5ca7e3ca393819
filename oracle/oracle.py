"""CPU restatement of the reference's contextual-sparse decode math (plain torch, no kernels).

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this file; it is the checker used by
tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference arm.

Every function cites the reference text (path inside FMInference/DejaVu, file:line) it restates.
Parity status: PINNED for the operator level (gather_gemv, gather_transposed_gemv, mlp_sparse,
qkv_proj_sparse, out_proj_sparse, k/v_cache_copy_sparse) against outputs of the reference's own Triton
kernels executed with Triton's CPU interpreter, and for the mask-form block against the reference's
Decentralized_FM_alpha/modules/hf_opt_sparse_mlp_attention.py run on CPU; the vectors and the script that
made them are in tests/golden/. Decode attention and top-K tie-breaking live in third-party code the
reference does not vendor (flash-attention v0.2.8 csrc/ft_attention; torch.topk): they are restated as
standard softmax attention and as a stable "score descending, index ascending" selection, and are
cross-checked against the mask-form attention of hf_opt_sparse_mlp_attention.py.

Arithmetic convention: inputs keep their dtype (fp16 on the latency path), every product is accumulated
in fp32, and results are rounded to the activation dtype at exactly the places the reference does.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

KV_WINDOW = 16  # Dejavu/src/models/modules/mha_dejavu.py:1243 (x_cache of 16 rows)


def _act(x: torch.Tensor, activation: str) -> torch.Tensor:
    # Dejavu/src/ops/triton/k_activations.py:56-162
    if activation == "id":
        return x
    if activation == "relu":
        return torch.relu(x)
    if activation == "gelu":
        return F.gelu(x)
    if activation == "gelu_approx":
        return F.gelu(x, approximate="tanh")
    if activation == "squared_relu":
        return torch.relu(x) ** 2
    raise ValueError(activation)


# ---------------------------------------------------------------------------------------------
# sparse MLP operators
# ---------------------------------------------------------------------------------------------
def gather_gemv(x, weight, idx, bias=None, activation="id"):
    """y = activation(x @ weight[idx, :].T + bias[idx]) — Dejavu/src/ops/triton/gather_gemv.py:206
    (kernel docstring :68-75); fp32 accumulate, output in x.dtype (:233)."""
    w = torch.index_select(weight, 0, idx.long()).float()
    y = x.float() @ w.T
    if bias is not None:
        y = y + torch.index_select(bias, 0, idx.long()).float()
    return _act(y, activation).to(x.dtype)


def gather_transposed_gemv(x, weight, idx, bias=None):
    """y = weight[idx, :]^T @ x + bias — Dejavu/src/ops/triton/gather_gemv.py:579; fp32 accumulate
    (:608-613), cast to x.dtype at the end (:644)."""
    w = torch.index_select(weight, 0, idx.long()).float()
    y = x.float() @ w
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def mlp_sparse(x, W1, W2t, idx, bias1=None, bias2=None):
    """Dejavu/src/ops/triton/gather_gemv.py:647-657: relu gather-GEMV then transposed gather-GEMV; the
    intermediate is an x.dtype tensor."""
    h = gather_gemv(x, W1, idx, bias1, activation="relu")
    return gather_transposed_gemv(h, W2t, idx, bias2)


def mlp_mask_form(x, W1, b1, W2, b2, idx):
    """The accuracy path's formulation of the same product:
    fc1 -> * mask -> ReLU -> F.linear(., fc2) with mask = scatter(idx)
    (Decentralized_FM_alpha/modules/hf_opt_sparse_mlp_attention.py:549-556, mask built at :493-501).
    W2 is (d, ffn). All math in the dtype promoted to fp32."""
    h = F.linear(x.float(), W1.float(), None if b1 is None else b1.float())
    mask = torch.zeros(W1.shape[0], dtype=torch.float32)
    mask[idx.long()] = 1.0
    h = torch.relu(h * mask)
    return F.linear(h, W2.float(), None if b2 is None else b2.float())


def predictor_scores(x, fc0_w, fc1_w):
    """logit = fc1(fc0(x)), two bias-free linears (Dejavu/src/ops/fused_dense_sparse_dejavu.py:59-76,
    Decentralized_FM_alpha/modules/hf_opt_sparse_mlp_attention.py:430-433). Each linear returns a tensor
    of x.dtype, so the rank-R intermediate is rounded once."""
    t = (x.float() @ fc0_w.float().T).to(x.dtype)
    return (t.float() @ fc1_w.float().T).to(x.dtype)


def topk_indices(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Index set of the k largest scores (mlp_sp_logit.topk(k, sorted=False),
    Dejavu/src/models/modules/mha_dejavu.py:1369, 1506). torch.topk leaves tie order unspecified; the rule
    here is score descending, then index ascending; NaN ranks highest. Returned ascending by index."""
    assert scores.dim() == 1
    s = scores.float()
    s = torch.where(torch.isnan(s), torch.full_like(s, float("inf")), s)
    # NaN > +inf: give NaN its own top rank
    rank_key = torch.where(torch.isnan(scores.float()), torch.ones_like(s), torch.zeros_like(s))
    order = sorted(range(s.numel()), key=lambda i: (-rank_key[i].item(), -s[i].item(), i))
    return torch.tensor(sorted(order[:k]), dtype=torch.int64)


def topk_indices_fast(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Same rule as topk_indices, vectorised (stable sort) for large vectors."""
    s = scores.float()
    nan = torch.isnan(s)
    s = torch.where(nan, torch.full_like(s, float("inf")), s)
    key = torch.stack([nan.float(), s], 0)
    # stable sort by score descending keeps index-ascending order among ties; NaN first
    order = torch.argsort(-key[1], stable=True)
    order = order[torch.argsort(-key[0][order], stable=True)]
    return torch.sort(order[:k]).values.to(torch.int64)


# ---------------------------------------------------------------------------------------------
# head-sparse attention operators
# ---------------------------------------------------------------------------------------------
def qkv_proj_sparse(x, weight, head_idx, batch_idx, bias=None):
    """einsum("thdn,bn->bthd", W, x) + bias restricted to head_idx and to the rows named by the
    non-negative entries of batch_idx (Dejavu/src/ops/triton/attention_proj_sparse.py:118-125, smoke
    block :625). Entries that the reference leaves uninitialised are returned as NaN."""
    three, nheads, hd, d = weight.shape
    T = x.shape[0]
    y = torch.full((T, 3, nheads, hd), float("nan"), dtype=torch.float32)
    for i, h in enumerate(head_idx.tolist()):
        for t in batch_idx[i].tolist():
            if t < 0:
                continue
            v = torch.einsum("qdn,n->qd", weight[:, h].float(), x[t].float())
            if bias is not None:
                v = v + bias[:, h].float()
            y[t, :, h] = v
    return y.to(x.dtype)


def out_proj_sparse(x, weight, head_idx, bias=None):
    """einsum("nhd,bhd->bn", W[:, head_idx], x[:, head_idx]) + bias
    (Dejavu/src/ops/triton/attention_proj_sparse.py:281-286, smoke block :646)."""
    hi = head_idx.long()
    y = torch.einsum("nhd,bhd->bn", weight[:, hi].float(), x[:, hi].float())
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def k_cache_copy_sparse(k, k_cache, head_idx, seqlen_idx, padding=None):
    """k (T,nheads,hd) -> k_cache (1,nheads,hd/8,S,8) at position seqlen_idx+padding, source row
    seqlen_idx (Dejavu/src/ops/triton/attention_proj_sparse.py:459-523)."""
    pad = 0 if padding is None else int(padding.item())
    hd = k.shape[2]
    for i, h in enumerate(head_idx.tolist()):
        for t in seqlen_idx[i].tolist():
            if t >= 0:
                k_cache[0, h, :, t + pad, :] = k[t, h].reshape(hd // 8, 8)


def v_cache_copy_sparse(v, v_cache, head_idx, seqlen_idx, padding=None):
    """v (T,nheads,hd) -> v_cache (1,nheads,S,hd) (attention_proj_sparse.py:341-393)."""
    pad = 0 if padding is None else int(padding.item())
    for i, h in enumerate(head_idx.tolist()):
        for t in seqlen_idx[i].tolist():
            if t >= 0:
                v_cache[0, h, t + pad, :] = v[t, h]


def pack_k_cache(k: torch.Tensor) -> torch.Tensor:
    """(B, S, nheads, hd) -> (B, nheads, hd/8, S, 8): the decode kernel's K layout
    (Dejavu/src/models/modules/mha_dejavu.py:385-447, packsize 8 for fp16)."""
    B, S, nh, hd = k.shape
    return k.permute(0, 2, 3, 1).reshape(B, nh, hd // 8, 8, S).permute(0, 1, 2, 4, 3).contiguous()


def unpack_k_cache(k_cache: torch.Tensor) -> torch.Tensor:
    """(B, nheads, hd/8, S, 8) -> (B, nheads, S, hd)."""
    B, nh, c, S, p = k_cache.shape
    return k_cache.permute(0, 1, 3, 2, 4).reshape(B, nh, S, c * p)


def decode_attention(q, k_cache, v_cache, head_idx, length, softmax_scale):
    """softmax(scale * q.K^T) V for one query per head over the first `length` cache positions — the
    pure-torch decode attention of the reference, CrossAttention.forward
    (Dejavu/src/models/modules/mha_dejavu.py:333-375), scale head_dim**-0.5
    (Dejavu/src/models/gpt_dejavu.py:175). fp32 softmax; rows of heads outside head_idx are NaN."""
    B, nheads, hd = q.shape
    K = unpack_k_cache(k_cache)[:, :, :length].float()
    V = v_cache[:, :, :length].float()
    ctx = torch.full((B, nheads, hd), float("nan"), dtype=torch.float32)
    heads = range(nheads) if head_idx is None else head_idx.tolist()
    for h in heads:
        s = torch.einsum("bd,bsd->bs", q[:, h].float() * softmax_scale, K[:, h])
        p = torch.softmax(s, dim=-1)
        ctx[:, h] = torch.einsum("bs,bsd->bd", p, V[:, h])
    return ctx.to(q.dtype)


def head_masked_attention(x, Wq, bq, Wk, bk, Wv, bv, Wo, bo, past_k, past_v, head_idx, num_heads):
    """The accuracy path's attention for one new token: dense q,k,v for ALL heads, softmax over past + new
    token, context of unselected heads zeroed, dense out_proj
    (Decentralized_FM_alpha/modules/hf_opt_sparse_mlp_attention.py:288-373, mask applied :365-366, scaling
    :194). x (1,d); past_k/past_v (num_heads, S, hd). Returns (out (1,d), k_new, v_new (num_heads, hd))."""
    d = x.shape[-1]
    hd = d // num_heads
    xf = x.float()
    q = (F.linear(xf, Wq.float(), bq.float()) * hd ** -0.5).view(num_heads, 1, hd)
    k_new = F.linear(xf, Wk.float(), bk.float()).view(num_heads, 1, hd)
    v_new = F.linear(xf, Wv.float(), bv.float()).view(num_heads, 1, hd)
    K = torch.cat([past_k.float(), k_new], 1)
    V = torch.cat([past_v.float(), v_new], 1)
    p = torch.softmax(torch.bmm(q, K.transpose(1, 2)), dim=-1)
    ctx = torch.bmm(p, V)  # (H,1,hd)
    mask = torch.zeros(num_heads, 1, 1)
    mask[head_idx.long()] = 1.0
    ctx = (ctx * mask).transpose(0, 1).reshape(1, d)
    return F.linear(ctx, Wo.float(), bo.float()), k_new[:, 0], v_new[:, 0]


def add_layernorm(x, residual, gamma, beta, eps, xbias=None):
    """residual = x + residual (in the activation dtype); y = LayerNorm(residual)
    (Dejavu/src/models/modules/block_dejavu.py:575-584, 625-636). Returns (y, residual)."""
    r = x.float()
    if residual is not None:
        r = r + residual.float()
    if xbias is not None:
        r = r + xbias.float()
    r = r.to(x.dtype)
    y = F.layer_norm(r.float(), (r.shape[-1],), gamma.float(), beta.float(), eps)
    return y.to(x.dtype), r


# ---------------------------------------------------------------------------------------------
# lazy K/V bookkeeping (host model of the device state machine)
# ---------------------------------------------------------------------------------------------
class LazyKVState:
    """ParallelTracker + x_cache + counter + cache_offset of the sparse mixer
    (Dejavu/src/models/modules/mha_dejavu.py:1124-1149, 1243-1253, 1318-1329, 1355-1359, 1485-1492):
    a head that is skipped at a step gets no K,V for that token until it is next selected; every 16th
    step all heads are used, which empties the window."""

    def __init__(self, nheads: int, prompt_len: int):
        self.nheads = nheads
        self.slot = 0
        self.base = prompt_len
        self.pending = [0] * nheads  # bit s: window slot s lacks K,V for this head

    def begin_step(self, head_idx: Optional[Sequence[int]]) -> Tuple[List[int], List[int]]:
        """Returns (heads in use ascending, rowmask per head in use) and updates `pending`."""
        flush = head_idx is None or self.slot == KV_WINDOW - 1
        heads = list(range(self.nheads)) if flush else sorted(set(int(h) for h in head_idx))
        bit = 1 << self.slot
        masks = []
        sel = set(heads)
        for h in range(self.nheads):
            if h in sel:
                masks.append(self.pending[h] | bit)
                self.pending[h] = 0
            else:
                self.pending[h] |= bit
        return heads, masks

    def finish_step(self):
        self.slot += 1
        if self.slot == KV_WINDOW:
            self.slot = 0
            self.base += KV_WINDOW


def attn_sparse_step(state: LazyKVState, x, x_ring, Wqkv, bqkv, k_cache, v_cache, head_idx, softmax_scale):
    """One decode step of the head-sparse attention (mha_dejavu.py:1312-1359, 1422-1446) on the lazy state:
    x (d,) is stored in the window, K,V of every missing window slot of the heads in use are projected
    and written to the caches, attention runs for the heads in use. Wqkv (3,nheads,hd,d).
    Returns (ctx (nheads,hd) with NaN rows for unused heads, heads in use)."""
    three, nheads, hd, d = Wqkv.shape
    x_ring[state.slot] = x
    heads, masks = state.begin_step(head_idx)
    q = torch.full((1, nheads, hd), float("nan"), dtype=x.dtype)
    for h, m in zip(heads, masks):
        for s in range(state.slot + 1):
            if m >> s & 1:
                kv = torch.einsum("qdn,n->qd", Wqkv[1:, h].float(), x_ring[s].float())
                if bqkv is not None:
                    kv = kv + bqkv[1:, h].float()
                kv = kv.to(x.dtype)
                pos = state.base + s
                k_cache[0, h, :, pos, :] = kv[0].reshape(hd // 8, 8)
                v_cache[0, h, pos, :] = kv[1]
        qh = Wqkv[0, h].float() @ x.float()
        if bqkv is not None:
            qh = qh + bqkv[0, h].float()
        q[0, h] = qh.to(x.dtype)
    length = state.base + state.slot + 1
    ctx = decode_attention(q, k_cache, v_cache, torch.tensor(heads, dtype=torch.int32), length, softmax_scale)
    return ctx[0], heads


# ---------------------------------------------------------------------------------------------
# tensor-parallel partitioning (Dejavu/src/utils/dejavu_util.py:139-234)
# ---------------------------------------------------------------------------------------------
def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n]


def mlp_sparse_tp(x, W1, b1, W2t, b2, scores, K, world):
    """Sparse MLP under TP: rank r owns ffn rows [r*F,(r+1)*F), picks K//world neurons inside its own
    shard (Dejavu/src/ops/fused_dense_sparse_dejavu.py:71), fc2 bias lives on rank 0 only (:299-306);
    the all-reduce is the sum of the ranks' fp16 partials. Returns (sum, [global idx per rank])."""
    F_loc = W1.shape[0] // world
    total = None
    picked = []
    for r in range(world):
        sl = slice(r * F_loc, (r + 1) * F_loc)
        idx = topk_indices_fast(scores[sl], K // world)
        part = mlp_sparse(x, W1[sl], W2t[sl], idx, None if b1 is None else b1[sl], b2 if r == 0 else None)
        total = part.float() if total is None else total + part.float()
        picked.append(idx + r * F_loc)
    return total.to(x.dtype), picked


# ---------------------------------------------------------------------------------------------
# BASELINE config 1: one OPT-125M-shaped sparse MLP block on CPU in fp32
# ---------------------------------------------------------------------------------------------
def sparse_mlp_block_fp32(x, ln_w, ln_b, W1, b1, W2, b2, P0, P1, K, eps=1e-5):
    """scores = P1 (P0 x) on the un-normalised block input; idx = top-K; y = W2[:,idx] relu(W1[idx] LN(x)
    + b1[idx]) + b2 + x (index_select form of hf_opt_sparse_mlp_attention.py:493-501, 534-560)."""
    scores = (x @ P0.T) @ P1.T
    idx = topk_indices_fast(scores[0], K)
    h = F.layer_norm(x, (x.shape[-1],), ln_w, ln_b, eps)
    a = torch.relu(h @ torch.index_select(W1, 0, idx).T + torch.index_select(b1, 0, idx))
    y = a @ torch.index_select(W2, 1, idx).T + b2 + x
    return y, idx, scores
