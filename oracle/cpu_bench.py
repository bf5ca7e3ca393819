"""Times the reference's torch formulation of one sparse decode step on the host cores.

TEST / MEASUREMENT INFRASTRUCTURE (used only by bench.py's cpu_baseline and its `--impl reference` arm).
The reference's latency model cannot run without its CUDA extensions, so the CPU arm is this port of its
math: per layer, in fp32 (fp16 matmul on CPU is not representative),
    predictor (two bias-free linears) + top-K            fused_dense_sparse_dejavu.py:59-76, mha_dejavu.py:1369
    index_select sparse MLP                              gather_gemv.py:206, 579, 647-657
    head-sparse QKV / one-query attention / out_proj     attention_proj_sparse.py:118-125, 281-286;
                                                         mha_dejavu.py:333-375
    residual add + LayerNorm (x2)                        block_dejavu.py:575-584, 625-636
plus the LM head once per token. A bounded number of layers is built and timed, then scaled to the
model's depth: layers are identical in shape, so time per layer x n_layer (+ LM head) is the token time.
"""
from __future__ import annotations

import time

import torch
import torch.nn.functional as F

from . import oracle as O


def _rand(*shape):
    """N(0, 0.02), the synthetic weight distribution of every benchmark configuration."""
    return torch.empty(*shape, dtype=torch.float32).normal_(0.0, 0.02)


class CpuLayer:
    def __init__(self, d, H, ffn, R_mlp, R_att, S):
        hd = d // H
        self.d, self.H, self.hd, self.ffn = d, H, hd, ffn
        self.Wqkv, self.bqkv = _rand(3, H, hd, d), _rand(3, H, hd)
        self.Wo, self.bo = _rand(d, H, hd), _rand(d)
        self.W1, self.b1 = _rand(ffn, d), _rand(ffn)
        self.W2t, self.b2 = _rand(ffn, d), _rand(d)
        self.P0, self.P1 = _rand(R_mlp, d), _rand(ffn, R_mlp)
        self.A0, self.A1 = _rand(R_att, d), _rand(H, R_att)
        self.ln = (torch.ones(d), torch.zeros(d))
        self.K = torch.randn(H, S, hd)
        self.V = torch.randn(H, S, hd)

    def step(self, h, residual, mlp_logit, att_idx, mlp_K, att_K, length):
        d, H, hd = self.d, self.H, self.hd
        residual = h + residual
        x = F.layer_norm(residual, (d,), *self.ln)
        heads = att_idx if att_idx is not None else torch.arange(H)
        qkv = torch.einsum("qhdn,n->qhd", self.Wqkv[:, heads], x[0]) + self.bqkv[:, heads]
        self.K[heads, length - 1] = qkv[1]
        self.V[heads, length - 1] = qkv[2]
        s = torch.einsum("hd,hkd->hk", qkv[0] * hd ** -0.5, self.K[heads, :length])
        ctx = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), self.V[heads, :length])
        out = torch.einsum("nhd,hd->n", self.Wo[:, heads], ctx) + self.bo
        mlp_idx = None if mlp_logit is None else torch.topk(mlp_logit, mlp_K, sorted=False).indices
        next_att = None
        if att_K is not None:
            next_att = torch.topk(self.A1 @ (self.A0 @ residual[0]), att_K, sorted=False).indices
        residual = out[None] + residual
        x = F.layer_norm(residual, (d,), *self.ln)
        if mlp_idx is not None:
            a = torch.relu(x @ torch.index_select(self.W1, 0, mlp_idx).T + self.b1[mlp_idx])
            h = a @ torch.index_select(self.W2t, 0, mlp_idx) + self.b2
        else:
            h = torch.relu(x @ self.W1.T + self.b1) @ self.W2t + self.b2
        next_logit = None
        if mlp_K is not None:
            next_logit = self.P1 @ (self.P0 @ residual[0])
        return h, residual, next_logit, next_att


def host_threads() -> int:
    """Host threads this process may use (launchers such as torch.distributed.run export OMP_NUM_THREADS=1,
    which would otherwise leave the CPU arm on a single core)."""
    import os

    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def time_decode(d, H, ffn, n_layer, vocab, mlp_K, att_K, S=256, sample_layers=2, reps=3, R_mlp=1000, R_att=1000,
                threads=None):
    """Returns dict(ms_per_token, ms_per_layer, ms_lm_head, cores, sample). mlp_K / att_K None = dense.
    threads: host threads to use (default: every core this process may run on)."""
    torch.set_num_threads(threads or host_threads())
    cores = torch.get_num_threads()
    sample_layers = max(1, min(sample_layers, n_layer))
    layers = [CpuLayer(d, H, ffn, R_mlp, R_att, S) for _ in range(sample_layers)]
    W_lm = _rand(vocab, d) if vocab else None
    h, residual = torch.randn(1, d), torch.randn(1, d)
    times = []
    with torch.inference_mode():
        for rep in range(reps + 1):
            logit = None if mlp_K is None else torch.randn(ffn)
            att = None if att_K is None else torch.randperm(H)[:att_K]
            t0 = time.perf_counter()
            hh, rr = h, residual
            for L in layers:
                hh, rr, logit, att = L.step(hh, rr, logit, att, mlp_K, att_K, S // 2 + rep)
            t1 = time.perf_counter()
            if rep > 0:  # first pass warms the pages
                times.append((t1 - t0) / sample_layers)
        lm = 0.0
        if W_lm is not None:
            t0 = time.perf_counter()
            for _ in range(2):
                (W_lm @ h[0]).argmax()
            lm = (time.perf_counter() - t0) / 2
    per_layer = sorted(times)[len(times) // 2]
    return {
        "ms_per_token": (per_layer * n_layer + lm) * 1e3,
        "ms_per_layer": per_layer * 1e3,
        "ms_lm_head": lm * 1e3,
        "cores": cores,
        "sample": f"{sample_layers} of {n_layer} layers x {reps} decode steps in fp32 (index_select form) + LM head, "
                  f"scaled to {n_layer} layers",
    }
