"""CPU restatement of the sparse OPT decoder's decode step (test infrastructure, like oracle.py).

Wiring of the latency path (Dejavu/src/models/gpt_dejavu.py:574-594, modules/block_dejavu.py:555-663,
modules/mha_dejavu.py:1283-1511, ops/fused_dense_sparse_dejavu.py:889-951):
  * layer L's MLP predictor reads layer L's MLP-input residual and its logits pick layer L+1's neurons;
    layer L's attention predictor reads layer L's attention-input residual and picks layer L+1's heads;
    layer 0 is always dense; the prompt pass is dense;
  * selection is per tensor-parallel shard: K // shards neurons / heads inside each contiguous shard
    (fused_dense_sparse_dejavu.py:71);
  * every 16th decode step uses all heads (mha_dejavu.py:1320-1325).
Attention is computed with a full K/V cache and the unselected heads' context dropped, which
tests/test_oracle_golden.py proves equal to the lazy-K/V bookkeeping for the heads in use.

Parity of index sets is defined "given identical predictor scores": `decode(..., forced=...)` takes the index
sets another implementation chose, checks that each is a valid top-K of the oracle's own scores up to a
score margin (fp16 rounding of the scores can swap near-ties), and continues with those sets.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from . import oracle as O


class OracleDecoder:
    def __init__(self, state_dict: Dict[str, torch.Tensor], cfg, num_shards: int = 1, score_margin: float = 2e-3,
                 cache_fp32: bool = False):
        """cache_fp32: keep an fp32 copy of every matrix after its first use (wide models: converting a
        12288 x 49152 matrix at every call dominates the run time otherwise)."""
        self.sd = {k: v.detach().cpu() for k, v in state_dict.items()}
        self._fp32 = {} if cache_fp32 else None
        self.free_running_checks = 0  # selections that were decisive and therefore compared exactly
        self.cfg = cfg
        self.L, self.d, self.H = cfg.n_layer, cfg.hidden_size, cfg.n_head
        self.hd = self.d // self.H
        self.shards = num_shards
        self.margin = score_margin
        self.dtype = self.sd["transformer.ln_f.weight"].dtype
        self.k = [None] * self.L  # (H, S, hd) per layer, activation dtype
        self.v = [None] * self.L
        self.step = 0

    # -- helpers ---------------------------------------------------------------------------------
    def _p(self, i, name):
        return self.sd[f"transformer.layers.{i}.{name}"]

    def _lin(self, x, w, b=None):
        if self._fp32 is not None:
            key = (w.data_ptr(), tuple(w.shape))
            if key not in self._fp32:
                self._fp32[key] = w.float()
            wf = self._fp32[key]
        else:
            wf = w.float()
        y = x.float() @ wf.T
        if b is not None:
            y = y + b.float()
        return y.to(self.dtype)

    def _mlp_k(self):
        return (self.cfg.mlp_K // self.shards) if getattr(self.cfg, "mlp_sparse", False) else None

    def _att_k(self, i):
        if not getattr(self.cfg, "att_sparse", False):
            return None
        l1, l2 = int(0.35 * self.L), int(0.65 * self.L)
        k = self.cfg.att_K[0] if (l1 <= i and i >= l2) else self.cfg.att_K[1]
        return k // self.shards

    def _select(self, scores, k_per_shard, forced, what):
        """top-k inside each shard; with `forced`, validate the given set against the scores instead."""
        n = scores.numel() // self.shards
        out = []
        for r in range(self.shards):
            sl = scores[r * n:(r + 1) * n]
            if forced is None:
                out.append(O.topk_indices_fast(sl, k_per_shard) + r * n)
                continue
            f = torch.as_tensor(forced).long().flatten()
            f = f[(f >= r * n) & (f < (r + 1) * n)] - r * n
            assert f.numel() == k_per_shard and f.unique().numel() == k_per_shard, \
                f"{what}: shard {r} got {f.numel()} indices, expected {k_per_shard} distinct ones"
            if k_per_shard < n:
                rest = torch.ones(n, dtype=torch.bool)
                rest[f] = False
                worst_in, best_out = sl.float()[f].min().item(), sl.float()[rest].max().item()
                assert worst_in >= best_out - self.margin * max(1.0, abs(best_out)), \
                    f"{what}: not a top-{k_per_shard} set (min selected {worst_in} < max unselected {best_out})"
                # free-running agreement: when this oracle's own K-th and (K+1)-th scores are further apart than
                # the margin, there is only one admissible set, and the other implementation must have found it
                own = O.topk_indices_fast(sl, k_per_shard)
                mine = torch.ones(n, dtype=torch.bool)
                mine[own] = False
                gap = sl.float()[own].min().item() - sl.float()[mine].max().item()
                if gap > self.margin * max(1.0, abs(best_out)):
                    assert torch.equal(own.sort().values, f.sort().values), f"{what}: decisive scores, different set"
                    self.free_running_checks += 1
            out.append(f.sort().values + r * n)
        return torch.cat(out)

    # -- prompt (dense) ----------------------------------------------------------------------------
    def prompt(self, ids: torch.Tensor) -> torch.Tensor:
        """ids (P,) -> logits of the last position (vocab,); ids (B, P) -> (B, vocab), one K/V history per
        sequence."""
        single = ids.dim() == 1
        batch = ids[None] if single else ids
        B, P = batch.shape
        sd = self.sd
        ks = [[None] * B for _ in range(self.L)]
        vs = [[None] * B for _ in range(self.L)]
        out = []
        for b in range(B):
            row = batch[b]
            h = (sd["transformer.embeddings.word_embeddings.weight"][row].float()
                 + sd["transformer.embeddings.position_embeddings.weight"][:P].float()).to(self.dtype)
            residual = None
            for i in range(self.L):
                x, residual = O.add_layernorm(h, residual, self._p(i, "norm1.weight"), self._p(i, "norm1.bias"),
                                              self.cfg.layer_norm_epsilon)
                qkv = self._lin(x, self._p(i, "mixer.Wqkv.weight"), self._p(i, "mixer.Wqkv.bias")).view(P, 3, self.H, self.hd)
                q, k, v = qkv[:, 0].transpose(0, 1), qkv[:, 1].transpose(0, 1), qkv[:, 2].transpose(0, 1)
                ks[i][b], vs[i][b] = k.contiguous(), v.contiguous()
                s = torch.einsum("hqd,hkd->hqk", q.float() * self.hd ** -0.5, k.float())
                s = s + torch.full((P, P), float("-inf")).triu(1)
                ctx = torch.einsum("hqk,hkd->hqd", torch.softmax(s, -1), v.float()).to(self.dtype)
                ctx = ctx.transpose(0, 1).reshape(P, self.d)
                h = self._lin(ctx, self._p(i, "mixer.out_proj.weight"), self._p(i, "mixer.out_proj.bias"))
                x, residual = O.add_layernorm(h, residual, self._p(i, "norm2.weight"), self._p(i, "norm2.bias"),
                                              self.cfg.layer_norm_epsilon)
                a = torch.relu(self._lin(x, self._p(i, "mlp.fc1.weight"), self._p(i, "mlp.fc1.bias")))
                h = self._lin(a, self._p(i, "mlp.fc2.weight"), self._p(i, "mlp.fc2.bias"))
            x, _ = O.add_layernorm(h, residual, sd["transformer.ln_f.weight"], sd["transformer.ln_f.bias"],
                                   self.cfg.layer_norm_epsilon)
            out.append(self._lin(x[-1:], sd["lm_head.weight"])[0])
        for i in range(self.L):
            self.k[i], self.v[i] = torch.stack(ks[i]), torch.stack(vs[i])  # (B, H, S, hd)
        self.step = 0
        return out[0] if single else torch.stack(out)

    # -- one decode step ---------------------------------------------------------------------------
    def decode(self, token, pos: int, forced: Optional[List[dict]] = None):
        """token: int -> (logits (vocab,), chosen); a list of B ints (one per sequence, all at position `pos`) ->
        (logits (B, vocab), chosen). chosen[i] = {"mlp_idx": ..., "att_idx": ...} are the sets layer i produced
        (mlp_idx: used by layer i's own MLP; att_idx: for layer i+1's attention); forced[i] holds the sets another
        implementation produced at layer i (or None entries).
        Batches share ONE index set per layer and step: the top-K of the predictor logits summed over the batch
        (fp32 sum of the fp16 logits, rounded to fp16). The reference's decode path keeps a single sequence
        (Dejavu/src/models/modules/mha_dejavu.py:1318, 1469); its kernels take one index list for all rows of a
        batch (Dejavu/src/ops/triton/gather_gemv.py:198-254), which is what this rule feeds."""
        single = not isinstance(token, (list, tuple))
        tokens = torch.tensor([token] if single else list(token))
        B = tokens.numel()
        sd, eps = self.sd, self.cfg.layer_norm_epsilon
        h = (sd["transformer.embeddings.word_embeddings.weight"][tokens].float()
             + sd["transformer.embeddings.position_embeddings.weight"][pos].float()).to(self.dtype)
        residual, mlp_logit, att_idx = None, None, None
        flush = (self.step % O.KV_WINDOW) == O.KV_WINDOW - 1
        chosen = []

        def shared(scores):  # (B, n) per-sequence logits -> the batch's scores
            return scores[0] if B == 1 else scores.float().sum(0).to(self.dtype)

        for i in range(self.L):
            fi = forced[i] if forced is not None else {}
            x, residual = O.add_layernorm(h, residual, self._p(i, "norm1.weight"), self._p(i, "norm1.bias"), eps)
            # attention over heads att_idx (all heads for layer 0, dense models and flush steps)
            qkv = self._lin(x, self._p(i, "mixer.Wqkv.weight"), self._p(i, "mixer.Wqkv.bias")).view(B, 3, self.H, self.hd)
            if self.k[i].dim() == 3:  # histories written by older callers: (H, S, hd)
                self.k[i], self.v[i] = self.k[i][None], self.v[i][None]
            self.k[i] = torch.cat([self.k[i], qkv[:, 1][:, :, None]], 2)
            self.v[i] = torch.cat([self.v[i], qkv[:, 2][:, :, None]], 2)
            heads = torch.arange(self.H) if (att_idx is None or flush) else att_idx.long()
            s = torch.einsum("bhd,bhkd->bhk", qkv[:, 0].float() * self.hd ** -0.5, self.k[i].float())
            ctx = torch.einsum("bhk,bhkd->bhd", torch.softmax(s, -1), self.v[i].float()).to(self.dtype)
            Wo = self._p(i, "mixer.out_proj.weight").view(self.d, self.H, self.hd)
            attn_out = O.out_proj_sparse(ctx, Wo, heads.int(), self._p(i, "mixer.out_proj.bias"))
            # this layer's MLP neurons come from the previous layer's logits
            mlp_idx = None
            if mlp_logit is not None:
                mlp_idx = self._select(mlp_logit, self._mlp_k(), fi.get("mlp_idx"), f"layer {i} mlp_idx")
            # next layer's heads come from this layer's attention-input residual
            next_att_idx = None
            if self._att_k(i) is not None:
                a_scores = shared(O.predictor_scores(residual, self._p(i, "mixer.sp.fc0.weight"),
                                                     self._p(i, "mixer.sp.fc1.weight")))
                next_att_idx = self._select(a_scores, self._att_k(i), fi.get("att_idx"), f"layer {i} att_idx")
            x, residual = O.add_layernorm(attn_out, residual, self._p(i, "norm2.weight"), self._p(i, "norm2.bias"), eps)
            W1, b1 = self._p(i, "mlp.fc1.weight"), self._p(i, "mlp.fc1.bias")
            W2, b2 = self._p(i, "mlp.fc2.weight"), self._p(i, "mlp.fc2.bias")
            if mlp_idx is not None:
                h = O.mlp_sparse(x, W1, W2.t(), mlp_idx, b1, b2)
            else:
                h = self._lin(torch.relu(self._lin(x, W1, b1)), W2, b2)
            mlp_logit = None
            if self._mlp_k() is not None:
                mlp_logit = shared(O.predictor_scores(residual, self._p(i, "mlp.sp.fc0.weight"),
                                                      self._p(i, "mlp.sp.fc1.weight")))
            att_idx = next_att_idx
            chosen.append({"mlp_idx": mlp_idx, "att_idx": next_att_idx})
        x, _ = O.add_layernorm(h, residual, sd["transformer.ln_f.weight"], sd["transformer.ln_f.bias"], eps)
        self.step += 1
        logits = self._lin(x, sd["lm_head.weight"])
        return (logits[0] if single else logits), chosen
