"""GPTLMHeadModel for OPT-shaped decoders with contextual sparsity in decode.

Mirrors Dejavu/src/models/gpt_dejavu.py (sparse MLP + sparse attention: create_mixer_cls :168-254,
create_mlp_cls :257-329, create_block :332-380, GPTModel :464-623, GPTLMHeadModel :626-702),
gpt_mlp_sparse.py (sparse MLP only) and gpt_dense.py (the dense comparator); which one is built follows the
same config attributes the benchmark scripts set (Dejavu/benchmarks/benchmark_generation_opt_dejavu.py:77-100):
    mlp_sparse, mlp_K, mlp_sp_dim, att_sparse, att_K=[K1,K2], att_sp_dim.
State-dict keys follow the reference: transformer.layers.{i}.{mixer.Wqkv,mixer.out_proj,mlp.fc1,mlp.fc2,norm1,
norm2}.*, ...mixer.sp.{fc0,fc1}.weight, ...mlp.sp.{fc0,fc1}.weight, transformer.embeddings.*, lm_head.weight.
"""
from __future__ import annotations

import math
from collections import namedtuple
from functools import partial
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, modules, ops
from .generation import GenerationMixin
from .modules import (BlockDejavu, BlockMlpAttSparse, ColumnParallelLinear, ParallelFusedMLP,
                      ParallelFusedMLPDejavu, ParallelMHADejavu, ParallelMHASparseAttMlp, _rank, _world,
                      all_reduce, join_side_streams)

# (n_layer, d, heads, ffn) of the OPT family; vocab 50272, 2048 positions (+2 offset rows dropped at load,
# Dejavu/src/utils/dejavu_util.py:41-46), ReLU, pre-norm, tied embeddings, all biases present.
OPT_SHAPES = {
    "opt-125m": (12, 768, 12, 3072),
    "opt-1.3b": (24, 2048, 32, 8192),
    "opt-6.7b": (32, 4096, 32, 16384),
    "opt-13b": (40, 5120, 40, 20480),
    "opt-30b": (48, 7168, 56, 28672),
    "opt-66b": (64, 9216, 72, 36864),
    "opt-175b": (96, 12288, 96, 49152),
}


def opt_config(name: str, **overrides) -> SimpleNamespace:
    """A GPT2Config-like namespace for an OPT shape (stands in for OPTConfig.from_pretrained +
    opt_config_to_gpt2_config of benchmark_generation_opt_dejavu.py:64-74, which need the model hub)."""
    L, d, H, ffn = OPT_SHAPES[name.split("/")[-1]]
    cfg = SimpleNamespace(
        model_name=name, n_layer=L, n_embd=d, hidden_size=d, n_head=H, n_inner=ffn, vocab_size=50272,
        n_positions=2048, max_position_embeddings=2048, activation_function="relu", layer_norm_epsilon=1e-5,
        initializer_range=0.02, pad_vocab_size_multiple=8, tie_word_embeddings=True, prenorm=True,
        mlp_sparse=False, mlp_K=ffn, mlp_sp_dim=1000, att_sparse=False, att_K=[H, H], att_sp_dim=1000,
        sequence_parallel=False, use_flash_attn=True, fused_bias_fc=True, fused_mlp=True, residual_in_fp32=False,
    )
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def apply_sparsity_knobs(cfg, mlp_K: int, att_K1: int, att_K2: int, world: int = 1):
    """--mlp-K / --att-K1 / --att-K2 -> config attributes, exactly as the benchmark does
    (benchmark_generation_opt_dejavu.py:81-100): sparsity is on iff K is below the dense size."""
    cfg.pad_vocab_size_multiple = 8 * world
    cfg.sequence_parallel = False
    if mlp_K < cfg.n_inner:
        cfg.mlp_sparse, cfg.mlp_K = True, mlp_K
    else:
        cfg.mlp_sparse, cfg.mlp_K = False, cfg.n_inner
    if att_K1 < cfg.n_head or att_K2 < cfg.n_head:
        cfg.att_sparse, cfg.att_K = True, [att_K1, att_K2]
    else:
        cfg.att_sparse, cfg.att_K = False, [cfg.n_head, cfg.n_head]
    return cfg


def att_k_for_layer(config, layer_idx: int) -> int:
    """Per-layer head budget, as written in gpt_dejavu.py:221-226: l1 = int(.35 L), l2 = int(.65 L),
    att_K[0] if (l1 <= i and i >= l2) else att_K[1] — i.e. only layers i >= l2 get K1."""
    l1, l2 = int(0.35 * config.n_layer), int(0.65 * config.n_layer)
    return config.att_K[0] if (l1 <= layer_idx and layer_idx >= l2) else config.att_K[1]


def create_mixer_cls(config, layer_idx=None, process_group=None, device=None, dtype=None):
    factory = {"device": device, "dtype": dtype}
    head_dim = config.hidden_size // config.n_head
    softmax_scale = head_dim ** -0.5  # gpt_dejavu.py:175
    common = dict(num_heads=config.n_head, process_group=process_group, softmax_scale=softmax_scale, causal=True,
                  layer_idx=layer_idx, sequence_parallel=getattr(config, "sequence_parallel", False), **factory)
    if getattr(config, "att_sparse", False):
        sp_kwargs = {"embed_dim": config.hidden_size, "low_rank_dim": config.att_sp_dim, "out_dim": config.n_head,
                     "K": att_k_for_layer(config, layer_idx)}
        return partial(ParallelMHASparseAttMlp, sp_kwargs=sp_kwargs, **common)
    return partial(ParallelMHADejavu, **common)


def create_mlp_cls(config, layer_idx=None, process_group=None, device=None, dtype=None):
    factory = {"device": device, "dtype": dtype}
    inner = config.n_inner if config.n_inner is not None else 4 * config.hidden_size
    common = dict(hidden_features=inner, activation=config.activation_function, layer_idx=layer_idx,
                  process_group=process_group, sequence_parallel=getattr(config, "sequence_parallel", False),
                  **factory)
    if getattr(config, "mlp_sparse", False):
        sp_kwargs = {"embed_dim": config.hidden_size, "low_rank_dim": config.mlp_sp_dim, "out_dim": inner,
                     "K": config.mlp_K}
        return partial(ParallelFusedMLPDejavu, sp_kwargs=sp_kwargs, **common)
    return partial(ParallelFusedMLP, **common)


def create_block(config, layer_idx=None, process_group=None, device=None, dtype=None):
    factory = {"device": device, "dtype": dtype}
    mixer_cls = create_mixer_cls(config, layer_idx, process_group=process_group, **factory)
    mlp_cls = create_mlp_cls(config, layer_idx, process_group=process_group, **factory)
    norm_cls = partial(nn.LayerNorm, eps=config.layer_norm_epsilon, **factory)
    block_cls = BlockMlpAttSparse if getattr(config, "att_sparse", False) else BlockDejavu
    block = block_cls(config.hidden_size, mixer_cls, mlp_cls, norm_cls=norm_cls, prenorm=True)
    block.layer_idx = layer_idx
    return block


class ParallelGPT2Embeddings(nn.Module):
    """Word embeddings split by vocabulary rows over the group (each rank looks up its own range, the
    all-reduce adds the pieces) + replicated learned position embeddings."""

    def __init__(self, embed_dim, vocab_size, max_position_embeddings, process_group, device=None, dtype=None):
        super().__init__()
        self.process_group = process_group
        world = _world(process_group)
        assert vocab_size % world == 0
        self.vocab_local = vocab_size // world
        self.word_embeddings = nn.Embedding(self.vocab_local, embed_dim, device=device, dtype=dtype)
        self.position_embeddings = nn.Embedding(max_position_embeddings, embed_dim, device=device, dtype=dtype)

    def forward(self, input_ids, position_ids=None):
        B, L = input_ids.shape
        if position_ids is None:
            position_ids = torch.arange(L, dtype=torch.long, device=input_ids.device)
        world = _world(self.process_group)
        if world == 1:
            e = self.word_embeddings(input_ids)
        else:
            lo = _rank(self.process_group) * self.vocab_local
            local = input_ids - lo
            inside = (local >= 0) & (local < self.vocab_local)
            e = self.word_embeddings(local.clamp(0, self.vocab_local - 1)) * inside.unsqueeze(-1).to(
                self.word_embeddings.weight.dtype)
            e = all_reduce(e, self.process_group)
        return e + self.position_embeddings(position_ids)


class GPTModel(nn.Module):
    def __init__(self, config, process_group=None, device=None, dtype=None):
        super().__init__()
        factory = {"device": device, "dtype": dtype}
        self.process_group = process_group
        self.config = config
        world = _world(process_group)
        mult = getattr(config, "pad_vocab_size_multiple", 1)
        vocab_size = math.ceil(config.vocab_size / mult) * mult  # gpt_dejavu.py:476-479
        if vocab_size % world:
            vocab_size = math.ceil(vocab_size / world) * world
        self.vocab_size_padded = vocab_size
        self.embeddings = ParallelGPT2Embeddings(config.hidden_size, vocab_size, config.max_position_embeddings,
                                                 process_group, **factory)
        self.layers = nn.ModuleList(
            [create_block(config, layer_idx=i, process_group=process_group, **factory) for i in range(config.n_layer)])
        for a, b in zip(self.layers[:-1], self.layers[1:]):
            if hasattr(a.mixer, "link_next"):
                a.mixer.link_next(b.mixer)
        self.ln_f = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon, **factory)
        self.att_sparse = getattr(config, "att_sparse", False)
        self.mlp_sparse = getattr(config, "mlp_sparse", False)
        self.comm = None

    def enable_fused_allreduce(self, comm, fused_mlp=None):
        """Route every TP all-reduce of the decode step through the one-shot all-reduce + add + LayerNorm.
        fused_mlp: "1" / "0" / "auto" = whether the second half of a block (exchange, residual, norm2, sparse MLP,
        send) runs as one kernel; None keeps the process-wide default (DJV_FUSED_MLP)."""
        self.comm = comm
        for layer in self.layers:
            layer.enable_fused_allreduce(comm)
            layer.mlp.fused_mlp = fused_mlp

    def set_dense(self, dense: bool, cublas: bool = True):
        """Dense comparator mode on the SAME weights: every head and every neuron, no predictors (what
        --mlp-K ffn --att-K heads gives, Dejavu/benchmarks/benchmark_generation_opt.py); with `cublas` the
        dense MLP GEMVs of the decode step go through torch."""
        self.force_dense = dense
        for layer in self.layers:
            layer.mixer.run_predictor = not dense
            layer.mlp.run_predictor = not dense
            layer.mlp.dense_decode_cublas = dense and cublas

    def forward(self, input_ids, position_ids=None, inference_params=None):
        hidden_states = self.embeddings(input_ids, position_ids=position_ids)
        residual = None
        mixer_kwargs = {"inference_params": inference_params} if inference_params is not None else {}
        next_mlp_sp_logit, next_att_idx = None, None
        partial_in = False
        for layer in self.layers:  # gpt_dejavu.py:574-594
            if self.att_sparse:
                hidden_states, residual, next_mlp_sp_logit, next_att_idx = layer(
                    hidden_states, residual, head_idx=next_att_idx, mlp_sp_logit=next_mlp_sp_logit,
                    mixer_kwargs=mixer_kwargs, hidden_is_partial=partial_in)
            else:
                hidden_states, residual, next_mlp_sp_logit = layer(
                    hidden_states, residual, mlp_sp_logit=next_mlp_sp_logit if self.mlp_sparse else None,
                    mixer_kwargs=mixer_kwargs, hidden_is_partial=partial_in)
            partial_in = self.comm is not None
        # final residual add + ln_f (gpt_dejavu.py:606-610)
        last = self.layers[-1]
        hidden_states, _ = last._add_norm(hidden_states, residual, self.ln_f, partial_in)
        if hidden_states.is_cuda:
            join_side_streams(hidden_states.device)  # the last layer's look-ahead results have no consumer
            if self.comm is not None:
                self.comm.end_step()  # every kernel of the step that reads the exchange is queued before this
        return hidden_states


CausalLMOutput = namedtuple("CausalLMOutput", ["logits"])


class GPTLMHeadModel(nn.Module, GenerationMixin):
    def __init__(self, config, process_group=None, device=None, dtype=None):
        super().__init__()
        self.process_group = process_group if process_group is not None else _SingleRankGroup()
        self.config = config
        self.transformer = GPTModel(config, self.process_group, device=device, dtype=dtype)
        self.lm_head = ColumnParallelLinear(config.hidden_size, self.transformer.vocab_size_padded,
                                            self.process_group, bias=False, device=device, dtype=dtype)
        self.tie_weights()

    def tie_weights(self):
        self.lm_head.weight = self.transformer.embeddings.word_embeddings.weight

    def forward(self, input_ids, position_ids=None, inference_params=None):
        # A decode step of several sequences runs kernels of several waves of blocks: programmatic dependent launch
        # then costs more than it hides (see djv_set_programmatic_launch), so the step's kernels are launched plain.
        plain = (input_ids.is_cuda and input_ids.size(0) > 1 and input_ids.size(1) == 1
                 and not modules.BATCH_PROGRAMMATIC_LAUNCH)
        if plain:
            _lib.load().djv_set_programmatic_launch(0)
        try:
            return self._forward(input_ids, position_ids, inference_params)
        finally:
            if plain:
                _lib.load().djv_set_programmatic_launch(1)

    def _forward(self, input_ids, position_ids=None, inference_params=None):
        hidden_states = self.transformer(input_ids, position_ids=position_ids, inference_params=inference_params)
        B, L, d = hidden_states.shape
        if L == 1 and hidden_states.is_cuda and B <= 32:
            lm_logits = ops.dense_gemv(hidden_states.view(B, d), self.lm_head.weight).view(B, 1, -1)
        else:
            lm_logits = self.lm_head(hidden_states)
        world = _world(self.process_group)
        if world > 1:  # gather the vocabulary shards (gpt_dejavu.py:693-700)
            parts = [torch.empty_like(lm_logits) for _ in range(world)]
            torch.distributed.all_gather(parts, lm_logits.contiguous(), group=self.process_group)
            lm_logits = torch.cat(parts, dim=-1)
        return CausalLMOutput(logits=lm_logits)

    # ---- synthetic weights ----------------------------------------------------------------------
    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02):
        """Random N(0, std) weights (benchmark_generation_opt_dejavu.py:110-124 runs on random init). Every
        tensor is generated at its FULL (unsharded) shape from a seed derived from its name, and a rank keeps
        its slice: the model is the same function for every tensor-parallel degree. LayerNorm weight 1,
        bias 0; every Linear bias ~N(0, std) as well."""
        world, rank = _world(self.process_group), _rank(self.process_group)
        dev = self.lm_head.weight.device
        gen = torch.Generator(device=dev)

        def fill(param, name, shard_dim=None, full_shape=None, transposed=False):
            gen.manual_seed((seed * 1000003 + _stable_hash(name)) % (2 ** 63))
            tgt = param.t() if transposed else param
            if shard_dim is None or world == 1:
                tgt.copy_(_randn_big(tuple(tgt.shape), gen, dev, std, tgt.dtype))
                return
            full = _randn_big(full_shape, gen, dev, std, param.dtype)
            n = full_shape[shard_dim] // world
            tgt.copy_(full.narrow(shard_dim, rank * n, n))
            del full

        t = self.transformer
        d = self.config.hidden_size
        fill(t.embeddings.word_embeddings.weight, "wte", 0, (t.vocab_size_padded, d))
        fill(t.embeddings.position_embeddings.weight, "wpe")
        H, hd = self.config.n_head, d // self.config.n_head
        for i, layer in enumerate(t.layers):
            p = f"l{i}."
            mx, ml = layer.mixer, layer.mlp
            n = mx.num_head_per_node
            # Wqkv rows are (three, head, head_dim): shard on the head axis inside each of q, k, v
            # (shard_qkv_headdim, Dejavu/src/utils/dejavu_util.py:164-169)
            gen.manual_seed((seed * 1000003 + _stable_hash(p + "Wqkv")) % (2 ** 63))
            full = _randn_big((3, H, hd, d), gen, dev, std, mx.Wqkv.weight.dtype)
            mx.Wqkv.weight.copy_(full[:, rank * n:(rank + 1) * n].reshape(3 * n * hd, d))
            gen.manual_seed((seed * 1000003 + _stable_hash(p + "bqkv")) % (2 ** 63))
            fullb = torch.randn((3, H, hd), generator=gen, device=dev).mul_(std)
            mx.Wqkv.bias.copy_(fullb[:, rank * n:(rank + 1) * n].reshape(-1))
            del full
            fill(mx.out_proj.weight, p + "Wo", 1, (d, d))
            if mx.out_proj.bias is not None:
                fill(mx.out_proj.bias, p + "bo")
            inner = self.config.n_inner
            fill(ml.fc1.weight, p + "W1", 0, (inner, d))
            fill(ml.fc1.bias, p + "b1", 0, (inner,))
            fill(ml.fc2.weight, p + "W2t", 0, (inner, d), transposed=True)
            if ml.fc2.bias is not None:
                fill(ml.fc2.bias, p + "b2")
            if getattr(ml, "sp", None) is not None:
                fill(ml.sp.fc0.weight, p + "P0")
                fill(ml.sp.fc1.weight, p + "P1", 0, (inner, ml.sp.fc0.weight.shape[0]))
            if getattr(mx, "sp", None) is not None:
                fill(mx.sp.fc0.weight, p + "A0")
                fill(mx.sp.fc1.weight, p + "A1", 0, (H, mx.sp.fc0.weight.shape[0]))
            for norm in (layer.norm1, layer.norm2):
                norm.weight.fill_(1.0)
                norm.bias.zero_()
        t.ln_f.weight.fill_(1.0)
        t.ln_f.bias.zero_()
        return self


class _SingleRankGroup:
    """Stand-in for a process group of size 1 (the reference's modules assert that a group is given)."""

    def size(self):
        return 1

    def rank(self):
        return 0


def _stable_hash(name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) % (2 ** 61)
    return h


def _randn_big(shape, gen, dev, std, dtype):
    """N(0, std) of `shape` in `dtype`, generated in fp32 slabs so no full-size fp32 copy is held."""
    out = torch.empty(shape, device=dev, dtype=dtype)
    flat = out.view(-1)
    step = 1 << 26
    for s in range(0, flat.numel(), step):
        e = min(flat.numel(), s + step)
        flat[s:e].copy_(torch.randn(e - s, generator=gen, device=dev, dtype=torch.float32).mul_(std))
    return out
