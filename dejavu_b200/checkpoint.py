"""Checkpoint plumbing: Hugging Face OPT state dict -> this model's keys, tensor-parallel shards, and the
trained sparsity predictors.

Same function names and results as Dejavu/src/utils/dejavu_util.py (remap_state_dict_opt :12-136,
shard_state_dict_tp :139-234), so `model.load_state_dict(shard_state_dict_tp(remap_state_dict_opt(sd, cfg),
cfg, world, rank))` works as in Dejavu/benchmarks/benchmark_generation_opt.py:59-69. Two differences, both
because of how this package lays tensors out: the position table is replicated (not split on its last
dimension), and the final LayerNorm is always called transformer.ln_f.
The reference latency model has no loader for predictor weights; `load_predictors` reads the files its
trainer writes (sparse_predictor/main_mlp.py:160-161: state dict of Sequential(Linear, Linear), found by
the glob patterns of Decentralized_FM_alpha/modules/hf_opt_sparse_mlp_attention.py:434-441, 455-462).
"""
from __future__ import annotations

import glob
import math
import os
import re
from collections import OrderedDict

import torch
import torch.nn.functional as F

_RENAMES = [
    (r"^model\.decoder\.", "transformer."),
    (r"^decoder\.", "transformer."),  # OPT-350m style
    (r"^transformer\.embed_tokens\.", "transformer.embeddings.word_embeddings."),
    (r"^transformer\.final_layer_norm\.", "transformer.ln_f."),
    (r"^transformer\.layers\.(\d+)\.self_attn_layer_norm\.", r"transformer.layers.\1.norm1."),
    (r"^transformer\.layers\.(\d+)\.final_layer_norm\.", r"transformer.layers.\1.norm2."),
    (r"^transformer\.layers\.(\d+)\.fc(1|2)\.", r"transformer.layers.\1.mlp.fc\2."),
    (r"^transformer\.layers\.(\d+)\.self_attn\.out_proj\.", r"transformer.layers.\1.mixer.out_proj."),
]


def _padded_vocab(config, world_size: int = 1) -> int:
    mult = getattr(config, "pad_vocab_size_multiple", 1)
    v = math.ceil(config.vocab_size / mult) * mult
    return math.ceil(v / world_size) * world_size


def _n_layers(config) -> int:
    return getattr(config, "num_hidden_layers", None) or config.n_layer


def remap_state_dict_opt(state_dict, config):
    """HF `OPTForCausalLM.state_dict()` -> keys of GPTLMHeadModel. Drops the two padding rows of the
    position table, pads the vocabulary, concatenates q/k/v into Wqkv (q rows, then k, then v), ties
    lm_head to the word embeddings."""
    out = OrderedDict()
    for key, value in state_dict.items():
        if key == "lm_head.weight":
            continue  # tied; rebuilt below
        for pattern, repl in _RENAMES:
            key = re.sub(pattern, repl, key)
        out[key] = value
    if "transformer.embed_positions.weight" in out:
        out["transformer.embeddings.position_embeddings.weight"] = out.pop("transformer.embed_positions.weight")[2:]
    emb_key = "transformer.embeddings.word_embeddings.weight"
    emb = out[emb_key]
    out[emb_key] = F.pad(emb, (0, 0, 0, _padded_vocab(config) - emb.shape[0]))
    out["lm_head.weight"] = out[emb_key]
    for layer in range(_n_layers(config)):
        p = f"transformer.layers.{layer}."
        for kind in ("weight", "bias"):
            parts = [out.pop(f"{p}self_attn.{n}_proj.{kind}") for n in ("q", "k", "v")]
            out[f"{p}mixer.Wqkv.{kind}"] = torch.cat(parts, dim=0)
    return out


def shard_state_dict_tp(state_dict, config, world_size, rank):
    """Slice a full (remapped) state dict for tensor-parallel rank `rank` of `world_size`:
    vocabulary rows; heads inside each of q, k, v; out_proj / fc2 input columns; fc1 rows; predictor fc1 rows;
    row-parallel biases on rank 0 only; everything else replicated."""
    vocab = _padded_vocab(config, world_size)
    inner = config.n_inner if getattr(config, "n_inner", None) is not None else 4 * config.hidden_size
    assert vocab % world_size == 0 and config.hidden_size % world_size == 0 and inner % world_size == 0

    def rows(x):
        n = x.shape[0] // world_size
        return x[rank * n:(rank + 1) * n]

    def cols(x):
        n = x.shape[-1] // world_size
        return x[..., rank * n:(rank + 1) * n]

    def qkv(x):
        three = x.reshape(3, x.shape[0] // 3, *x.shape[1:])
        n = three.shape[1] // world_size
        return three[:, rank * n:(rank + 1) * n].reshape(3 * n, *x.shape[1:])

    out = {}
    for key, x in state_dict.items():
        if key in ("transformer.embeddings.word_embeddings.weight", "lm_head.weight"):
            if x.shape[0] < vocab:
                x = F.pad(x, (0, 0, 0, vocab - x.shape[0]))
            out[key] = rows(x)
        elif key.endswith(("mixer.Wqkv.weight", "mixer.Wqkv.bias")):
            out[key] = qkv(x)
        elif key.endswith(("mixer.out_proj.weight", "mlp.fc2.weight")):
            out[key] = cols(x)
        elif key.endswith(("mlp.fc1.weight", "mlp.fc1.bias", "sp.fc1.weight")):
            out[key] = rows(x)
        elif key.endswith(("mixer.out_proj.bias", "mlp.fc2.bias")):
            if rank == 0:
                out[key] = x
        else:
            out[key] = x
    return out


def load_predictors(model, predictor_path: str, strict: bool = False) -> dict:
    """Loads trained predictors into model.transformer.layers[i].{mlp,mixer}.sp from
    `<predictor_path>/c4_layer{i}*.pt` (MLP) and `c4_att_layer{i}*.pt` (attention); each file holds the
    state dict of Sequential(Linear(d, R, no bias), Linear(R, n, no bias)). The second matrix is row-sharded
    for the model's tensor-parallel rank. Returns {"mlp": [layers loaded], "att": [...]}."""
    pg = model.process_group
    world, rank = pg.size(), pg.rank()
    loaded = {"mlp": [], "att": []}
    for i, layer in enumerate(model.transformer.layers):
        for kind, module, pattern in (("mlp", layer.mlp, f"c4_layer{i}*.pt"), ("att", layer.mixer, f"c4_att_layer{i}*.pt")):
            sp = getattr(module, "sp", None)
            if sp is None:
                continue
            files = sorted(glob.glob(os.path.join(predictor_path, pattern)))
            # c4_layer1*.pt would also match layer 10..19: keep exact layer numbers only
            files = [f for f in files if re.search(rf"layer{i}(\D|$)", os.path.basename(f))]
            if not files:
                if strict:
                    raise FileNotFoundError(os.path.join(predictor_path, pattern))
                continue
            sd = torch.load(files[0], map_location="cpu")
            w0, w1 = sd["0.weight"], sd["1.weight"]
            n = w1.shape[0] // world
            with torch.no_grad():
                sp.fc0.weight.copy_(w0)
                sp.fc1.weight.copy_(w1[rank * n:(rank + 1) * n])
            loaded[kind].append(i)
    return loaded
