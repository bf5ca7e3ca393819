"""Tensor-parallel host logic on CPU: two gloo ranks against the single-rank model.

Covers the partitioning rules (heads / ffn neurons / vocabulary by rank, bias on rank 0, K // world), the
TP-invariant random init, the vocab-parallel embedding all-reduce, the row-parallel all-reduces and the
logits all-gather, on the dense prompt pass (the only pass that has a torch path; the decode kernels are
CUDA-only and are covered by the GPU tests).
"""
import os
import sys
import tempfile
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _cfg():
    from dejavu_b200.gpt import apply_sparsity_knobs, opt_config

    cfg = opt_config("opt-125m", n_layer=2, n_embd=64, hidden_size=64, n_head=4, n_inner=256, vocab_size=90,
                     max_position_embeddings=32, n_positions=32, mlp_sp_dim=16, att_sp_dim=8)
    return cfg


def _worker(rank, world, init_file, out_file):
    sys.path.insert(0, str(ROOT))
    from dejavu_b200.gpt import GPTLMHeadModel, apply_sparsity_knobs

    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    pg = dist.group.WORLD
    cfg = apply_sparsity_knobs(_cfg(), 64, 2, 2, world)
    model = GPTLMHeadModel(cfg, process_group=pg, device="cpu", dtype=torch.float32).eval().init_random(3, std=0.05)
    ids = torch.arange(11).remainder(90)[None]
    with torch.inference_mode():
        logits = model(ids).logits
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    budgets = (model.transformer.layers[0].mixer.mlp_k, model.transformer.layers[0].mixer.att_k)
    gathered = [None] * world
    dist.all_gather_object(gathered, (sd, budgets))
    if rank == 0:
        torch.save({"logits": logits, "shards": gathered, "vocab_padded": model.transformer.vocab_size_padded}, out_file)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_single_rank():
    from dejavu_b200.gpt import GPTLMHeadModel, apply_sparsity_knobs

    world = 2
    with tempfile.TemporaryDirectory() as tmp:
        init_file, out_file = os.path.join(tmp, "init"), os.path.join(tmp, "out.pt")
        mp.spawn(_worker, args=(world, init_file, out_file), nprocs=world, join=True)
        res = torch.load(out_file, weights_only=False)
    # the single-rank model, vocabulary padded as the 2-rank run pads it (8 * world)
    cfg = apply_sparsity_knobs(_cfg(), 64, 2, 2, world)
    ref = GPTLMHeadModel(cfg, device="cpu", dtype=torch.float32).eval().init_random(3, std=0.05)
    assert ref.transformer.vocab_size_padded == res["vocab_padded"] == 96
    ids = torch.arange(11).remainder(90)[None]
    with torch.inference_mode():
        want = ref(ids).logits
    assert torch.allclose(res["logits"], want, atol=1e-4, rtol=1e-4), (res["logits"] - want).abs().max()
    # shards are slices of the single-rank tensors
    full = ref.state_dict()
    (sd0, b0), (sd1, b1) = res["shards"]
    assert b0 == b1 == (64 // world, 2 // world)  # K // world per rank (fused_dense_sparse_dejavu.py:71)
    H, hd, d = 4, 16, 64
    n = H // world
    for r, sd in enumerate((sd0, sd1)):
        p = "transformer.layers.1."
        assert torch.equal(sd[p + "mlp.fc1.weight"], full[p + "mlp.fc1.weight"][r * 128:(r + 1) * 128])
        assert torch.equal(sd[p + "mlp.fc1.bias"], full[p + "mlp.fc1.bias"][r * 128:(r + 1) * 128])
        assert torch.equal(sd[p + "mlp.fc2.weight"], full[p + "mlp.fc2.weight"][:, r * 128:(r + 1) * 128])
        assert torch.equal(sd[p + "mlp.sp.fc0.weight"], full[p + "mlp.sp.fc0.weight"])  # replicated
        assert torch.equal(sd[p + "mlp.sp.fc1.weight"], full[p + "mlp.sp.fc1.weight"][r * 128:(r + 1) * 128])
        assert torch.equal(sd[p + "mixer.sp.fc1.weight"], full[p + "mixer.sp.fc1.weight"][r * n:(r + 1) * n])
        wq = full[p + "mixer.Wqkv.weight"].view(3, H, hd, d)[:, r * n:(r + 1) * n].reshape(3 * n * hd, d)
        assert torch.equal(sd[p + "mixer.Wqkv.weight"], wq)
        assert torch.equal(sd[p + "mixer.out_proj.weight"], full[p + "mixer.out_proj.weight"][:, r * n * hd:(r + 1) * n * hd])
        assert (p + "mixer.out_proj.bias" in sd) == (r == 0)  # row-parallel bias lives on rank 0 only
        assert (p + "mlp.fc2.bias" in sd) == (r == 0)
        assert torch.equal(sd["lm_head.weight"], full["lm_head.weight"][r * 48:(r + 1) * 48])


def test_att_k_rule_as_written():
    from dejavu_b200.gpt import att_k_for_layer, opt_config

    cfg = opt_config("opt-175b")
    cfg.att_K = [24, 48]
    ks = [att_k_for_layer(cfg, i) for i in range(96)]
    l2 = int(0.65 * 96)
    assert ks[:l2] == [48] * l2 and ks[l2:] == [24] * (96 - l2)  # only the last 35 % of layers get att-K1


def test_sparsity_knobs_follow_the_benchmark_script():
    from dejavu_b200.gpt import apply_sparsity_knobs, opt_config

    cfg = apply_sparsity_knobs(opt_config("opt-66b"), 4096, 24, 24, world=8)
    assert cfg.mlp_sparse and cfg.att_sparse and cfg.mlp_K == 4096 and cfg.att_K == [24, 24]
    assert cfg.pad_vocab_size_multiple == 64
    cfg = apply_sparsity_knobs(opt_config("opt-66b"), 36864, 72, 72)
    assert not cfg.mlp_sparse and not cfg.att_sparse
