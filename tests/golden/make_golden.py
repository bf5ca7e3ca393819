"""Generates tests/golden/*.npz by RUNNING THE REFERENCE ITSELF on CPU.

Run once in a container that has the reference checkout (it does not travel to the GPU box):

    python tests/golden/make_golden.py --reference /path/to/DejaVu

Two sources:
  (A) the reference's Triton kernels (Dejavu/src/ops/triton/gather_gemv.py, attention_proj_sparse.py),
      executed by Triton's CPU interpreter (TRITON_INTERPRET=1). The autotuner's timing step needs a GPU
      driver, so its `_bench` is replaced by a constant: the first config of each list is used. Kernel
      code and wrappers run unmodified.
  (B) the accuracy path's block, Decentralized_FM_alpha/modules/hf_opt_sparse_mlp_attention.py
      (GPTBlock.forward with MLP mask and head mask), in fp32 on CPU at BASELINE config 1's shape. The
      block's constructor asks torch for CUDA streams; those three constructors are stubbed here.

Inputs come from numpy's PCG64 generator with the seeds below; small cases store inputs and outputs,
the config-1 case stores outputs plus a checksum of the inputs (tests regenerate them from the seed).
"""
from __future__ import annotations

import argparse
import os
import sys
import types
from pathlib import Path

import numpy as np

os.environ["TRITON_INTERPRET"] = "1"  # must be set before anything imports triton

HERE = Path(__file__).resolve().parent


def rng_normal(rng, shape, std, dtype):
    return (rng.standard_normal(shape) * std).astype(dtype)


def config1_inputs(seed: int = 0):
    """BASELINE config 1 tensors (fp32): d=768, ffn=3072, 12 heads, predictor rank 1000."""
    rng = np.random.Generator(np.random.PCG64(seed))
    d, ffn, R, H = 768, 3072, 1000, 12
    t = {
        "W1": rng_normal(rng, (ffn, d), 0.02, np.float32),
        "W2": rng_normal(rng, (d, ffn), 0.02, np.float32),
        "b1": np.zeros(ffn, np.float32),
        "b2": np.zeros(d, np.float32),
        "P0": rng_normal(rng, (R, d), 0.02, np.float32),
        "P1": rng_normal(rng, (ffn, R), 0.02, np.float32),
        "A0": rng_normal(rng, (R, d), 0.02, np.float32),
        "A1": rng_normal(rng, (H, R), 0.02, np.float32),
        "x": rng_normal(rng, (1, 1, d), 1.0, np.float32),
        "prev": rng_normal(rng, (1, 1, d), 1.0, np.float32),
        "past_k": rng_normal(rng, (1, H, 8, d // H), 1.0, np.float32),
        "past_v": rng_normal(rng, (1, H, 8, d // H), 1.0, np.float32),
    }
    for name in ("q", "k", "v", "o"):
        t["W" + name] = rng_normal(rng, (d, d), 0.02, np.float32)
        t["b" + name] = rng_normal(rng, (d,), 0.02, np.float32)
    return t


def checksum(arrays: dict) -> float:
    return float(sum(np.abs(a.astype(np.float64)).sum() for a in arrays.values()))


def triton_cases(ref_root: Path):
    sys.path.insert(0, str(ref_root / "Dejavu"))
    import torch
    import triton.runtime.autotuner as autotuner

    autotuner.Autotuner._bench = lambda self, *a, config=None, **k: [0.0, 0.0, 0.0]
    from src.ops.triton.attention_proj_sparse import (k_cache_copy_sparse, out_proj_sparse,
                                                      qkv_proj_sparse, v_cache_copy_sparse)
    from src.ops.triton.gather_gemv import gather_gemv, gather_transposed_gemv, mlp_sparse

    out = {}
    rng = np.random.Generator(np.random.PCG64(1))
    T = torch.from_numpy
    # ---- gather GEMV pair ----
    Z, N, M = 96, 256, 40
    W1 = rng_normal(rng, (Z, N), 0.1, np.float16)
    W2t = rng_normal(rng, (Z, N), 0.1, np.float16)
    b1 = rng_normal(rng, (Z,), 0.1, np.float16)
    b2 = rng_normal(rng, (N,), 0.1, np.float16)
    idx = rng.permutation(Z)[:M].astype(np.int64)
    out.update(g_W1=W1, g_W2t=W2t, g_b1=b1, g_b2=b2, g_idx=idx)
    for B in (1, 2, 3, 4):
        x = rng_normal(rng, (B, N), 1.0, np.float16)
        h_id = gather_gemv(T(x), T(W1), T(idx), T(b1), "id").numpy()
        h = gather_gemv(T(x), T(W1), T(idx), T(b1), "relu").numpy()
        y = gather_transposed_gemv(T(h), T(W2t), T(idx), T(b2)).numpy()
        y_nobias = gather_transposed_gemv(T(h), T(W2t), T(idx), None).numpy()
        y_mlp = mlp_sparse(T(x), T(W1), T(W2t), T(idx), T(b1), T(b2)).numpy()
        out.update({f"g_x{B}": x, f"g_hid{B}": h_id, f"g_h{B}": h, f"g_y{B}": y, f"g_ynb{B}": y_nobias,
                    f"g_ymlp{B}": y_mlp})
    # ---- head-sparse projections ----
    nheads, hd, d, Tn = 6, 64, 256, 5
    Wqkv = rng_normal(rng, (3, nheads, hd, d), 0.1, np.float16)
    bqkv = rng_normal(rng, (3, nheads, hd), 0.1, np.float16)
    xq = rng_normal(rng, (Tn, d), 1.0, np.float16)
    head_idx = np.array([4, 1, 3], np.int32)
    batch_idx = np.array([[0, 1, 2, 3, 4], [-1, -1, 2, -1, 4], [-1, 1, -1, -1, -1]], np.int32)
    yq = qkv_proj_sparse(T(xq), T(Wqkv), T(head_idx), T(batch_idx), T(bqkv)).numpy()
    out.update(q_W=Wqkv, q_b=bqkv, q_x=xq, q_head_idx=head_idx, q_batch_idx=batch_idx, q_y=yq)
    Wo = rng_normal(rng, (d, nheads, hd), 0.1, np.float16)
    bo = rng_normal(rng, (d,), 0.1, np.float16)
    ctx = rng_normal(rng, (3, nheads, hd), 1.0, np.float16)
    yo = out_proj_sparse(T(ctx), T(Wo), T(head_idx), T(bo)).numpy()
    out.update(o_W=Wo, o_b=bo, o_x=ctx, o_y=yo)
    # ---- cache scatter ----
    S = 24
    kc = np.zeros((1, nheads, hd // 8, S, 8), np.float16)
    vc = np.zeros((1, nheads, S, hd), np.float16)
    pad = np.array([7], np.int32)
    kt, vt = T(kc.copy()), T(vc.copy())
    k_src = np.ascontiguousarray(np.nan_to_num(yq[:, 1]))
    v_src = np.ascontiguousarray(np.nan_to_num(yq[:, 2]))
    k_cache_copy_sparse(T(k_src), kt, T(head_idx), T(batch_idx), T(pad))
    v_cache_copy_sparse(T(v_src), vt, T(head_idx), T(batch_idx), T(pad))
    out.update(c_k=k_src, c_v=v_src, c_pad=pad, c_kcache=kt.numpy(), c_vcache=vt.numpy())
    return out


def block_case(ref_root: Path):
    """GPTBlock.forward of the accuracy path on config 1 (fp32, CPU), one decode token with 8 cached ones."""
    import torch
    from torch import nn

    sys.path.insert(0, str(ref_root / "Decentralized_FM_alpha"))
    from modules.hf_opt_sparse_mlp_attention import GPTBlock

    # stub the CUDA stream constructors only after transformers has been imported
    torch.cuda.default_stream = lambda *a, **k: None
    torch.cuda.Stream = lambda *a, **k: None
    torch.cuda.Event = lambda *a, **k: None

    t = config1_inputs(0)
    d, ffn, H, K, KH = 768, 3072, 12, 384, 4
    cfg = types.SimpleNamespace(hidden_size=d, num_attention_heads=H, attention_dropout=0.0,
                                do_layer_norm_before=True, dropout=0.0, activation_function="relu",
                                activation_dropout=0.0, ffn_dim=ffn)
    blk = GPTBlock(cfg, device="cpu").eval()
    T = torch.from_numpy
    with torch.no_grad():
        blk.fc1.weight.copy_(T(t["W1"])); blk.fc1.bias.copy_(T(t["b1"]))
        # from_pretrained stores fc2 transposed and forward multiplies by its .T (:485, :556)
        blk.fc2.weight.data = T(t["W2"]).t().contiguous(); blk.fc2.bias.copy_(T(t["b2"]))
        for nm, lin in (("q", blk.self_attn.q_proj), ("k", blk.self_attn.k_proj),
                        ("v", blk.self_attn.v_proj), ("o", blk.self_attn.out_proj)):
            lin.weight.copy_(T(t["W" + nm])); lin.bias.copy_(T(t["b" + nm]))
        blk.predictor = nn.Sequential(nn.Linear(d, 1000, bias=None), nn.Linear(1000, ffn, bias=None))
        blk.predictor[0].weight.copy_(T(t["P0"])); blk.predictor[1].weight.copy_(T(t["P1"]))
        blk.topk = K
        blk.self_attn.predictor = nn.Sequential(nn.Linear(d, 1000, bias=None), nn.Linear(1000, H, bias=None))
        blk.self_attn.predictor[0].weight.copy_(T(t["A0"])); blk.self_attn.predictor[1].weight.copy_(T(t["A1"]))
        blk.self_attn.topk = float(KH)
        y, present = blk(T(t["x"]), layer_past=(T(t["past_k"]), T(t["past_v"])), mask=None,
                         previous_emb=T(t["prev"]))
        mlp_idx = torch.nonzero(blk._mask[0]).flatten().numpy()
        head_mask = blk.self_attn.prepare_head_mask(T(t["prev"]))
        head_idx = torch.nonzero(head_mask[0, :, 0]).flatten().numpy()
    return {
        "b_y": y.numpy(), "b_mlp_idx": mlp_idx.astype(np.int64), "b_head_idx": head_idx.astype(np.int64),
        "b_k_new": present[0][0, :, -1].numpy(), "b_v_new": present[1][0, :, -1].numpy(),
        "b_input_checksum": np.array(checksum(t)),
    }


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of FMInference/DejaVu to import and run")
    a = ap.parse_args()
    root = Path(a.reference)
    blk = block_case(root)
    np.savez_compressed(HERE / "block_config1.npz", **blk)
    tri = triton_cases(root)
    np.savez_compressed(HERE / "triton_ops.npz", **tri)
    for f in ("block_config1.npz", "triton_ops.npz"):
        print(f, (HERE / f).stat().st_size, "bytes")
