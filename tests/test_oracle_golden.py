"""The CPU oracle against vectors produced by the reference itself (tests/golden/make_golden.py)."""
import sys
from pathlib import Path

import numpy as np
import torch

from oracle import oracle as O

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
from make_golden import checksum, config1_inputs  # noqa: E402

ATOL, RTOL = 1e-3, 1e-2  # fp16 tolerance named by the north star


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def close(a, b, atol=ATOL, rtol=RTOL):
    a, b = torch.as_tensor(a).float(), torch.as_tensor(b).float()
    assert a.shape == b.shape
    assert torch.allclose(a, b, atol=atol, rtol=rtol), f"max abs diff {(a - b).abs().max().item()}"


def test_gather_gemv_matches_reference_kernel(golden_ops):
    g = golden_ops
    W1, b1, idx = T(g["g_W1"]), T(g["g_b1"]), T(g["g_idx"])
    for B in (1, 2, 3, 4):
        x = T(g[f"g_x{B}"])
        close(O.gather_gemv(x, W1, idx, b1, "id"), g[f"g_hid{B}"])
        close(O.gather_gemv(x, W1, idx, b1, "relu"), g[f"g_h{B}"])


def test_gather_transposed_gemv_matches_reference_kernel(golden_ops):
    g = golden_ops
    W2t, b2, idx = T(g["g_W2t"]), T(g["g_b2"]), T(g["g_idx"])
    for B in (1, 2, 3, 4):
        h = T(g[f"g_h{B}"])
        close(O.gather_transposed_gemv(h, W2t, idx, b2), g[f"g_y{B}"])
        close(O.gather_transposed_gemv(h, W2t, idx, None), g[f"g_ynb{B}"])


def test_mlp_sparse_matches_reference_kernel(golden_ops):
    g = golden_ops
    for B in (1, 2, 3, 4):
        y = O.mlp_sparse(T(g[f"g_x{B}"]), T(g["g_W1"]), T(g["g_W2t"]), T(g["g_idx"]), T(g["g_b1"]), T(g["g_b2"]))
        close(y, g[f"g_ymlp{B}"])


def test_qkv_proj_sparse_matches_reference_kernel(golden_ops):
    g = golden_ops
    y = O.qkv_proj_sparse(T(g["q_x"]), T(g["q_W"]), T(g["q_head_idx"]), T(g["q_batch_idx"]), T(g["q_b"]))
    computed = ~torch.isnan(y.float())
    # every (row, head) the reference computes is computed by the oracle, and agrees
    for i, h in enumerate(g["q_head_idx"].tolist()):
        for t in g["q_batch_idx"][i].tolist():
            if t >= 0:
                assert computed[t, :, h].all()
                close(y[t, :, h], g["q_y"][t, :, h])
    assert int(computed[:, 0, :, 0].sum()) == int((g["q_batch_idx"] >= 0).sum())


def test_out_proj_sparse_matches_reference_kernel(golden_ops):
    g = golden_ops
    close(O.out_proj_sparse(T(g["o_x"]), T(g["o_W"]), T(g["q_head_idx"]), T(g["o_b"])), g["o_y"], atol=2e-3)


def test_cache_copy_matches_reference_kernel(golden_ops):
    g = golden_ops
    kc = torch.zeros_like(T(g["c_kcache"]))
    vc = torch.zeros_like(T(g["c_vcache"]))
    O.k_cache_copy_sparse(T(g["c_k"]), kc, T(g["q_head_idx"]), T(g["q_batch_idx"]), T(g["c_pad"]))
    O.v_cache_copy_sparse(T(g["c_v"]), vc, T(g["q_head_idx"]), T(g["q_batch_idx"]), T(g["c_pad"]))
    assert torch.equal(kc, T(g["c_kcache"]))
    assert torch.equal(vc, T(g["c_vcache"]))


def test_k_cache_pack_roundtrip():
    k = torch.randn(2, 7, 3, 64)
    packed = O.pack_k_cache(k)
    assert packed.shape == (2, 3, 8, 7, 8)
    assert torch.equal(O.unpack_k_cache(packed), k.permute(0, 2, 1, 3))


def test_block_config1_matches_reference_block(golden_block):
    """Oracle pieces assembled into the accuracy path's block equal the reference block's output."""
    gb = golden_block
    t = {k: T(v) for k, v in config1_inputs(0).items()}
    assert abs(checksum(config1_inputs(0)) - float(gb["b_input_checksum"])) < 1e-6, "input generator drifted"
    d, H, K, KH = 768, 12, 384, 4
    x, prev = t["x"][0], t["prev"][0]  # (1, d)
    ln_w, ln_b = torch.ones(d), torch.zeros(d)
    # attention half: head mask from the predictor on previous_emb
    a_scores = (prev @ t["A0"].T) @ t["A1"].T
    head_idx = O.topk_indices(a_scores[0], KH)
    assert head_idx.tolist() == gb["b_head_idx"].tolist()
    h = torch.nn.functional.layer_norm(x, (d,), ln_w, ln_b, 1e-5)
    att, k_new, v_new = O.head_masked_attention(h, t["Wq"], t["bq"], t["Wk"], t["bk"], t["Wv"], t["bv"],
                                                t["Wo"], t["bo"], t["past_k"][0], t["past_v"][0], head_idx, H)
    close(k_new, gb["b_k_new"], atol=1e-5, rtol=1e-5)
    close(v_new, gb["b_v_new"], atol=1e-5, rtol=1e-5)
    hidden = x + att
    # MLP half: scores on the block input, index_select form
    scores = (x @ t["P0"].T) @ t["P1"].T
    idx = O.topk_indices_fast(scores[0], K)
    assert idx.tolist() == gb["b_mlp_idx"].tolist()
    h2 = torch.nn.functional.layer_norm(hidden, (d,), ln_w, ln_b, 1e-5)
    a = torch.relu(h2 @ t["W1"][idx].T + t["b1"][idx])
    y = a @ t["W2"][:, idx].T + t["b2"] + hidden
    close(y, gb["b_y"][0], atol=1e-4, rtol=1e-4)
    # and the mask form gives the same MLP product
    y_mask = O.mlp_mask_form(h2, t["W1"], t["b1"], t["W2"], t["b2"], idx) + hidden
    close(y_mask, gb["b_y"][0], atol=1e-4, rtol=1e-4)


def test_config1_sparse_mlp_block_index_equals_mask_form():
    t = {k: T(v) for k, v in config1_inputs(0).items()}
    d = 768
    x = t["x"][0]
    y, idx, scores = O.sparse_mlp_block_fp32(x, torch.ones(d), torch.zeros(d), t["W1"], t["b1"], t["W2"],
                                             t["b2"], t["P0"], t["P1"], 384)
    assert idx.numel() == 384 and torch.equal(idx, torch.sort(idx).values)
    rest = torch.ones(scores.shape[1], dtype=torch.bool)
    rest[idx] = False
    assert scores[0][idx].min() >= scores[0][rest].max()
    h = torch.nn.functional.layer_norm(x, (d,), torch.ones(d), torch.zeros(d), 1e-5)
    y_mask = O.mlp_mask_form(h, t["W1"], t["b1"], t["W2"], t["b2"], idx) + x
    close(y, y_mask, atol=1e-5, rtol=1e-5)
    # fp16 operator form against fp32 block within the fp16 tolerance
    y16 = O.mlp_sparse(h.half(), t["W1"].half(), t["W2"].t().contiguous().half(), idx, t["b1"].half(),
                       t["b2"].half()).float() + x
    close(y16, y, atol=5e-3, rtol=1e-2)


def test_topk_rule_and_ties():
    s = torch.tensor([1.0, 3.0, 3.0, 2.0, 3.0, float("nan"), -1.0, 2.0], dtype=torch.float16)
    assert O.topk_indices(s, 1).tolist() == [5]
    assert O.topk_indices(s, 3).tolist() == [1, 2, 5]
    assert O.topk_indices(s, 4).tolist() == [1, 2, 4, 5]
    assert O.topk_indices(s, 5).tolist() == [1, 2, 3, 4, 5]
    for k in range(0, 9):
        assert O.topk_indices(s, k).tolist() == O.topk_indices_fast(s, k).tolist()
    g = torch.Generator().manual_seed(3)
    r = torch.randn(5000, generator=g).half()  # fp16 rounding makes ties common
    for k in (1, 17, 512, 4999, 5000):
        a, b = O.topk_indices_fast(r, k), torch.topk(r.float(), k).indices
        assert r[a].float().sort().values.tolist() == r[b].float().sort().values.tolist()
        if k < 5000:
            rest = torch.ones(5000, dtype=torch.bool)
            rest[a] = False
            assert r[a].min() >= r[rest].max()


def test_tp_sharded_mlp_equals_unsharded_with_sharded_selection():
    g = torch.Generator().manual_seed(0)
    d, F, K, world = 128, 512, 64, 4
    W1 = (torch.randn(F, d, generator=g) * 0.05).half()
    W2t = (torch.randn(F, d, generator=g) * 0.05).half()
    b1 = (torch.randn(F, generator=g) * 0.05).half()
    b2 = (torch.randn(d, generator=g) * 0.05).half()
    x = torch.randn(1, d, generator=g).half()
    scores = torch.randn(F, generator=g).half()
    y_tp, picked = O.mlp_sparse_tp(x, W1, b1, W2t, b2, scores, K, world)
    idx_all = torch.cat(picked)
    assert idx_all.numel() == K and idx_all.unique().numel() == K
    close(y_tp, O.mlp_sparse(x, W1, W2t, idx_all, b1, b2), atol=2e-3)


def test_lazy_kv_equals_full_kv_with_head_mask():
    """The lazy K/V state machine produces, for the heads in use, exactly the context of full-KV attention."""
    g = torch.Generator().manual_seed(1)
    nheads, hd, d, P, steps, S = 6, 32, 64, 5, 37, 64
    Wqkv = (torch.randn(3, nheads, hd, d, generator=g) * 0.1).half()
    bqkv = (torch.randn(3, nheads, hd, generator=g) * 0.1).half()
    scale = hd ** -0.5
    # prompt K,V (dense)
    xp = torch.randn(P, d, generator=g).half()
    kv_p = torch.einsum("qhdn,tn->tqhd", Wqkv.float(), xp.float()) + bqkv.float()
    k_lazy = torch.zeros(1, nheads, hd // 8, S, 8, dtype=torch.float16)
    v_lazy = torch.zeros(1, nheads, S, hd, dtype=torch.float16)
    k_lazy[0, :, :, :P] = O.pack_k_cache(kv_p[None, :, 1].half())[0]
    v_lazy[0, :, :P] = kv_p[:, 2].half().permute(1, 0, 2)
    k_full, v_full = k_lazy.clone(), v_lazy.clone()
    state = O.LazyKVState(nheads, P)
    ring = torch.zeros(O.KV_WINDOW, d, dtype=torch.float16)
    for t in range(steps):
        x = torch.randn(d, generator=g).half()
        sel = torch.randperm(nheads, generator=g)[:2].tolist()
        flush_expected = state.slot == O.KV_WINDOW - 1
        ctx, heads = O.attn_sparse_step(state, x, ring, Wqkv, bqkv, k_lazy, v_lazy, sel, scale)
        assert heads == (list(range(nheads)) if flush_expected else sorted(sel))
        # full-KV reference: every head gets K,V every step
        qkv = torch.einsum("qhdn,n->qhd", Wqkv.float(), x.float()) + bqkv.float()
        pos = P + t
        k_full[0, :, :, pos, :] = qkv[1].half().reshape(nheads, hd // 8, 8)
        v_full[0, :, pos] = qkv[2].half()
        full = O.decode_attention(qkv[0].half()[None], k_full, v_full, None, pos + 1, scale)[0]
        for h in heads:
            close(ctx[h], full[h], atol=1e-3)
        state.finish_step()
        if state.slot == 0:
            assert all(p == 0 for p in state.pending)
            assert torch.equal(k_lazy[..., : pos + 1, :], k_full[..., : pos + 1, :])
            assert torch.equal(v_lazy[:, :, : pos + 1], v_full[:, :, : pos + 1])


def test_head_masked_attention_equals_decode_attention_on_selected_heads():
    g = torch.Generator().manual_seed(2)
    H, hd, S = 4, 32, 9
    d = H * hd
    W = {n: torch.randn(d, d, generator=g) * 0.1 for n in "qkvo"}
    b = {n: torch.randn(d, generator=g) * 0.1 for n in "qkvo"}
    x = torch.randn(1, d, generator=g)
    pk, pv = torch.randn(H, S, hd, generator=g), torch.randn(H, S, hd, generator=g)
    sel = torch.tensor([0, 2])
    out, k_new, v_new = O.head_masked_attention(x, W["q"], b["q"], W["k"], b["k"], W["v"], b["v"], W["o"], b["o"],
                                                pk, pv, sel, H)
    K = torch.cat([pk, k_new[:, None]], 1)
    V = torch.cat([pv, v_new[:, None]], 1)
    q = (x @ W["q"].T + b["q"]).view(1, H, hd)
    ctx = O.decode_attention(q, O.pack_k_cache(K.permute(1, 0, 2)[None]), V[None], sel.int(), S + 1, hd ** -0.5)
    y = O.out_proj_sparse(ctx, W["o"].view(d, H, hd), sel.int(), b["o"])
    close(y, out, atol=1e-4, rtol=1e-4)


def test_add_layernorm():
    g = torch.Generator().manual_seed(4)
    x, r = torch.randn(2, 64, generator=g).half(), torch.randn(2, 64, generator=g).half()
    w, b = torch.randn(64, generator=g).half(), torch.randn(64, generator=g).half()
    y, rr = O.add_layernorm(x, r, w, b, 1e-5)
    assert torch.equal(rr, (x.float() + r.float()).half())
    ref = torch.nn.functional.layer_norm(rr.float(), (64,), w.float(), b.float(), 1e-5)
    close(y, ref)
