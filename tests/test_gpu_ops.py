"""Parity of the sm_100a kernels (called through the C ABI) with the CPU oracle and with the vectors
the reference's own kernels produced. Tolerances: fp16 outputs atol 1e-3 / rtol 1e-2; index sets exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-3, 1e-2


def T(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def close(a, b, atol=ATOL, rtol=RTOL):
    a, b = torch.as_tensor(a).float().cpu(), torch.as_tensor(b).float().cpu()
    assert a.shape == b.shape
    bad = ~torch.isclose(a, b, atol=atol, rtol=rtol)
    assert not bad.any(), f"{int(bad.sum())} mismatches, max abs diff {(a - b).abs().max().item()}"


def rand(gen, shape, std=1.0):
    return (torch.randn(shape, generator=gen) * std).half()


# ---------------------------------------------------------------------------------------------
# golden vectors from the reference's Triton kernels
# ---------------------------------------------------------------------------------------------
def test_golden_gather_pair(cuda, golden_ops):
    from dejavu_b200 import ops

    g = golden_ops
    W1, W2t, b1, b2, idx = (T(g[k], cuda) for k in ("g_W1", "g_W2t", "g_b1", "g_b2", "g_idx"))
    for B in (1, 2, 3, 4):
        x = T(g[f"g_x{B}"], cuda)
        close(ops.gather_gemv(x, W1, idx, b1, "id"), g[f"g_hid{B}"])
        h = ops.gather_gemv(x, W1, idx, b1, "relu")
        close(h, g[f"g_h{B}"])
        close(ops.gather_transposed_gemv(T(g[f"g_h{B}"], cuda), W2t, idx, b2), g[f"g_y{B}"])
        close(ops.gather_transposed_gemv(T(g[f"g_h{B}"], cuda), W2t, idx, None), g[f"g_ynb{B}"])
        close(ops.mlp_sparse(x, W1, W2t, idx, b1, b2), g[f"g_ymlp{B}"])
        close(ops.mlp_sparse(x, W1, W2t, idx.int(), b1, b2), g[f"g_ymlp{B}"])


def test_golden_attention_projections(cuda, golden_ops):
    from dejavu_b200 import ops

    g = golden_ops
    hi, bi = T(g["q_head_idx"], cuda), T(g["q_batch_idx"], cuda)
    y = ops.qkv_proj_sparse(T(g["q_x"], cuda), T(g["q_W"], cuda), hi, bi, T(g["q_b"], cuda))
    for i, h in enumerate(g["q_head_idx"].tolist()):
        for t in g["q_batch_idx"][i].tolist():
            if t >= 0:
                close(y[t, :, h], g["q_y"][t, :, h])
    close(ops.out_proj_sparse(T(g["o_x"], cuda), T(g["o_W"], cuda), hi, T(g["o_b"], cuda)), g["o_y"], atol=2e-3)
    kc = torch.zeros(g["c_kcache"].shape, dtype=torch.float16, device=cuda)
    vc = torch.zeros(g["c_vcache"].shape, dtype=torch.float16, device=cuda)
    ops.k_cache_copy_sparse(T(g["c_k"], cuda), kc, hi, bi, T(g["c_pad"], cuda))
    ops.v_cache_copy_sparse(T(g["c_v"], cuda), vc, hi, bi, T(g["c_pad"], cuda))
    assert torch.equal(kc.cpu(), torch.from_numpy(g["c_kcache"]))
    assert torch.equal(vc.cpu(), torch.from_numpy(g["c_vcache"]))


# ---------------------------------------------------------------------------------------------
# gather GEMV pair against the oracle
# ---------------------------------------------------------------------------------------------
GATHER_CASES = [
    # Z, N, M, B, idx kind
    (3072, 768, 384, 1, "rand64"),     # BASELINE config 1 shape
    (3072, 768, 384, 3, "sorted32"),
    (6144, 12288, 512, 1, "rand64"),   # 175B TP8 shard, K/8 = 512
    (6144, 12288, 130, 2, "rand32"),   # K not a multiple of any tile
    (6144, 12288, 1, 1, "rand32"),
    (6144, 12288, 6144, 1, "perm32"),  # dense via a permutation
    (4608, 9216, 512, 4, "dup32"),     # 66B TP8 shard, duplicate indices
    (16384, 4096, 2048, 1, "rand64"),  # 6.7B
    (2048, 1000, 2048, 1, "none"),     # predictor fc1: rows of 2000 bytes, identity index
    (1000, 4096, 1000, 1, "none"),     # predictor fc0
    (512, 256, 77, 7, "rand32"),
    (512, 256, 64, 8, "rand32"),
    (512, 256, 64, 16, "rand32"),      # batch cut into slices
    (512, 256, 33, 32, "rand64"),
    (6144, 12288, 512, 16, "rand32"),  # tensor-core path at the 175B shard shape
    (6144, 12288, 100, 9, "rand64"),
    (2048, 1000, 300, 24, "rand32"),   # row length not a multiple of 32
    (4608, 9216, 77, 32, "dup32"),
    (6144, 2048, 5000, 12, "rand32"),  # long lists: several 16-row tiles per block (fc1), many ring steps (fc2)
    (6144, 1024, 4800, 32, "rand32"),
    (6144, 1024, 4805, 20, "rand64"),  # ragged last tile; activations not 16-byte aligned per row
    (2048, 1000, 304, 24, "sorted32"), # last column tile partly outside the rows
    (8192, 512, 2500, 5, "dup64"),
    (12000, 1000, 10000, 16, "rand32"),  # short rows, long list: a 16-row tile per warp
    (16384, 1000, 16384, 9, "none"),     # the predictor's second layer for a batch
    (10000, 264, 9999, 32, "rand64"),
]


def make_idx(kind, Z, M, gen):
    if kind == "none":
        return None
    if kind.startswith("dup"):
        idx = torch.randint(0, Z, (M,), generator=gen)
    elif kind.startswith("perm"):
        idx = torch.randperm(Z, generator=gen)[:M]
    else:
        idx = torch.randperm(Z, generator=gen)[:M]
        if kind.startswith("sorted"):
            idx = idx.sort().values
    return idx.to(torch.int32 if kind.endswith("32") else torch.int64)


@pytest.mark.parametrize("Z,N,M,B,kind", GATHER_CASES)
def test_gather_gemv_vs_oracle(cuda, Z, N, M, B, kind):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(Z * 7 + M)
    W, bias = rand(gen, (Z, N), 0.02), rand(gen, (Z,), 0.1)
    x = rand(gen, (B, N))
    idx = make_idx(kind, Z, M, gen)
    idx_o = torch.arange(M) if idx is None else idx
    for act, bb in (("relu", bias), ("id", None)):
        ref = O.gather_gemv(x, W, idx_o, bb, act)
        if idx is None:
            got = ops.dense_gemv(x.to(cuda), W.to(cuda)[:M], None if bb is None else bb.to(cuda), act)
        else:
            got = ops.gather_gemv(x.to(cuda), W.to(cuda), idx.to(cuda), None if bb is None else bb.to(cuda), act)
        close(got, ref)


@pytest.mark.parametrize("act", ["gelu", "gelu_approx", "squared_relu"])
def test_gather_gemv_activations(cuda, act):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(11)
    W, bias, x = rand(gen, (256, 512), 0.05), rand(gen, (256,), 0.1), rand(gen, (2, 512))
    idx = torch.randperm(256, generator=gen)[:100]
    close(ops.gather_gemv(x.to(cuda), W.to(cuda), idx.to(cuda), bias.to(cuda), act), O.gather_gemv(x, W, idx, bias, act))


@pytest.mark.parametrize("Z,N,M,B,kind", [c for c in GATHER_CASES if c[4] != "none"])
def test_gather_transposed_gemv_vs_oracle(cuda, Z, N, M, B, kind):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(Z * 3 + M)
    W, bias = rand(gen, (Z, N), 0.02), rand(gen, (N,), 0.1)
    h = torch.relu(rand(gen, (B, M)))
    idx = make_idx(kind, Z, M, gen)
    ref = O.gather_transposed_gemv(h, W, idx, bias)
    got = ops.gather_transposed_gemv(h.to(cuda), W.to(cuda), idx.to(cuda), bias.to(cuda))
    # |y| grows with sqrt(M): keep the relative tolerance, scale the absolute one with the output size
    close(got, ref, atol=max(ATOL, 2e-3 * float(ref.float().abs().max())))
    again = ops.gather_transposed_gemv(h.to(cuda), W.to(cuda), idx.to(cuda), bias.to(cuda))
    assert torch.equal(got, again), "summation order must be fixed"
    close(ops.gather_transposed_gemv(h.to(cuda), W.to(cuda), idx.to(cuda), None), O.gather_transposed_gemv(h, W, idx, None),
          atol=max(ATOL, 2e-3 * float(ref.float().abs().max())))


def test_empty_index_list(cuda):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(5)
    W, b1, b2, x = rand(gen, (64, 128)), rand(gen, (64,)), rand(gen, (128,)), rand(gen, (2, 128))
    idx = torch.zeros(0, dtype=torch.int64)
    h = ops.gather_gemv(x.to(cuda), W.to(cuda), idx.to(cuda), b1.to(cuda), "relu")
    assert h.shape == (2, 0)
    y = ops.gather_transposed_gemv(h, W.to(cuda), idx.to(cuda), b2.to(cuda))
    assert torch.equal(y.cpu(), b2.expand(2, 128))
    y0 = ops.gather_transposed_gemv(h, W.to(cuda), idx.to(cuda), None)
    assert torch.equal(y0.cpu(), torch.zeros(2, 128, dtype=torch.float16))


def test_full_size_properties_175b_shard(cuda):
    """BASELINE config 5 shapes (d 12288, ffn shard 6144): properties that need no CPU product."""
    from dejavu_b200 import ops

    gen = torch.Generator(device=cuda).manual_seed(0)
    F_, d = 6144, 12288
    W1 = (torch.randn(F_, d, device=cuda, generator=gen) * 0.02).half()
    W2t = (torch.randn(F_, d, device=cuda, generator=gen) * 0.02).half()
    b1 = (torch.randn(F_, device=cuda, generator=gen) * 0.02).half()
    x = torch.randn(4, d, device=cuda, generator=gen).half()
    for K in (128, 512, 4096, 6144):
        idx = torch.randperm(F_, device=cuda, generator=gen)[:K]
        h = ops.gather_gemv(x, W1, idx, b1, "relu")
        # 1. permuting idx permutes fc1's output bit-exactly
        perm = torch.randperm(K, device=cuda, generator=gen)
        assert torch.equal(ops.gather_gemv(x, W1, idx[perm], b1, "relu"), h[:, perm])
        # 2. sorted and unsorted index lists give the same fc2 sum (different order -> tolerance)
        y = ops.gather_transposed_gemv(h, W2t, idx, None)
        order = idx.sort().indices
        y_sorted = ops.gather_transposed_gemv(h[:, order], W2t, idx[order], None)
        close(y_sorted, y, atol=2e-3)
        # 3. the gathered product equals the dense product with unselected neurons zeroed (mask form)
        mask = torch.zeros(F_, device=cuda, dtype=torch.float32)
        mask[idx] = 1
        dense = torch.relu((x.float() @ W1.float().T + b1.float()) * mask)
        close(h, dense[:, idx])
        close(y, dense.half().float() @ W2t.float(), atol=3e-3)
        # 4. batch rows are independent (batch 1 and batch 4 use different lane layouts, so the fp32
        #    sums are added in a different order: tolerance, not bits)
        close(ops.gather_gemv(x[2:3], W1, idx, b1, "relu")[0], h[2])
    # 5. linearity of fc2 in its input
    idx = torch.randperm(F_, device=cuda, generator=gen)[:1024]
    a = torch.relu(torch.randn(1, 1024, device=cuda, generator=gen)).half()
    y1 = ops.gather_transposed_gemv(a, W2t, idx, None).float()
    y2 = ops.gather_transposed_gemv((a * 2).half(), W2t, idx, None).float()
    close(y2, 2 * y1, atol=2e-3)


@pytest.mark.parametrize("B,N", [(2, 4096), (5, 1000), (32, 36864), (1, 7)])
def test_batch_sum_adds_rows_in_fp32_in_order(cuda, B, N):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(B * N)
    x = rand(gen, (B, N))
    acc = torch.zeros(N, dtype=torch.float32)
    for b in range(B):
        acc += x[b].float()
    got = ops.batch_sum(x.to(cuda))
    assert got.shape == (1, N)
    assert torch.equal(got[0].cpu(), acc.half())


def test_outputs_stay_inside_their_buffers(cuda):
    """Canary words around y: the kernels must not write outside (B,M) / (B,N)."""
    from dejavu_b200 import _lib

    gen = torch.Generator().manual_seed(9)
    Z, N, M, B = 300, 264, 77, 3
    W, x = rand(gen, (Z, N)).to(cuda), rand(gen, (B, N)).to(cuda)
    idx = torch.randperm(Z, generator=gen)[:M].int().to(cuda)
    st = torch.cuda.current_stream().cuda_stream
    pad = 64
    buf = torch.full((pad + B * M + pad,), 7.0, dtype=torch.float16, device=cuda)
    _lib.call("djv_gather_gemv", buf.data_ptr() + pad * 2, W.data_ptr(), x.data_ptr(), idx.data_ptr(), None,
              B, N, M, N, 0, 1, st)
    assert (buf[:pad] == 7).all() and (buf[pad + B * M:] == 7).all()
    h = buf[pad:pad + B * M].clone().view(B, M)
    need = _lib.load().djv_gather_transposed_gemv_scratch_bytes(B, N, M)
    scratch = torch.zeros(need + 256, dtype=torch.uint8, device=cuda)
    buf2 = torch.full((pad + B * N + pad,), 7.0, dtype=torch.float16, device=cuda)
    _lib.call("djv_gather_transposed_gemv", buf2.data_ptr() + pad * 2, W.data_ptr(), h.data_ptr(), idx.data_ptr(),
              None, B, N, M, N, 0, scratch.data_ptr(), need, st)
    assert (buf2[:pad] == 7).all() and (buf2[pad + B * N:] == 7).all()
    assert (scratch[:4096] == 0).all(), "block counters must be left at zero"
    assert (scratch[need:] == 0).all(), "scratch overrun"
    with pytest.raises(_lib.DejavuKernelError) as e:
        _lib.call("djv_gather_transposed_gemv", buf2.data_ptr() + pad * 2, W.data_ptr(), h.data_ptr(),
                  idx.data_ptr(), None, B, N, M, N, 0, scratch.data_ptr(), 4096, st)
    assert e.value.status == _lib.ERR_SCRATCH


# ---------------------------------------------------------------------------------------------
# top-K
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k", [(1, 1), (12, 4), (96, 32), (1000, 0), (1000, 1000), (4608, 512), (16384, 2048),
                                 (36864, 4096), (49152, 6144), (50272, 1), (4096, 4096), (4100, 7), (4099, 0),
                                 (200000, 5000)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_topk_exact_index_sets(cuda, n, k, dtype):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(n + k)
    s = torch.randn(n, generator=gen).to(dtype)
    if dtype == torch.float16 and n > 100:
        s = (s * 4).round() / 4  # many exact ties
    ref = O.topk_indices_fast(s, k)
    for out_dtype in (torch.int32, torch.int64):
        got = ops.topk_indices(s.to(cuda), k, out_dtype)
        assert got.dtype == out_dtype
        assert got.cpu().tolist() == ref.tolist()


def test_topk_special_values(cuda):
    from dejavu_b200 import ops

    s = torch.tensor([1.0, float("inf"), -0.0, 0.0, float("nan"), -float("inf"), 3.0, 3.0, -2.0], dtype=torch.float16)
    for k in range(0, 10):
        assert ops.topk_indices(s.to(cuda), k, torch.int32).cpu().tolist() == O.topk_indices(s, k).tolist()
    # the same special values inside a vector long enough for the cluster kernel, spread over its blocks
    gen = torch.Generator().manual_seed(3)
    long = torch.randn(6000, generator=gen).half()
    for i, v in enumerate(s.tolist()):
        long[(i * 677) % 6000] = v
    long[5999] = float("nan")
    for k in (1, 2, 3, 5, 2999, 5998, 6000):
        assert ops.topk_indices(long.to(cuda), k, torch.int32).cpu().tolist() == O.topk_indices_fast(long, k).tolist()
    s2 = torch.randn(300).half()
    got = ops.topk_indices(s2.to(cuda), 50, torch.int64).cpu()
    rest = torch.ones(300, dtype=torch.bool)
    rest[got] = False
    assert s2[got].min() >= s2[rest].max()


# ---------------------------------------------------------------------------------------------
# attention operators
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("nheads,hd,d,T_,nnz", [(12, 128, 12288, 16, 4), (9, 128, 9216, 1, 3), (32, 128, 4096, 5, 12),
                                                 (8, 64, 512, 16, 8), (4, 32, 256, 3, 1)])
@pytest.mark.parametrize("rpb", [0, 32, 16, 8, 1])  # 0: the library's own choice; 32, 16, 8 run on tensor cores
def test_qkv_proj_sparse_vs_oracle(cuda, monkeypatch, nheads, hd, d, T_, nnz, rpb):
    from dejavu_b200 import ops

    if rpb:
        monkeypatch.setenv("DJV_QKV_RPB", str(rpb))
    gen = torch.Generator().manual_seed(nheads * d)
    W, b = rand(gen, (3, nheads, hd, d), 0.02), rand(gen, (3, nheads, hd), 0.1)
    x = rand(gen, (T_, d))
    head_idx = torch.randperm(nheads, generator=gen)[:nnz].int()
    batch_idx = torch.arange(T_, dtype=torch.int32).repeat(nnz, 1)
    batch_idx[torch.rand(nnz, T_, generator=gen) < 0.4] = -1
    batch_idx[:, -1] = T_ - 1
    ref = O.qkv_proj_sparse(x, W, head_idx, batch_idx, b)
    got = ops.qkv_proj_sparse(x.to(cuda), W.to(cuda), head_idx.to(cuda), batch_idx.to(cuda), b.to(cuda)).cpu()
    m = ~torch.isnan(ref.float())
    close(got[m], ref[m])


@pytest.mark.parametrize("nheads,hd,d,B,nnz", [(12, 128, 12288, 1, 4), (12, 128, 12288, 16, 4), (9, 128, 9216, 1, 3),
                                                (32, 128, 4096, 1, 12), (8, 64, 512, 3, 5), (4, 32, 256, 2, 4),
                                                (12, 128, 1536, 1, 0)])
def test_out_proj_sparse_vs_oracle(cuda, nheads, hd, d, B, nnz):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(nheads * d + B)
    W, b = rand(gen, (d, nheads, hd), 0.02), rand(gen, (d,), 0.1)
    x = rand(gen, (B, nheads, hd))
    head_idx = torch.randperm(nheads, generator=gen)[:nnz].int()
    ref = O.out_proj_sparse(x, W, head_idx, b)
    got = ops.out_proj_sparse(x.to(cuda), W.to(cuda), head_idx.to(cuda), b.to(cuda))
    close(got, ref, atol=2e-3)


@pytest.mark.parametrize("B,nheads,hd,S,length,nnz", [(1, 12, 128, 768, 700, 4), (1, 12, 128, 2048, 2048, 12),
                                                       (2, 8, 64, 96, 1, 3), (1, 4, 32, 300, 129, 2),
                                                       (1, 36, 128, 256, 130, 12), (3, 4, 128, 1100, 1100, 4)])
def test_decode_attention_vs_oracle(cuda, B, nheads, hd, S, length, nnz):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(S + length)
    q = rand(gen, (B, nheads, hd))
    k = rand(gen, (B, S, nheads, hd))
    v = rand(gen, (B, nheads, S, hd))
    kc = O.pack_k_cache(k)
    head_idx = None if nnz == nheads else torch.randperm(nheads, generator=gen)[:nnz].int()
    ref = O.decode_attention(q, kc, v, head_idx, length, hd ** -0.5)
    got = ops.decode_attention(q.to(cuda), kc.to(cuda), v.to(cuda), None if head_idx is None else head_idx.to(cuda),
                               length, hd ** -0.5).cpu()
    m = ~torch.isnan(ref.float())
    close(got[m], ref[m], atol=2e-3)


@pytest.mark.parametrize("B,d", [(1, 768), (1, 4096), (2, 9216), (1, 12288), (3, 264)])
def test_add_layernorm_vs_oracle(cuda, B, d):
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(d)
    x, r = rand(gen, (B, d)), rand(gen, (B, d))
    w, b, xb = 1 + rand(gen, (d,), 0.1), rand(gen, (d,), 0.1), rand(gen, (d,), 0.1)
    for res, bias in ((r, None), (None, None), (r, xb)):
        y_ref, r_ref = O.add_layernorm(x, res, w, b, 1e-5, bias)
        y, rr = ops.add_layernorm(x.to(cuda), None if res is None else res.to(cuda), w.to(cuda), b.to(cuda), 1e-5,
                                  None if bias is None else bias.to(cuda))
        assert torch.equal(rr.cpu(), r_ref), "residual stream must be bit-exact"
        close(y, y_ref, atol=2e-3)


# ---------------------------------------------------------------------------------------------
# lazy K/V decode step (device-resident state) against the host model
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("nheads,hd,d,P,steps,nsel", [(6, 32, 256, 5, 37, 2), (12, 128, 1536, 40, 35, 4),
                                                       (9, 128, 1152, 130, 20, 3)])
@pytest.mark.parametrize("rpb", [0, 32, 16, 8, 1])  # rows per block of the QKV kernel; 32, 16, 8: tensor cores
@pytest.mark.parametrize("opened", [False, True])  # True: the top-K kernel opens the step (djv_topk_attn_prep)
def test_attn_step_state_machine_vs_oracle(cuda, monkeypatch, nheads, hd, d, P, steps, nsel, rpb, opened):
    from dejavu_b200 import _lib

    if rpb:
        monkeypatch.setenv("DJV_QKV_RPB", str(rpb))
    lib = _lib.load()
    gen = torch.Generator().manual_seed(nheads + P)
    S = P + steps + 8
    Wqkv, bqkv = rand(gen, (3, nheads, hd, d), 0.05), rand(gen, (3, nheads, hd), 0.1)
    scale = hd ** -0.5
    xp = rand(gen, (P, d))
    kv_p = torch.einsum("qhdn,tn->tqhd", Wqkv.float(), xp.float()) + bqkv.float()
    k_ref = torch.zeros(1, nheads, hd // 8, S, 8, dtype=torch.float16)
    v_ref = torch.zeros(1, nheads, S, hd, dtype=torch.float16)
    k_ref[0, :, :, :P] = O.pack_k_cache(kv_p[None, :, 1].half())[0]
    v_ref[0, :, :P] = kv_p[:, 2].half().permute(1, 0, 2)
    k_dev, v_dev = k_ref.to(cuda), v_ref.to(cuda)
    Wd, bd = Wqkv.to(cuda), bqkv.to(cuda)
    state_o = O.LazyKVState(nheads, P)
    ring_o = torch.zeros(O.KV_WINDOW, d, dtype=torch.float16)
    words = _lib.ATTN_STATE_HDR + 3 * nheads
    state_d = torch.full((words,), -7, dtype=torch.int32, device=cuda)
    ring_d = torch.zeros(O.KV_WINDOW, d, dtype=torch.float16, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    _lib.call("djv_attn_state_reset", state_d.data_ptr(), nheads, P, st)
    need = lib.djv_attn_step_scratch_bytes(nheads, hd, S)
    scratch = torch.zeros(max(need, 4096), dtype=torch.uint8, device=cuda)
    ctx_d = torch.zeros(nheads, hd, dtype=torch.float16, device=cuda)
    q_d = torch.zeros(nheads, hd, dtype=torch.float16, device=cuda)
    for t in range(steps):
        x = rand(gen, (d,))
        sel = torch.randperm(nheads, generator=gen)[:nsel].int()
        dense_step = (t == 3)  # a step without a head list uses every head
        ctx_o, heads = O.attn_sparse_step(state_o, x, ring_o, Wqkv, bqkv, k_ref, v_ref,
                                          None if dense_step else sel.tolist(), scale)
        xd, seld = x.to(cuda), sel.to(cuda)
        if opened and not dense_step:
            scores = torch.zeros(nheads, dtype=torch.float16)
            scores[sel.long()] = 1.0 + torch.rand(nsel, generator=gen).half()
            seld = torch.full((nsel,), -1, dtype=torch.int32, device=cuda)
            _lib.call("djv_topk_attn_prep", seld.data_ptr(), scores.to(cuda).data_ptr(), nheads, nsel, 0,
                      state_d.data_ptr(), S, st)
            assert seld.cpu().tolist() == sorted(sel.tolist())
            _lib.call("djv_attn_step_project", q_d.data_ptr(), Wd.data_ptr(), bd.data_ptr(), xd.data_ptr(),
                      ring_d.data_ptr(), k_dev.data_ptr(), v_dev.data_ptr(), state_d.data_ptr(), seld.data_ptr(),
                      nsel, d, nheads, hd, S, 1, st)
            _lib.call("djv_attn_step_attend", ctx_d.data_ptr(), q_d.data_ptr(), k_dev.data_ptr(), v_dev.data_ptr(),
                      state_d.data_ptr(), nheads, hd, S, scale, scratch.data_ptr(), scratch.numel(), st)
        else:
            _lib.call("djv_attn_step", ctx_d.data_ptr(), q_d.data_ptr(), Wd.data_ptr(), bd.data_ptr(),
                      xd.data_ptr(), ring_d.data_ptr(), k_dev.data_ptr(), v_dev.data_ptr(), state_d.data_ptr(),
                      None if dense_step else seld.data_ptr(), nsel, d, nheads, hd, S, scale, scratch.data_ptr(),
                      scratch.numel(), st)
        sd = state_d.cpu().tolist()
        n_eff = sd[2]
        assert sd[3] == 0
        eff = sd[_lib.ATTN_STATE_HDR + nheads:_lib.ATTN_STATE_HDR + nheads + n_eff]
        assert eff == heads, f"step {t}: heads in use {eff} != {heads}"
        assert sd[_lib.ATTN_STATE_HDR:_lib.ATTN_STATE_HDR + nheads] == state_o.pending
        got = ctx_d.cpu()
        for h in heads:
            close(got[h], ctx_o[h], atol=2e-3)
        _lib.call("djv_attn_step_finish", state_d.data_ptr(), nheads, st)
        state_o.finish_step()
        sd = state_d.cpu().tolist()
        assert (sd[0], sd[1]) == (state_o.slot, state_o.base)
    # caches agree wherever the host model has written K,V
    close(k_dev, k_ref, atol=2e-3)
    close(v_dev, v_ref, atol=2e-3)


# ---------------------------------------------------------------------------------------------
# tensor-parallel exchange on one GPU: the peers' pieces are written by the test before the launch
# (no kernel ever waits for another kernel), then a wait that nothing satisfies runs out
# ---------------------------------------------------------------------------------------------
SLOTS = 4
SENT = -32768  # 0x8000 as int16: fp16 -0.0


def _make_comm(lib, cuda, world, slot_bytes):
    import ctypes as C

    nbytes = lib.djv_comm_buffer_bytes(world, slot_bytes)
    assert nbytes == SLOTS * world * slot_bytes
    bufs_t = [torch.zeros(nbytes // 2, dtype=torch.int16, device=cuda) for _ in range(world)]
    bufs = (C.c_void_p * world)(*[t.data_ptr() for t in bufs_t])
    comm = C.c_void_p()
    from dejavu_b200 import _lib

    _lib.check("djv_comm_create", lib.djv_comm_create(C.byref(comm), 0, world, bufs, slot_bytes))
    return comm, bufs_t


def _no_neg_zero(t):
    t = t.clone()
    t[t == 0] = 0.0
    return t


@pytest.mark.parametrize("world,B,d,slack", [(2, 1, 9216, 1), (4, 2, 1024, 1), (8, 1, 12288, 1), (1, 3, 256, 1),
                                             (2, 1, 20480, 1), (8, 4, 12288, 4), (2, 3, 1024, 2)])
def test_allreduce_push_protocol_single_gpu(cuda, world, B, d, slack):
    """slack > 1: slots larger than an exchange needs, and the number of rows changes from step to step (the refill
    covers what the slot's last exchange wrote, not the whole slot)."""
    from dejavu_b200 import _lib

    lib = _lib.load()
    B_max = B
    slot_bytes = (B_max * d * 2 + 255) // 256 * 256 * slack
    comm, bufs_t = _make_comm(lib, cuda, world, slot_bytes)
    own = bufs_t[0].view(SLOTS, world, slot_bytes // 2)
    assert bool((own == SENT).all()), "comm_create fills the rank's own buffer with the sentinel"
    gen = torch.Generator().manual_seed(world * d)
    gamma, beta = (1 + rand(gen, (d,), 0.1)).to(cuda), rand(gen, (d,), 0.1).to(cuda)
    st = torch.cuda.current_stream().cuda_stream
    e = 0  # exchanges so far; steps of 3 exchanges each, so that the slot sequence wraps inside a step
    for step in range(4):
        B = B_max if (slack == 1 or step % 2 == 0) else 1
        for seq in range(3):
            parts = rand(gen, (world, B, d))
            parts[:, :, :3] = -0.0  # the sentinel value inside real data
            res = rand(gen, (B, d))
            slot = e % SLOTS
            for p in range(1, world):  # what rank p's kernel would have stored here (it sends -0.0 as +0.0)
                own[slot, p, :B * d] = _no_neg_zero(parts[p]).reshape(-1).view(torch.int16).to(cuda)
            y = torch.empty(B, d, dtype=torch.float16, device=cuda)
            r = torch.empty(B, d, dtype=torch.float16, device=cuda)
            part0, resd = parts[0].to(cuda), res.to(cuda)
            _lib.call("djv_allreduce_add_layernorm", comm, seq, _lib.EXCHANGE_REFILL, y.data_ptr(), r.data_ptr(),
                      part0.data_ptr(), resd.data_ptr(), gamma.data_ptr(), beta.data_ptr(), B, d, 1e-5, st)
            assert lib.djv_comm_status(comm) == 0
            acc = torch.zeros(B, d)
            for p in range(world):  # rank order, fp32, rounded once
                acc += parts[p].float()
            total = acc.half()
            y_ref, r_ref = O.add_layernorm(total, res, gamma.cpu(), beta.cpu(), 1e-5)
            assert torch.equal(r.cpu(), r_ref), "residual stream must be bit-exact"
            close(y, y_ref, atol=2e-3)
            # this rank's partial went to piece 0 of the same slot of every rank, with -0.0 sent as +0.0
            for p in range(world):
                got = bufs_t[p].view(SLOTS, world, slot_bytes // 2)[slot, 0, :B * d].cpu()
                assert torch.equal(got, _no_neg_zero(parts[0]).reshape(-1).view(torch.int16))
            # the slot used two exchanges ago is free again, whole extent; the one of the exchange before is not
            assert bool((own[(slot + 2) % SLOTS] == SENT).all())
            if e >= 1 and world > 1:
                assert not bool((own[(slot + 3) % SLOTS, :, :B * d] == SENT).all())
            # a second consumer of the same exchange (no refill, no LayerNorm) sees the same sum
            r2 = torch.empty(B, d, dtype=torch.float16, device=cuda)
            _lib.call("djv_allreduce_add_layernorm", comm, seq, 0, None, r2.data_ptr(), None, resd.data_ptr(), None,
                      None, B, d, 0.0, st)
            assert torch.equal(r2.cpu(), r_ref)
            e += 1
        _lib.call("djv_comm_end_step", comm, 3, st)
    lib.djv_comm_destroy(comm)


def test_allreduce_wait_runs_out_and_reports(cuda):
    """A peer that never sends: the bounded wait gives up, the status word says so, later calls return at once."""
    import time

    from dejavu_b200 import _lib

    lib = _lib.load()
    d = 1024
    comm, bufs_t = _make_comm(lib, cuda, 2, d * 2)
    gen = torch.Generator().manual_seed(5)
    x, g, b = rand(gen, (1, d)).to(cuda), torch.ones(d, dtype=torch.float16, device=cuda), torch.zeros(
        d, dtype=torch.float16, device=cuda)
    y, r = torch.empty_like(x), torch.empty_like(x)
    st = torch.cuda.current_stream().cuda_stream
    args = (comm, 0, _lib.EXCHANGE_REFILL, y.data_ptr(), r.data_ptr(), x.data_ptr(), None, g.data_ptr(), b.data_ptr(),
            1, d, 1e-5, st)
    t0 = time.time()
    _lib.call("djv_allreduce_add_layernorm", *args)
    assert lib.djv_comm_status(comm) == _lib.ERR_TIMEOUT
    assert 1.0 < time.time() - t0 < 20.0
    t0 = time.time()
    _lib.call("djv_allreduce_add_layernorm", *args)
    assert lib.djv_comm_status(comm) == _lib.ERR_TIMEOUT
    assert time.time() - t0 < 1.0, "a dead exchange must not wait again"
    # the context is still usable
    assert torch.equal((x + 1).cpu(), x.cpu() + 1)
    lib.djv_comm_destroy(comm)


@pytest.mark.parametrize("world", [2, 8])
def test_push_producers_feed_the_allreduce(cuda, world):
    """fc2 and out_proj store their result straight into every rank's receive buffer; the consumer that
    follows (partial = NULL) finds this rank's piece there. Peers' pieces are written by the test."""
    from dejavu_b200 import _lib, ops

    lib = _lib.load()
    d, M, Z, nheads, hd = 1024, 96, 512, 4, 128
    slot_bytes = d * 2
    comm, bufs_t = _make_comm(lib, cuda, world, slot_bytes)
    own = bufs_t[0].view(SLOTS, world, d)
    gen = torch.Generator().manual_seed(world)
    gamma, beta = (1 + rand(gen, (d,), 0.1)).to(cuda), rand(gen, (d,), 0.1).to(cuda)
    st = torch.cuda.current_stream().cuda_stream

    def finish(seq, mine, res):
        """pre-fill the peers' pieces, run the consumer with partial = NULL, compare with the oracle"""
        slot = seq % SLOTS
        for p in range(world):
            got = bufs_t[p].view(SLOTS, world, d)[slot, 0].cpu().view(torch.float16)
            assert torch.equal(got, mine.reshape(-1)), f"piece of rank 0 in rank {p}'s buffer"
        others = _no_neg_zero(rand(gen, (world - 1, 1, d)))
        for p in range(1, world):
            own[slot, p] = others[p - 1].reshape(-1).view(torch.int16).to(cuda)
        y = torch.empty(1, d, dtype=torch.float16, device=cuda)
        r = torch.empty(1, d, dtype=torch.float16, device=cuda)
        _lib.call("djv_allreduce_add_layernorm", comm, seq, _lib.EXCHANGE_REFILL, y.data_ptr(), r.data_ptr(), None,
                  res.to(cuda).data_ptr(), gamma.data_ptr(), beta.data_ptr(), 1, d, 1e-5, st)
        assert lib.djv_comm_status(comm) == 0
        acc = mine.float().reshape(1, d).clone()
        for p in range(world - 1):
            acc += others[p].float()
        y_ref, r_ref = O.add_layernorm(acc.half(), res, gamma.cpu(), beta.cpu(), 1e-5)
        assert torch.equal(r.cpu(), r_ref)
        close(y, y_ref, atol=2e-3)

    # exchange 0: fc2 (gather transposed GEMV)
    W2t, b2 = rand(gen, (Z, d), 0.05), rand(gen, (d,), 0.1)
    h = rand(gen, (1, M))
    idx = torch.randperm(Z, generator=gen)[:M].sort().values.int()
    want = _no_neg_zero(ops.gather_transposed_gemv(h.to(cuda), W2t.to(cuda), idx.to(cuda), b2.to(cuda)).cpu())
    need = lib.djv_gather_transposed_gemv_scratch_bytes(1, d, M)
    scratch = torch.zeros(need, dtype=torch.uint8, device=cuda)
    Wd, hd_, idxd, bd = W2t.to(cuda), h.to(cuda), idx.to(cuda), b2.to(cuda)
    _lib.call("djv_gather_transposed_gemv_push", comm, 0, Wd.data_ptr(), hd_.data_ptr(), idxd.data_ptr(),
              bd.data_ptr(), 1, d, M, d, 0, scratch.data_ptr(), need, st)
    finish(0, want, rand(gen, (1, d)))

    # exchange 1: out_proj over selected heads
    Wo, bo = rand(gen, (d, nheads, hd), 0.05), rand(gen, (d,), 0.1)
    ctx = rand(gen, (1, nheads, hd))
    heads = torch.tensor([1, 3], dtype=torch.int32)
    want = _no_neg_zero(ops.out_proj_sparse(ctx.to(cuda), Wo.to(cuda), heads.to(cuda), bo.to(cuda)).cpu())
    Wod, ctxd, headsd, bod = Wo.to(cuda), ctx.to(cuda), heads.to(cuda), bo.to(cuda)
    _lib.call("djv_out_proj_sparse_push", comm, 1, Wod.data_ptr(), ctxd.data_ptr(), headsd.data_ptr(), None,
              bod.data_ptr(), 1, d, nheads, hd, 2, st)
    finish(1, want, rand(gen, (1, d)))
    lib.djv_comm_destroy(comm)
