"""The one-pass sparse MLP kernel (fc1 -> ReLU -> fc2 per gathered row, shared-memory ring fed by bulk
asynchronous copies) against the CPU oracle, alone and behind the tensor-parallel exchange + LayerNorm.
Tolerances: fp16 outputs atol 1e-3 / rtol 1e-2 (absolute part scaled with the output magnitude for long
sums); the residual stream and repeated runs are bit-exact."""
import ctypes as C

import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-3, 1e-2
SLOTS = 4


def close(a, b, atol=ATOL, rtol=RTOL):
    a, b = torch.as_tensor(a).float().cpu(), torch.as_tensor(b).float().cpu()
    assert a.shape == b.shape
    bad = ~torch.isclose(a, b, atol=atol, rtol=rtol)
    assert not bad.any(), f"{int(bad.sum())} mismatches, max abs diff {(a - b).abs().max().item()}"


def rand(gen, shape, std=1.0):
    return (torch.randn(shape, generator=gen) * std).half()


def _mlp_inputs(gen, Z, N, M, B, kind):
    W1, W2t = rand(gen, (Z, N), 0.02), rand(gen, (Z, N), 0.02)
    b1, b2 = rand(gen, (Z,), 0.1), rand(gen, (N,), 0.1)
    x = rand(gen, (B, N))
    if kind.startswith("dup"):
        idx = torch.randint(0, Z, (M,), generator=gen)
    else:
        idx = torch.randperm(Z, generator=gen)[:M]
        if kind.startswith("sorted"):
            idx = idx.sort().values
    return W1, W2t, b1, b2, x, idx.to(torch.int32 if kind.endswith("32") else torch.int64)


FUSED_CASES = [
    # Z, N, M, B, idx kind
    (3072, 768, 384, 1, "rand64"),      # BASELINE config 1 shape
    (3072, 768, 384, 3, "sorted32"),
    (6144, 12288, 512, 1, "rand64"),    # 175B TP8 shard, K/8 = 512: everything in flight at once
    (6144, 12288, 1024, 2, "rand32"),
    (6144, 12288, 130, 2, "rand32"),    # ragged: last cluster short, batches not full
    (6144, 12288, 1, 1, "rand32"),
    (6144, 12288, 3, 4, "dup32"),
    (6144, 12288, 6144, 1, "perm32"),   # dense through a permutation: many refills of the ring
    (4608, 9216, 512, 4, "dup32"),      # 66B TP8 shard, duplicate indices
    (36864, 9216, 4096, 1, "rand64"),   # 66B TP1
    (16384, 4096, 2048, 1, "rand64"),   # 6.7B
    (1024, 256, 256, 2, "rand32"),      # toy width of the model tests (32 columns per block)
    (512, 64, 100, 1, "rand32"),        # smallest width: one 16-byte chunk per block
]


@pytest.mark.parametrize("Z,N,M,B,kind", FUSED_CASES)
def test_mlp_sparse_fused_vs_oracle(cuda, Z, N, M, B, kind):
    from dejavu_b200 import _lib, ops

    lib = _lib.load()
    assert lib.djv_mlp_sparse_fused_supported(B, N, M)
    gen = torch.Generator().manual_seed(Z + 13 * M + B)
    W1, W2t, b1, b2, x, idx = _mlp_inputs(gen, Z, N, M, B, kind)
    dev = [t.to(cuda) for t in (W1, W2t, b1, b2, x, idx)]
    before = lib.djv_launch_count()
    got = ops.mlp_sparse(dev[4], dev[0], dev[1], dev[5], dev[2], dev[3], fused=True)
    assert lib.djv_launch_count() == before + 1, "the sparse MLP must be one launch"
    ref = O.mlp_sparse(x, W1, W2t, idx, b1, b2)
    tol = max(ATOL, 2e-3 * float(ref.float().abs().max()))
    close(got, ref, atol=tol)
    again = ops.mlp_sparse(dev[4], dev[0], dev[1], dev[5], dev[2], dev[3], fused=True)
    assert torch.equal(got, again), "summation order must be fixed"
    # without biases
    close(ops.mlp_sparse(dev[4], dev[0], dev[1], dev[5], None, None, fused=True), O.mlp_sparse(x, W1, W2t, idx, None, None), atol=tol)
    # and the two-kernel formulation of the same product
    h = ops.gather_gemv(dev[4], dev[0], dev[5], dev[2], "relu")
    two = ops.gather_transposed_gemv(h, dev[1], dev[5], dev[3])
    close(got, two, atol=tol)
    assert lib.djv_mlp_ring_timeouts() == 0


def test_mlp_sparse_fused_with_early_weight_stream(cuda):
    """With the caller's promise that the index list is complete, the kernel starts its copies before it waits
    for the kernel in front of it; results are the same."""
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(3)
    W1, W2t, b1, b2, x, idx = [t.to(cuda) for t in _mlp_inputs(gen, 6144, 12288, 700, 1, "rand32")]
    want = ops.mlp_sparse(x, W1, W2t, idx, b1, b2, fused=True)
    torch.cuda.synchronize()
    with ops.indices_ready(True):
        filler = x * 2  # some kernel in front
        got = ops.mlp_sparse(x, W1, W2t, idx, b1, b2, fused=True)
    assert torch.equal(got, want) and filler is not None


@pytest.mark.parametrize("Z,N,M,B", [(6144, 12288, 512, 1), (4608, 9216, 200, 3), (1024, 256, 64, 4)])
def test_ring_pipeline_runs_fc1_and_fc2_alone(cuda, monkeypatch, Z, N, M, B):
    """The same pipeline behind djv_gather_gemv / djv_gather_transposed_gemv (development knob)."""
    from dejavu_b200 import ops

    gen = torch.Generator().manual_seed(Z + M)
    W1, W2t, b1, b2, x, idx = _mlp_inputs(gen, Z, N, M, B, "rand32")
    monkeypatch.setenv("DJV_RING_GEMV", "100000")
    h = ops.gather_gemv(x.to(cuda), W1.to(cuda), idx.to(cuda), b1.to(cuda), "relu")
    close(h, O.gather_gemv(x, W1, idx, b1, "relu"))
    hid = ops.gather_gemv(x.to(cuda), W1.to(cuda), idx.to(cuda), None, "id")
    close(hid, O.gather_gemv(x, W1, idx, None, "id"))
    hh = torch.relu(rand(gen, (B, M)))
    y = ops.gather_transposed_gemv(hh.to(cuda), W2t.to(cuda), idx.to(cuda), b2.to(cuda))
    ref = O.gather_transposed_gemv(hh, W2t, idx, b2)
    close(y, ref, atol=max(ATOL, 2e-3 * float(ref.float().abs().max())))
    monkeypatch.setenv("DJV_RING_GEMV", "0")
    y_old = ops.gather_transposed_gemv(hh.to(cuda), W2t.to(cuda), idx.to(cuda), b2.to(cuda))
    close(y, y_old, atol=max(ATOL, 2e-3 * float(ref.float().abs().max())))


def _make_comm(lib, cuda, world, slot_bytes):
    from dejavu_b200 import _lib

    nbytes = lib.djv_comm_buffer_bytes(world, slot_bytes)
    bufs_t = [torch.zeros(nbytes // 2, dtype=torch.int16, device=cuda) for _ in range(world)]
    bufs = (C.c_void_p * world)(*[t.data_ptr() for t in bufs_t])
    comm = C.c_void_p()
    _lib.check("djv_comm_create", lib.djv_comm_create(C.byref(comm), 0, world, bufs, slot_bytes))
    return comm, bufs_t


def _no_neg_zero(t):
    t = t.clone()
    t[t == 0] = 0.0
    return t


@pytest.mark.parametrize("world,Z,N,M,B", [(1, 1024, 256, 128, 1), (2, 4608, 9216, 512, 1), (8, 6144, 12288, 512, 1),
                                           (4, 6144, 12288, 300, 2), (8, 6144, 12288, 2048, 1)])
def test_fused_mlp_behind_the_exchange_single_gpu(cuda, world, Z, N, M, B):
    """exchange -> residual add -> LayerNorm -> sparse MLP -> send, one launch. The peers' pieces of the incoming
    exchange are written by the test before the launch (no kernel waits for another kernel); this rank's piece
    comes from a real producer (out_proj with push). Checked: the new residual bit-exact, the sent result
    against the oracle in every rank's buffer, the recycled slot."""
    from dejavu_b200 import _lib, ops

    lib = _lib.load()
    d = N
    slot_bytes = (B * d * 2 + 255) // 256 * 256
    comm, bufs_t = _make_comm(lib, cuda, world, slot_bytes)
    own = bufs_t[0].view(SLOTS, world, slot_bytes // 2)
    gen = torch.Generator().manual_seed(world * 1000 + M)
    W1, W2t, b1, b2, _, idx = _mlp_inputs(gen, Z, N, M, B, "rand32")
    gamma, beta = 1 + rand(gen, (d,), 0.1), rand(gen, (d,), 0.1)
    st = torch.cuda.current_stream().cuda_stream
    need = lib.djv_mlp_sparse_fused_scratch_bytes(B, N, M)
    scratch = torch.zeros(need, dtype=torch.uint8, device=cuda)
    dW1, dW2t, db1, db2, didx, dg, dbt = [t.to(cuda) for t in (W1, W2t, b1, b2, idx, gamma, beta)]
    e = 0
    for step in range(3):
        parts = rand(gen, (world, B, d), 0.5)
        parts[:, :, :5] = -0.0
        res = rand(gen, (B, d))
        seq_in, seq_out = 0, 1
        slot_in, slot_out = e % SLOTS, (e + 1) % SLOTS
        # this rank's piece through the consumer-side send of the stand-alone kernel would consume the exchange;
        # write it like a producer would (piece 0 of every rank's buffer), peers' pieces into the own buffer
        for p in range(world):
            bufs_t[p].view(SLOTS, world, slot_bytes // 2)[slot_in, 0, :B * d] = \
                _no_neg_zero(parts[0]).reshape(-1).view(torch.int16).to(cuda)
        for p in range(1, world):
            own[slot_in, p, :B * d] = _no_neg_zero(parts[p]).reshape(-1).view(torch.int16).to(cuda)
        r = torch.empty(B, d, dtype=torch.float16, device=cuda)
        resd = res.to(cuda)
        _lib.call("djv_mlp_sparse_fused_exchange", comm, seq_in, _lib.EXCHANGE_REFILL, seq_out, None, r.data_ptr(),
                  resd.data_ptr(), dg.data_ptr(), dbt.data_ptr(), 1e-5, dW1.data_ptr(), dW2t.data_ptr(),
                  didx.data_ptr(), db1.data_ptr(), db2.data_ptr(), B, N, M, Z, N, N, 0, scratch.data_ptr(), need, st)
        assert lib.djv_comm_status(comm) == 0
        acc = torch.zeros(B, d)
        for p in range(world):
            acc += parts[p].float()
        x_ref, r_ref = O.add_layernorm(acc.half(), res, gamma, beta, 1e-5)
        assert torch.equal(r.cpu(), r_ref), "residual stream must be bit-exact"
        y_ref = O.mlp_sparse(x_ref, W1, W2t, idx, b1, b2)
        tol = max(2e-3, 4e-3 * float(y_ref.float().abs().max()))  # x itself carries one fp16 rounding of the LayerNorm
        sent = [bufs_t[p].view(SLOTS, world, slot_bytes // 2)[slot_out, 0, :B * d].cpu().view(torch.float16)
                for p in range(world)]
        close(sent[0].view(B, d), y_ref, atol=tol)
        for p in range(1, world):
            assert torch.equal(sent[p], sent[0]), "every rank receives the same piece"
        assert bool((own[(slot_in + 2) % SLOTS] == SENT_I16).all()), "the slot used two exchanges ago is recycled"
        # stored instead of sent: same bits
        y = torch.empty(B, d, dtype=torch.float16, device=cuda)
        for p in range(1, world):  # (the recycling above may have hit nothing these pieces need)
            own[slot_in, p, :B * d] = _no_neg_zero(parts[p]).reshape(-1).view(torch.int16).to(cuda)
        _lib.call("djv_mlp_sparse_fused_exchange", comm, seq_in, 0, -1, y.data_ptr(), None, resd.data_ptr(),
                  dg.data_ptr(), dbt.data_ptr(), 1e-5, dW1.data_ptr(), dW2t.data_ptr(), didx.data_ptr(),
                  db1.data_ptr(), db2.data_ptr(), B, N, M, Z, N, N, 0, scratch.data_ptr(), need, st)
        assert torch.equal(_no_neg_zero(y.cpu()).view(-1), sent[0])
        _lib.call("djv_comm_end_step", comm, 2, st)
        # the consumer of exchange seq_out would recycle slot_in + 3; do it by hand so that slots stay clean
        own[slot_out] = SENT_I16
        for p in range(1, world):
            bufs_t[p].view(SLOTS, world, slot_bytes // 2)[slot_out] = SENT_I16
        e += 2
    assert lib.djv_mlp_ring_timeouts() == 0
    lib.djv_comm_destroy(comm)


SENT_I16 = -32768


def test_fused_mlp_wait_on_a_missing_peer_runs_out(cuda):
    """A peer that never sends: the prologue's bounded wait gives up, nothing is sent, the status word says so."""
    from dejavu_b200 import _lib

    lib = _lib.load()
    Z, N, M, B = 1024, 1024, 64, 1
    comm, bufs_t = _make_comm(lib, cuda, 2, N * 2)
    gen = torch.Generator().manual_seed(9)
    W1, W2t, b1, b2, _, idx = [t.to(cuda) for t in _mlp_inputs(gen, Z, N, M, B, "rand32")]
    g, bt = torch.ones(N, dtype=torch.float16, device=cuda), torch.zeros(N, dtype=torch.float16, device=cuda)
    need = lib.djv_mlp_sparse_fused_scratch_bytes(B, N, M)
    scratch = torch.zeros(need, dtype=torch.uint8, device=cuda)
    r = torch.zeros(B, N, dtype=torch.float16, device=cuda)
    _lib.call("djv_mlp_sparse_fused_exchange", comm, 0, _lib.EXCHANGE_REFILL, 1, None, r.data_ptr(), None,
              g.data_ptr(), bt.data_ptr(), 1e-5, W1.data_ptr(), W2t.data_ptr(), idx.data_ptr(), b1.data_ptr(),
              b2.data_ptr(), B, N, M, Z, N, N, 0, scratch.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
    assert lib.djv_comm_status(comm) == _lib.ERR_TIMEOUT
    own = bufs_t[0].view(SLOTS, 2, N)
    assert bool((own[1, 0] == SENT_I16).all()), "nothing was sent"
    assert bool((scratch[:4096] == 0).all()), "the arrival counters are left at zero"
    assert torch.equal((r + 1).cpu(), r.cpu() + 1)  # the context is still usable
    lib.djv_comm_destroy(comm)
