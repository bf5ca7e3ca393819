"""The allocation-free entry point, djv_gather_transposed_gemv_static.

Some hosts of this library cannot give it a scratch buffer: they handed every byte of device memory to
their own pool at start-up, or they call from a context in which allocating is not allowed, or their
binding simply has no workspace argument. For them the library carries a fixed built-in scratch array.
This test calls that entry point through the C ABI, twice in a row on different inputs, and requires the
same result as the regular entry point (which gets a caller-allocated scratch buffer). It lives in a file
of its own that pytest collects last, and it must pass both alone in a fresh process and after every
other test has used the library.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 4096 + (256 << 10)


def _inputs(cuda, seed, Z, N, M, B):
    gen = torch.Generator().manual_seed(seed)
    W = (torch.randn(Z, N, generator=gen) * 0.05).half().to(cuda)
    h = torch.relu(torch.randn(B, M, generator=gen)).half().to(cuda)
    bias = (torch.randn(N, generator=gen) * 0.1).half().to(cuda)
    idx = torch.randperm(Z, generator=gen)[:M].int().to(cuda)
    return W, h, bias, idx


def _regular(lib_mod, W, h, bias, idx, B, N, M):
    lib = lib_mod.load()
    y = torch.empty(B, N, dtype=torch.float16, device=W.device)
    need = lib.djv_gather_transposed_gemv_scratch_bytes(B, N, M)
    scratch = torch.zeros(need, dtype=torch.uint8, device=W.device)
    lib_mod.call("djv_gather_transposed_gemv", y.data_ptr(), W.data_ptr(), h.data_ptr(), idx.data_ptr(),
                 bias.data_ptr(), B, N, M, W.stride(0), 0, scratch.data_ptr(), need,
                 torch.cuda.current_stream().cuda_stream)
    return y


def _static(lib_mod, W, h, bias, idx, B, N, M):
    y = torch.empty(B, N, dtype=torch.float16, device=W.device)
    lib_mod.call("djv_gather_transposed_gemv_static", y.data_ptr(), W.data_ptr(), h.data_ptr(), idx.data_ptr(),
                 bias.data_ptr(), B, N, M, W.stride(0), 0, torch.cuda.current_stream().cuda_stream)
    return y


@pytest.mark.parametrize("Z,N,M,B", [(6144, 12288, 512, 1), (2048, 4096, 700, 2), (2048, 4096, 700, 3),
                                     (8192, 2048, 4096, 4)])
def test_static_scratch_entry_point_matches_regular_one_twice(cuda, Z, N, M, B):
    """Up to 2 rows of x both entry points run the same kernel with the same plan: identical bits. With 3 and 4 rows
    the regular entry point uses the tensor-core kernel (another summation order): equal within the tolerance."""
    from dejavu_b200 import _lib

    for call_no, seed in enumerate((21, 22)):  # two calls in a row: the array keeps the first call's leftovers
        W, h, bias, idx = _inputs(cuda, seed, Z, N, M, B)
        want = _regular(_lib, W, h, bias, idx, B, N, M)
        got = _static(_lib, W, h, bias, idx, B, N, M)
        torch.cuda.synchronize()
        # same kernel, same plan, same summation order: the tolerance of the other tests is met exactly
        assert torch.allclose(got.float(), want.float(), atol=1e-3, rtol=1e-2), f"call {call_no}"
        if B <= 2:
            assert torch.equal(got, want), f"call {call_no}: expected identical bits"


@pytest.mark.parametrize("Z,M,B,widths", [(8192, 4096, 1, (1024, 2048)), (8192, 4096, 2, (2048, 1024))])
def test_static_scratch_array_is_really_used_and_reused(cuda, Z, M, B, widths):
    """Shapes whose plan splits the index list over several clusters per column tile: the kernel then keeps
    per-cluster partial sums and arrival counters in the built-in array. Two calls in a row with DIFFERENT
    output widths, so the second one finds the first one's partial sums and counters in the array."""
    from dejavu_b200 import _lib

    lib = _lib.load()
    for call_no, N in enumerate(widths):
        need = lib.djv_gather_transposed_gemv_scratch_bytes(B, N, M)
        if need <= 4096 + B * N * 4:
            pytest.skip("the plan keeps one cluster per column tile on this device: no partial sums in scratch")
        assert need <= STATIC_SCRATCH_BYTES
        W, h, bias, idx = _inputs(cuda, 31 + call_no, Z, N, M, B)
        want = _regular(_lib, W, h, bias, idx, B, N, M)
        got = _static(_lib, W, h, bias, idx, B, N, M)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call_no} (N={N}): expected identical bits"


def test_static_scratch_entry_point_refuses_oversized_requests(cuda):
    from dejavu_b200 import _lib

    lib = _lib.load()
    Z, N, M, B = 64, 32768, 4096, 4  # several row chunks of a very wide output: more partials than the array holds
    need = lib.djv_gather_transposed_gemv_scratch_bytes(B, N, M)
    W = torch.zeros(Z, N, dtype=torch.float16, device=cuda)
    h = torch.zeros(B, M, dtype=torch.float16, device=cuda)
    idx = torch.zeros(M, dtype=torch.int32, device=cuda)
    y = torch.empty(B, N, dtype=torch.float16, device=cuda)
    if need <= STATIC_SCRATCH_BYTES:
        pytest.skip("this shape fits the built-in array on this device")
    before = lib.djv_launch_count()
    with pytest.raises(_lib.DejavuKernelError) as e:
        _lib.call("djv_gather_transposed_gemv_static", y.data_ptr(), W.data_ptr(), h.data_ptr(), idx.data_ptr(), None,
                  B, N, M, N, 0, torch.cuda.current_stream().cuda_stream)
    assert e.value.status == _lib.ERR_SCRATCH and "built-in array" in str(e.value)
    assert lib.djv_launch_count() == before
