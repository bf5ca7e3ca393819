"""Small single-kernel cases for profiler captures and the phase trace of the one-pass MLP kernel.

    python -m dejavu_b200.profile_cases <case>
        case: qkv | out_proj | attn | topk | exchange | ring | fc1 | fc2 | fc1_b16 | fc2_b16 | ring_trace

Every case launches ONE kind of kernel a dozen times at the per-rank shapes of an OPT-175B layer under 8-way
tensor parallelism (d 12288, 12 local heads of which 4 are active, 512 of 6144 ffn rows), rotating several weight
buffers so that a launch never finds its rows in L2, and holds well under 3 GB on the device: small enough for a
multi-pass `ncu` capture of one kernel (`-k regex:<kernel> -s <skip> -c 3`) to end by itself in seconds.
`ring_trace` needs a library built with the phase stamps (DJV_NVCC_FLAGS=-DDJV_RING_TRACE python -m
dejavu_b200.build --force) and prints, per phase of the one-pass kernel, when the blocks reached it.
"""

import ctypes as C
import sys

import numpy as np
import torch

from . import _lib, ops


def main(case: str) -> None:
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    def rnd(*shape, std=0.02): return (torch.randn(*shape, device=dev, generator=g) * std).half()
    d, n, hd, a = 12288, 12, 128, 4   # OPT-175B TP8 shard
    NB, REP = 6, 2
    if case == "qkv":
        Ws = [rnd(3, n, hd, d) for _ in range(NB)]; b = rnd(3, n, hd); x = rnd(1, d, std=1.0)
        heads = torch.tensor([1, 4, 7, 10], dtype=torch.int32, device=dev); bidx = torch.zeros(a, 1, dtype=torch.int32, device=dev)
        for _ in range(REP):
            for W in Ws: ops.qkv_proj_sparse(x, W, heads, bidx, b)
    elif case == "out_proj":
        Ws = [rnd(d, n, hd) for _ in range(NB)]; b = rnd(d); ctx = rnd(1, n, hd, std=1.0)
        heads = torch.tensor([1, 4, 7, 10], dtype=torch.int32, device=dev)
        for _ in range(REP):
            for W in Ws: ops.out_proj_sparse(ctx, W, heads, b)
    elif case == "attn":
        S = 2048
        caches = [(rnd(1, n, hd // 8, S, 8, std=1.0), rnd(1, n, S, hd, std=1.0)) for _ in range(10)]
        q = rnd(1, n, hd, std=1.0); heads = torch.tensor([1, 4, 7, 10], dtype=torch.int32, device=dev)
        for _ in range(REP):
            for k, v in caches: ops.decode_attention(q, k, v, heads, 2000, hd ** -0.5)
    elif case == "topk":
        for nn, kk in ((6144, 512), (36864, 4096)):
            sc = rnd(nn, std=1.0)
            for _ in range(3): ops.topk_indices(sc, kk, torch.int32)
    elif case == "exchange":
        from .comm import TensorParallelComm
        comm = TensorParallelComm(None, dev, max_bytes=d * 2)
        x = rnd(1, d, std=1.0); r = rnd(1, d, std=1.0); gm = torch.ones(d, device=dev).half(); bt = torch.zeros(d, device=dev).half()
        for _ in range(6): comm.allreduce_add_layernorm(x, r, gm, bt, 1e-5)
        comm.end_step()
    elif case in ("ring", "fc1", "fc2", "ring_trace"):
        Z, K = 6144, 512
        W1 = [rnd(Z, d) for _ in range(NB)]; W2 = [rnd(Z, d) for _ in range(NB)]
        b1 = rnd(Z); b2 = rnd(d); x = rnd(1, d, std=1.0); h = torch.relu(rnd(1, K, std=1.0))
        idxs = [torch.randperm(Z, device=dev, generator=g)[:K].int() for _ in range(NB)]
        for _ in range(REP):
            for i in range(NB):
                if case in ("ring", "ring_trace"): ops.mlp_sparse(x, W1[i], W2[i], idxs[i], b1, b2, fused=True)
                elif case == "fc1": ops.gather_gemv(x, W1[i], idxs[i], b1, "relu")
                else: ops.gather_transposed_gemv(h, W2[i], idxs[i], b2)
    elif case in ("fc1_b16", "fc2_b16"):  # the tensor-core kernels: 16 activation rows, 4096 of 6144 rows
        Z, K, Bt = 6144, 4096, 16
        Ws = [rnd(Z, d) for _ in range(4)]; b1 = rnd(Z); b2 = rnd(d)
        x = rnd(Bt, d, std=1.0); h = torch.relu(rnd(Bt, K, std=1.0))
        idxs = [torch.randperm(Z, device=dev, generator=g)[:K].int() for _ in range(4)]
        for _ in range(REP):
            for i in range(4):
                if case == "fc1_b16": ops.gather_gemv(x, Ws[i], idxs[i], b1, "relu")
                else: ops.gather_transposed_gemv(h, Ws[i], idxs[i], b2)
    torch.cuda.synchronize()
    if case == "ring_trace":
        lib = _lib.load()
        if not hasattr(lib, "djv_mlp_ring_trace"):
            sys.exit("this library was built without -DDJV_RING_TRACE")
        lib.djv_mlp_ring_trace.restype, lib.djv_mlp_ring_trace.argtypes = C.c_int, [C.c_void_p]
        buf = np.zeros((512, 12), dtype=np.uint64)
        assert lib.djv_mlp_ring_trace(buf.ctypes.data) == 0
        t = buf[:120].astype(np.float64)  # 15 clusters of 8 blocks
        names = ["start", "first copies issued", "wait on predecessor done", "input rows ready", "first product done",
                 "cluster barrier", "activations ready", "second product done", "partial sums written", "ticket taken",
                 "result stored (last block of a segment)"]
        print("phase: microseconds after the first block's start, min / median / max over blocks (last launch)")
        for i, nm in enumerate(names):
            col = t[:, i][t[:, i] > t[:, 0].min()] if i else t[:, 0]
            if len(col):
                print(f"  {nm:42s} {(col.min() - t[:, 0].min()) / 1e3:6.2f} {(np.median(col) - t[:, 0].min()) / 1e3:6.2f} "
                      f"{(col.max() - t[:, 0].min()) / 1e3:6.2f}")
    print("ok", case)


if __name__ == "__main__":
    main(sys.argv[1])
