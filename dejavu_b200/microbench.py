"""Gather-GEMV kernel microbench at the per-rank shard of an OPT-175B layer (d=12288, ffn shard 6144).

    python -m dejavu_b200.microbench [--batch 1 2 4 8 16 32] [--K 128 ... | --K-step 128] [--buffers N]
                                     [--d 12288] [--ffn 6144] [--fused] [--out file.jsonl]

For every (batch, K, sorted/unsorted index list) it reports the achieved GB/s of fc1 (gather GEMV) and fc2
(gather transposed GEMV) and the fraction of the measured HBM peak. Algorithmic bytes per launch:
    fc1: K*d*2 + K*2 (bias) + K*4 (idx) + B*d*2 (x) + B*K*2 (h)     fc2: K*d*2 + B*K*2 (h) + d*2 (bias) + B*d*2 (y)
Timing: CUDA events around replays of a CUDA graph holding one launch per weight buffer; distinct (W, idx) pairs
are rotated, as many per K as it takes for the rows touched between two uses of a buffer to exceed twice the
126 MB L2 ((buffers - 1) * K * d * 2 bytes >= 252 MB; `--buffers` caps the count, default: what K-step needs).
`--fused` adds the one-pass fc1 -> ReLU -> fc2 kernel (batch <= 4).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import _lib

ROOT = Path(__file__).resolve().parents[1]


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def time_launches(fns, iters):
    """Average microseconds per launch of `fns` replayed `iters` times as one CUDA graph."""
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fns:
            f(s.cuda_stream)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for f in fns:
                f(torch.cuda.current_stream().cuda_stream)
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(iters):
            g.replay()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * len(fns))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--d", type=int, default=12288)
    ap.add_argument("--ffn", type=int, default=6144)
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 2, 4, 8, 16, 32])
    ap.add_argument("--K", type=int, nargs="+", default=None)
    ap.add_argument("--K-step", type=int, default=512, help="sweep K from K-step to ffn in this step (config: 128)")
    ap.add_argument("--buffers", type=int, default=0, help="cap on the weight buffers rotated (0 = as many as needed)")
    ap.add_argument("--fused", action="store_true", help="also time the one-pass sparse MLP kernel (batch <= 4)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    lib = _lib.load()
    dev = torch.device("cuda:0")
    peak, kind = hbm_peak()
    gen = torch.Generator(device=dev).manual_seed(0)
    F_, d = a.ffn, a.d
    Ks = a.K or list(range(a.K_step, F_ + 1, a.K_step))
    L2_BYTES = 126e6

    def buffers_for(K):
        n = int(2 * L2_BYTES / (K * d * 2)) + 2
        n = max(n, 4)
        return min(n, a.buffers) if a.buffers else n

    free, _total = torch.cuda.mem_get_info()
    NB_MAX = min(buffers_for(min(Ks)), int(free * 0.6 / (F_ * d * 2)))
    Ws = [(torch.randn(F_, d, device=dev, generator=gen) * 0.02).half() for _ in range(NB_MAX)]
    W2s = Ws[::-1]  # the one-pass kernel reads two matrices per launch: pair each buffer with a different one
    b1 = (torch.randn(F_, device=dev, generator=gen) * 0.02).half()
    b2 = (torch.randn(d, device=dev, generator=gen) * 0.02).half()
    sink = open(a.out, "w") if a.out else None
    for B in a.batch:
        x = torch.randn(B, d, device=dev, generator=gen).half()
        for K in Ks:
            NB = min(NB_MAX, buffers_for(K))
            for sorted_ in (False, True):
                idxs = []
                for _ in range(NB):
                    idx = torch.randperm(F_, device=dev, generator=gen)[:K].int()
                    idxs.append(idx.sort().values.int() if sorted_ else idx)
                h = torch.empty(B, K, device=dev, dtype=torch.float16)
                y = torch.empty(B, d, device=dev, dtype=torch.float16)
                need = lib.djv_gather_transposed_gemv_scratch_bytes(B, d, K)
                scratch = torch.zeros(need, dtype=torch.uint8, device=dev)

                def fc1(i):
                    return lambda st: _lib.call("djv_gather_gemv", h.data_ptr(), Ws[i].data_ptr(), x.data_ptr(),
                                                idxs[i].data_ptr(), b1.data_ptr(), B, d, K, d, 0, 1, st)

                def fc2(i):
                    return lambda st: _lib.call("djv_gather_transposed_gemv", y.data_ptr(), Ws[i].data_ptr(),
                                                h.data_ptr(), idxs[i].data_ptr(), b2.data_ptr(), B, d, K, d, 0,
                                                scratch.data_ptr(), need, st)

                t1 = time_launches([fc1(i) for i in range(NB)], a.iters)
                t2 = time_launches([fc2(i) for i in range(NB)], a.iters)
                bytes1 = K * d * 2 + K * 2 + K * 4 + B * d * 2 + B * K * 2
                bytes2 = K * d * 2 + B * K * 2 + d * 2 + B * d * 2
                rec = {"batch": B, "K": K, "sorted": sorted_, "d": d, "ffn": F_, "buffers": NB,
                       "fc1_us": round(t1, 2), "fc1_gbs": round(bytes1 / t1 / 1e3, 1),
                       "fc1_frac": round(bytes1 / t1 / 1e3 / peak, 3),
                       "fc2_us": round(t2, 2), "fc2_gbs": round(bytes2 / t2 / 1e3, 1),
                       "fc2_frac": round(bytes2 / t2 / 1e3 / peak, 3), "peak_gbs": peak, "peak_kind": kind}
                if a.fused and B <= 4 and lib.djv_mlp_sparse_fused_supported(B, d, K):
                    need3 = lib.djv_mlp_sparse_fused_scratch_bytes(B, d, K)
                    scratch3 = torch.zeros(need3, dtype=torch.uint8, device=dev)

                    def fused(i):
                        return lambda st: _lib.call("djv_mlp_sparse_fused", y.data_ptr(), Ws[i].data_ptr(),
                                                    W2s[i].data_ptr(), x.data_ptr(), idxs[i].data_ptr(), b1.data_ptr(),
                                                    b2.data_ptr(), B, d, K, F_, d, d, 0, scratch3.data_ptr(), need3, st)

                    t3 = time_launches([fused(i) for i in range(NB)], a.iters)
                    bytes3 = 2 * K * d * 2 + K * 2 + K * 4 + d * 2 + 2 * B * d * 2
                    rec.update({"fused_us": round(t3, 2), "fused_frac": round(bytes3 / t3 / 1e3 / peak, 3)})
                line = json.dumps(rec)
                print(line, flush=True)
                if sink:
                    sink.write(line + "\n")
    if sink:
        sink.close()


if __name__ == "__main__":
    main()
