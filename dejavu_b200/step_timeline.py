"""Kernel timeline of the captured decode step (torch.profiler over graph replays): per-kernel totals and a slice of
the launch sequence with start offsets, durations and streams.

    # real tensor-parallel ranks (rank 0 prints)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m dejavu_b200.step_timeline opt-175b
    # ONE GPU running one rank's shard of an N-way split (no NVLink trip: the exchange kernels run with one rank),
    # for A/B runs of the kernel chain at tensor-parallel shard shapes
    python -m dejavu_b200.step_timeline opt-175b --shard-of 8 --layers 16 [--batch B] [--dense] [--no-exchange]

Durations are profiler durations: with programmatic dependent launch a kernel's interval starts when its
predecessor's blocks have all started and includes the wait for it, so the layer period is what to read, and
`DJV_PDL=0` gives the kernels' own execution times. `ms/step` is measured with CUDA events without the profiler.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import tempfile

import torch
import torch.distributed as dist
from torch.profiler import ProfilerActivity, profile

from . import gpt, modules
from .comm import TensorParallelComm
from .generation import update_graph_cache
from .gpt import GPTLMHeadModel, apply_sparsity_knobs, opt_config

SPARSITY = {"opt-6.7b": (2048, 12), "opt-66b": (4096, 24), "opt-175b": (4096, 32)}  # mlp-K, active heads


class _OneShardGroup:
    """Stands in for a process group of `world` ranks of which only rank 0 exists (collectives become no-ops)."""

    def __init__(self, world):
        self.world = world

    def size(self):
        return self.world

    def rank(self):
        return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=sorted(SPARSITY))
    ap.add_argument("--shard-of", type=int, default=0, help="single process: run one shard of this many ranks")
    ap.add_argument("--layers", type=int, default=0, help="keep only this many layers (0 = all)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--dense", action="store_true", help="every head and neuron (the dense comparator)")
    ap.add_argument("--no-exchange", action="store_true", help="plain all-reduce path instead of the exchange")
    ap.add_argument("--rows", type=int, default=32, help="launches of the timeline slice to print")
    a = ap.parse_args(argv)
    K, H = SPARSITY[a.workload]
    distributed = int(os.environ.get("WORLD_SIZE", "1")) > 1
    if distributed:
        world, rank, lr = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(lr)
        dev = torch.device("cuda", lr)
        dist.init_process_group("nccl", device_id=dev)
        pg = dist.group.WORLD
    else:
        world, rank, dev = max(1, a.shard_of), 0, torch.device("cuda:0")
        pg = _OneShardGroup(world)
        if world > 1:  # the other ranks do not exist: the collectives of the prompt pass and LM head do nothing
            modules.all_reduce = lambda x, group: x
            gpt.all_reduce = lambda x, group: x
            dist.all_gather = lambda parts, x, group=None: [p.copy_(x) for p in parts]
    cfg = apply_sparsity_knobs(opt_config(a.workload), K, H, H, world)
    if a.layers:
        cfg.n_layer = a.layers
    model = GPTLMHeadModel(cfg, process_group=pg, device=dev, dtype=torch.float16).eval().init_random(0)
    comm = None
    if world > 1 and not a.no_exchange:
        comm = TensorParallelComm(pg if distributed else None, dev, max_bytes=cfg.hidden_size * 2 * a.batch)
        model.transformer.enable_fused_allreduce(comm)
    if a.dense:
        model.transformer.set_dense(True)
    P, B = 128, a.batch
    with torch.inference_mode():
        cache = update_graph_cache(model, None, B, P, 512, greedy_feedback=True, vocab_size=cfg.vocab_size)
        ip = cache.inference_params
        ip.sequence_len_offset = 0
        prompt = torch.randint(0, cfg.vocab_size, (B, P), generator=torch.Generator().manual_seed(0)).to(dev)
        logits = model(prompt, inference_params=ip).logits[:, -1, :cfg.vocab_size]
        ip.sequence_len_offset = P
        cache.input_ids.copy_(logits.argmax(-1, keepdim=True))
        cache.position_ids.fill_(P)
        for _ in range(5):
            cache.graph.replay()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(30):
            cache.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 30
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                cache.graph.replay()
            torch.cuda.synchronize()
    if rank == 0:
        knobs = {k: v for k, v in os.environ.items() if k.startswith("DJV_")}
        print(f"{a.workload} tp{world} layers {cfg.n_layer} batch {B} dense {a.dense} {knobs}: {ms:.4f} ms/step, "
              f"{cache.launches_per_step} launches of this library per step")
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "trace.json")
            prof.export_chrome_trace(path)
            with open(path) as f:
                trace = json.load(f)
        evs = sorted((e for e in trace["traceEvents"] if e.get("cat") == "kernel"), key=lambda e: e["ts"])
        agg = collections.defaultdict(lambda: [0, 0.0])
        for e in evs:
            agg[e["name"][:60]][0] += 1
            agg[e["name"][:60]][1] += e["dur"]
        print("launches in 3 steps, total us, us per launch, kernel")
        for name, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:16]:
            print(f"{c:5d} {t:9.1f} {t / c:7.2f}  {name}")
        n = len(evs) // 3
        mid = evs[n + n // 2: n + n // 2 + a.rows]
        print("a slice of the second step: start us, + duration us, stream, kernel")
        for e in mid:
            print(f"{e['ts'] - mid[0]['ts']:8.1f} +{e['dur']:6.1f}  s{e['args'].get('stream')} {e['name'][:52]}")
    del cache
    if comm is not None:
        comm.close()
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
