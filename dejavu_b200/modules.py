"""Host-side mirror of the reference's sparse decode modules, same class names, constructor arguments,
forward signatures and state-dict keys, running the sm_100a kernels for the decode step.

  ParallelSP, ColumnParallelLinear, RowParallelLinear, RowParallelLinearNoReduce, ParallelFusedMLPDejavu
      <- Dejavu/src/ops/fused_dense_sparse_dejavu.py:33-76, 241-317, 783-818, 821-951
  ParallelMHASparseAttMlp, ParallelMHADejavu
      <- Dejavu/src/models/modules/mha_dejavu.py:1152-1511, 910-1075
  BlockMlpAttSparse, BlockDejavu
      <- Dejavu/src/models/modules/block_dejavu.py:464-663, 264-461

Differences that are deliberate (none changes results for heads / neurons that are read):
  * the lazy-K/V bookkeeping (ParallelTracker, x_cache, counter, cache_offset) lives in device memory, so
    a captured CUDA graph replays correctly;
  * decode attention runs only for the heads in use (the reference runs all local heads and discards
    the others);
  * fc2's weight is stored once, transposed (ffn_local, d); `fc2.weight` is a (d, ffn_local) view of it,
    so nothing is duplicated or built lazily inside forward;
  * the predictor look-ahead work runs on side streams like the reference's sp_stream, but consumers
    wait on per-result events where the result is used, not at the end of the producing module.
The prompt phase (seqlen > 1) is dense and uses torch (cuBLAS / SDPA), as in the reference.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, ops
from ._lib import call

KV_WINDOW = _lib.KV_WINDOW

# Look-ahead predictor work runs on two side streams per device ("att": head predictor, "mlp": MLP
# predictor + its top-K), forked from and joined to the main stream with events; inside a CUDA-graph
# capture these become parallel branches of the graph. DJV_SIDE_STREAMS=0 keeps everything on one stream.
SIDE_STREAMS_ENABLED = os.environ.get("DJV_SIDE_STREAMS", "1") != "0"
# the kernel that selects the next layer's heads also opens that layer's decode step (development knob)
FUSE_STEP_OPEN = os.environ.get("DJV_FUSE_STEP_OPEN", "1") != "0"
# fc2 and out_proj send their result into the peers' receive buffers themselves (development knob)
PUSH_PARTIALS = os.environ.get("DJV_PUSH_PARTIALS", "1") != "0"
# kernels whose index list is known to be complete prefetch weights before their PDL wait (development knob)
EARLY_PREFETCH = os.environ.get("DJV_EARLY_PREFETCH", "1") != "0"
# with a comm: exchange + residual + LayerNorm + fc1 + ReLU + fc2 (+ send) of a block in one kernel. "0" (default):
# off, the separate kernels measured faster at every tensor-parallel degree (OPT-66B TP8: 3.06 against 3.15
# ms/token; 16 layers of an OPT-175B TP8 shard on one GPU: 0.94 against 1.04 ms); "1": on wherever the shape allows; "auto": on for a real
# tensor-parallel group when the shard's index list is short enough to be in flight at once
FUSED_MLP = os.environ.get("DJV_FUSED_MLP", "0")
# where the main stream joins the side stream that selects this layer's MLP rows: "attend" = before the attention
# kernel (the fused MLP kernel then follows out_proj with a single programmatic edge and streams its weights while
# out_proj runs), "mlp" = right before the MLP (development knob)
MLP_IDX_JOIN = os.environ.get("DJV_MLP_IDX_JOIN", "attend")
# L2 warm-up of the rows an index list names, as soon as the list exists: "0" off (default: measured slower, the
# extra traffic lengthens the memory latency every kernel of the main chain is bound by), "1" on, "auto" = on when
# the weights a rank gathers per layer stay below DJV_L2_PREFETCH_MB (development knob)
L2_PREFETCH = os.environ.get("DJV_L2_PREFETCH", "0")
L2_PREFETCH_MB = float(os.environ.get("DJV_L2_PREFETCH_MB", "100"))
# batch > 1: the predictors run once, on the sum of the sequences' inputs (they are linear), instead of once per
# sequence; "0": per sequence, logits added afterwards (development knob)
SP_SUM_INPUTS = os.environ.get("DJV_SP_SUM_INPUTS", "1") != "0"
# batch > 1: keep programmatic dependent launch for the decode step's kernels ("1"); default off, measured slower
# (OPT-6.7B, 16 sequences: 6.3 ms per step with, 4.7 without; 4 sequences: 2.95 / 2.64) (development knob)
BATCH_PROGRAMMATIC_LAUNCH = os.environ.get("DJV_BATCH_PDL", "0") != "0"
# batch > 1: the attention of all sequences runs through the batch entry points (one state, one launch per kernel
# for the whole batch); "0": sequence by sequence through the batch-1 kernels (development knob)
BATCHED_ATTENTION = os.environ.get("DJV_BATCHED_ATTENTION", "1") != "0"
# sequence by sequence, batch >= 4: the attention chains of sequences 1.. run on up to this many extra streams (branches of
# the captured graph), at least two sequences per stream, once sequence 0 has brought the selected heads' weights
# into L2; 0 = all on the main stream. Measured on OPT-6.7B, one GPU, ms per step without / with: batch 8 7.95 /
# 5.65, batch 16 16.9 / 8.4; one sequence per stream (batch 4 on 3 streams) was slower than none (4.9 / 4.7).
BATCH_STREAMS = int(os.environ.get("DJV_BATCH_STREAMS", "8"))
_SIDE_STREAMS: dict = {}
_SIDE_DIRTY: dict = {}  # device index -> names of side streams forked since the last join


def side_streams(device) -> dict:
    key = torch.device(device).index
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = {"att": torch.cuda.Stream(device=device), "mlp": torch.cuda.Stream(device=device)}
    return _SIDE_STREAMS[key]


def batch_streams(device, n) -> list:
    """The first n of the streams that carry the attention chains of sequences 1.. of a batch."""
    streams = side_streams(device)
    for j in range(n):
        if f"batch{j}" not in streams:
            streams[f"batch{j}"] = torch.cuda.Stream(device=device)
    return [streams[f"batch{j}"] for j in range(n)]


class _side:
    """`with _side(ref, name, after=t) as done: r = work(); done(r)` runs work() on side stream `name` after
    everything queued on the current stream so far and after `t` is ready; done(r) attaches the completion
    event to r, which consumers honour with _wait_ready(r)."""

    def __init__(self, ref, name, after=None):
        self.active = SIDE_STREAMS_ENABLED and ref.is_cuda
        self.ref, self.name, self.after, self.ctx = ref, name, after, None

    def __enter__(self):
        if not self.active:
            return lambda t: None
        self.main = torch.cuda.current_stream()
        self.side = side_streams(self.ref.device)[self.name]
        fork = torch.cuda.Event()
        fork.record(self.main)
        self.side.wait_event(fork)
        _SIDE_DIRTY.setdefault(self.ref.device.index, set()).add(self.name)
        if self.after is not None:
            ev = getattr(self.after, "_ready_event", None)
            if ev is not None:
                self.side.wait_event(ev)
            self.after.record_stream(self.side)
        self.ctx = torch.cuda.stream(self.side)
        self.ctx.__enter__()
        return self._done

    def _done(self, t):
        ev = torch.cuda.Event()
        ev.record(self.side)
        t._ready_event = ev
        t.record_stream(self.main)

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
        return False


def _wait_ready(t):
    """Make the current stream wait for a tensor produced on a side stream (no-op otherwise)."""
    ev = None if t is None else getattr(t, "_ready_event", None)
    if ev is not None:
        stream = torch.cuda.current_stream()
        # once per stream: a second wait would add a second edge to the next kernel of a captured graph, and a
        # kernel with two incoming edges is not launched programmatically any more
        if getattr(t, "_waited_on", None) != stream.cuda_stream:
            stream.wait_event(ev)
            t._waited_on = stream.cuda_stream


def join_side_streams(device):
    """All side-stream work rejoins the current stream (needed before a graph capture ends)."""
    key = torch.device(device).index
    dirty = _SIDE_DIRTY.pop(key, None)
    if dirty:
        main = torch.cuda.current_stream()
        for name in dirty:
            main.wait_stream(_SIDE_STREAMS[key][name])


def _world(pg) -> int:
    return 1 if pg is None else pg.size()


def _rank(pg) -> int:
    return 0 if pg is None else pg.rank()


def all_reduce(x: torch.Tensor, process_group) -> torch.Tensor:
    """SUM over the tensor-parallel group (flash_attn.utils.distributed.all_reduce at
    Dejavu/src/models/modules/mha_dejavu.py:1498, fused_dense_sparse_dejavu.py:940)."""
    if _world(process_group) == 1:
        return x
    x = x.contiguous()
    torch.distributed.all_reduce(x, group=process_group)
    return x


class ColumnParallelLinear(nn.Module):
    """Linear whose OUTPUT features are split over the group: weight (out/world, in)
    (fused_dense_sparse_dejavu.py:241-277)."""

    def __init__(self, in_features, out_features, process_group, bias=True, sequence_parallel=False,
                 device=None, dtype=None):
        super().__init__()
        world = _world(process_group)
        if out_features % world != 0:
            raise ValueError(f"out_features ({out_features}) must be divisible by world_size ({world})")
        self.process_group = process_group
        self.in_features, self.out_features = in_features, out_features // world
        self.weight = nn.Parameter(torch.empty(self.out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.empty(self.out_features, device=device, dtype=dtype)) if bias else None

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


class RowParallelLinearNoReduce(nn.Module):
    """Linear whose INPUT features are split over the group: weight (out, in/world); bias on rank 0 only;
    the caller all-reduces (fused_dense_sparse_dejavu.py:783-818)."""

    def __init__(self, in_features, out_features, process_group, bias=True, sequence_parallel=False,
                 device=None, dtype=None):
        super().__init__()
        world = _world(process_group)
        if in_features % world != 0:
            raise ValueError(f"in_features ({in_features}) must be divisible by world_size ({world})")
        self.process_group = process_group
        self.in_features, self.out_features = in_features // world, out_features
        self.weight = nn.Parameter(torch.empty(out_features, self.in_features, device=device, dtype=dtype))
        has_bias = bias and _rank(process_group) == 0
        self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if has_bias else None

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


class RowParallelLinear(RowParallelLinearNoReduce):
    """Same, followed by the all-reduce (fused_dense_sparse_dejavu.py:280-317)."""

    def forward(self, x):
        return all_reduce(F.linear(x, self.weight, self.bias), self.process_group)


class _TransposedRowParallelLinear(RowParallelLinear):
    """fc2 of the sparse MLP: storage is the transposed weight (in/world, out), contiguous, which is what
    the gather kernel streams; `.weight` is the usual (out, in/world) view of the same memory."""

    def __init__(self, in_features, out_features, process_group, bias=True, sequence_parallel=False,
                 device=None, dtype=None):
        nn.Module.__init__(self)
        world = _world(process_group)
        if in_features % world != 0:
            raise ValueError(f"in_features ({in_features}) must be divisible by world_size ({world})")
        self.process_group = process_group
        self.in_features, self.out_features = in_features // world, out_features
        storage = torch.empty(self.in_features, out_features, device=device, dtype=dtype)
        self.weight = nn.Parameter(storage.t())
        has_bias = bias and _rank(process_group) == 0
        self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if has_bias else None

    @property
    def weight_t(self) -> torch.Tensor:
        return self.weight.t()  # contiguous (in/world, out)


class ParallelSP(nn.Module):
    """Low-rank sparsity predictor: fc1(fc0(x)), both bias-free; fc0 replicated, fc1 split by output;
    K is the PER-RANK budget K // world (fused_dense_sparse_dejavu.py:33-76, mha_dejavu.py:1078-1121)."""

    def __init__(self, layer_idx=None, embed_dim=None, low_rank_dim=None, out_dim=None, K=None,
                 process_group=None, sequence_parallel=False, device=None, dtype=None) -> None:
        super().__init__()
        assert process_group is not None, "sparse predictor only implemented with parallel for now"
        self.process_group = process_group
        self.layer_idx = layer_idx
        self.embed_dim = embed_dim
        self.fc0 = nn.Linear(embed_dim, low_rank_dim, bias=False, device=device, dtype=dtype)
        self.out = out_dim // _world(process_group)
        self.fc1 = ColumnParallelLinear(low_rank_dim, out_dim, process_group, bias=False,
                                        sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        self.K = K // _world(process_group)

    def forward(self, x):
        """x (1, 1, d) -> logits (out,). A batch (B, 1, d) gives ONE score vector: the sum of the sequences' logits,
        so that the whole batch shares one index set per step, as the reference's kernels expect (one idx for all
        rows, Dejavu/src/ops/triton/gather_gemv.py:198-254); its decode path itself keeps a single sequence
        (mha_dejavu.py:1318, 1469). Both layers are linear and bias-free, so the sum of the logits is the predictor
        applied to the sum of the inputs: the batch costs the two GEMVs of ONE sequence (SP_SUM_INPUTS; with it
        off, every sequence's logits are computed and added in fp32). The two forms differ by fp16 rounding only."""
        x = x.reshape(-1, self.embed_dim)
        def rows_sum(t):  # fp32 sum of the rows, rounded once
            if t.is_cuda and t.dtype == torch.float16:
                return ops.batch_sum(t)
            return t.float().sum(0, keepdim=True).to(t.dtype)

        if x.size(0) > 1 and SP_SUM_INPUTS:
            x = rows_sum(x)
        x = ops.dense_gemv(x, self.fc0.weight)  # B x low_rank
        x = ops.dense_gemv(x, self.fc1.weight)
        if x.size(0) > 1:
            x = rows_sum(x)
        return x.view(-1)


class ParallelFusedMLPDejavu(nn.Module):
    """MLP with contextual sparsity: forward(x, residual, idx) -> (out, mlp_logit). With idx (decode) only
    the rows idx of fc1 / fc2^T are read; mlp_logit = sp(residual) selects the NEXT layer's neurons
    (fused_dense_sparse_dejavu.py:821-951)."""

    has_predictor = True
    run_predictor = True         # False: dense comparator mode, skip the look-ahead predictor
    dense_decode_cublas = False  # True: dense decode GEMVs through torch (cuBLAS)
    push_comm = None             # TensorParallelComm: fc2 sends its result to the peers itself
    fused_mlp = None             # "0" / "1" / "auto" for this module, None = the process-wide DJV_FUSED_MLP

    def __init__(self, in_features, hidden_features, sp_kwargs, out_features=None, activation="gelu_approx",
                 layer_idx=None, process_group=None, bias1=True, bias2=True, sequence_parallel=True,
                 checkpoint_lvl=0, heuristic="auto", device=None, dtype=None):
        assert checkpoint_lvl in [0, 1, 2]
        assert activation in ["gelu_approx", "relu"]
        assert process_group is not None
        assert sp_kwargs is not None or not self.has_predictor, "sparse predictor parameters are not passed in."
        super().__init__()
        if out_features is None:
            out_features = in_features
        factory = {"device": device, "dtype": dtype}
        self.activation = activation
        self.process_group = process_group
        self.sequence_parallel = sequence_parallel
        self.layer_idx = layer_idx
        self.fc1 = ColumnParallelLinear(in_features, hidden_features, process_group, bias=bias1, **factory)
        self.fc2 = _TransposedRowParallelLinear(hidden_features, out_features, process_group, bias=bias2, **factory)
        if self.has_predictor:
            self.sp = ParallelSP(layer_idx=layer_idx, device=device, dtype=dtype, process_group=process_group,
                                 sequence_parallel=sequence_parallel, **sp_kwargs)
        self.skip_all_reduce = False  # set by the block when it fuses the all-reduce with add+LN

    @property
    def fc2_weight_t(self):
        return self.fc2.weight_t

    def forward(self, x, residual, idx=None):
        do_token_generation = x.size(1) == 1
        # the look-ahead predictor for the NEXT layer runs beside this MLP (fused_dense_sparse_dejavu.py:942-949)
        mlp_logit = None
        if do_token_generation and self.has_predictor and self.run_predictor:
            with _side(x, "mlp", after=residual) as done:
                mlp_logit = self.sp(residual)
                done(mlp_logit)
        if idx is not None:
            assert x.size(1) == 1
            assert self.activation == "relu", "the sparse path applies ReLU (gather_gemv.py:655)"
            # idx came from a side stream and the main stream has waited on its event already
            with ops.indices_ready(EARLY_PREFETCH and getattr(idx, "_ready_event", None) is not None):
                out = ops.mlp_sparse(x.view(x.size(0), -1), self.fc1.weight, self.fc2.weight_t, idx, self.fc1.bias,
                                     self.fc2.bias, push_comm=self.push_comm)
            out = out.view(x.size(0), 1, -1)
        elif do_token_generation and not self.dense_decode_cublas:
            act = "relu" if self.activation == "relu" else "gelu_approx"
            h = ops.dense_gemv(x.view(x.size(0), -1), self.fc1.weight, self.fc1.bias, act)
            out = ops.dense_transposed_gemv(h, self.fc2.weight_t, self.fc2.bias,
                                            push_comm=self.push_comm).view(x.size(0), 1, -1)
        else:
            h = F.linear(x, self.fc1.weight, self.fc1.bias)
            h = F.relu(h) if self.activation == "relu" else F.gelu(h, approximate="tanh")
            out = F.linear(h, self.fc2.weight, self.fc2.bias)
        if not self.skip_all_reduce:
            out = all_reduce(out, self.process_group)
        return out, mlp_logit


    def fuses_after_exchange(self, batch: int, d: int, rows: int) -> bool:
        """Whether the second half of the block runs as one kernel for this shape (see FUSED_MLP)."""
        mode = self.fused_mlp if self.fused_mlp is not None else FUSED_MLP
        if mode == "0" or self.push_comm is None or self.activation != "relu":
            return False
        lib = _lib.load()
        if mode == "1":
            return bool(lib.djv_mlp_sparse_fused_supported(batch, d, rows))
        return self.push_comm.world > 1 and bool(lib.djv_mlp_sparse_fused_single_batch(batch, d, rows))

    def can_fuse_after_exchange(self, partial, idx) -> bool:
        """Whether decode_after_exchange applies: a comm that producers push into, a sparse step, and a shape
        the one-pass kernel takes."""
        if self.push_comm is None or idx is None or partial.dim() != 3 or partial.size(1) != 1:
            return False
        if self.push_comm.pushed_seq(partial) is None:
            return False
        return self.fuses_after_exchange(partial.size(0), partial.size(2), idx.numel())

    def decode_after_exchange(self, partial, residual, norm, idx):
        """The block's second half in one kernel: residual = sum over ranks(partial) + residual;
        x = norm(residual); out = fc2(relu(fc1(x)[idx])) sent as the next exchange. The look-ahead predictor
        (fused_dense_sparse_dejavu.py:942-949) takes its own copy of the new residual from the same exchange on
        the side stream, so that it does not wait for this kernel. Returns (out, residual, mlp_logit)."""
        comm = self.push_comm
        B, _, d = partial.shape
        p2 = partial.view(B, d)
        r2 = None if residual is None else residual.reshape(B, d)
        mlp_logit = None
        if self.has_predictor and self.run_predictor:
            seq_in = comm.pushed_seq(p2)
            with _side(partial, "mlp", after=residual) as done:
                _, r_side = comm.allreduce_add_layernorm(p2, r2, None, None, norm.eps, refill=False, seq=seq_in)
                mlp_logit = self.sp(r_side)
                done(mlp_logit)
        with ops.indices_ready(EARLY_PREFETCH and getattr(idx, "_ready_event", None) is not None):
            out, r = ops.mlp_sparse_after_exchange(comm, p2, r2, norm.weight, norm.bias, norm.eps, self.fc1.weight,
                                                   self.fc2.weight_t, idx, self.fc1.bias, self.fc2.bias, push=True)
        return out.view(B, 1, d), r.view(B, 1, d), mlp_logit


class ParallelFusedMLP(ParallelFusedMLPDejavu):
    """The dense MLP of the comparator model (fused_dense_sparse_dejavu.py:696-780): no predictor; decode
    GEMVs go through cuBLAS (torch), which is the dense fp16 decode the sparse path is measured against."""

    has_predictor = False

    def __init__(self, in_features, hidden_features, out_features=None, activation="gelu_approx", layer_idx=None,
                 process_group=None, bias1=True, bias2=True, sequence_parallel=True, checkpoint_lvl=0,
                 heuristic="auto", device=None, dtype=None):
        super().__init__(in_features, hidden_features, None, out_features=out_features, activation=activation,
                         layer_idx=layer_idx, process_group=process_group, bias1=bias1, bias2=bias2,
                         sequence_parallel=sequence_parallel, device=device, dtype=dtype)

    def forward(self, x, residual=None, idx=None):
        h = F.linear(x, self.fc1.weight, self.fc1.bias)
        h = F.relu(h) if self.activation == "relu" else F.gelu(h, approximate="tanh")
        out = F.linear(h, self.fc2.weight, self.fc2.bias)
        if not self.skip_all_reduce:
            out = all_reduce(out, self.process_group)
        return out, None


class ParallelMHASparseAttMlp(nn.Module):
    """Self-attention with head sparsity in decode. forward(x, residual, head_idx, mlp_sp_logit, seqlen,
    inference_params) -> (out, mlp_idx, att_idx): mlp_idx = top-mlp_k of mlp_sp_logit for THIS layer's MLP,
    att_idx = top-att_k of sp(residual) for the NEXT layer's attention (mha_dejavu.py:1152-1511)."""

    sparse_attention = True
    run_predictor = True  # False: dense comparator mode, skip the look-ahead predictor
    next_mixer = None  # the attention module of the following block (set by the model; not a submodule)
    push_comm = None   # TensorParallelComm: out_proj sends its result to the peers itself

    def link_next(self, mixer):
        self.__dict__["next_mixer"] = mixer

    mlp_ref = None  # the MLP of the same block (set by the block; not a submodule)

    def l2_prefetch_enabled(self) -> bool:
        """Whether index lists are followed by an L2 warm-up of the rows they name."""
        if L2_PREFETCH in ("0", "1"):
            return L2_PREFETCH == "1"
        d, hd = self.embed_dim, self.head_dim
        a = self.att_k if (self.sparse_attention and self.att_k) else self.num_head_per_node
        k = self.mlp_k if self.mlp_k else (self.mlp_ref.fc1.weight.shape[0] if self.mlp_ref is not None else 0)
        return (4 * a * hd * d * 2 + 2 * k * d * 2) <= L2_PREFETCH_MB * 1e6

    def __init__(self, embed_dim, num_heads, process_group, sp_kwargs, bias=True, dropout=0.0,
                 softmax_scale=None, causal=False, layer_idx=None, rotary_emb_dim=0, rotary_emb_scale_base=0,
                 use_flash_attn=False, checkpointing=False, sequence_parallel=True, device=None,
                 dtype=None) -> None:
        super().__init__()
        assert rotary_emb_dim == 0, "OPT uses learned positions; rotary embeddings are not on this path"
        self.embed_dim = embed_dim
        self.causal = causal
        self.layer_idx = layer_idx
        self.process_group = process_group
        self.num_heads = num_heads
        assert embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.head_dim = embed_dim // num_heads
        world = _world(process_group)
        assert num_heads % world == 0
        self.num_head_per_node = num_heads // world
        self.softmax_scale = softmax_scale if softmax_scale is not None else self.head_dim ** -0.5
        factory = {"device": device, "dtype": dtype}
        self.Wqkv = ColumnParallelLinear(embed_dim, 3 * embed_dim, process_group, bias=bias,
                                         sequence_parallel=sequence_parallel, **factory)
        self.out_proj = RowParallelLinearNoReduce(embed_dim, embed_dim, process_group, bias=bias,
                                                  sequence_parallel=sequence_parallel, **factory)
        self.sp = None
        if self.sparse_attention:
            self.sp = ParallelSP(layer_idx=layer_idx, device=device, dtype=dtype, process_group=process_group,
                                 sequence_parallel=sequence_parallel, **sp_kwargs)
        self.mlp_k = None  # per-rank budgets, copied in by the block (block_dejavu.py:549-553)
        self.att_k = None
        self.skip_all_reduce = False
        self._bufs = None

    # ---- device-resident decode state --------------------------------------------------------
    def _decode_buffers(self, device, S, batch=1):
        """Per-sequence state of the decode step (one lazy-K/V window, query and context buffer per sequence; the
        sequences of a batch share the head selection, so their windows stay identical)."""
        n, hd, d = self.num_head_per_node, self.head_dim, self.embed_dim
        if (self._bufs is None or self._bufs["S"] != S or self._bufs["device"] != device
                or len(self._bufs["seqs"]) < batch):
            need = _lib.load().djv_attn_step_scratch_bytes(n, hd, S)
            self._bufs = {"S": S, "device": device, "seqs": [{
                "state": torch.zeros(_lib.ATTN_STATE_HDR + 3 * n, dtype=torch.int32, device=device),
                "x_ring": torch.zeros(KV_WINDOW, d, dtype=torch.float16, device=device),
                "q": torch.zeros(n, hd, dtype=torch.float16, device=device),
                "ctx": torch.zeros(1, n, hd, dtype=torch.float16, device=device),
                "scratch": torch.zeros(max(need, 4096), dtype=torch.uint8, device=device),
            } for _ in range(batch)]}
        return self._bufs["seqs"]

    def _batch_buffers(self, device, S, batch):
        """Buffers of the batched decode step: the sequences share sequence 0's state; windows, queries and
        contexts are contiguous over the batch."""
        seqs = self._decode_buffers(device, S, batch)
        bb = self._bufs.get("batch")
        if bb is None or bb["B"] < batch:
            n, hd, d = self.num_head_per_node, self.head_dim, self.embed_dim
            need = _lib.load().djv_decode_attn_scratch_bytes(n, batch, hd, S)
            bb = self._bufs["batch"] = {
                "B": batch,
                "x_ring": torch.zeros(batch, KV_WINDOW, d, dtype=torch.float16, device=device),
                "q": torch.zeros(batch, n, hd, dtype=torch.float16, device=device),
                "ctx": torch.zeros(batch, n, hd, dtype=torch.float16, device=device),
                "scratch": torch.zeros(max(need, 4096), dtype=torch.uint8, device=device),
            }
        bb["state"] = seqs[0]["state"]
        return bb

    def reset_decode_state(self, prompt_len: int, device, S: int, batch: int = 1):
        for b in self._decode_buffers(device, S, batch):
            call("djv_attn_state_reset", b["state"].data_ptr(), self.num_head_per_node, int(prompt_len), ops._stream())

    def decode_status(self) -> int:
        """0, or the negative status a kernel left in the state (synchronises)."""
        if self._bufs is None:
            return 0
        return min(int(b["state"][3].item()) for b in self._bufs["seqs"])

    # ---- prompt phase: dense ------------------------------------------------------------------
    def _prompt_attention(self, x, inference_params):
        B, L, _ = x.shape
        n, hd = self.num_head_per_node, self.head_dim
        qkv = self.Wqkv(x).view(B, L, 3, n, hd)
        q, k, v = qkv.unbind(2)
        if inference_params is not None:
            k_cache, v_cache = inference_params.key_value_memory_dict[self.layer_idx]
            S = v_cache.shape[2]
            off = inference_params.sequence_len_offset
            assert off == 0 and L <= S
            # K cache (B, n, hd/8, S, 8), V cache (B, n, S, hd)   (mha_dejavu.py:385-447)
            k_cache[:, :, :, :L, :] = k.permute(0, 2, 3, 1).reshape(B, n, hd // 8, 8, L).permute(0, 1, 2, 4, 3)
            v_cache[:, :, :L, :] = v.permute(0, 2, 1, 3)
            self.reset_decode_state(L, x.device, S, B)
        ctx = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                             is_causal=True, scale=self.softmax_scale)
        return ctx.transpose(1, 2).reshape(B, L, n * hd)

    # ---- decode step ---------------------------------------------------------------------------
    def _decode_attention(self, x, head_idx, inference_params, between=None):
        """One decode step of this layer's attention; `between()` is called after the projection kernels are
        queued and before the attention kernel (the place to fork look-ahead work onto a side stream).
        A batch shares the head selection and advances in lockstep, so its sequences have identical windows: it
        runs through the batch entry points with one state (one launch per kernel). With BATCHED_ATTENTION off it
        runs sequence by sequence through the batch-1 kernels: sequence 0 on the main stream, the others, whose
        weights then come from L2, as parallel chains on up to BATCH_STREAMS extra streams that rejoin before the
        result is used."""
        n, hd, d = self.num_head_per_node, self.head_dim, self.embed_dim
        B = x.size(0)
        k_cache, v_cache = inference_params.key_value_memory_dict[self.layer_idx]
        assert k_cache.size(0) >= B and v_cache.size(0) >= B
        S = v_cache.shape[2]
        seqs = self._decode_buffers(x.device, S, B)
        xf = x.reshape(B, d).contiguous()
        nnz = 0
        if head_idx is not None:
            assert head_idx.dtype == torch.int32
            head_idx = head_idx.contiguous()
            nnz = head_idx.numel()
        bias = self.Wqkv.bias
        # the layer before may have opened this step already, in the kernel that selected the heads
        step_is_open = 1 if (head_idx is not None and getattr(head_idx, "_step_opened_for", None) is self) else 0
        # an opened step means the state was written on a side stream whose event the main stream has waited on
        early = EARLY_PREFETCH and step_is_open == 1 and getattr(head_idx, "_ready_event", None) is not None
        out = torch.empty(B, d, dtype=x.dtype, device=x.device)
        ob = self.out_proj.bias
        if B > 1 and BATCHED_ATTENTION and x.is_cuda:
            # one state for the batch (shared selection, lockstep windows): one launch per kernel whatever B is
            assert k_cache.is_contiguous() and v_cache.is_contiguous()
            bb = self._batch_buffers(x.device, S, B)
            state = bb["state"]
            call("djv_attn_step_project_batch", bb["q"].data_ptr(), self.Wqkv.weight.data_ptr(),
                 None if bias is None else bias.data_ptr(), xf.data_ptr(), bb["x_ring"].data_ptr(),
                 k_cache.data_ptr(), v_cache.data_ptr(), state.data_ptr(),
                 None if head_idx is None else head_idx.data_ptr(), nnz, d, n, hd, S, B, ops._stream())
            if between is not None:
                between()
            call("djv_attn_step_attend_batch", bb["ctx"].data_ptr(), bb["q"].data_ptr(), k_cache.data_ptr(),
                 v_cache.data_ptr(), state.data_ptr(), B, n, hd, S, float(self.softmax_scale),
                 bb["scratch"].data_ptr(), bb["scratch"].numel(), ops._stream())
            eff_heads_ptr = state.data_ptr() + 4 * (_lib.ATTN_STATE_HDR + n)
            n_eff_ptr = state.data_ptr() + 4 * 2
            for b0 in range(0, B, 16):  # (djv_out_proj_sparse takes up to 16 rows per call)
                nb = min(16, B - b0)
                call("djv_out_proj_sparse", out[b0].data_ptr(), self.out_proj.weight.data_ptr(),
                     bb["ctx"][b0].data_ptr(), eff_heads_ptr, n_eff_ptr, None if ob is None else ob.data_ptr(), nb, d,
                     n, hd, n, ops._stream())
            return out.view(B, 1, d)

        def project(i, b):
            call("djv_attn_step_project", b["q"].data_ptr(), self.Wqkv.weight.data_ptr(),
                 None if bias is None else bias.data_ptr(), xf[i].data_ptr(), b["x_ring"].data_ptr(),
                 k_cache[i].data_ptr(), v_cache[i].data_ptr(), b["state"].data_ptr(),
                 None if head_idx is None else head_idx.data_ptr(), nnz, d, n, hd, S, step_is_open, ops._stream())

        def attend(i, b):
            call("djv_attn_step_attend", b["ctx"].data_ptr(), b["q"].data_ptr(), k_cache[i].data_ptr(),
                 v_cache[i].data_ptr(), b["state"].data_ptr(), n, hd, S, float(self.softmax_scale),
                 b["scratch"].data_ptr(), b["scratch"].numel(), ops._stream())

        def project_out(i, b):
            state = b["state"]
            eff_heads_ptr = state.data_ptr() + 4 * (_lib.ATTN_STATE_HDR + n)
            n_eff_ptr = state.data_ptr() + 4 * 2
            if self.push_comm is not None and B == 1:
                seq = self.push_comm.next_seq()
                call("djv_out_proj_sparse_push", self.push_comm.handle, seq, self.out_proj.weight.data_ptr(),
                     b["ctx"].data_ptr(), eff_heads_ptr, n_eff_ptr, None if ob is None else ob.data_ptr(), 1, d,
                     n, hd, n, ops._stream())
                self.push_comm.note_pushed(out, seq)
            else:
                call("djv_out_proj_sparse", out[i].data_ptr(), self.out_proj.weight.data_ptr(),
                     b["ctx"].data_ptr(), eff_heads_ptr, n_eff_ptr, None if ob is None else ob.data_ptr(), 1, d, n,
                     hd, n, ops._stream())

        n_extra = min((B - 1) // 2, BATCH_STREAMS) if (SIDE_STREAMS_ENABLED and x.is_cuda and B >= 4) else 0
        with ops.indices_ready(early):
            project(0, seqs[0])
            if n_extra == 0:
                for i in range(1, B):
                    project(i, seqs[i])
        joins = []
        if n_extra > 0:
            # Sequence 0 has pulled the selected heads' weights through L2; the other sequences' chains (projection,
            # attention, out_proj: independent of each other) now run side by side on extra streams and hit L2.
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            for j, stream in enumerate(batch_streams(x.device, n_extra)):
                stream.wait_event(fork)
                for t in (out, xf):
                    t.record_stream(stream)
                with torch.cuda.stream(stream):
                    for i in range(1 + j, B, n_extra):
                        project(i, seqs[i])
                        attend(i, seqs[i])
                        project_out(i, seqs[i])
                    done = torch.cuda.Event()
                    done.record(stream)
                joins.append(done)
        if between is not None:
            between()
        on_main = 1 if n_extra > 0 else B  # sequences whose chain continues on the main stream
        for i in range(on_main):
            attend(i, seqs[i])
        with ops.indices_ready(early):
            for i in range(on_main):
                project_out(i, seqs[i])
        for done in joins:
            torch.cuda.current_stream().wait_event(done)
        # the window advance is folded into the next step's first kernel (no djv_attn_step_finish launch)
        return out.view(B, 1, d)

    def forward(self, x, residual, head_idx=None, mlp_sp_logit=None, seqlen=None, inference_params=None, **kwargs):
        do_token_generation = x.size(1) == 1
        decoding = inference_params is not None and inference_params.sequence_len_offset > 0
        # Look-ahead work runs beside the attention, as in the reference (sp_stream, mha_dejavu.py:1364-1370,
        # 1501-1510): the MLP top-K continues on the stream that produced the logits, the head predictor
        # forks from the main stream; consumers wait on the event attached to each result.
        mlp_idx = None
        if mlp_sp_logit is not None:
            with _side(x, "mlp", after=mlp_sp_logit) as done:
                mlp_idx = ops.topk_indices(mlp_sp_logit, self.mlp_k, torch.int32)
                done(mlp_idx)
                if decoding and self.mlp_ref is not None and x.is_cuda and self.l2_prefetch_enabled():
                    # the rows this layer's MLP is going to gather, a good part of a layer ahead of it
                    ops.prefetch_rows_l2(mlp_idx, self.mlp_ref.fc1.weight, self.mlp_ref.fc2.weight_t)
        result = {"att_idx": None}

        def predict_heads():
            if do_token_generation and self.sp is not None and self.run_predictor:
                nxt = self.next_mixer if (decoding and FUSE_STEP_OPEN) else None
                with _side(x, "att", after=residual) as done:
                    scores = self.sp(residual)
                    if nxt is not None and nxt.sparse_attention and scores.dim() == 1 and x.size(0) == 1:
                        # the selection is for the next layer's attention: open its decode step in the same
                        # kernel, so that layer starts with its QKV projection
                        S_next = inference_params.key_value_memory_dict[nxt.layer_idx][1].shape[2]
                        state = nxt._decode_buffers(x.device, S_next)[0]["state"]
                        idx = ops.topk_indices_open_step(scores, self.att_k, state, S_next)
                        idx._step_opened_for = nxt
                    else:
                        idx = ops.topk_indices(scores, self.att_k, torch.int32)
                    result["att_idx"] = idx
                    done(idx)
                    if (nxt is not None and nxt.sparse_attention and x.size(0) == 1
                            and self.l2_prefetch_enabled()):
                        # the next layer's q, k, v slabs and out_proj columns of the heads just selected
                        n_n, hd_n = nxt.num_head_per_node, nxt.head_dim
                        wq = nxt.Wqkv.weight.view(3, n_n * hd_n, nxt.embed_dim)
                        ops.prefetch_rows_l2(idx, wq[0], wq[1], wq[2], rows_per_index=hd_n)
                        ops.prefetch_head_columns_l2(idx, nxt.out_proj.weight, hd_n)

        if decoding:
            assert do_token_generation
            _wait_ready(head_idx)

            def between():
                # the head predictor forks after the QKV projection: its GEMVs then overlap the attention kernel,
                # which leaves HBM mostly idle, instead of taking the multiprocessors just before the projection
                predict_heads()
                if (MLP_IDX_JOIN == "attend" and mlp_idx is not None and self.mlp_ref is not None
                        and self.mlp_ref.fuses_after_exchange(x.size(0), self.embed_dim, mlp_idx.numel())):
                    _wait_ready(mlp_idx)

            out = self._decode_attention(x, head_idx if self.sparse_attention else None, inference_params,
                                         between=between)
        else:
            predict_heads()
            out = self.out_proj(self._prompt_attention(x, inference_params))
        if not self.skip_all_reduce:
            out = all_reduce(out, self.process_group)
        _wait_ready(mlp_idx)  # this layer's MLP is next on the main stream
        return out, mlp_idx, result["att_idx"]


class ParallelMHADejavu(ParallelMHASparseAttMlp):
    """Dense attention + top-K of the MLP logits: forward(...) -> (out, mlp_idx) (mha_dejavu.py:910-1075)."""

    sparse_attention = False

    def __init__(self, embed_dim, num_heads, process_group, bias=True, dropout=0.0, softmax_scale=None,
                 causal=False, layer_idx=None, rotary_emb_dim=0, rotary_emb_scale_base=0, use_flash_attn=False,
                 checkpointing=False, sequence_parallel=True, device=None, dtype=None) -> None:
        super().__init__(embed_dim, num_heads, process_group, None, bias=bias, dropout=dropout,
                         softmax_scale=softmax_scale, causal=causal, layer_idx=layer_idx,
                         rotary_emb_dim=rotary_emb_dim, use_flash_attn=use_flash_attn,
                         sequence_parallel=sequence_parallel, device=device, dtype=dtype)

    def forward(self, x, residual=None, mlp_sp_logit=None, seqlen=None, inference_params=None, **kwargs):
        out, mlp_idx, _ = super().forward(x, residual, None, mlp_sp_logit, seqlen, inference_params)
        return out, mlp_idx


class BlockMlpAttSparse(nn.Module):
    """Pre-norm block threading the look-ahead state:
    forward(hidden, residual, mixer_subset, mixer_kwargs, head_idx, mlp_sp_logit)
        -> (hidden, residual, next_mlp_sp_logit, next_att_idx)              (block_dejavu.py:464-663)."""

    returns_att_idx = True

    def __init__(self, dim, mixer_cls=None, mlp_cls=None, norm_cls=nn.LayerNorm, dropout_cls=nn.Dropout,
                 prenorm=True, resid_dropout1=0.0, resid_dropout2=0.0, drop_path1=0.0, drop_path2=0.0,
                 fused_dropout_add_ln=False, return_residual=False, residual_in_fp32=False,
                 sequence_parallel=False, mark_shared_params=False):
        super().__init__()
        assert prenorm, "OPT decoder blocks are pre-norm"
        assert not residual_in_fp32, "the decode path keeps the residual stream in fp16"
        self.prenorm = prenorm
        self.mixer = mixer_cls(dim)
        self.norm1 = norm_cls(dim)
        self.mlp = mlp_cls(dim)
        self.norm2 = norm_cls(dim)
        # per-rank budgets (block_dejavu.py:549-553)
        self.mixer.__dict__["mlp_ref"] = self.mlp
        if hasattr(self.mlp, "sp"):
            self.mixer.mlp_k = self.mlp.sp.K
        if getattr(self.mixer, "sp", None) is not None:
            self.mixer.att_k = self.mixer.sp.K
        self.comm = None  # TensorParallelComm for the fused all-reduce + add + LayerNorm

    def enable_fused_allreduce(self, comm):
        self.comm = comm
        self.mixer.skip_all_reduce = comm is not None
        self.mlp.skip_all_reduce = comm is not None
        push = comm if PUSH_PARTIALS else None
        self.mixer.__dict__["push_comm"] = push
        self.mlp.__dict__["push_comm"] = push

    def _add_norm(self, hidden_states, residual, norm, reduce_first):
        """residual = hidden + residual; hidden = norm(residual); `hidden` may still be a rank-partial sum."""
        decode = hidden_states.dim() == 3 and hidden_states.size(1) == 1 and hidden_states.is_cuda
        if decode:
            B, _, d = hidden_states.shape
            x2 = hidden_states.reshape(B, d)
            r2 = None if residual is None else residual.reshape(B, d)
            if reduce_first and self.comm is not None:
                y, r = self.comm.allreduce_add_layernorm(x2, r2, norm.weight, norm.bias, norm.eps)
            else:
                y, r = ops.add_layernorm(x2, r2, norm.weight, norm.bias, norm.eps)
            return y.view(B, 1, d), r.view(B, 1, d)
        if reduce_first and self.comm is not None:
            hidden_states = all_reduce(hidden_states, self.mixer.process_group)
        residual = (hidden_states + residual) if residual is not None else hidden_states
        return norm(residual.to(dtype=norm.weight.dtype)), residual

    def forward(self, hidden_states, residual=None, mixer_subset=None, mixer_kwargs=None, head_idx=None,
                mlp_sp_logit=None, hidden_is_partial=False):
        # the wait for the head list goes before the LayerNorm launch, so that the QKV projection follows the
        # LayerNorm with a single (programmatic) edge and can prefetch its weights while the LayerNorm runs
        _wait_ready(head_idx)
        hidden_states, residual = self._add_norm(hidden_states, residual, self.norm1, hidden_is_partial)
        if mixer_kwargs is None:
            mixer_kwargs = {}
        if self.returns_att_idx:
            hidden_states, mlp_idx, next_att_idx = self.mixer(hidden_states, residual=residual, head_idx=head_idx,
                                                              mlp_sp_logit=mlp_sp_logit, **mixer_kwargs)
        else:
            hidden_states, mlp_idx = self.mixer(hidden_states, residual=residual, mlp_sp_logit=mlp_sp_logit,
                                                **mixer_kwargs)
            next_att_idx = None
        if self.comm is not None and self.mlp.can_fuse_after_exchange(hidden_states, mlp_idx):
            _wait_ready(mlp_idx)
            hidden_states, residual, next_mlp_sp_logit = self.mlp.decode_after_exchange(hidden_states, residual,
                                                                                          self.norm2, mlp_idx)
        else:
            hidden_states, residual = self._add_norm(hidden_states, residual, self.norm2, self.comm is not None)
            hidden_states, next_mlp_sp_logit = self.mlp(hidden_states, residual, mlp_idx)
        if self.returns_att_idx:
            return hidden_states, residual, next_mlp_sp_logit, next_att_idx
        return hidden_states, residual, next_mlp_sp_logit


class BlockDejavu(BlockMlpAttSparse):
    """Block of the MLP-sparse-only model: forward(...) -> (hidden, residual, next_mlp_sp_logit)
    (block_dejavu.py:264-461)."""

    returns_att_idx = False
