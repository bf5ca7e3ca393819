"""Tensor-parallel exchange for the decode step: one-shot all-reduce fused with residual add + LayerNorm.

Replaces the NCCL all_reduce after out_proj and after fc2 (Dejavu/src/models/modules/mha_dejavu.py:1498,
Dejavu/src/ops/fused_dense_sparse_dejavu.py:937-940) plus the add + norm that follows it in the block
(Dejavu/src/models/modules/block_dejavu.py:575-584, 625-636). torch.distributed is only used to exchange
the CUDA IPC handles at set-up; the data path is the kernel in csrc/comm.cu storing each rank's partial
into the peers' receive buffers with plain stores over NVLink.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from ._lib import call


class TensorParallelComm:
    """One exchange object per rank. Exchanges of a decode step are numbered 0, 1, 2, ... in the order their
    producers are launched (`next_seq`), identically on every rank; `end_step` closes the step. With
    process_group = None the object is local (world 1): the same kernels then run on a single GPU, each
    "exchange" being a hand-over from the producing kernel to the consuming one through the receive buffer."""

    def __init__(self, process_group, device, max_bytes: int):
        self.pg = process_group
        self.rank = 0 if process_group is None else process_group.rank()
        self.world = 1 if process_group is None else process_group.size()
        self.device = device
        lib = _lib.load()
        self.slot_bytes = (max_bytes + 255) // 256 * 256
        buf = C.c_void_p()
        with torch.cuda.device(device):
            _lib.check("djv_ipc_alloc", lib.djv_ipc_alloc(lib.djv_comm_buffer_bytes(self.world, self.slot_bytes),
                                                          C.byref(buf)))
            self._own = (buf,)
            self._opened = []
            bufs = (C.c_void_p * self.world)()
            if self.world == 1:
                bufs[0] = buf
            else:
                hb = C.create_string_buffer(64)
                _lib.check("djv_ipc_get_handle", lib.djv_ipc_get_handle(buf, hb))
                gathered = [None] * self.world
                dist.all_gather_object(gathered, hb.raw, group=process_group)
                for r, b_raw in enumerate(gathered):
                    if r == self.rank:
                        bufs[r] = buf
                        continue
                    pb = C.c_void_p()
                    _lib.check("djv_ipc_open", lib.djv_ipc_open(b_raw, C.byref(pb)))
                    self._opened.append(pb)
                    bufs[r] = pb
            self._comm = C.c_void_p()
            _lib.check("djv_comm_create", lib.djv_comm_create(C.byref(self._comm), self.rank, self.world, bufs,
                                                              self.slot_bytes))
        # every rank has mapped every buffer and initialised its own before the first call
        if self.world > 1:
            dist.barrier(group=process_group)
        self._pushed = {}  # data_ptr of a placeholder -> exchange number a producer kernel sent it under
        self._seq = 0      # exchanges started in the current step

    @property
    def handle(self):
        return self._comm

    def next_seq(self) -> int:
        """Number of the next exchange of this step (call once per exchange, same order on every rank)."""
        s = self._seq
        self._seq += 1
        return s

    def note_pushed(self, placeholder: torch.Tensor, seq: int):
        """The kernel that produced this rank's partial has stored it into every rank's receive buffer as
        exchange `seq`; `placeholder` (never written) stands for it until a consumer takes it."""
        self._pushed[placeholder.data_ptr()] = seq

    def pushed_seq(self, t: torch.Tensor):
        """Exchange number under which `t`'s content was sent by its producer, or None."""
        return self._pushed.get(t.data_ptr())

    def take_pushed(self, t: torch.Tensor):
        return self._pushed.pop(t.data_ptr(), None)

    def end_step(self):
        """Closes the step on the current stream: call after every kernel of the step that touches the exchange
        has been queued and all side streams have been joined."""
        n, self._seq = self._seq, 0
        self._pushed.clear()
        if n:
            call("djv_comm_end_step", self._comm, n, torch.cuda.current_stream().cuda_stream)

    def allreduce_add_layernorm(self, partial, residual, weight, bias, eps, refill=True, seq=None):
        """r = sum over ranks(partial) + residual; y = LayerNorm(r) (y = r when weight is None). partial, residual
        (B, d) fp16. Returns (y, r); identical bits on every rank. `partial` may be a placeholder whose content a
        producer kernel has sent already; `seq` names an exchange explicitly (a second consumer of it)."""
        B, d = partial.shape
        partial = partial.contiguous()
        y, r = torch.empty_like(partial), torch.empty_like(partial)
        send = None
        if seq is None:
            seq = self.take_pushed(partial)
            if seq is None:
                seq = self.next_seq()
                send = partial.data_ptr()
        call("djv_allreduce_add_layernorm", self._comm, seq, _lib.EXCHANGE_REFILL if refill else 0, y.data_ptr(),
             r.data_ptr(), send, None if residual is None else residual.contiguous().data_ptr(),
             None if weight is None else weight.data_ptr(), None if bias is None else bias.data_ptr(),
             B, d, float(eps), torch.cuda.current_stream().cuda_stream)
        return y, r

    def status(self) -> int:
        """0, or DJV_ERR_TIMEOUT if a wait on a peer ran out (synchronises the last stream used)."""
        return int(_lib.load().djv_comm_status(self._comm))

    def close(self):
        lib = _lib.load()
        if self._comm:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.pg)  # nobody is still reading a peer's buffer
            lib.djv_comm_destroy(self._comm)
            for p in self._opened:
                lib.djv_ipc_close(p)
            for p in self._own:
                lib.djv_ipc_free(p)
            self._comm = None
