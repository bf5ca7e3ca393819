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
    def __init__(self, process_group, device, max_bytes: int):
        self.pg = process_group
        self.rank, self.world = process_group.rank(), process_group.size()
        self.device = device
        lib = _lib.load()
        self.slot_bytes = (max_bytes + 255) // 256 * 256
        buf = C.c_void_p()
        _lib.check("djv_ipc_alloc", lib.djv_ipc_alloc(lib.djv_comm_buffer_bytes(self.world, self.slot_bytes),
                                                      C.byref(buf)))
        self._own = (buf,)
        hb = C.create_string_buffer(64)
        _lib.check("djv_ipc_get_handle", lib.djv_ipc_get_handle(buf, hb))
        gathered = [None] * self.world
        dist.all_gather_object(gathered, hb.raw, group=process_group)
        self._opened = []
        bufs = (C.c_void_p * self.world)()
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
        dist.barrier(group=process_group)
        self._pushed = set()  # data_ptr of placeholders whose content a producer kernel has sent already

    @property
    def handle(self):
        return self._comm

    def note_pushed(self, placeholder: torch.Tensor):
        """The kernel that produced this rank's partial has stored it into every rank's receive buffer;
        `placeholder` (never written) stands for it until allreduce_add_layernorm consumes it."""
        self._pushed.add(placeholder.data_ptr())

    def allreduce_add_layernorm(self, partial, residual, weight, bias, eps):
        """r = sum over ranks(partial) + residual; y = LayerNorm(r). partial, residual (B, d) fp16.
        Returns (y, r); identical bits on every rank."""
        B, d = partial.shape
        partial = partial.contiguous()
        y, r = torch.empty_like(partial), torch.empty_like(partial)
        sent = partial.data_ptr() in self._pushed
        self._pushed.discard(partial.data_ptr())
        call("djv_allreduce_add_layernorm", self._comm, y.data_ptr(), r.data_ptr(),
             None if sent else partial.data_ptr(),
             None if residual is None else residual.contiguous().data_ptr(), weight.data_ptr(), bias.data_ptr(),
             B, d, float(eps), torch.cuda.current_stream().cuda_stream)
        return y, r

    def status(self) -> int:
        """0, or DJV_ERR_TIMEOUT if a wait on a peer ran out (synchronises the last stream used)."""
        return int(_lib.load().djv_comm_status(self._comm))

    def close(self):
        lib = _lib.load()
        if self._comm:
            torch.cuda.synchronize()
            dist.barrier(group=self.pg)  # nobody is still reading a peer's buffer
            lib.djv_comm_destroy(self._comm)
            for p in self._opened:
                lib.djv_ipc_close(p)
            for p in self._own:
                lib.djv_ipc_free(p)
            self._comm = None
