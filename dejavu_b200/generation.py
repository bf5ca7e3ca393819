"""Greedy generation with a CUDA-graph decode step, with the call surface the reference's benchmarks use:

    update_graph_cache(model, cache, batch_size, seqlen_og, max_seqlen, tensor_parallel=1)
    model.generate(input_ids=, max_length=, fused_ft_kernel=, cg=, vocab_size=, return_dict_in_generate=,
                   output_scores=, timing=)                -> .sequences (, .scores)

(Dejavu/benchmarks/benchmark_generation_opt_dejavu.py:182-194; the implementation the reference imports is
flash_attn.utils.generation of flash-attention v0.2.8, which is not part of the reference tree.)

The K/V caches use the decode kernel's layouts, per layer: K (B, heads_local, head_dim/8, S, 8),
V (B, heads_local, S, head_dim). Everything the decode step needs to know about the position (cache
length, lazy-K/V window) is device-resident state advanced by the kernels, so one captured graph is valid
for every step; only input_ids and position_ids are rewritten between replays.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Optional

import torch


@dataclass
class InferenceParams:
    """Fields the reference's mixers read (mha_dejavu.py:385-447, 1395-1446)."""

    max_sequence_len: int
    max_batch_size: int
    sequence_len_offset: int = 0
    batch_size_offset: int = 0
    key_value_memory_dict: dict = field(default_factory=dict)
    fused_ft_kernel: bool = True
    lengths_per_sample: Optional[torch.Tensor] = None


def allocate_kv_cache(model, batch_size: int, max_seqlen: int, device, dtype=torch.float16) -> dict:
    cfg = model.config
    hd = cfg.hidden_size // cfg.n_head
    assert hd % 8 == 0
    caches = {}
    for i, layer in enumerate(model.transformer.layers):
        n = layer.mixer.num_head_per_node
        k = torch.zeros(batch_size, n, hd // 8, max_seqlen, 8, device=device, dtype=dtype)
        v = torch.zeros(batch_size, n, max_seqlen, hd, device=device, dtype=dtype)
        caches[i] = (k, v)
    return caches


@dataclass
class DecodingCGCache:
    max_batch_size: int = 0
    max_seqlen: int = 0
    device: object = None
    inference_params: Optional[InferenceParams] = None
    graph: Optional[torch.cuda.CUDAGraph] = None
    input_ids: Optional[torch.Tensor] = None
    position_ids: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    next_token: Optional[torch.Tensor] = None
    launches_per_step: int = 0

    def run(self, new_input_ids, new_position_ids):
        self.input_ids.copy_(new_input_ids)
        self.position_ids.copy_(new_position_ids)
        self.graph.replay()
        return self.logits


@torch.inference_mode()
def update_graph_cache(model, cache, batch_size, seqlen_og, max_seqlen, tensor_parallel=1, dtype=None,
                       n_warmups=2, greedy_feedback=False, vocab_size=None):
    """(Re)allocates the K/V caches for (batch_size, max_seqlen) and captures ONE decode step of `model`
    into a CUDA graph. Capture launches nothing; the warm-up steps before it do run, and leave the lazy-K/V
    state wherever they leave it — the prompt pass of every generate() call resets that state.
    With greedy_feedback the graph also takes the arg-max of the logits, writes it back into input_ids and
    advances position_ids, so a replay is one complete greedy decode step with no host work."""
    if cache is None:
        cache = DecodingCGCache()
    param = next(iter(model.parameters()))
    device = param.device
    dtype = dtype or param.dtype
    if (cache.graph is not None and cache.device == device and cache.max_batch_size >= batch_size
            and cache.max_seqlen >= max_seqlen):
        return cache
    cache.graph = None
    cache.device, cache.max_batch_size, cache.max_seqlen = device, batch_size, max_seqlen
    cache.inference_params = InferenceParams(
        max_sequence_len=max_seqlen, max_batch_size=batch_size, sequence_len_offset=seqlen_og,
        key_value_memory_dict=allocate_kv_cache(model, batch_size, max_seqlen, device, dtype),
        fused_ft_kernel=True,
        lengths_per_sample=torch.full((batch_size,), seqlen_og, dtype=torch.int32, device=device))
    cache.input_ids = torch.zeros(batch_size, 1, dtype=torch.long, device=device)
    cache.position_ids = torch.full((batch_size, 1), seqlen_og, dtype=torch.long, device=device)
    # the decode state must describe a decodable position while warming up
    for layer in model.transformer.layers:
        layer.mixer.reset_decode_state(seqlen_og, device, max_seqlen, batch_size)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    def step():
        cache.logits = model(cache.input_ids, position_ids=cache.position_ids,
                             inference_params=cache.inference_params).logits
        if greedy_feedback:
            cache.next_token = cache.logits[:, -1, :vocab_size].argmax(dim=-1, keepdim=True)
            cache.input_ids.copy_(cache.next_token)
            cache.position_ids.add_(1)

    with torch.cuda.stream(s):
        for _ in range(n_warmups):
            step()
        s.synchronize()
        if torch.distributed.is_initialized():
            torch.distributed.barrier()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    from . import _lib

    launches_before = _lib.launch_count()
    # captured on a high-priority stream: when a main-chain kernel and look-ahead work on a side stream both
    # have blocks waiting for a multiprocessor, the main chain goes first
    priority = int(os.environ.get("DJV_MAIN_PRIORITY", "-1"))  # development knob; 0 = same as the side streams
    with torch.cuda.graph(graph, stream=torch.cuda.Stream(device=device, priority=priority)):
        step()
    cache.launches_per_step = _lib.launch_count() - launches_before  # kernels of libdejavu_b200 per replay
    cache.graph = graph
    return cache


class GenerationMixin:
    @torch.inference_mode()
    def generate(self, input_ids, max_length, top_k=1, top_p=0.0, temperature=1.0, fused_ft_kernel=True,
                 cg=False, vocab_size=None, return_dict_in_generate=False, output_scores=False, timing=False,
                 **kwargs):
        """Greedy decoding (top_k=1 is the only sampler the benchmarks use). Returns an object with
        .sequences (B, max_length) and, when asked, .scores (list of (B, vocab) logits per new token)."""
        assert top_k == 1, "only greedy decoding is implemented"
        B, seqlen_og = input_ids.shape
        device = input_ids.device
        if timing:
            torch.cuda.synchronize()
            t0 = time.time()
        if cg:
            self._decoding_cache = update_graph_cache(self, getattr(self, "_decoding_cache", None), B, seqlen_og,
                                                      max_length)
            ip = self._decoding_cache.inference_params
            ip.max_sequence_len, ip.max_batch_size = max_length, B
        else:
            ip = InferenceParams(max_sequence_len=max_length, max_batch_size=B, fused_ft_kernel=fused_ft_kernel,
                                 key_value_memory_dict=allocate_kv_cache(self, B, max_length, device))
        ip.sequence_len_offset = 0
        # prompt pass (dense); fills the caches and resets the lazy-K/V state to base = prompt length
        logits = self(input_ids, inference_params=ip).logits[:, -1]
        scores, sequences = [], [input_ids]
        ip.sequence_len_offset = seqlen_og
        pos = torch.full((B, 1), seqlen_og, dtype=torch.long, device=device)
        while True:
            if vocab_size is not None:
                logits = logits[..., :vocab_size]
            if output_scores:
                scores.append(logits.clone())
            token = logits.argmax(dim=-1, keepdim=True)
            sequences.append(token)
            if ip.sequence_len_offset >= max_length - 1:
                break
            if cg:
                logits = self._decoding_cache.run(token, pos)[:, -1]
            else:
                logits = self(token, position_ids=pos, inference_params=ip).logits[:, -1]
            ip.sequence_len_offset += 1
            pos += 1
        if timing:
            torch.cuda.synchronize()
            print(f"Prompt processing + decoding time: {(time.time() - t0) * 1000:.0f}ms")
        out = SimpleNamespace(sequences=torch.cat(sequences, dim=1))
        if output_scores:
            out.scores = scores
        return out if return_dict_in_generate else out.sequences
