"""Model-level parity: the sparse decoder on the GPU against the CPU restatement of the reference's wiring."""
import pytest
import torch

from oracle.model_oracle import OracleDecoder

pytestmark = pytest.mark.gpu


def tiny_config(mlp_K, att_K, n_layer=4):
    from dejavu_b200.gpt import apply_sparsity_knobs, opt_config

    cfg = opt_config("opt-125m", n_layer=n_layer, n_embd=256, hidden_size=256, n_head=4, n_inner=1024,
                     vocab_size=512, max_position_embeddings=128, n_positions=128, mlp_sp_dim=64, att_sp_dim=32)
    return apply_sparsity_knobs(cfg, mlp_K, att_K, att_K)


def build(cfg, cuda, seed=0, local_exchange=False):
    """local_exchange: route the block's hand-overs through a one-rank exchange object, which turns on the
    kernels a tensor-parallel run uses (producers that send, the exchange + LayerNorm consumer, the one-launch
    second half of a block) on a single GPU."""
    from dejavu_b200.gpt import GPTLMHeadModel

    model = GPTLMHeadModel(cfg, device=cuda, dtype=torch.float16).eval()
    model.init_random(seed, std=0.05)
    if local_exchange:
        from dejavu_b200.comm import TensorParallelComm

        model.transformer.enable_fused_allreduce(TensorParallelComm(None, cuda, max_bytes=cfg.hidden_size * 2),
                                                 fused_mlp="1")
    return model


def record_selections(model):
    rec = []

    def hook(layer_idx):
        def fn(_m, _inp, out):
            mlp_idx = out[1]
            att_idx = out[2] if len(out) > 2 else None
            rec[-1][layer_idx] = {"mlp_idx": None if mlp_idx is None else mlp_idx.cpu(),
                                  "att_idx": None if att_idx is None else att_idx.cpu()}
        return fn

    handles = [l.mixer.register_forward_hook(hook(i)) for i, l in enumerate(model.transformer.layers)]
    return rec, handles


@pytest.mark.parametrize("mlp_K,att_K,local_exchange", [(256, 2, False), (256, 4, False), (1024, 2, False),
                                                       (1024, 4, False), (256, 2, True), (256, 4, True),
                                                       (1024, 2, True)])
def test_decode_matches_oracle(cuda, mlp_K, att_K, local_exchange):
    """Sparse MLP + sparse attention, sparse MLP only, sparse attention only, dense; and the same through the
    exchange kernels (one rank)."""
    cfg = tiny_config(mlp_K, att_K)
    model = build(cfg, cuda, local_exchange=local_exchange)
    oracle = OracleDecoder(model.state_dict(), cfg)
    gen = torch.Generator().manual_seed(0)
    P, steps = 9, 36  # crosses two 16-step lazy-K/V windows
    ids = torch.randint(0, cfg.vocab_size, (1, P), generator=gen)
    rec, handles = record_selections(model)
    rec.append({})
    out = model.generate(ids.to(cuda), max_length=P + steps, cg=False, return_dict_in_generate=True,
                         output_scores=True)
    # replay the GPU's token sequence through the oracle, forcing (and validating) the GPU's index sets
    ref_logits = oracle.prompt(ids[0])
    seq = out.sequences[0].cpu()
    assert torch.allclose(out.scores[0][0].float().cpu(), ref_logits.float(), atol=3e-2, rtol=3e-2)
    for h in handles:
        h.remove()
    # the hooks fired once for the prompt pass (no selections) and once per decode step
    model2 = build(cfg, cuda, local_exchange=local_exchange)
    rec2, handles2 = record_selections(model2)
    from dejavu_b200.generation import InferenceParams, allocate_kv_cache

    ip = InferenceParams(max_sequence_len=P + steps, max_batch_size=1,
                         key_value_memory_dict=allocate_kv_cache(model2, 1, P + steps, cuda))
    rec2.append({})
    model2(ids.to(cuda), inference_params=ip)
    ip.sequence_len_offset = P
    for t in range(steps - 1):
        tok = seq[P + t].view(1, 1).to(cuda)
        rec2.append({})
        logits = model2(tok, position_ids=torch.tensor([[P + t]], device=cuda), inference_params=ip).logits[0, -1]
        ip.sequence_len_offset += 1
        forced = [rec2[-1].get(i, {}) for i in range(cfg.n_layer)]
        ref, chosen = oracle.decode(int(seq[P + t]), P + t, forced=forced)
        assert torch.allclose(logits.float().cpu(), ref.float(), atol=3e-2, rtol=3e-2), \
            f"step {t}: max diff {(logits.float().cpu() - ref.float()).abs().max().item()}"
        assert torch.allclose(logits.float().cpu(), out.scores[t + 1][0].float().cpu(), atol=1e-3), \
            "teacher-forced replay and generate() disagree"
    for m in model2.transformer.layers:
        assert m.mixer.decode_status() == 0
    for h in handles2:
        h.remove()
    for m in (model, model2):
        if m.transformer.comm is not None:
            assert m.transformer.comm.status() == 0
            m.transformer.comm.close()


@pytest.mark.parametrize("d,heads,mlp_K,att_K,steps", [(4096, 32, 2048, 12, 20), (9216, 72, 4096, 24, 10),
                                                       (12288, 96, 4096, 32, 10)])
def test_decode_matches_oracle_at_real_widths(cuda, d, heads, mlp_K, att_K, steps):
    """Two layers at the hidden size, head count and sparsity of OPT-6.7B / 66B / 175B (BASELINE configs 2-4; ffn =
    4 d, 128-wide heads; a small vocabulary keeps the LM head out of the way). Logit tolerance 3e-2 absolute and
    relative: the logits of these random models are O(1) and carry the fp16 rounding of two residual blocks whose
    sums run over up to 49152 terms in a different order than the oracle's."""
    from dejavu_b200.generation import InferenceParams, allocate_kv_cache
    from dejavu_b200.gpt import GPTLMHeadModel, apply_sparsity_knobs, opt_config

    cfg = opt_config("opt-125m", n_layer=2, n_embd=d, hidden_size=d, n_head=heads, n_inner=4 * d, vocab_size=1024,
                     max_position_embeddings=64, n_positions=64)
    apply_sparsity_knobs(cfg, mlp_K, att_K, att_K)
    model = GPTLMHeadModel(cfg, device=cuda, dtype=torch.float16).eval().init_random(3)
    oracle = OracleDecoder(model.state_dict(), cfg, score_margin=2e-3, cache_fp32=True)
    P = 8
    ids = torch.randint(0, cfg.vocab_size, (1, P), generator=torch.Generator().manual_seed(d))
    rec, handles = record_selections(model)
    ip = InferenceParams(max_sequence_len=P + steps, max_batch_size=1,
                         key_value_memory_dict=allocate_kv_cache(model, 1, P + steps, cuda))
    rec.append({})
    with torch.inference_mode():
        logits = model(ids.to(cuda), inference_params=ip).logits[0, -1].float().cpu()
    assert torch.allclose(logits, oracle.prompt(ids[0]).float(), atol=3e-2, rtol=3e-2)
    ip.sequence_len_offset = P
    for t in range(steps):
        tok = int(logits.argmax())
        rec.append({})
        with torch.inference_mode():
            logits = model(torch.tensor([[tok]], device=cuda), position_ids=torch.tensor([[P + t]], device=cuda),
                           inference_params=ip).logits[0, -1].float().cpu()
        ip.sequence_len_offset += 1
        ref, _ = oracle.decode(tok, P + t, forced=[rec[-1].get(i, {}) for i in range(cfg.n_layer)])
        assert torch.allclose(logits, ref.float(), atol=3e-2, rtol=3e-2), \
            f"step {t}: max diff {(logits - ref.float()).abs().max().item()}"
    assert oracle.free_running_checks > 0, "no selection was decisive enough to be compared exactly"
    for h in handles:
        h.remove()
    assert all(m.mixer.decode_status() == 0 for m in model.transformer.layers)


@pytest.mark.parametrize("B,mlp_K,att_K,local_exchange,batched", [
    (3, 256, 2, False, True), (4, 256, 2, True, True), (2, 1024, 4, False, True), (5, 256, 2, True, True),
    (18, 256, 2, False, True),   # more rows than one out_proj launch takes
    (5, 256, 2, False, False),   # sequence by sequence, two extra streams
    (9, 1024, 4, False, False)])
def test_batched_decode_shares_one_index_set_and_matches_oracle(cuda, monkeypatch, B, mlp_K, att_K, local_exchange,
                                                                batched):
    """Several sequences decode in lockstep with ONE index set per layer and step (top-K of the predictor logits
    summed over the batch); every sequence's logits follow the oracle, which applies the same rule. `batched`: the
    attention of the whole batch through the batch entry points (one state), else through the batch-1 kernels."""
    from dejavu_b200 import modules
    from dejavu_b200.generation import InferenceParams, allocate_kv_cache

    monkeypatch.setattr(modules, "BATCHED_ATTENTION", batched)
    cfg = tiny_config(mlp_K, att_K, n_layer=3)
    model = build(cfg, cuda, local_exchange=False)
    if local_exchange:
        from dejavu_b200.comm import TensorParallelComm

        model.transformer.enable_fused_allreduce(TensorParallelComm(None, cuda, max_bytes=B * cfg.hidden_size * 2),
                                                 fused_mlp="1")
    oracle = OracleDecoder(model.state_dict(), cfg, score_margin=1e-2)
    gen = torch.Generator().manual_seed(B)
    P, steps = 6, 20  # crosses a 16-step lazy-K/V window
    ids = torch.randint(0, cfg.vocab_size, (B, P), generator=gen)
    rec, handles = record_selections(model)
    ip = InferenceParams(max_sequence_len=P + steps, max_batch_size=B,
                         key_value_memory_dict=allocate_kv_cache(model, B, P + steps, cuda))
    rec.append({})
    with torch.inference_mode():
        logits = model(ids.to(cuda), inference_params=ip).logits[:, -1].float().cpu()
    ref = oracle.prompt(ids)
    assert torch.allclose(logits, ref.float(), atol=3e-2, rtol=3e-2)
    ip.sequence_len_offset = P
    for t in range(steps):
        toks = logits.argmax(-1)
        rec.append({})
        with torch.inference_mode():
            logits = model(toks.view(B, 1).to(cuda), position_ids=torch.full((B, 1), P + t, device=cuda),
                           inference_params=ip).logits[:, -1].float().cpu()
        ip.sequence_len_offset += 1
        forced = [rec[-1].get(i, {}) for i in range(cfg.n_layer)]
        ref, _ = oracle.decode(toks.tolist(), P + t, forced=forced)
        assert torch.allclose(logits, ref.float(), atol=3e-2, rtol=3e-2), \
            f"step {t}: max diff {(logits - ref.float()).abs().max().item()}"
    for m in model.transformer.layers:
        assert m.mixer.decode_status() == 0
    for h in handles:
        h.remove()
    if model.transformer.comm is not None:
        assert model.transformer.comm.status() == 0
        model.transformer.comm.close()


@pytest.mark.parametrize("local_exchange", [False, True])
def test_cuda_graph_decode_equals_eager(cuda, local_exchange):
    cfg = tiny_config(256, 2)
    model = build(cfg, cuda, local_exchange=local_exchange)
    gen = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (1, 7), generator=gen).to(cuda)
    eager = model.generate(ids, max_length=7 + 40, cg=False, return_dict_in_generate=True, output_scores=True)
    graph = model.generate(ids, max_length=7 + 40, cg=True, return_dict_in_generate=True, output_scores=True)
    again = model.generate(ids, max_length=7 + 40, cg=True, return_dict_in_generate=True, output_scores=True)
    assert torch.equal(eager.sequences, graph.sequences)
    assert torch.equal(graph.sequences, again.sequences)
    for a, b in zip(eager.scores, graph.scores):
        assert torch.equal(a, b), "graph replay must reproduce the eager step bit for bit"
    if local_exchange:
        # the exchange path computes the same function as the plain path: same logits within fp16 rounding for
        # as long as both have decoded the same tokens (a near-tie may then send them different ways)
        plain = build(cfg, cuda).generate(ids, max_length=7 + 40, cg=False, return_dict_in_generate=True,
                                          output_scores=True)
        same = 0
        for t, (a, b) in enumerate(zip(plain.scores, eager.scores)):
            if not torch.equal(plain.sequences[0, :7 + t], eager.sequences[0, :7 + t]):
                break
            assert torch.allclose(a.float(), b.float(), atol=3e-2, rtol=3e-2), f"step {t}"
            same += 1
        assert same >= 3
        assert model.transformer.comm.status() == 0
        del model._decoding_cache
        model.transformer.comm.close()


@pytest.mark.parametrize("B", [2, 4, 18])
def test_cuda_graph_batched_decode_equals_eager(cuda, B):
    """A batch decodes through the batch entry points (one state, plain launches): the captured graph replays the
    eager step bit for bit, and a second generation on the same model starts from a clean state."""
    cfg = tiny_config(256, 2)
    model = build(cfg, cuda)
    gen = torch.Generator().manual_seed(B)
    ids = torch.randint(0, cfg.vocab_size, (B, 7), generator=gen).to(cuda)
    eager = model.generate(ids, max_length=7 + 36, cg=False, return_dict_in_generate=True, output_scores=True)
    graph = model.generate(ids, max_length=7 + 36, cg=True, return_dict_in_generate=True, output_scores=True)
    again = model.generate(ids, max_length=7 + 36, cg=True, return_dict_in_generate=True, output_scores=True)
    assert eager.sequences.shape == (B, 7 + 36)
    assert torch.equal(eager.sequences, graph.sequences)
    assert torch.equal(graph.sequences, again.sequences)
    for a, b in zip(eager.scores, graph.scores):
        assert torch.equal(a, b), "graph replay must reproduce the eager step bit for bit"
    for m in model.transformer.layers:
        assert m.mixer.decode_status() == 0


def test_state_dict_keys_follow_the_reference(cuda):
    cfg = tiny_config(256, 2, n_layer=2)
    model = build(cfg, cuda)
    keys = set(model.state_dict().keys())
    for k in ("transformer.embeddings.word_embeddings.weight", "transformer.embeddings.position_embeddings.weight",
              "transformer.layers.0.mixer.Wqkv.weight", "transformer.layers.0.mixer.Wqkv.bias",
              "transformer.layers.0.mixer.out_proj.weight", "transformer.layers.0.mixer.out_proj.bias",
              "transformer.layers.1.mixer.sp.fc0.weight", "transformer.layers.1.mixer.sp.fc1.weight",
              "transformer.layers.0.mlp.fc1.weight", "transformer.layers.0.mlp.fc1.bias",
              "transformer.layers.0.mlp.fc2.weight", "transformer.layers.0.mlp.fc2.bias",
              "transformer.layers.1.mlp.sp.fc0.weight", "transformer.layers.1.mlp.sp.fc1.weight",
              "transformer.layers.0.norm1.weight", "transformer.layers.1.norm2.bias", "transformer.ln_f.weight",
              "lm_head.weight"):
        assert k in keys, k
    sd = model.state_dict()
    assert sd["transformer.layers.0.mlp.fc2.weight"].shape == (256, 1024)
    assert sd["transformer.layers.0.mixer.Wqkv.weight"].shape == (768, 256)
    assert model.transformer.layers[0].mixer.mlp_k == 256 and model.transformer.layers[0].mixer.att_k == 2
