"""Checkpoint remap / tensor-parallel shard / predictor loading, on CPU, against Hugging Face's OPT itself."""
import os

import pytest
import torch


def tiny_hf_opt():
    from transformers import OPTConfig, OPTForCausalLM

    cfg = OPTConfig(vocab_size=90, hidden_size=64, num_hidden_layers=2, ffn_dim=256, num_attention_heads=4,
                    max_position_embeddings=32, word_embed_proj_dim=64, do_layer_norm_before=True,
                    activation_function="relu", dropout=0.0)
    torch.manual_seed(0)
    return cfg, OPTForCausalLM(cfg).eval()


def my_config(world=1):
    from dejavu_b200.gpt import apply_sparsity_knobs, opt_config

    cfg = opt_config("opt-125m", n_layer=2, num_hidden_layers=2, n_embd=64, hidden_size=64, n_head=4, n_inner=256,
                     vocab_size=90, max_position_embeddings=32, n_positions=32, mlp_sp_dim=16, att_sp_dim=8)
    return apply_sparsity_knobs(cfg, 64, 2, 2, world)


def test_remapped_hf_checkpoint_reproduces_hf_logits():
    from dejavu_b200.checkpoint import remap_state_dict_opt
    from dejavu_b200.gpt import GPTLMHeadModel

    hf_cfg, hf = tiny_hf_opt()
    cfg = my_config()
    model = GPTLMHeadModel(cfg, device="cpu", dtype=torch.float32).eval().init_random(1)
    sd = remap_state_dict_opt(hf.state_dict(), cfg)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all(".sp." in k for k in missing), missing  # only the predictors are not part of an OPT checkpoint
    ids = torch.arange(13).remainder(90)[None]
    with torch.inference_mode():
        want = hf(ids).logits
        got = model(ids).logits[..., :90]
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), (got - want).abs().max()
    # fc2 is stored transposed internally but presents the reference shape
    assert model.state_dict()["transformer.layers.0.mlp.fc2.weight"].shape == (64, 256)
    assert torch.equal(model.transformer.layers[0].mlp.fc2_weight_t, hf.model.decoder.layers[0].fc2.weight.t())


def test_shards_concatenate_back_to_the_full_checkpoint():
    from dejavu_b200.checkpoint import remap_state_dict_opt, shard_state_dict_tp

    _, hf = tiny_hf_opt()
    cfg = my_config(world=2)
    full = remap_state_dict_opt(hf.state_dict(), cfg)
    s0, s1 = (shard_state_dict_tp(full, cfg, 2, r) for r in (0, 1))
    p = "transformer.layers.1."
    assert torch.equal(torch.cat([s0[p + "mlp.fc1.weight"], s1[p + "mlp.fc1.weight"]]), full[p + "mlp.fc1.weight"])
    assert torch.equal(torch.cat([s0[p + "mlp.fc2.weight"], s1[p + "mlp.fc2.weight"]], 1), full[p + "mlp.fc2.weight"])
    assert torch.equal(torch.cat([s0[p + "mixer.out_proj.weight"], s1[p + "mixer.out_proj.weight"]], 1),
                       full[p + "mixer.out_proj.weight"])
    w = full[p + "mixer.Wqkv.weight"].view(3, 4, 16, 64)
    assert torch.equal(s1[p + "mixer.Wqkv.weight"], w[:, 2:].reshape(96, 64))
    assert p + "mlp.fc2.bias" in s0 and p + "mlp.fc2.bias" not in s1
    assert p + "mixer.out_proj.bias" in s0 and p + "mixer.out_proj.bias" not in s1
    assert s0["lm_head.weight"].shape == (48, 64) and torch.equal(s0["transformer.ln_f.weight"], full["transformer.ln_f.weight"])
    assert torch.equal(s1["transformer.embeddings.position_embeddings.weight"],
                       hf.model.decoder.embed_positions.weight[2:])


def test_load_predictors_from_trainer_files(tmp_path):
    from dejavu_b200.checkpoint import load_predictors
    from dejavu_b200.gpt import GPTLMHeadModel

    cfg = my_config()
    model = GPTLMHeadModel(cfg, device="cpu", dtype=torch.float32).eval().init_random(2)
    g = torch.Generator().manual_seed(3)
    files = {}
    for i in range(2):
        files[f"c4_layer{i}_best.pt"] = {"0.weight": torch.randn(16, 64, generator=g), "1.weight": torch.randn(256, 16, generator=g)}
    files["c4_att_layer1_x.pt"] = {"0.weight": torch.randn(8, 64, generator=g), "1.weight": torch.randn(4, 8, generator=g)}
    files["c4_layer10_other.pt"] = {"0.weight": torch.zeros(16, 64), "1.weight": torch.zeros(256, 16)}  # not layer 1
    for name, sd in files.items():
        torch.save(sd, os.path.join(tmp_path, name))
    loaded = load_predictors(model, str(tmp_path))
    assert loaded == {"mlp": [0, 1], "att": [1]}
    assert torch.equal(model.transformer.layers[1].mlp.sp.fc1.weight, files["c4_layer1_best.pt"]["1.weight"])
    assert torch.equal(model.transformer.layers[1].mixer.sp.fc0.weight, files["c4_att_layer1_x.pt"]["0.weight"])
    with pytest.raises(FileNotFoundError):
        load_predictors(model, str(tmp_path), strict=True)  # attention predictor of layer 0 is missing
