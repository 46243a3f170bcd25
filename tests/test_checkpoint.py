"""Packed checkpoints: the on-disk layout of the reference's converter (htr/quantize.py:252-289) written synthetically,
then read back through the plugin's method selection and weight loaders (htr/vllm_plugin.py:40-125) into the decoder."""
import json
import os

import pytest
import torch

vllm = pytest.importorskip("vllm")


def tiny_config():
    from htr_b200.decoder import DecoderConfig

    return DecoderConfig(layers=2, hidden=256, q_heads=2, kv_heads=1, head_dim=128, intermediate=384, vocab=512, K=3, K_head=4, max_len=64)


def same_weights(a, b):
    for la, lb in zip(a.layers, b.layers):
        for key in ("qkv", "o", "gate_up", "down"):
            assert all(torch.equal(x.cpu(), y.cpu()) for x, y in zip(la[key], lb[key])), key
        assert torch.equal(la["ln1"].cpu(), lb["ln1"].cpu()) and torch.equal(la["ln2"].cpu(), lb["ln2"].cpu())
    assert all(torch.equal(x.cpu(), y.cpu()) for x, y in zip(a.head, b.head))
    assert torch.equal(a.embed.cpu(), b.embed.cpu()) and torch.equal(a.ln_f.cpu(), b.ln_f.cpu())


def test_checkpoint_layout_and_round_trip(tmp_path):
    from htr_b200 import checkpoint
    from htr_b200.decoder import PackedDecoder

    cpu = torch.device("cpu")
    model = PackedDecoder(tiny_config(), cpu, seed=3)
    model.layers[1]["ln1"].mul_(1.5)                                        # something other than ones in a norm
    out = str(tmp_path / "ckpt")
    weight_map = model.export_checkpoint(out, shards=3)
    # layout: shards + index + config with the converter's quantization_config
    files = sorted(os.listdir(out))
    assert files == ["config.json", "model-00001-of-00003.safetensors", "model-00002-of-00003.safetensors",
                     "model-00003-of-00003.safetensors", "model.safetensors.index.json"]
    qc = checkpoint.read_config(out)["quantization_config"]
    assert (qc["quant_method"], qc["wire"], qc["generator"], qc["L"], qc["tile"], qc["rht_block"]) == ("htr", "HTR-W1", "rdna24", 16, 16, 128)
    assert qc["modules"]["model.layers.0.self_attn.k_proj"] == {"K": 3} and qc["modules"]["lm_head"] == {"K": 4}
    assert len(qc["modules"]) == 2 * 7 + 1
    assert "model.layers.1.mlp.up_proj.htr_qweight" in weight_map and "model.layers.1.mlp.gate_up_proj.htr_qweight" not in weight_map
    names = dict(checkpoint.iter_tensors(out))
    assert tuple(names["model.layers.0.self_attn.q_proj.htr_qweight"].shape) == (16, 16, 24)
    assert tuple(names["model.layers.0.self_attn.v_proj.htr_sv"].shape) == (16,)
    assert torch.equal(names["model.layers.0.self_attn.q_proj.htr_su"], names["model.layers.0.self_attn.v_proj.htr_su"])
    # back through HTRConfig / HTRLinearMethod / weight loaders
    loaded = PackedDecoder.from_checkpoint(out, cpu)
    assert (loaded.cfg.K, loaded.cfg.K_head, loaded.cfg.layers, loaded.cfg.intermediate) == (3, 4, 2, 384)
    same_weights(model, loaded)


def test_loader_rejects_bad_checkpoints(tmp_path):
    from htr_b200 import checkpoint
    from htr_b200.decoder import PackedDecoder
    from safetensors.torch import load_file, save_file

    cpu = torch.device("cpu")
    model = PackedDecoder(tiny_config(), cpu, seed=4)
    out = str(tmp_path / "ckpt")
    model.export_checkpoint(out, shards=1)
    shard = os.path.join(out, "model-00001-of-00001.safetensors")
    tensors = {k: v.clone() for k, v in load_file(shard).items()}          # the file is rewritten below
    # members of a fused module must share the input signs (docs/FORMAT.md:31-32)
    broken = dict(tensors)
    broken["model.layers.0.self_attn.k_proj.htr_su"] = tensors["model.layers.0.self_attn.k_proj.htr_su"] ^ 1
    save_file(broken, shard, metadata={"format": "pt"})
    with pytest.raises(ValueError):
        PackedDecoder.from_checkpoint(out, cpu)
    # a tensor nobody owns
    broken = dict(tensors)
    broken["model.layers.0.self_attn.w_proj.htr_su"] = tensors["model.layers.0.self_attn.k_proj.htr_su"].clone()
    save_file(broken, shard, metadata={"format": "pt"})
    index = os.path.join(out, "model.safetensors.index.json")
    idx = json.load(open(index))
    idx["weight_map"]["model.layers.0.self_attn.w_proj.htr_su"] = "model-00001-of-00001.safetensors"
    json.dump(idx, open(index, "w"))
    with pytest.raises(KeyError):
        PackedDecoder.from_checkpoint(out, cpu)
    # mixed widths inside a fused module are refused by the method selection (htr/vllm_plugin.py:60-63)
    save_file(tensors, shard, metadata={"format": "pt"})
    del idx["weight_map"]["model.layers.0.self_attn.w_proj.htr_su"]
    json.dump(idx, open(index, "w"))
    cfg = checkpoint.read_config(out)
    cfg["quantization_config"]["modules"]["model.layers.0.mlp.up_proj"] = {"K": 4}
    json.dump(cfg, open(os.path.join(out, "config.json"), "w"))
    with pytest.raises(ValueError):
        PackedDecoder.from_checkpoint(out, cpu)


@pytest.mark.gpu
def test_loaded_checkpoint_decodes_like_the_source_model(tmp_path):
    from htr_b200.decoder import PackedDecoder

    dev = torch.device("cuda:0")
    model = PackedDecoder(tiny_config(), dev, seed=5)
    out = str(tmp_path / "ckpt")
    model.export_checkpoint(out)
    loaded = PackedDecoder.from_checkpoint(out, dev)
    same_weights(model, loaded)
    prompt = torch.randint(0, 512, (8,), generator=torch.Generator().manual_seed(6))
    a, _, _ = model.generate(prompt, 12)
    b, _, _ = loaded.generate(prompt, 12)
    assert torch.equal(a, b)
    ids, pos = prompt.to(dev), torch.arange(8, device=dev)
    assert torch.equal(model.forward(ids, pos), loaded.forward(ids, pos))
