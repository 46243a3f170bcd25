"""Packed checkpoints on disk: the layout the reference's converter writes, read back through the plugin's weight loaders.

On-disk layout (htr/quantize.py:252-289 of the reference; docs/FORMAT.md:25-36): safetensors shards
`model-0000i-of-0000N.safetensors` + `model.safetensors.index.json` (`weight_map`: tensor name -> shard file); every
replaced `<module>.weight` is stored as the four tensors `<module>.htr_qweight / .htr_scales / .htr_su / .htr_sv`;
`config.json` carries `quantization_config = {"quant_method": "htr", "wire": "HTR-W1", "generator": "rdna24", "L": 16,
"tile": 16, "rht_block": 128, "modules": {<module>: {"K": k}}}`.  Fused modules (q|k|v, gate|up) are stored per member
and share the input sign vector; the loaders place them by rows (htr/vllm_plugin.py:67-125).

`write_checkpoint` exists because no packed checkpoint can be downloaded here: it writes synthetic ones in exactly that
layout.  `load_checkpoint` does what a serving stack's weight loading does for these tensors: it walks the index, maps a
member name to its fused parameter and shard id, and calls the parameter's `weight_loader`.
"""
import json
import os

import torch
from safetensors import safe_open
from safetensors.torch import save_file

SUFFIXES = (".htr_qweight", ".htr_scales", ".htr_su", ".htr_sv")

# member module -> (fused module, shard id), as the model code of a decoder-only transformer stacks them
STACKED = {"q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
           "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}


def quantization_config(widths):
    """`widths`: {module name: K}.  The dictionary the reference's converter stores in config.json (htr/quantize.py:281-283)."""
    return {"quant_method": "htr", "wire": "HTR-W1", "generator": "rdna24", "L": 16, "tile": 16, "rht_block": 128,
            "modules": {name: {"K": int(k)} for name, k in widths.items()}}


def write_checkpoint(out_dir, packed, plain, config, shards=2):
    """packed: {module name: (qweight, scales, su, sv)}; plain: {tensor name: tensor} (embeddings, norms);
    config: the model's config.json content without quantization_config.  Tensors are dealt to `shards` files in name order."""
    os.makedirs(out_dir, exist_ok=True)
    tensors, widths = {}, {}
    for name, (qw, sc, su, sv) in packed.items():
        widths[name] = qw.shape[-1] // 8
        for suffix, t in zip(SUFFIXES, (qw, sc, su, sv)):
            tensors[name + suffix] = t.detach().cpu().contiguous().clone()   # members of a fused module arrive as views
    for name, t in plain.items():
        tensors[name] = t.detach().cpu().contiguous()
    names = sorted(tensors)
    weight_map, total = {}, 0
    for i in range(shards):
        fname = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        part = {k: tensors[k] for k in names[i::shards]}
        save_file(part, os.path.join(out_dir, fname), metadata={"format": "pt"})
        for k, v in part.items():
            weight_map[k] = fname
            total += v.numel() * v.element_size()
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    cfg = dict(config)
    cfg["quantization_config"] = quantization_config(widths)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return weight_map


def read_config(ckpt_dir):
    with open(os.path.join(ckpt_dir, "config.json")) as f:
        return json.load(f)


def iter_tensors(ckpt_dir):
    """(name, tensor) for every tensor of the checkpoint, shard by shard (each file is opened once)."""
    with open(os.path.join(ckpt_dir, "model.safetensors.index.json")) as f:
        weight_map = json.load(f)["weight_map"]
    by_file = {}
    for name, fname in weight_map.items():
        by_file.setdefault(fname, []).append(name)
    for fname in sorted(by_file):
        with safe_open(os.path.join(ckpt_dir, fname), "pt", device="cpu") as fh:
            for name in sorted(by_file[fname]):
                yield name, fh.get_tensor(name)


def load_checkpoint(ckpt_dir, params, stacked=STACKED):
    """Feeds every tensor of the checkpoint to its parameter.

    params: {parameter name: torch Parameter}, named as the model owns them (fused modules under their fused name, e.g.
    `model.layers.0.self_attn.qkv_proj.htr_qweight`).  A checkpoint tensor of a member (`…q_proj.htr_qweight`) goes to the
    fused parameter's `weight_loader(param, tensor, shard_id)`; other tensors to `weight_loader(param, tensor)` or a plain
    copy.  Returns the set of parameter names that received data; unknown tensors raise KeyError."""
    loaded = set()
    for name, tensor in iter_tensors(ckpt_dir):
        target, shard_id = name, None
        module, _, leaf = name.rpartition(".")
        parent, _, member = module.rpartition(".")
        if member in stacked:
            fused, shard_id = stacked[member]
            target = f"{parent}.{fused}.{leaf}" if parent else f"{fused}.{leaf}"
        if target not in params:
            raise KeyError(f"checkpoint tensor {name} has no parameter {target}")
        par = params[target]
        loader = getattr(par, "weight_loader", None)
        if loader is None:
            assert par.shape == tensor.shape, (target, tuple(par.shape), tuple(tensor.shape))
            par.data.copy_(tensor)
        elif shard_id is None:
            loader(par, tensor)
        else:
            loader(par, tensor, shard_id)
        loaded.add(target)
    return loaded
