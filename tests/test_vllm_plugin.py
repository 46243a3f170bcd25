"""Host-side behaviour of the vLLM quantization method: config parsing, module selection, parameter creation and
the shard loaders (reference behaviour: htr/vllm_plugin.py:14-138).  The GPU case runs apply() against the oracle."""
import numpy as np
import pytest
import torch

vllm = pytest.importorskip("vllm")


@pytest.fixture(scope="module")
def P():
    from htr_b200 import vllm_plugin

    return vllm_plugin


def test_canon_and_shard_ranges(P):
    assert P.canon("model.layers.3.mlp.down_proj.weight") == "layers.3.mlp.down_proj"
    assert P.canon("lm_head.weight") == "lm_head"
    sizes = [4096, 1024, 1024]
    assert P._shard_range(sizes, "q", 16) == (0, 256)
    assert P._shard_range(sizes, "k", 16) == (256, 64)
    assert P._shard_range(sizes, "v", 8) == (640, 128)
    assert P._shard_range(sizes, None, 1) == (0, 6144)
    assert P._shard_range(sizes, (1, 2), 1) == (4096, 2048)
    assert P._shard_range([128, 128], 1, 16) == (8, 8)
    with pytest.raises(AssertionError):
        P._shard_range(sizes, (0, 2), 1)


def test_config_registration_and_method_selection(P):
    from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
    from vllm.model_executor.layers.quantization import get_quantization_config

    assert get_quantization_config("htr") is P.HTRConfig
    cfg = P.HTRConfig.from_config({"quant_method": "htr", "wire": "HTR-W1", "modules": {
        "model.layers.0.self_attn.q_proj": {"K": 4}, "model.layers.0.self_attn.k_proj": {"K": 4},
        "model.layers.0.self_attn.v_proj": {"K": 4}, "model.layers.0.mlp.gate_proj": {"K": 3},
        "model.layers.0.mlp.up_proj": {"K": 4}, "model.layers.0.mlp.down_proj.weight": {"K": 5}}})
    assert cfg.get_name() == "htr" and cfg.get_min_capability() == 0
    assert cfg.get_supported_act_dtypes() == [torch.bfloat16, torch.float16]
    cfg.packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}
    lin = LinearBase.__new__(LinearBase)            # only its type matters here
    m = cfg.get_quant_method(lin, "model.layers.0.self_attn.qkv_proj")
    assert isinstance(m, P.HTRLinearMethod) and m.K == 4
    assert cfg.get_quant_method(lin, "model.layers.0.mlp.down_proj").K == 5
    assert isinstance(cfg.get_quant_method(lin, "model.layers.1.mlp.down_proj"), UnquantizedLinearMethod)
    assert isinstance(cfg.get_quant_method(lin, "model.visual.layers.0.mlp.down_proj"), UnquantizedLinearMethod)
    with pytest.raises(ValueError):
        cfg.get_quant_method(lin, "model.layers.0.mlp.gate_up_proj")          # K3 fused with K4
    assert cfg.get_quant_method(torch.nn.LayerNorm(8), "model.layers.0.norm") is None
    with pytest.raises(AssertionError):
        P.HTRConfig({}, wire="HTR-W2")


def test_create_weights_and_shard_loaders(P):
    from htr_b200 import wire

    layer = torch.nn.Module()
    meth = P.HTRLinearMethod(4)
    sizes = [256, 128, 128]
    meth.create_weights(layer, 384, sizes, 384, sum(sizes), torch.bfloat16)
    assert tuple(layer.htr_qweight.shape) == (32, 24, 32) and layer.htr_qweight.dtype == torch.int32
    assert tuple(layer.htr_scales.shape) == (512,) and layer.htr_scales.dtype == torch.float16
    assert tuple(layer.htr_su.shape) == (48,) and tuple(layer.htr_sv.shape) == (64,) and layer.htr_K == 4
    parts = [wire.random_packed(s, 384, 4, seed=i) for i, s in enumerate(sizes)]
    su = parts[0][2]
    for sid, (qw, sc, _, sv) in zip(("q", "k", "v"), parts):
        layer.htr_qweight.weight_loader(layer.htr_qweight, qw, sid)
        layer.htr_scales.weight_loader(layer.htr_scales, sc, sid)
        layer.htr_sv.weight_loader(layer.htr_sv, sv, sid)
        layer.htr_su.weight_loader(layer.htr_su, su, sid)
    assert torch.equal(layer.htr_qweight.data, torch.cat([p[0] for p in parts]))
    assert torch.equal(layer.htr_scales.data, torch.cat([p[1] for p in parts]))
    assert torch.equal(layer.htr_sv.data, torch.cat([p[3] for p in parts]))
    assert torch.equal(layer.htr_su.data, su)
    with pytest.raises(ValueError):
        layer.htr_su.weight_loader(layer.htr_su, parts[1][2], "k")            # a different sign vector
    with pytest.raises(AssertionError):
        layer.htr_qweight.weight_loader(layer.htr_qweight, parts[0][0][:4], "q")   # wrong shard shape
    with pytest.raises(AssertionError):
        meth.create_weights(torch.nn.Module(), 192, [256], 384, 256, torch.bfloat16)   # tensor parallel input split
    with pytest.raises(AssertionError):
        meth.create_weights(torch.nn.Module(), 384, [200], 384, 200, torch.bfloat16)   # not a multiple of 128
    assert P.register() is None


@pytest.mark.gpu
def test_apply_matches_oracle(P, coracle):
    from htr_b200 import wire

    dev = torch.device("cuda:0")
    layer = torch.nn.Module()
    meth = P.HTRLinearMethod(3)
    meth.create_weights(layer, 512, [256, 256], 512, 512, torch.bfloat16)
    a, b = wire.random_packed(256, 512, 3, seed=11), wire.random_packed(256, 512, 3, seed=12)
    for sid, (qw, sc, su, sv) in enumerate((a, b)):
        layer.htr_qweight.weight_loader(layer.htr_qweight, qw, sid)
        layer.htr_scales.weight_loader(layer.htr_scales, sc, sid)
        layer.htr_sv.weight_loader(layer.htr_sv, sv, sid)
        layer.htr_su.weight_loader(layer.htr_su, a[2], sid)
    layer.to(dev)
    x = torch.randn(2, 3, 512, generator=torch.Generator().manual_seed(1)).bfloat16()
    y = meth.apply(layer, x.to(dev))
    assert tuple(y.shape) == (2, 3, 512) and y.dtype == torch.bfloat16
    ref = coracle.linear(x.reshape(6, 512).float().numpy(), layer.htr_qweight.cpu().numpy(), layer.htr_scales.cpu().numpy(),
                         layer.htr_su.cpu().numpy(), layer.htr_sv.cpu().numpy())
    err = np.linalg.norm(y.reshape(6, 512).float().cpu().numpy() - ref) / np.linalg.norm(ref)
    assert err <= 4e-3
