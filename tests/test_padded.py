"""Padded (non-%128) linears: the stored tensors cover a zero-padded matrix, the activations come unpadded and only the first
m_out outputs are kept (reference: HTRHCLinearMethod, htr/vllm_plugin.py:279-326, which pads with F.pad and slices with
.contiguous(); here both are done inside the GEMV).  Oracle: the unpadded call must equal the padded call's slice."""
import numpy as np
import pytest
import torch

vllm = pytest.importorskip("vllm")


@pytest.fixture(autouse=True)
def gemv_up_to_eight_rows(monkeypatch):
    """The padded form runs on the GEMV; keep the unpadded comparison calls of 5..8 rows on the same kernel so that the
    results can be compared bit for bit."""
    from htr_b200 import ops

    monkeypatch.setattr(ops, "GEMV_ROUTE_MAX", 8)


def test_method_creates_padded_parameters_and_checks_spec():
    from htr_b200 import vllm_plugin as P

    spec = {"K": 3, "m": 320, "n": 336, "m_pad": 384, "n_pad": 384}
    meth = P.HTRHCLinearMethod(spec)
    layer = torch.nn.Module()
    meth.create_weights(layer, 336, [336], 336, 336, torch.bfloat16)
    assert tuple(layer.htr_qweight.shape) == (24, 24, 24) and tuple(layer.htr_scales.shape) == (384,)
    assert tuple(layer.htr_su.shape) == (48,) and tuple(layer.htr_sv.shape) == (48,)
    assert tuple(layer.weight.shape) == (336, 336) and layer.weight.dtype == torch.uint8 and layer._htr_weight_carrier
    assert (layer._htr_n, layer._htr_n_pad, layer._htr_m_out, layer._htr_m_pad) == (336, 384, 336, 384)
    good = torch.zeros(24, 24, 24, dtype=torch.int32)
    layer.htr_qweight.weight_loader(layer.htr_qweight, good)
    with pytest.raises(AssertionError):
        layer.htr_qweight.weight_loader(layer.htr_qweight, good, 0)                      # padded modules are never fused
    with pytest.raises(AssertionError):
        layer.htr_qweight.weight_loader(layer.htr_qweight, good[:8])
    with pytest.raises(AssertionError):
        meth.create_weights(torch.nn.Module(), 336, [400], 336, 400, torch.bfloat16)     # wider than the stored matrix
    with pytest.raises(AssertionError):
        meth.create_weights(torch.nn.Module(), 320, [336], 320, 336, torch.bfloat16)     # not the module the spec describes
    with pytest.raises(AssertionError):
        P.HTRHCLinearMethod({"K": 3, "m": 320, "n": 330, "m_pad": 384, "n_pad": 384}).create_weights(
            torch.nn.Module(), 330, [336], 330, 336, torch.bfloat16)                     # widths must be multiples of 8


@pytest.mark.gpu
@pytest.mark.parametrize("K", (2, 3, 4, 5))
@pytest.mark.parametrize("n_in,m_out,n_pad,m_pad,M", ((336, 336, 384, 384, 1), (200, 72, 256, 128, 3), (1000, 520, 1024, 640, 8),
                                                       (384, 384, 384, 384, 2), (8, 8, 128, 128, 1), (4000, 4096, 4096, 4096, 11)))
def test_padded_equals_explicit_padding(coracle, K, n_in, m_out, n_pad, m_pad, M):
    from htr_b200 import ops, wire

    dev = torch.device("cuda:0")
    qw, sc, su, sv = wire.random_packed(m_pad, n_pad, K, seed=K * 1000 + n_in + m_out)
    g = torch.Generator().manual_seed(n_in + M)
    x = torch.randn(M, n_in, generator=g)
    bias = torch.randn(m_out, generator=g)
    d = [t.to(dev) for t in (qw, sc, su, sv)]
    xp = torch.nn.functional.pad(x, (0, n_pad - n_in))
    ref = coracle.linear(xp.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())[:, :m_out] + bias.numpy()
    y = ops.linear_padded(x.to(dev), *d, bias=bias.to(dev), m_out=m_out)
    assert tuple(y.shape) == (M, m_out) and y.is_contiguous()
    err = np.linalg.norm(y.cpu().numpy() - ref) / np.linalg.norm(ref)
    assert err <= 1e-5
    # the explicit route of the reference (pad, full linear, slice) gives the same numbers from the same kernel
    full = torch.cat([ops.linear(xp[r:r + 8].to(dev), *d) for r in range(0, M, 8)])
    assert torch.equal(y, full[:, :m_out] + bias.to(dev))
    # bf16, no bias, leading dimensions kept
    xb = x.bfloat16().reshape(1, M, n_in)
    yb = ops.linear_padded(xb.to(dev), *d, m_out=m_out)
    assert tuple(yb.shape) == (1, M, m_out) and yb.dtype == torch.bfloat16
    fullb = torch.cat([ops.linear(torch.nn.functional.pad(xb[0, r:r + 8], (0, n_pad - n_in)).to(dev), *d) for r in range(0, M, 8)])
    assert torch.equal(yb[0], fullb[:, :m_out])


@pytest.mark.gpu
def test_padded_method_apply_and_errors():
    from htr_b200 import _lib, ops, wire
    from htr_b200 import vllm_plugin as P

    dev = torch.device("cuda:0")
    spec = {"K": 4, "m": 320, "n": 336, "m_pad": 384, "n_pad": 384}
    meth = P.HTRHCLinearMethod(spec)
    layer = torch.nn.Module()
    meth.create_weights(layer, 336, [336], 336, 336, torch.bfloat16)
    qw, sc, su, sv = wire.random_packed(384, 384, 4, seed=9)
    for name, t in (("htr_qweight", qw), ("htr_scales", sc), ("htr_su", su), ("htr_sv", sv)):
        par = getattr(layer, name)
        par.weight_loader(par, t)
    layer.to(dev)
    x = torch.randn(5, 336, generator=torch.Generator().manual_seed(2)).bfloat16().to(dev)
    y = meth.apply(layer, x)
    want = ops.linear(torch.nn.functional.pad(x, (0, 48)), layer.htr_qweight, layer.htr_scales, layer.htr_su, layer.htr_sv)[:, :336]
    assert tuple(y.shape) == (5, 336) and torch.equal(y, want)
    with pytest.raises(_lib.HTRError):
        ops.linear_padded(x[:, :331].contiguous(), layer.htr_qweight, layer.htr_scales, layer.htr_su, layer.htr_sv, m_out=336)
    with pytest.raises(_lib.HTRError):
        ops.linear_padded(x, layer.htr_qweight, layer.htr_scales, layer.htr_su, layer.htr_sv, m_out=400)
