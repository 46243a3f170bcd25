"""The tensor-core packed GEMM (five or more activation rows by default) against the CPU oracle.  Activations reach the MMA as two
fp16 planes (hi + lo), so float32 inputs are reproduced to ~1e-5 and bf16 outputs to their rounding:
  float32 in/out: norm-relative error <= 5e-5;  bf16 / fp16: <= 4e-3 norm-relative (the tolerances of the GEMV tests,
  the float32 one widened for the fp16-split activations)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


@pytest.mark.parametrize("K", (2, 3, 4, 5, 6, 8))
@pytest.mark.parametrize("m,n,M", ((128, 128, 16), (256, 1024, 9), (384, 512, 33), (128, 2048, 64), (512, 256, 128), (256, 384, 100), (256, 256, 256), (128, 640, 200), (128, 256, 300), (256, 1024, 5), (128, 2048, 8)))
def test_gemm_matches_oracle(coracle, K, m, n, M):
    from htr_b200 import ops, wire

    dev = torch.device("cuda:0")
    qw, sc, su, sv = wire.random_packed(m, n, K, seed=3 * K + m + n + M)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, n, generator=g)
    x[0, :7] *= 300.0                                                       # outliers exercise the per-row range scale
    bias = torch.randn(m, generator=g)
    ref = coracle.linear(x.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy(), bias=bias.numpy())
    y = ops.linear(x.to(dev), qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev), bias.to(dev))
    assert ops.gemm_error_codes() and all(c == 0 for c in ops.gemm_error_codes())
    assert tuple(y.shape) == (M, m)
    assert rel(y.cpu().numpy(), ref) <= 5e-5
    xb = x.bfloat16()
    refb = coracle.linear(xb.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    yb = ops.linear(xb.to(dev), qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev))
    assert yb.dtype == torch.bfloat16 and rel(yb.float().cpu().numpy(), refb) <= 4e-3


@pytest.mark.parametrize("K,m,n,M", ((4, 20480, 512, 64), (3, 12288, 1024, 100), (5, 24576, 256, 16)))
def test_gemm_tall_matrices(coracle, K, m, n, M):
    """Tall matrices: more row blocks than resident CTAs (the grid runs in more than one wave)."""
    from htr_b200 import ops, wire

    dev = torch.device("cuda:0")
    qw, sc, su, sv = wire.random_packed(m, n, K, seed=K + M)
    x = torch.randn(M, n, generator=torch.Generator().manual_seed(M)).bfloat16()
    ref = coracle.linear(x.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    d = [t.to(dev) for t in (qw, sc, su, sv)]
    y = ops.linear(x.to(dev), *d)
    assert rel(y.float().cpu().numpy(), ref) <= 4e-3
    assert torch.equal(ops.linear(x.to(dev), *d), y) and all(c == 0 for c in ops.gemm_error_codes())
    yf = ops.linear(x.float().to(dev), *d)
    assert rel(yf.cpu().numpy(), ref) <= 5e-5


def test_gemm_full_size_and_bit_stability(coracle):
    from htr_b200 import ops, wire

    dev = torch.device("cuda:0")
    m, n, K, M = 4096, 12288, 4, 64
    qw, sc, su, sv = wire.random_packed(m, n, K, seed=21)
    x = torch.randn(M, n, generator=torch.Generator().manual_seed(5)).bfloat16()
    d = [t.to(dev) for t in (qw, sc, su, sv)]
    y = ops.linear(x.to(dev), *d)
    ref = coracle.linear(x[:2].float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    assert rel(y[:2].float().cpu().numpy(), ref) <= 4e-3
    for _ in range(3):
        assert torch.equal(ops.linear(x.to(dev), *d), y)
    # the batch-1 GEMV and the GEMM agree on the same row
    y1 = ops.linear(x[:1].to(dev), *d)
    assert rel(y1.float().cpu().numpy(), y[:1].float().cpu().numpy()) <= 4e-3
    assert all(c == 0 for c in ops.gemm_error_codes())
