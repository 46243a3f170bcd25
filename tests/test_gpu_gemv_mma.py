"""The warp-MMA GEMV (htr_linear with up to four activation rows; hash words as int8 mma.sync fragments) forced for every
call it can serve: parity with the CPU oracle and with the CUDA-core GEMV, through the same entry points.

The kernel works in exact integers (hash bytes x byte planes of the activations, s32 accumulators), so beyond the tolerances
of tests/test_gpu_parity.py it must be bit-stable from run to run and must agree with the CUDA-core GEMV to float32 rounding.
  float32 activations/outputs: norm-relative error <= 1e-5 against the oracle, <= 2e-6 against the CUDA-core GEMV
  bf16 outputs:                the tolerances of tests/test_gpu_parity.py
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

WIDTHS = (2, 3, 4, 5, 6, 8)


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def warp_mma_gemv():
    from htr_b200 import _lib

    _lib.lib.htr_set_gemv_kernel(1)
    yield
    _lib.lib.htr_set_gemv_kernel(-1)


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def check_bf16(y, ref):
    y = y.float().cpu().numpy()
    assert rel(y, ref) <= 4e-3
    rms = float(np.sqrt(np.mean(np.square(ref))))
    assert np.all(np.abs(y - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-2 * rms)


def cuda_core(fn):
    """The same call on the CUDA-core GEMV."""
    from htr_b200 import _lib

    _lib.lib.htr_set_gemv_kernel(0)
    try:
        return fn()
    finally:
        _lib.lib.htr_set_gemv_kernel(1)


@pytest.mark.parametrize("K", (2, 3, 4, 5))
def test_reference_outputs(golden, dev, K):
    """fixtures computed by the reference: x.float() @ wire.dequant(...).T, 256 x 384, up to three activation rows"""
    from htr_b200 import ops

    g = golden(f"linear_K{K}")
    qw, sc, su, sv = [torch.from_numpy(g[k]).to(dev) for k in ("qweight", "scales", "su", "sv")]
    x = torch.from_numpy(g["x_f32"]).to(dev)
    for rows in (1, 2, 3):
        assert rel(ops.linear(x[:rows], qw, sc, su, sv).cpu().numpy(), g["y"][:rows]) <= 1e-5
        check_bf16(ops.linear(x[:rows].bfloat16(), qw, sc, su, sv), g["y"][:rows])
    bias = torch.from_numpy(g["bias_f32"]).to(dev)
    assert rel(ops.linear(x, qw, sc, su, sv, bias).cpu().numpy(), g["y_bias"]) <= 1e-5


@pytest.mark.parametrize("K", WIDTHS)
@pytest.mark.parametrize("m,n,M", ((128, 128, 1), (128, 1280, 4), (384, 2048, 2), (1024, 256, 3), (256, 4096, 1), (256, 3200, 4)))
def test_shapes_against_oracle(coracle, dev, K, m, n, M):
    from htr_b200 import ops, wire

    qw, sc, su, sv = wire.random_packed(m, n, K, seed=11 * K + m + n + M)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, n, generator=g)
    bias = torch.randn(m, generator=g)
    ref = coracle.linear(x.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy(), bias=bias.numpy())
    args = [t.to(dev) for t in (qw, sc, su, sv)]
    assert rel(ops.linear(x.to(dev), *args, bias.to(dev)).cpu().numpy(), ref) <= 1e-5
    xb = x.bfloat16()
    check_bf16(ops.linear(xb.to(dev), *args), coracle.linear(xb.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy()))
    xh = x.half()
    yh = ops.linear(xh.to(dev), *args)
    assert yh.dtype == torch.float16
    assert rel(yh.float().cpu().numpy(), coracle.linear(xh.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())) <= 1e-3


@pytest.mark.parametrize("K,m,n", ((4, 4096, 12288), (3, 12288, 4096), (2, 4096, 4096), (5, 20480, 1024)))
@pytest.mark.parametrize("M", (1, 4))
def test_full_sizes_bit_stable_and_close_to_cuda_core(dev, K, m, n, M):
    """Benchmark shapes (split and flat decompositions, several windows of activations per CTA): run-to-run bit stability,
    agreement with the CUDA-core GEMV, independence of 128-row blocks."""
    from htr_b200 import ops, wire

    args = wire.random_packed(m, n, K, 2000 + K, dev)
    x = torch.randn(M, n, generator=torch.Generator().manual_seed(K)).to(dev)
    y = ops.linear(x, *args)
    for _ in range(4):
        assert torch.equal(ops.linear(x, *args), y)
    ref = cuda_core(lambda: ops.linear(x, *args))
    assert rel(y.cpu().numpy(), ref.cpu().numpy()) <= 2e-6
    qw, sc, su, sv = args
    lo, hi = m // 128 // 3 * 128, m // 128 // 3 * 128 + 256
    ysl = ops.linear(x, qw[lo // 16:hi // 16].contiguous(), sc[lo:hi].contiguous(), su, sv[lo // 8:hi // 8].contiguous())
    assert rel(ysl.cpu().numpy(), y[:, lo:hi].cpu().numpy()) <= 2e-6


def test_activation_ranges(coracle, dev):
    """The planes are cut around a power-of-two scale per window of columns: rows of very different magnitude, a row of
    zeros, one huge outlier, and tiny values next to large ones must all keep float32 accuracy."""
    from htr_b200 import ops, wire

    m, n, K = 256, 2048, 4
    qw, sc, su, sv = wire.random_packed(m, n, K, seed=5)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(4, n, generator=g)
    x[0] *= 1e-20
    x[1] = 0
    x[2, 100] = 3e8
    x[3, ::2] *= 1e-6
    x[3, 1::2] *= 1e4
    ref = coracle.linear(x.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    y = ops.linear(x.to(dev), *[t.to(dev) for t in (qw, sc, su, sv)]).cpu().numpy()
    for r in (0, 2, 3):
        assert rel(y[r], ref[r]) <= 1e-5
    assert np.all(y[1] == 0)


def test_non_finite_activations_give_non_finite_rows(dev):
    from htr_b200 import ops, wire

    args = wire.random_packed(128, 256, 4, 3, dev)
    x = torch.randn(2, 256, device=dev)
    x[1, 17] = float("inf")
    y = ops.linear(x, *args)
    assert torch.isfinite(y[0]).all() and not torch.isfinite(y[1]).any()
    x[1, 17] = float("nan")
    y = ops.linear(x, *args)
    assert torch.isfinite(y[0]).all() and torch.isnan(y[1]).all()


def test_padded_and_fused_forms_agree_with_cuda_core(dev):
    """The other entry points that share the kernel: missing input columns / dropped output rows, RMSNorm and SwiGLU prologues,
    residual epilogue (bf16: both kernels reproduce the same roundings of the unfused operators, so they may differ by one
    bf16 step where a float32 sum sits next to a rounding boundary)."""
    from htr_b200 import ops, wire

    m, n, K = 384, 512, 3
    args = wire.random_packed(m, n, K, 21, dev)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 336, generator=g).to(dev)
    a = ops.linear_padded(x, *args, m_out=344)
    b = cuda_core(lambda: ops.linear_padded(x, *args, m_out=344))
    assert tuple(a.shape) == (2, 344) and rel(a.cpu().numpy(), b.cpu().numpy()) <= 2e-6

    xb = torch.randn(3, n, generator=g).bfloat16().to(dev)
    w = (1 + 0.1 * torch.randn(n, generator=g)).bfloat16().to(dev)
    a = ops.linear_fused(xb, *args, prologue=ops.PROLOGUE_RMSNORM, norm_weight=w, eps=1e-6)
    b = cuda_core(lambda: ops.linear_fused(xb, *args, prologue=ops.PROLOGUE_RMSNORM, norm_weight=w, eps=1e-6))
    assert rel(a.float().cpu().numpy(), b.float().cpu().numpy()) <= 2e-3
    gu = torch.randn(3, 2 * n, generator=g).bfloat16().to(dev)
    res = torch.randn(3, m, generator=g).bfloat16().to(dev)
    ra, rb = res.clone(), res.clone()
    ops.linear_fused(gu, *args, out=ra, prologue=ops.PROLOGUE_SWIGLU, residual=True)
    cuda_core(lambda: ops.linear_fused(gu, *args, out=rb, prologue=ops.PROLOGUE_SWIGLU, residual=True))
    assert rel(ra.float().cpu().numpy(), rb.float().cpu().numpy()) <= 2e-3


def test_plan_and_workspace_cover_both_kernels(dev):
    from htr_b200 import _lib

    grid, slots = ctypes.c_int(0), ctypes.c_int(0)
    for (M, m, n, K) in ((1, 4096, 12288, 4), (4, 151936, 4096, 4), (2, 128, 128, 2)):
        assert _lib.lib.htr_linear_plan(M, m, n, K, ctypes.byref(grid), ctypes.byref(slots)) == 0
        need = _lib.lib.htr_linear_workspace_bytes(M, m, n, K)
        rows_t = 1 if M <= 1 else 2 if M <= 2 else 4
        assert need >= _lib.lib.htr_linear_counter_bytes(m) + (m // 128) * slots.value * rows_t * 128 * 4
        assert 1 <= grid.value <= 3 * torch.cuda.get_device_properties(dev).multi_processor_count


@pytest.mark.parametrize("K,m,n", ((4, 20480, 4096), (3, 4096, 12288), (2, 2560, 1024), (5, 37888, 2048)))
@pytest.mark.parametrize("M", (1, 2))
def test_exact_sums_do_not_depend_on_the_launch_decomposition(coracle, dev, K, m, n, M):
    """HTR_LINEAR_EXACT_SUMS (ops.exact_sums): one scale per activation row and 64-bit integer sums across windows and thread
    blocks.  A run of row blocks cut out of the weight is launched with another grid and other column splits, and must still
    reproduce its rows of the full result bit for bit (what row sharding over several GPUs relies on); accuracy as usual."""
    from htr_b200 import ops, wire

    qw, sc, su, sv = wire.random_packed(m, n, K, 4000 + K)
    args = [t.to(dev) for t in (qw, sc, su, sv)]
    x = torch.randn(M, n, generator=torch.Generator().manual_seed(K + M))
    x[0, 5] = 37.0                                               # an outlier: the row scale follows a bound on the whole row
    with ops.exact_sums():
        y = ops.linear(x.to(dev), *args)
        yb = ops.linear(x.bfloat16().to(dev), *args)
        for lo, hi in ((0, 128), (m // 128 // 3 * 128, m // 128 // 3 * 128 + 896), (m - 384, m)):
            part = [args[0][lo // 16:hi // 16].contiguous(), args[1][lo:hi].contiguous(), args[2], args[3][lo // 8:hi // 8].contiguous()]
            assert torch.equal(ops.linear(x.to(dev), *part), y[:, lo:hi])
            assert torch.equal(ops.linear(x.bfloat16().to(dev), *part), yb[:, lo:hi])
    ref = coracle.linear(x.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    assert rel(y.cpu().numpy(), ref) <= 1e-5
    check_bf16(yb, coracle.linear(x.bfloat16().float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy()))


def test_exact_sums_hold_at_the_bound_of_the_row_scale(coracle, dev):
    """The exact form scales a row by a bound on its transform, 128 max|x|.  An input that meets it (su * x constant: the first
    output of every 128-column block is 128 times that constant) must not overflow the integer grid."""
    from htr_b200 import ops, wire

    m, n, K = 256, 2048, 4
    qw, sc, su, sv = wire.random_packed(m, n, K, seed=5)
    signs = 1.0 - 2.0 * torch.from_numpy(np.unpackbits(su.numpy(), bitorder="little").astype(np.float32))
    x = (1.75 * signs).reshape(1, n)
    ref = coracle.linear(x.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    with ops.exact_sums():
        y = ops.linear(x.to(dev), *[t.to(dev) for t in (qw, sc, su, sv)]).cpu().numpy()
    assert rel(y, ref) <= 1e-5
