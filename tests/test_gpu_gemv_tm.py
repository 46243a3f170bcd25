"""The tensor-memory GEMV (htr_linear with up to four activation rows; hash words as the A operand of tcgen05.mma.kind::i8 in
tensor memory) forced for every call it can serve: parity with the CPU oracle and with the CUDA-core GEMV, through the same
entry points.

The kernel works in exact integers on one grid per activation row (hash bytes x signed base-256 digits of the activations, s32
accumulators in tensor memory, 64-bit sums across windows and thread blocks), so beyond the tolerances of
tests/test_gpu_parity.py it must be bit-stable from run to run, must not depend on how a launch is cut into thread blocks, and
must agree with the CUDA-core GEMV to float32 rounding.
  float32 activations/outputs: norm-relative error <= 1e-5 against the oracle, <= 2e-6 against the CUDA-core GEMV
  bf16 outputs:                the tolerances of tests/test_gpu_parity.py
After every test the fault word of the operator's workspace must still be zero (no bounded wait ran out).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

WIDTHS = (2, 3, 4, 5, 6, 8)


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def fault_word(dev):
    from htr_b200 import _lib, ops

    ws = ops.workspace(dev, 1 << 16)
    off = _lib.lib.htr_linear_fault_offset()
    return int(ws[off:off + 4].view(torch.int32).item())


@pytest.fixture(autouse=True)
def tensor_memory_gemv(dev):
    from htr_b200 import _lib

    _lib.lib.htr_set_gemv_kernel(2)
    yield
    _lib.lib.htr_set_gemv_kernel(-1)
    torch.cuda.synchronize()
    assert fault_word(dev) == 0


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
        _lib.lib.htr_set_gemv_kernel(2)


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
    """Benchmark shapes (thread blocks that cross row blocks, several windows of activations per thread block): run-to-run bit
    stability, agreement with the CUDA-core GEMV, and independence of the decomposition: a run of row blocks cut out of the weight
    is launched with another grid and must reproduce its rows of the full result bit for bit."""
    from htr_b200 import ops, wire

    args = wire.random_packed(m, n, K, 2000 + K, dev)
    x = torch.randn(M, n, generator=torch.Generator().manual_seed(K)).to(dev)
    y = ops.linear(x, *args)
    for _ in range(4):
        assert torch.equal(ops.linear(x, *args), y)
    ref = cuda_core(lambda: ops.linear(x, *args))
    assert rel(y.cpu().numpy(), ref.cpu().numpy()) <= 2e-6
    qw, sc, su, sv = args
    for lo, hi in ((0, 128), (m // 128 // 3 * 128, m // 128 // 3 * 128 + 896), (m - 384, m)):
        ysl = ops.linear(x, qw[lo // 16:hi // 16].contiguous(), sc[lo:hi].contiguous(), su, sv[lo // 8:hi // 8].contiguous())
        assert torch.equal(ysl, y[:, lo:hi])
    xb = x.bfloat16()
    yb = ops.linear(xb, *args)
    assert torch.equal(ops.linear(xb, *args), yb)
    assert rel(yb.float().cpu().numpy(), cuda_core(lambda: ops.linear(xb, *args)).float().cpu().numpy()) <= 4e-3


def test_activation_ranges(coracle, dev):
    """One power-of-two scale per activation row, from a bound on the whole row: rows of very different magnitude, a row of zeros,
    one huge outlier, tiny values next to large ones, and a row that meets the bound (all of one sign under the input signs, i.e.
    a transform output of 128 max|x|) must all keep float32 accuracy."""
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
    signs = 1.0 - 2.0 * torch.from_numpy(np.unpackbits(su.numpy(), bitorder="little").astype(np.float32))
    xw = (1.75 * signs).reshape(1, n)                              # su * x is constant: the first output of every block is 128 * 1.75
    refw = coracle.linear(xw.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    yw = ops.linear(xw.to(dev), *[t.to(dev) for t in (qw, sc, su, sv)]).cpu().numpy()
    assert rel(yw, refw) <= 1e-5


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


def test_padded_form_and_fallbacks(dev):
    """Missing input columns / dropped output rows run on the kernel; the fused prologues and more than four rows do not and fall
    back to the kernels that serve them."""
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
    x8 = torch.randn(8, n, generator=g).to(dev)
    assert rel(ops.linear(x8, *args).cpu().numpy(), cuda_core(lambda: ops.linear(x8, *args)).cpu().numpy()) <= 2e-6


def test_independent_launches_in_a_row(dev):
    """Back-to-back launches with HTR_LINEAR_INPUT_INDEPENDENT (consecutive kernels overlap: a thread block of the next launch
    waits for the tensor memory of the one that is leaving) give the results of the same launches run one at a time."""
    from htr_b200 import ops, wire

    ws = [wire.random_packed(1024, 2048, K, 70 + K, dev) for K in (2, 3, 4, 5)]
    x = torch.randn(1, 2048, generator=torch.Generator().manual_seed(1)).bfloat16().to(dev)
    want = []
    for w in ws:
        want.append(ops.linear(x, *w))
        torch.cuda.synchronize()
    for _ in range(3):
        with ops.independent_inputs():
            got = [ops.linear(x, *w) for w in ws for _ in range(4)]
        torch.cuda.synchronize()
        for i, y in enumerate(got):
            assert torch.equal(y, want[i // 4])
