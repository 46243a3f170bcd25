"""htr_linear_static, the entry point for callers that cannot allocate device memory (its scratch is a fixed array
inside the library).  Called through the C interface several times in a row and compared with htr_linear_ex, which takes a
caller-provided workspace (same kernel, same plan: the results must be equal bit for bit), and with the CPU oracle.
Collected last on purpose: a failure here cannot hide the other tests of a run that stops at the first failure."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _static(x, qw, sc, su, sv, bias, like):
    from htr_b200 import _lib

    code = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}[x.dtype]
    got = torch.full_like(like, float("nan"))
    mt, nt, W = qw.shape
    rc = _lib.lib.htr_linear_static(x.data_ptr(), code, x.shape[0], qw.data_ptr(), mt, nt, W // 8, sc.data_ptr(), su.data_ptr(),
                                    sv.data_ptr(), None if bias is None else bias.data_ptr(), got.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.lib.htr_status_string(rc)
    torch.cuda.synchronize()
    return got


@pytest.mark.parametrize("K,m,n,M,dtype", ((4, 512, 4096, 1, torch.bfloat16), (3, 4096, 1024, 3, torch.float32),
                                           (5, 1024, 2048, 2, torch.bfloat16), (2, 768, 1536, 4, torch.bfloat16)))
def test_static_scratch_entry_matches_workspace_entry(coracle, K, m, n, M, dtype):
    from htr_b200 import ops, wire

    dev = torch.device("cuda:0")
    packed = wire.random_packed(m, n, K, seed=77 + K)
    qw, sc, su, sv = [t.to(dev) for t in packed]
    for call in range(2):                                     # two calls in a row share the array
        x = torch.randn(M, n, generator=torch.Generator().manual_seed(call)).to(dtype)
        bias = torch.randn(m, generator=torch.Generator().manual_seed(5)).to(dtype) if call else None
        xd, bd = x.to(dev), None if bias is None else bias.to(dev)
        want = ops.linear(xd, qw, sc, su, sv, bd)              # existing entry point (htr_linear_ex with a workspace)
        got = _static(xd, qw, sc, su, sv, bd, want)
        assert torch.equal(got, want)
        ref = coracle.linear(x.float().numpy(), *[t.numpy() for t in packed], bias=None if bias is None else bias.float().numpy())
        assert _rel(got.float().cpu().numpy(), ref) <= (1e-5 if dtype == torch.float32 else 4e-3)


def test_static_scratch_entry_mixed_shapes_in_a_row(coracle):
    """Calls of different shapes, widths and row counts share the array one after the other (split and flat plans, both GEMV
    kernels): each result is checked against the CPU oracle."""
    from htr_b200 import wire

    dev = torch.device("cuda:0")
    for i, (K, m, n, M) in enumerate(((4, 256, 4096, 1), (3, 8192, 256, 2), (2, 128, 128, 4), (5, 2048, 1024, 8), (4, 256, 4096, 1))):
        packed = wire.random_packed(m, n, K, seed=300 + i)
        x = torch.randn(M, n, generator=torch.Generator().manual_seed(i))
        like = torch.empty(M, m, device=dev)
        got = _static(x.to(dev), *[t.to(dev) for t in packed], None, like)
        ref = coracle.linear(x.numpy(), *[t.numpy() for t in packed])
        assert _rel(got.cpu().numpy(), ref) <= 1e-5


def test_static_scratch_entry_rejects_oversized_problems():
    from htr_b200 import _lib, wire

    dev = torch.device("cuda:0")
    m, n, K, M = 151936, 4096, 4, 8                            # scratch of this case is larger than the fixed array
    need = _lib.lib.htr_linear_workspace_bytes(M, m, n, K)
    assert need > 4 << 20
    x = torch.zeros(M, n, device=dev, dtype=torch.bfloat16)
    y = torch.zeros(M, 128, device=dev, dtype=torch.bfloat16)
    qw = torch.zeros(8, n // 16, 8 * K, dtype=torch.int32, device=dev)   # never dereferenced: the size check comes first
    sc = torch.zeros(128, dtype=torch.float16, device=dev)
    sg = torch.zeros(n // 8, dtype=torch.uint8, device=dev)
    rc = _lib.lib.htr_linear_static(x.data_ptr(), _lib.BF16, M, qw.data_ptr(), m // 16, n // 16, K, sc.data_ptr(), sg.data_ptr(),
                                    sg.data_ptr(), None, y.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -8
