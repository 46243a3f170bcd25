"""htr_linear_static, the entry point for callers that cannot allocate device memory (its scratch is a fixed array
inside the library).  Called through the C interface twice in a row and compared with htr_linear, which takes a
caller-provided workspace.  Collected last on purpose: a failure here cannot hide the other tests of a run that
stops at the first failure."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu().numpy().astype(np.float64), b.float().cpu().numpy().astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("K,m,n,M,dtype", ((4, 512, 4096, 1, torch.bfloat16), (3, 4096, 1024, 3, torch.float32)))
def test_static_scratch_entry_matches_workspace_entry(K, m, n, M, dtype):
    from htr_b200 import _lib, ops, wire

    dev = torch.device("cuda:0")
    code = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}[dtype]
    qw, sc, su, sv = wire.random_packed(m, n, K, seed=77 + K, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    tol = 1e-5 if dtype == torch.float32 else 4e-3
    for call in range(2):                                     # two calls in a row share the array
        x = torch.randn(M, n, device=dev, generator=torch.Generator(device=dev).manual_seed(call)).to(dtype)
        bias = torch.randn(m, device=dev).to(dtype) if call else None
        want = ops.linear(x, qw, sc, su, sv, bias)             # existing entry point (htr_linear_ex with a workspace)
        got = torch.full_like(want, float("nan"))
        rc = _lib.lib.htr_linear_static(x.data_ptr(), code, M, qw.data_ptr(), m // 16, n // 16, K, sc.data_ptr(), su.data_ptr(),
                                        sv.data_ptr(), None if bias is None else bias.data_ptr(), got.data_ptr(), stream)
        assert rc == 0, _lib.lib.htr_status_string(rc)
        torch.cuda.synchronize()
        assert _rel(got, want) <= tol


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
