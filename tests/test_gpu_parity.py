"""Parity of the CUDA path with the CPU oracle, through the C interface (ctypes -> libhtr_b200.so).

Integer work (decode) must be bit-exact.  Floating-point outputs are compared with
x.float() @ wire.dequant(...).T as restated by the oracle:
  float32 activations/outputs: norm-relative error <= 1e-5
  bf16 / fp16 outputs:         norm-relative error <= 4e-3 and |err| <= 2^-7 |y| + 1e-2 rms(y) elementwise
(the oracle's own result rounded to bf16 sits at 1.7e-3 / 0.9e-2 rms).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

WIDTHS = (2, 3, 4, 5, 6, 8)
TORCH_OF = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def gemv_up_to_eight_rows(monkeypatch):
    """This file is about the streaming GEMV: keep batches of 5..8 rows on it (by default they take the tensor-core GEMM,
    which tests/test_gpu_gemm.py covers)."""
    from htr_b200 import ops

    monkeypatch.setattr(ops, "GEMV_ROUTE_MAX", 8)


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def check_output(y, ref, dtype):
    y = y.float().cpu().numpy()
    if dtype == "f32":
        assert rel(y, ref) <= 1e-5
    else:
        assert rel(y, ref) <= 4e-3
        rms = float(np.sqrt(np.mean(np.square(ref))))
        assert np.all(np.abs(y - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-2 * rms)


def packed(m, n, K, seed, dev):
    from htr_b200 import wire

    return wire.random_packed(m, n, K, seed, dev)


# ------------------------------------------------------------------------------------------- integers
@pytest.mark.parametrize("K", WIDTHS)
def test_decode_raw_bit_exact_on_reference_draw(golden, dev, K):
    from htr_b200 import wire

    g = golden("bit_layout")
    got = wire.decode_raw(torch.from_numpy(g[f"words_K{K}"]).to(dev))
    assert np.array_equal(got.cpu().numpy(), g[f"values_K{K}"])


@pytest.mark.parametrize("K", WIDTHS)
@pytest.mark.parametrize("ntiles", (1, 7, 1000))
def test_decode_raw_bit_exact_random_and_extreme_streams(coracle, dev, K, ntiles):
    from htr_b200 import wire

    rng = np.random.default_rng(100 * K + ntiles)
    words = rng.integers(-2 ** 31, 2 ** 31, size=(ntiles, 8 * K), dtype=np.int64).astype(np.int32)
    words[0] = -1                       # all ones: every window is 0xFFFF
    if ntiles > 1:
        words[1] = 0                    # all zeros
    got = wire.decode_raw(torch.from_numpy(words).to(dev)).cpu().numpy()
    assert np.array_equal(got, coracle.decode_raw(words, K))


def test_decode_raw_empty(dev):
    from htr_b200 import wire

    assert wire.decode_raw(torch.empty((0, 4, 32), dtype=torch.int32, device=dev)).shape == (0, 256)


# ------------------------------------------------------------------------------------------- transform
@pytest.mark.parametrize("dtype", ("bf16", "f16", "f32"))
@pytest.mark.parametrize("M,n", ((1, 128), (3, 384), (8, 4096)))
def test_rht_matches_oracle(coracle, dev, dtype, M, n):
    from htr_b200 import _lib

    g = torch.Generator().manual_seed(n + M)
    x = torch.randn(M, n, generator=g).to(TORCH_OF[dtype])
    su = torch.randint(0, 256, (n // 8,), dtype=torch.uint8, generator=g)
    xd, sud = x.to(dev), su.to(dev)
    out = torch.empty(M, n, dtype=torch.float32, device=dev)
    rc = _lib.lib.htr_rht(xd.data_ptr(), {"bf16": 0, "f16": 1, "f32": 2}[dtype], M, n, sud.data_ptr(), out.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    ref = coracle.rht(x.float().numpy(), su.numpy())
    assert rel(out.cpu().numpy(), ref) <= 1e-6


@pytest.mark.parametrize("K", (2, 3, 4, 5))
def test_dequant_w_matches_reference_output(golden, dev, K):
    from htr_b200 import wire

    g = golden(f"linear_K{K}")
    args = [torch.from_numpy(g[k]).to(dev) for k in ("qweight", "scales", "su", "sv")]
    W = wire.dequant(*args, dtype=torch.float32).cpu().numpy()
    assert np.abs(W - g["W"]).max() <= 1e-5 * np.abs(g["W"]).max()
    Wb = wire.dequant(*args, dtype=torch.bfloat16).float().cpu().numpy()
    assert np.abs(Wb - g["W"]).max() <= 2.0 ** -8 * np.abs(g["W"]).max()


# ------------------------------------------------------------------------------------------- linear
@pytest.mark.parametrize("K", (2, 3, 4, 5))
@pytest.mark.parametrize("dtype", ("f32", "bf16", "f16"))
def test_linear_against_reference_outputs(golden, dev, K, dtype):
    """fixtures computed by the reference: x.float() @ wire.dequant(...).T, 256 x 384, three activation rows"""
    from htr_b200 import ops

    g = golden(f"linear_K{K}")
    qw, sc, su, sv = [torch.from_numpy(g[k]).to(dev) for k in ("qweight", "scales", "su", "sv")]
    x = torch.from_numpy(g["x_f32"]).to(dev).to(TORCH_OF[dtype])          # bf16-representable values: exact in all three
    for rows in (1, 2, 3):
        y = ops.linear(x[:rows], qw, sc, su, sv)
        assert y.dtype == x.dtype and tuple(y.shape) == (rows, 256)
        check_output(y, g["y"][:rows], dtype)
    bias = torch.from_numpy(g["bias_f32"]).to(dev).to(TORCH_OF[dtype])
    check_output(ops.linear(x, qw, sc, su, sv, bias), g["y_bias"], dtype)


@pytest.mark.parametrize("name", ("encoded_K4", "encoded_hessian_K2", "encoded_hessian_K3"))
def test_linear_on_real_encoder_streams(golden, dev, name):
    from htr_b200 import ops

    g = golden(name)
    qw, sc, su, sv = [torch.from_numpy(g[k]).to(dev) for k in ("qweight", "scales", "su", "sv")]
    n = g["What"].shape[1]
    x = torch.randn(2, n, generator=torch.Generator().manual_seed(3)).bfloat16()
    ref = x.float().numpy().astype(np.float64) @ g["What"].astype(np.float64).T
    check_output(ops.linear(x.to(dev).float(), qw, sc, su, sv), ref.astype(np.float32), "f32")
    check_output(ops.linear(x.to(dev), qw, sc, su, sv), ref.astype(np.float32), "bf16")


@pytest.mark.parametrize("K", WIDTHS)
@pytest.mark.parametrize("m,n,M", ((128, 128, 1), (128, 1280, 4), (384, 2048, 8), (1024, 256, 5), (256, 4096, 7)))
def test_linear_shapes_against_oracle(coracle, dev, K, m, n, M):
    from htr_b200 import ops

    qw, sc, su, sv = packed(m, n, K, seed=7 * K + m + n + M, dev="cpu")
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, n, generator=g)
    bias = torch.randn(m, generator=g)
    ref = coracle.linear(x.numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy(), bias=bias.numpy())
    y = ops.linear(x.to(dev), qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev), bias.to(dev))
    check_output(y, ref, "f32")
    xb = x.bfloat16()
    refb = coracle.linear(xb.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    check_output(ops.linear(xb.to(dev), qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev)), refb, "bf16")


@pytest.mark.parametrize("M", (0, 9, 17, 64, 70))
def test_linear_row_counts_beyond_one_launch(coracle, dev, M):
    """M == 0 is empty, 8 < M <= 64 loops the GEMV over 8-row chunks, M > 64 goes through dequant + GEMM"""
    from htr_b200 import ops

    m, n, K = 256, 512, 4
    qw, sc, su, sv = packed(m, n, K, seed=M + 1, dev="cpu")
    x = torch.randn(M, n, generator=torch.Generator().manual_seed(M)).bfloat16()
    y = ops.linear(x.to(dev), qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev))
    assert tuple(y.shape) == (M, m) and y.dtype == torch.bfloat16
    if M:
        ref = coracle.linear(x.float().numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
        check_output(y, ref, "bf16")
    y3 = ops.linear(x.to(dev).reshape(1, M, n), qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev))   # leading dims are kept
    assert tuple(y3.shape) == (1, M, m)


def test_linear_bad_arguments_raise(dev):
    from htr_b200 import ops

    qw, sc, su, sv = packed(128, 128, 4, seed=2, dev=dev)
    x = torch.zeros(1, 128, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError):
        ops.linear(x[:, :64], qw, sc, su, sv)                              # wrong inner size
    with pytest.raises(RuntimeError):
        ops.linear(x.to(torch.float64), qw, sc, su, sv)                    # unsupported dtype
    with pytest.raises(RuntimeError):
        ops.linear(x, qw[:, :, :28].contiguous(), sc, su, sv)             # 28 words per tile is no wire width
    with pytest.raises(RuntimeError):
        ops.linear(x, qw, sc.float(), su, sv)


# ------------------------------------------------------------------------------------------- full sizes
@pytest.mark.parametrize("K,m,n", ((4, 4096, 12288), (3, 12288, 4096), (2, 4096, 4096), (5, 4096, 4096)))
def test_full_size_linear_and_properties(coracle, dev, K, m, n):
    """Benchmark shapes: compared with the oracle once, then size-independent properties: run-to-run bit
    stability, linearity in the activations, and independence of 128-row blocks (a row slice of the weight
    gives the same rows)."""
    from htr_b200 import ops, wire

    qw, sc, su, sv = packed(m, n, K, seed=1000 + K, dev="cpu")
    g = torch.Generator().manual_seed(K)
    x = torch.randn(2, n, generator=g)
    dq, dsc, dsu, dsv = qw.to(dev), sc.to(dev), su.to(dev), sv.to(dev)
    y = ops.linear(x.to(dev), dq, dsc, dsu, dsv)
    ref = coracle.linear(x[:1].numpy(), qw.numpy(), sc.numpy(), su.numpy(), sv.numpy())
    check_output(y[:1], ref, "f32")
    for _ in range(5):
        assert torch.equal(ops.linear(x.to(dev), dq, dsc, dsu, dsv), y)
    ysum = ops.linear((x[0] + x[1]).to(dev)[None], dq, dsc, dsu, dsv)
    assert rel(ysum.cpu().numpy(), (y[0] + y[1])[None].cpu().numpy()) <= 2e-6
    lo, hi = m // 128 // 3 * 128, m // 128 // 3 * 128 + 256
    ysl = ops.linear(x.to(dev), dq[lo // 16:hi // 16].contiguous(), dsc[lo:hi].contiguous(), dsu, dsv[lo // 8:hi // 8].contiguous())
    assert rel(ysl.cpu().numpy(), y[:, lo:hi].cpu().numpy()) <= 2e-6
    # integer check at full size: checksum of the decoded integers against the C oracle on a sample of strips
    raw = wire.decode_raw(dq[:8])
    assert np.array_equal(raw.cpu().numpy(), coracle.decode_raw(qw[:8].reshape(-1, 8 * K).numpy(), K))


def test_workspace_counters_stay_zero(dev):
    from htr_b200 import ops, _lib

    qw, sc, su, sv = packed(512, 4096, 4, seed=9, dev=dev)
    x = torch.randn(1, 4096, device=dev).bfloat16()
    ops.linear(x, qw, sc, su, sv)
    torch.cuda.synchronize()
    for buf in ops._WORKSPACES.values():
        nb = _lib.lib.htr_linear_counter_bytes(512 * 64)
        assert int(buf[:nb].to(torch.int64).sum()) == 0


@pytest.mark.parametrize("K", (2, 3, 4, 5))
def test_routed_launch_equals_one_call_per_problem(dev, K):
    """htr_linear_routed: device-side route into per-expert pointer tables, shared activation rows, a skipped (null) expert,
    and the SwiGLU prologue -- each problem bit-identical to its own htr_linear call."""
    from htr_b200 import ops

    E, m, n, T, k = 5, 256, 384, 3, 2
    experts = [packed(m, n, K, 70 + e, dev) for e in range(E)]
    tables = [torch.tensor([experts[e][i].data_ptr() if e != 3 else 0 for e in range(E)], dtype=torch.int64, device=dev) for i in range(4)]
    route = torch.tensor([0, 4, 2, 2, 3, 1], dtype=torch.int64, device=dev)          # pair (token 2, slot 0) hits the absent expert
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(T, n, device=dev).to(dtype)
        out = torch.full((T * k, m), 7.0, dtype=dtype, device=dev)
        got = ops.linear_routed(x, route, tables, m // 16, n // 16, K, x_div=k, out=out)
        assert got is out
        for i, e in enumerate(route.tolist()):
            if e == 3:
                assert bool((out[i] == 7.0).all())                                     # untouched
            else:
                assert torch.equal(out[i:i + 1], ops.linear(x[i // k:i // k + 1], *experts[e]))
    # down-projection form: rows of [gate | up], SwiGLU applied while staging
    gu = torch.randn(T * k, 2 * n, device=dev).bfloat16()
    got = ops.linear_routed(gu, route, tables, m // 16, n // 16, K, prologue=ops.PROLOGUE_SWIGLU)
    for i, e in enumerate(route.tolist()):
        if e != 3:
            want = ops.linear_fused(gu[i:i + 1].contiguous(), *experts[e], prologue=ops.PROLOGUE_SWIGLU)
            assert torch.equal(got[i:i + 1], want)
    # planned for a rank that owns one problem in four (htr_linear_routed_peers without peers: four times the thread blocks, other
    # column splits): the same rows to float32 rounding, absent experts untouched
    x = torch.randn(T, n, device=dev)
    base = ops.linear_routed(x, route, tables, m // 16, n // 16, K, x_div=k, out=torch.full((T * k, m), 7.0, device=dev))
    wide = ops.linear_routed(x, route, tables, m // 16, n // 16, K, x_div=k, out=torch.full((T * k, m), 7.0, device=dev), share=4)
    assert bool((wide[4] == 7.0).all())
    assert float((wide - base).norm() / base.norm()) <= 2e-6
    # route entries outside the tables are skipped like absent experts (the kernel compares them with the table length first)
    wild = torch.tensor([0, E, 2, -1, 3, 1], dtype=torch.int64, device=dev)
    x = torch.randn(T, n, device=dev)
    out = torch.full((T * k, m), 7.0, device=dev)
    ops.linear_routed(x, wild, tables, m // 16, n // 16, K, x_div=k, out=out)
    for i, e in enumerate(wild.tolist()):
        if e in (E, -1, 3):
            assert bool((out[i] == 7.0).all())
        else:
            assert torch.equal(out[i:i + 1], ops.linear(x[i // k:i // k + 1], *experts[e]))
