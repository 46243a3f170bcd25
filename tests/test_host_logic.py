"""CPU-side checks of the product: the shared library loads and exports every symbol of the header, argument
validation answers with status codes before any CUDA work, the decode index arithmetic of the kernels (compiled
as host code) matches a bit-by-bit reading of the stream, and the wire helpers agree with the oracle.  No GPU."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from htr_b200 import build

    build.build()
    from htr_b200 import _lib

    return _lib


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "htr_b200.h")).read()
    declared = set(re.findall(r"\b(htr_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    raw = ctypes.CDLL(lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} declared in include/htr_b200.h but not exported"
    assert declared == set(lib.EXPORTS)
    assert lib.lib.htr_version() >= 100


def test_status_codes_without_touching_the_gpu(lib):
    L = lib.lib
    assert L.htr_decode_raw(None, 4, 7, None, None) == -1                 # K = 7 is not a wire width
    assert L.htr_decode_raw(None, 4, 4, None, None) == -5                 # NULL pointers
    assert L.htr_decode_raw(None, 0, 4, None, None) == 0                  # nothing to do
    assert L.htr_rht(None, 5, 1, 128, None, None, None) == -3
    assert L.htr_rht(None, 0, 1, 100, None, None, None) == -2
    assert L.htr_linear(None, 0, 9, None, 8, 8, 4, None, None, None, None, None, None, 0, None) == -2    # M > 8
    assert L.htr_linear(None, 0, 1, None, 8, 7, 4, None, None, None, None, None, None, 0, None) == -2    # n % 128
    assert L.htr_linear(None, 0, 1, None, 8, 8, 9, None, None, None, None, None, None, 0, None) == -1
    assert L.htr_linear(None, 0, 0, None, 8, 8, 4, None, None, None, None, None, None, 0, None) == 0     # M == 0
    assert L.htr_linear(None, 0, 1, None, 8, 8, 4, None, None, None, None, None, None, 0, None) == -5
    assert L.htr_linear(16, 0, 1, 8, 8, 8, 4, 16, 16, 16, None, 16, None, 0, None) == -6                 # misaligned qweight
    assert L.htr_dequant_w(None, 8, 8, 4, None, None, None, None, 7, None) == -3
    assert b"K" in L.htr_status_string(-1)
    assert L.htr_linear_counter_bytes(4096) == 65536
    # the later entry points validate their arguments the same way, before any CUDA call
    import ctypes

    f = ctypes.c_float(1e-6)
    assert L.htr_linear_padded(None, 0, 1, 100, None, 8, 8, 4, None, None, None, None, None, 128, None, 0, None) == -2   # n_in % 8
    assert L.htr_linear_padded(None, 0, 1, 136, None, 8, 8, 4, None, None, None, None, None, 128, None, 0, None) == -2   # n_in > n
    assert L.htr_linear_padded(None, 0, 1, 128, None, 8, 8, 4, None, None, None, None, None, 132, None, 0, None) == -2   # m_out % 8, > m
    assert L.htr_linear_padded(None, 0, 1, 120, None, 8, 8, 4, None, None, None, None, None, 72, None, 0, None) == -5    # NULL tensors
    assert L.htr_linear_padded(None, 0, 0, 120, None, 8, 8, 4, None, None, None, None, None, 72, None, 0, None) == 0     # no rows
    assert L.htr_linear_fused(None, 1, None, 8, 8, 4, None, None, None, None, None, 0, None, 3, None, f, 0) == -2        # unknown prologue
    assert L.htr_linear_fused(None, 1, None, 8, 8, 4, None, None, None, None, None, 0, None, 1, None, f, 0) == -5        # norm weight missing
    assert L.htr_linear_fused(None, 1, None, 8, 8, 4, None, None, None, None, None, 0, None, 0, None, f, 2) == -2        # residual flag
    assert L.htr_linear_fused(None, 9, None, 8, 8, 4, None, None, None, None, None, 0, None, 0, None, f, 0) == -2        # more than 8 rows
    assert L.htr_linear_gemm(None, 0, 257, None, 8, 8, 4, None, None, None, None, None, None, 0, None) == -2             # more than 256 rows
    assert L.htr_linear_gemm(None, 0, 16, None, 8, 8, 7, None, None, None, None, None, None, 0, None) == -1
    assert L.htr_linear_gemm(None, 0, 16, None, 8, 8, 4, None, None, None, None, None, None, 0, None) == -5
    assert L.htr_linear_gemm(None, 0, 0, None, 8, 8, 4, None, None, None, None, None, None, 0, None) == 0
    assert L.htr_viterbi(None, None, 4, 256, 7, 1, None, None, None, 0, None) == -1
    assert L.htr_viterbi(None, None, 4, 300, 4, 1, None, None, None, 0, None) == -2                                       # more than 256 steps
    assert L.htr_viterbi(None, None, 4, 256, 4, 1, None, None, None, 0, None) == -5
    assert L.htr_viterbi(None, None, 0, 256, 4, 1, None, None, None, 0, None) == 0
    assert L.htr_codebook_f32(None, None) == -5
    assert L.htr_dec_rope_attention(None, None, None, None, None, None, None, 8, 2, 128, 64, None, None) == -5
    one = ctypes.c_int(0)
    ptr = ctypes.addressof(one)                                             # any non-NULL address: the checks below come before a launch
    assert L.htr_dec_rope_attention(ptr, ptr, ptr, ptr, ptr, ptr, ptr, 8, 2, 128, 0, None, None) == -2          # a cache without rows
    assert L.htr_dec_attention(ptr, ptr, ptr, ptr, ptr, 1, 8, 2, 128, 0, None, None) == -2
    assert L.htr_dec_rope_cache(ptr, ptr, ptr, ptr, ptr, ptr, ptr, 1, 8, 2, 128, -3, None, None) == -2
    assert L.htr_linear_grouped(None, 0, None, 8, 8, 4, None, None, None, None, 0, None, 0, None) == 0                    # no problems
    assert L.htr_linear_routed(None, 0, 1, 128, None, 0, 0, None, None, None, None, 8, 8, 4, None, 0, None, 0, None) == -2  # tables without rows


def test_kernel_decode_arithmetic_on_the_host(tmp_path):
    exe = tmp_path / "host_codec_check"
    subprocess.run(["g++", "-std=c++17", "-O1", "-o", str(exe), os.path.join(ROOT, "tests", "host_codec_check.cpp")], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout


def test_wire_helpers_agree_with_the_oracle(lib):
    from htr_b200 import wire
    from oracle import oracle as O

    s = torch.arange(65536)
    assert np.array_equal(wire.gen_values(s).numpy(), O.value_table())
    assert wire.cbscale() == O.cbscale()
    rng = np.random.default_rng(5)
    for K in (2, 3, 4, 5, 8):
        words = rng.integers(-2 ** 31, 2 ** 31, size=(3, 8 * K), dtype=np.int64).astype(np.int32)
        st = O.unpack_states(words, K)
        assert np.array_equal(wire.pack_states(torch.from_numpy(st), K).numpy(), words)
    sg = torch.from_numpy(rng.choice([-1.0, 1.0], size=128).astype(np.float32))
    assert np.array_equal(wire.pack_signs(sg).numpy(), O.pack_signs(sg.numpy()))
    assert np.array_equal(wire.unpack_signs(wire.pack_signs(sg), 128).numpy(), sg.numpy())
    assert wire.payload_bytes(4096, 4096, 4) == 8397824


def test_operator_refuses_cpu_tensors(lib):
    from htr_b200 import ops, wire

    qw, sc, su, sv = wire.random_packed(128, 128, 4, seed=1)
    with pytest.raises(RuntimeError):
        ops.linear(torch.zeros(1, 128, dtype=torch.bfloat16), qw, sc, su, sv)


def test_unit_partition_covers_every_unit_once():
    """CTA b owns units [floor(b*U/G), floor((b+1)*U/G)); the closed-form owner used by the kernel to size the
    split reduction must agree with that partition for awkward U, G."""
    for U, G in ((2048, 444), (6144, 592), (75968, 592), (64, 64), (7, 3), (1187 * 64, 444)):
        owner = [((x + 1) * G - 1) // U for x in range(U)]
        for b in range(G):
            lo, hi = b * U // G, (b + 1) * U // G
            assert hi > lo
            assert all(owner[x] == b for x in range(lo, hi))
