"""The CPU oracle (numpy and C restatements) against fixtures produced by running the reference's
htr/wire.py (tests/golden/make_golden.py) and against the vectors of the reference's own
tests/test_release.py.  No GPU."""
import hashlib

import numpy as np
import pytest

from oracle import oracle as O

WIDTHS = (2, 3, 4, 5)


def test_codebook_known_answers(golden, coracle):
    g = golden("codebook")
    table = O.value_table()
    assert np.array_equal(table[g["probe_states"]], g["probe_values"])
    assert int(table.min()) == int(g["vmin"]) and int(table.max()) == int(g["vmax"])
    assert len(np.unique(table)) == int(g["distinct"])
    assert hashlib.sha256(table.astype("<i2").tobytes()).hexdigest() == str(g["sha256_int16"])
    assert hashlib.sha256(O.codebook_f32().tobytes()).hexdigest() == str(g["sha256_cb_f32"])
    assert O.cbscale() == float(g["cbscale"])
    # C restatement
    assert [coracle.gen_value(int(s)) for s in g["probe_states"]] == list(g["probe_values"])
    assert hashlib.sha256(coracle.codebook_f32().tobytes()).hexdigest() == str(g["sha256_cb_f32"])
    assert coracle.cbscale() == float(g["cbscale"])


@pytest.mark.parametrize("K", (2, 3, 4, 5, 6, 8))
def test_bit_layout_matches_reference_draw(golden, coracle, K):
    """words drawn exactly as tests/test_release.py:30-31; states from the reference's unpack_states."""
    g = golden("bit_layout")
    words, states, values = g[f"words_K{K}"], g[f"states_K{K}"].astype(np.int64), g[f"values_K{K}"]
    for impl in (O, coracle):
        assert np.array_equal(impl.unpack_states(words, K), states)
        assert np.array_equal(impl.pack_states(states, K), words)
        assert np.array_equal(impl.decode_raw(words, K), values)


@pytest.mark.parametrize("K", WIDTHS)
def test_independent_bit_string_oracle(K):
    """the string-of-bits check of tests/test_release.py:28-38, applied to the oracle itself"""
    rng = np.random.default_rng(K)
    words = rng.integers(-2 ** 31, 2 ** 31, size=(2, 8 * K), dtype=np.int64).astype(np.int32)
    expected = []
    for row in words.tolist():
        bits = "".join(format(w & 0xFFFFFFFF, "032b") for w in row)
        expected.append([int("".join(bits[(K * (t + 1) - 16 + j) % len(bits)] for j in range(16)), 2) for t in range(256)])
    assert np.array_equal(O.unpack_states(words, K), np.array(expected))


def test_sign_convention_and_hadamard(golden, coracle):
    g = golden("signs_hadamard")
    for impl in (O, coracle):
        assert int(impl.pack_signs(g["alt_signs"])[0]) == 170 == int(g["alt_byte"])     # tests/test_release.py:40-43
        assert np.array_equal(impl.pack_signs(g["rand_signs"]), g["rand_packed"])
        assert np.array_equal(impl.unpack_signs(g["rand_packed"], 256), g["rand_signs"])
        h = impl.hadamard128()
        assert np.array_equal(h, g["h128"])
        assert np.allclose(h @ h.T, np.eye(128), atol=2e-6)                             # tests/test_release.py:45-47


@pytest.mark.parametrize("K", WIDTHS)
def test_dequant_and_linear_against_reference_outputs(golden, coracle, K):
    g = golden(f"linear_K{K}")
    args = (g["qweight"], g["scales"], g["su"], g["sv"])
    Wref, scale = g["W"], np.abs(g["W"]).max()
    for impl in (O, coracle):
        W = impl.dequant(*args)
        # same float32 operations in a different summation order: a few ulp of the largest entry
        assert np.abs(W - Wref).max() <= 4e-6 * scale
    assert np.abs(O.rht(g["x_f32"], g["su"]) - g["xt"]).max() <= 1e-5 * np.abs(g["xt"]).max()
    assert np.abs(coracle.rht(g["x_f32"], g["su"]) - g["xt"]).max() <= 1e-5 * np.abs(g["xt"]).max()
    for impl in (O, coracle):
        y = impl.linear(g["x_f32"], *args)
        assert np.linalg.norm(y - g["y"]) <= 2e-6 * np.linalg.norm(g["y"])
        yb = impl.linear(g["x_f32"], *args, bias=g["bias_f32"])
        assert np.linalg.norm(yb - g["y_bias"]) <= 2e-6 * np.linalg.norm(g["y_bias"])


@pytest.mark.parametrize("name", ("encoded_K4", "encoded_hessian_K2", "encoded_hessian_K3"))
def test_real_encoder_streams_decode_to_the_encoder_output(golden, coracle, name):
    """tests/test_release.py:53-73: the packed tensors decode to the encoder's own What."""
    g = golden(name)
    args = (g["qweight"], g["scales"], g["su"], g["sv"])
    K = g["qweight"].shape[-1] // 8
    # real tail-biting paths obey the shift relation of the trellis
    st = O.unpack_states(g["qweight"].reshape(-1, 8 * K), K)
    assert np.array_equal(st[:, 1:] >> K, st[:, :-1] & ((1 << (16 - K)) - 1))
    assert np.array_equal(st[:, 0] >> K, st[:, -1] & ((1 << (16 - K)) - 1))
    scale = np.abs(g["What"]).max()
    for impl in (O, coracle):
        assert np.abs(impl.dequant(*args) - g["What"]).max() <= 4e-6 * scale
    err = np.square(g["What"] - g["W_in"]).sum() / np.square(g["W_in"]).sum()
    assert err < (0.02 if K >= 4 else 0.2)


def test_payload_accounting():
    # docs/EVIDENCE.md:36-41 of the reference
    assert [O.payload_bytes(4096, 4096, K) for K in WIDTHS] == [4203520, 6300672, 8397824, 10494976]


VITERBI_CASES = (("K2", 2, True), ("K3", 3, True), ("K4", 4, True), ("K5", 5, True), ("K4_open", 4, False), ("K6", 6, True), ("K8", 8, True))


@pytest.mark.parametrize("tag,K,tailbite", VITERBI_CASES)
def test_trellis_search_reproduces_the_reference_search(golden, coracle, tag, K, tailbite):
    """htr/reference.py:7-50 run on seeded tiles when the fixture was made: same states, same cost."""
    g = golden("viterbi")
    x, w, want = g[tag + "_x"], g[tag + "_w"], g[tag + "_states"]
    states, total = coracle.viterbi(x, w, K, tailbite=tailbite)
    assert np.array_equal(states, want)
    # the trellis constraint and, with tail-biting, the circular closure (rate exactly K bits per weight)
    mask = 0xFFFF
    assert np.array_equal(states[:, 1:] >> K, states[:, :-1] & (mask >> K))
    if tailbite:
        assert np.array_equal(states[:, 0] >> K, states[:, -1] & (mask >> K))
    for b in range(x.shape[0]):
        assert abs(coracle.path_cost(x[b], w[b], states[b]) - float(g[tag + "_cost"][b])) <= 1e-4 * float(g[tag + "_cost"][b])
        assert abs(float(total[b]) - float(g[tag + "_cost"][b])) <= 1e-4 * float(g[tag + "_cost"][b])
