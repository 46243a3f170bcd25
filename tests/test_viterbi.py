"""The sm_100a trellis search (htr_viterbi) against the reference's search: golden states produced by running
htr/reference.py (tests/golden/viterbi.npz), the C oracle on fresh seeded tiles, and size-independent properties
(trellis constraint, circular closure, reported cost = cost of the returned path, search -> pack -> decode round trip)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = (("K2", 2, True), ("K3", 3, True), ("K4", 4, True), ("K5", 5, True), ("K4_open", 4, False), ("K6", 6, True), ("K8", 8, True))


def tiles(B, T, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, generator=g) * (1.0 + 0.25 * torch.rand(B, 1, generator=g))
    rs = (torch.rand(B, (T + 15) // 16, generator=g) + 0.5).repeat_interleave(16, dim=1)[:, :T] ** 2
    return x, rs / rs.mean(dim=1, keepdim=True)


def test_device_codebook_is_the_reference_table_bit_for_bit(coracle):
    from htr_b200 import encoder

    cb = encoder.codebook_f32(torch.device("cuda:0")).cpu().numpy()
    assert np.array_equal(cb.view(np.uint32), coracle.codebook_f32().view(np.uint32))


@pytest.mark.parametrize("tag,K,tailbite", CASES)
def test_search_returns_the_reference_states(golden, tag, K, tailbite):
    from htr_b200 import encoder

    dev = torch.device("cuda:0")
    g = golden("viterbi")
    x, w = torch.from_numpy(g[tag + "_x"]).to(dev), torch.from_numpy(g[tag + "_w"]).to(dev)
    states, cost = encoder.viterbi(x, w, None, K, tailbite=tailbite, return_cost=True)
    assert states.dtype == torch.int64 and np.array_equal(states.cpu().numpy(), g[tag + "_states"])
    assert np.allclose(cost.cpu().numpy(), g[tag + "_cost"], rtol=1e-4)


@pytest.mark.parametrize("K", (2, 3, 4, 5, 6, 8))
def test_search_matches_the_oracle_on_fresh_tiles(coracle, K):
    from htr_b200 import encoder, wire

    dev = torch.device("cuda:0")
    x, w = tiles(12, 256, 40 + K)
    x[3] *= 3.0                                                         # a tile mostly outside the codebook's range
    w[5] = 1.0                                                          # unit weights: many exactly equal costs, ties matter
    x[5] = torch.round(x[5] * 4) / 4
    x[7] = 0.0                                                          # degenerate tiles: all-zero targets,
    x[8] = x[8, :1]                                                     # a constant target (every step ties),
    w[9, ::2] = 1e-6                                                    # weights spanning six orders of magnitude
    want, want_cost = coracle.viterbi(x.numpy(), w.numpy(), K)
    cb = torch.from_numpy(wire.codebook_f32()).to(dev)                  # the hook's third argument, as the reference passes it
    got, cost = encoder.viterbi(x.to(dev), w.to(dev), cb, K, return_cost=True)
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(cost.cpu().numpy().view(np.uint32), want_cost.view(np.uint32))   # same float operations, same bits


@pytest.mark.parametrize("T,tailbite", ((64, True), (17, False), (8, True), (256, False)))   # T*K >= 16: a closed path always exists
def test_short_and_open_searches(coracle, T, tailbite):
    from htr_b200 import encoder

    dev = torch.device("cuda:0")
    x, w = tiles(5, T, 7 * T + int(tailbite))
    want, _ = coracle.viterbi(x.numpy(), w.numpy(), 3, tailbite=tailbite)
    got = encoder.viterbi(x.to(dev), w.to(dev), None, 3, tailbite=tailbite)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("K", (2, 3, 4, 5))
def test_properties_at_encoder_batch_size(coracle, K):
    """One encoder call for a 4096-row matrix is 256 tiles per 16-column block times the group size; 1024 is the reference's
    max_batch (htr/encode.py:47).  Too many tiles for the CPU oracle, so: structure, cost accounting, round trip, optimality
    against perturbed paths."""
    from htr_b200 import _lib, encoder, wire

    dev = torch.device("cuda:0")
    B = 1024
    x, w = tiles(B, 256, 900 + K)
    st, cost = encoder.viterbi(x.to(dev), w.to(dev), None, K, return_cost=True)
    s = st.cpu().numpy()
    low = 0xFFFF >> K
    assert s.min() >= 0 and s.max() <= 0xFFFF
    assert np.array_equal(s[:, 1:] >> K, s[:, :-1] & low) and np.array_equal(s[:, 0] >> K, s[:, -1] & low)
    cb = wire.codebook_f32()
    path = (w.numpy().astype(np.float64) * (x.numpy().astype(np.float64) - cb[s].astype(np.float64)) ** 2).sum(axis=1)
    assert np.allclose(cost.cpu().numpy(), path, rtol=2e-4)
    # search -> pack -> device decode returns the codebook integers of the chosen states
    words = encoder.pack(st, K)
    out = torch.empty(B, 256, dtype=torch.int16, device=dev)
    _lib.check(_lib.lib.htr_decode_raw(words.contiguous().data_ptr(), B, K, out.data_ptr(), torch.cuda.current_stream().cuda_stream), "htr_decode_raw")
    assert np.array_equal(out.cpu().numpy(), wire.gen_values(st.cpu()).numpy().astype(np.int16))
    # no cheaper closed path nearby: re-searching from the same inputs on the CPU for a few tiles gives the same cost
    ref_states, ref_cost = coracle.viterbi(x[:3].numpy(), w[:3].numpy(), K)
    assert np.array_equal(s[:3], ref_states)
    # rate-distortion sanity: more bits per weight never cost more
    if K > 2:
        _, coarser = encoder.viterbi(x[:64].to(dev), w[:64].to(dev), None, K - 1, return_cost=True)
        assert float(cost[:64].sum()) < float(coarser.sum())


def test_arguments_are_checked():
    from htr_b200 import _lib, encoder

    dev = torch.device("cuda:0")
    x, w = tiles(2, 256, 1)
    with pytest.raises(_lib.HTRError):
        encoder.viterbi(x, w, None, 4)                                  # CPU tensors
    with pytest.raises(_lib.HTRError):
        encoder.viterbi(x.to(dev), w.to(dev), None, 7)
    with pytest.raises(_lib.HTRError):
        encoder.viterbi(torch.zeros(2, 300, device=dev), torch.ones(2, 300, device=dev), None, 4)
    with pytest.raises(_lib.HTRError):
        encoder.viterbi(x.to(dev), w.to(dev), torch.zeros(65536, device=dev), 4)   # not the codebook
    assert encoder.viterbi(x[:0].to(dev), w[:0].to(dev), None, 4).shape == (0, 256)
