"""Generate the golden fixtures of tests/golden/ by RUNNING the reference's own CPU code.

Run where the reference checkout is available (it is not on the GPU box, so the outputs are
committed):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/HTR

Everything written here comes from htr/wire.py (decoder), htr/encode.py + htr/reference.py
(encoder, to obtain real tail-biting streams) of that checkout; nothing is recomputed by this
repository's code.  Fixtures:

  codebook.npz      v(s) anchors, sha256 of the int16 / float32 tables, cbscale
  bit_layout.npz    the seeded words of tests/test_release.py:28-38 with states and values, K2..K5
                    (+K6, K8, which the wire also allows)
  signs_hadamard.npz sign-byte and H128 known answers (tests/test_release.py:40-47)
  linear_K{2..5}.npz random packed linears: inputs, wire.dequant W, x.float() @ W.T
  encoded_K4.npz    encoder round trip of tests/test_release.py:53-73 (seed 12, 128x128, H = I)
  encoded_hessian_K{2,3}.npz  small Hessian-weighted encodes (the outlier-channel recipe of the
                    benchmark configs, shrunk to 128x256)
  viterbi.npz       htr/reference.py viterbi (the encoder's trellis search) on seeded tiles: targets, weights, the states it
                    returns and their cost, K2..K5 tail-biting + K4 without tail-biting + K6/K8 on one tile
                    (only with --viterbi, it takes a few minutes)
  encode_K3.npz     htr/encode.py encode_group on a 128x256 matrix with an outlier-channel Hessian, inputs included
                    (W, H), two members sharing the input signs (only with --encode)
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the HTR checkout")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--viterbi", action="store_true", help="write viterbi.npz only")
    ap.add_argument("--encode", action="store_true", help="write encode_K3.npz only")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from htr import encode, wire

    torch.set_num_threads(os.cpu_count())
    out = a.out
    if a.viterbi:
        return viterbi_fixture(out)
    if a.encode:
        return encode_fixture(out)

    # ---- codebook
    v = wire.gen_values(torch.arange(65536))
    cb = wire.codebook_f32()
    probe = np.array([0, 1, 2, 3, 255, 256, 4096, 32768, 65535], dtype=np.int64)
    np.savez(os.path.join(out, "codebook.npz"),
             probe_states=probe, probe_values=v[torch.from_numpy(probe)].numpy(),
             vmin=int(v.min()), vmax=int(v.max()), distinct=int(v.unique().numel()),
             sha256_int16=hashlib.sha256(v.to(torch.int16).numpy().tobytes()).hexdigest(),
             sha256_cb_f32=hashlib.sha256(cb.numpy().tobytes()).hexdigest(),
             cbscale=np.float64(wire.cbscale()), cb_probe=cb[torch.from_numpy(probe)].numpy())

    # ---- bit layout: the exact draw of tests/test_release.py:30-31
    d = {}
    for K in (2, 3, 4, 5, 6, 8):
        g = torch.Generator().manual_seed(K)
        words = torch.randint(-(2 ** 31), 2 ** 31, (2, 8 * K), dtype=torch.int32, generator=g)
        st = wire.unpack_states(words, K)
        assert torch.equal(words, wire.pack_states(st, K))
        d[f"words_K{K}"] = words.numpy()
        d[f"states_K{K}"] = st.numpy().astype(np.uint16)
        d[f"values_K{K}"] = wire.gen_values(st).numpy().astype(np.int16)
    np.savez_compressed(os.path.join(out, "bit_layout.npz"), **d)

    # ---- signs / Hadamard
    signs = torch.tensor([1., -1., 1., -1., 1., -1., 1., -1.])
    g = torch.Generator().manual_seed(77)
    rs = (torch.randint(0, 2, (256,), generator=g) * 2 - 1).float()
    h = wire.hadamard(128, "cpu")
    np.savez_compressed(os.path.join(out, "signs_hadamard.npz"), alt_signs=signs.numpy(),
                        alt_byte=int(wire.pack_signs(signs).item()), rand_signs=rs.numpy(),
                        rand_packed=wire.pack_signs(rs).numpy(), h128=h.numpy())

    # ---- random packed linears (every bit pattern is a valid stream)
    for K in (2, 3, 4, 5):
        g = torch.Generator().manual_seed(4000 + K)
        m, n, M = 256, 384, 3
        qw = torch.randint(-(2 ** 31), 2 ** 31, (m // 16, n // 16, 8 * K), dtype=torch.int32, generator=g)
        sc = (torch.randn(m, generator=g).abs() * 0.01 + 0.01).half()
        su = torch.randint(0, 256, (n // 8,), dtype=torch.uint8, generator=g)
        sv = torch.randint(0, 256, (m // 8,), dtype=torch.uint8, generator=g)
        x = torch.randn(M, n, generator=g).bfloat16()
        bias = torch.randn(m, generator=g).bfloat16()
        W = wire.dequant(qw, sc, su, sv)
        y = x.float() @ W.T
        xt = wire.blk_had_cols_T(x.float() * wire.unpack_signs(su, n)[None, :])
        np.savez_compressed(os.path.join(out, f"linear_K{K}.npz"), qweight=qw.numpy(), scales=sc.numpy(), su=su.numpy(),
                            sv=sv.numpy(), x_f32=x.float().numpy(), bias_f32=bias.float().numpy(),
                            W=W.numpy(), y=y.numpy(), y_bias=(y + bias.float()[None, :]).numpy(), xt=xt.numpy())

    # ---- encoder round trip of tests/test_release.py:53-73
    g = torch.Generator().manual_seed(12)
    w = torch.randn(128, 128, generator=g) * 0.02
    old = encode.VITERBI
    encode.VITERBI = None
    try:
        r = encode.encode_group([{"W": w, "H": torch.eye(128)}], 4, max_batch=8)[0]
        assert torch.equal(wire.dequant(r["qweight"], r["scales"], r["su"], r["sv"]), r["What"])
        np.savez_compressed(os.path.join(out, "encoded_K4.npz"), W_in=w.numpy(), qweight=r["qweight"].numpy(),
                            scales=r["scales"].numpy(), su=r["su"].numpy(), sv=r["sv"].numpy(), What=r["What"].numpy())
        # Hessian-weighted encodes: X ~ N(0,1) with 1% of channels x10, H = X^T X / rows
        for K in (2, 3):
            g = torch.Generator().manual_seed(900 + K)
            m, n = 128, 256
            w = torch.randn(m, n, generator=g) * 0.02
            X = torch.randn(512, n, generator=g)
            hot = torch.randperm(n, generator=g)[: max(1, n // 100)]
            X[:, hot] *= 10.0
            H = X.T @ X / X.shape[0]
            r = encode.encode_group([{"W": w, "H": H}], K, seed=1234, max_batch=64)[0]
            x = torch.randn(2, n, generator=g).bfloat16()
            np.savez_compressed(os.path.join(out, f"encoded_hessian_K{K}.npz"), W_in=w.numpy(), qweight=r["qweight"].numpy(),
                                scales=r["scales"].numpy(), su=r["su"].numpy(), sv=r["sv"].numpy(), What=r["What"].numpy(),
                                x_f32=x.float().numpy(), y=(x.float() @ r["What"].T).numpy())
    finally:
        encode.VITERBI = old
    print("wrote fixtures to", out)


def encode_fixture(out):
    """A group of two matrices that share their input (as gate/up or q/k/v members do), encoded by the reference."""
    from htr import encode

    g = torch.Generator().manual_seed(4242)
    n = 256
    X = torch.randn(512, n, generator=g)
    X[:, torch.randperm(n, generator=g)[:3]] *= 10.0
    H = X.T @ X / X.shape[0]
    Ws = [torch.randn(128, n, generator=g) * 0.02, torch.randn(256, n, generator=g) * 0.03]
    old, encode.VITERBI = encode.VITERBI, None
    try:
        res = encode.encode_group([{"W": w, "H": H} for w in Ws], 3, seed=1234, max_batch=64)
    finally:
        encode.VITERBI = old
    d = {"H": H.numpy()}
    for i, (w, r) in enumerate(zip(Ws, res)):
        err = (w - r["What"]).double()
        d[f"W{i}"], d[f"qweight{i}"], d[f"scales{i}"] = w.numpy(), r["qweight"].numpy(), r["scales"].numpy()
        d[f"su{i}"], d[f"sv{i}"] = r["su"].numpy(), r["sv"].numpy()          # What = wire.dequant of these four (htr/encode.py:103-105)
        d[f"proxy{i}"] = np.float64(torch.trace(err @ H.double() @ err.T))
        print(i, "proxy loss", float(d[f"proxy{i}"]))
    np.savez_compressed(os.path.join(out, "encode_K3.npz"), **d)
    print("wrote", os.path.join(out, "encode_K3.npz"))


def viterbi_fixture(out):
    """Inputs shaped like the encoder's calls (htr/encode.py:77-86): targets = rows of a rotated weight divided by the row
    scale (about unit variance in codebook units), weights = squared row scales normalised to mean 1 per tile."""
    from htr import reference, wire

    cb = wire.codebook_f32()
    d = {}
    cases = [(2, 3, True), (3, 3, True), (4, 3, True), (5, 3, True), (4, 2, False), (6, 1, True), (8, 1, True)]
    for K, B, tb in cases:
        g = torch.Generator().manual_seed(100 * K + int(tb))
        x = torch.randn(B, 256, generator=g) * (1.0 + 0.25 * torch.rand(B, 1, generator=g))
        x[0, :5] *= 4.0                                             # a few outliers beyond the codebook range
        rs = (torch.rand(B, 16, generator=g) + 0.5).repeat_interleave(16, dim=1) ** 2
        w = rs / rs.mean(dim=1, keepdim=True)
        st = reference.viterbi(x, w, cb, K, tailbite=tb)
        cost = (w * (x - cb[st]) ** 2).sum(dim=1)
        tag = f"K{K}" + ("" if tb else "_open")
        d[tag + "_x"], d[tag + "_w"] = x.numpy(), w.numpy()
        d[tag + "_states"], d[tag + "_cost"] = st.numpy().astype(np.int32), cost.numpy()
        print(tag, "cost", cost.tolist())
    np.savez_compressed(os.path.join(out, "viterbi.npz"), **d)
    print("wrote", os.path.join(out, "viterbi.npz"))


if __name__ == "__main__":
    main()
