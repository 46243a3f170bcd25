"""CPU oracle for the HTR-W1 packed-linear decode path.  TEST INFRASTRUCTURE ONLY.

Two independent restatements of the reference's CPU decoder (htr/wire.py) and of the
dense contraction it feeds (htr/ops.py:93):

* numpy functions in this file (vectorised, written from the format text), and
* the C library ``htr_oracle.c`` beside it, reached through :class:`COracle`.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
The product package never does; it fails loudly when its CUDA library is missing.

Parity pin: both restatements are compared with fixtures produced by *running* the
reference's htr/wire.py (tests/golden/make_golden.py) and with the vectors of the
reference's tests/test_release.py (:28-38 bit layout, :40-43 sign byte, :45-47 Hadamard,
:53-73 encoder round trip).
"""
import ctypes
import os
import subprocess

import numpy as np

MUL, ADD = 0xDF6ADF, 0x34983
HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhtr_oracle.so")


# ----------------------------------------------------------------------------- numpy restatement
def gen_values(states):
    """v(s) = bytesum((s*0xDF6ADF + 0x34983) mod 2^32) - 510  (htr/wire.py:10-13)."""
    x = (np.asarray(states).astype(np.uint64) * np.uint64(MUL) + np.uint64(ADD)) & np.uint64(0xFFFFFFFF)
    total = np.zeros(x.shape, dtype=np.int64)
    for sh in (0, 8, 16, 24):
        total += ((x >> np.uint64(sh)) & np.uint64(0xFF)).astype(np.int64)
    return total - 510


def value_table():
    return gen_values(np.arange(65536))


def cbscale():
    """1/rms of the 65536 codebook integers in float64 (htr/wire.py:27-30)."""
    v = value_table().astype(np.float64)
    return float(1.0 / np.sqrt(np.mean(v * v)))


def codebook_f32():
    """cb[s] = float32(v/rms64) (htr/wire.py:19-24)."""
    v = value_table().astype(np.float64)
    return (v / np.sqrt(np.mean(v * v))).astype(np.float32)


def stream_bits(words):
    """[B, 8K] words -> [B, 256K] bits, word p>>5, bit 31-(p&31) (htr/wire.py:46-51)."""
    u = np.asarray(words).astype(np.int64) & 0xFFFFFFFF
    be = u.astype(">u4").view(np.uint8).reshape(u.shape[0], -1)     # big-endian bytes == MSB-first stream
    return np.unpackbits(be, axis=1, bitorder="big").astype(np.int64)


def unpack_states(words, K):
    """s_t = the 16 stream bits ending at bit (t+1)K-1 of the circular stream (htr/wire.py:54-63)."""
    bits = stream_bits(words)
    nbits = 256 * K
    assert bits.shape[1] == nbits
    ends = (np.arange(256) + 1) * K                                  # one past the last bit of step t
    out = np.zeros((bits.shape[0], 256), dtype=np.int64)
    for back in range(16):                                           # bit `back` positions before the end has weight 2^back
        out |= bits[:, (ends - 1 - back) % nbits] << back
    return out


def pack_states(states, K):
    """Inverse of unpack_states for a tail-biting path: low K bits of each state, MSB first (htr/wire.py:33-43)."""
    st = np.asarray(states).astype(np.int64)
    fresh = st & ((1 << K) - 1)
    bits = np.stack([(fresh >> (K - 1 - j)) & 1 for j in range(K)], axis=-1).reshape(st.shape[0], 256 * K)
    by = np.packbits(bits.astype(np.uint8), axis=1, bitorder="big")
    return by.view(">u4").astype(np.uint32).view(np.int32).reshape(st.shape[0], 8 * K)


def decode_raw(words, K):
    """int16 codebook integers [ntiles, 256] in stream order."""
    return gen_values(unpack_states(words, K)).astype(np.int16)


def unpack_signs(packed, n):
    """LSB-first bits, set bit = -1 (htr/wire.py:72-74)."""
    bits = np.unpackbits(np.asarray(packed, dtype=np.uint8), bitorder="little")[:n]
    return (1.0 - 2.0 * bits).astype(np.float32)


def pack_signs(signs):
    return np.packbits((np.asarray(signs) < 0).astype(np.uint8), bitorder="little")


def hadamard128():
    """Sylvester H128/sqrt(128) as float32 (htr/wire.py:80-87)."""
    idx = np.arange(128)
    par = np.array([[bin(a & b).count("1") & 1 for b in idx] for a in idx])
    return ((1.0 - 2.0 * par) / np.sqrt(128.0)).astype(np.float32)


def blk_had(A):
    """Right-multiply every 128-column block by H128/sqrt(128) (htr/wire.py:90-92)."""
    r, c = A.shape
    return (A.reshape(r, c // 128, 128) @ hadamard128()).reshape(r, c)


def dequant_Q(qweight, scales):
    """Rotated-domain Q [m, n] float32 (htr/wire.py:95-102)."""
    mt, nt, W = qweight.shape
    st = unpack_states(qweight.reshape(-1, W), W // 8)
    tiles = codebook_f32()[st].reshape(mt, nt, 16, 16)
    Q = tiles.transpose(0, 2, 1, 3).reshape(mt * 16, nt * 16)
    return Q * np.asarray(scales).astype(np.float32)[:, None]


def dequant(qweight, scales, su8, sv8):
    """Original-basis W [m, n] float32, rows first then columns then signs (htr/wire.py:105-113)."""
    Q = dequant_Q(qweight, scales)
    m, n = Q.shape
    W = blk_had(np.ascontiguousarray(Q.T)).T
    W = blk_had(np.ascontiguousarray(W))
    return np.ascontiguousarray(W * unpack_signs(sv8, m)[:, None] * unpack_signs(su8, n)[None, :])


def rht(x, su8):
    """xt = blk_had(su * x): the activation transform of docs/FORMAT.md:8."""
    x = np.asarray(x, dtype=np.float32)
    return blk_had(x * unpack_signs(su8, x.shape[1])[None, :])


def linear(x, qweight, scales, su8, sv8, bias=None):
    """y = x @ dequant(...).T (+ bias), float64 accumulation, float32 result (htr/ops.py:93)."""
    W = dequant(qweight, scales, su8, sv8).astype(np.float64)
    y = np.asarray(x, dtype=np.float64) @ W.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)[None, :]
    return y.astype(np.float32)


def payload_bytes(m, n, K):
    """Packed payload of one linear: m*n*K/8 + 2m + n/8 + m/8 (docs/METHODOLOGY.md:89)."""
    return m * n * K // 8 + 2 * m + n // 8 + m // 8


# ----------------------------------------------------------------------------- C restatement
def build(force=False):
    """Compile htr_oracle.c beside this file (gcc, OpenMP).  Building the checker is not using it."""
    src = os.path.join(HERE, "htr_oracle.c")
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= os.path.getmtime(src):
        return LIB_PATH
    subprocess.run(["gcc", "-O3", "-march=x86-64-v2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-o", LIB_PATH, src, "-lm"], check=True)
    return LIB_PATH


def _p(a, ty):
    return a.ctypes.data_as(ctypes.POINTER(ty))


class COracle:
    """ctypes view of libhtr_oracle.so (same contract as the numpy functions above)."""

    def __init__(self, path=None):
        path = path or LIB_PATH
        if not os.path.exists(path):
            build()
        self.lib = ctypes.CDLL(path)
        self.lib.htro_cbscale.restype = ctypes.c_double
        self.lib.htro_gen_value.restype = ctypes.c_int

    def gen_value(self, s):
        return int(self.lib.htro_gen_value(ctypes.c_uint32(int(s))))

    def cbscale(self):
        return float(self.lib.htro_cbscale())

    def codebook_f32(self):
        cb = np.empty(65536, dtype=np.float32)
        self.lib.htro_codebook_f32(_p(cb, ctypes.c_float))
        return cb

    def unpack_states(self, words, K):
        w = np.ascontiguousarray(words).view(np.uint32)
        out = np.empty((w.shape[0], 256), dtype=np.uint16)
        rc = self.lib.htro_unpack_states(_p(w, ctypes.c_uint32), K, ctypes.c_size_t(w.shape[0]), _p(out, ctypes.c_uint16))
        assert rc == 0
        return out.astype(np.int64)

    def pack_states(self, states, K):
        st = np.ascontiguousarray(np.asarray(states).astype(np.uint16))
        out = np.empty((st.shape[0], 8 * K), dtype=np.uint32)
        rc = self.lib.htro_pack_states(_p(st, ctypes.c_uint16), K, ctypes.c_size_t(st.shape[0]), _p(out, ctypes.c_uint32))
        assert rc == 0
        return out.view(np.int32)

    def decode_raw(self, words, K):
        w = np.ascontiguousarray(words).view(np.uint32)
        out = np.empty((w.shape[0], 256), dtype=np.int16)
        rc = self.lib.htro_decode_raw(_p(w, ctypes.c_uint32), K, ctypes.c_size_t(w.shape[0]), _p(out, ctypes.c_int16))
        assert rc == 0
        return out

    def unpack_signs(self, packed, n):
        pk = np.ascontiguousarray(packed, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        self.lib.htro_unpack_signs(_p(pk, ctypes.c_uint8), ctypes.c_size_t(n), _p(out, ctypes.c_float))
        return out

    def pack_signs(self, signs):
        s = np.ascontiguousarray(signs, dtype=np.float32)
        out = np.empty(s.size // 8, dtype=np.uint8)
        self.lib.htro_pack_signs(_p(s, ctypes.c_float), ctypes.c_size_t(s.size), _p(out, ctypes.c_uint8))
        return out

    def hadamard128(self):
        h = np.empty((128, 128), dtype=np.float32)
        self.lib.htro_hadamard128(_p(h, ctypes.c_float))
        return h

    def dequant(self, qweight, scales, su8, sv8):
        qw = np.ascontiguousarray(qweight).view(np.uint32)
        mt, nt, W = qw.shape
        sc = np.ascontiguousarray(np.asarray(scales, dtype=np.float16)).view(np.uint16)
        su, sv = np.ascontiguousarray(su8, dtype=np.uint8), np.ascontiguousarray(sv8, dtype=np.uint8)
        out = np.empty((mt * 16, nt * 16), dtype=np.float32)
        rc = self.lib.htro_dequant(_p(qw, ctypes.c_uint32), _p(sc, ctypes.c_uint16), _p(su, ctypes.c_uint8),
                                   _p(sv, ctypes.c_uint8), mt, nt, W // 8, _p(out, ctypes.c_float))
        assert rc == 0
        return out

    def rht(self, x, su8):
        x = np.ascontiguousarray(x, dtype=np.float32)
        su = np.ascontiguousarray(su8, dtype=np.uint8)
        out = np.empty_like(x)
        rc = self.lib.htro_rht(_p(x, ctypes.c_float), x.shape[0], x.shape[1], _p(su, ctypes.c_uint8), _p(out, ctypes.c_float))
        assert rc == 0
        return out

    def linear(self, x, qweight, scales, su8, sv8, bias=None, threads=None):
        """Decode + contract, the reference's CPU path, on `threads` host cores (default: all)."""
        if threads:
            self.lib.htro_set_num_threads(int(threads))
        x = np.ascontiguousarray(x, dtype=np.float32)
        qw = np.ascontiguousarray(qweight).view(np.uint32)
        mt, nt, W = qw.shape
        sc = np.ascontiguousarray(np.asarray(scales, dtype=np.float16)).view(np.uint16)
        su, sv = np.ascontiguousarray(su8, dtype=np.uint8), np.ascontiguousarray(sv8, dtype=np.uint8)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        out = np.empty((x.shape[0], mt * 16), dtype=np.float32)
        rc = self.lib.htro_linear(_p(x, ctypes.c_float), x.shape[0], _p(qw, ctypes.c_uint32), _p(sc, ctypes.c_uint16),
                                  _p(su, ctypes.c_uint8), _p(sv, ctypes.c_uint8),
                                  None if b is None else _p(b, ctypes.c_float), mt, nt, W // 8, _p(out, ctypes.c_float))
        assert rc == 0
        return out

    def viterbi(self, x, w, K, tailbite=True, threads=None):
        """Tail-biting trellis search per row of x [B, T] with weights w (htr/reference.py:7-50).  Returns (states int32 [B, T],
        float32 [B] cost of the winning final state)."""
        if threads:
            self.lib.htro_set_num_threads(int(threads))
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        B, T = x.shape
        states = np.empty((B, T), dtype=np.int32)
        total = np.empty(B, dtype=np.float32)
        rc = self.lib.htro_viterbi(_p(x, ctypes.c_float), _p(w, ctypes.c_float), ctypes.c_size_t(B), T, int(K), int(bool(tailbite)),
                                   _p(states, ctypes.c_int32), _p(total, ctypes.c_float))
        assert rc == 0
        return states, total

    def path_cost(self, x, w, states):
        """Cost of a path under the same error measure, accumulated in float64."""
        self.lib.htro_path_cost.restype = ctypes.c_double
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        st = np.ascontiguousarray(states, dtype=np.int32)
        return float(self.lib.htro_path_cost(_p(x, ctypes.c_float), _p(w, ctypes.c_float), x.shape[-1], _p(st, ctypes.c_int32)))

    def num_threads(self):
        return int(self.lib.htro_num_threads())


if __name__ == "__main__":
    print(build(force=True))
