"""HTR-W1 wire helpers of the package (host side of htr/wire.py of the reference).

Decoding runs on the GPU through the C library (`decode_raw`, `dequant`); the helpers that only
*produce* wire tensors (sign and state packing, random fixtures) are small torch routines because the
offline encoder side calls them on the host.  There is no CPU decoder here.
"""
import math

import torch

from . import _lib

L = 16
S = 1 << L
GEN_A, GEN_B = 0xDF6ADF, 0x34983
WIDTHS = (2, 3, 4, 5, 6, 8)


def gen_values(states):
    """Codebook integer v(s) = bytesum((s*GEN_A + GEN_B) mod 2^32) - 510 (htr/wire.py:10-13)."""
    x = (states.to(torch.int64) * GEN_A + GEN_B) % (1 << 32)
    return (x % 256) + (x // 256 % 256) + (x // 65536 % 256) + (x // 16777216) - 510


_CBSCALE = None


def cbscale():
    """1/rms of v over all 65536 states, float64 (htr/wire.py:27-30)."""
    global _CBSCALE
    if _CBSCALE is None:
        v = gen_values(torch.arange(S)).double()
        _CBSCALE = 1.0 / math.sqrt(float((v * v).mean()))
    return _CBSCALE


def codebook_f32():
    """cb[s] = float32(v(s) / rms) with the division in float64 (htr/wire.py:19-24), as a numpy array of 65536 values."""
    v = gen_values(torch.arange(S)).double()
    return (v / v.pow(2).mean().sqrt()).float().numpy()


def pack_signs(s):
    """+-1 vector [N] -> uint8 [N/8], LSB-first, set bit = -1 (htr/wire.py:66-69)."""
    neg = (s.reshape(-1, 8) < 0).to(torch.int32)
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32, device=s.device)
    return (neg * weights).sum(-1).to(torch.uint8)


def unpack_signs(u8, N):
    """uint8 [N/8] -> float +-1 [N] (htr/wire.py:72-74)."""
    shifts = torch.arange(8, device=u8.device, dtype=torch.int32)
    bits = (u8.to(torch.int32)[:, None] >> shifts) & 1
    return (1 - 2 * bits).reshape(-1)[:N].float()


def pack_states(states, K):
    """Tail-biting state path int64 [B, 256] -> int32 words [B, 8K] (htr/wire.py:33-43)."""
    B, T = states.shape
    if T != 256 or not 2 <= K <= 8:
        raise ValueError("pack_states wants [B, 256] states and 2 <= K <= 8")
    fresh = states.to(torch.int64) & ((1 << K) - 1)
    # value of word w = sum of the steps' fresh bits shifted to their place in the 32-bit word
    pos = torch.arange(256, device=states.device) * K                      # first stream bit of each step
    words = torch.zeros(B, 8 * K, dtype=torch.int64, device=states.device)
    for j in range(K):                                                     # bit j of a step, MSB first
        p = pos + j
        words.scatter_add_(1, (p >> 5).expand(B, -1), ((fresh >> (K - 1 - j)) & 1) << (31 - (p & 31)))
    return torch.where(words >= 1 << 31, words - (1 << 32), words).to(torch.int32)


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def decode_raw(qweight):
    """int16 codebook integers [ntiles, 256] in stream order, decoded on the GPU
    (decode_raw of htr/csrc/htr_kernels.cpp:4; equals gen_values(unpack_states(words, K)))."""
    if not qweight.is_cuda or qweight.dtype != torch.int32:
        raise _lib.HTRError("decode_raw wants a CUDA int32 tensor")
    qw = qweight.contiguous()
    K = qw.shape[-1] // 8
    ntiles = qw.numel() // (8 * K) if K else 0
    out = torch.empty((ntiles, 256), dtype=torch.int16, device=qw.device)
    with torch.cuda.device(qw.device):
        _lib.check(_lib.lib.htr_decode_raw(qw.data_ptr(), ntiles, K, out.data_ptr(), _stream(qw)), "htr_decode_raw")
    return out


def dequant(qweight, scales, su8, sv8, dtype=torch.float32):
    """Original-basis W [m, n] = Sv Ho Q Hi Su on the GPU (htr/wire.py:105-113; dequant_w of the reference)."""
    if not qweight.is_cuda:
        raise _lib.HTRError("dequant wants CUDA tensors")
    code = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}[dtype]
    qw = qweight.contiguous()
    mt, nt, W = qw.shape
    out = torch.empty((mt * 16, nt * 16), dtype=dtype, device=qw.device)
    with torch.cuda.device(qw.device):
        _lib.check(_lib.lib.htr_dequant_w(qw.data_ptr(), mt, nt, W // 8, scales.contiguous().data_ptr(), su8.contiguous().data_ptr(),
                                          sv8.contiguous().data_ptr(), out.data_ptr(), code, _stream(qw)), "htr_dequant_w")
    return out


def payload_bytes(m, n, K):
    """Packed bytes of one linear: m*n*K/8 + 2m + n/8 + m/8 (docs/METHODOLOGY.md:89)."""
    return m * n * K // 8 + 2 * m + n // 8 + m // 8


def random_packed(m, n, K, seed, device="cpu"):
    """Synthetic HTR-W1 tensors: every bit pattern is a valid circular stream, so uniform random words,
    positive fp16 scales around 0.02 and uniform sign bytes make a well-formed weight."""
    g = torch.Generator().manual_seed(seed)
    qw = torch.randint(-(2 ** 31), 2 ** 31, (m // 16, n // 16, 8 * K), dtype=torch.int32, generator=g)
    sc = (torch.randn(m, generator=g).abs() * 0.01 + 0.01).half()
    su = torch.randint(0, 256, (n // 8,), dtype=torch.uint8, generator=g)
    sv = torch.randint(0, 256, (m // 8,), dtype=torch.uint8, generator=g)
    return tuple(t.to(device) for t in (qw, sc, su, sv))
