"""Encoder-side trellis search on the GPU: the callable the reference's encoder expects behind `encode.VITERBI`.

The reference's encoder (htr/encode.py:46-110) quantises one 16-column block of all rows at a time and hands the resulting
[tiles, 256] targets to `VITERBI(x, w, cb, K) -> states int64 [tiles, 256]` (htr/encode.py:7,48,86); its portable
implementation is htr/reference.py:7-50 (31-53 ms per tile on a CPU core) and its CUDA one (htr/vit_v2.py) is built for
sm_86 / sm_120 only.  `viterbi` below has that signature and runs `htr_viterbi` of the library on sm_100a; a maintainer of the
reference switches with

    from htr import encode; from htr_b200 import encoder; encode.VITERBI = encoder.viterbi

`pack` turns states into the HTR-W1 words of a tile (htr/wire.py:33-43), so that search -> pack -> `htr_decode_raw` closes the
loop on the device.
"""
import torch

from . import _lib, wire

_WS = {}


def _workspace(device, nbytes):
    buf = _WS.get(device.index)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        _WS[device.index] = buf
    return buf


def codebook_f32(device):
    """cb[s] = float32(v(s) / rms) for all 65536 states, computed by the device function the search uses."""
    out = torch.empty(65536, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(_lib.lib.htr_codebook_f32(out.data_ptr(), torch.cuda.current_stream(device).cuda_stream), "htr_codebook_f32")
    return out


def viterbi(x, w, cb=None, K=4, tailbite=True, return_cost=False):
    """x, w: [B, T] float targets and per-element weights on a CUDA device (T <= 256); returns int64 states [B, T]
    (and the float32 path costs with return_cost).  `cb` is accepted for signature compatibility with the reference's hook and
    must be the HTR-W1 codebook (it is spot-checked, not used: the kernel recomputes the values from the state hash)."""
    if not x.is_cuda:
        raise _lib.HTRError("htr_viterbi has no CPU path: tensors must live on a CUDA device")
    if x.dim() != 2 or w.shape != x.shape:
        raise _lib.HTRError("htr_viterbi: x and w must be [tiles, steps] of equal shape")
    B, T = x.shape
    if cb is not None:
        probe = torch.tensor([0, 1, 255, 4096, 65535], device=cb.device)
        if cb.numel() != 65536 or not torch.equal(cb.flatten()[probe].float().cpu(), torch.from_numpy(wire.codebook_f32()[probe.cpu().numpy()])):
            raise _lib.HTRError("htr_viterbi: cb is not the HTR-W1 codebook")
    x32, w32 = x.float().contiguous(), w.float().contiguous()
    states = torch.empty((B, T), dtype=torch.int32, device=x.device)
    total = torch.empty(B, dtype=torch.float32, device=x.device)
    if B:
        with torch.cuda.device(x.device):
            need = _lib.lib.htr_viterbi_workspace_bytes(B, T, int(K))
            if need == 0:
                raise _lib.HTRError(f"htr_viterbi: unsupported sizes B={B} T={T} K={K}")
            ws = _workspace(x.device, need)
            rc = _lib.lib.htr_viterbi(x32.data_ptr(), w32.data_ptr(), B, T, int(K), int(bool(tailbite)), states.data_ptr(), total.data_ptr(),
                                      ws.data_ptr(), ws.numel(), torch.cuda.current_stream(x.device).cuda_stream)
            _lib.check(rc, "htr_viterbi")
    out = states.long()
    return (out, total) if return_cost else out


def pack(states, K):
    """states [tiles, 256] (any integer dtype, any device) -> int32 words [tiles, 8K] of the circular stream."""
    return wire.pack_states(states.cpu(), K).to(states.device)
