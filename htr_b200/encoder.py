"""Encoder-side trellis search on the GPU: the callable the reference's encoder expects behind `encode.VITERBI`.

The reference's encoder (htr/encode.py:46-110) quantises one 16-column block of all rows at a time and hands the resulting
[tiles, 256] targets to `VITERBI(x, w, cb, K) -> states int64 [tiles, 256]` (htr/encode.py:7,48,86); its portable
implementation is htr/reference.py:7-50 (31-53 ms per tile on a CPU core) and its CUDA one (htr/vit_v2.py) is built for
sm_86 / sm_120 only.  `viterbi` below has that signature and runs `htr_viterbi` of the library on sm_100a; a maintainer of the
reference switches with

    from htr import encode; from htr_b200 import encoder; encode.VITERBI = encoder.viterbi

`pack` turns states into the HTR-W1 words of a tile (htr/wire.py:33-43), so that search -> pack -> `htr_decode_raw` closes the
loop on the device.  `encode_group` is the whole encoder on the device (same algorithm and return values as
htr/encode.py:46-110: rotation by the sign vectors and block Hadamard transforms, Hessian damping, block LDLQ with error
feedback through the block-normalised Cholesky factor, trellis search per 16-column block, packing), so that a real matrix can be
turned into HTR-W1 tensors on a B200 in seconds; it exists for tests and benchmarks that want real encoder streams at full size.
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
    return wire.pack_states(states, K)


def _hadamard128(device, dtype):
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < 128:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h / 128 ** 0.5).to(dtype).to(device)


def _rotate_columns(A, H):
    """Block-diagonal 128-point transform of the columns: A [r, n] -> A . blockdiag(H) (H is symmetric)."""
    r, n = A.shape
    return (A.reshape(r, n // 128, 128) @ H).reshape(r, n)


def _rotate_both(A, H):
    return _rotate_columns(_rotate_columns(A, H).T.contiguous(), H).T.contiguous()


def sign_vectors(n, m, seed, index, shared_su=True):
    """The +-1 vectors of job `index` of a group, drawn as the reference draws them (htr/encode.py:20-32), so that encodes are
    reproducible across the two implementations."""
    def draw(count, gen):
        return (torch.randint(0, 2, (count,), generator=gen) * 2 - 1).float()

    if not shared_su:
        gen = torch.Generator().manual_seed(seed + 7919 * index)
        su = draw(n, gen)
        return su, draw(m, gen)
    return draw(n, torch.Generator().manual_seed(seed)), draw(m, torch.Generator().manual_seed(seed + 7919 * (index + 1)))


@torch.no_grad()
def encode_group(jobs, K, seed=1234, shared_su=True, damp=0.01, max_batch=4096):
    """jobs: list of dict(W=[m, n], H=[n, n]) that share n (and, with shared_su, their input sign vector: the members of a
    fused module).  Returns a list of dict(qweight int32 [m/16, n/16, 8K], scales fp16 [m], su u8 [n/8], sv u8 [m/8],
    What float32 [m, n] = the matrix the packed tensors decode to, Q = the quantised matrix in the rotated basis).
    Everything runs on the device of W; the trellis search is `viterbi` above."""
    dev = jobs[0]["W"].device
    n = jobs[0]["W"].shape[1]
    if n % 128:
        raise ValueError("encode_group: the input width must be a multiple of 128")
    blocks = n // 16
    H128 = _hadamard128(dev, torch.float32)
    cb = torch.from_numpy(wire.codebook_f32()).to(dev)
    work = []
    for index, job in enumerate(jobs):
        W = job["W"].float()
        m = W.shape[0]
        if m % 128 or W.shape[1] != n:
            raise ValueError("encode_group: every matrix must be [multiple of 128, n]")
        su, sv = (t.to(dev) for t in sign_vectors(n, m, seed, index, shared_su))
        Wr = _rotate_both(W * sv[:, None] * su[None, :], H128)                       # rotated weight
        Hr = _rotate_both(job["H"].float().to(dev) * su[:, None] * su[None, :], H128).double()
        dead = torch.diag(Hr) == 0                                                     # channels never seen in calibration
        Hr[dead, dead] = 1.0
        Wr[:, dead] = 0
        Hr += damp * torch.diag(Hr).mean() * torch.eye(n, device=dev, dtype=Hr.dtype)
        row_scale = Wr.pow(2).mean(dim=1).sqrt().half().float().clamp(min=1e-8)
        C = torch.linalg.cholesky(Hr)
        diag_blocks = C.view(blocks, 16, blocks, 16).diagonal(dim1=0, dim2=2).permute(2, 0, 1)      # [blocks, 16, 16]
        feedback = torch.einsum("ikj,kjl->ikl", C.view(n, blocks, 16), torch.linalg.inv(diag_blocks)).reshape(n, n).float()
        work.append(dict(Wr=Wr, rs=row_scale, L=feedback, su=su, sv=sv, Q=torch.zeros_like(Wr), F=torch.zeros_like(Wr),
                         S=torch.zeros((m // 16, blocks, 256), dtype=torch.int64, device=dev)))
    for k in range(blocks - 1, -1, -1):                                               # last block first: errors feed the earlier ones
        cols = slice(16 * k, 16 * k + 16)
        targets, weights = [], []
        for p in work:
            targets.append(((p["Wr"][:, cols] + p["F"][:, cols]) / p["rs"][:, None]).reshape(-1, 256))
            weights.append((p["rs"][:, None] ** 2).expand(-1, 16).contiguous().reshape(-1, 256))
        X = torch.cat(targets)
        Wt = torch.cat(weights)
        Wt = Wt / Wt.mean(dim=1, keepdim=True)
        states = torch.cat([viterbi(X[b:b + max_batch].contiguous(), Wt[b:b + max_batch].contiguous(), None, K)
                            for b in range(0, X.shape[0], max_batch)])
        values = cb[states]
        at = 0
        for p in work:
            tiles = p["S"].shape[0]
            p["S"][:, k] = states[at:at + tiles]
            q = values[at:at + tiles].reshape(-1, 16) * p["rs"][:, None]
            at += tiles
            p["Q"][:, cols] = q
            if k:
                p["F"][:, :16 * k] += (p["Wr"][:, cols] - q) @ p["L"][cols, :16 * k]
    out = []
    for p in work:
        mt = p["S"].shape[0]
        qweight = wire.pack_states(p["S"].reshape(-1, 256), K).reshape(mt, blocks, 8 * K)
        What = (_rotate_both(p["Q"], H128) * p["sv"][:, None] * p["su"][None, :]).contiguous()
        out.append(dict(qweight=qweight, scales=p["rs"].half(), su=wire.pack_signs(p["su"]), sv=wire.pack_signs(p["sv"]), What=What, Q=p["Q"]))
    return out
