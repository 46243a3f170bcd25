"""Operator boundary of the packed linear: `linear()` and the torch custom op `htr::linear`.

Same signature and meaning as htr/ops.py:107-122 of the reference, so a caller (the vLLM quantization
method, or any torch code) switches by importing this module instead.  The dispatch policy is re-derived
for one B200 (148 SMs, HBM3e) rather than copied from the 40-CU part the reference was tuned on:

  M == 0            empty result                                             (htr/ops.py:73-74)
  1 <= M <= 4       one launch of the streaming GEMV (activation transform, decode + dot, split reduce,
                    output transform fused)                                  (replaces htr/ops.py:75-76,95-101)
  4 < M <= 512      the tensor-core packed GEMM (tcgen05 + TMEM), up to 256 rows per launch (128 for float32
                    activations); decoded tiles go straight into the MMA operand    (replaces htr/ops.py:77-93).
                    The GEMV handles up to 8 rows and HTR_GEMV_ROUTE_MAX=8 keeps them there; measured, the GEMM wins from 5.
  M > 512           original-basis bf16 weight from the dequant kernel (decoded once), then a library GEMM
                                                                             (htr/ops.py:89-93)
  HTR_GEMM=0        instead: GEMV over 8-row chunks up to HTR_GEMV_LOOP_MAX rows, beyond that the original-basis bf16
                    weight from the dequant kernel + a library GEMM (the reference's own routes, kept for comparison)

All work is enqueued on the current torch stream without a host synchronisation, so the op can be
captured in a CUDA graph.  Nothing here runs on the CPU: without the CUDA library the import fails.
"""
import os
import threading

import torch

from . import _lib, wire

CB = wire.cbscale()
GEMV_MAX_M = _lib.GEMV_MAX_ROWS
GEMV_LOOP_MAX = int(os.environ.get("HTR_GEMV_LOOP_MAX", "64"))
USE_GEMM = os.environ.get("HTR_GEMM", "1") == "1"
GEMM_MAX_M = _lib.GEMM_MAX_ROWS
# above this many rows the weight is decoded once to bf16 and a library GEMM runs (the packed GEMM decodes once per 256-row launch)
GEMM_ROUTE_MAX = int(os.environ.get("HTR_GEMM_ROUTE_MAX", "512"))
# batches above this many rows leave the GEMV for the tensor-core GEMM (the GEMV itself handles up to 8 rows, but from 5 rows
# on the GEMM is faster: 25 us against 41-44 us at 4096x12288, 190 us against 384-408 us on the 151936x4096 head)
GEMV_ROUTE_MAX = min(GEMV_MAX_M, int(os.environ.get("HTR_GEMV_ROUTE_MAX", "4")))

class _ThreadState(threading.local):
    flags = 0       # flags of htr_linear_ex applied to every GEMV launch of this thread (see independent_inputs)


_STATE = _ThreadState()

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}
_WORKSPACES = {}
_NEED = {}
_MIN_WORKSPACE = 1 << 22


def workspace(device, nbytes, stream=None):
    """Scratch of the GEMV (split partial sums + arrival counters), one per (device, stream).

    The counters at its start must be zero before first use and every launch leaves them zero, so the buffer
    is zero-filled once and then reused (the reference keeps a per-device `counters` tensor the same way,
    htr/ops.py:24-28).  Calls on different streams get different buffers."""
    stream = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
    key = (device.index, stream)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(_MIN_WORKSPACE, 1 << (int(nbytes) - 1).bit_length())
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf


def _check(x2, qweight, scales, su, sv, bias):
    if not x2.is_cuda:
        raise _lib.HTRError("htr::linear has no CPU path: tensors must live on a CUDA device")
    if x2.dtype not in _DTYPES:
        raise _lib.HTRError(f"htr::linear: unsupported activation dtype {x2.dtype}")
    if qweight.dtype != torch.int32 or qweight.dim() != 3 or qweight.shape[2] % 8:
        raise _lib.HTRError("htr::linear: qweight must be int32 [m/16, n/16, 8K]")
    mt, nt, W = qweight.shape
    if x2.shape[1] != nt * 16:
        raise _lib.HTRError(f"htr::linear: activations have {x2.shape[1]} columns, the weight expects {nt * 16}")
    if scales.dtype != torch.float16 or scales.numel() != mt * 16:
        raise _lib.HTRError("htr::linear: scales must be float16 [m]")
    if su.dtype != torch.uint8 or su.numel() != nt * 2 or sv.dtype != torch.uint8 or sv.numel() != mt * 2:
        raise _lib.HTRError("htr::linear: su / sv must be uint8 [n/8] / [m/8]")
    if bias is not None and (bias.dtype != x2.dtype or bias.numel() != mt * 16):
        raise _lib.HTRError("htr::linear: bias must have the activation dtype and m elements")


def _gemv(x2, qweight, scales, su, sv, bias, out):
    """One C call: rows of x2 (<= 8) against the packed weight, result written into `out`."""
    M = x2.shape[0]
    mt, nt, W = qweight.shape
    K = W // 8
    key = (x2.device.index, M, mt, nt, K)
    need = _NEED.get(key)
    if need is None:
        need = _lib.lib.htr_linear_workspace_bytes(M, mt * 16, nt * 16, K)
        if need == 0:
            _lib.check(_lib.lib.htr_linear_plan(M, mt * 16, nt * 16, K, None, None), "htr_linear")
        _NEED[key] = need
    ws = workspace(x2.device, need)
    st = torch.cuda.current_stream(x2.device).cuda_stream
    rc = _lib.lib.htr_linear_ex(x2.data_ptr(), _DTYPES[x2.dtype], M, qweight.data_ptr(), mt, nt, K, scales.data_ptr(), su.data_ptr(),
                                sv.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), st,
                                _STATE.flags)
    _lib.check(rc, "htr_linear")


def linear_padded(x, qweight, scales, su, sv, bias=None, m_out=None):
    """Packed linear whose stored tensors cover a zero-padded [m_pad, n_pad] matrix: x[..., n_in] with n_in <= n_pad,
    result [..., m_out] with m_out <= m_pad (bias, if any, has m_out elements).

    The reference's `HTRHCLinearMethod.apply` (htr/vllm_plugin.py:313-326) pads the input with `F.pad` and slices the output
    with `.contiguous()`; here both happen inside the kernel (missing columns are read as zeros, rows beyond m_out are not
    written).  n_in and m_out must be multiples of 8.  Batches above 8 rows run as 8-row launches."""
    mt, nt, W = qweight.shape
    m_out = mt * 16 if m_out is None else int(m_out)
    n_in = x.shape[-1]
    x2 = x.reshape(-1, n_in).contiguous()
    if not x2.is_cuda:
        raise _lib.HTRError("htr::linear has no CPU path: tensors must live on a CUDA device")
    if x2.dtype not in _DTYPES:
        raise _lib.HTRError(f"htr::linear: unsupported activation dtype {x2.dtype}")
    if bias is not None and (bias.dtype != x2.dtype or bias.numel() != m_out):
        raise _lib.HTRError("htr::linear: bias must have the activation dtype and m_out elements")
    M, K = x2.shape[0], W // 8
    y = torch.empty((M, m_out), dtype=x2.dtype, device=x2.device)
    if M:
        qweight, scales, su, sv = qweight.contiguous(), scales.contiguous(), su.contiguous(), sv.contiguous()
        with torch.cuda.device(x2.device):
            st = torch.cuda.current_stream(x2.device).cuda_stream
            for r0 in range(0, M, GEMV_MAX_M):
                rows = min(GEMV_MAX_M, M - r0)
                ws = workspace(x2.device, _lib.lib.htr_linear_workspace_bytes(rows, mt * 16, nt * 16, K))
                rc = _lib.lib.htr_linear_padded(x2[r0:].data_ptr(), _DTYPES[x2.dtype], rows, n_in, qweight.data_ptr(), mt, nt, K,
                                                scales.data_ptr(), su.data_ptr(), sv.data_ptr(), None if bias is None else bias.data_ptr(),
                                                y[r0:].data_ptr(), m_out, ws.data_ptr(), ws.numel(), st)
                _lib.check(rc, "htr_linear_padded")
    return y.reshape(*x.shape[:-1], m_out)


PROLOGUE_NONE, PROLOGUE_RMSNORM, PROLOGUE_SWIGLU = 0, 1, 2


def linear_fused(x2, qweight, scales, su, sv, out=None, prologue=PROLOGUE_NONE, norm_weight=None, eps=0.0, residual=False):
    """GEMV with the element-wise neighbours of a decoder layer folded in (bf16, at most 8 rows; `htr_linear_fused`):

      prologue=PROLOGUE_RMSNORM  the linear sees rmsnorm(x2) * norm_weight
      prologue=PROLOGUE_SWIGLU   x2 is [rows, 2n] = [gate | up]; the linear sees silu(gate) * up
      residual=True              `out` is the residual stream [rows, m]: out += result, in place

    Returns `out` (allocated when not given and residual is False).  The reference runs these steps as separate kernels of its
    serving stack; results equal the unfused bf16 operators up to the summation order of the norm."""
    if x2.dtype != torch.bfloat16 or not x2.is_cuda or x2.dim() != 2:
        raise _lib.HTRError("htr_linear_fused: activations must be a 2-D bf16 CUDA tensor")
    M = x2.shape[0]
    mt, nt, W = qweight.shape
    K = W // 8
    cols = nt * 16 * (2 if prologue == PROLOGUE_SWIGLU else 1)
    if x2.shape[1] != cols or M > GEMV_MAX_M or not x2.is_contiguous():
        raise _lib.HTRError(f"htr_linear_fused: activations must be contiguous [rows <= {GEMV_MAX_M}, {cols}]")
    if out is None:
        if residual:
            raise _lib.HTRError("htr_linear_fused: residual=True needs the residual stream as `out`")
        out = torch.empty((M, mt * 16), dtype=x2.dtype, device=x2.device)
    elif out.dtype != x2.dtype or tuple(out.shape) != (M, mt * 16) or not out.is_contiguous():
        raise _lib.HTRError("htr_linear_fused: `out` must be a contiguous bf16 [rows, m] tensor")
    if M == 0:
        return out
    with torch.cuda.device(x2.device):
        ws = workspace(x2.device, _lib.lib.htr_linear_workspace_bytes(M, mt * 16, nt * 16, K))
        rc = _lib.lib.htr_linear_fused(x2.data_ptr(), M, qweight.data_ptr(), mt, nt, K, scales.data_ptr(), su.data_ptr(), sv.data_ptr(),
                                       out.data_ptr(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(x2.device).cuda_stream,
                                       int(prologue), None if norm_weight is None else norm_weight.data_ptr(), float(eps), int(bool(residual)))
        _lib.check(rc, "htr_linear_fused")
    return out


_GEMM_WS = {}


def _gemm(x2, qweight, scales, su, sv, bias, out, peer_ptrs=None, elem_offset=0):
    """One C call of the tensor-core GEMM: up to 256 rows of x2 (128 for float32) against the packed weight.  With peer_ptrs the
    rows go to element offset `elem_offset` of every buffer in the list instead of `out` (htr_linear_gemm_peers)."""
    M = x2.shape[0]
    mt, nt, W = qweight.shape
    K = W // 8
    need = _lib.lib.htr_linear_gemm_workspace_bytes(M, mt * 16, nt * 16, K)
    if need == 0:
        raise _lib.HTRError("htr_linear_gemm: unsupported sizes")
    st = torch.cuda.current_stream(x2.device).cuda_stream
    key = (x2.device.index, st)
    ws = _GEMM_WS.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 24), dtype=torch.uint8, device=x2.device)
        _GEMM_WS[key] = ws
    if peer_ptrs is None:
        rc = _lib.lib.htr_linear_gemm(x2.data_ptr(), _DTYPES[x2.dtype], M, qweight.data_ptr(), mt, nt, K, scales.data_ptr(), su.data_ptr(),
                                      sv.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), st)
    else:
        import ctypes

        arr = (ctypes.c_void_p * len(peer_ptrs))(*[int(p) for p in peer_ptrs])
        rc = _lib.lib.htr_linear_gemm_peers(x2.data_ptr(), _DTYPES[x2.dtype], M, qweight.data_ptr(), mt, nt, K, scales.data_ptr(),
                                            su.data_ptr(), sv.data_ptr(), None if bias is None else bias.data_ptr(), arr, len(peer_ptrs),
                                            int(elem_offset), ws.data_ptr(), ws.numel(), st)
    _lib.check(rc, "htr_linear_gemm")


def gemm_into_peers(x2, qweight, scales, su, sv, bias, peer_ptrs, elem_offset):
    """Row-shard form of the tensor-core GEMM (5 .. 256 activation rows, one launch): the result rows [M, m_local] are stored, from
    inside the kernel, at element offset `elem_offset` of every buffer in `peer_ptrs`; the caller orders the ranks afterwards."""
    _check(x2, qweight, scales, su, sv, bias)
    _gemm(x2, qweight, scales, su, sv, bias, None, peer_ptrs, elem_offset)


def gemm_error_codes():
    """Status words of the GEMM workspaces (synchronises; for tests): non-zero means a bounded device-side wait expired."""
    off = _lib.lib.htr_linear_gemm_error_offset()
    return [int(ws[off:off + 4].view(torch.int32).item()) for ws in _GEMM_WS.values()]


def linear_into_peers(x2, qweight, scales, su, sv, bias, peer_ptrs, elem_offset, flag_ptrs=None):
    """Row-shard form of the GEMV (M <= 8): the result rows [M, m_local] are stored, from inside the kernel, at element
    offset `elem_offset` of every buffer in `peer_ptrs` (device addresses of the gather buffers of all ranks as mapped
    into this process).  Nothing is returned.  With `flag_ptrs` (the addresses of this rank's delivery word in every rank's
    flag array) the kernel also signals the peers when its rows have arrived (htr_linear_peers_signal) and the consumers order
    themselves with `peer_wait`; without it the caller orders the ranks (a barrier) before reading the buffers."""
    _check(x2, qweight, scales, su, sv, bias)
    M = x2.shape[0]
    if not 1 <= M <= GEMV_MAX_M:
        raise _lib.HTRError("linear_into_peers handles 1..8 activation rows")
    mt, nt, W = qweight.shape
    K = W // 8
    need = _lib.lib.htr_linear_workspace_bytes(M, mt * 16, nt * 16, K)
    ws = workspace(x2.device, need)
    st = torch.cuda.current_stream(x2.device).cuda_stream
    import ctypes

    arr = (ctypes.c_void_p * len(peer_ptrs))(*[int(p) for p in peer_ptrs])
    if flag_ptrs is None:
        rc = _lib.lib.htr_linear_peers(x2.data_ptr(), _DTYPES[x2.dtype], M, qweight.data_ptr(), mt, nt, K, scales.data_ptr(), su.data_ptr(),
                                       sv.data_ptr(), None if bias is None else bias.data_ptr(), None, arr, len(peer_ptrs), int(elem_offset),
                                       ws.data_ptr(), ws.numel(), st, _STATE.flags)
    else:
        farr = (ctypes.c_void_p * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
        rc = _lib.lib.htr_linear_peers_signal(x2.data_ptr(), _DTYPES[x2.dtype], M, qweight.data_ptr(), mt, nt, K, scales.data_ptr(),
                                              su.data_ptr(), sv.data_ptr(), None if bias is None else bias.data_ptr(), arr, farr,
                                              len(peer_ptrs), int(elem_offset), ws.data_ptr(), ws.numel(), st, _STATE.flags)
    _lib.check(rc, "htr_linear_peers")


def peer_wait(flags, epoch, nranks, status=None, count=1):
    """Consumer side of the delivery flags (htr_peer_wait): wait, on the current stream, until every rank has delivered `count`
    more times into this GPU's buffer.  flags: int32 CUDA tensor [nranks] (this GPU's words), epoch / status: int32 CUDA tensors [1]."""
    st = torch.cuda.current_stream(flags.device).cuda_stream
    rc = _lib.lib.htr_peer_wait(flags.data_ptr(), epoch.data_ptr(), int(nranks), int(count), None if status is None else status.data_ptr(), st)
    _lib.check(rc, "htr_peer_wait")


def peer_barrier(peer_words, flags, epoch, nranks, status=None):
    """Barrier across the ranks of one NVLink box on the current stream (htr_peer_barrier: one small kernel per rank, bounded wait).
    peer_words: int64 CUDA tensor [nranks] with the address of this rank's word in every rank's flag array; flags: int32 CUDA
    tensor (this GPU's words); epoch / status: int32 CUDA tensors [1]."""
    st = torch.cuda.current_stream(flags.device).cuda_stream
    rc = _lib.lib.htr_peer_barrier(peer_words.data_ptr(), flags.data_ptr(), epoch.data_ptr(), int(nranks),
                                   None if status is None else status.data_ptr(), st)
    _lib.check(rc, "htr_peer_barrier")


def linear_grouped(x_ptrs, qw_ptrs, sc_ptrs, su_ptrs, sv_ptrs, y_ptrs, mt, nt, K, dtype):
    """`count` packed linears of one shape in one launch, one activation row each (htr_linear_grouped).  Every argument is
    an int64 CUDA tensor of `count` device addresses (built on the device, e.g. by indexing per-expert address tables with
    the routing result), so the call needs no host synchronisation and can be captured in a CUDA graph."""
    count = x_ptrs.numel()
    dev = x_ptrs.device
    need = _lib.lib.htr_linear_grouped_workspace_bytes(count, mt * 16, nt * 16, K)
    if need == 0:
        raise _lib.HTRError("htr_linear_grouped: unsupported sizes")
    ws = workspace(dev, need)
    st = torch.cuda.current_stream(dev).cuda_stream
    rc = _lib.lib.htr_linear_grouped(x_ptrs.data_ptr(), _DTYPES[dtype], qw_ptrs.data_ptr(), mt, nt, K, sc_ptrs.data_ptr(), su_ptrs.data_ptr(),
                                     sv_ptrs.data_ptr(), y_ptrs.data_ptr(), count, ws.data_ptr(), ws.numel(), st)
    _lib.check(rc, "htr_linear_grouped")


def linear_routed(x, route, tables, mt, nt, K, x_div=1, prologue=PROLOGUE_NONE, out=None, peer_ptrs=None, share=1):
    """One launch over `route.numel()` problems (htr_linear_routed): problem i multiplies activation row i // x_div of `x` by the
    packed matrix whose four tensor addresses sit in row route[i] of `tables` (four int64 CUDA tensors, one row per expert; a
    zero weight address, or a route entry outside the tables, skips the problem) and writes row i of the result [count, m].  With prologue=PROLOGUE_SWIGLU the rows of
    x are [gate | up] of 2n bf16 values.  Nothing touches the host: the routing result stays on the device.
    peer_ptrs (a list of device addresses: the [count, m] result matrix of every rank of an NVLink box as mapped into this process,
    this rank's `out` among them) turns the launch into htr_linear_routed_peers: each row this rank computes is stored into all of them."""
    count = route.numel()
    dev = x.device
    if route.dtype != torch.int64 or not route.is_cuda or not x.is_contiguous() or x.dim() != 2:
        raise _lib.HTRError("htr_linear_routed: route must be an int64 CUDA tensor and x a contiguous matrix")
    if out is None:
        out = torch.empty((count, mt * 16), dtype=x.dtype, device=dev)
    need = _lib.lib.htr_linear_grouped_workspace_bytes(max(count, 1), mt * 16, nt * 16, K)
    if need == 0:
        raise _lib.HTRError("htr_linear_routed: unsupported sizes")
    with torch.cuda.device(dev):
        ws = workspace(dev, need)
        st = torch.cuda.current_stream(dev).cuda_stream
        if peer_ptrs is None and share <= 1:
            rc = _lib.lib.htr_linear_routed(x.data_ptr(), _DTYPES[x.dtype], int(x_div), x.shape[1], route.data_ptr(), count, int(tables[0].numel()),
                                            tables[0].data_ptr(), tables[1].data_ptr(), tables[2].data_ptr(), tables[3].data_ptr(), mt, nt, K,
                                            out.data_ptr(), int(prologue), ws.data_ptr(), ws.numel(), st)
        else:
            import ctypes

            peers = [] if peer_ptrs is None else [int(v) for v in peer_ptrs]
            host = (ctypes.c_void_p * max(len(peers), 1))(*peers)
            rc = _lib.lib.htr_linear_routed_peers(x.data_ptr(), _DTYPES[x.dtype], int(x_div), x.shape[1], route.data_ptr(), count,
                                                  int(tables[0].numel()), tables[0].data_ptr(), tables[1].data_ptr(), tables[2].data_ptr(),
                                                  tables[3].data_ptr(), mt, nt, K, out.data_ptr(), host if peers else None, len(peers),
                                                  int(share), int(prologue), ws.data_ptr(), ws.numel(), st)
        _lib.check(rc, "htr_linear_routed")
    return out


class independent_inputs:
    """Context manager: inside it, every packed linear promises that its activations, bias and output are not
    touched by the kernel launched just before it on the stream (e.g. the experts of one MoE layer, or the
    shards of one activation).  Such launches overlap their predecessor completely (HTR_LINEAR_INPUT_INDEPENDENT)."""

    def __enter__(self):
        self._old = _STATE.flags
        _STATE.flags = self._old | _lib.INPUT_INDEPENDENT
        return self

    def __exit__(self, *exc):
        _STATE.flags = self._old
        return False


class exact_sums:
    """Context manager: inside it, packed linears of up to four rows run on the kernel that accumulates in exact integers
    (HTR_LINEAR_EXACT_SUMS), whose results do not depend on the launch decomposition: row shards of a linear then reproduce the
    unsharded result bit for bit.  Calls the integer kernel cannot serve are unaffected."""

    def __enter__(self):
        self._old = _STATE.flags
        _STATE.flags = self._old | _lib.EXACT_SUMS
        return self

    def __exit__(self, *exc):
        _STATE.flags = self._old
        return False


def _linear_impl(x2, qweight, scales, su, sv, bias):
    _check(x2, qweight, scales, su, sv, bias)
    M = x2.shape[0]
    mt = qweight.shape[0]
    if M == 0:
        return x2.new_empty((0, mt * 16))
    qweight, scales, su, sv = qweight.contiguous(), scales.contiguous(), su.contiguous(), sv.contiguous()
    bias = None if bias is None else bias.contiguous()
    with torch.cuda.device(x2.device):
        if GEMV_ROUTE_MAX < M <= GEMM_ROUTE_MAX and USE_GEMM:
            y = torch.empty((M, mt * 16), dtype=x2.dtype, device=x2.device)
            step = _lib.GEMM_MAX_ROWS_F32 if x2.dtype == torch.float32 else GEMM_MAX_M
            for r0 in range(0, M, step):
                r1 = min(M, r0 + step)
                _gemm(x2[r0:r1], qweight, scales, su, sv, bias, y[r0:r1])
            return y
        if M <= GEMV_LOOP_MAX and not (USE_GEMM and M > GEMV_MAX_M):
            y = torch.empty((M, mt * 16), dtype=x2.dtype, device=x2.device)
            for r0 in range(0, M, GEMV_MAX_M):
                r1 = min(M, r0 + GEMV_MAX_M)
                _gemv(x2[r0:r1], qweight, scales, su, sv, bias, y[r0:r1])
            return y
        W = wire.dequant(qweight, scales, su, sv, dtype=torch.bfloat16 if x2.dtype == torch.float32 else x2.dtype)
        return torch.nn.functional.linear(x2, W.to(x2.dtype), bias)


@torch.library.custom_op("htr::linear", mutates_args=())
def htr_linear_op(x2: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, su: torch.Tensor, sv: torch.Tensor,
                  bias: torch.Tensor | None) -> torch.Tensor:
    return _linear_impl(x2.contiguous(), qweight, scales, su, sv, bias)


@htr_linear_op.register_fake
def _(x2, qweight, scales, su, sv, bias):
    return x2.new_empty((x2.shape[0], qweight.shape[0] * 16))


def linear(x, qweight, scales, su, sv, bias=None):
    """y = x @ W^T (+ bias) for an HTR-W1 weight; x [..., n] -> [..., m] in x.dtype (htr/ops.py:118-122)."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if torch.compiler.is_compiling():
        y = htr_linear_op(x2, qweight, scales, su, sv, bias)      # traced programs see the registered op
    else:
        y = _linear_impl(x2.contiguous(), qweight, scales, su, sv, bias)   # eager: skip the dispatcher round trip
    return y.reshape(*lead, qweight.shape[0] * 16)
