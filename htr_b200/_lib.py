"""ctypes binding of libhtr_b200.so (the C interface declared in include/htr_b200.h).

There is no fallback: if the shared library has not been built (`python -m htr_b200.build`) importing
this module raises, and every operator of the package fails with it.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HTR_B200_LIB") or os.path.join(_HERE, "libhtr_b200.so")   # HTR_B200_LIB: alternative build

BF16, F16, F32 = 0, 1, 2
GEMV_MAX_ROWS = 8
GEMM_MAX_ROWS = 256
GEMM_MAX_ROWS_F32 = 128
INPUT_INDEPENDENT = 1
EXACT_SUMS = 2

EXPORTS = ("htr_status_string", "htr_last_cuda_error", "htr_version", "htr_decode_raw", "htr_rht",
           "htr_linear_workspace_bytes", "htr_linear_counter_bytes", "htr_linear", "htr_linear_ex", "htr_linear_peers", "htr_linear_grouped", "htr_linear_grouped_workspace_bytes", "htr_linear_routed", "htr_linear_static", "htr_linear_padded", "htr_linear_fused", "htr_linear_gemm", "htr_linear_gemm_peers", "htr_linear_gemm_workspace_bytes", "htr_linear_gemm_error_offset", "htr_linear_gemm_last_cuda_error", "htr_dequant_w", "htr_viterbi", "htr_viterbi_workspace_bytes", "htr_viterbi_last_cuda_error", "htr_codebook_f32",
           "htr_linear_plan", "htr_set_gemv_kernel", "htr_linear_fault_offset", "htr_linear_peers_signal", "htr_linear_routed_peers", "htr_peer_wait", "htr_peer_barrier", "htr_moe_combine_peers", "htr_moe_weighted_sum", "htr_rank_sum", "htr_dec_add_rmsnorm", "htr_dec_rope_cache", "htr_dec_attention",
           "htr_dec_swiglu", "htr_dec_rope_attention")


class HTRError(RuntimeError):
    """A C entry point returned a negative status (the reference raises RuntimeError from TORCH_CHECK)."""


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m htr_b200.build` (nvcc, sm_100a). "
                          "htr_b200 has no CPU or eager fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
    lib.htr_status_string.restype = ctypes.c_char_p
    lib.htr_status_string.argtypes = [i32]
    lib.htr_last_cuda_error.restype = i32
    lib.htr_version.restype = i32
    lib.htr_decode_raw.argtypes = [vp, i64, i32, vp, vp]
    lib.htr_rht.argtypes = [vp, i32, i32, i32, vp, vp, vp]
    lib.htr_linear_workspace_bytes.restype = sz
    lib.htr_linear_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.htr_linear_counter_bytes.restype = sz
    lib.htr_linear_counter_bytes.argtypes = [i32]
    lib.htr_linear.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.htr_linear_ex.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, sz, vp, ctypes.c_uint]
    lib.htr_linear_peers.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, ctypes.POINTER(vp), i32, i64, vp, sz, vp, ctypes.c_uint]
    lib.htr_linear_grouped.argtypes = [vp, i32, vp, i32, i32, i32, vp, vp, vp, vp, i32, vp, sz, vp]
    lib.htr_linear_routed.argtypes = [vp, i32, i32, i64, vp, i32, i32, vp, vp, vp, vp, i32, i32, i32, vp, i32, vp, sz, vp]
    lib.htr_linear_grouped_workspace_bytes.restype = sz
    lib.htr_linear_grouped_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.htr_linear_static.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp]
    lib.htr_linear_padded.argtypes = [vp, i32, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp, sz, vp]
    lib.htr_viterbi_workspace_bytes.restype = sz
    lib.htr_viterbi_workspace_bytes.argtypes = [i32, i32, i32]
    lib.htr_viterbi.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp, sz, vp]
    lib.htr_codebook_f32.argtypes = [vp, vp]
    lib.htr_linear_fused.argtypes = [vp, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, sz, vp, i32, vp, ctypes.c_float, i32]
    lib.htr_linear_gemm.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.htr_linear_gemm_peers.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, ctypes.POINTER(vp), i32, i64, vp, sz, vp]
    lib.htr_linear_gemm_workspace_bytes.restype = sz
    lib.htr_linear_gemm_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.htr_linear_gemm_error_offset.restype = sz
    lib.htr_dequant_w.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, i32, vp]
    lib.htr_dec_add_rmsnorm.argtypes = [vp, vp, vp, vp, i32, i32, ctypes.c_float, vp]
    lib.htr_dec_rope_cache.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]
    lib.htr_dec_attention.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]
    lib.htr_dec_swiglu.argtypes = [vp, vp, i32, i32, vp]
    lib.htr_dec_rope_attention.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
    lib.htr_linear_plan.argtypes = [i32, i32, i32, i32, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.htr_linear_peers_signal.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32, i64, vp, sz, vp, ctypes.c_uint]
    lib.htr_linear_routed_peers.argtypes = [vp, i32, i32, i64, vp, i32, i32, vp, vp, vp, vp, i32, i32, i32, vp, vp, i32, i32, i32, vp, sz, vp]
    lib.htr_peer_barrier.argtypes = [vp, vp, vp, i32, vp, vp]
    lib.htr_peer_wait.argtypes = [vp, vp, i32, i32, vp, vp]
    lib.htr_moe_combine_peers.argtypes = [vp, i32, vp, i32, i32, i32, vp, i32, i64, vp, vp, vp]
    lib.htr_moe_weighted_sum.argtypes = [vp, i32, vp, i32, i32, i32, vp, vp]
    lib.htr_rank_sum.argtypes = [vp, i32, i64, i32, i32, vp, i32, vp]
    lib.htr_linear_fault_offset.restype = sz
    lib.htr_set_gemv_kernel.restype = None
    lib.htr_set_gemv_kernel.argtypes = [i32]
    return lib


lib = _load()


def check(status, what):
    if status != 0:
        msg = lib.htr_status_string(status).decode()
        if status == -7:
            code = (lib.htr_linear_gemm_last_cuda_error() if what.startswith("htr_linear_gemm") else
                    lib.htr_viterbi_last_cuda_error() if what.startswith(("htr_viterbi", "htr_codebook")) else lib.htr_last_cuda_error())
            msg += f" (cudaError {code})"
        raise HTRError(f"{what}: {msg}")
