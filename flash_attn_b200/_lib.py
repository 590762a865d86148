"""ctypes binding of libfa_b200.so, the C-ABI declared in include/fa_b200.h.

There is no fallback: if the library is missing or fails to load, importing the
compute entry points raises."""
import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libfa_b200.so")

FA_DTYPE_FP16, FA_DTYPE_BF16, FA_DTYPE_FP32 = 0, 1, 2
FA_OK = 0
FA_ACCUM_FIRST, FA_ACCUM_FINAL = 1, 2

#: every symbol include/fa_b200.h declares
EXPORTS = ["fa_fwd", "fa_fwd_workspace_bytes", "fa_fwd_resolve_splits", "fa_num_splits_heuristic",
           "fa_dropout_mask", "fa_merge_partial", "fa_cast_output", "fa_fwd_host", "fa_fwd_host_release",
           "fa_fwd_static_scratch", "fa_static_scratch_bytes", "fa_launch_reference_params", "fa_strerror", "fa_version",
           "fa_ring_fwd", "fa_ring_message_bytes", "fa_ring_unique_id", "fa_ring_comm_create", "fa_ring_comm_destroy"]


class FwdParams(ctypes.Structure):
    """struct fa_fwd_params"""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("dtype", ctypes.c_int), ("o_dtype", ctypes.c_int),
        ("batch", ctypes.c_int), ("heads", ctypes.c_int),
        ("seqlen_q", ctypes.c_int), ("seqlen_k", ctypes.c_int),
        ("head_dim", ctypes.c_int),
        ("softmax_scale", ctypes.c_float),
        ("is_causal", ctypes.c_int),
        ("window_left", ctypes.c_int), ("window_right", ctypes.c_int),
        ("alibi_slopes", ctypes.c_void_p),
        ("p_dropout", ctypes.c_float),
        ("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64), ("unit0", ctypes.c_uint64),
        ("num_splits", ctypes.c_int),
        ("q_pos0", ctypes.c_int64), ("k_pos0", ctypes.c_int64),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p),
        ("stream", ctypes.c_void_p),
        ("heads_k", ctypes.c_int),
        ("accum_o", ctypes.c_void_p), ("accum_lse", ctypes.c_void_p), ("accum_flags", ctypes.c_int),
        ("launch_index", ctypes.c_uint64),
    ]


class RingParams(ctypes.Structure):
    """struct fa_ring_params"""
    _fields_ = [
        ("q", ctypes.c_void_p * 2), ("k", ctypes.c_void_p * 2), ("v", ctypes.c_void_p * 2), ("o", ctypes.c_void_p * 2),
        ("lse", ctypes.c_void_p * 2),
        ("dtype", ctypes.c_int), ("batch", ctypes.c_int), ("heads", ctypes.c_int), ("heads_k", ctypes.c_int),
        ("chunk_rows", ctypes.c_int), ("head_dim", ctypes.c_int),
        ("softmax_scale", ctypes.c_float),
        ("is_causal", ctypes.c_int), ("window_left", ctypes.c_int), ("window_right", ctypes.c_int),
        ("alibi_slopes", ctypes.c_void_p),
        ("p_dropout", ctypes.c_float),
        ("rank", ctypes.c_int), ("world", ctypes.c_int),
        ("comm", ctypes.c_void_p),
        ("message", ctypes.c_void_p * 2),
        ("accum_o", ctypes.c_void_p * 2), ("accum_lse", ctypes.c_void_p * 2),
        ("compute_stream", ctypes.c_void_p), ("comm_stream", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
    ]


class RefKernelParams(ctypes.Structure):
    """struct fa_ref_kernel_params: the reference's mykernelParamType, field for field"""
    _fields_ = [("Q", ctypes.c_void_p), ("K", ctypes.c_void_p), ("V", ctypes.c_void_p), ("O", ctypes.c_void_p),
                ("O_tmp", ctypes.c_void_p), ("L", ctypes.c_void_p), ("M", ctypes.c_void_p),
                ("N", ctypes.c_int), ("d", ctypes.c_int), ("Br", ctypes.c_int), ("Bc", ctypes.c_int),
                ("Tr", ctypes.c_int), ("Tc", ctypes.c_int),
                ("softmax_scale", ctypes.c_float), ("dropout_prob", ctypes.c_float),
                ("seed", ctypes.c_ulonglong), ("states", ctypes.c_void_p),
                ("window_size_left", ctypes.c_int), ("window_size_right", ctypes.c_int),
                ("alibi_slopes_ptr", ctypes.c_void_p), ("split_num", ctypes.c_int)]


class FaError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what} failed: {code} ({strerror(code)})")


_lib = None


def load():
    """Loads the library (building nothing: run `python -m flash_attn_b200.build` first)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m flash_attn_b200.build`; "
                          "there is no non-CUDA fallback")
    L = ctypes.CDLL(LIB_PATH)
    pp = ctypes.POINTER(FwdParams)
    L.fa_fwd.argtypes = [pp]
    L.fa_fwd.restype = ctypes.c_int
    L.fa_fwd_host.argtypes = [pp]
    L.fa_fwd_host.restype = ctypes.c_int
    L.fa_fwd_host_release.argtypes = []
    L.fa_fwd_host_release.restype = None
    L.fa_fwd_static_scratch.argtypes = [pp]
    L.fa_fwd_static_scratch.restype = ctypes.c_int
    L.fa_static_scratch_bytes.argtypes = []
    L.fa_static_scratch_bytes.restype = ctypes.c_size_t
    L.fa_launch_reference_params.argtypes = [ctypes.POINTER(RefKernelParams)] + [ctypes.c_int] * 6 + [
        ctypes.c_ulonglong, ctypes.c_void_p]
    L.fa_launch_reference_params.restype = ctypes.c_int
    L.fa_fwd_workspace_bytes.argtypes = [pp]
    L.fa_fwd_workspace_bytes.restype = ctypes.c_size_t
    L.fa_fwd_resolve_splits.argtypes = [pp]
    L.fa_fwd_resolve_splits.restype = ctypes.c_int
    L.fa_num_splits_heuristic.argtypes = [ctypes.c_int] * 5
    L.fa_num_splits_heuristic.restype = ctypes.c_int
    L.fa_dropout_mask.argtypes = [pp, ctypes.c_void_p]
    L.fa_dropout_mask.restype = ctypes.c_int
    L.fa_merge_partial.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                   ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
    L.fa_merge_partial.restype = ctypes.c_int
    L.fa_cast_output.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]
    L.fa_cast_output.restype = ctypes.c_int
    rp = ctypes.POINTER(RingParams)
    L.fa_ring_fwd.argtypes = [rp]
    L.fa_ring_fwd.restype = ctypes.c_int
    L.fa_ring_message_bytes.argtypes = [rp]
    L.fa_ring_message_bytes.restype = ctypes.c_size_t
    L.fa_ring_unique_id.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    L.fa_ring_unique_id.restype = ctypes.c_int
    L.fa_ring_comm_create.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                      ctypes.c_size_t]
    L.fa_ring_comm_create.restype = ctypes.c_int
    L.fa_ring_comm_destroy.argtypes = [ctypes.c_void_p]
    L.fa_ring_comm_destroy.restype = ctypes.c_int
    L.fa_strerror.argtypes = [ctypes.c_int]
    L.fa_strerror.restype = ctypes.c_char_p
    L.fa_version.argtypes = []
    L.fa_version.restype = ctypes.c_int
    _lib = L
    return L


def strerror(code):
    return load().fa_strerror(int(code)).decode()


def check(code, what):
    if code != FA_OK:
        raise FaError(code, what)
