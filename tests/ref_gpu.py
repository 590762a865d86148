"""ctypes binding of oracle/_ref/libref_gpu.so: the REFERENCE's own CUDA kernels
(src/flash_forward.h, src/flash_forward_splitkv.h), compiled from the reference
checkout for sm_100a behind oracle/ref_gpu_driver.cu.  Test infrastructure."""
import ctypes
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so")
_L = None


def available():
    return os.path.exists(PATH)


def lib():
    global _L
    if _L is None:
        L = ctypes.CDLL(PATH)
        L.ref_gpu_forward.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_float,
                                      ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_float),
                                      ctypes.c_int]
        L.ref_gpu_forward.restype = ctypes.c_int
        _L = L
    return _L


def forward(q, k, v, scale, causal=False, window=(-1, -1), slopes=None, p_dropout=0.0, seed=0, split_num=1,
            iters=0, prior_launches=0):
    """q/k/v fp16 CUDA [B,H,N,d].  Returns (o fp32, splits used, mean us per launch or None).
    prior_launches: launches made on the same generator states before the one that is returned."""
    B, H, N, d = q.shape
    o = torch.zeros((B, H, N, d), device=q.device, dtype=torch.float32)
    t = ctypes.c_float(0.0)
    torch.cuda.synchronize()
    rc = lib().ref_gpu_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, N, d, float(scale),
                               int(causal), int(window[0]), int(window[1]),
                               slopes.data_ptr() if slopes is not None else None, float(p_dropout), int(seed),
                               int(split_num), int(iters), ctypes.byref(t), int(prior_launches))
    if rc < 0:
        raise RuntimeError(f"ref_gpu_forward failed: {rc}")
    return o, rc, (t.value if iters > 0 else None)
