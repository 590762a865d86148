"""ctypes binding of the CPU oracle (oracle/liboracle.so) for the tests, the
smoke check and the benchmark's cpu_baseline leg.  Test infrastructure: the
shipped package never imports this module."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = None

c_f = ctypes.POINTER(ctypes.c_float)
c_i64 = ctypes.POINTER(ctypes.c_int64)


class DropoutGeom(ctypes.Structure):
    _fields_ = [("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64), ("p", ctypes.c_float),
                ("heads", ctypes.c_int), ("seqlen_q", ctypes.c_int), ("seqlen_k", ctypes.c_int),
                ("num_splits", ctypes.c_int), ("causal", ctypes.c_int), ("window_left", ctypes.c_int),
                ("q_pos0", ctypes.c_int64), ("k_pos0", ctypes.c_int64),
                ("window_right", ctypes.c_int), ("launch_index", ctypes.c_uint64)]


class Params(ctypes.Structure):
    _fields_ = [("q", c_f), ("k", c_f), ("v", c_f),
                ("batch", ctypes.c_int), ("heads", ctypes.c_int), ("seqlen_q", ctypes.c_int),
                ("seqlen_k", ctypes.c_int), ("head_dim", ctypes.c_int),
                ("softmax_scale", ctypes.c_float), ("causal", ctypes.c_int),
                ("window_left", ctypes.c_int), ("window_right", ctypes.c_int),
                ("alibi_slopes", c_f), ("p_dropout", ctypes.c_float),
                ("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64), ("dropout_splits", ctypes.c_int),
                ("q_pos0", ctypes.c_int64), ("k_pos0", ctypes.c_int64),
                ("rows", c_i64), ("n_rows", ctypes.c_int64),
                ("o", c_f), ("lse", c_f), ("num_threads", ctypes.c_int), ("launch_index", ctypes.c_uint64)]


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(ROOT, "oracle", "liboracle.so")
        if not os.path.exists(path):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), path])
        L = ctypes.CDLL(path)
        L.fa_oracle_forward.argtypes = [ctypes.POINTER(Params)]
        L.fa_oracle_forward.restype = ctypes.c_int
        L.fa_oracle_curand_draw.argtypes = [ctypes.c_uint64] * 4
        L.fa_oracle_curand_draw.restype = ctypes.c_uint32
        L.fa_oracle_uniform.argtypes = [ctypes.c_uint32]
        L.fa_oracle_uniform.restype = ctypes.c_float
        L.fa_oracle_keep_threshold.argtypes = [ctypes.c_float]
        L.fa_oracle_keep_threshold.restype = ctypes.c_uint64
        L.fa_oracle_dropout_mask.argtypes = [ctypes.POINTER(DropoutGeom), ctypes.c_int, ctypes.c_int,
                                             ctypes.POINTER(ctypes.c_uint8)]
        L.fa_oracle_dropout_mask.restype = None
        L.fa_oracle_num_splits_heuristic.argtypes = [ctypes.c_int] * 5
        L.fa_oracle_num_splits_heuristic.restype = ctypes.c_int
        _LIB = L
    return _LIB


def forward(q, k, v, scale, causal=False, window=(-1, -1), alibi_slopes=None, p_dropout=0.0, seed=0,
            offset=0, dropout_splits=1, q_pos0=0, k_pos0=0, rows=None, num_threads=0, launch_index=0):
    """q [B,H,Nq,d], k/v [B,H,Nk,d] fp32 numpy.  Returns (o, lse) for all rows, or
    for the flat row indices in `rows` ((b*H+h)*Nq + i)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    B, H, Nq, d = q.shape
    Nk = k.shape[2]
    p = Params()
    p.q, p.k, p.v = (a.ctypes.data_as(c_f) for a in (q, k, v))
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim = B, H, Nq, Nk, d
    p.softmax_scale = float(scale)
    p.causal = int(bool(causal))
    p.window_left, p.window_right = int(window[0]), int(window[1])
    keep = [q, k, v]
    if alibi_slopes is not None:
        s = np.ascontiguousarray(alibi_slopes, dtype=np.float32)
        keep.append(s)
        p.alibi_slopes = s.ctypes.data_as(c_f)
    p.p_dropout, p.seed, p.offset, p.dropout_splits = float(p_dropout), int(seed), int(offset), int(dropout_splits)
    p.q_pos0, p.k_pos0 = int(q_pos0), int(k_pos0)
    if rows is not None:
        r = np.ascontiguousarray(rows, dtype=np.int64)
        keep.append(r)
        p.rows, p.n_rows = r.ctypes.data_as(c_i64), r.size
        o = np.empty((r.size, d), dtype=np.float32)
        lse = np.empty((r.size,), dtype=np.float32)
    else:
        o = np.empty((B, H, Nq, d), dtype=np.float32)
        lse = np.empty((B, H, Nq), dtype=np.float32)
    p.o, p.lse = o.ctypes.data_as(c_f), lse.ctypes.data_as(c_f)
    p.num_threads = int(num_threads)
    p.launch_index = int(launch_index)
    rc = lib().fa_oracle_forward(ctypes.byref(p))
    if rc != 0:
        raise RuntimeError(f"fa_oracle_forward failed: {rc}")
    return o, lse


def dropout_mask(B, H, Nq, Nk, p, seed, offset=0, num_splits=1, window_left=-1, q_pos0=0, k_pos0=0, causal=False,
                 window_right=-1, launch_index=0):
    g = DropoutGeom(seed=seed, offset=offset, p=p, heads=H, seqlen_q=Nq, seqlen_k=Nk, num_splits=num_splits,
                    causal=int(causal), window_left=window_left, q_pos0=q_pos0, k_pos0=k_pos0,
                    window_right=window_right, launch_index=launch_index)
    out = np.empty((B, H, Nq, Nk), dtype=np.uint8)
    for b in range(B):
        for h in range(H):
            lib().fa_oracle_dropout_mask(ctypes.byref(g), b, h,
                                         out[b, h].ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
    return out


def reference_lib():
    """The reference's own code (oracle/_ref/libref.so) if it was built, else None."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref.so")
    if not os.path.exists(path):
        return None
    L = ctypes.CDLL(path)
    fn = L._Z21attention_forward_cpuPfS_S_fiiiiS_biS_
    fn.argtypes = [c_f, c_f, c_f, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   c_f, ctypes.c_bool, ctypes.c_int, c_f]
    fn.restype = None
    return L


def reference_cpu_forward(q, k, v, scale, causal=False, window=-1, alibi_slopes=None):
    """Calls the reference's attention_forward_cpu (src/main.cu:279-388) on one
    [B,H,N,d] problem.  Releases the GIL, so callers may thread over heads."""
    L = reference_lib()
    if L is None:
        raise RuntimeError("oracle/_ref/libref.so not built")
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    B, H, N, d = q.shape
    o = np.zeros_like(q)
    s = None if alibi_slopes is None else np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    L._Z21attention_forward_cpuPfS_S_fiiiiS_biS_(
        q.ctypes.data_as(c_f), k.ctypes.data_as(c_f), v.ctypes.data_as(c_f), float(scale), B, H, N, d,
        o.ctypes.data_as(c_f), bool(causal), int(window), None if s is None else s.ctypes.data_as(c_f))
    return o
