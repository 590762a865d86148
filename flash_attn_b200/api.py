"""Host-side mirror of the reference's launcher surface on torch tensors.

The reference drives its kernels from main() (src/main.cu:109-205): it fills a
parameter block with Q/K/V/O pointers, sizes, softmax scale, causal flag, local
window, ALiBi slopes, dropout probability and split count, and launches.
`flash_attn_forward` takes the same arguments and hands raw device pointers to
the C ABI (include/fa_b200.h); torch only owns the memory and the stream.
"""
import ctypes
import math

import torch

from . import _lib

_DT = {torch.float16: _lib.FA_DTYPE_FP16, torch.bfloat16: _lib.FA_DTYPE_BF16, torch.float32: _lib.FA_DTYPE_FP32}


def _params(q, k, v, o, lse, softmax_scale, causal, window, alibi_slopes, p_dropout, seed, offset, unit0, num_splits,
            q_pos0, k_pos0):
    B, H, Nq, d = q.shape
    Hk, Nk = k.shape[1], k.shape[2]
    if k.shape != (B, Hk, Nk, d) or v.shape != (B, Hk, Nk, d) or Hk < 1 or H % Hk != 0:
        raise ValueError("k and v must be [batch, heads_k, seqlen_k, head_dim] with heads a multiple of heads_k")
    for t in (q, k, v, o):
        if not t.is_contiguous():
            raise ValueError("q, k, v, o must be contiguous [batch, heads, seqlen, head_dim]")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share dtype float16 or bfloat16")
    p = _lib.FwdParams()
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.dtype, p.o_dtype = _DT[q.dtype], _DT[o.dtype]
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim = B, H, Nq, Nk, d
    p.softmax_scale = float(softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d))
    p.is_causal = int(bool(causal))
    p.window_left, p.window_right = int(window[0]), int(window[1])
    p.alibi_slopes = alibi_slopes.data_ptr() if alibi_slopes is not None else None
    p.p_dropout, p.seed, p.offset, p.unit0 = float(p_dropout), int(seed), int(offset), int(unit0)
    p.num_splits = int(num_splits)
    p.q_pos0, p.k_pos0 = int(q_pos0), int(k_pos0)
    p.heads_k = Hk  # grouped-query attention when Hk < H
    return p


def flash_attn_forward(q, k, v, softmax_scale=None, causal=False, window=(-1, -1), alibi_slopes=None,
                       p_dropout=0.0, seed=0, offset=0, num_splits=1, out=None, out_dtype=None, return_lse=True,
                       q_pos0=0, k_pos0=0, unit0=0, workspace=None, status=None, accum=None, accum_first=False,
                       accum_final=False, launch_index=0):
    """O, LSE = attention(Q, K, V) on the current CUDA device and stream.

    q [B,H,Nq,d], k/v [B,Hk,Nk,d] (Hk divides H; query head h reads K/V head
    h // (H // Hk)), fp16 or bf16, contiguous.  `window` = (left,
    right) with -1 = unbounded; `alibi_slopes` fp32 [H]; `num_splits` 0 = the
    reference heuristic, 1 = none, n = forced; `q_pos0`/`k_pos0` = global positions
    of row/column 0 (for one block of a sharded sequence).  Returns (o, lse).

    `accum` = (o_acc fp32 [B,H,Nq,d], lse_acc fp32 [B,H,Nq]): the launch merges its
    result into this running pair in its epilogue (key blocks that arrive one launch
    at a time); `accum_first` marks the first block (the pair is only written),
    `accum_final` the last one, and only that call writes and returns (o, lse) --
    the others return (None, None).
    """
    L = _lib.load()
    if not q.is_cuda:
        raise ValueError("flash_attn_forward needs CUDA tensors (use flash_attn_forward_host for host buffers)")
    B, H, Nq, d = q.shape
    writes_output = accum is None or accum_final
    if out is None and writes_output:
        out = torch.empty((B, H, Nq, d), device=q.device, dtype=out_dtype or q.dtype)
    lse = torch.empty((B, H, Nq), device=q.device, dtype=torch.float32) if (return_lse and writes_output) else None
    if alibi_slopes is not None:
        alibi_slopes = alibi_slopes.to(device=q.device, dtype=torch.float32).contiguous()
    if not writes_output:
        out = None
    p = _params(q, k, v, out if out is not None else q, lse, softmax_scale, causal, window, alibi_slopes, p_dropout,
                seed, offset, unit0, num_splits, q_pos0, k_pos0)
    if out is None:
        p.o = None
    p.launch_index = int(launch_index)  # dropout mask of the k-th launch of a loop of the reference's kernels
    if accum is not None:
        o_acc, lse_acc = accum
        if o_acc.dtype != torch.float32 or lse_acc.dtype != torch.float32 or not o_acc.is_contiguous() or \
                not lse_acc.is_contiguous() or o_acc.shape != (B, H, Nq, d) or lse_acc.shape != (B, H, Nq):
            raise ValueError("accum = (fp32 [B,H,Nq,d], fp32 [B,H,Nq]), contiguous")
        p.accum_o, p.accum_lse = o_acc.data_ptr(), lse_acc.data_ptr()
        p.accum_flags = (_lib.FA_ACCUM_FIRST if accum_first else 0) | (_lib.FA_ACCUM_FINAL if accum_final else 0)
    with torch.cuda.device(q.device):
        need = L.fa_fwd_workspace_bytes(ctypes.byref(p))
        if need:
            if workspace is None or workspace.numel() * workspace.element_size() < need:
                workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
            p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
        if status is not None:
            p.status = status.data_ptr()
        p.stream = torch.cuda.current_stream(q.device).cuda_stream
        _lib.check(L.fa_fwd(ctypes.byref(p)), "fa_fwd")
    return out, lse


def flash_attn_forward_host(q, k, v, softmax_scale=None, causal=False, window=(-1, -1), alibi_slopes=None,
                            p_dropout=0.0, seed=0, offset=0, num_splits=1, out=None, out_dtype=None, return_lse=True,
                            device=None):
    """Same computation on HOST tensors (pinned memory overlaps best): the library
    stages slices through device memory, as the reference's main() does around its
    kernel (src/main.cu:105-107, 219).  Synchronous."""
    L = _lib.load()
    if q.is_cuda:
        raise ValueError("flash_attn_forward_host takes host tensors")
    B, H, Nq, d = q.shape
    if out is None:
        out = torch.empty((B, H, Nq, d), dtype=out_dtype or q.dtype, pin_memory=True)
    lse = torch.empty((B, H, Nq), dtype=torch.float32, pin_memory=True) if return_lse else None
    if alibi_slopes is not None:
        alibi_slopes = alibi_slopes.to(device="cpu", dtype=torch.float32).contiguous()
    p = _params(q, k, v, out, lse, softmax_scale, causal, window, alibi_slopes, p_dropout, seed, offset, 0,
                num_splits, 0, 0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _lib.check(L.fa_fwd_host(ctypes.byref(p)), "fa_fwd_host")
    return out, lse


def dropout_mask(B, H, Nq, Nk, p_dropout, seed, offset=0, num_splits=1, window_left=-1, q_pos0=0, k_pos0=0,
                 unit0=0, device="cuda", causal=False, window_right=-1, launch_index=0):
    """uint8 [B,H,Nq,Nk] keep-mask (1 = kept) that flash_attn_forward applies."""
    L = _lib.load()
    keep = torch.empty((B, H, Nq, Nk), device=device, dtype=torch.uint8)
    dummy = torch.empty(16, device=device, dtype=torch.float16)
    p = _lib.FwdParams()
    p.q = p.k = p.v = p.o = dummy.data_ptr()
    p.dtype = p.o_dtype = _lib.FA_DTYPE_FP16
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim = B, H, Nq, Nk, 64
    p.softmax_scale = 1.0
    p.window_left, p.window_right = int(window_left), int(window_right)
    p.is_causal = int(bool(causal))
    p.p_dropout, p.seed, p.offset, p.unit0 = float(p_dropout), int(seed), int(offset), int(unit0)
    p.num_splits = int(num_splits)
    p.q_pos0, p.k_pos0 = int(q_pos0), int(k_pos0)
    p.launch_index = int(launch_index)
    with torch.cuda.device(keep.device):
        p.stream = torch.cuda.current_stream(keep.device).cuda_stream
        _lib.check(L.fa_dropout_mask(ctypes.byref(p), keep.data_ptr()), "fa_dropout_mask")
    return keep


def merge_partial(o_acc, lse_acc, o_part, lse_part):
    """In-place LSE merge of a partial result into fp32 accumulators."""
    L = _lib.load()
    d = o_acc.shape[-1]
    rows = o_acc.numel() // d
    with torch.cuda.device(o_acc.device):
        _lib.check(L.fa_merge_partial(o_acc.data_ptr(), lse_acc.data_ptr(), o_part.data_ptr(), lse_part.data_ptr(),
                                      _DT[o_part.dtype], rows, d,
                                      torch.cuda.current_stream(o_acc.device).cuda_stream), "fa_merge_partial")


def cast_output(o_acc, dtype):
    L = _lib.load()
    out = torch.empty_like(o_acc, dtype=dtype)
    with torch.cuda.device(o_acc.device):
        _lib.check(L.fa_cast_output(o_acc.data_ptr(), out.data_ptr(), _DT[dtype], o_acc.numel(),
                                    torch.cuda.current_stream(o_acc.device).cuda_stream), "fa_cast_output")
    return out


def num_splits_heuristic(batch_nheads_mblocks, num_sms, num_n_blocks, max_splits, seq_len):
    """The reference's split policy (src/main.cu:391-422)."""
    return _lib.load().fa_num_splits_heuristic(batch_nheads_mblocks, num_sms, num_n_blocks, max_splits, seq_len)
