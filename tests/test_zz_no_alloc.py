"""fa_fwd_static_scratch: the split-KV forward for callers that cannot allocate.

A process whose device memory is wholly owned by another allocator (an inference
server's pool, a host application that loads this library as a plugin) cannot
cudaMalloc a workspace for the split partials and may not be able to hand one
over either.  The entry point keeps the partials in a fixed 32 MiB array inside
the library image instead.  This test calls it through the C ABI, twice in a
row (the second call finds the first call's partials in the scratch), and checks
both results against fa_fwd with an ordinary caller-provided workspace: the same
kernels run on the same inputs, so the results must be equal bit for bit.  One case
is also held against the CPU oracle.

Collected last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

import gpu_util
import synth

pytestmark = pytest.mark.gpu


def _params(q, k, v, o, lse, causal, q_pos0, splits, p_dropout=0.0):
    from flash_attn_b200 import _lib
    B, H, Nq, d = q.shape
    p = _lib.FwdParams()
    p.q, p.k, p.v, p.o, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    p.dtype = p.o_dtype = _lib.FA_DTYPE_BF16
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim = B, H, Nq, k.shape[2], d
    p.softmax_scale = d ** -0.5
    p.is_causal = int(causal)
    p.window_left = p.window_right = -1
    p.p_dropout, p.seed = p_dropout, 42
    p.num_splits = splits
    p.q_pos0 = q_pos0
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def _run_pair(shape_q, nk, causal, q_pos0, splits, seed, p_dropout=0.0):
    from flash_attn_b200 import _lib
    L = _lib.load()
    B, H, Nq, d = shape_q
    q, k, v = (gpu_util.to_dev(x, "bfloat16") for x in synth.qkv(seed, B, H, Nq, nk, d, "bfloat16"))
    # existing entry point, workspace from the caller
    o_ref = torch.empty_like(q)
    lse_ref = torch.empty((B, H, Nq), device="cuda", dtype=torch.float32)
    p = _params(q, k, v, o_ref, lse_ref, causal, q_pos0, splits, p_dropout)
    need = L.fa_fwd_workspace_bytes(ctypes.byref(p))
    assert need > 0
    ws = torch.empty(need, device="cuda", dtype=torch.uint8)
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    _lib.check(L.fa_fwd(ctypes.byref(p)), "fa_fwd")
    # new entry point, no workspace
    o_new = torch.full_like(q, float("nan"))
    lse_new = torch.full_like(lse_ref, float("nan"))
    p2 = _params(q, k, v, o_new, lse_new, causal, q_pos0, splits, p_dropout)
    _lib.check(L.fa_fwd_static_scratch(ctypes.byref(p2)), "fa_fwd_static_scratch")
    torch.cuda.synchronize()
    assert torch.equal(o_new, o_ref), (o_new.float() - o_ref.float()).abs().max().item()
    assert torch.equal(lse_new, lse_ref)
    return q, k, v, o_new, lse_new


def test_static_scratch_matches_workspace_path_on_two_calls_in_a_row():
    # two different launches back to back: the second reuses the scratch the first one filled
    _run_pair((2, 4, 300, 128), 1024, causal=True, q_pos0=724, splits=4, seed=31)
    _run_pair((4, 8, 1, 128), 4096, causal=False, q_pos0=0, splits=16, seed=32)
    _run_pair((2, 4, 300, 128), 1024, causal=True, q_pos0=724, splits=4, seed=31, p_dropout=0.1)


def test_static_scratch_result_matches_the_oracle():
    import oracle_lib
    B, H, Nq, Nk, d = 2, 4, 300, 1024, 128
    q, k, v, o, lse = _run_pair((B, H, Nq, d), Nk, causal=True, q_pos0=724, splits=4, seed=33)
    want_o, want_lse = oracle_lib.forward(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                          d ** -0.5, causal=True, q_pos0=724)
    err = abs(o.float().cpu().numpy() - want_o)
    assert err.max() <= gpu_util.O_MAX_ABS and err.mean() <= gpu_util.O_MEAN_ABS
    assert abs(lse.cpu().numpy() - want_lse).max() <= gpu_util.LSE_ABS


def test_static_scratch_rejects_what_does_not_fit():
    from flash_attn_b200 import _lib
    L = _lib.load()
    limit = L.fa_static_scratch_bytes()
    assert limit == 32 << 20
    # 64 units x 8 splits x 1024 rows x (128+1) x 4 B = 258 MiB of partials
    B, H, Nq, Nk, d = 4, 16, 1024, 1024, 128
    q = torch.zeros(B, H, Nq, d, dtype=torch.bfloat16, device="cuda")
    o = torch.empty_like(q)
    lse = torch.empty(B, H, Nq, dtype=torch.float32, device="cuda")
    p = _params(q, q, q, o, lse, False, 0, 8)
    assert L.fa_fwd_workspace_bytes(ctypes.byref(p)) > limit
    assert L.fa_fwd_static_scratch(ctypes.byref(p)) == -7  # FA_ERR_TOO_LARGE
    assert "limit" in _lib.strerror(-7)
