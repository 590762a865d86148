"""The give-up path of the kernels' bounded waits, exercised on a GPU without faulting, trapping or
hanging anything: a test build of the library (-DFA_TEST_SHORT_WAIT: waits give up after about 2 ms)
whose TMA producer is told to leave out the loads of one KV tile.  The MMA warp's wait for that tile
runs out, the kernel records 100 + n in the status word, drains, frees its tensor memory and returns;
the host-buffer entry point turns the word into FA_ERR_DEVICE_TIMEOUT; the next ordinary launch on
the same device and context is correct."""
import ctypes
import os

import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib
import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def test_lib():
    from flash_attn_b200 import _lib, build
    path = build.TEST_LIB
    if not os.path.exists(path):
        path = build.build_test_variant()
    L = ctypes.CDLL(path)
    pp = ctypes.POINTER(_lib.FwdParams)
    for name in ("fa_fwd", "fa_fwd_host"):
        getattr(L, name).argtypes = [pp]
        getattr(L, name).restype = ctypes.c_int
    L.fa_test_skip_kv_tile.argtypes = [ctypes.c_int]
    L.fa_test_skip_kv_tile.restype = ctypes.c_int
    return L


def _params(q, k, v, o, lse, status=None):
    from flash_attn_b200 import _lib
    B, H, N, d = q.shape
    p = _lib.FwdParams()
    p.q, p.k, p.v, p.o, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    p.dtype = p.o_dtype = _lib.FA_DTYPE_BF16
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim = B, H, N, k.shape[2], d
    p.softmax_scale = d ** -0.5
    p.window_left = p.window_right = -1
    p.num_splits = 1
    if status is not None:
        p.status = status.data_ptr()
    if q.is_cuda:
        p.stream = torch.cuda.current_stream().cuda_stream
    return p


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(test_lib):
    L = test_lib
    B, H, N, d = 1, 2, 256, 128
    qh, kh, vh = synth.qkv(40, B, H, N, N, d, "bfloat16")
    q, k, v = (gpu_util.to_dev(x, "bfloat16") for x in (qh, kh, vh))
    o = torch.empty_like(q)
    lse = torch.empty((B, H, N), device="cuda", dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    try:
        assert L.fa_test_skip_kv_tile(1) == 0  # the second KV tile of every CTA never arrives
        assert L.fa_fwd(ctypes.byref(_params(q, k, v, o, lse, status))) == 0  # the launch itself succeeds
        torch.cuda.synchronize()  # ... and the kernel returns by itself
        code = int(status.item())
        assert 100 < code < 200, code  # a wait of the tiled kernel gave up
        # the synchronous host-buffer entry point reads the word itself
        pin = lambda x: torch.from_numpy(x).bfloat16().pin_memory()
        hq, hk, hv = pin(qh), pin(kh), pin(vh)
        ho = torch.empty((B, H, N, d), dtype=torch.bfloat16).pin_memory()
        hl = torch.empty((B, H, N), dtype=torch.float32).pin_memory()
        assert L.fa_fwd_host(ctypes.byref(_params(hq, hk, hv, ho, hl))) == -5  # FA_ERR_DEVICE_TIMEOUT
    finally:
        assert L.fa_test_skip_kv_tile(-1) == 0
    # same device, same context, same library: an ordinary launch is correct again
    status.zero_()
    assert L.fa_fwd(ctypes.byref(_params(q, k, v, o, lse, status))) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want_o, want_lse = oracle_lib.forward(qh, kh, vh, d ** -0.5)
    err = np.abs(o.float().cpu().numpy() - want_o)
    assert err.max() <= gpu_util.O_MAX_ABS and err.mean() <= gpu_util.O_MEAN_ABS
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= gpu_util.LSE_ABS
    assert L.fa_fwd_host(ctypes.byref(_params(hq, hk, hv, ho, hl))) == 0
    assert np.abs(ho.float().numpy() - want_o).max() <= gpu_util.O_MAX_ABS
