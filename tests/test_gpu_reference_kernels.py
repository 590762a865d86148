"""Parity with the reference's own CUDA kernels, run on the same GPU.

The dropout mask is read out of the reference's forward_kernel itself (unmodified,
recompiled for sm_100a): with Q = K = 0 every probability is 1/N, and with V a
tile-weighted identity the fp32 output encodes which entries were kept.  This pins
the stateless Philox map against the real thing, not only against the host
simulation.  Skipped when oracle/_ref/libref_gpu.so was not built."""
import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib
import ref_gpu
import synth

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_gpu.available(), reason="reference kernels not built")]


def _reference_mask(B, H, N, p, seed, split_num=1, causal=False, prior_launches=0):
    """Keep mask the reference kernel applies in launch number `prior_launches` on one set of generator states
    (entries a causal mask hides read as 0)."""
    d, tiles = 128, (N + 127) // 128
    q = torch.zeros(B, H, N, d, dtype=torch.float16, device="cuda")
    v = torch.zeros(B, H, N, d, dtype=torch.float32, device="cuda")
    idx = torch.arange(N, device="cuda")
    v[:, :, idx, idx % 128] = (2.0 ** (idx // 128)).float()
    o, used, _ = ref_gpu.forward(q, q, v.half(), 1.0, causal=causal, p_dropout=p, seed=seed, split_num=split_num,
                                 prior_launches=prior_launches)
    visible = (idx + 1).float() if causal else torch.full((N,), float(N), device="cuda")  # keys each row attends to
    code = torch.round(o * (visible * (1.0 - np.float32(p).item()))[None, None, :, None]).to(torch.int64)
    keep = torch.zeros(B, H, N, tiles * 128, dtype=torch.uint8, device="cuda")
    for t in range(tiles):
        keep[..., t * 128:(t + 1) * 128] = ((code >> t) & 1).to(torch.uint8)
    return keep[..., :N].cpu().numpy(), used


@pytest.mark.parametrize("case", [dict(B=1, H=2, N=256, p=0.1, seed=42), dict(B=2, H=1, N=512, p=0.25, seed=48),
                                  dict(B=1, H=2, N=512, p=0.1, seed=7, split_num=2)])
def test_reference_kernel_mask_equals_the_stateless_map(case):
    import flash_attn_b200 as fa
    splits = case.get("split_num", 1)
    got_ref, used = _reference_mask(case["B"], case["H"], case["N"], case["p"], case["seed"], splits)
    assert used == splits
    want = oracle_lib.dropout_mask(case["B"], case["H"], case["N"], case["N"], np.float32(case["p"]).item(),
                                   case["seed"], 0, splits)
    assert np.array_equal(got_ref, want)
    ours = fa.dropout_mask(case["B"], case["H"], case["N"], case["N"], case["p"], case["seed"], 0, splits).cpu().numpy()
    assert np.array_equal(ours, got_ref)


@pytest.mark.parametrize("case", [
    dict(B=1, H=4, N=256, d=64, causal=False),
    dict(B=2, H=2, N=512, d=128, causal=True),
    dict(B=1, H=2, N=384, d=128, causal=False, window=(128, 128)),
    dict(B=1, H=4, N=256, d=64, causal=False, split_num=2),
    dict(B=1, H=2, N=256, d=31, causal=True),   # head_dim of the reference's default launch (zero-padded to 32 there)
])
def test_outputs_match_the_reference_kernels(case):
    import flash_attn_b200 as fa
    B, H, N, d = case["B"], case["H"], case["N"], case["d"]
    q, k, v = (gpu_util.to_dev(x, "float16") for x in synth.qkv(40, B, H, N, N, d, "float16"))
    window = case.get("window", (-1, -1))
    o_ref, _, _ = ref_gpu.forward(q, k, v, d ** -0.5, causal=case["causal"], window=window,
                                  split_num=case.get("split_num", 1))
    o, _ = fa.flash_attn_forward(q, k, v, causal=case["causal"], window=window, out_dtype=torch.float32,
                                 num_splits=case.get("split_num", 1))
    err = (o - o_ref).abs()
    assert err.max().item() <= gpu_util.O_MAX_ABS and err.mean().item() <= gpu_util.O_MEAN_ABS, (err.max(), err.mean())


def test_launch_with_the_reference_parameter_block():
    """fa_launch_reference_params takes the reference's own argument struct and flags: the run of the
    reference's default main() (fp16 [1,8,1021,31], fp32 O, src/main.cu:39-42) against the oracle, and a
    causal + dropout launch against the reference kernels' own result."""
    import ctypes
    from flash_attn_b200 import _lib
    L = _lib.load()

    def launch(q, k, v, o, N, d, scale, p=0.0, causal=0, seed=0, split=1):
        prm = _lib.RefKernelParams()
        prm.Q, prm.K, prm.V, prm.O = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
        prm.N, prm.d, prm.Br, prm.Bc = N, d, 128, 128
        prm.Tr = prm.Tc = (N + 127) // 128
        prm.softmax_scale, prm.dropout_prob = scale, p
        prm.window_size_left = prm.window_size_right = -1
        prm.split_num = split
        _lib.check(L.fa_launch_reference_params(ctypes.byref(prm), q.shape[1], q.shape[0], int(p > 0), causal, 0, 0,
                                                seed, torch.cuda.current_stream().cuda_stream), "shim")
        torch.cuda.synchronize()

    B, H, N, d = 1, 8, 1021, 31
    qn, kn, vn = synth.qkv(41, B, H, N, N, d, "float16")
    q, k, v = (gpu_util.to_dev(x, "float16") for x in (qn, kn, vn))
    o = torch.zeros(B, H, N, d, dtype=torch.float32, device="cuda")
    launch(q, k, v, o, N, d, 1 / np.sqrt(d))
    want, _ = oracle_lib.forward(qn, kn, vn, 1 / np.sqrt(d))
    err = np.abs(o.cpu().numpy() - want)
    assert err.max() <= gpu_util.O_MAX_ABS and err.mean() <= gpu_util.O_MEAN_ABS

    B, H, N, d = 2, 2, 512, 128
    q, k, v = (gpu_util.to_dev(x, "float16") for x in synth.qkv(42, B, H, N, N, d, "float16"))
    o = torch.zeros(B, H, N, d, dtype=torch.float32, device="cuda")
    launch(q, k, v, o, N, d, d ** -0.5, p=0.1, causal=1, seed=48)
    o_ref, _, _ = ref_gpu.forward(q, k, v, d ** -0.5, causal=True, p_dropout=0.1, seed=48)
    err = (o - o_ref).abs()
    assert err.max().item() <= gpu_util.O_MAX_ABS and err.mean().item() <= gpu_util.O_MEAN_ABS


@pytest.mark.parametrize("case", [dict(N=384, causal=False, k=1), dict(N=512, causal=True, k=1), dict(N=512, causal=True, k=3),
                                  dict(N=512, causal=False, k=2, split_num=2), dict(N=512, causal=True, k=2, split_num=2)])
def test_later_launches_of_the_reference_loop_continue_the_streams(case):
    # the reference writes the generator states back (src/flash_forward.h:302-305): launch k of its loop
    # starts every CTA's stream 64 draws per visited KV tile per earlier launch further on -- fewer tiles for
    # the upper query blocks of a causal launch, so a single offset cannot express it.  launch_index does.
    import flash_attn_b200 as fa
    B, H, N, p, seed, k = 1, 2, case["N"], 0.1, 48, case["k"]
    splits, causal = case.get("split_num", 1), case["causal"]
    got_ref, _ = _reference_mask(B, H, N, p, seed, splits, causal=causal, prior_launches=k)
    first, _ = _reference_mask(B, H, N, p, seed, splits, causal=causal)
    visible = np.tril(np.ones((N, N), dtype=bool)) if causal else np.ones((N, N), dtype=bool)
    assert not np.array_equal(got_ref, first)  # the loop really moves on
    want = oracle_lib.dropout_mask(B, H, N, N, np.float32(p).item(), seed, 0, splits, causal=causal, launch_index=k)
    assert np.array_equal(got_ref[..., visible], want[..., visible])
    ours = fa.dropout_mask(B, H, N, N, p, seed, 0, splits, causal=causal, launch_index=k).cpu().numpy()
    assert np.array_equal(ours[..., visible], got_ref[..., visible])
    # and the forward kernel applies that mask: same launch of the reference kernels, same numbers
    q, kk, v = (gpu_util.to_dev(x, "float16") for x in synth.qkv(43, B, H, N, N, 128, "float16"))
    o_ref, _, _ = ref_gpu.forward(q, kk, v, 128 ** -0.5, causal=causal, p_dropout=p, seed=seed, split_num=splits,
                                  prior_launches=k)
    o, _ = fa.flash_attn_forward(q, kk, v, causal=causal, p_dropout=p, seed=seed, num_splits=splits,
                                 out_dtype=torch.float32, launch_index=k)
    err = (o - o_ref).abs()
    assert err.max().item() <= gpu_util.O_MAX_ABS and err.mean().item() <= gpu_util.O_MEAN_ABS, (err.max(), err.mean())
