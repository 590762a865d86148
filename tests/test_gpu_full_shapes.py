"""The two large baseline shapes at their stated sizes against the CPU oracle, on sampled rows: the
tensors are generated on the GPU from a seed and only the sampled (batch, head) units travel to
the host (a whole-tensor host copy of config 3 is 1.6 GB per tensor in fp32)."""
import numpy as np
import pytest
import torch

import gpu_util
import synth

pytestmark = pytest.mark.gpu


def _randn(shape, seed, sigma=1.0):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (sigma * torch.randn(shape, generator=g, device="cuda", dtype=torch.float32)).bfloat16()


def test_config3_full_shape_sampled_rows():
    # bf16 [4,32,8192,128], causal + window(1024, 0) + ALiBi slopes 2^(-8(h+1)/32)
    import flash_attn_b200 as fa
    B, H, N, d = 4, 32, 8192, 128
    q, k, v = (_randn((B, H, N, d), 30 + i) for i in range(3))
    slopes = synth.alibi_slopes(H)
    o, lse = fa.flash_attn_forward(q, k, v, causal=True, window=(1024, 0), alibi_slopes=torch.from_numpy(slopes))
    torch.cuda.synchronize()
    rng = np.random.default_rng(3)
    # first and last row, tile boundaries, the rows where the window's left edge starts to cut
    # (1023-1025) and crosses tile boundaries, the last tile, plus random rows
    fixed = [0, 1, 127, 128, 129, 1023, 1024, 1025, 1151, 1152, 2047, 2048, 4095, 4096, N - 129, N - 128, N - 1]
    units = [0, 1, 31, 32, 77, B * H - 1]  # smallest and largest slope, both ends of the batch
    res = gpu_util.check_sampled_units(q, k, v, o, lse, units, lambda u: fixed + list(rng.integers(0, N, 48)),
                                       d ** -0.5, causal=True, window=(1024, 0), slopes=slopes)
    gpu_util.assert_close(res, "config 3 at full size")


def test_config5_geometry_on_one_gpu():
    # config 5's sequence (N = 131072, 1024 KV tiles, N(0, 0.5) inputs, causal) with two heads
    # (K + V = 134 MB); rows of the first, a middle and the last tile
    import flash_attn_b200 as fa
    B, H, N, d = 1, 2, 131072, 128
    q, k, v = (_randn((B, H, N, d), 50 + i, sigma=0.5) for i in range(3))
    o, lse = fa.flash_attn_forward(q, k, v, causal=True)
    torch.cuda.synchronize()
    rng = np.random.default_rng(5)
    fixed = [0, 127, 128, 8191, 8192, 65535, 65536, 122879, 122880, N - 128, N - 127, N - 1]
    res = gpu_util.check_sampled_units(q, k, v, o, lse, [0, 1], lambda u: fixed + list(rng.integers(0, N, 40)),
                                       d ** -0.5, causal=True)
    gpu_util.assert_close(res, "config 5 geometry")
    # one block of the ring at config 5's largest offsets: the last query chunk against the
    # next-to-last key chunk (q_pos0 = 122880, k_pos0 = 114688), merged into a running result
    C = 8192
    qa = q[:, :, N - C:].contiguous()
    acc = (torch.empty((B, H, C, d), device="cuda"), torch.empty((B, H, C), device="cuda"))
    fa.flash_attn_forward(qa, k[:, :, N - 2 * C:N - C].contiguous(), v[:, :, N - 2 * C:N - C].contiguous(),
                          q_pos0=N - C, k_pos0=N - 2 * C, accum=acc, accum_first=True)
    o2, lse2 = fa.flash_attn_forward(qa, k[:, :, N - C:].contiguous(), v[:, :, N - C:].contiguous(), causal=True,
                                     q_pos0=N - C, k_pos0=N - C, accum=acc, accum_final=True)
    torch.cuda.synchronize()
    # oracle on the same two key chunks (k_pos0 = N - 2C)
    res = gpu_util.check_sampled_units(qa, k[:, :, N - 2 * C:].contiguous(), v[:, :, N - 2 * C:].contiguous(), o2, lse2,
                                       [0, 1], lambda u: [0, 1, 127, 128, C - 1] + list(rng.integers(0, C, 32)),
                                       d ** -0.5, causal=True, q_pos0=N - C, k_pos0=N - 2 * C)
    gpu_util.assert_close(res, "config 5 ring block with merged running result")
