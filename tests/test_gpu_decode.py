"""GPU parity of the decode kernel (seqlen_q = 1, keys on the tensor-memory lanes)
against the CPU oracle, same tolerances as the tiled path."""
import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("nk,splits", [(128, 1), (1000, 1), (4096, 16), (5000, 7), (32768, 16), (300, 8)])
def test_decode_plain(dtype, nk, splits):
    gpu_util.assert_close(gpu_util.run_case(2, 4, 1, nk, 128, dtype, seed=50, num_splits=splits), f"nk={nk} s={splits}")


@pytest.mark.parametrize("d", [64, 96, 128, 32])
def test_decode_head_dims(d):
    gpu_util.assert_close(gpu_util.run_case(2, 3, 1, 2000, d, "bfloat16", seed=51, num_splits=4), f"d={d}")


def test_decode_masks_and_bias():
    # the query sits at the end of the sequence (bottom-right causal), some keys lie after it
    gpu_util.assert_close(gpu_util.run_case(1, 4, 1, 3000, 128, "bfloat16", seed=52, causal=True, q_pos0=2500,
                                            num_splits=6), "causal q_pos0 (empty splits)")
    gpu_util.assert_close(gpu_util.run_case(1, 4, 1, 3000, 128, "bfloat16", seed=53, causal=True, q_pos0=2999,
                                            window=(700, 0), alibi=True, num_splits=4), "causal + window + alibi")
    gpu_util.assert_close(gpu_util.run_case(1, 2, 1, 1500, 128, "float16", seed=54, window=(100, 50), q_pos0=800,
                                            num_splits=3), "two-sided window")
    # nothing visible at all: O = 0, LSE = -inf
    gpu_util.assert_close(gpu_util.run_case(1, 2, 1, 600, 128, "bfloat16", seed=55, causal=True, k_pos0=10,
                                            num_splits=2), "fully masked row")


def test_decode_dropout_follows_the_reference_streams():
    gpu_util.assert_close(gpu_util.run_case(2, 4, 1, 2048, 128, "bfloat16", seed=56, p_dropout=0.2, drop_seed=11,
                                            num_splits=1), "dropout")
    gpu_util.assert_close(gpu_util.run_case(2, 4, 1, 4096, 128, "bfloat16", seed=57, p_dropout=0.1, drop_seed=42,
                                            num_splits=4, offset=8), "dropout split")


def test_decode_config4_shape_sampled_units():
    # bf16 B=64 H=32 q=1 kv=32768 d=128, 16 splits: every unit is computed, a sample is checked
    import flash_attn_b200 as fa
    B, H, Nk, d = 64, 32, 32768, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    q = torch.randn((B, H, 1, d), generator=g, device="cuda").bfloat16()
    k = torch.randn((B, H, Nk, d), generator=g, device="cuda").bfloat16()
    v = torch.randn((B, H, Nk, d), generator=g, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o, lse = fa.flash_attn_forward(q, k, v, num_splits=16, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for b, h in ((0, 0), (63, 31), (17, 5), (40, 20)):
        want_o, want_lse = oracle_lib.forward(q[b:b + 1, h:h + 1].float().cpu().numpy(), k[b:b + 1, h:h + 1].float().cpu().numpy(),
                                              v[b:b + 1, h:h + 1].float().cpu().numpy(), d ** -0.5)
        err = np.abs(o[b, h].float().cpu().numpy() - want_o[0, 0])
        assert err.max() <= gpu_util.O_MAX_ABS and err.mean() <= gpu_util.O_MEAN_ABS, (b, h, err.max())
        assert abs(lse[b, h, 0].item() - want_lse[0, 0, 0]) <= gpu_util.LSE_ABS
