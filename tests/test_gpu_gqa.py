"""Grouped-query attention (K/V with fewer heads than Q) against the oracle run on K/V
repeated per query head.  The reference has a single head count (gridDim.y,
src/main.cu:142); this is the decode-side generalisation of its split-KV path."""
import pytest

import gpu_util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H,Hk", [(8, 2), (4, 1), (6, 3)])
def test_gqa_tiled_causal(H, Hk):
    res = gpu_util.run_case(2, H, 384, 384, 128, causal=True, heads_k=Hk, seed=11)
    gpu_util.assert_close(res, f"gqa causal H={H} Hk={Hk}")


def test_gqa_tiled_dropout_alibi_fp16():
    res = gpu_util.run_case(1, 8, 256, 512, 64, dtype="float16", causal=True, q_pos0=256, alibi=True, p_dropout=0.1,
                            heads_k=2, seed=12)
    gpu_util.assert_close(res, "gqa dropout alibi fp16")


def test_gqa_split_and_padded_head_dim():
    res = gpu_util.run_case(1, 4, 130, 700, 72, heads_k=2, num_splits=3, seed=13)
    gpu_util.assert_close(res, "gqa split")
    res = gpu_util.run_case(1, 4, 100, 300, 31, dtype="float16", heads_k=1, seed=14)
    gpu_util.assert_close(res, "gqa head_dim 31")


@pytest.mark.parametrize("Hk,splits", [(2, 1), (1, 4), (8, 2)])
def test_gqa_decode(Hk, splits):
    res = gpu_util.run_case(2, 8, 1, 1500, 128, heads_k=Hk, num_splits=splits, q_pos0=1499, causal=True, seed=15)
    gpu_util.assert_close(res, f"gqa decode Hk={Hk} splits={splits}")


@pytest.mark.parametrize("H,Hk", [(16, 1), (6, 2), (24, 2)])
def test_gqa_decode_group_sizes(H, Hk):
    # groups of 16 and 12 heads are cut into sub-groups of eight; a group of 3 leaves operand rows unused
    res = gpu_util.run_case(1, H, 1, 2100, 128, heads_k=Hk, num_splits=3, seed=17)
    gpu_util.assert_close(res, f"gqa decode H={H} Hk={Hk}")


def test_gqa_decode_dropout_alibi_window_fp16():
    res = gpu_util.run_case(2, 8, 1, 1000, 64, dtype="float16", heads_k=2, num_splits=2, q_pos0=999, causal=True,
                            window=(600, 0), alibi=True, p_dropout=0.2, seed=18)
    gpu_util.assert_close(res, "gqa decode dropout alibi window")


@pytest.mark.parametrize("H,Hk,Nq,splits", [(4, 4, 4, 3), (8, 2, 2, 2), (4, 2, 3, 1), (8, 1, 8, 4), (2, 2, 8, 1), (6, 3, 5, 2)])
def test_short_query_blocks_on_the_decode_kernel(H, Hk, Nq, splits):
    # 2..8 query rows per head (bottom-right causal: the last rows of the sequence), packed with the
    # heads of a K/V group into the eight columns of the decode kernel
    Nk = 1300
    res = gpu_util.run_case(2, H, Nq, Nk, 128, heads_k=Hk, num_splits=splits, q_pos0=Nk - Nq, causal=True, seed=19)
    gpu_util.assert_close(res, f"short q H={H} Hk={Hk} Nq={Nq} splits={splits}")


def test_short_query_dropout_alibi_window_fp16():
    res = gpu_util.run_case(1, 4, 5, 900, 64, dtype="float16", heads_k=2, num_splits=2, q_pos0=895, causal=True,
                            window=(500, 0), alibi=True, p_dropout=0.2, seed=20)
    gpu_util.assert_close(res, "short q dropout alibi window")
    res = gpu_util.run_case(1, 2, 7, 640, 128, q_pos0=100, causal=True, p_dropout=0.1, seed=21)  # rows that see few keys
    gpu_util.assert_close(res, "short q early rows")


def test_gqa_host_buffers():
    res = gpu_util.run_case(3, 6, 256, 256, 128, causal=True, heads_k=2, host=True, seed=16)
    gpu_util.assert_close(res, "gqa host path")


def test_gqa_rejects_bad_group():
    import torch
    import flash_attn_b200 as fa
    q = torch.zeros(1, 6, 128, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 4, 128, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        fa.flash_attn_forward(q, k, k)
