"""GPU parity tests of the tiled forward path: CUDA result through the C ABI
versus the CPU oracle, on exactly reproducible inputs.

Tolerances (16-bit O against the fp32 oracle): max-abs 2e-2, mean-abs 2e-3, LSE
1e-3 -- the values in gpu_util.py.  Dropout masks must be bit-exact."""
import json
import os

import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib
import synth

pytestmark = pytest.mark.gpu


def test_config1_fp16_noncausal_full_tensor():
    # fp16 [B=1,H=4,N=256,d=64], scale 1/8, no masks: the reference's CPU-runnable case
    gpu_util.assert_close(gpu_util.run_case(1, 4, 256, 256, 64, "float16", seed=0), "config 1")


def test_config1_matches_reference_cpu_fixture(golden_dir):
    import flash_attn_b200 as fa
    z = np.load(os.path.join(golden_dir, "reference_cpu.npz"))
    for c in json.loads(bytes(z["meta"]).decode()):
        q, k, v = synth.qkv(c["seed"], c["B"], c["H"], c["N"], c["N"], c["d"], c["dtype"], c["sigma"])
        slopes = torch.from_numpy(synth.alibi_slopes(c["H"])) if c["alibi"] else None
        o, _ = fa.flash_attn_forward(gpu_util.to_dev(q, c["dtype"]), gpu_util.to_dev(k, c["dtype"]),
                                     gpu_util.to_dev(v, c["dtype"]), softmax_scale=c["scale"], causal=c["causal"],
                                     window=(c["window"], c["window"]), alibi_slopes=slopes)
        got = o.float().cpu().numpy()[:, :, ::c["row_step"], :]
        want = z[c["name"] + ".o"]
        err = np.abs(got - want)
        assert err.max() <= gpu_util.O_MAX_ABS and err.mean() <= gpu_util.O_MEAN_ABS, (c["name"], err.max(), err.mean())


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("d", [64, 128])
def test_plain_shapes(dtype, d):
    gpu_util.assert_close(gpu_util.run_case(2, 3, 384, 384, d, dtype, seed=1), f"{dtype} d={d}")


@pytest.mark.parametrize("n", [1, 17, 127, 128, 129, 200, 333])
def test_ragged_sequence_lengths(n):
    # rows and key columns beyond the end are zero-filled by TMA and masked
    gpu_util.assert_close(gpu_util.run_case(1, 2, n, n, 64, "bfloat16", seed=2), f"N={n}")
    gpu_util.assert_close(gpu_util.run_case(1, 2, n, n, 128, "float16", seed=3, causal=True), f"N={n} causal")


def test_seqlen_q_differs_from_seqlen_k():
    gpu_util.assert_close(gpu_util.run_case(2, 2, 100, 700, 128, "bfloat16", seed=4), "Nq=100 Nk=700")
    gpu_util.assert_close(gpu_util.run_case(1, 2, 300, 50, 64, "float16", seed=5), "Nq=300 Nk=50")


def test_causal_and_positions():
    gpu_util.assert_close(gpu_util.run_case(1, 2, 512, 512, 128, "bfloat16", seed=6, causal=True), "causal")
    # bottom-right aligned causal: the last 130 queries of a 600-key sequence
    gpu_util.assert_close(gpu_util.run_case(1, 2, 130, 600, 64, "bfloat16", seed=7, causal=True, q_pos0=470),
                          "causal q_pos0")
    # keys that start after some queries: the first rows are fully masked -> O = 0, LSE = -inf
    gpu_util.assert_close(gpu_util.run_case(1, 1, 256, 256, 64, "float16", seed=8, causal=True, k_pos0=100),
                          "causal k_pos0 (fully masked rows)")


@pytest.mark.parametrize("window", [(128, 0), (1024, 0), (130, 5), (0, 0), (17, 17), (-1, 40), (64, -1)])
def test_local_windows(window):
    gpu_util.assert_close(gpu_util.run_case(1, 2, 640, 640, 128, "bfloat16", seed=9, causal=window[1] == 0,
                                            window=window), f"window {window}")


def test_alibi():
    gpu_util.assert_close(gpu_util.run_case(1, 4, 384, 384, 128, "bfloat16", seed=10, alibi=True), "alibi")
    gpu_util.assert_close(gpu_util.run_case(2, 4, 300, 300, 64, "float16", seed=11, alibi=True, causal=True,
                                            window=(100, 0)), "alibi + causal + window")


def test_alibi_far_keys_and_ring_positions():
    # pure causal ALiBi over 1536 keys (the bias of the far tiles is large; the part linear in the key
    # column comes from the tensor core, the row constant from the softmax), in both 16-bit formats, with a
    # small softmax scale (large bias entries in units of the raw scores), and on a key block that lies
    # wholly before the query block (positions as in a sequence ring: q_pos0 > k_pos0, no causal test)
    gpu_util.assert_close(gpu_util.run_case(1, 4, 1536, 1536, 128, "bfloat16", seed=13, alibi=True, causal=True),
                          "alibi causal bf16")
    gpu_util.assert_close(gpu_util.run_case(1, 4, 1536, 1536, 128, "float16", seed=14, alibi=True, causal=True),
                          "alibi causal fp16")
    gpu_util.assert_close(gpu_util.run_case(1, 2, 512, 512, 64, "float16", seed=15, alibi=True, causal=True,
                                            scale=0.01), "alibi causal fp16, small scale")
    gpu_util.assert_close(gpu_util.run_case(1, 4, 512, 512, 128, "bfloat16", seed=16, alibi=True,
                                            window=(-1, 0), q_pos0=2048, k_pos0=1024), "alibi, keys before queries")


def test_alibi_steep_and_negative_slopes():
    # slopes far outside the usual 2^(-8(h+1)/H): steep ones keep the bias in the softmax, negative ones
    # (the sign the reference's own main() passes) go through the tensor core like any other
    import flash_attn_b200 as fa
    B, H, N, d = 1, 4, 512, 128
    q, k, v = synth.qkv(17, B, H, N, N, d, "bfloat16", 1.0)
    slopes = np.array([6.0, -0.5, 0.02, -3.0], dtype=np.float32)
    scale = 1.0 / np.sqrt(d)
    o, lse = fa.flash_attn_forward(gpu_util.to_dev(q, "bfloat16"), gpu_util.to_dev(k, "bfloat16"),
                                   gpu_util.to_dev(v, "bfloat16"), softmax_scale=scale, causal=True,
                                   alibi_slopes=torch.from_numpy(slopes))
    want_o, want_lse = oracle_lib.forward(q, k, v, scale, causal=True, alibi_slopes=slopes)
    assert np.abs(o.float().cpu().numpy() - want_o).max() < 2e-2
    assert np.abs(lse.cpu().numpy() - want_lse).max() < 2e-3


def test_config3_shape_scaled_down():
    # causal + window(1024, 0) + ALiBi slopes 2^(-8(h+1)/H), as config 3, at N = 2304
    gpu_util.assert_close(gpu_util.run_case(1, 4, 2304, 2304, 128, "bfloat16", seed=12, causal=True,
                                            window=(1024, 0), alibi=True), "config 3 (scaled)")


def test_fp32_output_like_the_reference():
    res = gpu_util.run_case(1, 2, 256, 256, 64, "float16", seed=13, out_dtype=torch.float32)
    gpu_util.assert_close(res, "fp32 O")


@pytest.mark.parametrize("d", [8, 32, 40, 96, 120])
def test_head_dims_below_the_tile(d):
    gpu_util.assert_close(gpu_util.run_case(1, 2, 200, 200, d, "float16", seed=14, causal=True), f"d={d}")


def test_head_dims_that_are_not_multiples_of_8():
    # the reference's default launch: fp16 [1,8,1021,31] -> fp32 O (src/main.cu:39-42); served by a padded copy
    gpu_util.assert_close(gpu_util.run_case(1, 8, 1021, 1021, 31, "float16", seed=24, out_dtype=torch.float32),
                          "reference default shape")
    gpu_util.assert_close(gpu_util.run_case(2, 2, 300, 500, 20, "bfloat16", seed=25, causal=True, q_pos0=200,
                                            p_dropout=0.1, num_splits=2), "d=20 causal dropout split")
    gpu_util.assert_close(gpu_util.run_case(1, 3, 1, 900, 100, "bfloat16", seed=26, num_splits=3), "d=100 decode")


@pytest.mark.parametrize("splits", [2, 3, 4])
def test_split_kv_and_combine(splits):
    gpu_util.assert_close(gpu_util.run_case(1, 2, 256, 1024, 64, "float16", seed=15, num_splits=splits),
                          f"splits={splits}")
    gpu_util.assert_close(gpu_util.run_case(1, 2, 300, 900, 128, "bfloat16", seed=16, causal=True, q_pos0=600,
                                            num_splits=splits), f"splits={splits} causal (empty splits)")


def test_split_invariance():
    # property: the result does not depend on the split count beyond rounding
    import flash_attn_b200 as fa
    q, k, v = (gpu_util.to_dev(x, "bfloat16") for x in synth.qkv(17, 1, 4, 128, 2048, 128, "bfloat16"))
    o1, l1 = fa.flash_attn_forward(q, k, v, num_splits=1)
    for s in (2, 8, 16):
        o2, l2 = fa.flash_attn_forward(q, k, v, num_splits=s)
        assert (o1.float() - o2.float()).abs().max().item() <= 8e-3
        assert (l1 - l2).abs().max().item() <= 1e-4


def test_decode_shape_single_query():
    gpu_util.assert_close(gpu_util.run_case(4, 8, 1, 4096, 128, "bfloat16", seed=18, num_splits=16), "decode")
    gpu_util.assert_close(gpu_util.run_case(2, 4, 1, 1000, 128, "bfloat16", seed=19, num_splits=1), "decode ragged")


def test_heuristic_split_is_used_when_num_splits_is_zero():
    gpu_util.assert_close(gpu_util.run_case(1, 4, 256, 256, 64, "float16", seed=0, num_splits=0), "auto split")


def test_determinism():
    import flash_attn_b200 as fa
    q, k, v = (gpu_util.to_dev(x, "bfloat16") for x in synth.qkv(20, 2, 4, 512, 512, 128, "bfloat16"))
    o1, l1 = fa.flash_attn_forward(q, k, v, causal=True, p_dropout=0.1, seed=3)
    o2, l2 = fa.flash_attn_forward(q, k, v, causal=True, p_dropout=0.1, seed=3)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_argument_errors():
    import flash_attn_b200 as fa
    from flash_attn_b200 import _lib
    q = torch.zeros(1, 1, 128, 136, dtype=torch.float16, device="cuda")
    with pytest.raises(_lib.FaError) as e:
        fa.flash_attn_forward(q, q, q)
    assert e.value.code == -2  # head_dim > 128
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(_lib.FaError) as e:
        fa.flash_attn_forward(q, q, q, softmax_scale=-1.0)
    assert e.value.code == -1
    with pytest.raises(_lib.FaError) as e:
        fa.flash_attn_forward(q, q, q, p_dropout=1.0)
    assert e.value.code == -1
