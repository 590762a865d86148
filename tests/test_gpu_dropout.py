"""Dropout parity: the stateless Philox mask must equal, bit for bit, the mask of
the reference's cuRAND draw order (pinned on the CPU by tests/test_oracle.py)."""
import json
import os

import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib
import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", [
    dict(B=1, H=2, Nq=200, Nk=200, p=0.1, seed=42),
    dict(B=2, H=3, Nq=300, Nk=500, p=0.25, seed=48, offset=0),
    dict(B=1, H=2, Nq=256, Nk=512, p=0.1, seed=7, num_splits=2),
    dict(B=1, H=1, Nq=400, Nk=400, p=0.5, seed=9, window_left=130),
    dict(B=1, H=2, Nq=130, Nk=260, p=0.1, seed=42, offset=6),
    dict(B=1, H=2, Nq=130, Nk=260, p=0.1, seed=42, offset=64),
])
def test_mask_kernel_matches_oracle_map(case):
    import flash_attn_b200 as fa
    c = dict(offset=0, num_splits=1, window_left=-1)
    c.update(case)
    got = fa.dropout_mask(c["B"], c["H"], c["Nq"], c["Nk"], c["p"], c["seed"], c["offset"], c["num_splits"],
                          c["window_left"]).cpu().numpy()
    want = oracle_lib.dropout_mask(c["B"], c["H"], c["Nq"], c["Nk"], np.float32(c["p"]).item(), c["seed"],
                                   c["offset"], c["num_splits"], c["window_left"])
    assert np.array_equal(got, want)


def test_mask_kernel_matches_simulated_reference_kernel(golden_dir):
    import flash_attn_b200 as fa
    z = np.load(os.path.join(golden_dir, "dropout_mask_sim.npz"))
    for i, c in enumerate(json.loads(bytes(z["meta"]).decode())):
        want = z[f"mask{i}"]
        p = np.uint32(c["p_bits"]).view(np.float32).item()
        got = fa.dropout_mask(c["B"], c["H"], c["N"], c["N"], p, c["seed"], 0, c["splits"], c["wl"]).cpu().numpy()
        visited = want != 2
        assert np.array_equal(got[visited], want[visited]), c


def _mask_applied_by_forward(B, H, N, d, p, seed, dtype, **kw):
    """Reads the mask out of the forward kernel itself: with Q = 0 every P is 1/N,
    and with V = a tile-weighted identity O[row, c] = sum_t 2^t * keep[row, 128 t + c] / (N (1-p))."""
    import flash_attn_b200 as fa
    tiles = (N + 127) // 128
    assert tiles <= 8 and d == 128
    q = torch.zeros(B, H, N, d, dtype=dtype, device="cuda")
    k = torch.zeros(B, H, N, d, dtype=dtype, device="cuda")
    v = torch.zeros(B, H, N, d, dtype=torch.float32, device="cuda")
    idx = torch.arange(N, device="cuda")
    v[:, :, idx, idx % 128] = (2.0 ** (idx // 128)).float()
    o, _ = fa.flash_attn_forward(q, k, v.to(dtype), softmax_scale=1.0, p_dropout=p, seed=seed,
                                 out_dtype=torch.float32, **kw)
    # keys a row attends to: all N, or with a causal mask those up to the row itself
    visible = (idx + 1).double() if kw.get("causal") else torch.full((N,), float(N), device="cuda", dtype=torch.float64)
    code = torch.round(o.double() * (visible * (1.0 - np.float32(p).item()))[None, None, :, None]).to(torch.int64)  # [B,H,N,128]
    keep = torch.zeros(B, H, N, tiles * 128, dtype=torch.uint8, device="cuda")
    for t in range(tiles):
        keep[..., t * 128:(t + 1) * 128] = ((code >> t) & 1).to(torch.uint8)
    return keep[..., :N].cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_forward_kernel_applies_exactly_the_reference_mask(dtype):
    B, H, N, p, seed = 1, 2, 512, 0.1, 42
    got = _mask_applied_by_forward(B, H, N, 128, p, seed, dtype)
    want = oracle_lib.dropout_mask(B, H, N, N, np.float32(p).item(), seed)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("N,causal", [(640, False), (1024, False), (1024, True), (900, True)])
def test_forward_kernel_mask_over_many_kv_tiles(N, causal):
    # five to eight KV tiles per query tile: the keep bits pass through the helper warp's ring of four
    # tiles several times, with an odd tile count (a last chunk of one tile) and, under the causal mask,
    # a different tile count for every query tile
    B, H, p, seed = 1, 2, 0.2, 11
    got = _mask_applied_by_forward(B, H, N, 128, p, seed, torch.bfloat16, causal=causal)
    want = oracle_lib.dropout_mask(B, H, N, N, np.float32(p).item(), seed)
    if causal:
        vis = np.tril(np.ones((N, N), dtype=bool))[None, None]
        assert np.array_equal(got[np.broadcast_to(vis, got.shape)], want[np.broadcast_to(vis, want.shape)])
    else:
        assert np.array_equal(got, want)


def test_forward_with_dropout_matches_oracle():
    gpu_util.assert_close(gpu_util.run_case(1, 2, 384, 384, 128, "bfloat16", seed=21, causal=True, p_dropout=0.1,
                                            drop_seed=42), "dropout causal")
    gpu_util.assert_close(gpu_util.run_case(2, 2, 200, 456, 64, "float16", seed=22, p_dropout=0.3, drop_seed=5,
                                            offset=12), "dropout offset")
    gpu_util.assert_close(gpu_util.run_case(1, 2, 256, 1024, 64, "float16", seed=23, p_dropout=0.1, drop_seed=7,
                                            num_splits=2), "dropout split")


def test_config2_shape_sampled_rows():
    # bf16 [8,16,2048,128] causal, dropout 0.1, Philox seed 42, offset 0: sampled rows against the oracle
    B, H, N, d = 8, 16, 2048, 128
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([
        rng.integers(0, B * H * N, 256),
        np.array([0, 127, 128, N - 1, N, B * H * N - 1, (B * H - 1) * N + 1023])])).astype(np.int64)
    res = gpu_util.run_case(B, H, N, N, d, "bfloat16", seed=2, causal=True, p_dropout=0.1, drop_seed=42, rows=rows)
    gpu_util.assert_close(res, "config 2")
