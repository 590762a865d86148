"""Pins the CPU oracle: cuRAND host KATs, the simulated reference dropout mask,
the reference's own CPU attention outputs and its split policy."""
import json
import os

import numpy as np
import pytest

import oracle_lib
import synth


def _load_meta(npz):
    return json.loads(bytes(npz["meta"]).decode())


def test_philox_matches_curand_kats(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "philox_kat.json")))
    L = oracle_lib.lib()
    for c in kat["cases"]:
        raw = [L.fa_oracle_curand_draw(c["seed"], c["subsequence"], c["offset"], n) for n in range(len(c["raw"]))]
        assert raw == c["raw"]
        uni = [np.float32(L.fa_oracle_uniform(x)).view(np.uint32).item() for x in raw]
        assert uni == c["uniform_hex"]


def test_keep_threshold_matches_curand_uniform(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "philox_kat.json")))
    L = oracle_lib.lib()
    for t in kat["thresholds"]:
        p = np.uint32(t["p_bits"]).view(np.float32).item()
        assert L.fa_oracle_keep_threshold(p) == t["first_kept"]
    # the value quoted for p = 0.1f: raw draws below 429496721 are dropped
    assert L.fa_oracle_keep_threshold(np.float32(0.1).item()) == 429496721


def test_dropout_map_matches_simulated_reference_kernel(golden_dir):
    z = np.load(os.path.join(golden_dir, "dropout_mask_sim.npz"))
    for i, c in enumerate(_load_meta(z)):
        want = z[f"mask{i}"]
        p = np.uint32(c["p_bits"]).view(np.float32).item()
        got = oracle_lib.dropout_mask(c["B"], c["H"], c["N"], c["N"], p, c["seed"], 0, c["splits"], c["wl"])
        visited = want != 2
        assert visited.any()
        assert np.array_equal(got[visited], want[visited]), f"case {i}: {c}"
        frac = got[visited].mean()
        assert abs(frac - (1 - p)) < 0.08


def test_attention_matches_reference_cpu_bit_for_bit(golden_dir):
    z = np.load(os.path.join(golden_dir, "reference_cpu.npz"))
    for c in _load_meta(z):
        q, k, v = synth.qkv(c["seed"], c["B"], c["H"], c["N"], c["N"], c["d"], c["dtype"], c["sigma"])
        slopes = synth.alibi_slopes(c["H"]) if c["alibi"] else None
        o, lse = oracle_lib.forward(q, k, v, np.float32(c["scale"]), causal=c["causal"],
                                    window=(c["window"], c["window"]), alibi_slopes=slopes)
        want = z[c["name"] + ".o"]
        got = o[:, :, ::c["row_step"], :]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), c["name"]
        assert np.isfinite(lse).all()


def test_attention_matches_live_reference_when_built():
    if oracle_lib.reference_lib() is None:
        pytest.skip("oracle/_ref/libref.so not built in this checkout")
    q, k, v = synth.qkv(11, 1, 2, 150, 150, 24, "float16")
    want = oracle_lib.reference_cpu_forward(q, k, v, 0.2, causal=True, window=40)
    got, _ = oracle_lib.forward(q, k, v, 0.2, causal=True, window=(40, 40))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_lse_and_row_subset_and_extensions():
    q, k, v = synth.qkv(5, 1, 2, 70, 190, 32, "bfloat16")
    scale = 1 / np.sqrt(32)
    o, lse = oracle_lib.forward(q, k, v, scale, causal=True, q_pos0=120)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) * scale
    qi = 120 + np.arange(70)[:, None]
    kj = np.arange(190)[None, :]
    s = np.where(kj > qi, -np.inf, s)
    m = s.max(-1, keepdims=True)
    pe = np.exp(s - m)
    want_lse = (m + np.log(pe.sum(-1, keepdims=True)))[..., 0]
    want_o = np.einsum("bhqk,bhkd->bhqd", pe / pe.sum(-1, keepdims=True), v.astype(np.float64))
    assert np.abs(lse - want_lse).max() < 1e-4
    assert np.abs(o - want_o).max() < 1e-4
    rows = np.array([0, 69, 70, 139, 33], dtype=np.int64)
    o2, lse2 = oracle_lib.forward(q, k, v, scale, causal=True, q_pos0=120, rows=rows)
    assert np.array_equal(o2, o.reshape(-1, 32)[rows])
    assert np.array_equal(lse2, lse.reshape(-1)[rows])
    # a fully masked row gives O = 0 and LSE = -inf instead of the reference's NaN
    o3, lse3 = oracle_lib.forward(q, k, v, scale, causal=True, k_pos0=10)
    assert np.all(o3[:, :, :10] == 0) and np.all(np.isneginf(lse3[:, :, :10]))
    assert np.isfinite(o3).all()


def test_dropout_in_oracle_scales_and_zeroes():
    q, k, v = synth.qkv(6, 1, 1, 130, 130, 16, "float16")
    p = np.float32(0.1).item()
    o0, lse0 = oracle_lib.forward(q, k, v, 0.25)
    o1, lse1 = oracle_lib.forward(q, k, v, 0.25, p_dropout=p, seed=42)
    assert np.array_equal(lse0, lse1)
    keep = oracle_lib.dropout_mask(1, 1, 130, 130, p, 42)[0, 0].astype(np.float64)
    s = (q[0, 0].astype(np.float64) @ k[0, 0].astype(np.float64).T) * 0.25
    pm = np.exp(s - s.max(-1, keepdims=True))
    pm /= pm.sum(-1, keepdims=True)
    want = (pm * keep / (1 - p)) @ v[0, 0].astype(np.float64)
    assert np.abs(o1[0, 0] - want).max() < 1e-4
    assert np.abs(o1 - o0).max() > 1e-3


def test_split_policy_matches_reference(golden_dir):
    t = json.load(open(os.path.join(golden_dir, "num_splits_heuristic.json")))
    L = oracle_lib.lib()
    for a, b, c, d, e, want in t["rows"]:
        assert L.fa_oracle_num_splits_heuristic(a, b, c, d, e) == want, (a, b, c, d, e)
