"""Regenerates every fixture in tests/golden/ (run in a container that has the
reference checkout and the CUDA toolkit headers; the fixtures themselves are
committed so the tests need neither).

    python tests/golden/make_fixtures.py [--reference /path/to/reference]

Sources of truth:
  philox_kat.json, dropout_mask_sim.npz  <- NVIDIA cuRAND Philox4_32_10 device API run
                                            on the host (gen_curand_vectors.cpp)
  reference_cpu.npz                      <- the reference's attention_forward_cpu
                                            (src/main.cu:279-388) from oracle/_ref/libref.so
  num_splits_heuristic.json              <- the reference's num_splits_heuristic
                                            (src/main.cu:391-422) from the same library
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def curand_vectors():
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "gen_curand")
        subprocess.check_call(["g++", "-O2", "-w", "-I/usr/local/cuda/include",
                               os.path.join(HERE, "gen_curand_vectors.cpp"), "-o", exe])
        subprocess.check_call([exe, tmp])
        with open(os.path.join(tmp, "philox_kat.json")) as f:
            kat = json.load(f)
        with open(os.path.join(HERE, "philox_kat.json"), "w") as f:
            json.dump(kat, f, indent=1)
        with open(os.path.join(tmp, "dropout_mask_sim.json")) as f:
            sim = json.load(f)
    out = {}
    meta = []
    for i, c in enumerate(sim["cases"]):
        s = np.frombuffer(c.pop("mask").encode(), dtype=np.uint8)
        m = np.where(s == ord("."), 2, s - ord("0")).astype(np.uint8)
        out[f"mask{i}"] = m.reshape(c["B"], c["H"], c["N"], c["N"])
        meta.append(c)
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "dropout_mask_sim.npz"), **out)


def reference_cpu(libref):
    """Reference CPU attention on exactly reproducible inputs (tests/synth.py).
    Only every `row_step`-th query row of O is stored; inputs are regenerated
    from (seed, shape) by the tests."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth
    fn = libref._Z21attention_forward_cpuPfS_S_fiiiiS_biS_
    fp = ctypes.POINTER(ctypes.c_float)
    fn.argtypes = [fp, fp, fp, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   fp, ctypes.c_bool, ctypes.c_int, fp]
    fn.restype = None
    cases = [
        # name, B, H, N, d, dtype, causal, window, alibi, sigma, row_step
        ("c1_fp16_b1h4n256d64", 1, 4, 256, 64, "float16", False, -1, False, 1.0, 5),
        ("causal_bf16_b1h2n200d128", 1, 2, 200, 128, "bfloat16", True, -1, False, 1.0, 3),
        ("window_alibi_bf16_b2h3n160d64", 2, 3, 160, 64, "bfloat16", True, 48, True, 1.0, 3),
        ("sym_window_fp16_b1h2n130d32", 1, 2, 130, 32, "float16", False, 17, False, 1.0, 1),
        ("alibi_only_fp16_b1h2n96d40", 1, 2, 96, 40, "float16", False, -1, True, 0.5, 1),
        ("causal_window_bf16_b1h1n384d128", 1, 1, 384, 128, "bfloat16", True, 130, False, 1.0, 7),
    ]
    out = {}
    meta = []
    for seed, (name, B, H, N, d, dt, causal, window, alibi, sigma, step) in enumerate(cases):
        q, k, v = synth.qkv(seed, B, H, N, N, d, dt, sigma)
        o = np.zeros_like(q)
        slopes = synth.alibi_slopes(H) if alibi else None
        scale = np.float32(1.0 / np.sqrt(d))
        fn(q.ctypes.data_as(fp), k.ctypes.data_as(fp), v.ctypes.data_as(fp), scale, B, H, N, d,
           o.ctypes.data_as(fp), causal, window, slopes.ctypes.data_as(fp) if alibi else None)
        out[f"{name}.o"] = np.ascontiguousarray(o[:, :, ::step, :])
        meta.append(dict(name=name, seed=seed, B=B, H=H, N=N, d=d, dtype=dt, causal=causal, window=window,
                         alibi=alibi, sigma=sigma, scale=float(scale), row_step=step))
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "reference_cpu.npz"), **out)


def heuristic(libref):
    fn = libref._Z20num_splits_heuristiciiiii
    fn.argtypes = [ctypes.c_int] * 5
    fn.restype = ctypes.c_int
    rows = []
    for sms in (108, 148):
        for bh in (1, 2, 4, 8, 16, 32, 128, 2048):
            for n in (128, 256, 1021, 1024, 2048, 4096, 8192, 32768):
                tr = (n + 127) // 128
                padded = tr * 128
                # call shape of the reference launcher, src/main.cu:125
                rows.append([bh * tr, sms, tr, tr, padded, fn(bh * tr, sms, tr, tr, padded)])
    with open(os.path.join(HERE, "num_splits_heuristic.json"), "w") as f:
        json.dump({"columns": ["batch_nheads_mblocks", "num_sms", "num_n_blocks", "max_splits", "seq_len", "splits"],
                   "rows": rows}, f)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FA_REFERENCE_DIR"), required="FA_REFERENCE_DIR" not in os.environ,
                    help="path of the reference checkout (or the environment variable FA_REFERENCE_DIR)")
    args = ap.parse_args()
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), f"REF={args.reference}", "all"])
    curand_vectors()
    libref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref.so"))
    reference_cpu(libref)
    heuristic(libref)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    sys.exit(main())
