"""The C benchmark driver (csrc/fa_main.c, the successor of the reference's main()):
its dumped result must match the CPU oracle on the same, bit-reproducible inputs."""
import json
import os
import subprocess
import tempfile

import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib
import synth

pytestmark = pytest.mark.gpu


def _run(args):
    from flash_attn_b200 import build
    exe = build.build_driver()
    with tempfile.TemporaryDirectory() as tmp:
        dump = os.path.join(tmp, "o.bin")
        out = subprocess.check_output([exe] + args + ["--dump", dump], timeout=600).decode()
        return json.loads(out.strip().splitlines()[-1]), open(dump, "rb").read()


def _check(raw, units, Nq, Nk, d, dtype, data_seed, **kw):
    n = units * Nq * d
    tdt = gpu_util.TORCH_DT[dtype]
    o = torch.frombuffer(bytearray(raw[:2 * n]), dtype=tdt).float().numpy().reshape(1, units, Nq, d)
    lse = np.frombuffer(raw[2 * n:2 * n + 4 * units * Nq], dtype=np.float32).reshape(1, units, Nq)
    q, k, v = synth.qkv(data_seed, 1, units, Nq, Nk, d, dtype)
    want_o, want_lse = oracle_lib.forward(q, k, v, 1 / np.sqrt(d), **kw)
    err = np.abs(o - want_o)
    assert err.max() <= gpu_util.O_MAX_ABS and err.mean() <= gpu_util.O_MEAN_ABS, (err.max(), err.mean())
    assert np.abs(lse - want_lse).max() <= gpu_util.LSE_ABS


def test_driver_config1_full_tensor():
    line, raw = _run(["--config", "1", "--iters", "3"])
    assert line["driver"] == "fa_bench" and line["units"] == 4 and line["ms_per_iter"] > 0
    _check(raw, 4, 256, 256, 64, "float16", 0)


def test_driver_config2_first_units_with_dropout():
    line, raw = _run(["--config", "2", "--units", "3", "--iters", "2"])
    _check(raw, 3, 2048, 2048, 128, "bfloat16", 2, causal=True, p_dropout=np.float32(0.1).item(), seed=42)
    assert line["tflops"] > 0


def test_driver_config4_first_units_decode():
    line, raw = _run(["--config", "4", "--units", "2", "--iters", "2"])
    _check(raw, 2, 1, 32768, 128, "bfloat16", 4)
    assert line["gbs"] > 0
