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


@pytest.mark.parametrize("args", [["--config", "1"], ["--config", "2", "--units", "4"], ["--config", "3", "--units", "3"],
                                  ["--config", "4", "--units", "2"]])
def test_driver_checks_itself(args):
    # --check: the driver's own verification on sampled rows (plain fp32 attention in the driver, not the
    # oracle) and its CPU timing leg, as the reference's main() has them (src/main.cu:212-225)
    from flash_attn_b200 import build
    exe = build.build_driver()
    out = subprocess.run([exe] + args + ["--iters", "2", "--check"], capture_output=True, timeout=600)
    assert out.returncode == 0, out.stderr.decode()
    line = json.loads(out.stdout.decode().strip().splitlines()[-1])
    assert line["check"]["pass"] is True and line["check"]["rows"] >= 8
    assert line["cpu"]["ms_per_row"] > 0


def test_driver_config5_ring_on_one_gpu():
    # the ring through fa_ring_fwd with one rank (no exchange), at a shortened sequence
    from flash_attn_b200 import build
    exe = build.build_driver()
    out = subprocess.run([exe, "--config", "5", "--gpus", "1", "--iters", "1", "--warmup", "1", "--seq", "16384"],
                         capture_output=True, timeout=600)
    assert out.returncode == 0, out.stderr.decode()
    line = json.loads(out.stdout.decode().strip().splitlines()[-1])
    assert line["n_gpus"] == 1 and line["tflops"] > 0 and line["chunk_rows"] == 8192
