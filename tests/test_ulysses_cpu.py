"""Host logic of the head-sharded (all-to-all) multi-GPU path on CPU ranks (gloo, world_size 2
and 4): the two layout exchanges are inverses, and attention through them equals the
single-device result, with grouped-query K/V, ALiBi slopes and the dropout streams keyed on
global heads.  The kernels are replaced by the CPU oracle here."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib
import synth

HERE = os.path.dirname(os.path.abspath(__file__))


def _oracle_attend(q, k, v, scale, causal, slopes, p, seed, unit0):
    H, Hk = q.shape[1], k.shape[1]
    qq = q.float().numpy()
    kk = np.repeat(k.float().numpy(), H // Hk, axis=1)
    vv = np.repeat(v.float().numpy(), H // Hk, axis=1)
    sl = None if slopes is None else slopes.numpy()
    pad = 0
    if p > 0.0 and unit0 > 0:
        # the oracle numbers its dropout streams from unit 0: put unit0 dummy heads in front
        # (one batch entry, so unit = head), which gives the real heads their global numbers
        assert q.shape[0] == 1
        pad = unit0
        z = lambda x: np.concatenate([np.zeros((1, pad) + x.shape[2:], np.float32), x], axis=1)
        qq, kk, vv = z(qq), z(kk), z(vv)
        if sl is not None:
            sl = np.concatenate([np.zeros(pad, np.float32), sl])
    o, lse = oracle_lib.forward(qq, kk, vv, scale, causal=causal, alibi_slopes=sl, p_dropout=p, seed=seed,
                                num_threads=1)
    return torch.from_numpy(o[:, pad:].copy()), torch.from_numpy(lse[:, pad:].copy())


def _worker(rank, world, port, case, out):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from datetime import timedelta
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=30))
    try:
        from flash_attn_b200 import ulysses
        B, H, Hk, N, d = case["B"], 4 * world, case["Hk_per_rank"] * world, 32 * world, 16
        q, k, v = (torch.from_numpy(x) for x in synth.qkv(7, B, H, N, N, d, "bfloat16", 0.5))
        k, v = k[:, :Hk].contiguous(), v[:, :Hk].contiguous()
        slopes = torch.from_numpy(synth.alibi_slopes(H)) if case["alibi"] else None
        C = N // world
        sl = slice(rank * C, (rank + 1) * C)
        # the two exchanges are inverses of each other
        x = q[:, :, sl].contiguous()
        back = ulysses.heads_to_seq(ulysses.seq_to_heads(x))
        assert torch.equal(back, x)
        assert torch.equal(ulysses.seq_to_heads(x), q[:, rank * 4:(rank + 1) * 4])
        o, lse = ulysses.ulysses_attention_forward(x, k[:, :, sl].contiguous(), v[:, :, sl].contiguous(),
                                                   causal=case["causal"], alibi_slopes=slopes, p_dropout=case["p"],
                                                   seed=9, attend_fn=_oracle_attend)
        want_o, want_lse = _oracle_attend(q, k, v, d ** -0.5, case["causal"], slopes, case["p"], 9, 0)
        err = float((o - want_o[:, :, sl]).abs().max())
        err = max(err, float((lse - want_lse[:, :, sl]).abs().max()))
        out[rank] = err
    except Exception as exc:
        out[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


CASES = [
    dict(B=1, Hk_per_rank=4, causal=True, alibi=False, p=0.0),
    dict(B=2, Hk_per_rank=1, causal=True, alibi=True, p=0.0),    # grouped-query K/V, ALiBi
    dict(B=2, Hk_per_rank=4, causal=False, alibi=False, p=0.25),  # dropout: masks keyed on global heads
]


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", CASES)
def test_ulysses_equals_single_device(world, case):
    port = 31500 + (os.getpid() * 5 + world * 11 + CASES.index(case)) % 2000
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, case, out), nprocs=world, join=True)
    res = dict(out)
    assert len(res) == world
    for r, e in res.items():
        assert isinstance(e, float) and e == 0.0, (r, e)
