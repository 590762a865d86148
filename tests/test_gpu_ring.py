"""Sequence ring on real GPUs: 2 (or 4) NCCL ranks against the single-GPU result.
Skipped when the box has one GPU; NVLS is switched off for the test processes and a
rank only ever leaves between steps."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, out):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from datetime import timedelta
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=timedelta(seconds=60),
                            device_id=torch.device("cuda", rank))
    try:
        import flash_attn_b200 as fa
        from flash_attn_b200 import ring
        import synth
        B, H, N, d = 1, 4, 1024 * world, 128
        q, k, v = (torch.from_numpy(x).bfloat16().cuda() for x in synth.qkv(9, B, H, N, N, d, "bfloat16", 0.5))
        ql, kl, vl = (ring.shard_sequence(x, rank, world) for x in (q, k, v))
        o, lse = ring.ring_attention_forward(ql, kl, vl, causal=True)
        want_o, want_lse = fa.flash_attn_forward(q, k, v, causal=True)
        torch.cuda.synchronize()
        C = N // (2 * world)
        err = lerr = 0.0
        for i, c in enumerate(ring.zigzag_chunks(rank, world)):
            err = max(err, (o[i].float() - want_o[:, :, c * C:(c + 1) * C].float()).abs().max().item())
            lerr = max(lerr, (lse[i] - want_lse[:, :, c * C:(c + 1) * C]).abs().max().item())
        out[rank] = (err, lerr)
    except Exception as exc:
        out[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ring_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, 29700 + os.getpid() % 200, out), nprocs=world, join=True)
    for r in range(world):
        assert isinstance(out[r], tuple), out[r]
        assert out[r][0] <= 8e-3 and out[r][1] <= 1e-3, out[r]
