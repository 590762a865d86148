"""Host logic of the multi-GPU paths on CPU ranks (gloo, world_size 2 and 4): the
ring schedule, the zig-zag layout and the LSE merge give the single-device result;
a rank that fails is reported, not waited for forever.  The kernels are replaced by
the CPU oracle here; the GPU tests run the same module with the CUDA kernels."""
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


def oracle_block(q, k, v, scale, causal, q_pos0, k_pos0, acc, first, final, out, window, alibi_slopes):
    """One visiting block with the CPU oracle as the kernel: partial (O, LSE) of the block, merged into the
    running pair with the combine algebra (src/flash_forward_splitkv.h:359-397 in log-sum-exp form)."""
    o_part, lse_part = oracle_lib.forward(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale, causal=causal,
                                          window=window, alibi_slopes=None if alibi_slopes is None else alibi_slopes.numpy(),
                                          q_pos0=q_pos0, k_pos0=k_pos0, num_threads=1)
    o_part, lse_part = torch.from_numpy(o_part), torch.from_numpy(lse_part)
    o_acc, lse_acc = acc
    if first:
        o_acc.copy_(o_part)
        lse_acc.copy_(lse_part)
    else:
        new = torch.logaddexp(lse_acc, lse_part)
        wa = torch.where(torch.isneginf(new), torch.zeros_like(new), torch.exp(lse_acc - new))
        wb = torch.where(torch.isneginf(new), torch.zeros_like(new), torch.exp(lse_part - new))
        o_acc.mul_(wa.unsqueeze(-1)).add_(o_part * wb.unsqueeze(-1))
        lse_acc.copy_(new)
    if final:
        out.copy_(o_acc.to(out.dtype))
        return out, lse_acc.clone()
    return None, None


def _worker(rank, world, port, causal, fail_rank, out):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from datetime import timedelta
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    try:
        from flash_attn_b200 import ring
        B, H, N, d = 1, 2, 64 * world, 16
        q, k, v = (torch.from_numpy(x) for x in synth.qkv(5, B, H, N, N, d, "bfloat16", 0.5))
        if rank == fail_rank:
            raise RuntimeError("injected failure on the host")
        ql, kl, vl = (ring.shard_sequence(x, rank, world) for x in (q, k, v))
        o, lse = ring.ring_attention_forward(ql, kl, vl, causal=causal, block_fn=oracle_block, out_dtype=torch.float32)
        want_o, want_lse = oracle_lib.forward(q.numpy(), k.numpy(), v.numpy(), d ** -0.5, causal=causal, num_threads=1)
        C = N // (2 * world)
        err = 0.0
        for i, c in enumerate(ring.zigzag_chunks(rank, world)):
            err = max(err, float(np.abs(o[i].numpy() - want_o[:, :, c * C:(c + 1) * C]).max()))
            err = max(err, float(np.abs(lse[i].numpy() - want_lse[:, :, c * C:(c + 1) * C]).max()))
        out[rank] = err
    except Exception as exc:  # reported to the parent instead of hanging the group
        out[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


def _run(world, causal, fail_rank=-1):
    port = 29500 + (os.getpid() * 7 + world * 3 + int(causal)) % 2000
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, causal, fail_rank, out), nprocs=world, join=True)
    return dict(out)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal", [True, False])
def test_ring_equals_single_device(world, causal):
    res = _run(world, causal)
    assert len(res) == world
    for r, e in res.items():
        assert isinstance(e, float) and e < 2e-5, (r, e)


def test_a_failing_rank_is_reported_and_the_others_time_out():
    # rank 1 raises before its first send: the other rank's receive ends with an error
    # (process-group timeout), not a hang
    res = _run(2, True, fail_rank=1)
    assert "injected failure" in res[1]
    assert isinstance(res[0], str)


def test_unit_sharding_and_zigzag_layout():
    from flash_attn_b200 import ring
    for units, world in ((128, 8), (2048, 8), (10, 4), (3, 8)):
        slices = [ring.unit_slice(units, r, world) for r in range(world)]
        assert slices[0][0] == 0 and slices[-1][1] == units
        assert all(a[1] == b[0] for a, b in zip(slices, slices[1:]))
        assert max(h - l for l, h in slices) - min(h - l for l, h in slices) <= 1
    world = 4
    owned = sorted(c for r in range(world) for c in ring.zigzag_chunks(r, world))
    assert owned == list(range(2 * world))
    # causal work (number of key chunks at or before each query chunk) is the same on every rank
    work = [sum(c + 1 for c in ring.zigzag_chunks(r, world)) for r in range(world)]
    assert len(set(work)) == 1
    x = torch.arange(2 * 1 * 16 * 3, dtype=torch.float32).reshape(2, 1, 16, 3)
    a, b = ring.shard_sequence(x, 1, 4)
    assert torch.equal(a, x[:, :, 2:4]) and torch.equal(b, x[:, :, 12:14])


@pytest.mark.parametrize("world", [3, 8])
@pytest.mark.parametrize("opts", [dict(causal=True), dict(causal=False), dict(causal=True, window=(40, 0), alibi=True),
                                  dict(causal=False, window=(24, 9))])
def test_schedule_of_every_rank_in_one_process(world, opts):
    # the ranks' loops run one after the other with a transport that hands over the buffer the ring
    # would have delivered: same schedule, no process group
    from flash_attn_b200 import ring
    B, H, d = 1, 2, 16
    C = 16
    N = 2 * world * C
    q, k, v = (torch.from_numpy(x) for x in synth.qkv(6, B, H, N, N, d, "bfloat16", 0.5))
    window = opts.get("window", (-1, -1))
    slopes = torch.from_numpy(synth.alibi_slopes(H)) if opts.get("alibi") else None
    want_o, want_lse = oracle_lib.forward(q.numpy(), k.numpy(), v.numpy(), d ** -0.5, causal=opts["causal"], window=window,
                                          alibi_slopes=None if slopes is None else slopes.numpy(), num_threads=1)
    kv_of_rank = [ring.pack_kv(ring.shard_sequence(k, r, world), ring.shard_sequence(v, r, world)) for r in range(world)]
    for r in range(world):
        ql, kl, vl = (ring.shard_sequence(x, r, world) for x in (q, k, v))
        o, lse = ring.ring_attention_forward(ql, kl, vl, causal=opts["causal"], window=window, alibi_slopes=slopes,
                                             block_fn=oracle_block, transport=ring.LocalTransport(kv_of_rank, r, world),
                                             out_dtype=torch.float32)
        for i, c in enumerate(ring.zigzag_chunks(r, world)):
            sl = slice(c * C, (c + 1) * C)
            assert np.abs(o[i].numpy() - want_o[:, :, sl]).max() < 2e-5
            got, want = lse[i].numpy(), want_lse[:, :, sl]
            assert np.array_equal(np.isneginf(got), np.isneginf(want))
            fin = np.isfinite(want)
            assert np.abs(got[fin] - want[fin]).max() < 2e-5


def test_ring_schedule_marks_first_and_last_launch_of_each_query_chunk():
    from flash_attn_b200 import ring
    for world in (1, 2, 4, 8):
        for rank in range(world):
            sch = ring.ring_schedule(rank, world, 128, causal=True)
            a0, a1 = ring.zigzag_chunks(rank, world)
            # causal: chunk a sees chunks 0..a, each exactly once over the ring
            assert sorted(x["b"] for x in sch if x["qi"] == 0) == list(range(a0 + 1))
            assert sorted(x["b"] for x in sch if x["qi"] == 1) == list(range(a1 + 1))
            for qi in range(2):
                mine = [x for x in sch if x["qi"] == qi]
                assert [x["first"] for x in mine] == [True] + [False] * (len(mine) - 1)
                assert [x["final"] for x in mine] == [False] * (len(mine) - 1) + [True]
    with pytest.raises(ValueError):
        ring.ring_attention_forward([torch.zeros(1, 1, 8, 8)] * 2, [torch.zeros(1, 1, 8, 8)] * 2,
                                    [torch.zeros(1, 1, 8, 8)] * 2, p_dropout=0.1)
