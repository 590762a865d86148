"""Sequence-sharded attention on real GPUs (the K/V ring and the head all-to-all): 2 (or 4)
NCCL ranks against the single-GPU result.  Skipped when the box has one GPU; NVLS is
switched off for the test processes and a rank only ever leaves between steps."""
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


def _a2a_worker(rank, world, port, out):
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
        from flash_attn_b200 import ulysses
        import synth
        # grouped-query K/V, ALiBi and dropout: the mask is keyed on global heads, so the sharded
        # run must reproduce the single-GPU run of the same seed
        B, H, Hk, N, d = 2, 4 * world, world, 512 * world, 128
        q, k, v = (torch.from_numpy(x).bfloat16().cuda() for x in synth.qkv(10, B, H, N, N, d, "bfloat16", 0.5))
        k, v = k[:, :Hk].contiguous(), v[:, :Hk].contiguous()
        slopes = torch.from_numpy(synth.alibi_slopes(H)).cuda()
        C = N // world
        sl = slice(rank * C, (rank + 1) * C)
        o, lse = ulysses.ulysses_attention_forward(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(),
                                                   v[:, :, sl].contiguous(), causal=True, alibi_slopes=slopes,
                                                   p_dropout=0.1, seed=77)
        want_o, want_lse = fa.flash_attn_forward(q, k, v, causal=True, alibi_slopes=slopes, p_dropout=0.1, seed=77)
        torch.cuda.synchronize()
        out[rank] = ((o.float() - want_o[:, :, sl].float()).abs().max().item(),
                     (lse - want_lse[:, :, sl]).abs().max().item())
    except Exception as exc:
        out[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_head_all_to_all_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_a2a_worker, args=(world, 29950 + os.getpid() % 200, out), nprocs=world, join=True)
    for r in range(world):
        assert isinstance(out[r], tuple), out[r]
        # the same kernel on the same rows with the same mask: identical up to the summation order of
        # nothing at all (whole sequences per head), so the results are equal
        assert out[r][0] == 0.0 and out[r][1] == 0.0, out[r]


@pytest.mark.parametrize("world", [4, 8])
def test_ring_schedule_on_one_gpu_against_the_oracle(world):
    # every rank's loop of the ring on ONE device: all shards resident, a local transport hands over the
    # buffers the ring would deliver, the real forward launches with global positions and the merge in
    # their epilogue.  Checked against the CPU oracle at the chunk edges, not against the GPU kernel.
    import numpy as np
    import gpu_util
    import synth
    from flash_attn_b200 import ring
    B, H, d, C = 1, 2, 128, 384  # chunks of three tiles
    N = 2 * world * C
    q, k, v = (torch.from_numpy(x).bfloat16().cuda() for x in synth.qkv(11, B, H, N, N, d, "bfloat16", 0.5))
    kv_of_rank = [ring.pack_kv(ring.shard_sequence(k, r, world), ring.shard_sequence(v, r, world)) for r in range(world)]
    o = torch.empty_like(q)
    lse = torch.empty((B, H, N), device="cuda", dtype=torch.float32)
    for r in range(world):
        ql, kl, vl = (ring.shard_sequence(x, r, world) for x in (q, k, v))
        o_r, lse_r = ring.ring_attention_forward(ql, kl, vl, causal=True, transport=ring.LocalTransport(kv_of_rank, r, world))
        for i, c in enumerate(ring.zigzag_chunks(r, world)):
            o[:, :, c * C:(c + 1) * C] = o_r[i]
            lse[:, :, c * C:(c + 1) * C] = lse_r[i]
    torch.cuda.synchronize()
    rng = np.random.default_rng(world)
    edges = [c * C + off for c in range(2 * world) for off in (0, 1, 127, 128, C - 1)]
    res = gpu_util.check_sampled_units(q, k, v, o, lse, [0, 1], lambda u: edges + list(rng.integers(0, N, 64)),
                                       d ** -0.5, causal=True)
    gpu_util.assert_close(res, f"ring schedule, {world} ranks on one GPU")


def test_ring_with_window_and_alibi_on_one_gpu():
    import numpy as np
    import gpu_util
    import synth
    from flash_attn_b200 import ring
    world, B, H, d, C = 4, 1, 4, 128, 256
    N = 2 * world * C
    q, k, v = (torch.from_numpy(x).bfloat16().cuda() for x in synth.qkv(12, B, H, N, N, d, "bfloat16", 0.5))
    slopes = synth.alibi_slopes(H)
    kv_of_rank = [ring.pack_kv(ring.shard_sequence(k, r, world), ring.shard_sequence(v, r, world)) for r in range(world)]
    o = torch.empty_like(q)
    lse = torch.empty((B, H, N), device="cuda", dtype=torch.float32)
    for r in range(world):
        ql, kl, vl = (ring.shard_sequence(x, r, world) for x in (q, k, v))
        o_r, lse_r = ring.ring_attention_forward(ql, kl, vl, causal=True, window=(300, 0),
                                                 alibi_slopes=torch.from_numpy(slopes).cuda(),
                                                 transport=ring.LocalTransport(kv_of_rank, r, world))
        for i, c in enumerate(ring.zigzag_chunks(r, world)):
            o[:, :, c * C:(c + 1) * C] = o_r[i]
            lse[:, :, c * C:(c + 1) * C] = lse_r[i]
    torch.cuda.synchronize()
    rng = np.random.default_rng(2)
    res = gpu_util.check_sampled_units(q, k, v, o, lse, range(H), lambda u: [0, 255, 256, 300, 301, N - 1] + list(rng.integers(0, N, 64)),
                                       d ** -0.5, causal=True, window=(300, 0), slopes=slopes)
    gpu_util.assert_close(res, "ring with window and ALiBi")


def test_c_abi_ring_with_one_rank_matches_the_oracle():
    # fa_ring_fwd with world = 1: both chunks of the sequence on this GPU, no exchange
    import numpy as np
    import gpu_util
    import synth
    from flash_attn_b200 import ring
    B, H, d, C = 1, 2, 128, 384
    N = 2 * C
    q, k, v = (torch.from_numpy(x).bfloat16().cuda() for x in synth.qkv(13, B, H, N, N, d, "bfloat16", 0.5))
    ql, kl, vl = (ring.shard_sequence(x, 0, 1) for x in (q, k, v))
    o_l, lse_l = ring.ring_attention_forward_c(ql, kl, vl, None, 0, 1, causal=True)
    torch.cuda.synchronize()
    o = torch.cat(o_l, dim=2)
    lse = torch.cat(lse_l, dim=2)
    rng = np.random.default_rng(1)
    res = gpu_util.check_sampled_units(q, k, v, o, lse, [0, 1], lambda u: [0, 127, 128, C - 1, C, N - 1] + list(rng.integers(0, N, 64)),
                                       d ** -0.5, causal=True)
    gpu_util.assert_close(res, "fa_ring_fwd, one rank")


def _c_ring_worker(rank, world, port, out):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from datetime import timedelta
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=timedelta(seconds=60),
                            device_id=torch.device("cuda", rank))
    comm = None
    try:
        from flash_attn_b200 import ring
        import synth
        B, H, N, d = 1, 4, 1024 * world, 128
        q, k, v = (torch.from_numpy(x).bfloat16().cuda() for x in synth.qkv(9, B, H, N, N, d, "bfloat16", 0.5))
        ql, kl, vl = (ring.shard_sequence(x, rank, world) for x in (q, k, v))
        comm = ring.create_ring_comm()
        o_c, lse_c = ring.ring_attention_forward_c(ql, kl, vl, comm, rank, world, causal=True)
        o_c2, lse_c2 = ring.ring_attention_forward_c(ql, kl, vl, comm, rank, world, causal=True)  # buffers reused
        o_py, lse_py = ring.ring_attention_forward(ql, kl, vl, causal=True)
        torch.cuda.synchronize()
        # the same launches in the same order on the same data: equal bit for bit
        same = all(torch.equal(a, b) for a, b in zip(o_c + lse_c + o_c2 + lse_c2, o_py + lse_py + o_py + lse_py))
        out[rank] = bool(same)
    except Exception as exc:
        out[rank] = repr(exc)
    finally:
        if comm is not None:
            from flash_attn_b200 import ring
            ring.destroy_ring_comm(comm)
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_c_abi_ring_equals_the_python_ring(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_c_ring_worker, args=(world, 29300 + os.getpid() % 200, out), nprocs=world, join=True)
    for r in range(world):
        assert out[r] is True, out[r]
