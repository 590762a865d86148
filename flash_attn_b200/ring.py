"""Sequence-sharded (ring) causal attention over torch.distributed.

The reference has no multi-GPU path; its softmax couples key blocks only through
the per-row (max, sum) pair that forward_kernel_splitkv_combine merges
(src/flash_forward_splitkv.h:359-397).  The same algebra lets a sequence be
sharded across ranks: every rank keeps its query rows and output, the K/V shards
travel around a ring (send to rank+1, receive from rank-1; NCCL send/recv over
NVLink on GPUs), each visiting block contributes a partial (O, LSE) computed by
the ordinary forward kernel with global positions, and partials are merged by LSE.

Layout ("zig-zag"): the sequence is cut into 2*P chunks of C rows; rank r owns
chunks r and 2P-1-r, so with a causal mask every rank has the same amount of
unmasked work.  Tensors are passed per chunk: q, k, v = lists of two contiguous
[B, H, C, d] tensors.
"""
import torch
import torch.distributed as dist

from . import api


def zigzag_chunks(rank, world):
    """Global chunk indices owned by `rank` (chunks are numbered 0 .. 2*world-1)."""
    return (rank, 2 * world - 1 - rank)


def shard_sequence(x, rank, world):
    """[B,H,N,d] -> the two contiguous [B,H,C,d] chunks `rank` owns (N divisible by 2*world)."""
    n = x.shape[2]
    if n % (2 * world) != 0:
        raise ValueError("sequence length must be a multiple of 2 * world_size")
    c = n // (2 * world)
    return [x[:, :, i * c:(i + 1) * c].contiguous() for i in zigzag_chunks(rank, world)]


def unit_slice(units, rank, world):
    """Contiguous slice [lo, hi) of the flattened batch*heads units owned by `rank`
    (the communication-free sharding used for everything but the ring)."""
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _cuda_attend(q, k, v, scale, causal, q_pos0, k_pos0):
    return api.flash_attn_forward(q, k, v, softmax_scale=scale, causal=causal, q_pos0=q_pos0, k_pos0=k_pos0,
                                  out_dtype=torch.float32)


def _cuda_merge(o_acc, lse_acc, o_part, lse_part):
    api.merge_partial(o_acc, lse_acc, o_part, lse_part)


def ring_attention_forward(q, k, v, group=None, softmax_scale=None, causal=True, attend_fn=None, merge_fn=None,
                           out_dtype=None):
    """Attention over a sequence sharded in zig-zag chunks across `group`.

    q, k, v: lists of two [B,H,C,d] tensors (this rank's chunks, see shard_sequence).
    Returns (o, lse): lists of two tensors, [B,H,C,d] in out_dtype (default q dtype)
    and [B,H,C] fp32.  `attend_fn(q, k, v, scale, causal, q_pos0, k_pos0) -> (o fp32,
    lse)` and `merge_fn(o_acc, lse_acc, o_part, lse_part)` default to the CUDA
    kernels; the CPU tests substitute the oracle.
    """
    attend_fn = attend_fn or _cuda_attend
    merge_fn = merge_fn or _cuda_merge
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    B, H, C, d = q[0].shape
    scale = float(softmax_scale) if softmax_scale is not None else d ** -0.5
    my_chunks = zigzag_chunks(rank, world)
    dev = q[0].device

    o_acc = [torch.zeros((B, H, C, d), device=dev, dtype=torch.float32) for _ in range(2)]
    lse_acc = [torch.full((B, H, C), float("-inf"), device=dev, dtype=torch.float32) for _ in range(2)]

    # K/V travel as one contiguous buffer [2 (k|v), 2 (chunk), B, H, C, d], double-buffered
    kv = [torch.stack([torch.stack(list(k)), torch.stack(list(v))]).contiguous(), None]
    if world > 1:
        kv[1] = torch.empty_like(kv[0])
    nxt = (rank + 1) % world
    prv = (rank - 1) % world
    if group is not None and world > 1:
        nxt, prv = dist.get_global_rank(group, nxt), dist.get_global_rank(group, prv)

    for step in range(world):
        cur = kv[step % 2]
        reqs = []
        if step + 1 < world:
            # post the exchange first: it runs on the communication stream while the kernels below compute
            ops = [dist.P2POp(dist.isend, cur, nxt, group), dist.P2POp(dist.irecv, kv[(step + 1) % 2], prv, group)]
            reqs = dist.batch_isend_irecv(ops)
        src = (rank - step) % world
        src_chunks = zigzag_chunks(src, world)
        for qi, a in enumerate(my_chunks):
            for ki, b in enumerate(src_chunks):
                if causal and b > a:
                    continue  # every key of the block lies after every query of the chunk
                o_part, lse_part = attend_fn(q[qi], cur[0, ki], cur[1, ki], scale, causal and b == a, a * C, b * C)
                merge_fn(o_acc[qi], lse_acc[qi], o_part, lse_part)
        for r in reqs:
            r.wait()

    out_dtype = out_dtype or q[0].dtype
    if out_dtype == torch.float32:
        return o_acc, lse_acc
    if o_acc[0].is_cuda:
        return [api.cast_output(o, out_dtype) for o in o_acc], lse_acc
    return [o.to(out_dtype) for o in o_acc], lse_acc
