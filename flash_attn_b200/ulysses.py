"""Head-sharded (all-to-all) attention over torch.distributed: the alternative to the ring
for a sequence that is sharded across ranks.

Every (batch, head) unit of the reference is independent (grid y/z, src/main.cu:142), so
instead of moving K/V blocks around a ring the ranks can trade layouts: one all-to-all turns
"my slice of the sequence, all heads" into "the whole sequence, my slice of the heads", the
ordinary forward kernel runs once on whole sequences (no partial results, no LSE merge), and
a second all-to-all brings O and LSE back to the sequence-sharded layout.  Each rank sends
and receives (P-1)/P of its Q, K, V and O once, over NCCL (NVLink / NVSwitch) on GPUs.

Layout: rank r owns the contiguous rows [r*C, (r+1)*C) of the sequence, C = N / P, as
[B, H, C, d] tensors; H (and the K/V head count with grouped-query attention) must be a
multiple of P.
"""
import torch
import torch.distributed as dist

from . import api


def _world(group):
    if not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class _Exchange:
    """One all-to-all in flight: `finish()` waits for it (on the current stream for NCCL) and
    returns the tensor in its new layout.  Send and receive buffers stay referenced until then."""

    def __init__(self, send, group, rebuild):
        self.send = send
        self.recv = torch.empty_like(send)
        self.rebuild = rebuild
        self.work = dist.all_to_all_single(self.recv, send, group=group, async_op=True)

    def finish(self):
        self.work.wait()
        out = self.rebuild(self.recv)
        self.send = None
        return out


class _Ready:
    def __init__(self, x):
        self.x = x

    def finish(self):
        return self.x


def seq_to_heads_start(x, group=None):
    """Starts [B, H, C, ...] (sequence slice, all heads) -> [B, H/P, P*C, ...] (whole sequence, head slice)."""
    world, _ = _world(group)
    if world == 1:
        return _Ready(x)
    B, H, C = x.shape[:3]
    tail = x.shape[3:]
    if H % world != 0:
        raise ValueError("the head count must be a multiple of the group size")
    # block j (heads j*H/P ...) goes to rank j
    send = x.reshape(B, world, H // world, C, *tail).movedim(1, 0).contiguous()
    # recv[j] = rank j's sequence slice of my heads: concatenate along the sequence in rank order
    return _Exchange(send, group, lambda r: r.movedim(0, 2).reshape(B, H // world, world * C, *tail))


def heads_to_seq_start(x, group=None):
    """Starts the inverse exchange: [B, H/P, N, ...] -> [B, H, N/P, ...]."""
    world, _ = _world(group)
    if world == 1:
        return _Ready(x)
    B, Hl, N = x.shape[:3]
    tail = x.shape[3:]
    if N % world != 0:
        raise ValueError("the sequence length must be a multiple of the group size")
    C = N // world
    # sequence slice j goes to rank j
    send = x.reshape(B, Hl, world, C, *tail).movedim(2, 0).contiguous()
    # recv[j] = rank j's heads of my sequence slice: concatenate along the heads in rank order
    return _Exchange(send, group, lambda r: r.movedim(0, 1).reshape(B, world * Hl, C, *tail))


def seq_to_heads(x, group=None):
    return seq_to_heads_start(x, group).finish()


def heads_to_seq(x, group=None):
    return heads_to_seq_start(x, group).finish()


def _cuda_attend(q, k, v, scale, causal, alibi_slopes, p_dropout, seed, unit0):
    return api.flash_attn_forward(q, k, v, softmax_scale=scale, causal=causal, alibi_slopes=alibi_slopes,
                                  p_dropout=p_dropout, seed=seed, unit0=unit0)


def _head_groups(H, Hk, world, want):
    """Largest number of head groups <= want such that every group holds a multiple of
    `world` query heads and K/V heads."""
    for g in range(max(1, want), 0, -1):
        if H % (g * world) == 0 and Hk % (g * world) == 0:
            return g
    raise ValueError("the head counts must be multiples of the group size")


def ulysses_attention_forward(q, k, v, group=None, softmax_scale=None, causal=True, alibi_slopes=None,
                              p_dropout=0.0, seed=0, attend_fn=None, pipeline=4):
    """Attention over a sequence sharded in contiguous slices across `group`.

    q [B,H,C,d], k/v [B,Hk,C,d]: this rank's rows [rank*C, (rank+1)*C).  Returns (o [B,H,C,d]
    in q's dtype, lse [B,H,C] fp32) for the same rows.  `alibi_slopes` is the full fp32 [H]
    vector; dropout streams are keyed on the global (batch, head) index, so the mask does not
    depend on the group size.  The heads are worked on in up to `pipeline` groups: the
    exchange of the next group and the return of the previous one run (on the collective's
    stream) while the kernel works on the current group.  `attend_fn(q, k, v, scale, causal,
    slopes, p, seed, unit0) -> (o, lse)` defaults to the CUDA kernels; the CPU tests
    substitute the oracle.
    """
    attend_fn = attend_fn or _cuda_attend
    world, rank = _world(group)
    B, H, C, d = q.shape
    Hk = k.shape[1]
    scale = float(softmax_scale) if softmax_scale is not None else d ** -0.5
    G = _head_groups(H, Hk, world, pipeline)
    Hg, Hkg = H // G, Hk // G  # heads of one group, before the exchange
    Hl = Hg // world           # query heads of one group on this rank, after it

    def start(g):
        return tuple(seq_to_heads_start(x[:, g * n:(g + 1) * n], group) for x, n in ((q, Hg), (k, Hkg), (v, Hkg)))

    back = []
    nxt = start(0)
    for g in range(G):
        qh, kh, vh = (e.finish() for e in nxt)
        if g + 1 < G:
            nxt = start(g + 1)
        h0 = g * Hg + rank * Hl  # global index of this rank's first head of the group
        slopes = None if alibi_slopes is None else alibi_slopes[h0:h0 + Hl].contiguous()
        if p_dropout > 0.0 and B > 1:
            # the local heads of different batch entries are not contiguous in the global unit
            # numbering b*H + h, which is what keys the dropout streams: one call per batch entry
            outs = [attend_fn(qh[b:b + 1], kh[b:b + 1], vh[b:b + 1], scale, causal, slopes, p_dropout, seed,
                              b * H + h0) for b in range(B)]
            oh = torch.cat([o for o, _ in outs])
            lseh = torch.cat([l for _, l in outs])
        else:
            oh, lseh = attend_fn(qh, kh, vh, scale, causal, slopes, p_dropout, seed, h0)
        back.append((heads_to_seq_start(oh, group), heads_to_seq_start(lseh, group)))
    o = torch.cat([e.finish() for e, _ in back], dim=1)
    lse = torch.cat([e.finish() for _, e in back], dim=1)
    return o, lse
