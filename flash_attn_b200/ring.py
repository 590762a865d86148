"""Sequence-sharded (ring) attention: the host side of the path on torch tensors.

The reference has no multi-GPU path; its softmax couples key blocks only through
the per-row (max, sum) pair that forward_kernel_splitkv_combine merges
(src/flash_forward_splitkv.h:359-397).  The same algebra lets a sequence be
sharded across ranks: every rank keeps its query rows and output, the K/V shards
travel around a ring (send to rank+1, receive from rank-1; NCCL send/recv over
NVLink on GPUs), and every visiting block is one launch of the ordinary forward
kernel with global positions that merges its result into the rank's running fp32
(O, LSE) pair in its own epilogue (fa_fwd_params.accum_o); the launch of a query
chunk's last block also writes the 16-bit output.  No merge or cast pass runs.

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


def block_visible(a, b, chunk, causal, window):
    """Can any query of chunk `a` attend to any key of chunk `b`?  (Blocks that cannot are not launched.)"""
    q_lo, q_hi = a * chunk, (a + 1) * chunk - 1
    k_lo, k_hi = b * chunk, (b + 1) * chunk - 1
    if (causal or window[1] == 0) and k_lo > q_hi:
        return False
    if window[1] > 0 and k_lo > q_hi + window[1]:
        return False
    if window[0] >= 0 and k_hi < q_lo - window[0]:
        return False
    return True


def ring_schedule(rank, world, chunk, causal=True, window=(-1, -1)):
    """Launches of one rank, in execution order: dicts with step (ring step), qi / ki (which of the
    rank's query chunks, which of the visiting rank's key chunks), a / b (their global chunk
    indices), first / final (the query chunk's first / last launch)."""
    out = []
    for step in range(world):
        src = (rank - step) % world
        for qi, a in enumerate(zigzag_chunks(rank, world)):
            for ki, b in enumerate(zigzag_chunks(src, world)):
                if block_visible(a, b, chunk, causal, window):
                    out.append(dict(step=step, qi=qi, ki=ki, a=a, b=b, first=False, final=False))
    for qi in range(2):
        mine = [x for x in out if x["qi"] == qi]
        if mine:
            mine[0]["first"] = True
            mine[-1]["final"] = True
    return out


def cuda_block(q, k, v, scale, causal, q_pos0, k_pos0, acc, first, final, out, window, alibi_slopes):
    """One visiting block on the GPU: forward launch that merges into `acc` = (o_acc, lse_acc)."""
    return api.flash_attn_forward(q, k, v, softmax_scale=scale, causal=causal, window=window, alibi_slopes=alibi_slopes,
                                  q_pos0=q_pos0, k_pos0=k_pos0, accum=acc, accum_first=first, accum_final=final, out=out)


class DistTransport:
    """K/V exchange with the ring neighbours over torch.distributed (NCCL on GPUs, gloo on CPU ranks)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nxt, self.prv = (self.rank + 1) % self.world, (self.rank - 1) % self.world
        if group is not None and self.world > 1:
            self.nxt, self.prv = dist.get_global_rank(group, self.nxt), dist.get_global_rank(group, self.prv)

    def exchange(self, step, send_buf, recv_buf):
        """Posts the send of this step's K/V to rank+1 and the receive of the next step's from rank-1;
        returns the requests to wait on before recv_buf is read."""
        ops = [dist.P2POp(dist.isend, send_buf, self.nxt, self.group), dist.P2POp(dist.irecv, recv_buf, self.prv, self.group)]
        return dist.batch_isend_irecv(ops)


class LocalTransport:
    """All ranks' K/V on one device: the 'receive' of step s+1 copies the buffer of rank r-s-1.  Runs one
    rank's schedule exactly as the ring does, without a second GPU (tests, single-GPU runs)."""

    def __init__(self, kv_of_rank, rank, world):
        self.kv_of_rank, self.rank, self.world = kv_of_rank, rank, world

    def exchange(self, step, send_buf, recv_buf):
        recv_buf.copy_(self.kv_of_rank[(self.rank - step - 1) % self.world])
        return []


def pack_kv(k, v):
    """The K/V message of a rank: one contiguous buffer [2 (k|v), 2 (chunk), B, H, C, d]."""
    return torch.stack([torch.stack(list(k)), torch.stack(list(v))]).contiguous()


_buffers = {}


def _scratch(key, make):
    """Receive buffer and running accumulators are kept between calls of the same geometry."""
    if key not in _buffers:
        if len(_buffers) > 8:
            _buffers.clear()
        _buffers[key] = make()
    return _buffers[key]


def ring_attention_forward(q, k, v, group=None, softmax_scale=None, causal=True, window=(-1, -1), alibi_slopes=None,
                           p_dropout=0.0, block_fn=None, transport=None, out_dtype=None):
    """Attention over a sequence sharded in zig-zag chunks across `group`.

    q, k, v: lists of two [B,H,C,d] tensors (this rank's chunks, see shard_sequence).
    Returns (o, lse): lists of two tensors, [B,H,C,d] in out_dtype (default q dtype)
    and [B,H,C] fp32.  `window` and `alibi_slopes` act on global positions, as in one
    unsharded launch.  Dropout is refused: the reference's dropout streams are keyed on
    the tile grid of one whole-sequence launch, which a sharded launch does not have.
    `block_fn` (default: the CUDA kernel) runs one visiting block; the CPU tests
    substitute the oracle.  `transport` defaults to the process group.
    """
    if p_dropout:
        raise ValueError("ring attention does not support dropout: the reference's dropout streams are keyed on "
                         "the tile grid of a whole-sequence launch (use the head all-to-all path)")
    block_fn = block_fn or cuda_block
    transport = transport or DistTransport(group)
    world, rank = transport.world, transport.rank
    B, H, C, d = q[0].shape
    scale = float(softmax_scale) if softmax_scale is not None else d ** -0.5
    dev = q[0].device
    out_dtype = out_dtype or q[0].dtype
    key = (dev, B, H, C, d, q[0].dtype, k[0].shape[1])
    acc = _scratch(("acc",) + key, lambda: [(torch.empty((B, H, C, d), device=dev, dtype=torch.float32),
                                             torch.empty((B, H, C), device=dev, dtype=torch.float32)) for _ in range(2)])
    kv = [pack_kv(k, v), None]
    if world > 1:
        kv[1] = _scratch(("kv",) + key, lambda: torch.empty_like(kv[0]))
    out = [torch.empty((B, H, C, d), device=dev, dtype=out_dtype) for _ in range(2)]
    lse = [None, None]
    launches = ring_schedule(rank, world, C, causal, window)
    for step in range(world):
        cur = kv[step % 2]
        reqs = []
        if step + 1 < world:
            # post the exchange first: it runs on the communication stream while the kernels below compute
            reqs = transport.exchange(step, cur, kv[(step + 1) % 2])
        for x in (l for l in launches if l["step"] == step):
            # blocks that lie wholly before the query chunk need no causal test
            diag = causal and x["b"] == x["a"]
            res = block_fn(q[x["qi"]], cur[0, x["ki"]], cur[1, x["ki"]], scale, diag, x["a"] * C, x["b"] * C,
                           acc[x["qi"]], x["first"], x["final"], out[x["qi"]] if x["final"] else None, window, alibi_slopes)
            if x["final"]:
                lse[x["qi"]] = res[1]
        for r in reqs:
            r.wait()
    for qi in range(2):
        if lse[qi] is None:  # no key block was visible to this query chunk
            out[qi].zero_()
            lse[qi] = torch.full((B, H, C), float("-inf"), device=dev, dtype=torch.float32)
    return out, lse


# ------------------------------------------------------------------ the same ring through the C ABI

def create_ring_comm(group=None):
    """NCCL communicator for fa_ring_fwd, one per rank: rank 0 asks the library for an id and the
    process group hands it round.  Returns an opaque handle (destroy_ring_comm frees it)."""
    import ctypes
    from . import _lib
    L = _lib.load()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world == 1:
        return None
    dev = torch.device("cuda", torch.cuda.current_device())
    ident = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = (ctypes.c_ubyte * 128)()
        _lib.check(L.fa_ring_unique_id(buf, 128), "fa_ring_unique_id")
        ident = torch.tensor(list(buf), dtype=torch.uint8)
    ident = ident.to(dev) if dist.get_backend(group) == "nccl" else ident
    dist.broadcast(ident, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    raw = bytes(ident.cpu().tolist())
    comm = ctypes.c_void_p()
    with torch.cuda.device(dev):
        _lib.check(L.fa_ring_comm_create(ctypes.byref(comm), world, rank, raw, 128), "fa_ring_comm_create")
    return comm


def destroy_ring_comm(comm):
    from . import _lib
    if comm is not None:
        _lib.load().fa_ring_comm_destroy(comm)


_comm_streams = {}


def ring_attention_forward_c(q, k, v, comm, rank, world, softmax_scale=None, causal=True, window=(-1, -1),
                             alibi_slopes=None):
    """ring_attention_forward with the whole schedule -- exchange, launches, stream ordering -- inside
    the library (fa_ring_fwd): torch only owns the memory.  q, k, v as in ring_attention_forward; `comm`
    from create_ring_comm (None when world == 1)."""
    import ctypes
    from . import _lib
    L = _lib.load()
    B, H, C, d = q[0].shape
    Hk = k[0].shape[1]
    dev = q[0].device
    p = _lib.RingParams()
    out = [torch.empty_like(q[0]) for _ in range(2)]
    lse = [torch.empty((B, H, C), device=dev, dtype=torch.float32) for _ in range(2)]
    key = (dev, B, H, Hk, C, d, q[0].dtype)
    acc = _scratch(("c_acc",) + key, lambda: [(torch.empty((B, H, C, d), device=dev, dtype=torch.float32),
                                               torch.empty((B, H, C), device=dev, dtype=torch.float32)) for _ in range(2)])
    for i in range(2):
        for t in (q[i], k[i], v[i]):
            if not t.is_contiguous():
                raise ValueError("chunks must be contiguous")
        p.q[i], p.k[i], p.v[i] = q[i].data_ptr(), k[i].data_ptr(), v[i].data_ptr()
        p.o[i], p.lse[i] = out[i].data_ptr(), lse[i].data_ptr()
        p.accum_o[i], p.accum_lse[i] = acc[i][0].data_ptr(), acc[i][1].data_ptr()
    p.dtype = api._DT[q[0].dtype]
    p.batch, p.heads, p.heads_k, p.chunk_rows, p.head_dim = B, H, Hk, C, d
    p.softmax_scale = float(softmax_scale) if softmax_scale is not None else d ** -0.5
    p.is_causal, p.window_left, p.window_right = int(bool(causal)), int(window[0]), int(window[1])
    slopes = None
    if alibi_slopes is not None:
        slopes = alibi_slopes.to(device=dev, dtype=torch.float32).contiguous()
        p.alibi_slopes = slopes.data_ptr()
    p.rank, p.world = rank, world
    p.comm = comm
    nbytes = L.fa_ring_message_bytes(ctypes.byref(p))
    msgs = _scratch(("c_msg",) + key, lambda: [torch.empty(nbytes, device=dev, dtype=torch.uint8) for _ in range(2)])
    p.message[0], p.message[1] = msgs[0].data_ptr(), msgs[1].data_ptr()
    if dev not in _comm_streams:
        # highest priority: the exchange's few CTAs are placed as soon as an SM frees up instead of
        # queueing behind the attention launch they overlap
        _comm_streams[dev] = torch.cuda.Stream(device=dev, priority=-1)
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream(dev)
        p.compute_stream = cur.cuda_stream
        p.comm_stream = _comm_streams[dev].cuda_stream
        _lib.check(L.fa_ring_fwd(ctypes.byref(p)), "fa_ring_fwd")
    return out, lse
