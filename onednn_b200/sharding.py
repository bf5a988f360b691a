"""Sharding of one matmul across the GPUs of a node (one process per GPU).

Dense problems shard by output columns: rank r holds weights[:, r*N/g:(r+1)*N/g]
with the matching slices of every per-N parameter (weight scales and
zero-points, bias, binary post-op operands); src and per-row parameters are
replicated.  Each rank runs an ordinary matmul on its slice and the dst
slices are assembled with an all-gather (``gather_columns``).

Grouped (MoE) problems shard by experts, E / g per rank, chosen so that the
ranks' work is even (``expert_assignment``: heaviest expert first onto the
least loaded rank that still has room): a rank holds its experts' weights and
the src rows routed to them, concatenated in expert order; the dst row blocks
are assembled with a variable-size all-gather (``gather_rows``) and
``row_map`` says where each row of the unsharded problem lies in them.
"""
import numpy as np

from . import workloads as W


def _cols(data, dt, rows, N, lo, hi):
    """Columns [lo, hi) of a row-major [rows, N] buffer of data type dt."""
    if dt in (W.S4, W.U4):
        assert lo % 2 == 0 and hi % 2 == 0, "int4 column slices must start on a byte"
        return np.ascontiguousarray(data.reshape(rows, N // 2)[:, lo // 2:hi // 2])
    return np.ascontiguousarray(data.reshape(rows, N)[:, lo:hi])


def column_range(N, rank, world, align=16):
    """Near-equal column ranges whose boundaries are multiples of `align`."""
    units = N // align
    assert units * align == N, "N must be a multiple of %d" % align
    lo = (units * rank // world) * align
    hi = (units * (rank + 1) // world) * align
    return lo, hi


def shard_columns(p: W.Problem, rank: int, world: int) -> W.Problem:
    assert p.offsets is None
    lo, hi = column_range(p.N, rank, world)
    n = hi - lo
    wei = W.QTensor(_cols(p.wei.data, p.wei.dt, p.K, p.N, lo, hi), p.wei.dt, (p.K, n))
    bias = p.bias
    if bias is not None and bias.dims[1] == p.N:
        bias = W.QTensor(_cols(bias.data, bias.dt, bias.dims[0], p.N, lo, hi), bias.dt, (bias.dims[0], n))
    quant = {}
    for name, q in p.quant.items():
        per_n = name.startswith(("wei", "dst")) and (q.mask & 2)
        if per_n:
            assert q.groups[1] == 1, "N-grouped parameters are not sharded"
            rows = q.data.size * (2 if q.dt in (W.S4, W.U4) else 1) // p.N
            quant[name] = W.Quant(_cols(q.data, q.dt, rows, p.N, lo, hi), q.dt, q.mask, q.groups)
        else:
            quant[name] = q
    pos = []
    for po in p.post_ops:
        if po.src1 is not None and po.src1.dims[1] == p.N:
            t = po.src1
            pos.append(W.PostOp(po.kind, po.alg, po.alpha, po.beta, po.scale, po.zero_point,
                                W.QTensor(_cols(t.data, t.dt, t.dims[0], p.N, lo, hi), t.dt, (t.dims[0], n))))
        else:
            pos.append(po)
    return W.Problem("%s[n %d:%d]" % (p.name, lo, hi), p.M, n, p.K, p.src, wei, p.dst_dt, bias, quant, pos,
                     p.apply_to_int, p.fpmath)


def expert_range(E, rank, world):
    return E * rank // world, E * (rank + 1) // world


def expert_assignment(rows_per_expert, world):
    """Experts of every rank (sorted), E // world (+1 for the first E % world ranks) each.

    An expert costs its weight stream (the same for every non-empty expert) or
    its rows' arithmetic, whichever is larger: with K x N weights of one byte
    and a tensor rate of about 240 flop per byte of HBM, the two meet near 128
    rows.  Experts go, heaviest first, to the rank with the smallest cost so far
    that still has room (ties: lower rank), which is deterministic."""
    E = len(rows_per_expert)
    cap = [E // world + (1 if r < E % world else 0) for r in range(world)]
    cost = [0 if n == 0 else max(128, int(n)) for n in rows_per_expert]
    order = sorted(range(E), key=lambda e: (-cost[e], e))
    load, own = [0] * world, [[] for _ in range(world)]
    for e in order:
        r = min((r for r in range(world) if len(own[r]) < cap[r]), key=lambda r: (load[r], r))
        own[r].append(e)
        load[r] += cost[e]
    return [sorted(o) for o in own]


def _expert_rows(p):
    ends = p.offsets.astype(np.int64)
    begins = np.concatenate([[0], ends[:-1]])
    return begins, ends


def row_map(p: W.Problem, world: int):
    """(rank, row inside that rank's block) of every row of the unsharded grouped problem."""
    begins, ends = _expert_rows(p)
    own = expert_assignment((ends - begins).tolist(), world)
    rank_of = np.zeros(p.M, np.int64)
    local = np.zeros(p.M, np.int64)
    for r, experts in enumerate(own):
        at = 0
        for e in experts:
            n = int(ends[e] - begins[e])
            rank_of[begins[e]:ends[e]] = r
            local[begins[e]:ends[e]] = at + np.arange(n)
            at += n
    return rank_of, local


def shard_experts(p: W.Problem, rank: int, world: int) -> W.Problem:
    assert p.offsets is not None
    begins, ends = _expert_rows(p)
    experts = expert_assignment((ends - begins).tolist(), world)[rank]
    src2d = p.src.data.reshape(p.M, p.K)
    parts = [src2d[begins[e]:ends[e]] for e in experts]
    m = int(sum(len(x) for x in parts))
    src = W.QTensor(np.ascontiguousarray(np.concatenate(parts, axis=0)) if parts else src2d[:0].copy(), p.src.dt, (m, p.K))
    wei = W.QTensor(np.ascontiguousarray(p.wei.data[experts]), p.wei.dt, (len(experts), p.K, p.N))
    quant = {}
    for name, q in p.quant.items():
        assert name.startswith("wei") and (q.mask & 1), "only per-expert weight parameters are sharded"
        quant[name] = W.Quant(np.ascontiguousarray(q.data[experts]), q.dt, q.mask, q.groups)
    bias = p.bias
    if bias is not None:  # one row per expert
        bias = W.QTensor(np.ascontiguousarray(bias.data.reshape(p.groups, p.N)[experts]), bias.dt, (len(experts), p.N))
    for po in p.post_ops:
        assert po.src1 is None, "binary post-op operands of grouped problems are not sharded"
    off = np.cumsum([int(ends[e] - begins[e]) for e in experts]).astype(np.int32)
    return W.Problem("%s[experts of rank %d]" % (p.name, rank), m, p.N, p.K, src, wei, p.dst_dt, bias, quant,
                     list(p.post_ops), p.apply_to_int, p.fpmath, offsets=off)


def shard(p: W.Problem, rank: int, world: int) -> W.Problem:
    if world == 1:
        return p
    return shard_experts(p, rank, world) if p.offsets is not None else shard_columns(p, rank, world)


def gather_columns(local, N, world, dist=None, group=None):
    """All-gathers column slices [M, n_r] (torch tensors) into [M, N].

    Slices may differ in width by one alignment unit, so every rank
    contributes a buffer padded to the widest slice; the padding is dropped
    when the row-major result is put together."""
    import torch
    if world == 1:
        return local
    dist = dist or torch.distributed
    M = local.shape[0]
    widths = [column_range(N, r, world)[1] - column_range(N, r, world)[0] for r in range(world)]
    wmax = max(widths)
    send = local if local.shape[1] == wmax else torch.nn.functional.pad(local, (0, wmax - local.shape[1]))
    flat = torch.empty((world * M, wmax), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    out = flat.view(world, M, wmax)
    return torch.cat([out[r, :, :widths[r]] for r in range(world)], dim=1)


def gather_columns_blocked(local, N, world, dist=None, group=None):
    """All-gathers column slices [M, n_r] into the blocked layout [world, M, n_max]
    (slice r in block r, padded to the widest slice): the collective's own
    output, without the copy that would interleave the slices into [M, N]."""
    import torch
    if world == 1:
        return local.unsqueeze(0)
    dist = dist or torch.distributed
    M = local.shape[0]
    wmax = max(column_range(N, r, world)[1] - column_range(N, r, world)[0] for r in range(world))
    send = local if local.shape[1] == wmax else torch.nn.functional.pad(local, (0, wmax - local.shape[1]))
    flat = torch.empty((world * M, wmax), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    return flat.view(world, M, wmax)


def gather_rows_blocked(local, rows_per_rank, dist=None, group=None):
    """All-gathers row blocks [m_r, N] into [world, m_max, N] (block r holds
    rank r's rows, padded to the tallest block)."""
    import torch
    world = len(rows_per_rank)
    if world == 1:
        return local.unsqueeze(0)
    dist = dist or torch.distributed
    mmax = max(rows_per_rank)
    send = local if local.shape[0] == mmax else torch.nn.functional.pad(local, (0, 0, 0, mmax - local.shape[0]))
    flat = torch.empty((world * mmax, local.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    return flat.view(world, mmax, local.shape[1])


def gather_rows(local, rows_per_rank, dist=None, group=None):
    """All-gathers row blocks [m_r, N] of different heights into [sum m_r, N]."""
    import torch
    world = len(rows_per_rank)
    if world == 1:
        return local
    dist = dist or torch.distributed
    mmax = max(rows_per_rank)
    send = local if local.shape[0] == mmax else torch.nn.functional.pad(local, (0, 0, 0, mmax - local.shape[0]))
    flat = torch.empty((world * mmax, local.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    out = flat.view(world, mmax, local.shape[1])
    return torch.cat([out[r, :rows_per_rank[r]] for r in range(world)], dim=0)


class PeerGather:
    """Assembles the shards of one dst in every rank's full [M, N] buffer with the library's own
    peer-store kernels (``dnnl_cuda_interop_peer_scatter`` / ``_peer_wait``) instead of a collective
    library.  The full buffers and the flag words live in symmetric memory (torch's allocator does the
    CUDA IPC exchange once, at construction); after that a step is two kernel launches per rank.

    full: the unsharded problem, p: this rank's shard.  ``dst`` is the [M, N] torch view of this
    rank's full buffer."""

    def __init__(self, full, p, rank, world, torch, dist, dev):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        from . import api
        self.C, self.api, self.world, self.rank = C, api, world, rank
        es = W.nbytes(full.dst_dt, 1)
        self.nbytes = full.M * full.N * es
        self.buf = symm.empty(max(16, self.nbytes), dtype=torch.uint8, device=dev)
        self.flags = symm.empty(64, dtype=torch.int32, device=dev)
        self.buf.zero_()
        self.flags.zero_()
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        hb = symm.rendezvous(self.buf, dist.group.WORLD)
        hf = symm.rendezvous(self.flags, dist.group.WORLD)
        self.peer_dst = (C.c_void_p * world)(*[int(x) for x in hb.buffer_ptrs])
        self.peer_flags = (C.c_void_p * world)(*[int(x) for x in hf.buffer_ptrs])
        self._keep = (hb, hf)
        self.epoch = 0
        elem = {W.BF16: torch.bfloat16, W.F16: torch.float16, W.F32: torch.float32, W.S32: torch.int32,
                W.S8: torch.int8, W.U8: torch.uint8}[full.dst_dt]
        self.dst = self.buf[:self.nbytes].view(elem).view(full.M, full.N)
        if full.offsets is None:
            lo, hi = column_range(full.N, rank, world)
            segs = [(0, 0, full.M)]
            self.row_bytes, self.src_pitch, self.dst_pitch, self.col_bytes = (hi - lo) * es, (hi - lo) * es, full.N * es, lo * es
        else:
            begins, ends = _expert_rows(full)
            segs, at = [], 0
            for e in expert_assignment((ends - begins).tolist(), world)[rank]:
                n = int(ends[e] - begins[e])
                if n:
                    segs.append((at, int(begins[e]), n))
                at += n
            segs = segs or [(0, 0, 0)]
            self.row_bytes = self.src_pitch = self.dst_pitch = full.N * es
            self.col_bytes = 0
        self.nseg = len(segs)
        self.segs = (C.c_int64 * (3 * self.nseg))(*[v for t in segs for v in t])
        L = api.lib()
        L.dnnl_cuda_interop_peer_scatter.argtypes = [
            C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int,
            C.c_void_p, C.c_void_p, C.c_uint, C.c_void_p]
        L.dnnl_cuda_interop_peer_wait.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_uint]
        L.dnnl_cuda_interop_primitive_replicate_dst.argtypes = [
            C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_uint]
        self.L = L
        self.es = es
        self.full_N = full.N
        # where this rank's column slice begins inside its own full buffer (dense problems)
        self.slice_ptr = int(self.buf.data_ptr()) + (self.col_bytes if full.offsets is None else 0)

    def fused_step(self, strm, prep):
        """The exchange fused into the matmul kernel: `prep` (a runner.Prepared whose dst memory is
        this rank's slice INSIDE the full buffer, row pitch N) stores every dst element into all
        ranks' buffers and publishes the flag itself; only the wait is a launch of its own.  Raises
        api.error(unimplemented) for implementations without the fused form."""
        self.epoch += 1
        st = self.L.dnnl_cuda_interop_primitive_replicate_dst(
            prep.prim._h, self.world, self.rank, self.peer_dst, self.C.c_size_t(max(16, self.nbytes)), self.peer_flags,
            self.done.data_ptr(), self.epoch)
        if st != 0:
            self.epoch -= 1
            raise self.api.error(st, "replicate dst")
        prep.execute(strm)
        st = self.L.dnnl_cuda_interop_peer_wait(strm._h, self.world, self.flags.data_ptr(), self.epoch)
        if st != 0:
            raise self.api.error(st, "peer wait")

    def step(self, strm, local_dst_ptr):
        """Enqueues scatter + wait on the library stream; the assembled result is complete on this
        rank once the stream has passed the wait."""
        self.epoch += 1
        st = self.L.dnnl_cuda_interop_peer_scatter(strm._h, self.world, self.rank, local_dst_ptr, self.row_bytes,
                                                   self.src_pitch, self.peer_dst, self.dst_pitch, self.col_bytes,
                                                   self.nseg, self.segs, self.peer_flags, self.epoch, self.done.data_ptr())
        if st != 0:
            raise self.api.error(st, "peer scatter")
        st = self.L.dnnl_cuda_interop_peer_wait(strm._h, self.world, self.flags.data_ptr(), self.epoch)
        if st != 0:
            raise self.api.error(st, "peer wait")
