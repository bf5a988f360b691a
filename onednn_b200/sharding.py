"""Sharding of one matmul across the GPUs of a node (one process per GPU).

Dense problems shard by output columns: rank r holds weights[:, r*N/g:(r+1)*N/g]
with the matching slices of every per-N parameter (weight scales and
zero-points, bias, binary post-op operands); src and per-row parameters are
replicated.  Each rank runs an ordinary matmul on its slice and the dst
slices are assembled with an all-gather (``gather_columns``).

Grouped (MoE) problems shard by experts: rank r holds a contiguous block of
experts and the src rows routed to them; the dst row blocks are assembled
with a variable-size all-gather (``gather_rows``).
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


def shard_experts(p: W.Problem, rank: int, world: int) -> W.Problem:
    assert p.offsets is not None
    e0, e1 = expert_range(p.groups, rank, world)
    ends = p.offsets.astype(np.int64)
    r0 = int(ends[e0 - 1]) if e0 > 0 else 0
    r1 = int(ends[e1 - 1]) if e1 > e0 else r0
    src = W.QTensor(np.ascontiguousarray(p.src.data.reshape(p.M, p.K)[r0:r1]), p.src.dt, (r1 - r0, p.K))
    wei = W.QTensor(np.ascontiguousarray(p.wei.data[e0:e1]), p.wei.dt, (e1 - e0, p.K, p.N))
    quant = {}
    for name, q in p.quant.items():
        assert name.startswith("wei") and (q.mask & 1), "only per-expert weight parameters are sharded"
        quant[name] = W.Quant(np.ascontiguousarray(q.data[e0:e1]), q.dt, q.mask, q.groups)
    off = (ends[e0:e1] - r0).astype(np.int32)
    return W.Problem("%s[e %d:%d]" % (p.name, e0, e1), r1 - r0, p.N, p.K, src, wei, p.dst_dt, None, quant,
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
