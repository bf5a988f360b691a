"""N>1 host logic on CPU: two `gloo` ranks shard a problem the way the GPU
ranks do (columns for dense problems, experts for grouped ones), compute
their shard with the CPU oracle, all-gather, and the assembled result must
equal the unsharded oracle result bit for bit."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from onednn_b200 import workloads as W, sharding as S
from oracle import oracle as O

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)

def as_f32(p, out):
    return torch.from_numpy(np.ascontiguousarray(W.to_f32(out, p.dst_dt).reshape(p.M, p.N)))

def biased_moe():
    p = W.moe_grouped(48, 64, 32, 6, sizes=[20, 1, 0, 9, 15, 3])
    r = np.random.Generator(np.random.PCG64(3))
    p.bias = W.QTensor(r.standard_normal((6, p.N)).astype(np.float32), W.F32, (6, p.N))
    return p

problems = [W.int8_zp(24, 64, 96, per_n_scales=True), W.int8_postops(16, 64, 80), W.fp8_prefill(8, 64, 48),
            W.int4_decode(3, 128, 64), W.moe_grouped(40, 64, 32, 5, sizes=[7, 0, 13, 20, 0]), biased_moe()]
for p in problems:
    local = S.shard(p, rank, world)
    got_local = as_f32(local, O.run_port(local))
    if p.offsets is None:
        full = S.gather_columns(got_local, p.N, world)
        blocks = S.gather_columns_blocked(got_local, p.N, world)  # [rank][M][widest slice]
        widths = [S.column_range(p.N, r, world)[1] - S.column_range(p.N, r, world)[0] for r in range(world)]
        assert torch.equal(torch.cat([blocks[r, :, :widths[r]] for r in range(world)], dim=1), full)
    else:
        rows = [S.shard(p, r, world).M for r in range(world)]
        stacked = S.gather_rows(got_local, rows)  # rank blocks, one after the other
        blocks = S.gather_rows_blocked(got_local, rows)  # [rank][tallest block][N]
        assert torch.equal(torch.cat([blocks[r, :rows[r]] for r in range(world)], dim=0), stacked)
        rank_of, local_row = S.row_map(p, world)  # where each row of the unsharded problem lies
        full = blocks[torch.from_numpy(rank_of), torch.from_numpy(local_row)]
    want = as_f32(p, O.run_port(p))
    assert full.shape == want.shape, (p.name, full.shape, want.shape)
    assert torch.equal(full, want), "%s: sharded result differs on rank %d" % (p.name, rank)
dist.barrier()
dist.destroy_process_group()
print("rank %d ok" % rank)
"""


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_two_gloo_ranks_assemble_the_unsharded_result(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for pr in procs:
        try:
            out, _ = pr.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            pr.kill()
            out, _ = pr.communicate()
        outs.append(out)
    for rank, (pr, out) in enumerate(zip(procs, outs)):
        assert pr.returncode == 0, "rank %d failed:\n%s" % (rank, out[-3000:])
        assert "rank %d ok" % rank in out


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_column_ranges_partition_n(world):
    from onednn_b200.sharding import column_range
    for N in (16, 48, 4096, 28672, 16 * 13):
        edges = [column_range(N, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == N
        for (lo, hi), (lo2, _) in zip(edges, edges[1:]):
            assert hi == lo2 and lo % 16 == 0 and hi >= lo


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_shards_cover_all_rows(world):
    from onednn_b200 import workloads as W
    from onednn_b200.sharding import shard
    p = W.moe_grouped(64, 32, 16, 8)
    from onednn_b200.sharding import row_map, expert_assignment
    shards = [shard(p, r, world) for r in range(world)]
    assert sum(s.M for s in shards) == p.M
    assert sum(s.groups for s in shards) == p.groups
    assert all(s.groups == p.groups // world for s in shards)
    rank_of, local = row_map(p, world)
    src = p.src.data.reshape(p.M, p.K)
    for m in range(p.M):
        s = shards[rank_of[m]]
        assert np.array_equal(s.src.data.reshape(s.M, s.K)[local[m]], src[m])
    # the benchmark's distribution: the heaviest rank carries at most 1.3 x the mean cost, unless the
    # largest expert alone (with the cheapest companions its rank must take) already exceeds that
    big = W.moe_grouped(8192, 16, 16, 64)
    ends = big.offsets.astype(np.int64)
    rows = np.diff(np.concatenate([[0], ends])).tolist()
    own = expert_assignment(rows, world)
    cost = [sum(0 if rows[e] == 0 else max(128, rows[e]) for e in o) for o in own]
    assert sorted(sum(own, [])) == list(range(64))
    floor = max(rows) + (64 // world - 1) * 128
    assert max(cost) <= max(1.3 * (sum(cost) / world), floor)
