"""Benchmark of the quantized matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one execution of a workload's matmul through the library's C API.
Without --workload the run covers the five benchmark configurations (the int4
decode at M = 1, 8 and 32) and prints ONE JSON line: its top-level fields
describe the headline workload, the fp8 prefill GEMM (e4m3 [4096,4096] x e4m3
[4096,14336] -> bf16, per-tensor scales, bf16 bias), and `workloads` carries
the same fields for every workload.  For N > 1 (launched under torchrun) dense
problems are sharded by output columns and the grouped one by experts; every
rank computes its shard and the full dst is assembled on every rank by the
library's own peer-store kernels (fused into the GEMM epilogue at two ranks;
`--gather nccl`, or no peer-mapped memory: an NCCL all-gather); the total
problem is fixed, so scaling is "strong".

Per workload:
  value     whole-job throughput with inputs resident in HBM: blocks of K steps,
            each timed with CUDA events on the launching stream between
            barriers (max over ranks), repeated until 0.25 s of blocks have
            run; the median block is reported, the best beside it
  e2e       the same metric with the step's src copied from pinned host memory
            and this rank's dst read back to the host inside the timed region
  roofline  algorithmic work of one launch / its average duration, against the
            measured peaks of MEASURED_PEAKS.json (burst and sustained)
  parity    a seeded subset of dst rows of the (gathered) result against the
            CPU oracle, outside the timed region; a mismatch fails the run
  cpu_baseline  the reference's CPU matmul on a bounded sample (headline only)
`--impl reference` times that CPU implementation alone (rank 0 only).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from onednn_b200 import workloads as W  # noqa: E402

WORKLOADS = {
    # name: (factory, metric, unit, bound, compute dtype)
    "fp8_prefill": (lambda **kw: W.fp8_prefill(**kw), "fp8_matmul_tflops", "TFLOP/s", "tensor", "f8_e4m3"),
    "int8_postops": (lambda **kw: W.int8_postops(**kw), "int8_matmul_tops", "TOP/s", "tensor", "s8"),
    "int8_zp": (lambda **kw: W.int8_zp(**kw), "int8_matmul_tops", "TOP/s", "tensor", "u8"),
    "int4_decode": (lambda **kw: W.int4_decode(**kw), "int4_decode_hbm_gbs", "GB/s", "hbm", "bf16"),
    "moe_grouped": (lambda **kw: W.moe_grouped(**kw), "moe_matmul_tflops", "TFLOP/s", "tensor", "bf16"),
}
# the default run: the headline first, then the rest of the metric BASELINE.json names
SUITE = [("fp8_prefill", {}), ("int8_zp", {}), ("int8_postops", {}), ("int4_decode", {"M": 1}),
         ("int4_decode", {"M": 8}), ("int4_decode", {"M": 32}), ("moe_grouped", {})]
MIN_TIMED_S = 0.25
L2_BYTES = 126e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + ["reorder_quantize"],
                    help="one workload instead of the whole suite")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--kernel", default=None, help="pin an implementation by name substring")
    ap.add_argument("--M", type=int, default=None, help="override M (decode: 1, 8 or 32)")
    ap.add_argument("--K", type=int, default=None)
    ap.add_argument("--N", type=int, default=None)
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the results")
    ap.add_argument("--min-time", type=float, default=MIN_TIMED_S, help="seconds of timed blocks per workload")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: assemble dst with the library's peer-store kernels, or with an NCCL all-gather")
    return ap.parse_args()


def make_problem(name, kw, args):
    kw = dict(kw)
    if args.M is not None:
        kw["total_M" if name == "moe_grouped" else "M"] = args.M
    if args.K is not None:
        kw["K"] = args.K
    if args.N is not None:
        kw["N"] = args.N
    if args.small:
        small = {"fp8_prefill": dict(M=2048, K=2048, N=8192), "int8_postops": dict(M=1024, K=2048, N=4096),
                 "int4_decode": dict(K=8192, N=16384), "moe_grouped": dict(total_M=2048, K=2048, N=4096, experts=16),
                 "int8_zp": {}}[name]
        small.update(kw)
        kw = small
    return WORKLOADS[name][0](**kw)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0=None, t1=None):
        """Clocks seen between wall-clock times t0 and t1 (all samples when omitted)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in list(self.lines):
            if (t0 is not None and ts < t0) or (t1 is not None and ts > t1 + 0.05):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measure_8bit_yardstick(torch, dev):
    """A library 8-bit GEMM as a YARDSTICK for the tensor peak (never on the product path):
    torch._scaled_mm on e4m3 8192^3, best of 10, in TFLOP/s; None where it does not run."""
    try:
        n = 8192
        a = torch.randn((n, n), device=dev, dtype=torch.bfloat16).to(torch.float8_e4m3fn)
        b = torch.randn((n, n), device=dev, dtype=torch.bfloat16).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev, dtype=torch.float32)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e30
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        del a, b
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:  # the yardstick is optional
        return None


def dram_traffic(workload_key, world):
    """DRAM bytes of one launch of the dominant kernel, from the committed ncu
    capture of this exact workload (single GPU); None when there is none."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if world != 1 or not os.path.exists(path):
        return None
    entry = json.load(open(path)).get(workload_key)
    return entry["bytes"] if entry else None


# ------------------------------------------------------------------ GPU arm
def device_buffers(p, torch, dev):
    """Uploads every tensor of the problem once; returns (ptr dict, keepalive)."""
    keep, ptrs = {}, {}

    def up(name, arr):
        t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).to(dev)
        keep[name] = t
        ptrs[name] = t.data_ptr()
        return t

    up("src", p.src.data)
    up("wei", p.wei.data)
    if p.bias is not None:
        up("bias", p.bias.data)
    for name, q in p.quant.items():
        up(name, q.data)
    for i, po in enumerate(p.post_ops):
        if po.src1 is not None:
            up("po%d" % i, po.src1.data)
    if p.offsets is not None:
        up("offsets", p.offsets)
    dst = torch.zeros(max(1, W.nbytes(p.dst_dt, p.M * p.N)), dtype=torch.uint8, device=dev)
    keep["dst"] = dst
    ptrs["dst"] = dst.data_ptr()
    return ptrs, keep


def parity_rows(full):
    """The dst rows the oracle checks: spread over the row tiles (dense) or over the experts and
    thereby over the ranks' blocks (grouped), seeded."""
    r = np.random.Generator(np.random.PCG64(11))
    if full.offsets is None:
        n = min(full.M, 3 if full.K * full.N > 2e8 else 6)
        rows = [0, full.M - 1] + [int(x) for x in r.integers(0, full.M, max(0, n - 2))]
    else:
        ends = full.offsets.astype(np.int64)
        begins = np.concatenate([[0], ends[:-1]])
        live = [g for g in range(full.groups) if ends[g] > begins[g]]
        picks = [live[0], live[len(live) // 3], live[2 * len(live) // 3], live[-1]]
        rows = [int(begins[0]), int(ends[-1] - 1)] + [int(r.integers(begins[g], ends[g])) for g in picks]
    return np.unique(np.array(rows, dtype=np.int64))


def measure(args, name, kw, ctx):
    """One workload on this rank's GPU (and its peers'); returns the result dict on rank 0."""
    torch, dist, api, sharding, Prepared = ctx["torch"], ctx["dist"], ctx["api"], ctx["sharding"], ctx["Prepared"]
    world, rank, dev, eng, strm = ctx["world"], ctx["rank"], ctx["dev"], ctx["eng"], ctx["strm"]
    _, metric, unit, bound, dtype = WORKLOADS[name]
    full = make_problem(name, kw, args)
    p = sharding.shard(full, rank, world)
    grouped = full.offsets is not None

    # A step must not find its inputs in the 126 MB L2 left there by the step before: when one
    # rank's working set is not clearly larger than L2 (decode, and every workload once it is
    # sharded), consecutive steps use different copies of all buffers, enough of them that a
    # cycle through the copies moves 2.5 x L2.
    ws = float(p.algorithmic_bytes())
    nsets = 1 if ws > 1.5 * L2_BYTES else int(min(8, max(2, np.ceil(2.5 * L2_BYTES / max(ws, 1.0)))))
    sets, set_ptrs = [], []
    for _ in range(nsets):
        ptrs_s, keep_s = device_buffers(p, torch, dev)
        sets.append((Prepared(p, eng, args.kernel).bind_device(ptrs_s), keep_s))
        set_ptrs.append(ptrs_s)
    prep = sets[0][0]
    preps = [s[0] for s in sets]
    l2_note = ("working set %.0f MB > 126 MB L2" % (ws / 1e6)) if nsets == 1 else \
        ("%d copies of all buffers rotated, %.0f MB per cycle %s 126 MB L2" %
         (nsets, nsets * ws / 1e6, ">" if nsets * ws > L2_BYTES else "< (L2-resident workload)"))
    elem = {W.BF16: torch.bfloat16, W.F16: torch.float16, W.F32: torch.float32, W.S32: torch.int32,
            W.S8: torch.int8, W.U8: torch.uint8}[p.dst_dt]
    rows_per_rank = [sharding.shard(full, r, world).M for r in range(world)] if (grouped and world > 1) else None
    # N > 1: the library's own exchange (peer stores into every rank's full dst + flags) unless NCCL was asked for
    # or peer-mapped memory cannot be had; every rank must take the same path
    peers = None
    if world > 1 and args.gather == "peer":
        try:
            peers = [sharding.PeerGather(full, p, rank, world, torch, dist, dev) for _ in range(nsets)]
            ok_t = torch.ones(1, device=dev)
        except Exception as e:  # no peer access / no symmetric memory on this system
            if rank == 0:
                print("peer gather unavailable (%s): using NCCL" % e, file=sys.stderr)
            peers, ok_t = None, torch.zeros(1, device=dev)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        if float(ok_t[0]) == 0:
            peers = None
    # the tcgen05 GEMM stores into every rank's buffer from its own epilogue (no scatter pass): its
    # dst memory is this rank's column slice inside the full buffer
    # (two ranks: with more, the 64-byte runs a warp's dst store covers use NVLink half as well as the
    # scatter kernel's 512-byte ones, and every element leaves world - 1 times)
    fused = None
    if (peers is not None and world == 2 and not grouped and prep.impl in ("cuda:tcgen05:int8", "cuda:tcgen05:fp8")
            and not p.post_ops and (p.bias is None or p.bias.dims[0] == 1)):
        fused = []
        for i in range(nsets):
            ptrs_f = dict(set_ptrs[i])
            ptrs_f["dst"] = peers[i].slice_ptr
            fused.append(Prepared(p, eng, args.kernel, dst_ld=full.N).bind_device(ptrs_f))

    def gather(i=0):
        if world == 1:
            return None
        if peers is not None:
            if fused is None:
                peers[i % nsets].step(strm, sets[i % nsets][1]["dst"].data_ptr())
            return peers[i % nsets].dst
        local = sets[i % nsets][1]["dst"].view(elem).view(p.M, p.N)
        # the gathered result stays in the collective's blocked layout ([rank][M][N/g] column
        # slices, [rank][rows][N] expert blocks): no interleaving copy inside the step
        if rows_per_rank is not None:
            return sharding.gather_rows_blocked(local, rows_per_rank)
        return sharding.gather_columns_blocked(local, full.N, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def execute(i):
        if fused is not None:
            peers[i % nsets].fused_step(strm, fused[i % nsets])
        else:
            preps[i % nsets].execute(strm)

    K = args.steps
    for i in range(max(3, args.warmup)):
        execute(i)
        gather(i)
    barrier()

    # ---- device-timed blocks of K steps, inputs resident in HBM, for at least min_time seconds
    launches0 = api.launch_count()
    blocks, kernel_blocks, step_no = [], [], 0
    t_wall0 = time.time()
    budget = torch.zeros(1, dtype=torch.float64, device=dev)
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)] \
            if world > 1 else None
        barrier()
        e0.record()
        for j in range(K):
            if k_ev:
                k_ev[j][0].record()
            execute(step_no)
            if k_ev:
                k_ev[j][1].record()
            gather(step_no)
            step_no += 1
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        blocks.append(ms)
        # N = 1: the step is the kernel(s) of one execute; N > 1: events around each execute
        kernel_blocks.append(float(np.mean([a.elapsed_time(b) for a, b in k_ev])) if k_ev else ms / K)
        # every rank leaves the loop after the same block: the slowest rank's accumulated time decides
        budget[0] = sum(blocks)
        if world > 1:
            dist.all_reduce(budget, op=dist.ReduceOp.MAX)
        if float(budget[0]) >= args.min_time * 1e3 or len(blocks) >= 2000:
            break
    t_wall1 = time.time()
    launches_per_block = (api.launch_count() - launches0) / len(blocks)
    n_blocks = len(blocks)
    med_i = int(np.argsort(blocks)[n_blocks // 2])

    # ---- end to end: src from pinned host memory, this rank's dst slice back to the host, every step
    # (a result consumed on the host needs no device gather: each rank's slice lands in its own
    # region of the host buffer)
    src_host = torch.from_numpy(p.src.data.view(np.uint8).reshape(-1).copy()).pin_memory()
    out_bytes = int(sets[0][1]["dst"].numel())
    dst_host = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
    e2e_steps = max(3, min(K, 20))

    # Steps overlap as they would in a serving loop: the copy-in of step i + 1 and the copy-out of step
    # i - 1 run on streams of their own beside the matmul of step i (two or more src / dst buffer
    # pairs; weights and parameters shared).  Every step still pays both copies inside the timed region.
    e2e_slots = []
    for j in range(max(2, min(nsets, 3))):
        if j < nsets:
            e2e_slots.append((preps[j], sets[j][1]["src"], sets[j][1]["dst"]))
        else:
            src_d = torch.empty_like(sets[0][1]["src"])
            dst_d = torch.empty_like(sets[0][1]["dst"])
            ptrs_e = dict(set_ptrs[0])
            ptrs_e["src"], ptrs_e["dst"] = src_d.data_ptr(), dst_d.data_ptr()
            e2e_slots.append((Prepared(p, eng, args.kernel).bind_device(ptrs_e), src_d, dst_d))
    main_s = torch.cuda.current_stream()
    h2d_s, d2h_s = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in e2e_slots]
    ev_comp = [torch.cuda.Event() for _ in e2e_slots]
    ev_out = [torch.cuda.Event() for _ in e2e_slots]

    def e2e_step(i):
        j = i % len(e2e_slots)
        prep_j, src_d, dst_d = e2e_slots[j]
        with torch.cuda.stream(h2d_s):
            h2d_s.wait_event(ev_comp[j])  # the matmul that read this src buffer last
            src_d.copy_(src_host, non_blocking=True)
            ev_in[j].record(h2d_s)
        main_s.wait_event(ev_in[j])
        main_s.wait_event(ev_out[j])  # the copy-out that read this dst buffer last
        prep_j.execute(strm)
        ev_comp[j].record(main_s)
        with torch.cuda.stream(d2h_s):
            d2h_s.wait_event(ev_comp[j])
            dst_host.copy_(dst_d, non_blocking=True)
            ev_out[j].record(d2h_s)

    def e2e_drain():
        for e in ev_out:
            main_s.wait_event(e)

    e2e_step(0)
    e2e_drain()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_drain()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / e2e_steps

    # ---- parity of the assembled result, outside the timed region
    parity = None
    if not args.no_parity:
        execute(0)
        g = gather(0)
        torch.cuda.synchronize()
        if rank == 0:
            from oracle.parity import check_rows
            rows = parity_rows(full)
            if g is None:
                got_rows = sets[0][1]["dst"].view(elem).view(full.M, full.N)[torch.from_numpy(rows).to(dev)]
            elif peers is not None:  # this rank's full [M, N] buffer, filled by all ranks
                got_rows = g[torch.from_numpy(rows).to(dev)]
            elif grouped:
                rank_of, local_row = sharding.row_map(full, world)
                got_rows = g[torch.from_numpy(rank_of[rows]).to(dev), torch.from_numpy(local_row[rows]).to(dev)]
            else:
                widths = [sharding.column_range(full.N, r, world)[1] - sharding.column_range(full.N, r, world)[0]
                          for r in range(world)]
                sel = torch.from_numpy(rows).to(dev)
                got_rows = torch.cat([g[r, sel, :widths[r]] for r in range(world)], dim=1)
            got_np = got_rows.contiguous().view(torch.uint8).cpu().numpy().view(W.NP_STORAGE[full.dst_dt]).reshape(len(rows), full.N)
            scattered = np.zeros((full.M, full.N), W.NP_STORAGE[full.dst_dt])
            scattered[rows] = got_np
            reordered = not prep.impl.startswith("cuda:ref") and full.src.dt not in (W.S8, W.U8)
            res = check_rows(full, scattered, rows, reordered)
            parity = {"rows": res["rows"], "ok": bool(res["ok"] and res["strict_misses_explained"]),
                      "beyond_1ulp": res["beyond_strict"], "detail": res["msg"]}

    t = torch.tensor([blocks[med_i], min(blocks), kernel_blocks[med_i], e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    block_ms, best_ms, kernel_ms, e2e_ms = [float(x) for x in t.tolist()]
    ms_per_step = block_ms / K
    for s in sets:
        s[1].clear()
    del sets, preps
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    pk = ctx["peaks"]
    if bound == "hbm":
        work_full, work_launch = full.algorithmic_bytes() / 1e9, p.algorithmic_bytes() / 1e9
        peak, peak_sus, runit = pk["hbm_gbs"], pk["hbm_gbs"], "GB/s"
    else:
        work_full, work_launch = full.ops() / 1e12, p.ops() / 1e12
        # fp8 / int8 tensor peak: twice the measured dense bf16 figure (the 8-bit MMA rate is
        # twice the 16-bit one); bf16 workloads use it as is
        mult = 1.0 if dtype == "bf16" else 2.0
        peak, peak_sus, runit = mult * pk["bf16_tflops"], mult * pk["bf16_tflops_sustained"], "TFLOP/s"
    achieved = work_launch / (kernel_ms * 1e-3)
    wkey = "%s M=%d K=%d N=%d" % (name, full.M, full.K, full.N)
    clocks = ctx["sampler"].summary(t_wall0, t_wall1) if ctx["sampler"] else None
    if clocks is not None:
        clocks["sampled"] = "over this workload's timed blocks (%.2f s)" % (t_wall1 - t_wall0)
    roof = {"bound": bound, "achieved": achieved, "peak": peak, "unit": runit, "frac": achieved / peak,
            "peak_sustained": peak_sus, "frac_sustained": achieved / peak_sus,
            "traffic": dram_traffic(wkey, world),
            "traffic_unit": "bytes per launch (ncu, profiles/dram_traffic.json)",
            "algorithmic_bytes": int(p.algorithmic_bytes()), "peak_source": pk["source"], "kernel_ms": kernel_ms}
    if bound == "tensor" and dtype != "bf16" and ctx.get("peak_8bit"):
        roof["peak_8bit_measured"] = ctx["peak_8bit"]
        roof["frac_of_8bit_measured"] = achieved / ctx["peak_8bit"]
        roof["peak_8bit_how"] = "torch._scaled_mm e4m3 8192^3, best of 10 (a library GEMM as yardstick only)"
    return {
        "metric": metric, "value": work_full / (ms_per_step * 1e-3), "unit": unit, "n_gpus": world, "steps": K,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": wkey, "kernel": prep.impl,
                   "parallelism": ("%s x%d + %s"
                                   % ("expert-shard (balanced by rows)" if grouped else "n-shard", world,
                                      ("dst stores of the GEMM epilogue repeated into every rank's [M,N] dst, flag wait (own kernels)"
                                       if fused is not None else
                                       "peer stores of every rank's block into every rank's [M,N] dst, flag wait (own kernels)")
                                      if peers is not None else "NCCL all-gather into [rank][M][N/g] blocks"))
                   if world > 1 else "single",
                   "l2": l2_note,
                   "e2e": "src H2D from pinned memory and this rank's dst D2H every step (copies of neighbouring steps overlap the matmul on their own streams); weights resident"},
        "timing": {"blocks": n_blocks, "steps_per_block": K, "timed_region_s": sum(blocks) / 1e3,
                   "ms_per_step_median_block": ms_per_step, "ms_per_step_best_block": best_ms / K},
        "roofline": roof,
        "e2e": {"value": work_full / (e2e_ms * 1e-3), "unit": unit, "h2d_bytes_per_step": int(src_host.numel()),
                "d2h_bytes_per_step": int(out_bytes), "ms_per_step": e2e_ms},
        "gpu_launches": int(round(launches_per_block)), "clocks": clocks, "parity": parity,
    }, full


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from onednn_b200 import api, sharding
    from onednn_b200.runner import Prepared

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    eng = api.engine(api.engine.kind.gpu, local_rank)
    strm = api.stream(eng, torch.cuda.current_stream().cuda_stream)
    ctx = {"torch": torch, "dist": dist, "api": api, "sharding": sharding, "Prepared": Prepared, "world": world,
           "rank": rank, "dev": dev, "eng": eng, "strm": strm, "peaks": peaks(), "sampler": None}
    if rank == 0:
        ctx["peak_8bit"] = measure_8bit_yardstick(torch, dev)
        ctx["sampler"] = ClockSampler(local_rank).start()
    suite = [(args.workload, {})] if args.workload else SUITE
    results, head_full = {}, None
    for name, kw in suite:
        out = measure(args, name, kw, ctx)
        if rank == 0:
            res, full = out
            results[res["config"]["workload"]] = res
            if head_full is None:
                head_full, head = full, res
    if ctx["sampler"]:
        ctx["sampler"].stop()
    if rank == 0:
        line = dict(head)
        if len(results) > 1:
            line["workloads"] = results
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(head_full, suite[0][0], WORKLOADS[suite[0][0]][3], seconds=15.0)
        print(json.dumps(line), flush=True)
        bad = [k for k, v in results.items() if v["parity"] is not None and not v["parity"]["ok"]]
        if bad:
            print("parity check failed for: %s" % ", ".join(bad), file=sys.stderr, flush=True)
    ok = torch.tensor([0 if (rank == 0 and bad) else 1], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        dist.destroy_process_group()
    if int(ok[0]) == 0:
        sys.exit(3)


# ------------------------------------------------------- CPU reference arm
def host_threads():
    """All the host threads the CPU arm may use: torchrun exports OMP_NUM_THREADS=1 to its
    workers, which is not what a CPU baseline should run with."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(n)
    return n


def cpu_sample(full):
    """A bounded sample of the workload for the CPU: a seeded subset of src
    rows (dense) or a smaller token count (grouped); K, N and every attribute
    are those of the full problem."""
    if full.offsets is not None:
        def make(m):
            return W.moe_grouped(total_M=m, K=full.K, N=full.N, experts=full.groups), "total_M=%d of %d" % (m, full.M)
    else:
        def make(m):
            if m >= full.M:
                return full, "all %d src rows" % full.M
            rows = np.sort(np.random.Generator(np.random.PCG64(7)).choice(full.M, size=m, replace=False))
            return full.take_rows(rows), "%d of %d src rows" % (m, full.M)
    return make


def time_cpu(p, iters):
    """(ms, implementation, kind) of the reference CPU matmul on problem p:
    the unmodified reference library when a build of it is present (first
    implementation it dispatches), else the C restatement of its scalar code."""
    from oracle import oracle as O
    if O.ref_available():
        _, impl, ms = O.run_ref(p, pin_ref=False, iters=iters)
        return ms, impl, "reference"
    best = 1e30
    for _ in range(iters):
        t0 = time.perf_counter()
        O.run_port(p)
        best = min(best, (time.perf_counter() - t0) * 1e3)
    return best, "oracle port of ref*:any", "port"


def cpu_baseline(full, name, bound, seconds=15.0, iters=2):
    """Sizes the sample so that one execution takes a worthwhile fraction of `seconds`, then times
    `iters` executions (best).  Returns the cpu_baseline object; `executions` counts every timed run."""
    cores = host_threads()
    make = cpu_sample(full)
    m = min(full.M, 1 if full.offsets is None else full.groups)
    p, what = make(m)
    ms, impl, kind = time_cpu(p, 1)
    runs = 1
    # grow the sample until one execution is worth timing, within the budget (the whole problem
    # where the reference's own fast implementation makes that affordable)
    while ms * 4 < seconds * 1e3 / (iters + 1) and m < full.M:
        m = min(full.M, m * 4)
        p, what = make(m)
        ms, impl, kind = time_cpu(p, 1)
        runs += 1
    if ms * (iters + 1) < seconds * 1e3:
        ms2, impl, kind = time_cpu(p, iters)
        runs += iters
        ms = min(ms, ms2)
    work = (p.algorithmic_bytes() / 1e9) if bound == "hbm" else (p.ops() / 1e12)
    return {"value": work / (ms * 1e-3), "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
            "cores": cores, "kind": kind, "impl": impl, "ms": ms, "executions": runs,
            "sample": "%s, K=%d N=%d, %.1f ms per execution" % (what, p.K, p.N, ms)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload or SUITE[0][0]
    _, metric, unit, bound, dtype = WORKLOADS[name]
    full = make_problem(name, {}, args)
    base = cpu_baseline(full, name, bound, seconds=20.0, iters=max(1, min(args.steps, 3)))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    # steps / warmup: what was executed (a bounded sample of the workload per step, see cpu_baseline.sample)
    line = {"impl": "reference", "metric": metric, "value": base["value"], "unit": unit, "n_gpus": world,
            "steps": base["executions"], "warmup": 0, "ms_per_step": base["ms"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": "%s M=%d K=%d N=%d" % (name, full.M, full.K, full.N)},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------ reorder (weight quantization) arm
def reorder_problem(K, N, seed=20266):
    """f32 [K,N] -> s8 with one dst scale per column: the quantization of a weight matrix."""
    r = np.random.Generator(np.random.PCG64(seed))
    w = (r.standard_normal((K, N), dtype=np.float32) * 0.05)
    sc = (np.abs(w).max(axis=0, keepdims=True) / 127.0).astype(np.float32)
    return W.Reorder("reorder_quantize", W.QTensor(w, W.F32, (K, N)), W.S8, quant={"dst_scale": W.Quant(sc, W.F32, 2)})


def reorder_cpu(K, N, seconds=10.0):
    """The reference's CPU reorder on a sample of the rows (wall clock around one call of the
    reference library through its C++ API, primitive creation included; best of 3)."""
    from oracle import oracle as O
    cores = host_threads()
    rows = K  # the whole tensor: a call takes milliseconds
    r = reorder_problem(rows, N)
    run = (lambda: O.run_ref_reorder(r)[1]) if O.ref_available() else (lambda: (O.run_port_reorder(r), "oracle port")[1])
    best, impl, t_all = 1e30, "", time.perf_counter()
    for _ in range(3):
        t0 = time.perf_counter()
        impl = run()
        best = min(best, time.perf_counter() - t0)
        if time.perf_counter() - t_all > seconds:
            break
    gb = rows * N * 5 / 1e9
    return {"value": gb / best, "unit": "GB/s", "cores": cores,
            "kind": "reference" if O.ref_available() else "port", "impl": impl, "ms": best * 1e3,
            "sample": "%d of %d rows, N=%d, %.1f ms per call incl. primitive creation" % (rows, K, N, best * 1e3)}


def run_reorder_bench(args):
    K, N = args.K or 4096, args.N or 14336
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    wkey = "reorder_quantize f32[%d,%d] -> s8, per-column dst scales" % (K, N)
    if args.impl == "reference":
        if rank == 0:
            base = reorder_cpu(K, N)
            print(json.dumps({"impl": "reference", "metric": "reorder_hbm_gbs", "value": base["value"], "unit": "GB/s",
                              "n_gpus": world, "steps": 3, "warmup": 0, "ms_per_step": base["ms"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                              "data": "synthetic", "config": {"workload": wkey},
                              "cpu_baseline": base,
                              "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                                      "d2h_bytes_per_step": 0}}), flush=True)
        return
    import torch
    import torch.distributed as dist
    from onednn_b200 import api
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    Nl = N // world // 16 * 16 if world > 1 else N  # this rank's columns (a tensor of its own)
    if world > 1 and rank == world - 1:
        Nl = N - Nl * (world - 1)
    eng = api.engine(api.engine.kind.gpu, local_rank)
    strm = api.stream(eng, torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device=dev).manual_seed(20266 + rank)
    src_md, dst_md = api.memory.desc((K, Nl), W.F32, api.tag.ab), api.memory.desc((K, Nl), W.S8, api.tag.ab)
    attr = api.primitive_attr()
    attr.set_scales(api.ARG_DST, 2, (), W.F32)
    pd = api.reorder.primitive_desc(eng, src_md, eng, dst_md, attr)
    key = api.ARG_ATTR_SCALES | api.ARG_DST
    # as in the matmul arm: copies of the buffers in rotation when one rank's tensors do not exceed L2 clearly
    ws = float(K * Nl * 5)
    nsets = 1 if ws > 1.5 * 126e6 else int(min(8, max(2, np.ceil(2.5 * 126e6 / ws))))
    bufs = []
    for _ in range(nsets):
        s_ = torch.randn((K, Nl), generator=g, device=dev, dtype=torch.float32) * 0.05
        c_ = (s_.abs().amax(dim=0, keepdim=True) / 127.0).contiguous()
        d_ = torch.zeros((K, Nl), device=dev, dtype=torch.int8)
        bufs.append((s_, d_, c_, {api.ARG_FROM: api.memory(src_md, eng, s_.data_ptr()),
                                  api.ARG_TO: api.memory(dst_md, eng, d_.data_ptr()),
                                  key: api.memory(pd.query_md(api.QUERY_EXEC_ARG_MD, key), eng, c_.data_ptr())}))
    src, dst = bufs[0][0], bufs[0][1]

    class _Rotating:
        """Executes the reorder on the next set of buffers at every call."""
        def __init__(self):
            self.prim, self.i = api.reorder(pd), 0

        def execute(self, strm, _unused=None):
            self.prim.execute(strm, bufs[self.i % nsets][3])
            self.i += 1

    prim, ex_args = _Rotating(), None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        prim.execute(strm, ex_args)
    barrier()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    launches0 = api.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        prim.execute(strm, ex_args)
    e1.record()
    barrier()
    launches = api.launch_count() - launches0
    total_ms = e0.elapsed_time(e1)
    if sampler:
        t_end = time.time() + 1.5
        while time.time() < t_end:
            for _ in range(20):
                prim.execute(strm, ex_args)
            torch.cuda.synchronize()
    barrier()
    clocks = None
    if sampler:
        sampler.stop()
        clocks = sampler.summary()
        clocks["sampled"] = "over the timed region and a 1.5 s untimed repeat of the same step"
    # end to end: f32 weights from pinned host memory, s8 result back to the host
    src_host = src.cpu().pin_memory()
    dst_host = torch.empty((K, Nl), dtype=torch.int8).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    for _ in range(e2e_steps):
        src.copy_(src_host, non_blocking=True)
        prim.prim.execute(strm, bufs[0][3])  # the set whose src was just copied in
        dst_host.copy_(dst, non_blocking=True)
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / e2e_steps
    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = [float(x) for x in t.tolist()]
    if rank == 0:
        pk = peaks()
        ms = total_ms / args.steps
        full_gb, launch_gb = (K * N * 5 + N * 4) / 1e9, (K * Nl * 5 + Nl * 4) / 1e9
        line = {"metric": "reorder_hbm_gbs", "value": full_gb / (ms * 1e-3), "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wkey, "kernel": pd.impl_info_str(),
                           "parallelism": "column blocks, one tensor per rank, no collective" if world > 1 else "single",
                           "l2": ("working set %.0f MB > 126 MB L2" % (launch_gb * 1e3)) if nsets == 1 else
                                 ("%d copies of all buffers rotated, %.0f MB per cycle > 126 MB L2" % (nsets, nsets * ws / 1e6)),
                           "e2e": "f32 src H2D from pinned memory and s8 dst D2H every step"},
                "roofline": {"bound": "hbm", "achieved": launch_gb / (ms * 1e-3), "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": launch_gb / (ms * 1e-3) / pk["hbm_gbs"], "traffic": dram_traffic(wkey, world),
                             "algorithmic_bytes": int(launch_gb * 1e9), "peak_source": pk["source"], "kernel_ms": ms},
                "e2e": {"value": full_gb / (e2e_ms * 1e-3), "unit": "GB/s", "h2d_bytes_per_step": int(K * Nl * 4),
                        "d2h_bytes_per_step": int(K * Nl), "ms_per_step": e2e_ms},
                "gpu_launches": int(launches), "clocks": clocks}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = reorder_cpu(K, N)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.workload == "reorder_quantize":
        run_reorder_bench(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_gpu(a)
