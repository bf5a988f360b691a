"""Benchmark of the quantized matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one execution of the workload's matmul through the library's C API.
Default workload: the fp8 prefill GEMM (e4m3 [4096,4096] x e4m3 [4096,14336]
-> bf16, per-tensor scales, bf16 bias).  For N > 1 (launched under torchrun)
the weights are sharded by output columns, every rank computes its N-slice
and the slices are assembled with an NCCL all-gather; the total problem is
fixed, so scaling is "strong".

One JSON line is printed by rank 0:
  value     whole-job throughput with inputs resident in HBM, timed with CUDA
            events on the launching stream (max over ranks)
  e2e       the same metric with the step's src copied from pinned host memory
            and the dst read back to the host inside the timed region
  roofline  algorithmic work of one launch / its average duration, against the
            measured peak in MEASURED_PEAKS.json
  cpu_baseline  the reference's CPU matmul on a bounded sample of the workload
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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="fp8_prefill", choices=sorted(WORKLOADS) + ["reorder_quantize"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--kernel", default=None, help="pin an implementation by name substring")
    ap.add_argument("--M", type=int, default=None, help="override M (decode: 1, 8 or 32)")
    ap.add_argument("--K", type=int, default=None)
    ap.add_argument("--N", type=int, default=None)
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def make_problem(args):
    kw = {}
    if args.M is not None:
        kw["total_M" if args.workload == "moe_grouped" else "M"] = args.M
    if args.K is not None:
        kw["K"] = args.K
    if args.N is not None:
        kw["N"] = args.N
    if args.small:
        small = {"fp8_prefill": dict(M=2048, K=2048, N=8192), "int8_postops": dict(M=1024, K=2048, N=4096),
                 "int4_decode": dict(K=8192, N=16384), "moe_grouped": dict(total_M=2048, K=2048, N=4096, experts=16),
                 "int8_zp": {}}[args.workload]
        small.update(kw)
        kw = small
    return WORKLOADS[args.workload][0](**kw)


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
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
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

    name = args.workload
    _, metric, unit, bound, dtype = WORKLOADS[name]
    full = make_problem(args)
    p = sharding.shard(full, rank, world)

    eng = api.engine(api.engine.kind.gpu, local_rank)
    tstream = torch.cuda.current_stream()
    strm = api.stream(eng, tstream.cuda_stream)
    # A step must not find its inputs in the 126 MB L2 left there by the step before: when one
    # rank's working set is not clearly larger than L2 (decode, and every workload once it is
    # sharded), consecutive steps use different copies of all buffers, enough of them that a
    # cycle through the copies moves 2.5 x L2.
    L2_BYTES = 126e6
    ws = float(p.algorithmic_bytes())
    nsets = 1 if ws > 1.5 * L2_BYTES else int(min(8, max(2, np.ceil(2.5 * L2_BYTES / max(ws, 1.0)))))
    sets = []
    for _ in range(nsets):
        ptrs_s, keep_s = device_buffers(p, torch, dev)
        sets.append((Prepared(p, eng, args.kernel).bind_device(ptrs_s), keep_s))
    prep, keep = sets[0]
    preps = [s[0] for s in sets]
    l2_note = ("working set %.0f MB > 126 MB L2" % (ws / 1e6)) if nsets == 1 else \
        ("%d copies of all buffers rotated, %.0f MB per cycle %s 126 MB L2" %
         (nsets, nsets * ws / 1e6, ">" if nsets * ws > L2_BYTES else "< (L2-resident workload)"))
    elem = {W.BF16: torch.bfloat16, W.F16: torch.float16, W.F32: torch.float32, W.S32: torch.int32,
            W.S8: torch.int8, W.U8: torch.uint8}[p.dst_dt]
    rows_per_rank = None
    if full.offsets is not None and world > 1:
        ends = full.offsets.astype(np.int64)
        rows_per_rank = []
        for r in range(world):
            e0, e1 = sharding.expert_range(full.groups, r, world)
            rows_per_rank.append(int((ends[e1 - 1] if e1 > e0 else (ends[e0 - 1] if e0 else 0)) - (ends[e0 - 1] if e0 else 0)))

    def gather(i=0):
        if world == 1:
            return None
        local = sets[i % nsets][1]["dst"].view(elem).view(p.M, p.N)
        # the gathered result stays in the collective's blocked layout ([rank][M][N/g] column
        # slices, [rank][rows][N] expert blocks): no interleaving copy inside the step
        if rows_per_rank is not None:
            return sharding.gather_rows_blocked(local, rows_per_rank)
        return sharding.gather_columns_blocked(local, full.N, world)

    def step(i):
        preps[i % nsets].execute(strm)
        return gather(i)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()

    # ---- device-timed region: inputs resident in HBM
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    launches0 = api.launch_count()
    k_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        k_ev[i][0].record()
        preps[i % nsets].execute(strm)
        k_ev[i][1].record()
        gather(i)
    e1.record()
    barrier()
    launches = api.launch_count() - launches0
    total_ms = e0.elapsed_time(e1)
    # The timed region lasts milliseconds, less than one nvidia-smi sampling period: the same
    # step is repeated (untimed) for about 1.5 s so that the sampler sees the clocks under this load.
    if sampler:
        t_end = time.time() + 1.5
        i = 0
        while time.time() < t_end:
            for _ in range(50):
                preps[i % nsets].execute(strm)
                i += 1
            torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["sampled"] = "over the timed region and a 1.5 s untimed repeat of the same step"
    kernel_ms = float(np.mean([a.elapsed_time(b) for a, b in k_ev]))

    # ---- end-to-end: src from pinned host memory, dst back to the host, every step
    src_host = torch.from_numpy(p.src.data.view(np.uint8).reshape(-1).copy()).pin_memory()
    g0 = gather()
    out_bytes = int(g0.numel() * g0.element_size()) if g0 is not None else keep["dst"].numel()
    dst_host = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step(i):
        k = sets[i % nsets][1]
        k["src"].copy_(src_host, non_blocking=True)
        g = step(i)
        res = k["dst"] if g is None else g.reshape(-1).view(torch.uint8)
        dst_host[:res.numel()].copy_(res, non_blocking=True)

    e2e_step(0)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / e2e_steps

    t = torch.tensor([total_ms, kernel_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kernel_ms, e2e_ms = [float(x) for x in t.tolist()]
    ms_per_step = total_ms / args.steps

    if rank == 0:
        pk = peaks()
        if bound == "hbm":
            work_full, work_launch, per = full.algorithmic_bytes() / 1e9, p.algorithmic_bytes() / 1e9, 1e-3
            peak, runit = pk["hbm_gbs"], "GB/s"
        else:
            work_full, work_launch, per = full.ops() / 1e12, p.ops() / 1e12, 1e-3
            # fp8 / int8 tensor peak: twice the measured dense bf16 figure (the
            # 8-bit MMA rate is twice the 16-bit one); bf16 workloads use it as is
            mult = 1.0 if dtype == "bf16" else 2.0
            peak, runit = mult * pk["bf16_tflops"], "TFLOP/s"
        value = work_full / (ms_per_step * per)
        achieved = work_launch / (kernel_ms * per)
        wkey = "%s M=%d K=%d N=%d" % (name, full.M, full.K, full.N)
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": wkey,
                       "kernel": prep.impl, "parallelism": ("%s x%d + NCCL all-gather into [rank][M][N/g] blocks"
                                       % ("expert-shard" if full.offsets is not None else "n-shard", world))
                       if world > 1 else "single",
                       "l2": l2_note,
                       "e2e": "src H2D from pinned memory and dst D2H every step; weights resident"},
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": runit,
                         "frac": achieved / peak, "traffic": dram_traffic(wkey, world),
                         "traffic_unit": "bytes per launch (ncu, profiles/dram_traffic.json)",
                         "algorithmic_bytes": int(p.algorithmic_bytes()), "peak_source": pk["source"],
                         "kernel_ms": kernel_ms},
            "e2e": {"value": work_full / (e2e_ms * per), "unit": unit,
                    "h2d_bytes_per_step": int(src_host.numel()), "d2h_bytes_per_step": int(out_bytes),
                    "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(full, name, bound, seconds=15.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------- CPU reference arm
def cpu_sample(full, name, target_s):
    """A bounded sample of the workload for the CPU: a seeded subset of src
    rows (dense) or a smaller token count (grouped); K, N and every attribute
    are those of the full problem.  Sized from a short probe so one execution
    takes about target_s seconds."""
    if full.offsets is not None:
        def make(m):
            return W.moe_grouped(total_M=m, K=full.K, N=full.N, experts=full.groups), "total_M=%d of %d" % (m, full.M)
    else:
        def make(m):
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
    os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))
    make = cpu_sample(full, name, seconds)
    m = 1 if full.offsets is None else full.groups
    m = min(m, full.M)
    p, what = make(m)
    ms, impl, kind = time_cpu(p, 1)
    # grow the sample until one execution is worth timing, within the budget
    while ms * 4 < seconds * 1e3 / (iters + 1) and m < full.M:
        m = min(full.M, m * 4)
        p, what = make(m)
        ms, impl, kind = time_cpu(p, 1)
    if ms * (iters + 1) < seconds * 1e3:
        ms2, impl, kind = time_cpu(p, iters)
        ms = min(ms, ms2)
    work = (p.algorithmic_bytes() / 1e9) if bound == "hbm" else (p.ops() / 1e12)
    return {"value": work / (ms * 1e-3), "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
            "cores": int(os.environ["OMP_NUM_THREADS"]), "kind": kind, "impl": impl,
            "ms": ms, "sample": "%s, K=%d N=%d, %.1f ms per execution" % (what, p.K, p.N, ms)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    _, metric, unit, bound, dtype = WORKLOADS[name]
    full = make_problem(args)
    budget = 20.0
    base = cpu_baseline(full, name, bound, seconds=budget, iters=max(1, min(args.steps, 3)))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    line = {"impl": "reference", "metric": metric, "value": base["value"], "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": "%s M=%d K=%d N=%d" % (name, full.M, full.K, full.N), "sample": base["sample"]},
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
    os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))
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
    return {"value": gb / best, "unit": "GB/s", "cores": int(os.environ["OMP_NUM_THREADS"]),
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
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                              "data": "synthetic", "config": {"workload": wkey, "sample": base["sample"]},
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
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
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
