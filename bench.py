#!/usr/bin/env python
"""Benchmark of the PrivateUse1 operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass of every bandwidth-bound operator of the path over its
full-size seeded synthetic inputs (configurations 1-3 of BASELINE.json: the
fp32 op sweep, the index ops on the 128256x4096 bf16 table, the fused bf16
inference ops), called through the C ABI of libb200ops.so.

  value     algorithmic bytes of one pass / device time of one pass (GB/s),
            inputs resident in HBM, L2 flushed before every operator launch
  e2e       same metric with HOST buffers: pinned inputs copied H2D, the
            operator run, the result copied D2H, all inside the timed region
  roofline  the operator with the largest share of the pass, measured live
  ops       per-operator achieved GB/s against the measured copy bandwidth
  cpu_baseline / --impl reference: PyTorch CPU ATen (what the reference
            backend mirrors and checks itself against) on the host cores.

N > 1 (torchrun, one rank per GPU): the per-operator path does not shard --
every rank runs the same pass on its own GPU (replicas, no collective in the
data path) and the line reports the aggregate.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "torch-gcu_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "op_hbm_gbs"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
NSETS = 4


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", FALLBACK_HBM_GBS)), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------- workload --
class Op:
    def __init__(self, name, nbytes, launches, gpu_inputs, gpu_run, cpu_run, host_inputs, result):
        self.name = name
        self.bytes = nbytes          # algorithmic bytes per call
        self.launches = launches     # kernels (or copy nodes) per call
        self.gpu_inputs = gpu_inputs  # dict name -> device tensor (mutable, for e2e)
        self.gpu_run = gpu_run       # () -> None, enqueues on the current stream
        self.cpu_run = cpu_run       # () -> tensor, CPU ATen
        self.host_inputs = host_inputs  # dict name -> CPU tensor (pinned lazily)
        self.result = result         # () -> device tensor holding the result


def nbytes(*ts):
    return sum(t.numel() * t.element_size() for t in ts)


def make_data(scale=1.0):
    """Seeded CPU tensors of configs 1-3. scale < 1 shrinks the row counts (used
    by the bounded CPU sample only; the GPU arm always runs scale 1)."""
    import workloads
    R = lambda n: max(8, int(n * scale))  # noqa: E731
    return dict(sw=workloads.op_sweep(rows=R(4096)),
                ix=workloads.index_ops(vocab=R(128256), seq=R(2048), n_select=R(65536), gather_rows=R(8192),
                                       scatter_src=R(262144), scatter_dst=R(65536)),
                fu=workloads.fused_ops(tokens=R(16384), seq=R(2048)))


def build_ops(dev, data, want_gpu=True):
    """The operator list of one pass over `data`, with its own device buffers."""
    from oracle import aten_cpu as cpu  # used ONLY inside the cpu_run closures (CPU baseline leg)
    ops_mod = None
    if want_gpu:
        import b200ops as ops_mod
    out = []
    import ctypes
    cd, ci64, ci32, csz = ctypes.c_double, ctypes.c_int64, ctypes.c_int32, ctypes.c_size_t

    def i64s(v):
        return (ctypes.c_int64 * len(v))(*v)

    def B(name, *a, keep=()):
        # pre-marshalled C-ABI call (GPU arm only; the CPU arm never invokes it)
        return ops_mod.bind(name, *a, keep=keep) if want_gpu else None

    def wsa(w_):
        return ops_mod.ws_args(w_) if want_gpu else (None, None)

    def to_dev(d):
        if not want_gpu:
            import collections
            return collections.defaultdict(lambda: None)
        return {k: v.to(dev) for k, v in d.items() if torch.is_tensor(v)}

    # ---- config 1: fp32 op sweep ------------------------------------------
    sw = data["sw"]
    a, b, w, bias = sw["a"], sw["b"], sw["weight"], sw["bias"]
    rows, cols = a.shape
    g = to_dev(dict(a=a, b=b, w=w, bias=bias))
    if want_gpu:
        o32 = torch.empty_like(g["a"])
        o16 = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
        a16 = g["a"].to(torch.bfloat16)
        osum = torch.empty(rows, device=dev)
        mean = torch.empty(rows, device=dev)
        rstd = torch.empty(rows, device=dev)
    else:
        o32 = o16 = a16 = osum = mean = rstd = None
    a16_cpu = a.to(torch.bfloat16)
    out.append(Op("add", 3 * nbytes(a), 1, g, B("add", o32, g["a"], g["b"], cd(1.0)),
                  lambda: cpu.add(a, b), dict(a=a, b=b), lambda: o32))
    out.append(Op("mul", 3 * nbytes(a), 1, g, B("mul", o32, g["a"], g["b"]),
                  lambda: cpu.mul(a, b), dict(a=a, b=b), lambda: o32))
    out.append(Op("silu", 2 * nbytes(a), 1, g, B("silu", o32, g["a"]),
                  lambda: cpu.silu(a), dict(a=a), lambda: o32))
    out.append(Op("cast_f32_bf16", nbytes(a) + nbytes(a) // 2, 1, g, B("copy", o16, g["a"]),
                  lambda: cpu.cast(a, torch.bfloat16), dict(a=a), lambda: o16))
    g16 = dict(a=a16)  # a16 is None on the CPU arm
    out.append(Op("cast_bf16_f32", nbytes(a) + nbytes(a) // 2, 1, g16, B("copy", o32, g16["a"]),
                  lambda: cpu.cast(a16_cpu, torch.float32), dict(a=a16_cpu), lambda: o32))
    out.append(Op("sum_lastdim", nbytes(a) + rows * 4, 1, g, B("sum", osum, g["a"], i64s([1]), ci32(1), ci32(0), None, csz(0)),
                  lambda: cpu.sum_dim(a, [-1]), dict(a=a), lambda: osum))
    out.append(Op("softmax_lastdim", 2 * nbytes(a), 1, g, B("softmax", o32, g["a"], ci64(1)),
                  lambda: cpu.softmax(a, -1), dict(a=a), lambda: o32))
    out.append(Op("layer_norm", 2 * nbytes(a) + 2 * cols * 4 + 2 * rows * 4, 1, g,
                  B("native_layer_norm", o32, mean, rstd, g["a"], ci64(rows), ci64(cols), g["w"], g["bias"], cd(1e-5)),
                  lambda: cpu.native_layer_norm(a, (cols,), w, bias, 1e-5)[0], dict(a=a, w=w, bias=bias),
                  lambda: o32))

    # ---- config 2: index ops ------------------------------------------------
    ix = data["ix"]
    table, ids, sel = ix["table"], ix["ids"], ix["select_idx"]
    gsrc, gidx, svals, srows = ix["gather_src"], ix["gather_idx"], ix["scatter_vals"], ix["scatter_rows"]
    n_dst, scols = ix["scatter_dst"], ix["scatter_cols"]
    gi = to_dev(dict(table=table, ids=ids.reshape(-1), sel=sel, gsrc=gsrc, gidx=gidx, svals=svals, srows=srows))
    hidden = table.shape[1]
    zeros_cpu = torch.zeros(n_dst, scols)
    if want_gpu:
        emb_out = torch.empty(ids.numel(), hidden, dtype=torch.bfloat16, device=dev)
        sel_out = torch.empty(sel.numel(), hidden, dtype=torch.bfloat16, device=dev)
        gat_out = torch.empty_like(gi["gsrc"])
        gi["zeros"] = torch.zeros(n_dst, scols, device=dev)
        sc_out = torch.empty(n_dst, scols, device=dev)
        sidx = gi["srows"][:, None].expand(-1, scols)
        ws = torch.empty(ops_mod.scatter_add_workspace_size(gi["zeros"], 0, sidx, gi["svals"]), dtype=torch.uint8,
                         device=dev)
        ip_self = torch.zeros(n_dst, scols, device=dev)

        _ip = B("index_put", ip_self, gi["srows"], gi["svals"], ci32(1), *wsa(ws), keep=(ws,))

        def run_index_put():
            ip_self.zero_()  # restore the accumulator (a memset node, counted as a launch)
            _ip()
    else:
        emb_out = sel_out = gat_out = sc_out = sidx = ws = ip_self = run_index_put = None
    out.append(Op("embedding", 2 * ids.numel() * hidden * 2 + nbytes(ids), 1, gi,
                  B("index_select", emb_out, gi["table"], ci64(0), gi["ids"]),
                  lambda: cpu.embedding(table, ids), dict(table=table, ids=ids.reshape(-1)), lambda: emb_out))
    out.append(Op("index_select", 2 * sel.numel() * hidden * 2 + nbytes(sel), 1, gi,
                  B("index_select", sel_out, gi["table"], ci64(0), gi["sel"]),
                  lambda: cpu.index_select(table, 0, sel), dict(table=table, sel=sel), lambda: sel_out))
    out.append(Op("gather", nbytes(gidx) + 2 * nbytes(gsrc), 1, gi,
                  B("gather", gat_out, gi["gsrc"], ci64(1), gi["gidx"]),
                  lambda: cpu.gather(gsrc, 1, gidx), dict(gsrc=gsrc, gidx=gidx), lambda: gat_out))
    sc_bytes = nbytes(svals) + nbytes(srows) + 2 * n_dst * scols * 4
    out.append(Op("scatter_add", sc_bytes, 7, gi,
                  B("scatter_add", sc_out, gi["zeros"], ci64(0), sidx, gi["svals"], *wsa(ws), keep=(ws,)),
                  lambda: cpu.scatter_add(zeros_cpu, 0, srows[:, None].expand(-1, scols), svals),
                  dict(svals=svals, srows=srows, zeros=zeros_cpu), lambda: sc_out))
    out.append(Op("index_put_accumulate", sc_bytes, 8, gi, run_index_put,
                  lambda: cpu.index_put(zeros_cpu, [srows], svals, True),
                  dict(svals=svals, srows=srows), lambda: ip_self))

    # ---- config 3: fused bf16 inference ops ---------------------------------
    fu = data["fu"]
    x, res, wn, q, k, gate, up, cos, sin = (fu[n] for n in ("x", "res", "weight", "q", "k", "gate", "up", "cos", "sin"))
    gf = to_dev(dict(x=x, res=res, wn=wn, q=q, k=k, gate=gate, up=up, cos=cos, sin=sin))
    if want_gpu:
        y = torch.empty_like(gf["x"])
        hres = torch.empty_like(gf["x"])
        qo, ko = torch.empty_like(gf["q"]), torch.empty_like(gf["k"])
        so = torch.empty_like(gf["gate"])

        _rq = B("rope", qo, gf["q"], gf["cos"], gf["sin"], None)
        _rk = B("rope", ko, gf["k"], gf["cos"], gf["sin"], None)

        def run_rope():
            _rq()
            _rk()
    else:
        y = hres = qo = ko = so = run_rope = None
    out.append(Op("rms_norm_residual", 4 * nbytes(x) + nbytes(wn), 1, gf,
                  B("rms_norm_residual", y, hres, gf["x"], gf["res"], gf["wn"], cd(1e-6)),
                  lambda: cpu.rms_norm_residual(x, res, wn, 1e-6)[0], dict(x=x, res=res, wn=wn), lambda: y))
    out.append(Op("rope_q_k", 2 * (nbytes(q) + nbytes(k)), 2, gf, run_rope,
                  lambda: (cpu.rope(q, cos, sin), cpu.rope(k, cos, sin))[0], dict(q=q, k=k, cos=cos, sin=sin),
                  lambda: qo))
    out.append(Op("swiglu", 3 * nbytes(gate), 1, gf, B("swiglu", so, gf["gate"], gf["up"]),
                  lambda: cpu.swiglu(gate, up), dict(gate=gate, up=up), lambda: so))
    return out


# ------------------------------------------------------------------- clocks --
class ClockSampler:
    """Samples nvidia-smi during the timed region (read-only query)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ GPU arm --
def run_gpu(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    import b200ops
    b200ops.lib()  # fail loudly if the kernel library is missing
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    data = make_data()
    # NSETS independent copies of every operator's buffers, used round-robin, so
    # that a launch never finds its operands in the 126 MB L2: between two uses
    # of one buffer set the other sets stream >= 3x its footprint (>= 200 MB
    # even for the smallest operator).
    sets = [build_ops(dev, data) for _ in range(NSETS)]
    if args.only:
        keep = set(args.only.split(","))
        sets = [[op for op in st if op.name in keep] for st in sets]
    ops = sets[0]
    stream = torch.cuda.current_stream()

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_pass(per_op_ms):
        # one event pair around NSETS back-to-back launches of the same operator
        for i in range(len(ops)):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            for st in sets:
                st[i].gpu_run()
            e.record(stream)
            per_op_ms[i].append((s, e))

    for _ in range(max(args.warmup, 3)):
        timed_pass([[] for _ in ops])
    barrier()
    events = [[] for _ in ops]
    with ClockSampler(local) as clocks:
        for _ in range(args.steps):
            timed_pass(events)
        barrier()
    op_ms = [sum(s.elapsed_time(e) for s, e in ev) / args.steps / NSETS for ev in events]
    pass_ms = sum(op_ms)
    pass_bytes = sum(op.bytes for op in ops)

    # end to end: host buffers in, result out, per operator, inside the timing
    pinned = [{k: v.contiguous().pin_memory() for k, v in op.host_inputs.items()} for op in ops]
    host_out = [torch.empty(op.result().shape, dtype=op.result().dtype).pin_memory() for op in ops]
    h2d = sum(nbytes(*p.values()) for p in pinned)
    d2h = sum(nbytes(t) for t in host_out)

    def e2e_pass():
        for op, pin, ho in zip(ops, pinned, host_out):
            for kname, v in pin.items():
                op.gpu_inputs[kname].view(-1).copy_(v.view(-1), non_blocking=True)
            op.gpu_run()
            ho.copy_(op.result(), non_blocking=True)
    e2e_pass()
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(stream)
    for _ in range(args.steps):
        e2e_pass()
    e.record(stream)
    barrier()
    e2e_ms = s.elapsed_time(e) / args.steps

    t = torch.tensor([pass_ms, e2e_ms], dtype=torch.float64, device=dev)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    pass_ms_max, e2e_ms_max = t.tolist()

    if rank == 0:
        peak, peak_kind = measured_peaks()
        table = []
        for op, ms in zip(ops, op_ms):
            gbs = op.bytes / ms / 1e6
            table.append({"op": op.name, "ms": round(ms, 4), "bytes": op.bytes, "gbs": round(gbs, 1),
                          "frac_of_measured": round(gbs / peak, 3), "frac_of_8tbs": round(gbs / NOMINAL_HBM_GBS, 3),
                          "launches": op.launches})
        top = max(range(len(ops)), key=lambda i: op_ms[i])
        top_gbs = ops[top].bytes / op_ms[top] / 1e6
        value = world * pass_bytes / pass_ms_max / 1e6
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(pass_ms_max, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32+bf16", "data": "synthetic",
            "config": {"workload": "configs[0..2]: fp32 (4096,4096) op sweep + index ops on bf16 (128256,4096) "
                                   "table + fused bf16 RMSNorm/RoPE/SwiGLU, one pass of all 16 operators",
                       "l2": "%d rotating buffer sets per operator (no launch re-reads data resident in L2)" % NSETS, "parallelism": "replicas" if world > 1 else "1gpu",
                       "peak": "%s copy bandwidth %.1f GB/s" % (peak_kind, peak)},
            "clocks": clocks.summary(),
            "e2e": {"value": round(world * pass_bytes / e2e_ms_max / 1e6, 2), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps * NSETS * sum(op.launches for op in ops),
            "roofline": {"bound": "hbm", "kernel": ops[top].name, "achieved": round(top_gbs, 1), "peak": peak,
                         "unit": "GB/s", "frac": round(top_gbs / peak, 3), "traffic": None,
                         "peak_kind": peak_kind},
            "ops": table,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(pass_bytes, sample_steps=1)
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------ CPU arm --
def cpu_pass(ops):
    t0 = time.perf_counter()
    for op in ops:
        op.cpu_run()
    return time.perf_counter() - t0


def cpu_baseline(pass_bytes_full, sample_steps=1, scale=0.25):
    """CPU ATen over a bounded sample: the same 16 operators on `scale` of the rows."""
    torch.set_num_threads(os.cpu_count() or 1)
    ops = build_ops(None, make_data(scale), want_gpu=False)
    sample_bytes = sum(op.bytes for op in ops)
    cpu_pass(ops)  # warm-up
    dt = min(cpu_pass(ops) for _ in range(max(1, sample_steps)))
    return {"value": round(sample_bytes / dt / 1e9, 3), "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port", "sample": "all 16 operators on %.0f%% of the rows of each config (%.2f GB algorithmic), "
            "PyTorch CPU ATen, best of %d" % (scale * 100, sample_bytes / 1e9, max(1, sample_steps))}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    scale = 0.25
    ops = build_ops(None, make_data(scale), want_gpu=False)
    sample_bytes = sum(op.bytes for op in ops)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_pass(ops)
    steps = max(1, min(args.steps, 5))
    dts = [cpu_pass(ops) for _ in range(steps)]
    dt = sum(dts) / len(dts)
    value = round(sample_bytes / dt / 1e9, 3)
    sample = ("PyTorch CPU ATen (the implementation the reference mirrors and checks against; its own kernels are a "
              "closed vendor library), all 16 operators on %.0f%% of the rows of each config (%.2f GB algorithmic "
              "per step)" % (scale * 100, sample_bytes / 1e9))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": max(1, min(args.warmup, 2)), "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32+bf16", "data": "synthetic",
            "config": {"workload": "configs[0..2] operator pass (bounded sample)"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only", default="", help="comma-separated operator names (profiling aid)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
