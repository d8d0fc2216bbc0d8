#!/usr/bin/env python
"""Benchmark of the Granite 4.2 8B layer-glue kernels on B200.

Workload (the box-scale sweep the headline metric is quoted on): 65536 token rows, sharded
by rows over the N GPUs of one node, each shard running the full 40-layer glue sequence
(per layer: residual add + RMSNorm -> FP8, RoPE + int8 paged KV write, residual add +
RMSNorm -> FP8, SwiGLU -> FP8; then the final norm) on seeded random bf16 activations of
Granite 8B shape. No collective on the data path; NCCL only carries the timing reduction.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

prints ONE JSON line (rank 0). `value` is whole-job tokens/s with inputs resident in HBM;
`roofline` is the dominant op's algorithmic bytes over its CUDA-event time; `e2e` is the same
sequence through the host-buffer C-ABI entry point (host<->device copies inside the timed
region); `cpu_baseline` is the reference's CPU formulation on this box's cores.
`--impl reference` times only that CPU formulation and prints the reference arm's line.
After the timed regions every rank's outputs are checked (`check` in the line): the ranks
all_gather a fingerprint of what their last step left behind, and rank 0 rebuilds every other
rank's shard from its seed, runs it alone and compares bit for bit.
`--sweep-only` leaves out the other shapes (short profiler captures); `--traffic-from-ncu CSV`
is a converter, not a benchmark: it condenses an ncu raw CSV into the DRAM-traffic file the
roofline's `traffic` is read from.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOTAL_TOKENS = 65536
METRIC = "layer_glue_tokens_per_s"
UNIT = "tokens/s"
WORKLOAD = ("box-scale sweep: 65536 tokens row-sharded, 40-layer glue sequence "
            "(2x add+RMSNorm->FP8, RoPE+int8 paged KV, SwiGLU->FP8 per layer, final norm), "
            "Granite 8B shapes H4096/I12800/32q/8kv/d128")


def shard_bounds(total: int, world: int, rank: int):
    """Contiguous row range of `rank`: GPU g of N takes rows [g * total / N, (g + 1) * total / N)."""
    if total % world:
        raise SystemExit(f"the GPU count must divide {total}")
    per = total // world
    return rank * per, (rank + 1) * per


def max_over_ranks(value: float, device):
    """Max of a per-rank duration over the process group (the only collective in the bench; it
    carries a timing, never data of the path). device None: CPU tensor (gloo)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, MEASURED_PEAKS.json absent)"


# ------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        sm, smax, reasons = [], None, set()
        for ts, line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                clock, cmax = float(f[1]), float(f[2])
            except ValueError:
                continue
            smax = cmax
            if t0 - 0.05 <= ts <= t1 + 0.15:
                sm.append(clock)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm:  # region shorter than one sample: take what there is
            sm = [float(l.split(",")[1]) for _, l in self.lines[-3:] if len(l.split(",")) > 2] or [0.0]
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------- CPU arm
def np_f32_to_bf16(a):
    import numpy as np
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


class CpuGlue:
    """The same layer sequence on the host cores, through the oracle library (the reference's
    own compiled host code when oracle/_ref is present, else the C port). Rows are split over
    threads; the per-tensor FP8 amax is the max of the threads' maxima."""

    def __init__(self, rows: int, layers: int, threads: int):
        import numpy as np
        from oracle import g4_oracle
        self.np, self.g4 = np, g4_oracle
        self.kind = "reference" if g4_oracle.available("reference") else "port"
        self.lib = g4_oracle.load(self.kind)
        self.rows, self.layers, self.threads = rows, layers, max(1, min(threads, rows))
        rng = np.random.default_rng(0)

        def randn(*shape):
            return np_f32_to_bf16(rng.standard_normal(shape, dtype=np.float32))
        H, I, self.Hq, self.Hk, self.d = 4096, 12800, 32, 8, 128
        self.buf = {"y_attn": randn(rows, H), "y_mlp": randn(rows, H), "qkv": randn(rows, 6144),
                    "gate": randn(rows, I), "up": randn(rows, I)}
        self.h0 = randn(rows, H)
        self.w = np_f32_to_bf16(1.0 + 0.02 * rng.standard_normal((2, H), dtype=np.float32))
        self.cos, self.sin = self.lib.rope_tables(1e7, 128, rows)
        self.pos = np.arange(rows, dtype=np.int32)
        self.caches = (np.zeros((8, rows, 128), np.int8), np.zeros((8, rows, 128), np.int8),
                       np.zeros((8, rows), np.float32), np.zeros((8, rows), np.float32))

    def _quant(self, x):
        lib, par = self.lib, self.g4.parallel_rows
        amax = max(par(lambda lo, hi: lib.amax_bf16(x[lo:hi]), self.rows, self.threads))
        scale = lib.fp8_scale_from_amax(amax)
        par(lambda lo, hi: lib.quant_fp8_with_scale(x[lo:hi], scale), self.rows, self.threads)

    def step(self):
        lib, par, b = self.lib, self.g4.parallel_rows, self.buf
        h = self.h0
        for _ in range(self.layers):
            for y, w in ((b["y_attn"], self.w[0]), (b["y_mlp"], self.w[1])):
                parts = par(lambda lo, hi: lib.add_rmsnorm(y[lo:hi], h[lo:hi], w, 1e-5, 0.22), self.rows,
                            self.threads)
                h = self.np.concatenate([p[0] for p in parts])
                self._quant(self.np.concatenate([p[1] for p in parts]))
                if y is b["y_attn"]:
                    par(lambda lo, hi: lib.rope_kv_int8(b["qkv"][lo:hi], self.cos, self.sin, self.pos[lo:hi],
                                                        self.pos[lo:hi], self.Hq, self.Hk, self.d, self.rows, 0,
                                                        self.caches), self.rows, self.threads)
            act = self.np.concatenate(par(lambda lo, hi: lib.swiglu(b["gate"][lo:hi], b["up"][lo:hi]),
                                          self.rows, self.threads))
            self._quant(act)
        par(lambda lo, hi: lib.add_rmsnorm(h[lo:hi], None, self.w[0], 1e-5, 1.0, want_h=False), self.rows,
            self.threads)


def cpu_tokens_per_s(rows: int, layers: int, threads: int, steps: int, warmup: int):
    cpu = CpuGlue(rows, layers, threads)
    for _ in range(warmup):
        cpu.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.step()
    dt = time.perf_counter() - t0
    # tokens/s of the full 40-layer sequence: a step of `layers` layers stands for layers/40 of it
    tokens_per_s = rows * steps / dt * (layers / 40.0)
    return tokens_per_s, dt, cpu


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    threads = host_threads()
    rows = int(os.environ.get("G4_BENCH_CPU_ROWS", "256"))
    tps, dt, cpu = cpu_tokens_per_s(rows, 40, threads, args.steps, args.warmup)
    sample = (f"{rows} of the 65536 token rows through all 40 layers + final norm per step, rows split "
              f"over {cpu.threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cpu.threads, "kind": cpu.kind,
                         "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, rank: int, local_rank: int, world: int):
    import torch
    import torch.distributed as dist
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi, glue

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU fallback for the kernels)")
    capi.lib()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL writes its version banner (and anything NCCL_DEBUG asks for) to stdout when the
        # communicator is created, i.e. at the first collective; stdout is reserved for the one JSON
        # line, so file descriptor 1 points at stderr until that has happened.
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize(device)
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    shapes = glue.GraniteShapes()
    lo, hi = shard_bounds(TOTAL_TOKENS, world, rank)
    rows = int(os.environ.get("G4_BENCH_ROWS", hi - lo))  # override only for profiling
    total_tokens = rows * world
    prof_layers = os.environ.get("G4_BENCH_LAYERS")  # fewer layers: only for short profiler captures
    workspace = os.environ.get("G4_BENCH_WORKSPACE", "1") != "0"  # 0: the scratch-free second sweeps
    seq = glue.GlueSequence(rows, shapes, device=device, seed=rank, sets=2,
                            layers=int(prof_layers) if prof_layers else None, workspace=workspace)
    seq.reset()
    stream = torch.cuda.current_stream(device)
    warmup = max(args.warmup, 3)

    def sync_all():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    for _ in range(warmup):
        seq.run_fast()
    sync_all()

    # ---- timed region: K steps, CUDA events on the launching stream ---------------------
    gpu_index = local_rank
    if "CUDA_VISIBLE_DEVICES" in os.environ:
        try:
            gpu_index = int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
        except ValueError:
            pass
    sampler = ClockSampler(gpu_index)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    seq.launches = 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    wall0 = time.time()
    ev0.record(stream)
    for _ in range(args.steps):
        seq.run_fast()
    ev1.record(stream)
    sync_all()
    wall1 = time.time()
    launches = seq.launches
    ms = ev0.elapsed_time(ev1)

    # ---- a second, instrumented timed region: an event pair around every op ----------------
    op_events = {"add_rmsnorm_fp8": [], "rope_kv_int8": [], "swiglu_fp8": [], "final_norm": []}
    op_steps = min(args.steps, 3)
    evo0, evo1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    evo0.record(stream)
    for _ in range(op_steps):
        timed_step(seq, op_events, stream)
    evo1.record(stream)
    sync_all()
    wall2 = time.time()
    clocks = sampler.stop(wall0, wall2) if rank == 0 else None
    ms_ops = evo0.elapsed_time(evo1)

    ms_max = max_over_ranks(ms, device)
    status = capi.lib().device_status()

    # ---- the embedding gather (a1; not part of the sweep) and the small, latency-bound shapes ----
    extras = small_shapes_and_embed(seq, rows, device, stream) if rank == 0 and not args.sweep_only else None

    # ---- end to end through the host-buffer entry points ------------------------------------
    e2e = None
    if not args.no_e2e:
        e2e_ms_own, h2d, d2h, e2e_steps, placement = run_e2e(seq, rows, device, min(args.steps, 2))
        e2e_ms = max_over_ranks(e2e_ms_own, device)
        e2e = {"value": total_tokens * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e2e_steps,
               "rank0_h2d_gbs": h2d * e2e_steps / (e2e_ms_own * 1e-3) / 1e9,
               "rank0_d2h_gbs": d2h * e2e_steps / (e2e_ms_own * 1e-3) / 1e9, "placement": placement,
               "timing": "host clock around enqueue + granite4_host_glue_sync, max over ranks",
               "api": "granite4_host_glue_layer x layers + granite4_host_glue_final_norm, pinned "
                      "host buffers; the residual stream and the KV pool stay on the device"}

    check = check_outputs(seq, rows, rank, world, device, shapes, prof_layers, workspace)

    if rank == 0:
        peak, peak_src = load_peaks()
        bpr = glue.bytes_per_row(shapes)
        traffic = load_traffic()
        ops = {}
        for name, evs in op_events.items():
            dur = [a.elapsed_time(b) for a, b in evs]
            per_row = bpr[name]
            mean_ms = statistics.mean(dur)
            ops[name] = {"launches": len(dur), "mean_us": mean_ms * 1e3,
                         "share": sum(dur) / (ms_ops if ms_ops > 0 else 1.0),
                         "achieved_gbs": per_row * rows / (mean_ms * 1e-3) / 1e9,
                         "frac": per_row * rows / (mean_ms * 1e-3) / 1e9 / peak,
                         "frac_of_nominal_8000": per_row * rows / (mean_ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
                         "bytes_per_row": per_row,
                         "dram_bytes_per_row": traffic.get(name)}
        dominant = max(ops, key=lambda k: ops[k]["share"])
        tokens_per_s = total_tokens * args.steps / (ms_max * 1e-3)
        per_token = (seq.layers * (2 * bpr["add_rmsnorm_fp8"] + bpr["rope_kv_int8"] + bpr["swiglu_fp8"]) +
                     bpr["final_norm"])
        seq_gbs = per_token * total_tokens * args.steps / (ms_max * 1e-3) / 1e9 / world
        line = {
            "metric": METRIC, "value": tokens_per_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": rows, "total_tokens": total_tokens,
                       "layers": seq.layers, "parallelism": f"rows/{world}",
                       "fp8_sweep_scratch": workspace,
                       "l2": "inputs larger than L2: two rotated input sets, >= 1.1 GB touched per layer",
                       "bytes_per_token": per_token},
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": ops[dominant]["achieved_gbs"],
                         "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": ops[dominant]["frac"],
                         "traffic": traffic[dominant] * rows if dominant in traffic else None,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of the op's kernels "
                                           "from the committed profiler launch list, scaled by rows"
                                           if dominant in traffic else None,
                         "algorithmic_bytes_per_launch": ops[dominant]["bytes_per_row"] * rows,
                         "timing": f"event pair around each op, {op_steps} steps after the main region"},
            "sequence_roofline": {"achieved": seq_gbs, "unit": "GB/s per GPU", "frac": seq_gbs / peak},
            "ops": ops,
            "check": check,
            "clocks": clocks,
            "gpu_launches": launches,
            "device_status": status,
        }
        # CPU baseline on this box's cores (rank 0, N = 1 only), bounded sample
        if world == 1 and not args.no_cpu:
            threads = host_threads()
            c_rows = int(os.environ.get("G4_BENCH_CPU_ROWS", "256"))
            tps, dt, cpu = cpu_tokens_per_s(c_rows, 40, threads, 3, 1)
            line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cpu.threads, "kind": cpu.kind,
                                    "sample": f"{c_rows} token rows through all 40 layers + final norm, "
                                              f"3 steps after 1 warm-up, {dt:.1f} s"}
        line["e2e"] = e2e
        if extras is not None:
            line.update({"embed": extras["embed"], "small_shapes": extras["small"], "argmax": extras["argmax"],
                         "config2_decode_chain": extras["config2"], "config4_rope_kv": extras["config4"],
                         "attention_decode": extras["attention"], "decode_step": extras["decode_step"],
                         "gemm_fp8": extras["gemm"]})
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def check_outputs(seq, rows, rank, world, device, shapes, prof_layers, workspace):
    """After the timed regions, outside every timer: are the outputs the ranks computed the right
    ones? Each rank condenses what its last step left behind (GlueSequence.fingerprint: integer
    sums over every output buffer in full, plus the raw bits of 64 sample rows) and the ranks
    all_gather those fingerprints - the one data collective of the benchmark, and it carries
    results for checking, not data of the path. Rank 0 then rebuilds every other rank's shard
    from that rank's seed in buffers of its own, runs it alone, launch by launch instead of one
    library call per layer, and compares fingerprints bit for bit (same shard => same per-shard
    FP8 scales). With one GPU the rebuilt shard is rank 0's own."""
    import torch
    import torch.distributed as dist
    from granite4_b200 import glue
    seq.reset()
    seq.run_fast()
    torch.cuda.synchronize(device)
    mine = seq.fingerprint()
    prints = [mine]
    if world > 1:
        prints = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(prints, mine)
        torch.cuda.synchronize(device)
    if rank != 0:
        return None
    compared, equal = [], True
    for r in (range(1, world) if world > 1 else (0,)):
        other = glue.GlueSequence(rows, shapes, device=device, seed=r, sets=2,
                                  layers=int(prof_layers) if prof_layers else None, workspace=workspace)
        other.reset()
        other.run()
        torch.cuda.synchronize(device)
        same = bool(torch.equal(other.fingerprint(), prints[r]))
        compared.append(r)
        equal = equal and same
        del other
        torch.cuda.empty_cache()
    return {"ranks": world, "compared_ranks": compared, "rows": min(64, rows), "bytes_per_rank": mine.numel(),
            "covers": "sums over all rows of h, out, n_fp8, act_fp8, q_rot, KV pool and scales; bits of the "
                      "sample rows", "equal": equal}


NOMINAL_HBM_GBS = 8000.0  # the data-sheet figure the reference's target is stated against

TRAFFIC_FILE = os.path.join(ROOT, "profiles", "layer_kernels_dram_traffic.txt")


def op_of_kernel(kernel_name: str):
    """The op of the sweep a kernel (as the profiler names it) belongs to, or None."""
    if "add_rmsnorm_fast_kernel<0, 0>" in kernel_name:
        return "final_norm"
    if "add_rmsnorm" in kernel_name or "norm_encode_kernel" in kernel_name:
        return "add_rmsnorm_fp8"
    if "rope_kv" in kernel_name:
        return "rope_kv_int8"
    if "swiglu_kernel" in kernel_name:
        return "swiglu_fp8"
    return None


def traffic_from_ncu(csv_path: str, rows: int, out_path: str = TRAFFIC_FILE) -> dict:
    """Condense an `ncu --csv` launch list (one line per launch and metric; metrics
    dram__bytes_read.sum and dram__bytes_write.sum) of a sweep of `rows` token rows into DRAM
    bytes per launch of each op. Every kernel specialisation runs once per op, so an op's bytes
    are the sum over its kernels of each kernel's mean over its launches."""
    import csv
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    launches = {}  # (kernel name, launch id) -> bytes
    with open(csv_path, newline="") as f:
        rd = csv.DictReader(l for l in f if l.startswith('"'))
        for r in rd:
            if r["Metric Name"] in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
                key = (r["Kernel Name"], r["ID"])
                launches[key] = launches.get(key, 0.0) + float(r["Metric Value"].replace(",", "")) * scale[r["Metric Unit"]]
    per_kernel = {}
    for (name, _), v in launches.items():
        per_kernel.setdefault(name, []).append(v)
    ops = {}
    for name, vals in per_kernel.items():
        op = op_of_kernel(name)
        if op is not None:
            ops[op] = ops.get(op, 0.0) + sum(vals) / len(vals)
    with open(out_path, "w") as f:
        f.write("# DRAM bytes (read + written) per launch of each op of the layer sweep, from one profiler\n"
                "# launch list; written by: python bench.py --traffic-from-ncu <csv> --traffic-rows <rows>\n")
        f.write(f"rows {rows}\n")
        for op in sorted(ops):
            f.write(f"{op} {ops[op]:.0f}\n")
    return ops


def load_traffic():
    """{op: DRAM bytes per token row} from the committed profiler summary, or {} when it is absent."""
    if not os.path.isfile(TRAFFIC_FILE):
        return {}
    vals = {}
    with open(TRAFFIC_FILE) as f:
        for line in f:
            if line.startswith("#") or not line.strip():
                continue
            k, v = line.split()
            vals[k] = float(v)
    rows = vals.pop("rows", 0)
    return {k: v / rows for k, v in vals.items()} if rows else {}


def kernels_rope_tables(s, max_pos, device):
    from granite4_b200 import kernels
    return kernels.RopeTables(s.rope_theta, s.head_dim, max_pos, device)


def small_shapes_and_embed(seq, rows, device, stream):
    """(1) The embedding gather at the shard's row count on a Granite-size table (100352 x 4096,
    ids uniform, multiplier 12). (2) benchmark configurations 1-3: one decode row, the decode chain at 1
    and 8 rows replayed from a CUDA graph, one 500-row prefill layer - latency-bound shapes,
    reported in microseconds, not against the bandwidth roofline."""
    import torch
    from granite4_b200 import capi, glue, kernels as k
    s = seq.shapes
    peak, _ = load_peaks()

    def timed(fn, iters):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        a.record(stream)
        for _ in range(iters):
            fn()
        b.record(stream)
        torch.cuda.synchronize(device)
        return a.elapsed_time(b) / iters * 1e3

    g = torch.Generator(device=device).manual_seed(1234)
    table = (0.02 * torch.randn(s.vocab, s.hidden, generator=g, device=device)).to(torch.bfloat16)
    ids = torch.randint(0, s.vocab, (rows,), generator=g, device=device, dtype=torch.int32)
    out = torch.empty(rows, s.hidden, dtype=torch.bfloat16, device=device)
    us = timed(lambda: k.embed_gather(ids, table, s.embedding_multiplier, out), 10)
    bpr = glue.bytes_per_row(s)["embed"]
    embed = {"rows": rows, "mean_us": us, "achieved_gbs": bpr * rows / (us * 1e-6) / 1e9,
             "frac": bpr * rows / (us * 1e-6) / 1e9 / peak,
             "frac_of_nominal_8000": bpr * rows / (us * 1e-6) / 1e9 / NOMINAL_HBM_GBS, "bytes_per_row": bpr}

    def graph_replay_us(fn, iters=100):
        """fn captured once into a CUDA graph on a side stream, then replayed (every launcher is
        capturable: no allocation, no synchronisation, positions read from device memory)."""
        side = torch.cuda.Stream(device)
        with torch.cuda.stream(side):
            fn()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
            for _ in range(3):
                graph.replay()
            side.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side)
            for _ in range(iters):
                graph.replay()
            b.record(side)
            side.synchronize()
            return a.elapsed_time(b) / iters * 1e3

    small = {}
    for n in (1, 2, 4, 8, 500):
        sq = glue.GlueSequence(n, s, device=device, seed=7, sets=1, layers=1, pool_rows=8192, max_pos=8192)
        pos = torch.randint(0, 8192, (n,), generator=g, device=device, dtype=torch.int32)
        sq.set_rows(pos, torch.randperm(8192, generator=g, device=device)[:n].to(torch.int32))
        sq.reset()
        tok = ids[:n].contiguous()
        f32y = torch.randn(n, s.hidden, generator=g, device=device)
        f32r = torch.randn(n, s.hidden, generator=g, device=device)
        hb, nb = torch.empty_like(sq.h), torch.empty_like(sq.h)

        def chain():
            k.embed_gather(tok, table, s.embedding_multiplier, sq.h)
            for _, thunk in sq.layer_ops(0):
                thunk()
        entry = {"chain_eager_us": timed(chain, 50)}
        entry["chain_graph_us"] = graph_replay_us(chain)
        if n == 1:  # config 1: f32 x and residual, bf16 + FP8 out
            def c1():
                k.add_rmsnorm_fp8(f32y, f32r, sq.w[0, 0], s.eps, s.residual_multiplier, hb, nb, sq.n_fp8,
                                  sq.scales[0, 0])
            entry["add_rmsnorm_f32_fp8_us"] = timed(c1, 50)
            entry["add_rmsnorm_f32_fp8_graph_us"] = graph_replay_us(c1)
            # the same call straight through the C ABI (no Python wrapper around it): what a C host pays
            lib = capi.lib()
            c_args = (f32y.data_ptr(), 1, f32r.data_ptr(), 1, sq.w[0, 0].data_ptr(), s.eps, s.residual_multiplier,
                      1, s.hidden, hb.data_ptr(), nb.data_ptr(), sq.n_fp8.data_ptr(), sq.scales[0, 0].data_ptr(),
                      None)
            c_fn = lib.granite4_kernel_add_rmsnorm_fp8
            entry["add_rmsnorm_f32_fp8_c_abi_us"] = timed(lambda: c_fn(*c_args), 200)
        small[f"rows_{n}"] = entry
        del sq
    # Benchmark configuration 2 in its own shape: B decode sessions; gather from the Granite-size
    # table (ids uniform, multiplier 12) -> add + RMSNorm -> FP8 -> RoPE of Q [32 x 128] / K [8 x 128]
    # at positions uniform in [0, 8192) with the int8 KV append through per-session page tables
    # (the reference's decode entry point: K rounded to bf16 first) -> SwiGLU of gate / up [12800]
    # -> FP8. Four kernels, replayed from a CUDA graph.
    config2 = {}
    pool2 = 8 * 8192
    ck2 = torch.zeros(s.kv_heads, pool2, s.head_dim, dtype=torch.int8, device=device)
    cv2 = torch.zeros_like(ck2)
    ks2 = torch.zeros(s.kv_heads, pool2, dtype=torch.float32, device=device)
    vs2 = torch.zeros_like(ks2)
    tables2 = [((torch.randperm(512, generator=g, device=device) + 512 * r).repeat_interleave(16) * 16
                + torch.arange(8192, device=device) % 16).to(torch.int32) for r in range(8)]
    tabs2 = kernels_rope_tables(s, 8192, device)
    for n in (1, 2, 4, 8):
        desc = capi.MultiRows()
        desc.n = n
        pos_n = torch.randint(0, 8192, (n,), generator=g, device=device).tolist()
        for r in range(n):
            desc.pos[r] = pos_n[r]
            desc.pt[r] = tables2[r].data_ptr()
        d_rows = k.multi_rows_to_device(desc, device)
        b = {name: torch.randn(n, c, generator=g, device=device).to(torch.bfloat16)
             for name, c in (("y", s.hidden), ("q", s.q_heads * s.head_dim), ("k", s.kv_heads * s.head_dim),
                             ("v", s.kv_heads * s.head_dim), ("gate", s.intermediate), ("up", s.intermediate))}
        hid = torch.empty(n, s.hidden, dtype=torch.bfloat16, device=device)
        nf8 = torch.empty(n, s.hidden, dtype=torch.uint8, device=device)
        af8 = torch.empty(n, s.intermediate, dtype=torch.uint8, device=device)
        qr = torch.empty_like(b["q"])
        sc = torch.zeros(2, 2, dtype=torch.float32, device=device)
        tok = ids[:n].contiguous()
        wn = seq.w[0, 0]

        def chain2():
            k.embed_gather(tok, table, s.embedding_multiplier, hid)
            k.add_rmsnorm_fp8(b["y"], hid, wn, s.eps, s.residual_multiplier, h_out=hid, n_fp8=nf8, scale_amax=sc[0])
            k.gpu_multi_rope_append(b["q"], b["k"], b["v"], tabs2.cos, tabs2.sin, d_rows, n, s.q_heads, s.kv_heads,
                                    s.head_dim, 8, ck2, cv2, ks2, vs2, pool2, qr)
            k.swiglu_fp8(b["gate"], b["up"], None, af8, sc[1])
        config2[f"sessions_{n}"] = {"kernels": 4, "chain_eager_us": timed(chain2, 50),
                                    "chain_graph_us": graph_replay_us(chain2)}
    tabs2.close()
    del table, ck2, cv2, ks2, vs2
    torch.cuda.empty_cache()

    # Benchmark configuration 4, the long-context write: 4 sequences x 8192 tokens at RoPE offsets up to
    # 131071, K/V scattered into a 122880-row pool through a random permutation of its 7680
    # 16-token pages, against the same rows written to consecutive pool rows.
    from granite4_b200 import paging
    c4_rows = min(rows, 32768)
    per_seq = c4_rows // 4
    pool4, max_pos4 = 7680 * 16, 131072
    tabs4 = kernels_rope_tables(s, max_pos4, device)
    bt = paging.permuted_block_tables(4, (per_seq + 15) // 16, 7680, seed=44)
    pos4, kvr4 = paging.batch_rows(bt, [0, 40000, 90001, max_pos4 - per_seq], per_seq)
    pos4_d, kvr4_d = torch.from_numpy(pos4).to(device), torch.from_numpy(kvr4).to(device)
    ident = torch.arange(c4_rows, dtype=torch.int32, device=device)
    ck4 = torch.zeros(s.kv_heads, pool4, s.head_dim, dtype=torch.int8, device=device)
    cv4 = torch.zeros_like(ck4)
    ks4 = torch.zeros(s.kv_heads, pool4, dtype=torch.float32, device=device)
    vs4 = torch.zeros_like(ks4)
    qr4 = torch.empty(c4_rows, s.q_heads * s.head_dim, dtype=torch.bfloat16, device=device)
    flip4 = [0]

    def rope4(pos_t, kv_t):
        flip4[0] ^= 1  # rotate the two input sets: nothing is L2-hot
        qkv = seq.sets[flip4[0] % len(seq.sets)]["qkv"][:c4_rows]
        k.rope_kv_int8_paged(qkv, tabs4.cos, tabs4.sin, pos_t, kv_t, s.q_heads, s.kv_heads, s.head_dim, pool4,
                             max_pos4, 0, qr4, ck4, cv4, ks4, vs4)
    bpr4 = glue.bytes_per_row(s)["rope_kv_int8"]
    us_id = timed(lambda: rope4(ident, ident), 20)
    us_pg = timed(lambda: rope4(pos4_d, kvr4_d), 20)
    config4 = {"rows": c4_rows, "pool_rows": pool4, "pages": 7680,
               "consecutive_rows_us": us_id, "permuted_pages_us": us_pg,
               "permuted_over_consecutive": us_pg / us_id,
               "achieved_gbs": bpr4 * c4_rows / (us_pg * 1e-6) / 1e9,
               "frac": bpr4 * c4_rows / (us_pg * 1e-6) / 1e9 / peak}
    tabs4.close()
    del ck4, cv4, ks4, vs4, qr4
    torch.cuda.empty_cache()

    # Greedy pick over the logits (the decode step's last glue op; 2 V bytes read per row): a
    # prefill-size batch against the bandwidth roofline, decode sizes as latencies.
    a_rows = min(rows, 8192)
    logits = torch.randn(a_rows, s.vocab, generator=g, device=device).to(torch.bfloat16)
    picked = torch.empty(a_rows, dtype=torch.int32, device=device)
    us = timed(lambda: k.argmax_rows(logits, picked), 10)
    a_bytes = (2 * s.vocab + 4) * a_rows
    argmax = {"rows": a_rows, "mean_us": us, "achieved_gbs": a_bytes / (us * 1e-6) / 1e9,
              "frac": a_bytes / (us * 1e-6) / 1e9 / peak, "bytes_per_row": 2 * s.vocab + 4}
    for n in (1, 8):
        argmax[f"rows_{n}_graph_us"] = graph_replay_us(lambda: k.argmax_rows(logits[:n], picked[:n]))
    del logits
    torch.cuda.empty_cache()

    # Decode attention over the int8 paged pool (the reader of the KV write): 264 B per cache
    # position and kv head. One layer's pool of 131072 rows (270 MB, larger than L2), 16-token pages
    # in permuted order; a single sequence at full context, eight sequences of 32768, and a
    # four-row verify step.
    stride, page = 131072, 16
    ck = torch.randint(-127, 128, (s.kv_heads, stride, s.head_dim), generator=g, device=device, dtype=torch.int8)
    cv = torch.randint(-127, 128, (s.kv_heads, stride, s.head_dim), generator=g, device=device, dtype=torch.int8)
    ksc = torch.rand(s.kv_heads, stride, generator=g, device=device) * 0.02 + 0.005
    vsc = torch.rand(s.kv_heads, stride, generator=g, device=device) * 0.02 + 0.005
    pages = torch.randperm(stride // page, generator=g, device=device)
    table = (pages.repeat_interleave(page) * page + torch.arange(stride, device=device) % page).to(torch.int32)
    attention = {}
    for name, n, group, ctx in (("1_row_ctx_131072", 1, 1, 131072), ("8_rows_ctx_32768", 8, 1, 32768),
                                ("verify_4_rows_ctx_32768", 4, 4, 32768),
                                ("verify_8_groups_of_4_rows_ctx_32768", 32, 4, 32768)):
        qa = torch.randn(n, s.q_heads * s.head_dim, generator=g, device=device).to(torch.bfloat16)
        pos = torch.full((n,), ctx - 1, dtype=torch.int32, device=device)
        if group > 1:
            pos = pos - torch.arange(n - 1, -1, -1, device=device, dtype=torch.int32)
        oa = torch.empty_like(qa)
        need = k.attn_decode_scratch_bytes(n, group, s.kv_heads, ctx)
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
        us = timed(lambda: k.attn_decode_int8_paged(qa, ck, cv, ksc, vsc, pos, s.q_heads, s.kv_heads, s.head_dim,
                                                    stride, ctx, 1.0 / 128, oa, rows_per_group=group, pt=table,
                                                    scratch=scratch), 20)
        groups = (n + group - 1) // group
        nbytes = groups * s.kv_heads * ctx * (2 * s.head_dim + 8)
        attention[name] = {"mean_us": us, "achieved_gbs": nbytes / (us * 1e-6) / 1e9,
                           "frac": nbytes / (us * 1e-6) / 1e9 / peak, "bytes": nbytes}
    # Causal attention of a whole prefill chunk over the same pool (K/V of the chunk stay in L2):
    # 4 d Hq n^2 / 2 flops, against the measured bf16 GEMM rate. The tcgen05 kernel (default) and the
    # mma.sync kernel it replaced for chunks of 64 rows or more, through the same entry point.
    mp_attn = {}
    if os.path.isfile(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp_attn = json.load(f)
    bf16_peak = float(mp_attn.get("bf16_tflops", 1590.0))
    for n_pf in (2048, 8192):
        qa = torch.randn(n_pf, s.q_heads * s.head_dim, generator=g, device=device).to(torch.bfloat16)
        oa = torch.empty_like(qa)
        flops = 4.0 * s.head_dim * s.q_heads * n_pf * (n_pf + 1) / 2
        entry = {}
        for form, env in (("tcgen05", "1"), ("mma_sync", "0")):
            os.environ["G4_PREFILL_TC"] = env
            us = timed(lambda: k.prefill_attention_int8(qa, 1.0 / 128, s.q_heads, s.kv_heads, s.head_dim, 0, stride,
                                                        oa, ck, cv, ksc, vsc, pt=table), 5)
            entry[form] = {"mean_us": us, "tflops": flops / (us * 1e-6) / 1e12,
                           "frac_of_measured_bf16": flops / (us * 1e-6) / 1e12 / bf16_peak}
        os.environ.pop("G4_PREFILL_TC")
        entry.update({"mean_us": entry["tcgen05"]["mean_us"], "tflops": entry["tcgen05"]["tflops"],
                      "form": "tcgen05: S and O in tensor memory, 64 positions x 4 heads per CTA, K / V converted once per tile"})
        attention[f"prefill_{n_pf}_rows"] = entry
        del qa, oa
    # A whole decode step (one layer's glue + attention at ~4096 positions + final norm + greedy
    # pick with the token scatter folded in) of n sessions, captured into a CUDA graph and replayed: everything that
    # changes between steps is read from the device descriptor, so the replays chain by themselves.
    decode_step = {}
    emb_small = (0.02 * torch.randn(4096, s.hidden, generator=g, device=device)).to(torch.bfloat16)
    logits_small = torch.randn(16, 4096, generator=g, device=device).to(torch.bfloat16)
    w3 = (1.0 + 0.02 * torch.randn(3, s.hidden, generator=g, device=device)).to(torch.bfloat16)
    for n in (1, 8):
        sess_tables = [table[r * 8192:(r + 1) * 8192].contiguous() for r in range(n)]
        toks = [torch.zeros(8192, dtype=torch.int32, device=device) for _ in range(n)]
        desc = capi.MultiRows()
        desc.n = n
        for r in range(n):
            desc.pos[r] = 4000 + 3 * r
            desc.pt[r] = sess_tables[r].data_ptr()
            desc.tok[r] = toks[r].data_ptr()
        d_rows = k.multi_rows_to_device(desc, device)
        row_pos = d_rows[capi.MultiRows.pos.offset:capi.MultiRows.pos.offset + 4 * n].view(torch.int32)
        row_pt = d_rows[capi.MultiRows.pt.offset:capi.MultiRows.pt.offset + 8 * n].view(torch.int64)
        b = {name: torch.randn(n, c, generator=g, device=device).to(torch.bfloat16)
             for name, c in (("y_attn", s.hidden), ("y_mlp", s.hidden), ("q", s.q_heads * s.head_dim),
                             ("k", s.kv_heads * s.head_dim), ("v", s.kv_heads * s.head_dim),
                             ("gate", s.intermediate), ("up", s.intermediate))}
        hid = torch.empty(n, s.hidden, dtype=torch.bfloat16, device=device)
        fin = torch.empty_like(hid)
        nf8 = torch.empty(n, s.hidden, dtype=torch.uint8, device=device)
        af8 = torch.empty(n, s.intermediate, dtype=torch.uint8, device=device)
        sc = torch.zeros(3, 2, dtype=torch.float32, device=device)
        qr, ao = torch.empty_like(b["q"]), torch.empty_like(b["q"])
        idv = torch.zeros(n, dtype=torch.int32, device=device)
        scr = torch.empty(max(k.attn_decode_scratch_bytes(n, 1, s.kv_heads, 8192), 16), dtype=torch.uint8,
                          device=device)

        def step():
            k.gpu_multi_embed(d_rows, n, emb_small, s.embedding_multiplier, hid)
            k.add_rmsnorm_fp8(b["y_attn"], hid, w3[0], s.eps, s.residual_multiplier, h_out=hid, n_fp8=nf8,
                              scale_amax=sc[0])
            k.gpu_multi_rope_append(b["q"], b["k"], b["v"], seq.tables.cos, seq.tables.sin, d_rows, n, s.q_heads,
                                    s.kv_heads, s.head_dim, 8, ck, cv, ksc, vsc, stride, qr)
            k.attn_decode_int8_paged(qr, ck, cv, ksc, vsc, row_pos, s.q_heads, s.kv_heads, s.head_dim, stride,
                                     8192, 1.0 / 128, ao, rows_per_group=1, row_pt=row_pt, scratch=scr)
            k.add_rmsnorm_fp8(b["y_mlp"], hid, w3[1], s.eps, s.residual_multiplier, h_out=hid, n_fp8=nf8,
                              scale_amax=sc[1])
            k.swiglu_fp8(b["gate"], b["up"], None, af8, sc[2])
            k.rmsnorm(hid, w3[2], s.eps, n, s.hidden, fin, batched=True)
            k.argmax_advance(logits_small[:n], d_rows, idv)
        decode_step[f"sessions_{n}"] = {"kernels": 9, "graph_replay_us": graph_replay_us(step)}
    del ck, cv, ksc, vsc, table
    torch.cuda.empty_cache()

    # The FP8 x FP8 GEMMs on either side of the glue (tensor-core bound at prefill sizes, a stream
    # of the weights at decode sizes). Codes of N(0, 1) values scaled the way the glue's per-tensor
    # amax scales them (amax ~ 5 sigma -> 448). Prefill: one 8192-row chunk per projection, against
    # twice the measured bf16 GEMM rate (there is no measured FP8 figure) and the nominal dense FP8
    # peak. Decode: the four projections of a layer back to back in a CUDA graph over two rotated
    # weight sets (2 x 199 MB, larger than L2), against the HBM roofline on the weight bytes.
    mp = {}
    if os.path.isfile(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
    bf16_burst, bf16_sust = float(mp.get("bf16_tflops", 1590.0)), float(mp.get("bf16_tflops_sustained", 1400.0))

    def fp8_codes(r, c):
        # (clamped: e4m3 has no infinity, a value past 448 would become a NaN code)
        return (torch.randn(r, c, generator=g, device=device) * (448.0 / 5.0)).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    H, I, QKV = s.hidden, s.intermediate, (s.q_heads + 2 * s.kv_heads) * s.head_dim
    proj = (("qkv", QKV, H), ("o", H, H), ("gate_up", 2 * I, H), ("down", H, I))
    wsets = [{name: fp8_codes(N, Kd) for name, N, Kd in proj} for _ in range(2)]
    g_rows = min(rows, 8192)
    a_h, a_i = fp8_codes(g_rows, H), fp8_codes(g_rows, I)
    a_sc = torch.tensor([5.0 / 448.0, 5.0], device=device)
    gemm = {"prefill_rows": g_rows, "peaks": {"bf16_tflops_measured": bf16_burst,
                                              "bf16_tflops_sustained_measured": bf16_sust, "fp8_tflops_nominal": 4500.0}}
    for name, N, Kd in proj:
        a_in = a_i if Kd == I else a_h
        o = torch.empty(g_rows, N, dtype=torch.bfloat16, device=device)
        flip = [0]

        def run():
            flip[0] ^= 1
            k.gemm_fp8(a_in, wsets[flip[0]][name], o, a_scale=a_sc, w_scales=(0.01,))
        us = timed(run, 20)
        tf = 2.0 * g_rows * N * Kd / (us * 1e-6) / 1e12
        gemm[name] = {"M": g_rows, "N": N, "K": Kd, "mean_us": us, "tflops": tf,
                      "frac_of_2x_measured_bf16_sustained": tf / (2 * bf16_sust),
                      "frac_of_2x_measured_bf16_burst": tf / (2 * bf16_burst), "frac_of_nominal_4500": tf / 4500.0}
        del o
    # gate|up projection -> SwiGLU -> FP8, two ways: the projection writing gate|up (bf16) and the
    # standalone two-sweep SwiGLU kernel after it, or SwiGLU folded into the projection's epilogue
    # (which also leaves max |a| in the device slot) and the one-sweep encode after it.
    gu_o = torch.empty(g_rows, 2 * I, dtype=torch.bfloat16, device=device)
    act_b = torch.empty(g_rows, I, dtype=torch.bfloat16, device=device)
    act_8 = torch.empty(g_rows, I, dtype=torch.uint8, device=device)
    slot = torch.zeros(2, dtype=torch.float32, device=device)
    flip = [0]

    def unfused():
        flip[0] ^= 1
        k.gemm_fp8(a_h, wsets[flip[0]]["gate_up"], gu_o, a_scale=a_sc, w_scales=(0.01,))
        k.swiglu_fp8(gu_o[:, :I], gu_o[:, I:], None, act_8, slot, ld=2 * I)

    def fused():
        flip[0] ^= 1
        k.gemm_fp8(a_h, wsets[flip[0]]["gate_up"], act_b, a_scale=a_sc, w_scales=(0.01,), swiglu_scale_amax=slot)
        k.fp8_encode_with_amax(act_b, act_8, slot)
    gemm["gate_up_swiglu_fp8"] = {"M": g_rows, "unfused_us": timed(unfused, 10), "fused_epilogue_us": timed(fused, 10),
                                  "bytes_per_row_unfused": 2 * (2 * I) + 9 * I, "bytes_per_row_fused": 2 * I + 3 * I}
    del gu_o, act_b, act_8
    wbytes = sum(N * Kd for _, N, Kd in proj)
    # the prefill projections above ran under the power cap; a decode step does not follow such a burst,
    # so let the clocks come back before the latency-sized measurements
    torch.cuda.synchronize()
    time.sleep(1.0)
    for n in (1, 8, 16):
        outs = {name: torch.empty(n, N, dtype=torch.bfloat16, device=device) for name, N, _ in proj}
        wsp = {name: k.gemm_fp8_workspace(n, N, Kd, device) for name, N, Kd in proj}

        def layer_gemms():
            for ws_ in wsets:
                for name, N, Kd in proj:
                    k.gemm_fp8((a_i if Kd == I else a_h)[:n], ws_[name], outs[name], a_scale=a_sc, w_scales=(0.01,),
                               workspace=wsp[name])
        us = graph_replay_us(layer_gemms, 20) / 2
        gemm[f"decode_rows_{n}_layer_graph_us"] = us
        gemm[f"decode_rows_{n}_weight_gbs"] = wbytes / (us * 1e-6) / 1e9
        gemm[f"decode_rows_{n}_frac"] = wbytes / (us * 1e-6) / 1e9 / peak
    gemm["decode_weight_bytes_per_layer"] = wbytes

    # A complete decode step of a two-layer model with real projections, one CUDA graph: embedding of
    # the newest tokens, per layer {norm -> FP8, QKV GEMM, RoPE + int8 KV append, attention over
    # ~4100 cached positions, FP8 of the attention output, O GEMM + residual, norm -> FP8, gate|up
    # GEMM, SwiGLU -> FP8, down GEMM + residual}, final norm -> FP8, lm_head GEMM (100352 x 4096),
    # greedy pick + token scatter. 809 MB of weights per replay (two layer sets + lm_head).
    stride_d, page_d = 16384, 16
    ck = torch.zeros(s.kv_heads, stride_d, s.head_dim, device=device, dtype=torch.int8)
    cv = torch.zeros_like(ck)
    ksc = torch.full((s.kv_heads, stride_d), 0.01, device=device)
    vsc = torch.full((s.kv_heads, stride_d), 0.01, device=device)
    ck.random_(-127, 128, generator=g), cv.random_(-127, 128, generator=g)
    w_lm = fp8_codes(s.vocab, H)
    wn = (1.0 + 0.02 * torch.randn(3, H, generator=g, device=device)).to(torch.bfloat16)
    emb_d = (0.02 * torch.randn(4096, H, generator=g, device=device)).to(torch.bfloat16)
    full = {}
    for n in (1, 8):
        tables = [(torch.randperm(stride_d // 8 // page_d, generator=g, device=device).repeat_interleave(page_d) * page_d
                   + torch.arange(stride_d // 8, device=device) % page_d + r * (stride_d // 8)).to(torch.int32)
                  for r in range(n)]
        toks = [torch.zeros(stride_d // 8, dtype=torch.int32, device=device) for _ in range(n)]
        desc = capi.MultiRows()
        desc.n = n
        for r in range(n):
            desc.pos[r] = 1900 + 3 * r
            desc.pt[r] = tables[r].data_ptr()
            desc.tok[r] = toks[r].data_ptr()
        d_rows = k.multi_rows_to_device(desc, device)
        row_pos = d_rows[capi.MultiRows.pos.offset:capi.MultiRows.pos.offset + 4 * n].view(torch.int32)
        row_pt = d_rows[capi.MultiRows.pt.offset:capi.MultiRows.pt.offset + 8 * n].view(torch.int64)
        kv_rows = torch.stack([tables[r][1900 + 3 * r] for r in range(n)]).to(torch.int32)
        hid = torch.empty(n, H, dtype=torch.bfloat16, device=device)
        nf8 = torch.empty(n, H, dtype=torch.uint8, device=device)
        a8 = torch.empty(n, H, dtype=torch.uint8, device=device)
        act8 = torch.empty(n, I, dtype=torch.uint8, device=device)
        qkv = torch.empty(n, QKV, dtype=torch.bfloat16, device=device)
        qr = torch.empty(n, H, dtype=torch.bfloat16, device=device)
        ao = torch.empty_like(qr)
        gu = torch.empty(n, 2 * I, dtype=torch.bfloat16, device=device)
        logits = torch.empty(n, s.vocab, dtype=torch.bfloat16, device=device)
        sc = torch.zeros(12, 2, dtype=torch.float32, device=device)
        idv = torch.zeros(n, dtype=torch.int32, device=device)
        scr = torch.empty(max(k.attn_decode_scratch_bytes(n, 1, s.kv_heads, 2048), 16), dtype=torch.uint8, device=device)
        wsp = {name: k.gemm_fp8_workspace(n, N, Kd, device) for name, N, Kd in proj}
        wsp["lm"] = k.gemm_fp8_workspace(n, s.vocab, H, device)
        count = [0]

        def step():
            c = 0
            k.gpu_multi_embed(d_rows, n, emb_d, s.embedding_multiplier, hid)
            c += 1
            for li, ws_ in enumerate(wsets):
                b = 5 * li
                k.add_rmsnorm_fp8(hid, None, wn[0], s.eps, s.residual_multiplier, n_fp8=nf8, scale_amax=sc[b])
                k.gemm_fp8(nf8, ws_["qkv"], qkv, a_scale=sc[b], w_scales=(0.01,), workspace=wsp["qkv"])
                k.rope_kv_int8_paged(qkv, seq.tables.cos, seq.tables.sin, row_pos, kv_rows, s.q_heads, s.kv_heads,
                                     s.head_dim, stride_d, seq.max_pos, 0, qr, ck, cv, ksc, vsc)
                k.attn_decode_int8_paged(qr, ck, cv, ksc, vsc, row_pos, s.q_heads, s.kv_heads, s.head_dim, stride_d,
                                         2048, 1.0 / 128, ao, rows_per_group=1, row_pt=row_pt, scratch=scr)
                k.fp8_quant(ao, a8, sc[b + 1])
                k.gemm_fp8(a8, ws_["o"], hid, a_scale=sc[b + 1], w_scales=(0.01,), residual=hid,
                           resid_scale=s.residual_multiplier, workspace=wsp["o"])
                k.add_rmsnorm_fp8(hid, None, wn[1], s.eps, s.residual_multiplier, n_fp8=nf8, scale_amax=sc[b + 2])
                k.gemm_fp8(nf8, ws_["gate_up"], gu, a_scale=sc[b + 2], w_scales=(0.01,), workspace=wsp["gate_up"])
                k.swiglu_fp8(gu[:, :I], gu[:, I:], None, act8, sc[b + 3], ld=2 * I)
                k.gemm_fp8(act8, ws_["down"], hid, a_scale=sc[b + 3], w_scales=(0.01,), residual=hid,
                           resid_scale=s.residual_multiplier, workspace=wsp["down"])
                c += 11
            k.add_rmsnorm_fp8(hid, None, wn[2], s.eps, s.residual_multiplier, n_fp8=nf8, scale_amax=sc[10])
            k.gemm_fp8(nf8, w_lm, logits, a_scale=sc[10], w_scales=(0.01,), workspace=wsp["lm"])
            k.argmax_advance(logits, d_rows, idv)
            count[0] = c + 3
        us = graph_replay_us(step, 20)
        wb = 2 * wbytes + s.vocab * H
        full[f"sessions_{n}"] = {"layers": 2, "launches": count[0], "graph_replay_us": us, "weight_bytes": wb,
                                 "weight_gbs": wb / (us * 1e-6) / 1e9, "frac": wb / (us * 1e-6) / 1e9 / peak}
    gemm["decode_step_two_layers_lm_head"] = full
    del w_lm, logits

    # One whole prefill layer on device buffers only (the first chunk of a prompt, positions 0..n-1):
    # norm -> FP8, QKV GEMM, RoPE + int8 KV write, causal attention over the pool, FP8 of its output,
    # O GEMM + residual, norm -> FP8, gate|up GEMM with the fused SwiGLU epilogue, one-sweep encode,
    # down GEMM + residual. Event-timed per step to show where a layer's time goes.
    layer = {}
    for n_pf in (2048, 8192):
        if n_pf > stride_d:
            continue
        hid = torch.randn(n_pf, H, generator=g, device=device).to(torch.bfloat16)
        nf8 = torch.empty(n_pf, H, dtype=torch.uint8, device=device)
        a8 = torch.empty(n_pf, H, dtype=torch.uint8, device=device)
        qkv = torch.empty(n_pf, QKV, dtype=torch.bfloat16, device=device)
        qr = torch.empty(n_pf, H, dtype=torch.bfloat16, device=device)
        ao = torch.empty_like(qr)
        act_b = torch.empty(n_pf, I, dtype=torch.bfloat16, device=device)
        act8 = torch.empty(n_pf, I, dtype=torch.uint8, device=device)
        sc = torch.zeros(4, 2, dtype=torch.float32, device=device)
        pos = torch.arange(n_pf, dtype=torch.int32, device=device)
        ws_ = wsets[0]
        steps = (
            ("norm_fp8", lambda: k.add_rmsnorm_fp8(hid, None, wn[0], s.eps, s.residual_multiplier, n_fp8=nf8, scale_amax=sc[0])),
            ("qkv_gemm", lambda: k.gemm_fp8(nf8, ws_["qkv"], qkv, a_scale=sc[0], w_scales=(0.01,))),
            ("rope_kv", lambda: k.rope_kv_int8_paged(qkv, seq.tables.cos, seq.tables.sin, pos, pos, s.q_heads, s.kv_heads,
                                                      s.head_dim, stride_d, seq.max_pos, 0, qr, ck, cv, ksc, vsc)),
            ("attention", lambda: k.prefill_attention_int8(qr, 1.0 / 128, s.q_heads, s.kv_heads, s.head_dim, 0, stride_d, ao,
                                                           ck, cv, ksc, vsc)),
            ("attn_fp8", lambda: k.fp8_quant(ao, a8, sc[1])),
            ("o_gemm_residual", lambda: k.gemm_fp8(a8, ws_["o"], hid, a_scale=sc[1], w_scales=(0.01,), residual=hid,
                                                   resid_scale=s.residual_multiplier)),
            ("norm_fp8_2", lambda: k.add_rmsnorm_fp8(hid, None, wn[1], s.eps, s.residual_multiplier, n_fp8=nf8, scale_amax=sc[2])),
            ("gate_up_gemm_swiglu", lambda: k.gemm_fp8(nf8, ws_["gate_up"], act_b, a_scale=sc[2], w_scales=(0.01,),
                                                       swiglu_scale_amax=sc[3])),
            ("act_fp8_encode", lambda: k.fp8_encode_with_amax(act_b, act8, sc[3])),
            ("down_gemm_residual", lambda: k.gemm_fp8(act8, ws_["down"], hid, a_scale=sc[3], w_scales=(0.0001,), residual=hid,
                                                      resid_scale=s.residual_multiplier)),
        )

        def whole():
            for _, fn in steps:
                fn()
        total = timed(whole, 5)
        per = {name: timed(fn, 5) for name, fn in steps}
        layer[f"rows_{n_pf}"] = {"total_us": total, "steps_us": per}
    gemm["prefill_layer"] = layer
    del ck, cv, ksc, vsc
    del wsets, a_h, a_i
    torch.cuda.empty_cache()
    return {"embed": embed, "small": small, "argmax": argmax, "attention": attention, "decode_step": decode_step,
            "gemm": gemm, "config2": config2, "config4": config4}


def cpus_near_gpu(device):
    """CPUs of the NUMA node the GPU hangs off (sysfs local_cpulist of its PCI function), cut down
    to the ones this process may run on; an empty set when sysfs does not say."""
    import torch
    try:
        pr = torch.cuda.get_device_properties(device)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            text = f.read().strip()
    except (OSError, AttributeError):
        return set(), None
    cpus = set()
    for part in text.split(","):
        if part:
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus & os.sched_getaffinity(0), bdf


def run_e2e(seq, rows, device, steps):
    """The same sequence through the host-buffer C ABI: per step every layer's inputs are copied
    from pinned host memory, its FP8 / q_rot outputs are copied back. For the duration of this leg
    the process is bound to the CPUs next to its GPU, so the pinned buffers (allocated below, first
    touched here) and the enqueueing thread sit on the GPU's NUMA node."""
    import torch
    from granite4_b200 import glue
    s = seq.shapes
    before = os.sched_getaffinity(0)
    near, bdf = cpus_near_gpu(device)
    if near and os.environ.get("G4_BENCH_BIND", "1") != "0":
        os.sched_setaffinity(0, near)
    try:
        ms, h2d, d2h, steps = _run_e2e_bound(seq, rows, device, steps, s, glue, torch)
    finally:
        os.sched_setaffinity(0, before)
    return ms, h2d, d2h, steps, {"pci": bdf, "cpus_near_gpu": len(near), "bound": bool(near)}


def _run_e2e_bound(seq, rows, device, steps, s, glue, torch):
    hg = glue.HostGlue(rows, s, device=device, layers=seq.layers, pool_rows=seq.pool_rows,
                       max_pos=seq.max_pos)
    src = seq.sets[0]

    def pinned_copy(t):
        return t.cpu().pin_memory()

    def pinned_empty(shape, dtype):
        return torch.empty(shape, dtype=dtype).pin_memory()
    host = {k: pinned_copy(src[k]) for k in ("y_attn", "y_mlp", "qkv", "gate", "up")}
    host["w_attn_norm"] = pinned_copy(seq.w[0, 0])
    host["w_mlp_norm"] = pinned_copy(seq.w[0, 1])
    host["pos_rows"] = pinned_copy(seq.pos_rows)
    host["kv_rows"] = pinned_copy(seq.kv_rows)
    host["n_attn_fp8"] = pinned_empty((rows, s.hidden), torch.uint8)
    host["n_mlp_fp8"] = pinned_empty((rows, s.hidden), torch.uint8)
    host["q_rot"] = pinned_empty((rows, s.q_heads * s.head_dim), torch.bfloat16)
    host["act_fp8"] = pinned_empty((rows, s.intermediate), torch.uint8)
    host["scales"] = pinned_empty((6,), torch.float32)
    h_in = pinned_copy(seq.h0)
    h_out = pinned_empty((rows, s.hidden), torch.bfloat16)
    w_final = pinned_copy(seq.w_final)
    mid = glue.host_layer_io(host, rows, s.eps, s.residual_multiplier)
    first = glue.host_layer_io({**host, "hidden_in": h_in}, rows, s.eps, s.residual_multiplier)

    def step():
        for layer in range(seq.layers):
            hg.layer(layer, first if layer == 0 else mid)
        hg.final_norm(w_final, s.eps, rows, h_out)
    step()  # warm-up
    hg.sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    hg.sync()
    ms = (time.perf_counter() - t0) * 1e3
    h2d = seq.layers * hg.h2d_bytes(rows) + h_in.numel() * 2 + w_final.numel() * 2
    d2h = seq.layers * hg.d2h_bytes(rows) + h_out.numel() * 2
    hg.close()
    return ms, h2d, d2h, steps


def prefill_attention_only(rows, launches, local_rank):
    """The causal attention of one prefill chunk over an int8 pool of 16-token pages in permuted
    order, `launches` times after three warm-up launches: the small case a profiler capture runs."""
    import torch
    import granite4_b200  # noqa: F401
    from granite4_b200 import glue, kernels as k
    s = glue.GraniteShapes()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    g = torch.Generator(device=device).manual_seed(1234)
    stride = max(16384, (rows + 15) // 16 * 16)
    ck = torch.randint(-127, 128, (s.kv_heads, stride, s.head_dim), generator=g, device=device, dtype=torch.int8)
    cv = torch.randint(-127, 128, (s.kv_heads, stride, s.head_dim), generator=g, device=device, dtype=torch.int8)
    ksc = torch.rand(s.kv_heads, stride, generator=g, device=device) * 0.02 + 0.005
    vsc = torch.rand(s.kv_heads, stride, generator=g, device=device) * 0.02 + 0.005
    pages = torch.randperm(stride // 16, generator=g, device=device)
    table = (pages.repeat_interleave(16) * 16 + torch.arange(stride, device=device) % 16).to(torch.int32)
    q = torch.randn(rows, s.q_heads * s.head_dim, generator=g, device=device).to(torch.bfloat16)
    out = torch.empty_like(q)

    def run():
        return k.prefill_attention_int8(q, 1.0 / 128, s.q_heads, s.kv_heads, s.head_dim, 0, stride, out, ck, cv, ksc, vsc,
                                        pt=table)
    for _ in range(3):
        assert run() == 0
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    a.record()
    for _ in range(launches):
        run()
    b.record()
    torch.cuda.synchronize(device)
    us = a.elapsed_time(b) / launches * 1e3
    flops = 4.0 * s.head_dim * s.q_heads * rows * (rows + 1) / 2
    from granite4_b200 import capi
    return {"prefill_attention_rows": rows, "mean_us": us, "tflops": flops / (us * 1e-6) / 1e12,
            "device_status": capi.lib().device_status()}


def decode_gemm_only(shape, launches, local_rank):
    """One decode-size FP8 GEMM (shape "N,K,rows": weight rows, depth, activation rows) over three
    rotated weight matrices, `launches` times after six warm-up launches: the small case a profiler
    capture of the 16-row form runs."""
    import torch
    import granite4_b200  # noqa: F401
    from granite4_b200 import capi, kernels as k
    N, Kd, rows = (int(x) for x in shape.split(","))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    g = torch.Generator(device=device).manual_seed(1234)

    def codes(r, c):
        # (clamped: e4m3 has no infinity, a value past 448 would become a NaN code)
        return (torch.randn(r, c, generator=g, device=device) * (448.0 / 5.0)).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    ws = [codes(N, Kd) for _ in range(3)]
    a = codes(max(rows, 1), Kd)
    a_sc = torch.tensor([5.0 / 448.0, 5.0], device=device)
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=device)
    wsp = k.gemm_fp8_workspace(rows, N, Kd, device)
    for i in range(6):
        assert k.gemm_fp8(a, ws[i % 3], out, a_scale=a_sc, w_scales=(0.01,), workspace=wsp) == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record()
    for i in range(launches):
        k.gemm_fp8(a, ws[i % 3], out, a_scale=a_sc, w_scales=(0.01,), workspace=wsp)
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) / launches * 1e3
    return {"decode_gemm": {"N": N, "K": Kd, "rows": rows}, "mean_us_eager": us, "weight_gbs": N * Kd / (us * 1e-6) / 1e9,
            "device_status": capi.lib().device_status()}


def timed_step(seq, op_events, stream):
    """GlueSequence.run() with an event pair around every op (for the per-op durations)."""
    import torch

    def timed(name, thunk):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        rc = thunk()
        b.record(stream)
        op_events[name].append((a, b))
        return rc

    seq.run(wrap=timed)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--sweep-only", action="store_true", help="only the sweep (short profiler captures)")
    ap.add_argument("--prefill-attention-only", type=int, metavar="ROWS", default=0,
                    help="only the causal prefill attention of a chunk of ROWS rows, a few launches (profiler captures)")
    ap.add_argument("--decode-gemm-only", metavar="N,K,ROWS", default="",
                    help="only one decode-size FP8 GEMM of that shape, --steps launches (a small profiler case)")
    ap.add_argument("--traffic-from-ncu", metavar="CSV", help="convert a profiler launch list; no benchmark")
    ap.add_argument("--traffic-rows", type=int, default=8192, help="token rows of that capture")
    args = ap.parse_args()
    if args.traffic_from_ncu:
        print(json.dumps(traffic_from_ncu(args.traffic_from_ncu, args.traffic_rows)))
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs one process per GPU: launch with "
                         f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {args.gpus} "
                         f"--master-addr 127.0.0.1 --master-port <port> bench.py --gpus {args.gpus} ...")
    if args.prefill_attention_only:
        print(json.dumps(prefill_attention_only(args.prefill_attention_only, max(args.steps, 1), local_rank)))
        return
    if args.decode_gemm_only:
        print(json.dumps(decode_gemm_only(args.decode_gemm_only, max(args.steps, 1), local_rank)))
        return
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
    else:
        run_gpu_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
