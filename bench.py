#!/usr/bin/env python3
"""Benchmark of the GGUF row quantize / dequantize hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload `dequant_sweep` is the configuration the headline metric is quoted on: decode a
14336x4096 weight matrix (N(0, 0.02), seed 0) from Q8_0, Q6_K, Q5_K, Q4_K, Q3_K and Q2_K to fp16
and to bf16.  One step = the 12 decodes.  `value` counts algorithmic bytes (encoded bytes read +
2 bytes per element written) per second with inputs resident in HBM; `e2e` is the same metric
through the device-pointer C ABI with pinned HOST buffers, copies included, and `roofline_e2e`
sets it beside what plain copies of the same bytes reach on the same host link.  The same line
carries the quantize half of the metric (`quant`: Melem/s per type for the Q4_K round trip, the
six K/Q types, MXFP4 / NVFP4 and the four lattice types, each on its own workload matrix), the
whole-model conversion (`convert`: GB/s of fp32 source through the pinned-host streaming
pipeline) and a host-pointer figure (`host_api`).  Every input comes from the seeded NumPy
generators of tests/inputs.py, and after the timed regions one slice per type is compared with
the CPU checker (`verified`).  `--workload NAME` runs one of the secondary workloads alone
(bench_quant.py).

Under torchrun every rank runs the same per-GPU workload on its own device (weak scaling, no
collective on the data path; the conversion shards one model over the ranks, strong scaling);
every reported time is the maximum over ranks.

`--impl reference` times upstream's own CPU implementation (oracle/_ref, built from the upstream
sources; the C restatement if that library is absent) on the host cores, same rows, same types.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

ROWS, WIDTH = 14336, 4096
SWEEP = [("Q8_0", 8, 34, 32), ("Q6_K", 14, 210, 256), ("Q5_K", 13, 176, 256), ("Q4_K", 12, 144, 256),
         ("Q3_K", 11, 110, 256), ("Q2_K", 10, 84, 256)]
L2_BYTES = 126 * 1024 * 1024
METRIC = "dequant GB/s (encoded read + fp16/bf16 written)"


def sweep_config(rows: int) -> dict:
    """`config` of the bench line; the same dictionary for the GPU arm and the CPU reference arm."""
    return {"workload": f"dequant_sweep Q8_0,Q6_K,Q5_K,Q4_K,Q3_K,Q2_K {rows}x{WIDTH} -> fp16+bf16",
            "rows": rows, "width": WIDTH, "qtypes": [s[0] for s in SWEEP], "outputs": ["fp16", "bf16"],
            "inputs": "numpy default_rng(0) standard_normal * 0.02, encoded per type; every row of the matrix is decoded in every step",
            "bytes_per_step": 2 * sum(rows * (WIDTH // bel * bsz + WIDTH * 2) for _, _, bsz, bel in SWEEP),
            "l2": "no flush: every decode moves 137-180 MB (> 126 MB L2) and consecutive decodes use different buffers"}


def peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons from warm-up to the end of the last timed leg: NVML queries from a thread
    of this process (a sample every half millisecond), or, when the NVML binding is missing, an `nvidia-smi -lms`
    child process.  `window()` marks a stretch in which the GPU is kept busy; the reported clock is the median over
    the samples inside such stretches and `samples_under_load` is their number."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.file = None
        self.proc = None
        self.thread = None
        self.samples = []          # (host time, sm MHz, power W, reasons bitmask)
        self.windows = []          # [t0, t1] host times of the loaded stretches
        self.running = False
        self.nvml = None
        self.max_sm = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(device_index))
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    @staticmethod
    def _physical_index(device_index: int) -> int:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if device_index < len(ids) and ids[device_index].isdigit():
                return int(ids[device_index])
        return device_index

    def _loop(self):
        nv = self.nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while self.running:
            try:
                self.samples.append((time.perf_counter(), float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)),
                                     nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0, int(reasons_fn(self.handle))))
            except Exception:
                break
            time.sleep(0.0005)

    def start(self):
        if self.nvml is not None:
            self.running = True
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
            return
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    class _Window:
        def __init__(self, sampler):
            self.sampler = sampler

        def __enter__(self):
            self.t0 = time.perf_counter()

        def __exit__(self, *exc):
            self.sampler.windows.append((self.t0, time.perf_counter()))

    def window(self):
        return ClockSampler._Window(self)

    def stop(self) -> dict:
        if self.thread is not None:
            self.running = False
            self.thread.join(timeout=2)
            if not self.samples:
                return {"sm_mhz": None, "sm_max_mhz": self.max_sm, "reasons": ["no samples"]}
            loaded = [s for s in self.samples if any(a <= s[0] <= b for a, b in self.windows)]
            use = loaded or self.samples
            mask = 0
            for s in use:
                mask |= s[3]
            return {"sm_mhz": statistics.median(s[1] for s in use), "sm_max_mhz": self.max_sm, "samples": len(self.samples),
                    "samples_under_load": len(loaded), "seconds_under_load": round(sum(b - a for a, b in self.windows), 3),
                    "power_w_max": max(s[2] for s in use), "reasons": sorted(n for bit, n in self.REASON_BITS.items() if mask & bit),
                    "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8]
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            for name, v in zip(names, r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]), "samples": len(rows),
                "samples_under_load": None, "power_w_max": max(float(r[3]) for r in rows), "reasons": sorted(reasons),
                "source": "nvidia-smi"}


# ------------------------------------------------------------------------------------------------
def reference_checker():
    from oracle import reference
    if reference.available("ref"):
        return reference.load("ref"), "reference"
    if not reference.available("port"):
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    return reference.load("port"), "port"


def cpu_sweep_step(chk, enc_host: dict, out: np.ndarray, rows: int) -> None:
    """One step of the sweep on the host cores: the 12 decodes (the CPU API writes fp32, so fp16 and bf16 are the
    same call; it is credited with the 2 B/element of the 16-bit outputs all the same)."""
    for _ in range(2):
        for name, qtype, _, _ in SWEEP:
            chk._dequantize(qtype, enc_host[name].ctypes.data, out.ctypes.data, 0, rows, WIDTH)


def cpu_dequant_sweep(enc_host: dict, budget_s: float, rows: int) -> dict:
    """Times the checker's dequantize_chunk over whole steps of the sweep (all `rows` rows, as the GPU arm decodes
    them) until about budget_s seconds have been spent.  Returns GB/s of algorithmic bytes."""
    chk, kind = reference_checker()
    out = np.empty((rows, WIDTH), np.float32)
    step_bytes = 2 * sum(enc_host[name].nbytes + rows * WIDTH * 2 for name, *_ in SWEEP)
    cpu_sweep_step(chk, enc_host, out, rows)  # warm-up (page faults of `out`, thread pool)
    t_total, reps = 0.0, 0
    while t_total < budget_s and reps < 200:
        t0 = time.perf_counter()
        cpu_sweep_step(chk, enc_host, out, rows)
        t_total += time.perf_counter() - t0
        reps += 1
    threads = 1 if kind == "port" else (os.cpu_count() or 1)
    line = {"value": step_bytes * reps / t_total / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{reps} steps of 12 x dequantize_chunk->fp32 of all {rows}x{WIDTH} rows on the host cores, "
                      "credited with encoded + 2 B/elem per decode"}
    from oracle import reference
    if kind == "reference" and reference.available("avx2"):  # upstream's AVX2 build, same calls, a quarter of the time
        avx, t2, r2 = reference.load("avx2"), 0.0, 0
        while t2 < budget_s / 4 and r2 < 200:
            t0 = time.perf_counter()
            cpu_sweep_step(avx, enc_host, out, rows)
            t2 += time.perf_counter() - t0
            r2 += 1
        line["avx2_value"] = step_bytes * r2 / t2 / 1e9
    return line


# ------------------------------------------------------------------------------------------------
def run_reference_arm(args, rank: int, world: int) -> None:
    """upstream's CPU REF backend on the host cores: the same 12 decodes of all 14336 rows per step."""
    if rank != 0:
        return
    import inputs
    chk, kind = reference_checker()
    rows = args.rows
    x = inputs.decode_sweep_matrix(rows, WIDTH)
    enc = {name: chk.quantize_rows(x, qtype) for name, qtype, _, _ in SWEEP}
    out = np.empty((rows, WIDTH), np.float32)
    config = sweep_config(rows)
    for _ in range(max(args.warmup, 1)):
        cpu_sweep_step(chk, enc, out, rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_sweep_step(chk, enc, out, rows)
    dt = time.perf_counter() - t0
    value = config["bytes_per_step"] * args.steps / dt / 1e9
    threads = 1 if kind == "port" else (os.cpu_count() or 1)
    sample = (f"each step = 12 x dequantize_chunk->fp32 of all {rows}x{WIDTH} rows on the host cores, "
              "credited with encoded + 2 B/elem per decode")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dequant_sweep")
    ap.add_argument("--rows", type=int, default=ROWS, help="rows of the weight matrix (smaller for profiling captures)")
    ap.add_argument("--src-dtype", default="f32", choices=["f32", "f16", "bf16"],
                    help="convert workload: dtype of the pinned source tensors (16-bit sources are widened on the GPU)")
    ap.add_argument("--types", default="", help="secondary workloads: comma-separated subset of the workload's types")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="default workload: skip the quant, convert and host_api blocks")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL announces its version on stdout when the first communicator comes up; stdout is kept for the one JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    from libgguf_b200._native import lib
    from libgguf_b200.libgguf_cuda import ops

    if args.workload != "dequant_sweep":
        import bench_quant
        bench_quant.run(args, torch, dist, lib, ops, device, rank, world)
        if world > 1:
            dist.destroy_process_group()
        return

    import inputs
    import bench_quant

    rows = args.rows
    x_host = bench_quant.sweep_matrix(rows, WIDTH)
    x_dev = torch.from_numpy(x_host).to(device)
    enc = {name: ops.quantize(x_dev, qtype) for name, qtype, _, _ in SWEEP}
    del x_dev
    # NSETS distinct copies of every input and output so that consecutive launches of one kernel
    # never touch the same lines: a launch moves 137-180 MB and the L2 holds 126 MB.
    NSETS = 4
    enc_sets = {name: [enc[name]] + [enc[name].clone() for _ in range(NSETS - 1)] for name, *_ in SWEEP}
    out_sets = {dt: [torch.empty((rows, WIDTH), dtype=dt, device=device) for _ in range(NSETS)]
                for dt in (torch.float16, torch.bfloat16)}
    dtype_code = {torch.float16: 1, torch.bfloat16: 2}
    stream = torch.cuda.current_stream(device)
    algo_bytes = {name: enc[name].numel() + rows * WIDTH * 2 for name, *_ in SWEEP}
    step_bytes = 2 * sum(algo_bytes.values())
    config = sweep_config(rows)
    assert config["bytes_per_step"] == step_bytes

    def decode(name, qtype, dt, k):
        st = lib.libgguf_cuda_dequantize_rows_on_stream(enc_sets[name][k % NSETS].data_ptr(), qtype, rows, WIDTH, dtype_code[dt],
                                                        out_sets[dt][k % NSETS].data_ptr(), stream.cuda_stream)
        if st != 0:
            raise RuntimeError(lib.libgguf_cuda_thread_last_error().decode())

    def run_steps(nsteps, events=None):
        """nsteps passes over the sweep.  The launches are issued kernel-major (all nsteps launches of
        one (qtype, dtype) kernel back to back, each on its own buffer set) so that one event pair
        brackets every kernel's launches without sitting between two short kernels."""
        for dt in (torch.float16, torch.bfloat16):
            for name, qtype, _, _ in SWEEP:
                if events is not None:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                for k in range(nsteps):
                    decode(name, qtype, dt, k)
                if events is not None:
                    b.record(stream)
                    events.append((name, a, b))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return float(v)
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    sampler.start()
    warm = max(args.warmup, 3)
    with sampler.window():
        run_steps(warm)
        barrier()
        launches0 = lib.libgguf_cuda_kernel_launch_count()
        events = []
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_start.record(stream)
        run_steps(args.steps, events)
        t_end.record(stream)
        barrier()
    launches = lib.libgguf_cuda_kernel_launch_count() - launches0
    ms = max_over_ranks(t_start.elapsed_time(t_end))
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9

    # per-kernel durations inside the timed region
    per = {}
    for name, a, b in events:
        per.setdefault(name, []).append(a.elapsed_time(b) / args.steps)
    hbm, peak_kind = peaks()
    per_qtype = {}
    for name in per:
        mean_ms = statistics.fmean(per[name])
        gbs = algo_bytes[name] / (mean_ms * 1e-3) / 1e9
        per_qtype[name] = {"ms": round(mean_ms, 5), "GB/s": round(gbs, 1), "frac": round(gbs / hbm, 4)}
    dominant = max(per, key=lambda n: sum(per[n]))
    dom_ms = statistics.fmean(per[dominant])
    achieved = algo_bytes[dominant] / (dom_ms * 1e-3) / 1e9
    traffic = None
    tfile = ROOT / "profiles" / "traffic.json"
    if tfile.exists():
        t = json.loads(tfile.read_text()).get(f"dequant_{dominant}")
        if t:
            traffic = t["dram_bytes_per_elem"] * rows * WIDTH
    roofline = {"bound": "hbm", "kernel": f"dequant_fast_kernel<{dominant}, fp16|bf16>", "achieved": achieved, "peak": hbm,
                "unit": "GB/s", "frac": achieved / hbm, "traffic": traffic, "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": algo_bytes[dominant], "launch_ms": dom_ms}

    # what the timed kernels wrote, against the CPU checker (outside every timed region)
    verified = verify_sweep(torch, lib, x_host, enc, out_sets, rows, decode) if rank == 0 else None

    # end to end through the device-pointer C ABI with pinned host buffers, and the plain-copy ceiling beside it
    e2e = roofline_e2e = None
    if not args.no_e2e:
        with sampler.window():
            e2e = run_e2e(torch, lib, enc, rows, local_rank, world, dist if world > 1 else None, device,
                          max(2, min(args.steps, 5)))
        if e2e is not None:
            with sampler.window():
                roofline_e2e = link_ceiling(torch, lib, enc, rows, local_rank, world, dist if world > 1 else None, device, e2e)

    del enc_sets, out_sets
    torch.cuda.empty_cache()
    quant = convert = host_api = None
    if not args.no_extras:
        with sampler.window():
            quant = bench_quant.quant_block(torch, dist if world > 1 else None, lib, device, rank, world, hbm,
                                            check=(rank == 0), cpu=(rank == 0 and world == 1 and not args.no_cpu_baseline))
        if world == 1 and roofline_e2e is not None:
            host_api = host_pointer_e2e(lib, x_host, roofline_e2e)
        link = roofline_e2e if world > 1 or args.gpus == 1 else None
        convert = bench_quant.convert_block(torch, dist if world > 1 else None, lib, device, rank, world, link=link, gpus=args.gpus,
                                            keep_sources=True)
        # the same set from a bf16 checkpoint: the 16-bit values cross the host link as they are and are widened on the GPU
        convert["bf16_source"] = bench_quant.convert_block(torch, dist if world > 1 else None, lib, device, rank, world, link=link,
                                                           gpus=args.gpus, src_dtype="bf16", reuse=convert.pop("_sources"))
    clocks = sampler.stop()
    if quant is not None and clocks.get("sm_mhz"):
        bench_quant.add_issue_fractions(quant, clocks["sm_mhz"])

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        enc_host = {name: enc[name].cpu().numpy() for name, *_ in SWEEP}
        cpu = cpu_dequant_sweep(enc_host, budget_s=12.0, rows=rows)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "notes": {"per_gpu_bytes_per_step": step_bytes, "buffer_sets": NSETS,
                      "launch_order": "kernel-major: the K launches of each of the 12 kernels run back to back inside one CUDA-event pair"},
            "clocks": clocks, "e2e": e2e, "roofline_e2e": roofline_e2e, "gpu_launches": int(launches), "roofline": roofline,
            "per_qtype": per_qtype, "verified": verified, "quant": quant, "convert": convert, "host_api": host_api,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def verify_sweep(torch, lib, x_host, enc, out_sets, rows, decode) -> dict:
    """After the timed region: every (type, output dtype) kernel of the sweep is launched once more on the buffers the
    timed launches used (they share their output buffers, so only the last kernel's output survives the sweep itself),
    and the first and the last 256 rows are compared with the CPU checker: the encoded bytes the sweep decodes equal
    the checker's encoding of the same input rows, and the decode equals the checker's fp32 decode rounded to
    nearest-even (bit patterns).  The checker only checks here; nothing it computes is timed or shipped."""
    chk, kind = reference_checker()
    n = min(rows, 256)
    ok = True
    detail = {}
    for name, qtype, _, _ in SWEEP:
        good = True
        for sl in (slice(0, n), slice(rows - n, rows)):
            want = chk.quantize_rows(x_host[sl], qtype)
            good = good and bool(np.array_equal(enc[name][sl].cpu().numpy(), want))
            ref32 = torch.from_numpy(chk.dequantize_rows(want, qtype, WIDTH))
            for dt, outs in out_sets.items():
                decode(name, qtype, dt, 0)
                torch.cuda.synchronize()
                good = good and bool(torch.equal(outs[0][sl].cpu().view(torch.int16), ref32.to(dt).view(torch.int16)))
        detail[name] = good
        ok = ok and good
    return {"ok": ok, "rows_checked": 2 * n, "checker": kind, "per_qtype": detail}


class _Slot:
    pass


def _make_slots(lib, device_index, count, in_bytes, out_bytes):
    slots = []
    for _ in range(count):
        sl = _Slot()
        sl.ctx = ctypes.c_void_p()
        if lib.libgguf_cuda_context_create(device_index, ctypes.byref(sl.ctx)) != 0:
            return None
        sl.d_in, sl.d_out, sl.h_out, sl.ev = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        for st in (lib.libgguf_cuda_buffer_create(sl.ctx, in_bytes, ctypes.byref(sl.d_in)),
                   lib.libgguf_cuda_buffer_create(sl.ctx, out_bytes, ctypes.byref(sl.d_out)),
                   lib.libgguf_cuda_host_buffer_create(sl.ctx, out_bytes, ctypes.byref(sl.h_out)),
                   lib.libgguf_cuda_event_create(sl.ctx, ctypes.byref(sl.ev))):
            if st != 0:
                raise RuntimeError(lib.libgguf_cuda_last_error(sl.ctx).decode())
        slots.append(sl)
    return slots


def _free_slots(lib, slots):
    for sl in slots:
        lib.libgguf_cuda_event_destroy(sl.ctx, sl.ev)
        lib.libgguf_cuda_host_buffer_destroy(sl.ctx, sl.h_out)
        lib.libgguf_cuda_buffer_destroy(sl.ctx, sl.d_in)
        lib.libgguf_cuda_buffer_destroy(sl.ctx, sl.d_out)
        lib.libgguf_cuda_context_destroy(sl.ctx)


def _pinned_inputs(lib, ctx, enc):
    h_in = {}
    for name, t in enc.items():
        hb = ctypes.c_void_p()
        if lib.libgguf_cuda_host_buffer_create(ctx, t.numel(), ctypes.byref(hb)) != 0:
            raise RuntimeError(lib.libgguf_cuda_last_error(ctx).decode())
        host_copy = t.cpu().numpy()  # keep the array alive while memmove reads it
        ctypes.memmove(lib.libgguf_cuda_host_buffer_data(hb), host_copy.ctypes.data, host_copy.nbytes)
        del host_copy
        h_in[name] = hb
    return h_in


E2E_SLOTS = 3


def run_e2e(torch, lib, enc, rows, device_index, world, dist, device, steps):
    """h2d(encoded, pinned) -> dequantize_rows -> d2h(fp16/bf16, pinned) for the 12 decodes of a step,
    through libgguf_cuda_* with three library contexts used in turn (each owns a stream, a device
    input/output buffer and a pinned result buffer), so that one decode's upload and kernel overlap the
    downloads of the two before it the way the converter's slots do.  Timed with the host wall
    clock around a final event synchronize on every context; max over ranks."""
    max_enc = max(t.numel() for t in enc.values())
    out_bytes = rows * WIDTH * 2
    slots = _make_slots(lib, device_index, E2E_SLOTS, max_enc, out_bytes)
    if slots is None:
        return None

    def chk(sl, st):
        if st != 0:
            raise RuntimeError(lib.libgguf_cuda_last_error(sl.ctx).decode())

    first = slots[0]
    h_in = _pinned_inputs(lib, first.ctx, enc)
    h2d = d2h = 0

    def step():
        nonlocal h2d, d2h
        h2d = d2h = 0
        k = 0
        for dt in (1, 2):
            for name, qtype, _, _ in SWEEP:
                sl = slots[k % E2E_SLOTS]
                if k >= E2E_SLOTS:  # the slot's previous result has to be on the host before its buffers are reused
                    chk(sl, lib.libgguf_cuda_event_synchronize(sl.ctx, sl.ev))
                n = enc[name].numel()
                chk(sl, lib.libgguf_cuda_buffer_resize_discard(sl.ctx, sl.d_in, n))
                chk(sl, lib.libgguf_cuda_h2d(sl.ctx, sl.d_in, 0, lib.libgguf_cuda_host_buffer_data(h_in[name]), n))
                chk(sl, lib.libgguf_cuda_dequantize_rows(sl.ctx, lib.libgguf_cuda_buffer_data(sl.d_in), qtype, rows, WIDTH, dt,
                                                         lib.libgguf_cuda_buffer_data(sl.d_out)))
                chk(sl, lib.libgguf_cuda_d2h(sl.ctx, lib.libgguf_cuda_host_buffer_data(sl.h_out), sl.d_out, 0, out_bytes))
                chk(sl, lib.libgguf_cuda_event_record(sl.ctx, sl.ev))
                h2d += n
                d2h += out_bytes
                k += 1
        for sl in slots:
            chk(sl, lib.libgguf_cuda_event_synchronize(sl.ctx, sl.ev))

    step()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([dt], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    algo = 2 * sum(enc[name].numel() + out_bytes for name, *_ in SWEEP)
    for hb in h_in.values():
        lib.libgguf_cuda_host_buffer_destroy(first.ctx, hb)
    _free_slots(lib, slots)
    return {"value": world * algo * steps / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "seconds_per_step": dt / steps,
            "api": f"libgguf_cuda_h2d + libgguf_cuda_dequantize_rows + libgguf_cuda_d2h, pinned host buffers, {E2E_SLOTS} contexts in turn"}


def link_ceiling(torch, lib, enc, rows, device_index, world, dist, device, e2e) -> dict:
    """What the host link allows for the e2e leg: the same pinned buffers, the same byte counts per step in each
    direction, plain asynchronous copies and no kernels -- all uploads of a step on one stream, all downloads on
    another, both in flight together (a GPU has a copy engine per direction) -- on every rank at once.  Also each
    direction alone.  `ceiling` is the e2e metric a pipeline with free kernels would reach; times are max over ranks."""
    out_bytes = rows * WIDTH * 2
    max_enc = max(t.numel() for t in enc.values())
    slots = _make_slots(lib, device_index, 2, max_enc, out_bytes)
    if slots is None:
        return None
    up, down = slots

    def chk(sl, st):
        if st != 0:
            raise RuntimeError(lib.libgguf_cuda_last_error(sl.ctx).decode())

    h_in = _pinned_inputs(lib, up.ctx, enc)

    def uploads():
        for _ in range(2):
            for name, *_ in SWEEP:
                chk(up, lib.libgguf_cuda_h2d(up.ctx, up.d_in, 0, lib.libgguf_cuda_host_buffer_data(h_in[name]), enc[name].numel()))
        chk(up, lib.libgguf_cuda_event_record(up.ctx, up.ev))

    def downloads():
        for _ in range(2 * len(SWEEP)):
            chk(down, lib.libgguf_cuda_d2h(down.ctx, lib.libgguf_cuda_host_buffer_data(down.h_out), down.d_out, 0, out_bytes))
        chk(down, lib.libgguf_cuda_event_record(down.ctx, down.ev))

    def timed(fns, reps=3):
        for f in fns:
            f()
        for sl in (up, down):
            lib.libgguf_cuda_event_synchronize(sl.ctx, sl.ev)
        if dist is not None:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            for f in fns:
                f()
        for sl in (up, down):
            chk(sl, lib.libgguf_cuda_event_synchronize(sl.ctx, sl.ev))
        dt = (time.perf_counter() - t0) / reps
        if dist is not None:
            t = torch.tensor([dt], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt

    # a first record on both events so that synchronising an unused one is defined
    chk(up, lib.libgguf_cuda_event_record(up.ctx, up.ev))
    chk(down, lib.libgguf_cuda_event_record(down.ctx, down.ev))
    t_up, t_down, t_mix = timed([uploads]), timed([downloads]), timed([uploads, downloads])
    for hb in h_in.values():
        lib.libgguf_cuda_host_buffer_destroy(up.ctx, hb)
    _free_slots(lib, slots)
    h2d, d2h = e2e["h2d_bytes_per_step"], e2e["d2h_bytes_per_step"]
    algo = 2 * sum(enc[name].numel() + out_bytes for name, *_ in SWEEP)
    ceiling = world * algo / t_mix / 1e9
    return {"bound": "host_link", "unit": "GB/s", "ceiling": ceiling, "achieved": e2e["value"], "frac": e2e["value"] / ceiling,
            "h2d_alone_GBps": world * h2d / t_up / 1e9, "d2h_alone_GBps": world * d2h / t_down / 1e9,
            "mix_h2d_GBps": world * h2d / t_mix / 1e9, "mix_d2h_GBps": world * d2h / t_mix / 1e9,
            "seconds_per_step_copies_only": t_mix, "n_gpus": world,
            "how": "cudaMemcpyAsync of a step's bytes from / to the same pinned buffers, uploads and downloads on two streams, "
                   "no kernels, all ranks at once; aggregate over ranks, slowest rank's time"}


def host_pointer_e2e(lib, x_host, link) -> dict:
    """The host-pointer ABI a CPU caller binds (libgguf_quantize_chunk / libgguf_dequantize_chunk) on pageable
    memory: Q4_K of the 14336x4096 matrix and back, best of three, as GB/s of the bytes that cross the host link and
    as a fraction of the plain pinned-copy rate of the dominant direction."""
    rows, width = x_host.shape
    rs = int(lib.libgguf_row_size(12, width))
    enc = np.empty(rows * rs, np.uint8)
    dec = np.empty((rows, width), np.float32)
    tq, td = [], []
    for _ in range(4):
        t0 = time.perf_counter()
        wrote = lib.libgguf_quantize_chunk(12, x_host.ctypes.data, enc.ctypes.data, 0, rows, width, None)
        t1 = time.perf_counter()
        got = lib.libgguf_dequantize_chunk(12, enc.ctypes.data, dec.ctypes.data, 0, rows, width)
        t2 = time.perf_counter()
        if wrote != rows * rs or got != rows * width * 4:
            return {"error": "host-pointer call failed"}
        tq.append(t1 - t0)
        td.append(t2 - t1)
    moved = x_host.nbytes + enc.nbytes
    q, d = min(tq[1:]), min(td[1:])
    return {"workload": f"Q4_K {rows}x{width} from / to pageable host memory",
            "quantize_chunk": {"ms": round(q * 1e3, 3), "link_GBps": round(moved / q / 1e9, 2),
                               "frac_of_h2d_rate": round(moved / q / 1e9 / link["h2d_alone_GBps"], 3)},
            "dequantize_chunk": {"ms": round(d * 1e3, 3), "link_GBps": round(moved / d / 1e9, 2),
                                 "frac_of_d2h_rate": round(moved / d / 1e9 / link["d2h_alone_GBps"], 3)},
            "note": "pageable memory: the library copies through its two pinned slots with a pool of host threads, so the "
                    "bound is host memcpy + the link, not the link alone"}


if __name__ == "__main__":
    main()
