#!/usr/bin/env python3
"""Benchmark of the GGUF row quantize / dequantize hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload `dequant_sweep` is the BASELINE configuration the headline metric is quoted on:
decode a 14336x4096 weight matrix from Q8_0, Q6_K, Q5_K, Q4_K, Q3_K and Q2_K to fp16 and to
bf16.  One step = the 12 decodes.  `value` counts algorithmic bytes (encoded bytes read + 2 bytes
per element written) per second with inputs resident in HBM; `e2e` is the same metric through
the device-pointer C ABI with pinned HOST buffers, copies included.  Other workloads
(`q4k_roundtrip`, `kquant`, `fp4`, `iq`) time the quantizers of the remaining BASELINE
configurations in Melem/s.

Under torchrun every rank runs the same per-GPU workload on its own device (weak scaling, no
collective on the data path); the reported time is the maximum over ranks.

`--impl reference` times upstream's own CPU implementation (oracle/_ref, built from the upstream
sources; the C restatement if that library is absent) on the host cores.
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
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, WIDTH = 14336, 4096
SWEEP = [("Q8_0", 8, 34, 32), ("Q6_K", 14, 210, 256), ("Q5_K", 13, 176, 256), ("Q4_K", 12, 144, 256),
         ("Q3_K", 11, 110, 256), ("Q2_K", 10, 84, 256)]
L2_BYTES = 126 * 1024 * 1024


def peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons sampled while the timed region runs: NVML queries from a thread of this
    process (about a sample per millisecond, so even a region of a few milliseconds is covered), or, when the NVML
    binding is missing, an `nvidia-smi -lms` child process."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.file = None
        self.proc = None
        self.thread = None
        self.samples = []          # (sm MHz, power W, reasons bitmask)
        self.running = False
        self.nvml = None
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
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)),
                                     nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0, int(reasons_fn(self.handle))))
            except Exception:
                break
            time.sleep(0.0005)

    def start(self):
        if self.nvml is not None:
            import threading
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

    def stop(self) -> dict:
        if self.thread is not None:
            self.running = False
            self.thread.join(timeout=2)
            if not self.samples:
                return {"sm_mhz": None, "sm_max_mhz": self.max_sm, "reasons": ["no samples"]}
            mask = 0
            for _, _, r in self.samples:
                mask |= r
            return {"sm_mhz": statistics.median(s[0] for s in self.samples), "sm_max_mhz": self.max_sm, "samples": len(self.samples),
                    "power_w_max": max(s[1] for s in self.samples), "reasons": sorted(n for bit, n in self.REASON_BITS.items() if mask & bit),
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
                "power_w_max": max(float(r[3]) for r in rows), "reasons": sorted(reasons), "source": "nvidia-smi"}


# ------------------------------------------------------------------------------------------------
def reference_checker():
    from oracle import reference
    if reference.available("ref"):
        return reference.load("ref"), "reference"
    if not reference.available("port"):
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    return reference.load("port"), "port"


def cpu_dequant_sweep(enc_host: dict[str, np.ndarray], budget_s: float, rows: int) -> dict:
    """Times the checker's dequantize_chunk over the sweep on the first `rows` rows, repeated
    until about budget_s seconds have been spent.  Returns GB/s of algorithmic bytes."""
    chk, kind = reference_checker()
    out = np.empty((rows, WIDTH), np.float32)
    algo = 0
    t_total = 0.0
    reps = 0
    while t_total < budget_s and reps < 50:
        for name, qtype, bsz, bel in SWEEP:
            enc = enc_host[name][:rows]
            t0 = time.perf_counter()
            chk._dequantize(qtype, enc.ctypes.data, out.ctypes.data, 0, rows, WIDTH)
            t_total += time.perf_counter() - t0
            algo += enc.nbytes + rows * WIDTH * 2
        reps += 1
    threads = 1 if kind == "port" else (os.cpu_count() or 1)
    line = {"value": algo / t_total / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{reps} x dequantize_chunk->fp32 of {rows}x{WIDTH} for {len(SWEEP)} qtypes on host cores, "
                      "credited with encoded + 2 B/elem per decode"}
    from oracle import reference
    if kind == "reference" and reference.available("avx2"):  # upstream's AVX2 build, same calls, a quarter of the time
        avx, algo2, t2, r2 = reference.load("avx2"), 0, 0.0, 0
        while t2 < budget_s / 4 and r2 < 50:
            for name, qtype, bsz, bel in SWEEP:
                enc = enc_host[name][:rows]
                t0 = time.perf_counter()
                avx._dequantize(qtype, enc.ctypes.data, out.ctypes.data, 0, rows, WIDTH)
                t2 += time.perf_counter() - t0
                algo2 += enc.nbytes + rows * WIDTH * 2
            r2 += 1
        line["avx2_value"] = algo2 / t2 / 1e9
    return line


def make_encoded_on_gpu(torch, ops, device, rows=ROWS) -> dict:
    g = torch.Generator(device=device)
    g.manual_seed(0)
    w = torch.randn((rows, WIDTH), generator=g, device=device, dtype=torch.float32) * 0.02
    return {name: ops.quantize(w, qtype) for name, qtype, _, _ in SWEEP}


# ------------------------------------------------------------------------------------------------
def run_reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    chk, kind = reference_checker()
    rows = 2048  # bounded sample of the 14336-row matrix
    x = (np.random.default_rng(0).standard_normal((rows, WIDTH), dtype=np.float32) * np.float32(0.02))
    enc = {}
    for name, qtype, _, _ in SWEEP:
        enc[name] = chk.quantize_rows(x, qtype)
    out = np.empty((rows, WIDTH), np.float32)
    step_bytes = sum(2 * (enc[n].nbytes + rows * WIDTH * 2) for n, *_ in SWEEP)

    def step():
        for dt in range(2):
            for name, qtype, _, _ in SWEEP:
                chk._dequantize(qtype, enc[name].ctypes.data, out.ctypes.data, 0, rows, WIDTH)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = step_bytes * args.steps / dt / 1e9
    threads = 1 if kind == "port" else (os.cpu_count() or 1)
    sample = (f"each step = 12 x dequantize_chunk->fp32 of a {rows}x{WIDTH} slice (of {ROWS}x{WIDTH}) on host cores, "
              "credited with encoded + 2 B/elem per decode")
    print(json.dumps({
        "impl": "reference", "metric": "dequant GB/s (encoded read + fp16/bf16 written)", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "dequant_sweep Q8_0,Q6_K,Q5_K,Q4_K,Q3_K,Q2_K 14336x4096 -> fp16+bf16", "rows_timed": rows},
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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
        dist.init_process_group("nccl", device_id=device)

    from libgguf_b200._native import lib
    from libgguf_b200.libgguf_cuda import ops

    if args.workload != "dequant_sweep":
        import bench_quant
        bench_quant.run(args, torch, dist, lib, ops, device, rank, world)
        if world > 1:
            dist.destroy_process_group()
        return

    rows = args.rows
    enc = make_encoded_on_gpu(torch, ops, device, rows)
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

    run_steps(max(args.warmup, 3))
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = lib.libgguf_cuda_kernel_launch_count()
    events = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record(stream)
    run_steps(args.steps, events)
    t_end.record(stream)
    barrier()
    launches = lib.libgguf_cuda_kernel_launch_count() - launches0
    clocks = sampler.stop()
    ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
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

    # end to end through the device-pointer C ABI with pinned host buffers
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(torch, lib, enc, rows, local_rank, world, dist if world > 1 else None, device,
                      max(2, min(args.steps, 5)))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        enc_host = {name: enc[name].cpu().numpy() for name, *_ in SWEEP}
        cpu = cpu_dequant_sweep(enc_host, budget_s=12.0, rows=min(rows, 4096))

    if rank == 0:
        line = {
            "metric": "dequant GB/s (encoded read + fp16/bf16 written)", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"dequant_sweep Q8_0,Q6_K,Q5_K,Q4_K,Q3_K,Q2_K {rows}x{WIDTH} -> fp16+bf16",
                       "per_gpu_bytes_per_step": step_bytes,
                       "l2": "no flush: every launch moves 137-180 MB (> 126 MB L2) and consecutive launches rotate over 4 distinct input/output buffer sets",
                       "launch_order": "kernel-major: the K launches of each of the 12 kernels run back to back inside one CUDA-event pair"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "per_qtype": per_qtype,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_e2e(torch, lib, enc, rows, device_index, world, dist, device, steps):
    """h2d(encoded, pinned) -> dequantize_rows -> d2h(fp16/bf16, pinned) for the 12 decodes of a step,
    through libgguf_cuda_* with two library contexts used alternately (each owns a stream, a device
    input/output buffer and a pinned result buffer), so that one decode's upload overlaps the
    previous decode's download the way the converter's two slots do.  Timed with the host wall
    clock around a final event synchronize on both contexts; max over ranks."""
    NCTX = 2
    max_enc = max(t.numel() for t in enc.values())
    out_bytes = rows * WIDTH * 2

    class Slot:
        pass

    slots = []
    for _ in range(NCTX):
        sl = Slot()
        sl.ctx = ctypes.c_void_p()
        if lib.libgguf_cuda_context_create(device_index, ctypes.byref(sl.ctx)) != 0:
            return None
        sl.d_in, sl.d_out, sl.h_out, sl.ev = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        slots.append(sl)

    def chk(sl, st):
        if st != 0:
            raise RuntimeError(lib.libgguf_cuda_last_error(sl.ctx).decode())

    for sl in slots:
        chk(sl, lib.libgguf_cuda_buffer_create(sl.ctx, max_enc, ctypes.byref(sl.d_in)))
        chk(sl, lib.libgguf_cuda_buffer_create(sl.ctx, out_bytes, ctypes.byref(sl.d_out)))
        chk(sl, lib.libgguf_cuda_host_buffer_create(sl.ctx, out_bytes, ctypes.byref(sl.h_out)))
        chk(sl, lib.libgguf_cuda_event_create(sl.ctx, ctypes.byref(sl.ev)))
    first = slots[0]
    h_in = {}
    for name, t in enc.items():
        hb = ctypes.c_void_p()
        chk(first, lib.libgguf_cuda_host_buffer_create(first.ctx, t.numel(), ctypes.byref(hb)))
        host_copy = t.cpu().numpy()  # keep the array alive while memmove reads it
        ctypes.memmove(lib.libgguf_cuda_host_buffer_data(hb), host_copy.ctypes.data, host_copy.nbytes)
        del host_copy
        h_in[name] = hb
    h2d = d2h = 0

    def step():
        nonlocal h2d, d2h
        h2d = d2h = 0
        k = 0
        for dt in (1, 2):
            for name, qtype, _, _ in SWEEP:
                sl = slots[k % NCTX]
                if k >= NCTX:  # the slot's previous result has to be on the host before its buffers are reused
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
    for sl in slots:
        lib.libgguf_cuda_event_destroy(sl.ctx, sl.ev)
        lib.libgguf_cuda_host_buffer_destroy(sl.ctx, sl.h_out)
        lib.libgguf_cuda_buffer_destroy(sl.ctx, sl.d_in)
        lib.libgguf_cuda_buffer_destroy(sl.ctx, sl.d_out)
        lib.libgguf_cuda_context_destroy(sl.ctx)
    return {"value": world * algo * steps / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "api": "libgguf_cuda_h2d + libgguf_cuda_dequantize_rows + libgguf_cuda_d2h, pinned host buffers, 2 contexts alternating"}


if __name__ == "__main__":
    main()
