"""Secondary workloads of bench.py (`--workload NAME`): the quantizer and conversion configurations.

  q4k_roundtrip  BASELINE config 1: Q4_K quantize + dequantize->fp32 of 4096x4096 N(0, 0.02)
  kquant         quantize 14336x4096 to Q8_0, Q6_K, Q5_K, Q4_K, Q3_K, Q2_K
  legacy         quantize 14336x4096 to Q4_0, Q4_1, Q5_0, Q5_1, Q1_0, TQ1_0, TQ2_0, IQ4_NL, IQ4_XS
  iq             BASELINE config 4: IQ2_XXS, IQ2_S, IQ3_XXS, IQ1_S (+ IQ2_XS, IQ3_S, IQ1_M) on 4096x11008
                 Student-t(5)*0.02 with a chi-square(4)/4 imatrix
  fp4            BASELINE config 5: MXFP4 / NVFP4 quantize and dequantize->bf16 of 8192x8192 Laplace(0, 0.01)
  convert        BASELINE config 3: synthetic Llama-3-8B-shaped weight set through the multi-GPU streaming
                 pipeline (pinned host memory in and out), Q4_K_M-style mix

Each prints one JSON line: metric Melem/s (GB/s of source for `convert`), per-type table with the fraction of the
bound that applies (HBM for the cheap encoders, fp32 issue rate for the search-heavy ones).
Inputs live in HBM; every timed launch uses one of NSETS distinct input/output buffer sets."""
from __future__ import annotations

import json
import os
import statistics
import time

NSETS = 3
FP32_LANES = 148 * 128  # fp32 lanes of a B200

# flop per element of the upstream algorithm (no FMA), for the pipe-bound encoders: candidates x (operations per
# element and candidate) of the scale searches
FLOP_PER_ELEM = {"Q4_K": 480, "Q5_K": 370, "Q2_K": 375, "Q6_K": 280, "Q3_K": 125, "MXFP4": 85, "NVFP4": 85}

BLOCK = {"Q4_0": (32, 18), "Q4_1": (32, 20), "Q5_0": (32, 22), "Q5_1": (32, 24), "Q8_0": (32, 34), "Q1_0": (128, 18),
         "MXFP4": (32, 17), "NVFP4": (64, 36), "Q2_K": (256, 84), "Q3_K": (256, 110), "Q4_K": (256, 144),
         "Q5_K": (256, 176), "Q6_K": (256, 210), "TQ1_0": (256, 54), "TQ2_0": (256, 66), "IQ2_XXS": (256, 66),
         "IQ2_XS": (256, 74), "IQ2_S": (256, 82), "IQ3_XXS": (256, 98), "IQ3_S": (256, 110), "IQ1_S": (256, 50),
         "IQ1_M": (256, 56), "IQ4_NL": (32, 18), "IQ4_XS": (256, 136)}
CODE = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14,
        "IQ2_XXS": 16, "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19, "IQ4_NL": 20, "IQ3_S": 21, "IQ2_S": 22, "IQ4_XS": 23,
        "IQ1_M": 29, "TQ1_0": 34, "TQ2_0": 35, "MXFP4": 39, "NVFP4": 40, "Q1_0": 41}


def _time_launches(torch, stream, fn, reps):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for k in range(reps):
        fn(k)
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _make_input(torch, device, kind, rows, cols, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    if kind == "normal":
        return torch.randn((rows, cols), generator=g, device=device) * 0.02
    if kind == "student":
        z = torch.randn((rows, cols), generator=g, device=device)
        chi = sum(torch.randn((rows, cols), generator=g, device=device) ** 2 for _ in range(5))
        return z / torch.sqrt(chi / 5) * 0.02
    if kind == "laplace":
        u = torch.rand((rows, cols), generator=g, device=device) - 0.5
        x = -0.01 * torch.sign(u) * torch.log1p(-2 * u.abs())
        x = x.to(torch.bfloat16).to(torch.float32)
        nblk = rows * cols // 32
        pick = torch.randperm(nblk, generator=g, device=device)[: max(1, nblk // 100)]
        pos = torch.randint(0, 32, (pick.numel(),), generator=g, device=device)
        sign = torch.randint(0, 2, (pick.numel(),), generator=g, device=device).float() * 2 - 1
        flat = x.reshape(-1)
        flat[pick * 32 + pos] = (sign * 50 * 0.01 * 2 ** 0.5).to(torch.bfloat16).to(torch.float32)
        return flat.reshape(rows, cols)
    raise ValueError(kind)


def cpu_quantize_baseline(x_host, im_host, types, seconds_per_type=1.5):
    """Upstream's CPU quantizers (REF build, and the AVX2 build when present) on the first rows of the same input,
    all host threads: rows are doubled until a call lasts about `seconds_per_type`.  Melem/s per type and backend."""
    import numpy as np
    from oracle import reference
    kinds = [k for k in ("ref", "avx2") if reference.available(k)]
    if not kinds:
        kinds = ["port"]
    cores = os.cpu_count() or 1
    per_type, totals = {}, {k: [0.0, 0.0] for k in kinds}
    for kind in kinds:
        chk = reference.load(kind)
        for name in types:
            code = CODE[name]
            rs = chk.row_size(code, x_host.shape[1])
            rows = min(x_host.shape[0], max(cores, 16))
            one = np.ascontiguousarray(x_host[:1])  # first use builds the type's search tables: not timed
            one_out = np.empty(rs, np.uint8)
            chk._quantize(code, one.ctypes.data, one_out.ctypes.data, 0, 1, one.shape[1],
                          im_host.ctypes.data if im_host is not None else None)
            while True:
                src = np.ascontiguousarray(x_host[:rows])
                dst = np.empty(rows * rs, np.uint8)
                t0 = time.perf_counter()
                wrote = chk._quantize(code, src.ctypes.data, dst.ctypes.data, 0, rows, src.shape[1],
                                      im_host.ctypes.data if im_host is not None else None)
                dt = time.perf_counter() - t0
                if wrote != rows * rs:
                    raise RuntimeError(f"CPU {kind} quantize_chunk failed for {name}")
                if dt >= seconds_per_type / 4 or rows >= x_host.shape[0]:
                    break
                rows = min(x_host.shape[0], rows * 4)
            per_type.setdefault(name, {})[f"cpu_{kind}_Melem/s"] = round(rows * src.shape[1] / dt / 1e6, 1)
            per_type[name][f"cpu_{kind}_rows"] = rows
            totals[kind][0] += rows * src.shape[1]
            totals[kind][1] += dt
    first = kinds[0]
    out = {"value": round(totals[first][0] / totals[first][1] / 1e6, 1), "unit": "Melem/s",
           "cores": 1 if first == "port" else cores, "kind": "port" if first == "port" else "reference",
           "sample": "libgguf_quantize_chunk on the first rows of the same input per type (rows grown until a call lasts "
                     f"about {seconds_per_type / 4:.1f}-{seconds_per_type:.1f} s), all host threads; aggregate over the types"}
    if "avx2" in kinds:
        out["avx2_value"] = round(totals["avx2"][0] / totals["avx2"][1] / 1e6, 1)
    return out, per_type


def run(args, torch, dist, lib, ops, device, rank, world):
    import bench
    stream = torch.cuda.current_stream(device)
    hbm, peak_kind = bench.peaks()
    wl = args.workload
    if wl == "convert":
        return run_convert(args, torch, dist, lib, device, rank, world, hbm)
    if wl == "convert_file":
        return run_convert_file(args, torch, lib, rank, world)
    if wl == "dequant_all":
        return run_dequant_all(args, torch, lib, ops, device, rank, world, hbm, peak_kind)
    shapes = {"q4k_roundtrip": (4096, 4096, "normal", ["Q4_K"], False),
              "kquant": (14336, 4096, "normal", ["Q8_0", "Q6_K", "Q5_K", "Q4_K", "Q3_K", "Q2_K"], False),
              "legacy": (14336, 4096, "normal", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q1_0", "TQ1_0", "TQ2_0", "IQ4_NL", "IQ4_XS"], False),
              "iq": (4096, 11008, "student", ["IQ2_XXS", "IQ2_S", "IQ3_XXS", "IQ1_S", "IQ2_XS", "IQ3_S", "IQ1_M"], True),
              "fp4": (8192, 8192, "laplace", ["MXFP4", "NVFP4"], False)}
    rows, cols, kind, types, weighted = shapes[wl]
    if args.rows != bench.ROWS:
        rows = args.rows
    xs = [_make_input(torch, device, kind, rows, cols, seed) for seed in range(NSETS)]
    im = None
    if weighted:
        g = torch.Generator(device=device)
        g.manual_seed(1)
        im = (sum(torch.randn(cols, generator=g, device=device) ** 2 for _ in range(4)) / 4).contiguous()
    n = rows * cols
    sampler = bench.ClockSampler(int(device.index or 0))
    launches0 = lib.libgguf_cuda_kernel_launch_count()
    table = {}
    reps = max(1, args.steps)
    total_ms = 0.0
    sampler.start()
    for name in types:
        code, (bel, bby) = CODE[name], BLOCK[name]
        enc_bytes = n // bel * bby
        outs = [torch.empty((rows, cols // bel * bby), dtype=torch.uint8, device=device) for _ in range(NSETS)]

        def quant(k):
            st = lib.libgguf_cuda_quantize_f32_rows_on_stream(xs[k % NSETS].data_ptr(), im.data_ptr() if im is not None else None,
                                                              outs[k % NSETS].data_ptr(), code, rows, cols, stream.cuda_stream)
            if st != 0:
                raise RuntimeError(lib.libgguf_cuda_thread_last_error().decode())

        for k in range(max(3, args.warmup)):
            quant(k)
        torch.cuda.synchronize()
        ms = _time_launches(torch, stream, quant, reps)
        total_ms += ms
        row = {"quant_ms": round(ms, 4), "quant_Melem/s": round(n / ms / 1e3, 1),
               "quant_GB/s": round((4 * n + enc_bytes) / ms / 1e6, 1), "hbm_frac": round((4 * n + enc_bytes) / ms / 1e6 / hbm, 4)}
        if name in FLOP_PER_ELEM:
            row["fp32_issue_frac_at_max_clock"] = round(FLOP_PER_ELEM[name] * n / (ms * 1e-3) / (FP32_LANES * 1.965e9), 4)
        if wl in ("q4k_roundtrip", "fp4"):
            dt = torch.float32 if wl == "q4k_roundtrip" else torch.bfloat16
            code_dt = 0 if dt == torch.float32 else 2
            dec = [torch.empty((rows, cols), dtype=dt, device=device) for _ in range(NSETS)]

            def dequant(k):
                st = lib.libgguf_cuda_dequantize_rows_on_stream(outs[k % NSETS].data_ptr(), code, rows, cols, code_dt,
                                                                dec[k % NSETS].data_ptr(), stream.cuda_stream)
                if st != 0:
                    raise RuntimeError(lib.libgguf_cuda_thread_last_error().decode())

            for k in range(3):
                dequant(k)
            torch.cuda.synchronize()
            dms = _time_launches(torch, stream, dequant, reps)
            db = enc_bytes + n * dec[0].element_size()
            row.update({"dequant_ms": round(dms, 4), "dequant_GB/s": round(db / dms / 1e6, 1), "dequant_hbm_frac": round(db / dms / 1e6 / hbm, 4)})
            total_ms += dms
            del dec
        table[name] = row
        del outs
    clocks = sampler.stop()
    launches = lib.libgguf_cuda_kernel_launch_count() - launches0
    value = len(types) * n / total_ms / 1e3
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, cpu_rows = cpu_quantize_baseline(xs[0].cpu().numpy(), im.cpu().numpy() if im is not None else None, types)
        for name, extra in cpu_rows.items():
            table[name].update(extra)
    if rank == 0:
        print(json.dumps({
            "metric": "quant Melem/s", "value": value, "unit": "Melem/s", "n_gpus": world, "steps": reps, "warmup": max(3, args.warmup),
            "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{wl} {rows}x{cols} {kind}{' +imatrix' if weighted else ''}: {','.join(types)}",
                       "l2": f"{NSETS} rotating input/output buffer sets per kernel"},
            "clocks": clocks, "gpu_launches": int(launches), "per_qtype": table, "peak_source": peak_kind,
            **({"cpu_baseline": cpu} if cpu else {})}))


def run_dequant_all(args, torch, lib, ops, device, rank, world, hbm, peak_kind):
    """Decode throughput of every block type, 14336x4096 (or --rows) -> fp16, inputs resident in HBM."""
    import bench
    rows, cols = args.rows, 4096
    stream = torch.cuda.current_stream(device)
    g = torch.Generator(device=device)
    g.manual_seed(0)
    x = torch.randn((rows, cols), generator=g, device=device) * 0.02
    im = (torch.randn(cols, generator=g, device=device) ** 2 + 0.1).contiguous()
    table = {}
    reps = max(1, args.steps)
    launches0 = lib.libgguf_cuda_kernel_launch_count()
    for name in sorted(CODE, key=lambda n: CODE[n]):
        code, (bel, bby) = CODE[name], BLOCK[name]
        enc = [ops.quantize_weighted(x, code, im) if name.startswith("IQ") else ops.quantize(x, code)]
        enc += [enc[0].clone() for _ in range(NSETS - 1)]
        outs = [torch.empty((rows, cols), dtype=torch.float16, device=device) for _ in range(NSETS)]

        def dequant(k):
            st = lib.libgguf_cuda_dequantize_rows_on_stream(enc[k % NSETS].data_ptr(), code, rows, cols, 1,
                                                            outs[k % NSETS].data_ptr(), stream.cuda_stream)
            if st != 0:
                raise RuntimeError(lib.libgguf_cuda_thread_last_error().decode())

        for k in range(3):
            dequant(k)
        torch.cuda.synchronize()
        ms = _time_launches(torch, stream, dequant, reps)
        nbytes = enc[0].numel() + rows * cols * 2
        table[name] = {"ms": round(ms, 4), "GB/s": round(nbytes / ms / 1e6, 1), "hbm_frac": round(nbytes / ms / 1e6 / hbm, 4)}
        del enc, outs
    if rank == 0:
        print(json.dumps({"metric": "dequant GB/s per type", "value": statistics_mean([v["GB/s"] for v in table.values()]), "unit": "GB/s",
                          "n_gpus": world, "steps": reps, "warmup": 3, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": f"dequant_all {rows}x{cols} -> fp16, {NSETS} rotating buffer sets"},
                          "gpu_launches": int(lib.libgguf_cuda_kernel_launch_count() - launches0), "per_qtype": table, "peak_source": peak_kind}))


def statistics_mean(values):
    values = list(values)
    return sum(values) / len(values)


def run_convert_file(args, torch, lib, rank, world):
    """The converter as a user runs it: a Llama-shaped bf16 safetensors file (8 of the 32 layers by default, values
    synthetic) -> `libgguf_b200.quantize_gguf` with --gpus N -> GGUF file, both on a RAM-backed file system when
    there is one.  Reports fp32-equivalent GB/s of the whole command, file reads and writes included."""
    import shutil
    import struct
    import tempfile
    import numpy as np
    from libgguf_b200 import quantize_gguf as qg
    if rank != 0:
        return
    n_layers = int(os.environ.get("LIBGGUF_BENCH_LAYERS", "8"))
    base = "/dev/shm" if os.path.isdir("/dev/shm") else None
    tmp = tempfile.mkdtemp(prefix="libgguf_bench_", dir=base)
    try:
        shapes = [("model.embed_tokens.weight", (128256, 4096))]
        for i in range(n_layers):
            p = f"model.layers.{i}."
            shapes += [(p + "self_attn.q_proj.weight", (4096, 4096)), (p + "self_attn.k_proj.weight", (1024, 4096)),
                       (p + "self_attn.v_proj.weight", (1024, 4096)), (p + "self_attn.o_proj.weight", (4096, 4096)),
                       (p + "mlp.gate_proj.weight", (14336, 4096)), (p + "mlp.up_proj.weight", (14336, 4096)),
                       (p + "mlp.down_proj.weight", (4096, 14336)), (p + "input_layernorm.weight", (4096,))]
        shapes += [("model.norm.weight", (4096,)), ("lm_head.weight", (128256, 4096))]
        rng = np.random.default_rng(0)
        block = (rng.standard_normal(1 << 24, dtype=np.float32) * 0.02).view(np.uint32) >> 16
        block = block.astype(np.uint16)   # 16 Mi bf16 values, tiled over every tensor
        header, offset = {}, 0
        for name, shape in shapes:
            n = int(np.prod(shape)) * 2
            header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [offset, offset + n]}
            offset += n
        text = json.dumps(header, separators=(",", ":")).encode()
        text += b" " * (-len(text) % 8)
        src, dst = os.path.join(tmp, "model.safetensors"), os.path.join(tmp, "model.gguf")
        with open(src, "wb") as f:
            f.write(struct.pack("<Q", len(text)) + text)
            for name, shape in shapes:
                n = int(np.prod(shape))
                for start in range(0, n, block.size):
                    f.write(block[: min(block.size, n - start)].tobytes())
        elements = offset // 2
        ndev = min(args.gpus, torch.cuda.device_count())
        times = []
        for _ in range(1 + max(1, min(args.steps, 3))):
            t0 = time.perf_counter()
            qg.convert(qg.parse_args(["--src", src, "--dst", dst, "--qtype", "Q4_K_M", "--overwrite", "--gpus", str(ndev)]))
            times.append(time.perf_counter() - t0)
        best = min(times[1:])
        print(json.dumps({"metric": "conversion GB/s of fp32-equivalent source, file to file", "value": elements * 4 / best / 1e9, "unit": "GB/s",
                          "n_gpus": ndev, "steps": len(times) - 1, "warmup": 1, "ms_per_step": best * 1e3, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": f"convert_file: Llama-shaped bf16 safetensors, {n_layers} layers, Q4_K_M -> GGUF, through the command line front end",
                                     "elements": elements, "source_file_bytes": os.path.getsize(src), "output_file_bytes": os.path.getsize(dst),
                                     "directory": "RAM-backed" if base else "default temporary directory"},
                          "all_times_s": [round(t, 3) for t in times]}))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def bind_to_gpu_cpus(device_index):
    """One process per GPU: run on the CPUs NVML lists as local to the GPU, so that the pinned buffers this process
    allocates (first touch) sit on the memory node next to the GPU's PCIe root.  Returns the CPU list or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = [64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return allowed
    except Exception:
        return None
    return None


def as_numpy_source(torch, t):
    """Pinned torch tensor -> the numpy view the pipeline takes (bfloat16 as uint16 bit patterns)."""
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def widened(torch, a, src_dtype):
    t = torch.from_numpy(a)
    if src_dtype == "bf16":
        t = t.view(torch.bfloat16)
    return t.float()


def run_convert(args, torch, dist, lib, device, rank, world, hbm):
    """Whole-model conversion, pinned host fp32 in, pinned host blocks out.
    Plain `python bench.py --gpus N`: one process drives N GPUs through the in-process pool.
    Under torchrun (one process per GPU): every rank derives its share of the shards from the plan alone and
    streams it through its own GPU; no rank talks to another except for the barrier and the max-over-ranks time."""
    import numpy as np
    from libgguf_b200 import row_size
    from libgguf_b200.convert import ConversionPipeline, llama3_8b_plan, max_over_ranks, rank_batch
    per_process = world > 1
    affinity = None
    if per_process and os.environ.get("LIBGGUF_BENCH_CPU_AFFINITY", "1") != "0":
        affinity = bind_to_gpu_cpus(int(device.index or 0))
    ndev = world if per_process else min(args.gpus, torch.cuda.device_count())
    devices = [int(device.index or 0)] if per_process else list(range(ndev))
    plan = llama3_8b_plan()
    # one pinned source per distinct shape (layer tensors are re-used by all 32 layers), values N(0, 0.02) with
    # 0.1% of the columns scaled by 20; outputs are distinct pinned buffers per tensor
    g = torch.Generator(device=device)
    g.manual_seed(0)
    sources = {}
    for t in plan:
        key = (t.rows, t.cols)
        if key not in sources:
            x = torch.randn((t.rows, t.cols), generator=g, device=device) * 0.02
            cols = torch.randperm(t.cols, generator=g, device=device)[: max(1, t.cols // 1000)]
            x[:, cols] *= 20
            src_torch = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[args.src_dtype]
            host = torch.empty((t.rows, t.cols), dtype=src_torch).pin_memory()
            host.copy_(x.to(src_torch))
            sources[key] = host
            del x
    torch.cuda.synchronize()
    outs, batch = [], []
    for t in plan:
        o = torch.empty(t.rows * row_size(t.qtype, t.cols), dtype=torch.uint8).pin_memory()
        outs.append(o)
        batch.append((t.qtype, as_numpy_source(torch, sources[(t.rows, t.cols)]), None, o.numpy()))
    if per_process:
        batch = rank_batch(batch, world, rank)
    in_bytes = sum(t.rows * t.cols * 4 for t in plan)  # fp32-equivalent, whatever the source dtype
    link_bytes = in_bytes if args.src_dtype == "f32" else in_bytes // 2
    out_bytes = sum(o.numel() for o in outs)
    times = []
    with ConversionPipeline(devices, slots=3, chunk_bytes=128 << 20) as pipe:
        for it in range(1 + max(1, min(args.steps, 8))):
            if per_process:
                dist.barrier()
            t0 = time.perf_counter()
            pipe.quantize(batch)
            times.append(max_over_ranks(time.perf_counter() - t0, device))
        stats = pipe.stats()
    best = min(times[1:])
    # spot check against the single-GPU device path
    from libgguf_b200.libgguf_cuda import ops
    ok = True
    for q, s, _, d in batch[:: max(1, len(batch) // 4)]:
        rows = min(s.shape[0], 256)
        ref = ops.quantize(widened(torch, s[:rows], args.src_dtype).to(device), q).cpu().numpy().reshape(-1)
        ok = ok and bool(np.array_equal(ref, d[: ref.size]))
    if per_process:
        flag = torch.tensor([int(ok)], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
    if rank != 0:
        return
    print(json.dumps({
        "metric": "conversion GB/s of fp32 source", "value": in_bytes / best / 1e9, "unit": "GB/s", "n_gpus": ndev, "steps": len(times) - 1,
        "warmup": 1, "ms_per_step": best * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": "convert Llama-3-8B-shaped set, Q4_K_M mix, pinned host in/out", "tensors": len(plan),
                                       "launch": "one process per GPU, shards assigned from the plan" if per_process else "one process, in-process GPU pool",
                                       "source_dtype": args.src_dtype, "source_bytes_fp32_equivalent": in_bytes,
                                       "source_bytes_over_the_link": link_bytes, "output_bytes": out_bytes,
                                       "note": "layer sources shared by the 32 layers (one 0.87 GB layer + 2.1 GB embedding resident in pinned memory)"},
        "elements_per_s": in_bytes / 4 / best, "all_times_s": [round(x, 4) for x in times], "pipeline_rank0": stats, "spot_check_ok": ok,
        "cpu_affinity_rank0": (f"{affinity[0]}-{affinity[-1]} ({len(affinity)} cpus)" if affinity else None)}))
