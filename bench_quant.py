"""The quantizer and conversion workloads of bench.py.

As blocks of the default bench line (`quant_block`, `convert_block`) and alone (`--workload NAME`):

  q4k_roundtrip  Q4_K quantize + dequantize->fp32 of 4096x4096 N(0, 0.02)
  kquant         quantize 14336x4096 N(0, 0.02) to Q8_0, Q6_K, Q5_K, Q4_K, Q3_K, Q2_K
  legacy         quantize the same matrix to Q4_0, Q4_1, Q5_0, Q5_1, Q1_0, TQ1_0, TQ2_0, IQ4_NL, IQ4_XS
  iq             the lattice types IQ2_XXS, IQ2_S, IQ3_XXS, IQ1_S (+ IQ2_XS, IQ3_S, IQ1_M) on 4096x11008
                 Student-t(5)*0.02 with a chi-square(4)/4 importance matrix
  fp4            MXFP4 / NVFP4 quantize and dequantize->bf16 of 8192x8192 bf16-origin Laplace(0, 0.01) with 1% outlier blocks
  dequant_all    decode of every block type, 14336x4096 -> fp16
  convert        synthetic Llama-3-8B-shaped weight set (N(0, 0.02) with 0.1% outlier columns) through the multi-GPU
                 streaming pipeline (pinned host memory in and out), Q4_K_M-style mix
  convert_file   the same through the command-line front end, file to file

Metric Melem/s (GB/s of fp32 source for `convert`), per-type table with the fraction of the bound that applies: HBM
bytes for the cheap encoders; for the search-heavy ones the share of the SMs' warp-instruction issue slots, from the
warp instructions per element that profiles/quantizer_instruction_counts.json records (an ncu count on a small case)
and the SM clock sampled during the run.  Inputs are the seeded NumPy generators of tests/inputs.py, resident in HBM
when a timed region starts; every timed launch uses one of NSETS distinct input/output buffer sets; a slice of what
the timed launches wrote is compared with the CPU checker afterwards."""
from __future__ import annotations

import json
import os
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
NSETS = 3
SMS, SCHEDULERS_PER_SM = 148, 4

BLOCK = {"Q4_0": (32, 18), "Q4_1": (32, 20), "Q5_0": (32, 22), "Q5_1": (32, 24), "Q8_0": (32, 34), "Q1_0": (128, 18),
         "MXFP4": (32, 17), "NVFP4": (64, 36), "Q2_K": (256, 84), "Q3_K": (256, 110), "Q4_K": (256, 144),
         "Q5_K": (256, 176), "Q6_K": (256, 210), "TQ1_0": (256, 54), "TQ2_0": (256, 66), "IQ2_XXS": (256, 66),
         "IQ2_XS": (256, 74), "IQ2_S": (256, 82), "IQ3_XXS": (256, 98), "IQ3_S": (256, 110), "IQ1_S": (256, 50),
         "IQ1_M": (256, 56), "IQ4_NL": (32, 18), "IQ4_XS": (256, 136)}
CODE = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14,
        "IQ2_XXS": 16, "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19, "IQ4_NL": 20, "IQ3_S": 21, "IQ2_S": 22, "IQ4_XS": 23,
        "IQ1_M": 29, "TQ1_0": 34, "TQ2_0": 35, "MXFP4": 39, "NVFP4": 40, "Q1_0": 41}
# encoders whose time is set by HBM traffic (4 B/element in, the encoded bytes out); the others are bound by issue
HBM_BOUND = {"Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q1_0", "TQ1_0", "TQ2_0", "MXFP4", "NVFP4"}
LATTICE = ("IQ1", "IQ2", "IQ3")


def _inputs():
    import inputs  # tests/inputs.py (bench.py puts tests/ on the path)
    return inputs


_sweep_matrix_cache: dict = {}


def sweep_matrix(rows: int, cols: int):
    """inputs.decode_sweep_matrix, drawn once per process (bench.py's sweep and the K-quant workloads share it; the
    generator is a single sequential stream of 59 M normals)."""
    key = (rows, cols)
    if key not in _sweep_matrix_cache:
        _sweep_matrix_cache.clear()
        _sweep_matrix_cache[key] = _inputs().decode_sweep_matrix(rows, cols)
    return _sweep_matrix_cache[key]


def workload_spec(name: str) -> dict:
    """rows, cols, generator -> (matrix, imatrix or None), types, output dtype of the decode leg (or None)."""
    inp = _inputs()
    return {
        "q4k_roundtrip": dict(rows=4096, cols=4096, gen=lambda r, c: (inp.q4k_matrix(r, c), None), types=["Q4_K"], decode="fp32",
                              data="N(0, 0.02) seed 0"),
        "kquant": dict(rows=14336, cols=4096, gen=lambda r, c: (sweep_matrix(r, c), None),
                       types=["Q8_0", "Q6_K", "Q5_K", "Q4_K", "Q3_K", "Q2_K"], decode=None, data="N(0, 0.02) seed 0"),
        "legacy": dict(rows=14336, cols=4096, gen=lambda r, c: (sweep_matrix(r, c), None),
                       types=["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q1_0", "TQ1_0", "TQ2_0", "IQ4_NL", "IQ4_XS"], decode=None,
                       data="N(0, 0.02) seed 0"),
        "iq": dict(rows=4096, cols=11008, gen=lambda r, c: inp.lattice_matrix(r, c),
                   types=["IQ2_XXS", "IQ2_S", "IQ3_XXS", "IQ1_S", "IQ2_XS", "IQ3_S", "IQ1_M"], decode=None,
                   data="Student-t(5) * 0.02 seed 0, importance weights chi-square(4)/4 seed 1"),
        "fp4": dict(rows=8192, cols=8192, gen=lambda r, c: (inp.microscaling_matrix(r, c), None), types=["MXFP4", "NVFP4"],
                    decode="bf16", data="Laplace(0, 0.01) rounded to bf16, 1% of 32-blocks with a +-50 sigma element, seed 0"),
    }[name]


def _time_launches(torch, stream, fn, reps):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for k in range(reps):
        fn(k)
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _max_over_ranks(torch, dist, device, v):
    if dist is None:
        return float(v)
    t = torch.tensor([v], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _checker():
    from oracle import reference
    return reference.load("ref" if reference.available("ref") else "port")


def time_types(torch, dist, lib, device, world, hbm, x_host, im_host, types, decode, reps, warm, check):
    """Times lib.libgguf_cuda_quantize_f32_rows_on_stream (and the decode leg) per type on the matrix `x_host`;
    returns {type: row}.  `check`: compare the first rows of what the timed launches wrote with the CPU checker."""
    stream = torch.cuda.current_stream(device)
    rows, cols = x_host.shape
    n = rows * cols
    x0 = torch.from_numpy(x_host).to(device)
    xs = [x0] + [x0.clone() for _ in range(NSETS - 1)]
    im = torch.from_numpy(im_host).to(device) if im_host is not None else None
    table = {}
    chk = _checker() if check else None
    for name in types:
        code, (bel, bby) = CODE[name], BLOCK[name]
        enc_bytes = n // bel * bby
        outs = [torch.empty((rows, cols // bel * bby), dtype=torch.uint8, device=device) for _ in range(NSETS)]

        def quant(k):
            st = lib.libgguf_cuda_quantize_f32_rows_on_stream(xs[k % NSETS].data_ptr(), im.data_ptr() if im is not None else None,
                                                              outs[k % NSETS].data_ptr(), code, rows, cols, stream.cuda_stream)
            if st != 0:
                raise RuntimeError(lib.libgguf_cuda_thread_last_error().decode())

        for k in range(max(warm, NSETS)):   # at least once per buffer set: the check below reads all of them
            quant(k)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        ms = _max_over_ranks(torch, dist, device, _time_launches(torch, stream, quant, reps))
        gbs = (4 * n + enc_bytes) / ms / 1e6
        row = {"quant_ms": round(ms, 4), "quant_Melem/s": round(world * n / ms / 1e3, 1), "elements": n,
               "bound": "hbm" if name in HBM_BOUND else "issue"}
        if name in HBM_BOUND:
            row.update({"quant_GB/s": round(gbs, 1), "hbm_frac": round(gbs / hbm, 4)})
        if decode is not None:
            dt = torch.float32 if decode == "fp32" else torch.bfloat16
            code_dt = 0 if decode == "fp32" else 2
            dec = [torch.empty((rows, cols), dtype=dt, device=device) for _ in range(NSETS)]

            def dequant(k):
                st = lib.libgguf_cuda_dequantize_rows_on_stream(outs[k % NSETS].data_ptr(), code, rows, cols, code_dt,
                                                                dec[k % NSETS].data_ptr(), stream.cuda_stream)
                if st != 0:
                    raise RuntimeError(lib.libgguf_cuda_thread_last_error().decode())

            for k in range(3):
                dequant(k)
            torch.cuda.synchronize()
            dms = _max_over_ranks(torch, dist, device, _time_launches(torch, stream, dequant, reps))
            db = enc_bytes + n * dec[0].element_size()
            row.update({"dequant_ms": round(dms, 4), "dequant_GB/s": round(db / dms / 1e6, 1),
                        "dequant_hbm_frac": round(db / dms / 1e6 / hbm, 4), "dequant_to": decode})
        if chk is not None:
            nchk = min(rows, 16 if name.startswith(LATTICE) else 128)
            want = chk.quantize_rows(x_host[:nchk], code, im_host)
            ok = all(bool(np.array_equal(o[:nchk].cpu().numpy(), want)) for o in outs)
            if decode is not None:
                ref32 = torch.from_numpy(chk.dequantize_rows(want, code, cols))
                view = torch.int32 if decode == "fp32" else torch.int16
                ok = ok and all(bool(torch.equal(d[:nchk].cpu().view(view), ref32.to(dec[0].dtype).view(view))) for d in dec)
            row["verified"] = ok
        if decode is not None:
            del dec
        table[name] = row
        del outs
    del xs, x0
    torch.cuda.empty_cache()
    return table


def instruction_counts() -> dict:
    p = ROOT / "profiles" / "quantizer_instruction_counts.json"
    return json.loads(p.read_text()).get("types", {}) if p.exists() else {}


def add_issue_fractions(block: dict, sm_mhz: float) -> None:
    """issue_frac = warp instructions (ncu count per element x elements) / (time x 148 SMs x 4 schedulers x the SM clock
    sampled during this run): the share of the GPU's issue slots the kernel filled."""
    counts = instruction_counts()
    for group in block.get("workloads", {}).values():
        for name, row in group.get("per_qtype", {}).items():
            c = counts.get(name)
            if row.get("bound") != "issue" or not c:
                continue
            slots = row["quant_ms"] * 1e-3 * SMS * SCHEDULERS_PER_SM * sm_mhz * 1e6
            row["issue_frac"] = round(c["warp_inst_per_elem"] * row["elements"] / slots, 4)
            row["warp_inst_per_elem"] = c["warp_inst_per_elem"]
    block["issue_frac_clock_mhz"] = sm_mhz


def cpu_quantize_baseline(x_host, im_host, types, seconds_per_type=1.5):
    """Upstream's CPU quantizers (REF build, and the AVX2 build when present) on the first rows of the same input,
    all host threads: rows are grown until a call lasts about a quarter of `seconds_per_type`.  Melem/s per type."""
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


def quant_block(torch, dist, lib, device, rank, world, hbm, check=True, cpu=False) -> dict:
    """The quantize half of the metric inside the default bench line: every workload's matrix at full size, each type
    timed over a few launches (own CUDA events, max over ranks).  Every rank quantizes its own copy of the matrices:
    rows shard with no exchange, so N GPUs do N times the work in the same time (weak scaling)."""
    plan = [("q4k_roundtrip", None, 10), ("kquant", None, 10), ("fp4", None, 10),
            ("iq", ["IQ2_XXS", "IQ2_S", "IQ3_XXS", "IQ1_S"], 3)]
    out = {"unit": "Melem/s (all ranks)", "n_gpus": world, "workloads": {}}
    launches0 = lib.libgguf_cuda_kernel_launch_count()
    all_ok = True
    for wl, subset, reps in plan:
        spec = workload_spec(wl)
        types = subset or spec["types"]
        x_host, im_host = spec["gen"](spec["rows"], spec["cols"])
        table = time_types(torch, dist, lib, device, world, hbm, x_host, im_host, types, spec["decode"], reps, 3, check)
        entry = {"shape": f"{spec['rows']}x{spec['cols']}", "data": spec["data"], "launches_timed_per_type": reps, "per_qtype": table}
        if cpu:
            base, cpu_rows = cpu_quantize_baseline(x_host, im_host, types, seconds_per_type=0.6)
            for name, extra in cpu_rows.items():
                table[name].update(extra)
            entry["cpu_baseline"] = base
        if check:
            all_ok = all_ok and all(r.get("verified", False) for r in table.values())
        out["workloads"][wl] = entry
        del x_host
    out["gpu_launches"] = int(lib.libgguf_cuda_kernel_launch_count() - launches0)
    if check:
        out["verified"] = all_ok
    return out


# ------------------------------------------------------------------------------------------------
def run(args, torch, dist, lib, ops, device, rank, world):
    import bench
    hbm, peak_kind = bench.peaks()
    wl = args.workload
    if wl == "convert":
        sampler = bench.ClockSampler(int(device.index or 0))
        sampler.start()
        block = convert_block(torch, dist if world > 1 else None, lib, device, rank, world, link=None, gpus=args.gpus,
                              src_dtype=args.src_dtype, iterations=max(2, min(args.steps, 8)))
        clocks = sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": "conversion GB/s of fp32 source", "value": block["GB/s"], "unit": "GB/s", "n_gpus": block["n_gpus"],
                              "steps": block["passes_timed"], "warmup": 1, "ms_per_step": block["seconds"] * 1e3, "higher_is_better": True,
                              "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "clocks": clocks,
                              "config": {"workload": "convert Llama-3-8B-shaped set, Q4_K_M mix, pinned host in/out"}, "convert": block}))
        return
    if wl == "convert_file":
        return run_convert_file(args, torch, lib, rank, world)
    if wl == "dequant_all":
        return run_dequant_all(args, torch, lib, ops, device, rank, world, hbm, peak_kind)
    spec = workload_spec(wl)
    rows = spec["rows"] if args.rows == bench.ROWS else args.rows
    types = [t for t in spec["types"] if not args.types or t in args.types.split(",")]
    x_host, im_host = spec["gen"](rows, spec["cols"])
    sampler = bench.ClockSampler(int(device.index or 0))
    launches0 = lib.libgguf_cuda_kernel_launch_count()
    reps = max(1, args.steps)
    sampler.start()
    with sampler.window():
        table = time_types(torch, dist if world > 1 else None, lib, device, world, hbm, x_host, im_host, types, spec["decode"], reps,
                           max(1, args.warmup), check=(rank == 0))
    clocks = sampler.stop()
    launches = lib.libgguf_cuda_kernel_launch_count() - launches0
    block = {"workloads": {wl: {"per_qtype": table}}}
    if clocks.get("sm_mhz"):
        add_issue_fractions(block, clocks["sm_mhz"])
    total_ms = sum(r["quant_ms"] + r.get("dequant_ms", 0.0) for r in table.values())
    n = rows * spec["cols"]
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, cpu_rows = cpu_quantize_baseline(x_host, im_host, types)
        for name, extra in cpu_rows.items():
            table[name].update(extra)
    if rank == 0:
        print(json.dumps({
            "metric": "quant Melem/s", "value": world * len(types) * n / total_ms / 1e3, "unit": "Melem/s", "n_gpus": world, "steps": reps,
            "warmup": max(1, args.warmup), "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{wl} {rows}x{spec['cols']} {spec['data']}: {','.join(types)}",
                       "l2": f"{NSETS} rotating input/output buffer sets per kernel"},
            "clocks": clocks, "gpu_launches": int(launches), "per_qtype": table, "peak_source": peak_kind,
            "verified": all(r.get("verified", False) for r in table.values()),
            **({"cpu_baseline": cpu} if cpu else {})}))


def run_dequant_all(args, torch, lib, ops, device, rank, world, hbm, peak_kind):
    """Decode throughput of every block type, 14336x4096 (or --rows) -> fp16, inputs resident in HBM."""
    inp = _inputs()
    rows, cols = args.rows, 4096
    stream = torch.cuda.current_stream(device)
    x = torch.from_numpy(sweep_matrix(rows, cols)).to(device)
    im = torch.from_numpy(inp.imatrix_for(cols, 3)).to(device)
    only = set(args.types.split(",")) if args.types else None
    table = {}
    reps = max(1, args.steps)
    launches0 = lib.libgguf_cuda_kernel_launch_count()
    for name in sorted(CODE, key=lambda n: CODE[n]):
        if only and name not in only:
            continue
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
        values = [v["GB/s"] for v in table.values()]
        print(json.dumps({"metric": "dequant GB/s per type", "value": sum(values) / len(values), "unit": "GB/s",
                          "n_gpus": world, "steps": reps, "warmup": 3, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": f"dequant_all {rows}x{cols} -> fp16, {NSETS} rotating buffer sets"},
                          "gpu_launches": int(lib.libgguf_cuda_kernel_launch_count() - launches0), "per_qtype": table, "peak_source": peak_kind}))


def run_convert_file(args, torch, lib, rank, world):
    """The converter as a user runs it: a Llama-shaped bf16 safetensors file (8 of the 32 layers by default, values
    synthetic) -> `libgguf_b200.quantize_gguf` with --gpus N -> GGUF file, both on a RAM-backed file system when
    there is one.  Reports fp32-equivalent GB/s of the whole command, file reads and writes included."""
    import shutil
    import struct
    import tempfile
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
        times, stages = [], []
        for _ in range(1 + max(1, min(args.steps, 3))):
            t0 = time.perf_counter()
            result = qg.convert(qg.parse_args(["--src", src, "--dst", dst, "--qtype", "Q4_K_M", "--overwrite", "--gpus", str(ndev)]))
            times.append(time.perf_counter() - t0)
            stages.append({k: round(v, 3) for k, v in result["timings"].items() if isinstance(v, float)})
        best = min(times[1:])
        print(json.dumps({"metric": "conversion GB/s of fp32-equivalent source, file to file", "value": elements * 4 / best / 1e9, "unit": "GB/s",
                          "n_gpus": ndev, "steps": len(times) - 1, "warmup": 1, "ms_per_step": best * 1e3, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": f"convert_file: Llama-shaped bf16 safetensors, {n_layers} layers, Q4_K_M -> GGUF, through the command line front end",
                                     "elements": elements, "source_file_bytes": os.path.getsize(src), "output_file_bytes": os.path.getsize(dst),
                                     "directory": "RAM-backed" if base else "default temporary directory"},
                          "all_times_s": [round(t, 3) for t in times],
                          "stages_of_the_best_run_s": stages[times.index(best)]}))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def convert_block(torch, dist, lib, device, rank, world, link=None, gpus=1, src_dtype="f32", iterations=2, reuse=None,
                  keep_sources=False) -> dict:
    """Whole-model conversion, pinned host source in, pinned host blocks out: the Llama-3-8B-shaped tensor set
    (226 tensors, 8.03 G elements, Q4_K_M mix).  One process: the in-process pool over `gpus` GPUs.  Under torchrun
    (one process per GPU): every rank derives its share of the shards from the plan alone and streams it through its
    own GPU; no rank talks to another except for the barrier and the max-over-ranks time (strong scaling).
    The values of one tensor per distinct shape are generated (tests/inputs.conversion_tensor) and shared by the
    tensors of that shape; afterwards row ranges of the encoded output are compared with the CPU checker.
    `reuse`: the pinned fp32 sources of an earlier call (`keep_sources=True` returns them under "_sources"), from which a
    16-bit run derives its sources instead of drawing the values again."""
    from libgguf_b200 import row_size
    from libgguf_b200.convert import SOURCE_DTYPES, ConversionPipeline, assign_shards, llama3_8b_plan, plan_shards
    inp = _inputs()
    per_process = dist is not None
    ndev = world if per_process else max(1, min(gpus, torch.cuda.device_count()))
    devices = [int(device.index or 0)] if per_process else list(range(ndev))
    plan = llama3_8b_plan()
    src_torch = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[src_dtype]
    names = {(rows, cols): name for name, rows, cols in inp.CONVERSION_SHAPES}
    sources, pinned = {}, {}
    for key in names:
        if reuse is not None and src_dtype == "f32":
            pinned[key] = reuse[key]
            continue
        pinned[key] = torch.empty(key, dtype=src_torch).pin_memory()
        if src_dtype == "f32":   # drawn straight into the pinned buffer, blocks of rows on several threads
            inp.conversion_tensor(names[key], key[0], key[1], out=pinned[key].numpy())
        elif reuse is not None:
            pinned[key].copy_(reuse[key])
        else:
            pinned[key].copy_(torch.from_numpy(inp.conversion_tensor(names[key], key[0], key[1])).to(src_torch))
    for key, t in pinned.items():
        sources[key] = t.view(torch.uint16).numpy() if src_dtype == "bf16" else t.numpy()
    chunk = 128 << 20
    tensors = [(t.qtype, t.rows, t.cols) for t in plan]
    code = SOURCE_DTYPES[np.dtype(np.uint16 if src_dtype == "bf16" else (np.float16 if src_dtype == "f16" else np.float32))]
    rates = None
    if per_process:
        # Start-up probe of every rank's own host link (all ranks copying at once, the way the conversion runs), exchanged
        # once: the static shares follow the measured rates, like the in-process pool's pull queue finds by itself.  This
        # is planning input; no tensor data crosses between ranks.
        probe_src = pinned[(14336, 4096)].view(torch.uint8).reshape(-1)[: 128 << 20]
        probe_dst = torch.empty(probe_src.numel(), dtype=torch.uint8, device=device)
        probe_dst.copy_(probe_src, non_blocking=True)
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(4):
            probe_dst.copy_(probe_src, non_blocking=True)
        b.record()
        torch.cuda.synchronize()
        mine = torch.tensor([4 * probe_src.numel() / (a.elapsed_time(b) * 1e-3) / 1e9], device=device, dtype=torch.float64)
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        rates = [round(float(g.item()), 1) for g in gathered]
        del probe_dst
        shards = assign_shards(plan_shards(tensors, chunk, [code] * len(plan)), [t.cols for t in plan], world, rates)[rank]
    else:
        shards = [(i, 0, t.rows) for i, t in enumerate(plan)]
    pool_bytes = sum(rows * row_size(plan[i].qtype, plan[i].cols) for i, _, rows in shards)
    out_pool_t = torch.empty(max(pool_bytes, 1), dtype=torch.uint8).pin_memory()
    out_pool = out_pool_t.numpy()
    batch, at = [], 0
    for i, row0, rows in shards:
        t = plan[i]
        nbytes = rows * row_size(t.qtype, t.cols)
        batch.append((t.qtype, sources[(t.rows, t.cols)][row0:row0 + rows], None, out_pool[at:at + nbytes]))
        at += nbytes
    in_bytes = sum(t.rows * t.cols * 4 for t in plan)  # fp32-equivalent, whatever the source dtype
    link_bytes = in_bytes if src_dtype == "f32" else in_bytes // 2
    out_bytes = sum(t.rows * row_size(t.qtype, t.cols) for t in plan)
    times = []
    with ConversionPipeline(devices, slots=3, chunk_bytes=chunk) as pipe:
        for _ in range(1 + iterations):
            if per_process:
                dist.barrier()
            t0 = time.perf_counter()
            pipe.quantize(batch)
            times.append(_max_over_ranks(torch, dist, device, time.perf_counter() - t0))
        stats = pipe.stats()
    best = min(times[1:])

    def copies_only() -> float:
        """The same shards as plain copies, no kernels: every source row range uploaded from its pinned buffer in pieces
        of `chunk` bytes on one stream, the encoded bytes downloaded into the pinned output on another, both in flight
        together, every rank at once; seconds of the slowest rank, best of two."""
        up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
        d_in = torch.empty(chunk, dtype=torch.uint8, device=device)
        d_out = torch.empty(chunk, dtype=torch.uint8, device=device)
        pieces_in = []
        for i, row0, rows in shards:
            flat = pinned[(plan[i].rows, plan[i].cols)][row0:row0 + rows].view(torch.uint8).reshape(-1)
            pieces_in += [flat[a:a + chunk] for a in range(0, flat.numel(), chunk)]
        result = []
        for _ in range(3):
            torch.cuda.synchronize(device)
            if per_process:
                dist.barrier()
            t0 = time.perf_counter()
            with torch.cuda.stream(up):
                for piece in pieces_in:
                    d_in[:piece.numel()].copy_(piece, non_blocking=True)
            with torch.cuda.stream(down):
                for a in range(0, pool_bytes, chunk):
                    n = min(chunk, pool_bytes - a)
                    out_pool_t[a:a + n].copy_(d_out[:n], non_blocking=True)
            up.synchronize()
            down.synchronize()
            result.append(_max_over_ranks(torch, dist, device, time.perf_counter() - t0))
        return min(result[1:])
    # row ranges of what the pipeline wrote, against the CPU checker (rank 0; outside the timed passes)
    ok = None
    if rank == 0:
        chk = _checker()
        ok, seen = True, set()
        for (qtype, src, _, dst) in batch:
            key = (qtype, src.shape[1], src.shape[0] > 2048)
            if key in seen:
                continue
            seen.add(key)
            n = min(src.shape[0], 64)
            rows32 = src[:n]
            if src_dtype == "bf16":
                rows32 = (rows32.astype(np.uint32) << np.uint32(16)).view(np.float32)
            elif src_dtype == "f16":
                rows32 = rows32.astype(np.float32)
            want = chk.quantize_rows(np.ascontiguousarray(rows32), qtype)
            ok = ok and bool(np.array_equal(dst[:want.size], want.reshape(-1)))
    out = {"GB/s": in_bytes / best / 1e9, "unit": "GB/s of fp32-equivalent source", "seconds": best, "n_gpus": ndev, "scaling": "strong",
           "launch": "one process per GPU, shards assigned from the plan" if per_process else "one process, in-process GPU pool",
           "tensors": len(plan), "source_dtype": src_dtype, "source_bytes_fp32_equivalent": in_bytes,
           "source_bytes_over_the_link": link_bytes, "output_bytes": out_bytes, "passes_timed": iterations,
           "all_times_s": [round(x, 4) for x in times], "pipeline_rank0": stats, "verified": ok,
           "link_rates_GBps_per_rank": rates,
           "note": "one generated tensor per distinct shape, shared by the tensors of that shape (3.3 GB of pinned source)"}
    if keep_sources and src_dtype == "f32":
        out["_sources"] = pinned
    if link is not None:
        # what plain copies of the same bytes take on this host link at this N: the conversion's own uploads and
        # downloads together (measured here, after the timed passes and the check of their output),
        # and, for orientation, each direction alone at the rates of the e2e leg's probe
        t_alone = max(link_bytes / (link["h2d_alone_GBps"] * 1e9), out_bytes / (link["d2h_alone_GBps"] * 1e9))
        # (one process driving several GPUs: the probe's rates only)
        t_mix = copies_only() if (per_process or ndev == 1) else t_alone
        out["roofline"] = {"bound": "host_link", "ceiling": in_bytes / t_mix / 1e9, "achieved": out["GB/s"], "unit": out["unit"],
                           "frac": out["GB/s"] / (in_bytes / t_mix / 1e9), "seconds_copies_only": t_mix,
                           "ceiling_directions_alone": in_bytes / t_alone / 1e9,
                           "how": "the same shards as plain pinned copies without kernels, uploads and downloads on two streams, "
                                  "all ranks at once, slowest rank's time; `ceiling_directions_alone` = the slower of uploads "
                                  "alone and downloads alone at the rates the e2e leg's probe measured at the same N"}
    return out
