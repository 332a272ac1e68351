"""Benchmark of the packed INT4-g128 matvec path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One process per GPU (for N > 1 launch under ``python -m torch.distributed.run``).  Rank 0 prints one
JSON line.

N = 1: the workload is the seven block linears of a Llama-3-8B-shaped decoder block (q, k, v, o,
gate, up, down; INT4, group 128, fp16 scales; weights N(0, 0.02) from a seed, RTN-quantised on the
device by this package's own ``mk.int(4, group=128)``), with 1, 2, 4 and 8 activation rows.  A step is
one pass of the packed matvec over ``BLOCKS`` distinct blocks x 7 linears x 4 row counts.  The blocks
together hold ~0.9 GB of packed weights, so no weight is served from L2 twice in a row.

N > 1: the 70B-shaped tensor-parallel decode step of ``mlkit_b200.tp`` (see ``decode_workload``).

``value`` is algorithmic GB/s with every input resident in HBM; ``e2e`` is the same pass through the
public module call (``PackedLinear.forward``) with activations coming from pinned host memory and
results returned to it inside the timed region.  ``--impl reference`` times the reference's CPU route
(unpack, reconstruct, ``F.linear``) through ``oracle/cpu_path.py`` on the host cores.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA8B = {"q": (4096, 4096), "k": (1024, 4096), "v": (1024, 4096), "o": (4096, 4096),
           "gate": (14336, 4096), "up": (14336, 4096), "down": (4096, 14336)}
ROW_COUNTS = (1, 2, 4, 8)
BLOCKS = 8
BITS, GROUP = 4, 128
METRIC = "packed_int4_g128_gemv_hbm_gbps"
# dram__bytes_read.sum + dram__bytes_write.sum of one gate-shape launch (4096 -> 14336) from the profiler
# captures summarised in profiles/gemv_tiled_gate_4096x14336_M1.md and gemv_bulk_gate_4096x14336_M8.md;
# refreshed when a kernel changes
TILED_GATE_M1_DRAM_BYTES = 30.3293e6
BULK_GATE_M8_DRAM_BYTES = 30.3890e6


def gemv_bytes(out_rows: int, width: int, rows_in: int) -> int:
    """Algorithmic bytes of one INT4-g128 matvec: codes + fp16 scales + activations + outputs + table."""
    return out_rows * width * BITS // 8 + out_rows * (width // GROUP) * 2 + rows_in * width * 2 + rows_in * out_rows * 2 + 64


def pass_bytes(blocks: int) -> int:
    return blocks * sum(gemv_bytes(n, k, m) for (n, k) in LLAMA8B.values() for m in ROW_COUNTS)


def peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.process = None

    def __enter__(self) -> "ClockSampler":
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc) -> None:
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.process is None:
            return
        time.sleep(0.25)
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        clocks, reasons, maximum = [], set(), None
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 9:
                continue
            try:
                clocks.append(float(fields[1]))
                maximum = float(fields[2])
            except ValueError:
                continue
            for name, field in zip(names, fields[5:9]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.summary = {"sm_mhz": statistics.median(clocks), "sm_max_mhz": maximum, "reasons": sorted(reasons),
                            "samples": len(clocks)}


def build_blocks(device: torch.device, blocks: int):
    """``blocks`` decoder blocks of seven ``PackedLinear`` layers, RTN-quantised on the device."""
    import mlkit_b200 as mk
    from torch import nn

    generator = torch.Generator(device=device).manual_seed(1234)
    fmt = mk.int(BITS, group=GROUP)
    result = []
    for _ in range(blocks):
        layers = {}
        for name, (out_rows, width) in LLAMA8B.items():
            weight = (torch.randn(out_rows, width, generator=generator, device=device) * 0.02).half()
            linear = nn.Linear(width, out_rows, bias=False, device=device, dtype=torch.float16)
            with torch.no_grad():
                linear.weight.copy_(weight)
            q = fmt(weight.float(), mk.Ctx(name, device=device))
            layers[name] = mk.PackedLinear(linear, q)
            del linear, weight, q
        result.append(layers)
    torch.cuda.empty_cache()
    return result


def run_pass_resident(blocks, inputs, outputs) -> int:
    """One step with everything in HBM: bound launches on preallocated outputs.  Returns launches."""
    launches = 0
    for rows in ROW_COUNTS:
        for layers in blocks:
            for name, layer in layers.items():
                layer._plan(torch.float16)(inputs[rows][layer.in_features], outputs[rows][layer.out_features])
                launches += 1
    return launches


def capture_pass(blocks, inputs, outputs) -> tuple[torch.cuda.CUDAGraph, int]:
    """The resident step as one CUDA graph (decode loops are launch-bound; the reference itself relies
    on graph capture through ``torch.compile(mode="reduce-overhead")`` for generation)."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run_pass_resident(blocks, inputs, outputs)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            launches = run_pass_resident(blocks, inputs, outputs)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return graph, launches


def run_pass_e2e(blocks, host_inputs, host_outputs, device) -> tuple[int, int]:
    """One step through ``PackedLinear.forward`` with host-resident activations and results."""
    h2d = d2h = 0
    for rows in ROW_COUNTS:
        for layers in blocks:
            for name, layer in layers.items():
                x_host = host_inputs[rows][layer.in_features]
                x = x_host.to(device, non_blocking=True)
                y = layer(x)
                host_outputs[rows][layer.out_features].copy_(y, non_blocking=True)
                h2d += x_host.numel() * 2
                d2h += y.numel() * 2
    return h2d, d2h


def per_layer_table(blocks, inputs, outputs, peak: float) -> dict:
    """Average launch duration per layer shape and row count (CUDA events around the launches of all
    blocks, which keeps every weight cold in L2), as algorithmic GB/s and roofline fraction."""
    table = {}
    for name, (out_rows, width) in LLAMA8B.items():
        if name in ("v", "up"):
            continue
        for rows in ROW_COUNTS:
            def launch_all():
                for layers in blocks:
                    layers[name]._plan(torch.float16)(inputs[rows][width], outputs[rows][out_rows])
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                launch_all()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    launch_all()
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            best = None
            for _ in range(5):
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                graph.replay()
                stop.record()
                torch.cuda.synchronize()
                elapsed = start.elapsed_time(stop) / len(blocks)
                best = elapsed if best is None else min(best, elapsed)
            gbps = gemv_bytes(out_rows, width, rows) / best / 1e6
            table[f"{name}_{width}x{out_rows}_M{rows}"] = {"us": round(best * 1e3, 3), "gbps": round(gbps, 1),
                                                           "frac": round(gbps / peak, 4)}
    return table


def cpu_reference_layers(blocks: int = 1):
    """Host copies of the block linears for the CPU route (random codes: arithmetic cost is value-blind)."""
    generator = torch.Generator().manual_seed(99)
    layers = []
    for _ in range(blocks):
        for name, (out_rows, width) in LLAMA8B.items():
            layers.append({
                "packed": torch.randint(0, 256, (out_rows * width * BITS // 8,), dtype=torch.uint8, generator=generator),
                "scales": (torch.rand(out_rows, width // GROUP, generator=generator) * 0.01 + 0.001).half(),
                "values": torch.arange(-8, 8, dtype=torch.float32), "group": GROUP, "bits": BITS,
                "shape": (out_rows, width),
            })
    return layers


def time_cpu_route(repetitions: int, warmup: int):
    """Seconds per pass of unpack + reconstruct + F.linear over one block's seven linears, M = 1."""
    from oracle import cpu_path

    layers = cpu_reference_layers(1)
    seconds, threads = cpu_path.time_reconstruct_plus_matmul(layers, rows_in=1, repetitions=repetitions, warmup=warmup)
    bytes_per_pass = sum(gemv_bytes(n, k, 1) for (n, k) in LLAMA8B.values())
    return seconds, threads, bytes_per_pass


def time_transform(device: torch.device, rows: int, width: int, copies: int, repetitions: int = 5) -> float:
    """Microseconds per launch of the randomised Hadamard transform (signs, FWHT, Paley factor for
    14336 = 28 x 512) on fp16 ``[rows, width]``, over ``copies`` distinct inputs replayed as one CUDA graph."""
    import mlkit_b200 as mk

    generator = torch.Generator(device=device).manual_seed(11)
    inputs = [torch.randn(rows, width, device=device, generator=generator).half() for _ in range(copies)]
    signs = (torch.randint(0, 2, (width,), device=device, generator=generator) * 2 - 1).to(torch.int8)

    def launch_all():
        for x in inputs:
            mk.rht(x, signs=signs)
    launch_all()
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch_all()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            launch_all()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(repetitions):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        elapsed = start.elapsed_time(stop) * 1e3 / copies
        best = elapsed if best is None else min(best, elapsed)
    return best


def transform_table(device: torch.device, peak: float) -> dict:
    """The activation transform at decode sizes (latency-bound) and on a large batch (its bandwidth ceiling)."""
    table = {}
    for rows, width, copies in ((1, 4096, 16), (8, 4096, 16), (8, 14336, 16), (16384, 4096, 4), (8192, 14336, 4)):
        us = time_transform(device, rows, width, copies)
        moved = 2 * rows * width * 2 + width
        table[f"rht_{rows}x{width}"] = {"us": round(us, 2), "gbps": round(moved / us / 1e3, 1),
                                        "frac": round(moved / us / 1e3 / peak, 4)}
    return table


def run_case(spec: str, device: torch.device, launches: int) -> None:
    """One layer shape, ``launches`` launches over distinct weight copies (each cold in L2), nothing
    else on the device: the small case a profiler captures.  Prints the mean launch time.
    ``rht:ROWS:WIDTH`` runs the activation transform instead."""
    from mlkit_b200 import kernels

    fields = spec.split(":")
    if fields[0] == "rht":
        rows, width = int(fields[1]), int(fields[2])
        us = time_transform(device, rows, width, launches, repetitions=2)
        print(json.dumps({"case": spec, "launches": launches, "us_per_launch": round(us, 2),
                          "bytes_per_launch": 2 * rows * width * 2 + width}))
        return
    out_rows, width = LLAMA8B[fields[0]]
    rows = int(fields[1]) if len(fields) > 1 else 1
    kernel = fields[2] if len(fields) > 2 else "auto"
    generator = torch.Generator(device=device).manual_seed(5)
    packed = [torch.randint(0, 256, (out_rows * width * BITS // 8,), dtype=torch.uint8, device=device, generator=generator)
              for _ in range(launches)]
    scales = [(torch.rand(out_rows, width // GROUP, device=device, generator=generator) * 0.01 + 0.001).half()
              for _ in range(launches)]
    values = torch.arange(-8, 8, dtype=torch.float32, device=device)
    x = torch.randn(rows, width, device=device, generator=generator).half()
    out = torch.empty(rows, out_rows, device=device, dtype=torch.float16)

    def launch(i):
        kernels.packed_matvec(x, packed[i], scales[i], values, None, None, out, group=GROUP, bits=BITS,
                              integer_grid=True, grid_minimum=-8.0, kernel=kernel)
    launch(0)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(launches):
        launch(i)
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / launches
    print(json.dumps({"case": spec, "launches": launches, "us_per_launch_eager": round(us, 2),
                      "bytes_per_launch": gemv_bytes(out_rows, width, rows)}))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--case", default=None,
                        help="small single-shape run for a profiler: NAME[:ROWS[:KERNEL]], NAME one of " + ",".join(LLAMA8B))
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        seconds, threads, bytes_per_pass = time_cpu_route(max(1, args.steps), max(0, args.warmup))
        value = bytes_per_pass / seconds / 1e9
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama3-8b block linears int4 g128 (q,k,v,o,gate,up,down), M=1, CPU reconstruct+matmul"},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": "one decoder block (7 linears, 109 MB packed), M=1, per step"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        from mlkit_b200 import tp_bench

        tp_bench.run(args, rank, world, device, peaks())
        dist.destroy_process_group()
        return

    if args.case:
        run_case(args.case, device, max(1, args.steps))
        return

    peak, peak_kind = peaks()
    blocks = build_blocks(device, BLOCKS)
    generator = torch.Generator(device=device).manual_seed(7)
    widths = sorted({k for (_, k) in LLAMA8B.values()})
    outs = sorted({n for (n, _) in LLAMA8B.values()})
    inputs = {m: {k: torch.randn(m, k, generator=generator, device=device).half() for k in widths} for m in ROW_COUNTS}
    outputs = {m: {n: torch.empty(m, n, device=device, dtype=torch.float16) for n in outs} for m in ROW_COUNTS}
    host_inputs = {m: {k: inputs[m][k].cpu().pin_memory() for k in widths} for m in ROW_COUNTS}
    host_outputs = {m: {n: torch.empty(m, n, dtype=torch.float16).pin_memory() for n in outs} for m in ROW_COUNTS}

    # ---- resident-input timing: W warm-up steps, then exactly K steps between two events ----
    graph, launches_per_step = capture_pass(blocks, inputs, outputs)
    for _ in range(max(3, args.warmup)):
        graph.replay()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as sampler:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        resident_ms = start.elapsed_time(stop) / args.steps
        launches = launches_per_step * args.steps
        # the same step launched eagerly (host launch path included)
        start.record()
        for _ in range(args.steps):
            run_pass_resident(blocks, inputs, outputs)
        stop.record()
        torch.cuda.synchronize()
        eager_ms = start.elapsed_time(stop) / args.steps
        # ---- end-to-end timing through the module call with host activations ----
        with torch.inference_mode():
            for _ in range(max(3, args.warmup)):
                run_pass_e2e(blocks, host_inputs, host_outputs, device)
            torch.cuda.synchronize()
            start.record()
            for _ in range(args.steps):
                h2d, d2h = run_pass_e2e(blocks, host_inputs, host_outputs, device)
            stop.record()
            torch.cuda.synchronize()
            e2e_ms = start.elapsed_time(stop) / args.steps
        table = per_layer_table(blocks, inputs, outputs, peak)
    step_bytes = pass_bytes(BLOCKS)
    value = step_bytes / resident_ms / 1e6
    # the dominant kernel by share of device time is the tiled kernel (profiles/bench_launch_list.md);
    # its largest launch is the gate/up shape at one row.  The TMA-fed kernel takes the same shape at 8 rows.
    gate_bytes, gate_us = gemv_bytes(14336, 4096, 1), table["gate_4096x14336_M1"]["us"]
    achieved = gate_bytes / gate_us / 1e3
    bulk_bytes, bulk_us = gemv_bytes(14336, 4096, 8), table["gate_4096x14336_M8"]["us"]

    cpu_seconds, cpu_threads, cpu_bytes = time_cpu_route(repetitions=3, warmup=1)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": resident_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"llama3-8b block linears int4 g128 (q,k,v,o,gate,up,down) x M in {list(ROW_COUNTS)} x {BLOCKS} distinct blocks",
                   "l2": f"inputs larger than L2: {BLOCKS} blocks = {BLOCKS * 113} MB of packed weights cycled",
                   "pct_of_8tbs": round(value / 8000 * 100, 2), "launch": "one CUDA graph per step",
                   "eager_ms_per_step": round(eager_ms, 4)},
        "e2e": {"value": step_bytes / e2e_ms / 1e6, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": sampler.summary,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": TILED_GATE_M1_DRAM_BYTES, "peak_kind": peak_kind,
                     "kernel": "gemv_tiled_kernel<4, raw> on gate/up 4096->14336, M=1",
                     "bytes_per_launch": gate_bytes, "us_per_launch": gate_us},
        "roofline_bulk": {"bound": "hbm", "achieved": bulk_bytes / bulk_us / 1e3, "peak": peak, "unit": "GB/s",
                          "frac": bulk_bytes / bulk_us / 1e3 / peak, "traffic": BULK_GATE_M8_DRAM_BYTES,
                          "peak_kind": peak_kind, "kernel": "gemv_bulk_kernel on gate/up 4096->14336, M=8",
                          "bytes_per_launch": bulk_bytes, "us_per_launch": bulk_us},
        "per_layer": table,
        "cpu_baseline": {"value": cpu_bytes / cpu_seconds / 1e9, "unit": "GB/s", "cores": cpu_threads, "kind": "port",
                         "sample": "one decoder block (7 linears, 109 MB packed), M=1, median of 3 passes"},
    }
    try:   # an auxiliary table: a failure here must not cost the matvec numbers above
        line["transform"] = transform_table(device, peak)
    except Exception as error:
        line["transform"] = {"error": repr(error)[:200]}
    # the 70B-shaped decode step on this one GPU (the N > 1 runs shard the same model)
    del blocks, graph
    torch.cuda.empty_cache()
    from mlkit_b200 import tp_bench

    decode = tp_bench.measure(0, 1, device, steps=max(5, args.steps), warmup=3)
    line["decode"] = {
        "workload": f"llama3-70b-shaped int4 g128 decode, tp1, ctx {tp_bench.CONTEXT}, one CUDA graph per step",
        "tokens_per_s": {f"batch{b}": r["tokens_per_s"] for b, r in decode["batches"].items()},
        "e2e_tokens_per_s": {f"batch{b}": r["e2e_tokens_per_s"] for b, r in decode["batches"].items()},
        "ms_per_step": {f"batch{b}": r["ms_per_step"] for b, r in decode["batches"].items()},
        "per_gpu_roofline_frac": {f"batch{b}": r["per_gpu_gbps"] / peak for b, r in decode["batches"].items()},
        "launches_per_step": decode["launches_per_step"],
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
