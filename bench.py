"""Benchmark of the packed INT4-g128 matvec path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One process per GPU (for N > 1 launch under ``python -m torch.distributed.run``).  Rank 0 prints one
JSON line.

N = 1: the workload is the seven block linears of a Llama-3-8B-shaped decoder block (q, k, v, o,
gate, up, down; INT4, group 128, fp16 scales; weights N(0, 0.02) from a seed, RTN-quantised on the
device by this package's own ``mk.int(4, group=128)``), with 1, 2, 4 and 8 activation rows.  The block
is built the way ``mk.optimize`` builds it: q | k | v and gate | up share one launch each, so a block
is four launches.  A step is one pass of the packed matvec over ``BLOCKS`` distinct blocks x 7 linears
x 4 row counts.  The blocks together hold ~0.9 GB of packed weights, so no weight is served from L2
twice in a row.

N > 1: the 70B-shaped tensor-parallel decode step of ``mlkit_b200.tp`` (see ``bench_tp.py``).

``value`` is algorithmic GB/s with every input resident in HBM; ``e2e`` is the same pass through the
public module call (``mk.capture`` of a block whose forward calls its seven ``PackedLinear``: one
CUDA graph per call with its host copies as nodes) with activations coming from pinned host memory
and results returned to it inside the timed region.  ``--impl reference`` times the reference's CPU route
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
LLAMA70B_BLOCK = {"q": (8192, 8192), "k": (1024, 8192), "v": (1024, 8192), "o": (8192, 8192),
                  "gate": (28672, 8192), "up": (28672, 8192), "down": (8192, 28672)}
PROJECTION = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "gate": "gate_proj", "up": "up_proj",
              "down": "down_proj"}
ROW_COUNTS = (1, 2, 4, 8)
BLOCKS = 8
BITS, GROUP = 4, 128
METRIC = "packed_int4_g128_gemv_hbm_gbps"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the profiler
# capture summarised in the file named beside it (a past capture, not a counter of this run)
DOMINANT_DRAM_BYTES = 30352000
DOMINANT_DRAM_SOURCE = ("dram__bytes_read.sum + dram__bytes_write.sum of gemv_stream_kernel<4,0,1,2,3> on 4096->14336, M=1, "
                        "one ncu --set full capture (profiles/gemv_stream_gate_4096x14336_M1.md): 30.352 MB read, 0 written")


def matvec_bytes(out_rows: int, width: int, rows_in: int, bits: int = BITS, group: int = GROUP, levels: int = 16) -> int:
    """Algorithmic bytes of one packed matvec: codes + fp16 scales + activations + outputs + table."""
    return (out_rows * width * bits // 8 + out_rows * (width // group) * 2 + rows_in * width * 2 +
            rows_in * out_rows * 2 + 4 * levels)


E2E_STREAMS = 4


def pass_bytes(blocks: int) -> int:
    return blocks * sum(matvec_bytes(n, k, m) for (n, k) in LLAMA8B.values() for m in ROW_COUNTS)


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


def graph_of(launch_all) -> torch.cuda.CUDAGraph:
    """``launch_all`` captured as one CUDA graph (run once eagerly first, on a side stream)."""
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
    return graph


def replay_us(graph: torch.cuda.CUDAGraph, launches: int, repetitions: int = 7) -> dict:
    """Microseconds per launch over ``repetitions`` replays: median and minimum."""
    samples = []
    for _ in range(repetitions):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) * 1e3 / launches)
    return {"median": statistics.median(samples), "min": min(samples)}


def entry(us: dict, moved: int, peak: float) -> dict:
    gbps = moved / us["median"] / 1e3
    return {"us": round(us["median"], 3), "us_min": round(us["min"], 3), "gbps": round(gbps, 1), "frac": round(gbps / peak, 4)}


# ---------------------------------------------------------------- the decoder blocks
def build_blocks(device: torch.device, blocks: int):
    """``blocks`` decoder blocks of seven ``PackedLinear`` layers, RTN-quantised on the device, siblings
    grouped as ``mk.optimize`` groups them."""
    import mlkit_b200 as mk
    from torch import nn

    generator = torch.Generator(device=device).manual_seed(1234)
    fmt = mk.int(BITS, group=GROUP)
    result = []
    for _ in range(blocks):
        block = nn.Module()
        for name, (out_rows, width) in LLAMA8B.items():
            weight = (torch.randn(out_rows, width, generator=generator, device=device) * 0.02).half()
            linear = nn.Linear(width, out_rows, bias=False, device=device, dtype=torch.float16)
            with torch.no_grad():
                linear.weight.copy_(weight)
            q = fmt(weight.float(), mk.Ctx(name, device=device))
            setattr(block, PROJECTION[name], mk.PackedLinear(linear, q))
            del linear, weight, q
        assert mk.fuse_siblings(block) == 2
        result.append(block)
    torch.cuda.empty_cache()
    return result


def block_launches(block):
    """The four launches of one block: (plan, input width, output width)."""
    return [(block.q_proj._siblings.plan(torch.float16), 4096, 6144), (block.o_proj._plan(torch.float16), 4096, 4096),
            (block.gate_proj._siblings.plan(torch.float16), 4096, 28672), (block.down_proj._plan(torch.float16), 14336, 4096)]


def run_pass_resident(blocks, inputs, outputs) -> int:
    """One step with everything in HBM: bound launches on preallocated outputs.  Returns launches."""
    launches = 0
    for rows in ROW_COUNTS:
        for block in blocks:
            for plan, width, out_rows in block_launches(block):
                plan(inputs[rows][width], outputs[rows][out_rows])
                launches += 1
    return launches


class BlockCall(torch.nn.Module):
    """The seven linears of one block as a module call: (hidden, mlp) -> the seven outputs."""

    def __init__(self, block) -> None:
        super().__init__()
        self.block = block

    def forward(self, hidden, mlp):
        b = self.block
        return (b.q_proj(hidden), b.k_proj(hidden), b.v_proj(hidden), b.o_proj(hidden), b.gate_proj(hidden),
                b.up_proj(hidden), b.down_proj(mlp))


def run_pass_e2e(calls, host_inputs, streams) -> tuple[int, int]:
    """One step through the public module call (``mk.capture`` of a block of ``PackedLinear``) with
    host-resident activations and results: the copies from and to pinned host memory are part of
    every call.  The calls are independent, so they alternate between ``streams`` and one call's
    copies overlap another's kernels; the current stream waits for all of them at the end."""
    h2d = d2h = 0
    main = torch.cuda.current_stream()
    for stream in streams:
        stream.wait_stream(main)
    turn = 0
    for rows in ROW_COUNTS:
        hidden, mlp = host_inputs[rows][4096], host_inputs[rows][14336]
        for call in calls:
            with torch.cuda.stream(streams[turn % len(streams)]):
                outputs = call(hidden, mlp)
            turn += 1
            h2d += (hidden.numel() + mlp.numel()) * 2
            d2h += sum(y.numel() for y in outputs) * 2
    for stream in streams:
        main.wait_stream(stream)
    return h2d, d2h


def per_layer_tables(blocks, inputs, outputs, peak: float) -> tuple[dict, dict]:
    """Launch duration per layer shape and row count (all blocks' launches in one graph, which keeps
    every weight cold in L2), as algorithmic GB/s and roofline fraction: every linear alone, and the
    grouped launches the module path issues."""
    alone, grouped = {}, {}
    for name, (out_rows, width) in LLAMA8B.items():
        if name in ("v", "up"):
            continue
        for rows in ROW_COUNTS:
            out = torch.empty(rows, out_rows, device=inputs[rows][width].device, dtype=torch.float16)
            plans = [getattr(block, PROJECTION[name])._plan(torch.float16) for block in blocks]
            graph = graph_of(lambda: [plan(inputs[rows][width], out) for plan in plans])
            alone[f"{name}_{width}x{out_rows}_M{rows}"] = entry(replay_us(graph, len(blocks)),
                                                                matvec_bytes(out_rows, width, rows), peak)
    for label, member, out_rows in (("qkv", "q_proj", 6144), ("gate_up", "gate_proj", 28672)):
        for rows in ROW_COUNTS:
            plans = [getattr(block, member)._siblings.plan(torch.float16) for block in blocks]
            graph = graph_of(lambda: [plan(inputs[rows][4096], outputs[rows][out_rows]) for plan in plans])
            grouped[f"{label}_4096x{out_rows}_M{rows}"] = entry(replay_us(graph, len(blocks)),
                                                                matvec_bytes(out_rows, 4096, rows), peak)
    return alone, grouped


# ---------------------------------------------------------------- other configurations of the baseline
def single_layers(device, out_rows: int, width: int, fmt, copies: int, seed: int):
    """``copies`` distinct ``PackedLinear`` layers of one shape and format (weights N(0, 0.02))."""
    import mlkit_b200 as mk
    from torch import nn

    generator = torch.Generator(device=device).manual_seed(seed)
    layers = []
    for _ in range(copies):
        weight = (torch.randn(out_rows, width, generator=generator, device=device) * 0.02).half()
        linear = nn.Linear(width, out_rows, bias=False, device=device, dtype=torch.float16)
        with torch.no_grad():
            linear.weight.copy_(weight)
        layers.append(mk.PackedLinear(linear, fmt(weight.float(), mk.Ctx("layer", device=device))))
    return layers


def time_layers(layers, rows: int, peak: float, moved: int) -> dict:
    width, out_rows = layers[0].in_features, layers[0].out_features
    device = layers[0].packed.device
    x = torch.randn(rows, width, device=device).half()
    out = torch.empty(rows, out_rows, device=device, dtype=torch.float16)
    plans = [layer._plan(torch.float16) for layer in layers]
    graph = graph_of(lambda: [plan(x, out) for plan in plans])
    return entry(replay_us(graph, len(layers)), moved, peak)


def codec_table(device, peak: float) -> dict:
    """The codec sweep on one 4096 -> 14336 linear, M in {1, 8}."""
    import mlkit_b200 as mk

    codebook = torch.tensor([-1, -0.5, -0.25, 0, 0.25, 0.5, 1.0])
    formats = {
        "int2_g128": (mk.int(2, group=128), 2, 128, 4), "int3_g128": (mk.int(3, group=128), 3, 128, 8),
        "int4_g128": (mk.int(4, group=128), 4, 128, 16), "int5_g128": (mk.int(5, group=128), 5, 128, 32),
        "int6_g128": (mk.int(6, group=128), 6, 128, 64), "int7_g128": (mk.int(7, group=128), 7, 128, 128),
        "int8_g128": (mk.int(8, group=128), 8, 128, 256),
        "nf4_g64": (mk.nf4(group=64), 4, 64, 16),
        "codebook3_g64_mse": (mk.scaled(mk.grid.values(codebook, bits=3), group=64, scale="mse"), 3, 64, 7),
    }
    table = {}
    for name, (fmt, bits, group, levels) in formats.items():
        layers = single_layers(device, 14336, 4096, fmt, copies=4, seed=bits * 100 + group)
        for rows in (1, 8):
            table[f"{name}_M{rows}"] = time_layers(layers, rows, peak, matvec_bytes(14336, 4096, rows, bits, group, levels))
        del layers
        torch.cuda.empty_cache()
    return table


def rotated_table(device, peak: float) -> dict:
    """The Hadamard-rotated INT4 path: transform and matvec chained in one graph, against the matvec alone."""
    import mlkit_b200 as mk
    from mlkit_b200 import kernels

    table = {}
    generator = torch.Generator(device=device).manual_seed(21)
    for width, out_rows in ((4096, 4096), (14336, 4096)):
        layers = single_layers(device, out_rows, width, mk.int(4, group=128), copies=8, seed=width)
        signs = (torch.randint(0, 2, (width,), device=device, generator=generator) * 2 - 1).to(torch.int8)
        plans = [layer._plan(torch.float16) for layer in layers]
        for rows in (1, 2, 4, 8):
            x = torch.randn(rows, width, device=device, generator=generator)
            picks = torch.randperm(width, device=device, generator=generator)[: width // 100]
            x[:, picks] *= 50
            x = x.half()
            out = torch.empty(rows, out_rows, device=device, dtype=torch.float16)
            chained = graph_of(lambda: [plan(mk.rht(x, signs=signs), out) for plan in plans])
            alone = graph_of(lambda: [plan(x, out) for plan in plans])
            moved = matvec_bytes(out_rows, width, rows)
            both, only = replay_us(chained, len(plans)), replay_us(alone, len(plans))
            record = dict(entry(both, moved, peak), matvec_alone_us=round(only["median"], 3))
            if kernels.rotated_matvec_supported(rows, width, torch.float16):
                # rotation on load inside the matvec launch (mkb_gemv_hadamard): what the module path takes
                fused = graph_of(lambda: [kernels.packed_matvec_rotated(
                    x, signs, layer.packed, layer.scales, layer.values, None, out, group=GROUP, bits=BITS,
                    integer_grid=True, grid_minimum=-8.0) for layer in layers])
                record["fused_us"] = round(replay_us(fused, len(layers))["median"], 3)
            table[f"rht+matvec_{width}x{out_rows}_M{rows}"] = record
        del layers
        torch.cuda.empty_cache()
    return table


def time_transform(device: torch.device, rows: int, width: int, copies: int) -> dict:
    """The randomised Hadamard transform (signs, FWHT, Paley factor for 14336 = 28 x 512) on fp16
    ``[rows, width]``, over ``copies`` distinct inputs replayed as one CUDA graph."""
    import mlkit_b200 as mk

    generator = torch.Generator(device=device).manual_seed(11)
    inputs = [torch.randn(rows, width, device=device, generator=generator).half() for _ in range(copies)]
    signs = (torch.randint(0, 2, (width,), device=device, generator=generator) * 2 - 1).to(torch.int8)
    graph = graph_of(lambda: [mk.rht(x, signs=signs) for x in inputs])
    return replay_us(graph, copies, repetitions=5)


def transform_table(device: torch.device, peak: float) -> dict:
    """The activation transform at decode sizes (latency-bound) and on a large batch (its bandwidth ceiling)."""
    table = {}
    for rows, width, copies in ((1, 4096, 16), (8, 4096, 16), (8, 14336, 16), (16384, 4096, 4), (8192, 14336, 4)):
        table[f"rht_{rows}x{width}"] = entry(time_transform(device, rows, width, copies), 2 * rows * width * 2 + width, peak)
    return table


def gemm_table(device, peak: float) -> dict:
    """The fused dequantise + GEMM (``mkb_gemm``, 9..128 activation rows) on the gate and down shapes,
    beside the dense route it replaces (reconstruct the fp16 weight, then the library GEMM): per launch
    over 6 distinct weights in one graph, algorithmic GB/s and TFLOP/s."""
    from mlkit_b200 import kernels

    generator = torch.Generator(device=device).manual_seed(11)
    values = torch.arange(-8, 8, dtype=torch.float32, device=device)
    table = {}
    for name, (out_rows, width) in (("gate", (14336, 4096)), ("down", (4096, 14336))):
        packed = [torch.randint(0, 256, (out_rows * width // 2,), dtype=torch.uint8, device=device, generator=generator)
                  for _ in range(6)]
        scales = [(torch.rand(out_rows, width // GROUP, device=device, generator=generator) * 0.01 + 0.001).half()
                  for _ in range(6)]
        for rows in (16, 32, 64, 128):
            x = torch.randn(rows, width, device=device, generator=generator).half()
            out = torch.empty(rows, out_rows, device=device, dtype=torch.float16)

            def fused():
                for i in range(6):
                    kernels.packed_gemm(x, packed[i], scales[i], values, None, out, group=GROUP, bits=BITS,
                                        integer_grid=True, grid_minimum=-8.0)

            def dense():
                for i in range(6):
                    weight, _ = kernels.dequantize(packed[i], scales[i], values, None, shape=(out_rows, width),
                                                   group=GROUP, bits=BITS, dtype=torch.float16)
                    torch.nn.functional.linear(x, weight)

            moved = matvec_bytes(out_rows, width, rows)
            record = entry(replay_us(graph_of(fused), 6), moved, peak)
            record["tflops"] = round(2 * rows * out_rows * width / record["us"] / 1e6, 1)
            record["dense_route_us"] = round(replay_us(graph_of(dense), 6)["median"], 3)
            table[f"{name}_{width}x{out_rows}_M{rows}"] = record
        del packed, scales
        torch.cuda.empty_cache()
    table["status"] = kernels.gemm_status()
    return table


def comparator_table(device, peak: float) -> dict:
    """The reference's own Triton ``PackedLinear`` and dense fp16 ``F.linear`` on this GPU, with the
    per-layer protocol (8 weight copies in one graph).  Comparators only: nothing of the product runs
    through them.  The reference is imported from ``baseline/_ref`` when it was installed there."""
    from torch import nn

    shapes = {"gate": (14336, 4096), "down": (4096, 14336), "q": (4096, 4096), "k": (1024, 4096)}
    result = {"dense_fp16": {}, "triton_reference": {}}
    generator = torch.Generator(device=device).manual_seed(3)
    for name, (out_rows, width) in shapes.items():
        weights = [(torch.randn(out_rows, width, generator=generator, device=device) * 0.02).half() for _ in range(8)]
        for rows in (1, 8):
            x = torch.randn(rows, width, device=device).half()
            graph = graph_of(lambda: [torch.nn.functional.linear(x, w) for w in weights])
            result["dense_fp16"][f"{name}_M{rows}"] = entry(replay_us(graph, 8), out_rows * width * 2 + rows * (width + out_rows) * 2, peak)
        del weights
    reference_path = ROOT / "baseline" / "_ref"
    if not (reference_path / "mlkit").exists():
        result["triton_reference"] = {"unavailable": "baseline/_ref holds no installed reference"}
        return result
    sys.path.insert(0, str(reference_path))
    try:
        import mlkit as mk_ref

        for name, (out_rows, width) in shapes.items():
            modules = []
            for _ in range(8):
                linear = nn.Sequential(nn.Linear(width, out_rows, bias=False, device=device, dtype=torch.float16))
                with torch.no_grad():
                    linear[0].weight.normal_(0, 0.02, generator=generator)
                quantized = mk_ref.quantize(linear, mk_ref.int(4, group=128), calib=None)
                modules.append(mk_ref.optimize(quantized, backend="packed"))
            for rows in (1, 8):
                x = torch.randn(rows, width, device=device).half()
                with torch.inference_mode():
                    graph = graph_of(lambda: [module(x) for module in modules])
                    result["triton_reference"][f"{name}_M{rows}"] = entry(replay_us(graph, 8),
                                                                          matvec_bytes(out_rows, width, rows), peak)
            del modules
            torch.cuda.empty_cache()
    except Exception as error:  # Triton cannot compile here, or the reference refuses the device
        result["triton_reference"]["error"] = repr(error)[:300]
    finally:
        sys.path.remove(str(reference_path))
    return result


# ---------------------------------------------------------------- the CPU route (reference arm)
def cpu_reference_layers(shapes: dict):
    """Host copies of block linears for the CPU route (random codes: arithmetic cost is value-blind)."""
    generator = torch.Generator().manual_seed(99)
    layers = []
    for name, (out_rows, width) in shapes.items():
        layers.append({
            "packed": torch.randint(0, 256, (out_rows * width * BITS // 8,), dtype=torch.uint8, generator=generator),
            "scales": (torch.rand(out_rows, width // GROUP, generator=generator) * 0.01 + 0.001).half(),
            "values": torch.arange(-8, 8, dtype=torch.float32), "group": GROUP, "bits": BITS,
            "shape": (out_rows, width),
        })
    return layers


def time_cpu_route(repetitions: int, warmup: int, shapes: dict | None = None):
    """Seconds per pass of unpack + reconstruct + F.linear over one block's seven linears, M = 1, on
    every host core (a launcher such as torch.distributed.run pins OMP_NUM_THREADS to 1: undone here)."""
    from oracle import cpu_path

    torch.set_num_threads(os.cpu_count() or 1)
    shapes = shapes or LLAMA8B
    layers = cpu_reference_layers(shapes)
    seconds, threads = cpu_path.time_reconstruct_plus_matmul(layers, rows_in=1, repetitions=repetitions, warmup=warmup)
    bytes_per_pass = sum(matvec_bytes(n, k, 1) for (n, k) in shapes.values())
    return seconds, threads, bytes_per_pass


def reference_arm(args) -> None:
    """``--impl reference``: the reference's CPU route for the configuration the other arm times at this
    N.  N = 1: one Llama-3-8B block at one row, scaled to nothing (GB/s is size-free).  N > 1: one
    70B-shaped block, times 80 blocks per decode step, so that the line is the same step in the same unit."""
    if args.gpus > 1:
        seconds, threads, bytes_per_pass = time_cpu_route(max(1, min(args.steps, 2)), 0, LLAMA70B_BLOCK)
        step_seconds, step_bytes = seconds * 80, bytes_per_pass * 80
        workload = "llama3-70b-shaped int4 g128 decode step, batch 1: one block timed on the CPU x 80 blocks (head and cache left out)"
        sample = "one 70B-shaped decoder block (7 linears, 428 MB packed), M=1, per step; x 80 for the step"
    else:
        seconds, threads, bytes_per_pass = time_cpu_route(max(1, args.steps), max(0, args.warmup))
        step_seconds, step_bytes = seconds, bytes_per_pass
        workload = "llama3-8b block linears int4 g128 (q,k,v,o,gate,up,down), M=1, CPU reconstruct+matmul"
        sample = "one decoder block (7 linears, 109 MB packed), M=1, per step"
    value = step_bytes / step_seconds / 1e9
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_seconds * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def mk_nf4_levels() -> list:
    from mlkit_b200.quantization import NF4_VALUES

    return [float(v) for v in NF4_VALUES]


def run_case(spec: str, device: torch.device, launches: int) -> None:
    """One layer shape, ``launches`` launches over distinct weight copies (each cold in L2), nothing
    else on the device: the small case a profiler captures.  Prints the mean launch time.
    ``NAME[:ROWS[:KERNEL]]`` with NAME a block linear, ``qkv`` or ``gate_up``; ``gemm:NAME:ROWS`` runs the
    fused dequantise + GEMM on that shape; ``codec:NAME:ROWS`` one codec of the sweep on the gate shape; ``rht:ROWS:WIDTH`` runs
    the activation transform instead; ``tp_layer:WORLD:BATCH`` times the operators of one decoder layer with
    the shard shapes of WORLD ranks."""
    from mlkit_b200 import kernels

    fields = spec.split(":")
    if fields[0] == "tp_layer":     # tp_layer:WORLD:BATCH -- per-operator times of one tensor-parallel-shaped layer
        import bench_tp

        world, batch = int(fields[1]), int(fields[2]) if len(fields) > 2 else 1
        print(json.dumps({"case": spec, "us": bench_tp.layer_breakdown(world, batch, device)}))
        return
    if fields[0] == "rht":
        rows, width = int(fields[1]), int(fields[2])
        us = time_transform(device, rows, width, launches)
        print(json.dumps({"case": spec, "launches": launches, "us_per_launch": round(us["median"], 2),
                          "bytes_per_launch": 2 * rows * width * 2 + width}))
        return
    if fields[0] == "codec":        # codec:NAME:ROWS -- one codec of the sweep on the gate shape, random codes
        tables = {"nf4_g64": (4, 64, mk_nf4_levels()), "nf4_g128": (4, 128, mk_nf4_levels()),
                  "codebook3_g64": (3, 64, [-1, -0.5, -0.25, 0, 0.25, 0.5, 1.0]),
                  "int3_g128": (3, 128, list(range(-4, 4))), "int7_g128": (7, 128, list(range(-64, 64)))}
        bits, group, levels = tables[fields[1]]
        rows = int(fields[2]) if len(fields) > 2 else 1
        out_rows, width = LLAMA8B["gate"]
        generator = torch.Generator(device=device).manual_seed(5)
        packed = [torch.randint(0, 256, (out_rows * width * bits // 8,), dtype=torch.uint8, device=device, generator=generator)
                  for _ in range(launches)]
        scales = [(torch.rand(out_rows, width // group, device=device, generator=generator) * 0.01 + 0.001).half()
                  for _ in range(launches)]
        values = torch.tensor(levels, dtype=torch.float32, device=device)
        integer = fields[1].startswith("int")
        x = torch.randn(rows, width, device=device, generator=generator).half()
        out = torch.empty(rows, out_rows, device=device, dtype=torch.float16)
        run = lambda i: kernels.packed_matvec(x, packed[i], scales[i], values, None, None, out, group=group, bits=bits,
                                              integer_grid=integer, grid_minimum=float(levels[0]) if integer else 0.0)
        run(0)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(launches):
            run(i)
        stop.record()
        torch.cuda.synchronize()
        print(json.dumps({"case": spec, "launches": launches,
                          "us_per_launch_eager": round(start.elapsed_time(stop) * 1e3 / launches, 2),
                          "bytes_per_launch": matvec_bytes(out_rows, width, rows, bits, group, len(levels))}))
        return
    shapes = dict(LLAMA8B, qkv=(6144, 4096), gate_up=(28672, 4096))
    fused_gemm = fields[0] == "gemm"      # gemm:NAME:ROWS -- the fused dequantise + GEMM on that layer shape
    if fused_gemm:
        fields = fields[1:]
    out_rows, width = shapes[fields[0]]
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
        if fused_gemm:
            kernels.packed_gemm(x, packed[i], scales[i], values, None, out, group=GROUP, bits=BITS, integer_grid=True,
                                grid_minimum=-8.0)
        else:
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
                      "bytes_per_launch": matvec_bytes(out_rows, width, rows),
                      "flops_per_launch": 2 * rows * out_rows * width}))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--case", default=None,
                        help="small single-shape run for a profiler: NAME[:ROWS[:KERNEL]], NAME one of " +
                             ",".join(LLAMA8B) + ",qkv,gate_up, or rht:ROWS:WIDTH")
    parser.add_argument("--quick", action="store_true", help="skip the auxiliary tables and the 70B-shaped decode")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            reference_arm(args)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        import bench_tp

        dist.init_process_group("nccl", device_id=device)
        bench_tp.run(args, rank, world, device, peaks())
        dist.destroy_process_group()
        return

    if args.case:
        run_case(args.case, device, max(1, args.steps))
        return

    peak, peak_kind = peaks()
    blocks = build_blocks(device, BLOCKS)
    generator = torch.Generator(device=device).manual_seed(7)
    widths = (4096, 14336)
    outs = (4096, 6144, 28672)
    inputs = {m: {k: torch.randn(m, k, generator=generator, device=device).half() for k in widths} for m in ROW_COUNTS}
    outputs = {m: {n: torch.empty(m, n, device=device, dtype=torch.float16) for n in outs} for m in ROW_COUNTS}
    host_inputs = {m: {k: inputs[m][k].cpu().pin_memory() for k in widths} for m in ROW_COUNTS}

    # ---- resident-input timing: W warm-up steps, then exactly K steps between two events ----
    launches_per_step = run_pass_resident(blocks, inputs, outputs)
    graph = graph_of(lambda: run_pass_resident(blocks, inputs, outputs))
    for _ in range(max(3, args.warmup)):
        graph.replay()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as sampler:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()     # a profiler started with its collection off sees the timed region only
        start.record()
        for _ in range(args.steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
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
        import mlkit_b200 as mk

        calls = [mk.capture(BlockCall(block), synchronize=False) for block in blocks]
        streams = [torch.cuda.Stream() for _ in range(E2E_STREAMS)]
        for _ in range(max(3, args.warmup)):
            run_pass_e2e(calls, host_inputs, streams)
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            h2d, d2h = run_pass_e2e(calls, host_inputs, streams)
        stop.record()
        torch.cuda.synchronize()
        e2e_ms = start.elapsed_time(stop) / args.steps
        del calls
        alone, grouped = per_layer_tables(blocks, inputs, outputs, peak)
    step_bytes = pass_bytes(BLOCKS)
    value = step_bytes / resident_ms / 1e6
    # the dominant kernel by share of device time is the streaming kernel; its largest launch in the
    # pass is gate | up (4096 -> 28672) and the single-layer reference point is gate alone at one row
    top = alone["gate_4096x14336_M1"]
    top_bytes = matvec_bytes(14336, 4096, 1)

    cpu_seconds, cpu_threads, cpu_bytes = time_cpu_route(repetitions=3, warmup=1)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": resident_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"llama3-8b block linears int4 g128 (q,k,v,o,gate,up,down) x M in {list(ROW_COUNTS)} x {BLOCKS} distinct blocks; "
                               "q|k|v and gate|up share one launch each, as mk.optimize builds the block",
                   "l2": f"inputs larger than L2: {BLOCKS} blocks = {BLOCKS * 113} MB of packed weights cycled",
                   "pct_of_8tbs": round(value / 8000 * 100, 2), "launch": "one CUDA graph per step",
                   "eager_ms_per_step": round(eager_ms, 4)},
        "e2e": {"value": step_bytes / e2e_ms / 1e6, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": sampler.summary,
        "roofline": {"bound": "hbm", "achieved": top_bytes / top["us"] / 1e3, "peak": peak, "unit": "GB/s",
                     "frac": top_bytes / top["us"] / 1e3 / peak, "traffic": DOMINANT_DRAM_BYTES,
                     "traffic_source": DOMINANT_DRAM_SOURCE, "peak_kind": peak_kind,
                     "kernel": "gemv_stream_kernel<4, 2, 3> on gate/up 4096->14336, M=1 (median of 7 graph replays of 8 launches)",
                     "bytes_per_launch": top_bytes, "us_per_launch": top["us"]},
        "per_layer": alone,
        "per_layer_fused": grouped,
        "cpu_baseline": {"value": cpu_bytes / cpu_seconds / 1e9, "unit": "GB/s", "cores": cpu_threads, "kind": "port",
                         "sample": "one decoder block (7 linears, 109 MB packed), M=1, median of 3 passes"},
    }
    del blocks, graph
    torch.cuda.empty_cache()
    if not args.quick:
        for name, build in (("qwen_up", lambda: {"qwen_up_896x4864_M1": time_layers(
                                single_layers(device, 4864, 896, __import__("mlkit_b200").int(4, group=128), 16, 5), 1, peak,
                                matvec_bytes(4864, 896, 1))}),
                            ("per_codec", lambda: codec_table(device, peak)),
                            ("fused_gemm", lambda: gemm_table(device, peak)),
                            ("rotated", lambda: rotated_table(device, peak)),
                            ("transform", lambda: transform_table(device, peak)),
                            ("comparators", lambda: comparator_table(device, peak))):
            try:   # auxiliary tables: a failure here must not cost the matvec numbers above
                line[name] = build()
            except Exception as error:
                line[name] = {"error": repr(error)[:300]}
            torch.cuda.empty_cache()
        # the 70B-shaped decode step on this one GPU (the N > 1 runs shard the same model)
        import bench_tp

        decode = bench_tp.measure(0, 1, device, steps=max(5, args.steps), warmup=3)
        line["decode"] = {
            "workload": f"llama3-70b-shaped int4 g128 decode, tp1, ctx {bench_tp.CONTEXT}, one CUDA graph per step",
            "tokens_per_s": {f"batch{b}": r["tokens_per_s"] for b, r in decode["batches"].items()},
            "e2e_tokens_per_s": {f"batch{b}": r["e2e_tokens_per_s"] for b, r in decode["batches"].items()},
            "ms_per_step": {f"batch{b}": r["ms_per_step"] for b, r in decode["batches"].items()},
            "aggregate_gbps": {f"batch{b}": r["aggregate_gbps"] for b, r in decode["batches"].items()},
            "per_gpu_roofline_frac": {f"batch{b}": r["per_gpu_gbps"] / peak for b, r in decode["batches"].items()},
            "launches_per_step": decode["launches_per_step"],
        }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
