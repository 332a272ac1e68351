"""Timing of the 70B-shaped tensor-parallel decode step (the multi-GPU workload of ``bench.py``).

Random-initialised Llama-3-70B shape (80 layers, hidden 8192, 64 query / 8 key-value heads, MLP 28672,
vocabulary 128256 with an fp16 head); every block linear INT4 with group 128; a 512-token synthetic
context in the KV cache; 1 to 8 sequences decoding one token each.  Total work is fixed as ranks are
added (strong scaling): each rank streams 1/N of the packed weights per step.
"""

import json
import statistics

import torch
import torch.distributed as dist

from mlkit_b200 import tp

CONTEXT = 512
BATCHES = (1, 8)


def step_bytes_per_rank(model: tp.TensorParallelDecoder, batch: int) -> int:
    """Bytes one rank must read per step: its packed weights and head share, and the cached context."""
    c = model.config
    cache = 2 * batch * (c.kv_heads // model.world) * CONTEXT * c.head_dim * 2 * len(model.blocks)
    return model.weight_bytes + cache


def time_steps(captured: tp.CapturedStep, steps: int, warmup: int, world: int, host_io: bool) -> float:
    """Milliseconds per decode step (max over ranks), CUDA events around ``steps`` graph replays."""
    model = captured.model
    batch = captured.tokens.shape[0]
    host_tokens = torch.randint(0, model.config.vocab, (batch,), dtype=torch.int64).pin_memory()
    host_positions = torch.full((batch,), CONTEXT, dtype=torch.int32).pin_memory()
    host_next = torch.empty(batch, dtype=torch.int64).pin_memory()
    captured.tokens.copy_(host_tokens)
    captured.positions.copy_(host_positions)

    def one_step() -> None:
        if host_io:
            captured.tokens.copy_(host_tokens, non_blocking=True)
            captured.positions.copy_(host_positions, non_blocking=True)
        logits = captured.replay()
        if host_io:
            host_next.copy_(logits.argmax(-1), non_blocking=True)

    for _ in range(max(3, warmup)):
        one_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one_step()
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed = torch.tensor([start.elapsed_time(stop) / steps], device=model.device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    return float(elapsed)


def dominant_kernel(model: tp.TensorParallelDecoder, batch: int) -> tuple[float, int]:
    """Average duration (us) and algorithmic bytes of the gate|up matvec launch of this rank, timed over
    the distinct weights of all layers (cold in L2) inside one CUDA graph."""
    width, rows = model.config.hidden, model.blocks[0]["gate_up"].out_rows
    x = torch.randn(batch, width, device=model.device).half()
    out = torch.empty(batch, rows, device=model.device, dtype=torch.float16)
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for block in model.blocks:
            block["gate_up"](x, out)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for block in model.blocks:
                block["gate_up"](x, out)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    samples = []
    for _ in range(5):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop) * 1e3 / len(model.blocks))
    shard = model.blocks[0]["gate_up"]
    return min(samples), shard.nbytes + batch * width * 2 + batch * rows * 2 + 64


def layer_breakdown(world: int, batch: int, device: torch.device, layers: int = 16) -> dict:
    """Per-operator launch time of one decoder layer with the shard shapes of ``world`` ranks, on ONE GPU
    and without communication (the peer reduction is a plain add + norm here): every operator alone over
    ``layers`` distinct layers in one CUDA graph (weights cold in L2), then the chained layer.  Microseconds."""
    from mlkit_b200 import kernels

    c = tp.LLAMA3_70B
    generator = torch.Generator(device=device).manual_seed(1)
    q_heads, kv_heads, mlp = c.q_heads // world, c.kv_heads // world, c.intermediate // world
    shapes = {"qkv": ((q_heads + 2 * kv_heads) * c.head_dim, c.hidden), "o": (c.hidden, q_heads * c.head_dim),
              "gate_up": (2 * mlp, c.hidden), "down": (c.hidden, mlp)}
    shards = [{name: tp.PackedShard.synthetic(n, k, c, device, generator) for name, (n, k) in shapes.items()}
              for _ in range(layers)]
    capacity = CONTEXT + 64
    keys = [torch.randn(batch, kv_heads, capacity, c.head_dim, device=device).half() for _ in range(layers)]
    values = [torch.randn(batch, kv_heads, capacity, c.head_dim, device=device).half() for _ in range(layers)]
    positions = torch.full((batch,), CONTEXT, dtype=torch.int32, device=device)
    residual = torch.randn(batch, c.hidden, device=device).half()
    normed, weight = torch.empty_like(residual), torch.ones(c.hidden, device=device).half()
    out = {name: torch.empty(batch, n, device=device, dtype=torch.float16) for name, (n, _) in shapes.items()}
    attended = torch.randn(batch, q_heads * c.head_dim, device=device).half()

    def timed(launch_all) -> float:
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
        samples = []
        for _ in range(5):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            samples.append(start.elapsed_time(stop) * 1e3 / layers)
        return statistics.median(samples)

    activation = torch.empty(batch, mlp, device=device, dtype=torch.float16)
    operators = {
        "add_rmsnorm": lambda i: kernels.add_rmsnorm(residual, out["down"], weight, normed, 1e-5),
        "qkv": lambda i: shards[i]["qkv"](normed, out["qkv"]),
        "rope_attention": lambda i: kernels.rope_attention_decode(out["qkv"], positions, keys[i], values[i], attended,
                                                                  q_heads=q_heads, kv_heads=kv_heads,
                                                                  head_dim=c.head_dim, theta=c.rope_theta),
        "o": lambda i: shards[i]["o"](attended, out["o"]),
        "gate_up": lambda i: shards[i]["gate_up"](normed, out["gate_up"]),
        "silu_mul": lambda i: kernels.silu_mul(out["gate_up"], activation),
        "down": lambda i: shards[i]["down"](activation, out["down"]),
    }
    table = {}
    for name, operator in operators.items():
        table[name] = round(timed(lambda: [operator(i) for i in range(layers)]), 2)

    def layer(i: int) -> None:
        operators["add_rmsnorm"](i)
        operators["qkv"](i)
        operators["rope_attention"](i)
        operators["o"](i)
        kernels.add_rmsnorm(residual, out["o"], weight, normed, 1e-5)
        operators["gate_up"](i)
        operators["silu_mul"](i)
        operators["down"](i)

    table["layer_chained"] = round(timed(lambda: [layer(i) for i in range(layers)]), 2)
    table["sum_of_parts"] = round(sum(table[name] for name in operators) + table["add_rmsnorm"], 2)
    weights = sum(shard.nbytes for shard in shards[0].values())
    table["weight_mb_per_layer"] = round(weights / 1e6, 2)
    return table


def measure(rank: int, world: int, device: torch.device, steps: int, warmup: int, layers: int | None = None) -> dict:
    """Build the synthetic model on this rank and time decode for every batch in ``BATCHES``."""
    group = dist.group.WORLD if world > 1 else None
    model = tp.TensorParallelDecoder.synthetic(tp.LLAMA3_70B, rank=rank, world=world, device=device, seed=1,
                                               layers=layers, max_batch=max(BATCHES), capacity=CONTEXT + 64,
                                               group=group)
    model.fill_cache(CONTEXT)
    results = {"batches": {}, "launches_per_step": len(model.blocks) * 8 + 3,
               "collectives_per_step": 0 if world == 1 else 2 * len(model.blocks) + 1, "collective": "none"}
    if world > 1:
        # the library all-reduce first, as the yardstick; then the peer-memory reduction, which is the product path
        captured = model.capture(1)
        results["nccl_ms_per_step_batch1"] = time_steps(captured, steps, warmup, world, host_io=False)
        del captured
        results["collective"] = "nccl all-reduce"
        try:
            model.enable_peer_exchange()
            results["collective"] = "peer-memory all-reduce fused with add + norm, one kernel (mkb_peer_reduce_add_rmsnorm); logits by nccl all-gather"
            probe_tokens = torch.zeros(1, dtype=torch.int64, device=device)
            probe_positions = torch.full((1,), CONTEXT, dtype=torch.int32, device=device)
            model.step(probe_tokens, probe_positions)
            torch.cuda.synchronize()
            expired = torch.tensor([model.exchange.status()], device=device)
            dist.all_reduce(expired, op=dist.ReduceOp.MAX)
            if int(expired) != 0:   # a wait ran out on some rank: every rank goes back to the library collective
                model.exchange = None
                results["collective"] = "nccl all-reduce (a wait of the peer exchange expired)"
        except Exception as error:  # peer mapping refused on this node: stay on the library collective
            results["collective"] = f"nccl all-reduce (peer exchange unavailable: {error})"
    for batch in BATCHES:
        captured = model.capture(batch)
        resident = time_steps(captured, steps, warmup, world, host_io=False)
        e2e = time_steps(captured, steps, warmup, world, host_io=True)
        bytes_rank = step_bytes_per_rank(model, batch)
        results["batches"][batch] = {
            "ms_per_step": resident, "tokens_per_s": batch / resident * 1e3, "e2e_ms_per_step": e2e,
            "e2e_tokens_per_s": batch / e2e * 1e3, "bytes_per_rank": bytes_rank,
            "per_gpu_gbps": bytes_rank / resident / 1e6, "aggregate_gbps": world * bytes_rank / resident / 1e6,
        }
        del captured
    if model.exchange is not None:
        results["peer_status"] = model.exchange.status()
    kernel_us, kernel_bytes = dominant_kernel(model, 1)
    results["kernel"] = {"us": kernel_us, "bytes": kernel_bytes,
                         "shape": f"{model.config.hidden}->{model.blocks[0]['gate_up'].out_rows}"}
    del model
    torch.cuda.empty_cache()
    return results


def run(args, rank: int, world: int, device: torch.device, peak_info: tuple[float, str]) -> None:
    """The N > 1 arm of ``bench.py``: rank 0 prints the JSON line."""
    from bench import METRIC, ClockSampler

    peak, peak_kind = peak_info
    with ClockSampler(device.index) as sampler:
        results = measure(rank, world, device, args.steps, args.warmup)
    if rank != 0:
        return
    one, eight = results["batches"][1], results["batches"][8]
    achieved = results["kernel"]["bytes"] / results["kernel"]["us"] / 1e3
    print(json.dumps({
        "metric": METRIC, "value": one["aggregate_gbps"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": one["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"llama3-70b-shaped int4 g128 tensor-parallel decode, tp{world}, batch 1, ctx {CONTEXT}, "
                               "one CUDA graph per step",
                   "l2": "inputs larger than L2: every step streams all packed weights of the rank",
                   "pct_of_8tbs_per_gpu": round(one["per_gpu_gbps"] / 8000 * 100, 2)},
        "e2e": {"value": world * one["bytes_per_rank"] / one["e2e_ms_per_step"] / 1e6, "unit": "GB/s",
                "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 8},
        "gpu_launches": results["launches_per_step"] * args.steps,
        "clocks": sampler.summary,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind,
                     "kernel": f"the matvec kernel AUTO takes (gemv_stream_kernel) on the gate|up shard {results['kernel']['shape']}, M=1, rank 0",
                     "bytes_per_launch": results["kernel"]["bytes"], "us_per_launch": results["kernel"]["us"]},
        "decode": {
            "tokens_per_s": {"batch1": one["tokens_per_s"], "batch8": eight["tokens_per_s"]},
            "e2e_tokens_per_s": {"batch1": one["e2e_tokens_per_s"], "batch8": eight["e2e_tokens_per_s"]},
            "per_gpu_roofline_frac": {"batch1": one["per_gpu_gbps"] / peak, "batch8": eight["per_gpu_gbps"] / peak},
            "per_gpu_gbps": {"batch1": one["per_gpu_gbps"], "batch8": eight["per_gpu_gbps"]},
            "collectives_per_step": results["collectives_per_step"],
            "collective": results["collective"],
            "nccl_ms_per_step_batch1": results.get("nccl_ms_per_step_batch1"),
            "peer_status": results.get("peer_status"),
        },
    }))
