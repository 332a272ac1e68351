"""Tensor-parallel decode of a Llama-shaped model whose block linears are packed scalar codes.

This component has no counterpart in the reference (which is single-device and leaves the decoder
block to ``transformers``); it is what serves the packed matvec on one 8-GPU box:

* one process per GPU, ``torch.distributed`` (NCCL) for the exchange;
* column parallel (shard the output rows): q, k, v, gate, up, and the fp16 output head by vocabulary.
  A rank's rows of q, k and v are stored as one packed matrix, likewise gate and up, so each pair of
  sibling projections is one matvec launch;
* row parallel (shard the reduction axis): o and down.  Each rank multiplies its slice of the
  activations and the partial results are summed by one all-reduce per projection, two per layer;
* between the matvecs: fused residual-add + RMS norm, rotary embedding + KV-cache append,
  single-token grouped-query attention, SiLU * up (``csrc/decode_ops.cu``);
* a decode step for a fixed batch is captured once in a CUDA graph and replayed.

Sharding happens when the model is built; nothing sharded is ever written to a checkpoint.
"""

import math
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor

from mlkit_b200 import _native, kernels
from mlkit_b200.quantization import Q, pack


@dataclass(frozen=True)
class DecoderConfig:
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float = 500000.0
    eps: float = 1e-5
    bits: int = 4
    group: int = 128

    def validate(self, world: int) -> None:
        if self.q_heads % world or self.kv_heads % world or self.intermediate % world or self.vocab % world:
            raise ValueError(f"heads, MLP width and vocabulary must divide by the world size {world}")
        codes_per_word = 8 // math.gcd(self.bits, 8)
        for name, width in (("o", self.q_heads * self.head_dim // world), ("down", self.intermediate // world)):
            if width % math.lcm(self.group, codes_per_word):
                raise ValueError(f"the {name} shard of {width} columns splits a scale group or packing word")


LLAMA3_70B = DecoderConfig(layers=80, hidden=8192, q_heads=64, kv_heads=8, head_dim=128, intermediate=28672,
                           vocab=128256)
LLAMA3_8B = DecoderConfig(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, intermediate=14336,
                          vocab=128256)


# ---------------------------------------------------------------------------------- sharding


def best_keys(all_keys: Tensor) -> Tensor:
    """The unsigned maximum over axis 0 of ``argmax_keys`` words kept in int64 storage: flipping the top
    bit turns unsigned order into signed order and back."""
    top = -(1 << 63)
    return (all_keys ^ top).amax(0) ^ top


def rows_of(rank: int, world: int, total: int) -> slice:
    """Rows ``[rank * total / world, (rank + 1) * total / world)`` of a column-parallel projection."""
    share = total // world
    return slice(rank * share, (rank + 1) * share)


def shard_rows(packed: Tensor, scales: Tensor, rows: slice, width: int, bits: int) -> tuple[Tensor, Tensor]:
    """Column-parallel shard: a contiguous run of output rows (contiguous bytes of the stream)."""
    row_bytes = width * bits // 8
    return (packed.view(-1, row_bytes)[rows].reshape(-1).contiguous(), scales[rows].contiguous())


def shard_columns(packed: Tensor, scales: Tensor, rank: int, world: int, width: int, bits: int,
                  group: int) -> tuple[Tensor, Tensor]:
    """Row-parallel shard: columns ``[rank * width / world, ...)`` of every row, compacted."""
    share = width // world
    byte_share, group_share = share * bits // 8, share // group
    matrix = packed.view(-1, width * bits // 8)
    return (matrix[:, rank * byte_share:(rank + 1) * byte_share].reshape(-1).contiguous(),
            scales[:, rank * group_share:(rank + 1) * group_share].contiguous())


class PackedShard:
    """The packed weight one rank holds for one (possibly fused) projection, with its bound launch."""

    def __init__(self, packed: Tensor, scales: Tensor, values: Tensor, *, out_rows: int, width: int, bits: int,
                 group: int) -> None:
        self.packed, self.scales, self.values = packed, scales, values
        self.out_rows, self.width, self.bits, self.group = out_rows, width, bits, group
        integer, low = kernels.integer_grid_of(values)
        self.plan = kernels.MatvecPlan(packed, scales, values, None, None, outputs=out_rows, width=width,
                                       group=group, bits=bits, dtype=torch.float16, integer_grid=integer,
                                       grid_minimum=low)

    def __call__(self, x: Tensor, out: Tensor) -> Tensor:
        return self.plan(x, out)

    @property
    def nbytes(self) -> int:
        return self.packed.numel() + self.scales.numel() * 2

    @staticmethod
    def synthetic(out_rows: int, width: int, config: DecoderConfig, device: torch.device,
                  generator: torch.Generator) -> "PackedShard":
        """Random codes and scales of realistic size: throughput does not depend on the values."""
        packed = torch.randint(0, 256, (out_rows * width * config.bits // 8,), dtype=torch.uint8, device=device,
                               generator=generator)
        scales = (torch.rand(out_rows, width // config.group, device=device, generator=generator) * 0.003
                  + 0.003).half()
        low = -(2 ** (config.bits - 1))
        values = torch.arange(low, -low, dtype=torch.float32, device=device)
        return PackedShard(packed, scales, values, out_rows=out_rows, width=width, bits=config.bits,
                           group=config.group)


def _packed_parts(quantized: Q, device: torch.device) -> tuple[Tensor, Tensor, Tensor, int, int]:
    bits, group = int(quantized.metadata["code_bits"]), int(quantized.params["group"])
    if quantized.params.get("zero") is not None:
        raise ValueError("tensor-parallel decode covers symmetric formats")
    return (quantized.packed_stream(bits).to(device), quantized.params["scales"].to(device).half(),
            quantized.params["values"].to(device).float().contiguous(), bits, group)


def shard_block(block: dict[str, Q], config: DecoderConfig, rank: int, world: int,
                device: torch.device) -> dict[str, PackedShard]:
    """Shard the seven quantised projections of one block (keys q, k, v, o, gate, up, down)."""
    config.validate(world)
    parts = {name: _packed_parts(q, device) for name, q in block.items()}
    bits, group = parts["q"][3], parts["q"][4]
    hidden, inter = config.hidden, config.intermediate

    def fused_rows(names: list[str], totals: list[int], width: int) -> PackedShard:
        packed, scales = zip(*(shard_rows(parts[n][0], parts[n][1], rows_of(rank, world, total), width, bits)
                               for n, total in zip(names, totals)))
        rows = sum(total // world for total in totals)
        return PackedShard(torch.cat(packed), torch.cat(scales), parts[names[0]][2], out_rows=rows, width=width,
                           bits=bits, group=group)

    def columns(name: str, out_rows: int, width: int) -> PackedShard:
        packed, scales = shard_columns(parts[name][0], parts[name][1], rank, world, width, bits, group)
        return PackedShard(packed, scales, parts[name][2], out_rows=out_rows, width=width // world, bits=bits,
                           group=group)

    q_rows, kv_rows = config.q_heads * config.head_dim, config.kv_heads * config.head_dim
    return {
        "qkv": fused_rows(["q", "k", "v"], [q_rows, kv_rows, kv_rows], hidden),
        "o": columns("o", hidden, q_rows),
        "gate_up": fused_rows(["gate", "up"], [inter, inter], hidden),
        "down": columns("down", hidden, inter),
    }


def synthetic_block(config: DecoderConfig, world: int, device: torch.device,
                    generator: torch.Generator) -> dict[str, PackedShard]:
    """One rank's shards of a block with random codes (shapes exactly as ``shard_block`` makes them)."""
    config.validate(world)
    q_rows, kv_rows = config.q_heads * config.head_dim // world, config.kv_heads * config.head_dim // world
    make = lambda rows, width: PackedShard.synthetic(rows, width, config, device, generator)
    return {"qkv": make(q_rows + 2 * kv_rows, config.hidden), "o": make(config.hidden, q_rows),
            "gate_up": make(2 * config.intermediate // world, config.hidden),
            "down": make(config.hidden, config.intermediate // world)}


# ----------------------------------------------------------------------------------- peer exchange


class PeerExchange:
    """The exchange buffers of the one-shot peer-memory all-reduce (``mkb_peer_*``).

    Every rank allocates one buffer, the ranks swap its 64-byte handle through the process group, and
    each maps the others' buffers; ``reduce_add_rmsnorm`` then pushes a partial into all of them, waits for
    the other ranks' partials and consumes the sum, in one kernel.  Ranks must share a node (NVLink/NVSwitch peer access).
    """

    def __init__(self, *, rank: int, world: int, rows: int, width: int, device: torch.device,
                 group: "dist.ProcessGroup | None" = None) -> None:
        import ctypes

        self.rank, self.world, self.rows, self.width, self.device = rank, world, rows, width, device
        self.own: int | None = None
        self.opened: list[int] = []
        library = _native.library()

        def agreed(problem: str | None, stage: str) -> None:
            """Every rank learns whether every rank got through ``stage``: no rank may be left in a collective."""
            flag = torch.tensor([0 if problem is None else 1], dtype=torch.int32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
            if int(flag) != 0:
                self.close()
                raise RuntimeError(f"peer exchange: {stage} failed on " +
                                   ("this rank: " + problem if problem is not None else "another rank"))

        with torch.cuda.device(device):
            problem, handle = None, ctypes.create_string_buffer(64)
            try:
                size = library.mkb_peer_buffer_bytes(rows, width, world)
                if size <= 0:
                    raise ValueError(f"no layout for rows={rows} width={width} world={world}")
                own = ctypes.c_void_p()
                _native.check(library.mkb_peer_alloc(size, ctypes.byref(own)), "peer_alloc")
                self.own = own.value
                _native.check(library.mkb_peer_export(self.own, handle), "peer_export")
                parts = int(os.environ.get("MLKIT_B200_PEER_SPLIT", "0"))   # CTAs per row; 0: from the world size
                if parts:
                    _native.check(library.mkb_peer_set_split(self.own, parts), "peer_set_split")
            except Exception as error:  # reported to all ranks below
                problem = repr(error)
            agreed(problem, "allocating and exporting the buffer")
            handles: list = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            pointers = []
            try:
                for peer, raw in enumerate(handles):
                    if peer == rank:
                        pointers.append(self.own)
                        continue
                    mapped = ctypes.c_void_p()
                    _native.check(library.mkb_peer_open(ctypes.create_string_buffer(raw, 64), ctypes.byref(mapped)),
                                  "peer_open")
                    self.opened.append(mapped.value)
                    pointers.append(mapped.value)
            except Exception as error:
                problem = repr(error)
            agreed(problem, "mapping the other ranks' buffers")
            self.peers = torch.tensor(pointers, dtype=torch.int64, device=device)
        dist.barrier(group=group)

    def reduce_add_rmsnorm(self, partial: Tensor, residual: Tensor, weight: Tensor, normed: Tensor, eps: float,
                           reduced: Tensor | None = None) -> None:
        """All-reduce ``partial`` over the ranks, ``residual += sum``, ``normed = rms_norm(residual) * weight``:
        one kernel launch."""
        status = _native.library().mkb_peer_reduce_add_rmsnorm(
            partial.data_ptr(), self.peers.data_ptr(), self.own, residual.data_ptr(), weight.data_ptr(),
            normed.data_ptr(), None if reduced is None else reduced.data_ptr(), partial.shape[0], self.width,
            self.rows, self.world, self.rank, float(eps), torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(status, "peer_reduce_add_rmsnorm")

    def status(self) -> int:
        """Non-zero when a bounded wait of an earlier reduction expired."""
        import ctypes

        value = ctypes.c_int(0)
        _native.check(_native.library().mkb_peer_status(self.own, ctypes.byref(value)), "peer_status")
        return value.value

    def set_poll_limit(self, polls: int) -> None:
        """How long a reduction waits for the other ranks (polls of a flag) before it gives up."""
        _native.check(_native.library().mkb_peer_set_poll_limit(self.own, int(polls)), "peer_set_poll_limit")

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's.  Call it after the process group has been
        destroyed (tearing the library communicator down after these mappings were closed was seen to
        block), or leave it to process exit."""
        library = _native.library()
        for mapped in self.opened:
            library.mkb_peer_close(mapped)
        self.opened = []
        if self.own:
            library.mkb_peer_free(self.own)
            self.own = None


# ----------------------------------------------------------------------------------- the model


class TensorParallelDecoder:
    """One rank of a tensor-parallel Llama-shaped decoder with packed block linears."""

    def __init__(self, config: DecoderConfig, *, rank: int = 0, world: int = 1, device: torch.device | str = "cuda",
                 max_batch: int = 8, capacity: int = 1024, group: "dist.ProcessGroup | None" = None) -> None:
        config.validate(world)
        self.config, self.rank, self.world, self.group = config, rank, world, group
        self.device = torch.device(device)
        self.max_batch, self.capacity = max_batch, capacity
        self.blocks: list[dict[str, PackedShard]] = []
        self.norms: list[tuple[Tensor, Tensor]] = []
        self.embedding: Tensor | None = None
        self.final_norm: Tensor | None = None
        self.head: Tensor | None = None
        self.packed_head: PackedShard | None = None
        self.k_cache: list[Tensor] = []
        self.v_cache: list[Tensor] = []
        self._work: dict[int, dict[str, Tensor]] = {}
        self.exchange: PeerExchange | None = None

    def enable_peer_exchange(self) -> None:
        """Replace the library all-reduce after o and down by the one-shot peer-memory reduction."""
        if self.world > 1 and self.exchange is None:
            self.exchange = PeerExchange(rank=self.rank, world=self.world, rows=self.max_batch,
                                         width=self.config.hidden, device=self.device, group=self.group)

    # -- construction --
    def add_block(self, shards: dict[str, PackedShard], attention_norm: Tensor, mlp_norm: Tensor) -> None:
        config, local_kv = self.config, self.config.kv_heads // self.world
        self.blocks.append(shards)
        self.norms.append((attention_norm.to(self.device).half().contiguous(),
                           mlp_norm.to(self.device).half().contiguous()))
        shape = (self.max_batch, local_kv, self.capacity, config.head_dim)
        self.k_cache.append(torch.zeros(shape, dtype=torch.float16, device=self.device))
        self.v_cache.append(torch.zeros(shape, dtype=torch.float16, device=self.device))

    def set_head(self, embedding: Tensor, final_norm: Tensor, head: "Tensor | Q") -> None:
        """``embedding`` [vocab, hidden] replicated; ``head`` [vocab, hidden] is sharded by rows here.  A
        quantised head (a ``Q`` of a scalar codec, as head-quantised checkpoints carry) stays packed:
        this rank's rows of its code stream feed the packed matvec
        (``src/mlkit/inference/packed_linear.py:248-287`` runs such a head through ``PackedLinear``)."""
        self.embedding = embedding.to(self.device).half().contiguous()
        self.final_norm = final_norm.to(self.device).half().contiguous()
        if isinstance(head, Q):
            packed, scales, values, bits, group = _packed_parts(head, self.device)
            vocab, width = head.codes.shape
            rows = rows_of(self.rank, self.world, vocab)
            shard_packed, shard_scales = shard_rows(packed, scales, rows, width, bits)
            self.packed_head = PackedShard(shard_packed, shard_scales, values, out_rows=vocab // self.world, width=width,
                                           bits=bits, group=group)
            self.head = None
        else:
            self.head = head[rows_of(self.rank, self.world, head.shape[0])].to(self.device).half().contiguous()

    @staticmethod
    def synthetic(config: DecoderConfig, *, rank: int = 0, world: int = 1, device: torch.device | str = "cuda",
                  seed: int = 0, layers: int | None = None, with_head: bool = True, **options) -> "TensorParallelDecoder":
        model = TensorParallelDecoder(config, rank=rank, world=world, device=device, **options)
        generator = torch.Generator(device=model.device).manual_seed(seed * 1000 + rank)
        ones = torch.ones(config.hidden, dtype=torch.float16, device=model.device)
        for _ in range(config.layers if layers is None else layers):
            model.add_block(synthetic_block(config, world, model.device, generator), ones, ones)
        if with_head:
            shared = torch.Generator(device=model.device).manual_seed(seed)  # same on every rank
            embedding = (torch.randn(config.vocab, config.hidden, device=model.device, generator=shared) * 0.5).half()
            model.embedding, model.final_norm = embedding, ones
            share = config.vocab // world
            model.head = (torch.randn(share, config.hidden, device=model.device, generator=generator) * 0.02).half()
        return model

    def fill_cache(self, length: int, seed: int = 0) -> None:
        """A synthetic context: random keys and values for positions ``0..length-1`` of every sequence."""
        generator = torch.Generator(device=self.device).manual_seed(seed + 17 + self.rank)
        for cache in (*self.k_cache, *self.v_cache):
            cache[:, :, :length].copy_(torch.randn(cache[:, :, :length].shape, device=self.device,
                                                   generator=generator).half())

    @property
    def weight_bytes(self) -> int:
        """Bytes this rank streams per decode step: packed codes, scales and its share of the head."""
        total = sum(shard.nbytes for block in self.blocks for shard in block.values())
        if self.packed_head is not None:
            total += self.packed_head.nbytes
        return total + (0 if self.head is None else self.head.numel() * 2)

    # -- one decode step --
    def _buffers(self, batch: int) -> dict[str, Tensor]:
        work = self._work.get(batch)
        if work is None:
            c, w = self.config, self.world
            local_q, local_kv = c.q_heads // w, c.kv_heads // w
            half = lambda *shape: torch.empty(shape, dtype=torch.float16, device=self.device)
            work = self._work[batch] = {
                "residual": half(batch, c.hidden), "normed": half(batch, c.hidden),
                "qkv": half(batch, (local_q + 2 * local_kv) * c.head_dim), "attention": half(batch, local_q * c.head_dim),
                "o": half(batch, c.hidden), "gate_up": half(batch, 2 * c.intermediate // w),
                "act": half(batch, c.intermediate // w), "down": half(batch, c.hidden),
                "logits": half(batch, c.vocab // w),
                "keys": torch.empty(batch, dtype=torch.int64, device=self.device),
                "all_keys": torch.empty(w, batch, dtype=torch.int64, device=self.device),
                "gathered": half(w, batch, c.vocab // w),
            }
        return work

    def _all_reduce(self, tensor: Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(tensor, group=self.group)

    def step(self, tokens: Tensor, positions: Tensor, greedy: bool = False) -> Tensor:
        """Decode one token per sequence: ``tokens`` int64 [batch], ``positions`` int32 [batch] (the
        cache slot each new token takes).  Returns this step's logits [batch, vocab] in fp16, or, with
        ``greedy``, the next tokens int64 [batch]: every rank picks the best token of its vocabulary
        shard and the ranks exchange 8 bytes per sequence instead of their logits."""
        c, w = self.config, self.world
        batch = tokens.shape[0]
        if batch > self.max_batch:
            raise ValueError(f"batch {batch} exceeds max_batch {self.max_batch}")
        if not torch.cuda.is_current_stream_capturing():
            # an eager step checks its cache slots on the host (one small synchronisation).  A captured
            # step cannot: its caller keeps positions below the capacity; the kernels clamp a position
            # that is not and report it through kernels.decode_status()
            low, high = int(positions.min()), int(positions.max())
            if low < 0 or high >= self.capacity:
                raise ValueError(f"positions {low}..{high} leave the cache of {self.capacity} slots")
        work = self._buffers(batch)
        local_q, local_kv = c.q_heads // w, c.kv_heads // w
        residual, normed = work["residual"], work["normed"]
        torch.index_select(self.embedding, 0, tokens, out=residual)
        delta = None
        exchange = self.exchange
        for index, block in enumerate(self.blocks):
            attention_norm, mlp_norm = self.norms[index]
            k_cache, v_cache = self.k_cache[index], self.v_cache[index]
            if exchange is not None and delta is not None:
                exchange.reduce_add_rmsnorm(delta, residual, attention_norm, normed, c.eps)   # the down-projection shards
            else:
                kernels.add_rmsnorm(residual, delta, attention_norm, normed, c.eps)
            block["qkv"](normed, work["qkv"])
            if local_q <= 8 * local_kv and c.head_dim == 128:   # rotary embedding, cache append and attention in one launch
                kernels.rope_attention_decode(work["qkv"], positions, k_cache, v_cache, work["attention"],
                                              q_heads=local_q, kv_heads=local_kv, head_dim=c.head_dim,
                                              theta=c.rope_theta)
            else:
                kernels.rope_append(work["qkv"], positions, k_cache, v_cache, q_heads=local_q, kv_heads=local_kv,
                                    head_dim=c.head_dim, theta=c.rope_theta)
                kernels.attention_decode(work["qkv"], positions, k_cache, v_cache, work["attention"],
                                         q_heads=local_q, kv_heads=local_kv, head_dim=c.head_dim)
            block["o"](work["attention"], work["o"])
            if exchange is not None:
                exchange.reduce_add_rmsnorm(work["o"], residual, mlp_norm, normed, c.eps)
            else:
                self._all_reduce(work["o"])
                kernels.add_rmsnorm(residual, work["o"], mlp_norm, normed, c.eps)
            block["gate_up"](normed, work["gate_up"])
            # SwiGLU as its own 1.5 us launch: formed on load inside the down projection (MKB_GEMV_GATED) every
            # CTA would redo the activation of its K slice, which measured 3 us slower per layer at every shard size
            kernels.silu_mul(work["gate_up"], work["act"])
            block["down"](work["act"], work["down"])
            if exchange is None:
                self._all_reduce(work["down"])
            delta = work["down"]
        if exchange is not None and delta is not None:
            exchange.reduce_add_rmsnorm(delta, residual, self.final_norm, normed, c.eps)
        else:
            kernels.add_rmsnorm(residual, delta, self.final_norm, normed, c.eps)
        if self.packed_head is not None:   # a head-quantised checkpoint: the head is one more packed matvec
            self.packed_head(normed, work["logits"])
        else:
            torch.matmul(normed, self.head.t(), out=work["logits"])
        if greedy:
            share = work["logits"].shape[1]
            keys = kernels.argmax_keys(work["logits"], work["keys"], offset=self.rank * share)
            if w > 1:
                dist.all_gather_into_tensor(work["all_keys"], keys, group=self.group)
                keys = best_keys(work["all_keys"])
            return kernels.tokens_of_keys(keys)
        if w == 1:
            return work["logits"]
        dist.all_gather_into_tensor(work["gathered"], work["logits"], group=self.group)
        return work["gathered"].permute(1, 0, 2).reshape(batch, c.vocab)

    def capture(self, batch: int) -> "CapturedStep":
        return CapturedStep(self, batch)


class CapturedStep:
    """A decode step for a fixed batch as a CUDA graph: write ``tokens`` / ``positions``, ``replay()``."""

    def __init__(self, model: TensorParallelDecoder, batch: int) -> None:
        self.model = model
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=model.device)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=model.device)
        side = torch.cuda.Stream(device=model.device)
        side.wait_stream(torch.cuda.current_stream(model.device))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm up kernels, NCCL channels and the allocator before capturing
                model.step(self.tokens, self.positions)
            torch.cuda.synchronize(model.device)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.logits = model.step(self.tokens, self.positions)
        torch.cuda.current_stream(model.device).wait_stream(side)
        torch.cuda.synchronize(model.device)

    def replay(self) -> Tensor:
        self.graph.replay()
        return self.logits
