"""GPU tests of the decode operators and the tensor-parallel decoder.

The operators are compared with fp32 torch restatements of the same formulas.  The decoder is compared,
on one GPU, with a dense fp32 torch decoder built from the oracle's reconstruction of the same packed
weights; shards for 2, 4 and 8 ranks are summed on one GPU against the unsharded projection; the
NCCL path runs when two GPUs are visible.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import mlkit_b200 as mk
from mlkit_b200 import kernels, tp
from oracle import matvec

pytestmark = pytest.mark.gpu
SMALL = tp.DecoderConfig(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, intermediate=512, vocab=512)


def rel(a, b):
    return matvec.relative_l2(a.float().cpu().numpy(), b.float().cpu().numpy())


def test_add_rmsnorm_matches_torch():
    torch.manual_seed(0)
    for rows, hidden in ((1, 256), (8, 8192), (3, 4096)):
        residual = torch.randn(rows, hidden, device="cuda").half()
        delta = torch.randn(rows, hidden, device="cuda").half()
        weight = (torch.rand(hidden, device="cuda") + 0.5).half()
        expected_residual = (residual.float() + delta.float()).half()
        variance = expected_residual.float().pow(2).mean(-1, keepdim=True)
        expected = (expected_residual.float() * torch.rsqrt(variance + 1e-5)).half().float() * weight.float()
        normed = torch.empty_like(residual)
        kernels.add_rmsnorm(residual, delta, weight, normed, 1e-5)
        assert torch.equal(residual, expected_residual)
        assert rel(normed, expected) < 1e-3
        first = torch.empty_like(residual)
        kernels.add_rmsnorm(residual, None, weight, first, 1e-5)
        assert torch.equal(first, normed) and torch.equal(residual, expected_residual)


def rope_reference(vec, position, theta):
    dim = vec.shape[-1]
    freq = theta ** (-torch.arange(0, dim, 2, device=vec.device).float() / dim)
    angle = position * freq
    a, b = vec[..., : dim // 2].float(), vec[..., dim // 2:].float()
    return torch.cat((a * angle.cos() - b * angle.sin(), b * angle.cos() + a * angle.sin()), -1)


def test_rope_append_and_attention_match_torch():
    torch.manual_seed(1)
    batch, q_heads, kv_heads, dim, capacity = 3, 8, 2, 128, 96
    qkv = torch.randn(batch, (q_heads + 2 * kv_heads) * dim, device="cuda").half()
    original = qkv.clone()
    positions = torch.tensor([0, 17, 95], dtype=torch.int32, device="cuda")
    k_cache = torch.randn(batch, kv_heads, capacity, dim, device="cuda").half()
    v_cache = torch.randn(batch, kv_heads, capacity, dim, device="cuda").half()
    kernels.rope_append(qkv, positions, k_cache, v_cache, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim, theta=5e5)
    heads = original.view(batch, q_heads + 2 * kv_heads, dim)
    got = qkv.view(batch, q_heads + 2 * kv_heads, dim)
    for m in range(batch):
        p = int(positions[m])
        expected = rope_reference(heads[m, : q_heads + kv_heads], p, 5e5)
        assert rel(got[m, : q_heads + kv_heads], expected) < 1e-3
        assert torch.equal(got[m, q_heads + kv_heads:], heads[m, q_heads + kv_heads:])
        assert torch.equal(k_cache[m, :, p], got[m, q_heads:q_heads + kv_heads])
        assert torch.equal(v_cache[m, :, p], got[m, q_heads + kv_heads:])
    out = torch.empty(batch, q_heads * dim, device="cuda", dtype=torch.float16)
    kernels.attention_decode(qkv, positions, k_cache, v_cache, out, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim)
    for m in range(batch):
        length = int(positions[m]) + 1
        q = got[m, :q_heads].float()
        keys = k_cache[m, :, :length].float().repeat_interleave(q_heads // kv_heads, 0)
        values = v_cache[m, :, :length].float().repeat_interleave(q_heads // kv_heads, 0)
        weights = torch.softmax(torch.einsum("hd,hpd->hp", q, keys) / dim ** 0.5, -1)
        expected = torch.einsum("hp,hpd->hd", weights, values).reshape(-1)
        assert rel(out[m], expected) < 2e-3


def test_fused_rope_attention_equals_the_two_kernels():
    """rope_attention_decode: same cache contents and, up to the fp16 rounding of the rotated query,
    the same attention output as rope_append followed by attention_decode."""
    torch.manual_seed(4)
    for q_heads, kv_heads in ((8, 2), (8, 1), (16, 2)):
        batch, dim, capacity = 3, 128, 96
        qkv = torch.randn(batch, (q_heads + 2 * kv_heads) * dim, device="cuda").half()
        positions = torch.tensor([0, 40, 95], dtype=torch.int32, device="cuda")
        caches = [torch.randn(batch, kv_heads, capacity, dim, device="cuda").half() for _ in range(2)]
        k_two, v_two, k_one, v_one = caches[0].clone(), caches[1].clone(), caches[0].clone(), caches[1].clone()
        rotated = qkv.clone()
        kernels.rope_append(rotated, positions, k_two, v_two, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim, theta=5e5)
        expected = torch.empty(batch, q_heads * dim, device="cuda", dtype=torch.float16)
        kernels.attention_decode(rotated, positions, k_two, v_two, expected, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim)
        untouched = qkv.clone()
        got = torch.empty_like(expected)
        kernels.rope_attention_decode(qkv, positions, k_one, v_one, got, q_heads=q_heads, kv_heads=kv_heads,
                                      head_dim=dim, theta=5e5)
        assert torch.equal(qkv, untouched)
        assert torch.equal(v_one, v_two)
        assert rel(k_one, k_two) < 1e-3
        assert rel(got, expected) < 2e-3


def test_silu_mul_matches_torch():
    torch.manual_seed(2)
    gate_up = torch.randn(5, 2 * 1024, device="cuda").half()
    out = torch.empty(5, 1024, device="cuda", dtype=torch.float16)
    kernels.silu_mul(gate_up, out)
    expected = F.silu(gate_up[:, :1024].float()).half().float() * gate_up[:, 1024:].float()
    assert rel(out, expected) < 1e-3


def quantised_block(config, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    fmt = mk.int(config.bits, group=config.group)
    shapes = {"q": (config.q_heads * config.head_dim, config.hidden), "k": (config.kv_heads * config.head_dim, config.hidden),
              "v": (config.kv_heads * config.head_dim, config.hidden), "o": (config.hidden, config.q_heads * config.head_dim),
              "gate": (config.intermediate, config.hidden), "up": (config.intermediate, config.hidden),
              "down": (config.hidden, config.intermediate)}
    return {name: fmt((torch.randn(shape, device="cuda", generator=generator) * 0.05).half().float())
            for name, shape in shapes.items()}


def dense_reference_step(config, blocks, embedding, final_norm, head, tokens, positions, k_caches, v_caches):
    """fp32 torch decoder over the dense reconstructions; caches are [batch, kv, capacity, dim] fp32."""
    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + config.eps) * w

    x = embedding.float()[tokens]
    batch = tokens.shape[0]
    for index, block in enumerate(blocks):
        w = {name: q.w.half().float() for name, q in block.items()}
        h = norm(x, 1.0)
        q = (h @ w["q"].T).view(batch, config.q_heads, config.head_dim)
        k = (h @ w["k"].T).view(batch, config.kv_heads, config.head_dim)
        v = (h @ w["v"].T).view(batch, config.kv_heads, config.head_dim)
        outs = []
        for m in range(batch):
            p = int(positions[m])
            qm, km = rope_reference(q[m], p, config.rope_theta), rope_reference(k[m], p, config.rope_theta)
            k_caches[index][m, :, p], v_caches[index][m, :, p] = km, v[m]
            repeat = config.q_heads // config.kv_heads
            keys = k_caches[index][m, :, : p + 1].repeat_interleave(repeat, 0)
            values = v_caches[index][m, :, : p + 1].repeat_interleave(repeat, 0)
            weights = torch.softmax(torch.einsum("hd,hpd->hp", qm, keys) / config.head_dim ** 0.5, -1)
            outs.append(torch.einsum("hp,hpd->hd", weights, values).reshape(-1))
        x = x + torch.stack(outs) @ w["o"].T
        h = norm(x, 1.0)
        x = x + (F.silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T
    return norm(x, final_norm.float()) @ head.float().T


def build_model(config, blocks, embedding, final_norm, head, rank=0, world=1, **options):
    model = tp.TensorParallelDecoder(config, rank=rank, world=world, device="cuda", max_batch=4, capacity=64, **options)
    ones = torch.ones(config.hidden, device="cuda")
    for block in blocks:
        model.add_block(tp.shard_block(block, config, rank, world, torch.device("cuda")), ones, ones)
    model.set_head(embedding, final_norm, head)
    return model


def test_decoder_matches_dense_reference_and_graph_replay():
    torch.manual_seed(3)
    config = SMALL
    blocks = [quantised_block(config, 10 + i) for i in range(config.layers)]
    embedding = torch.randn(config.vocab, config.hidden, device="cuda").half()
    final_norm = (torch.rand(config.hidden, device="cuda") + 0.5).half()
    head = (torch.randn(config.vocab, config.hidden, device="cuda") * 0.05).half()
    model = build_model(config, blocks, embedding, final_norm, head)
    model.fill_cache(5, seed=1)
    k_ref = [cache.float().clone() for cache in model.k_cache]
    v_ref = [cache.float().clone() for cache in model.v_cache]
    tokens = torch.tensor([3, 500, 77], device="cuda")
    positions = torch.tensor([5, 5, 5], dtype=torch.int32, device="cuda")
    captured = None
    for step in range(3):
        expected = dense_reference_step(config, blocks, embedding, final_norm, head, tokens, positions, k_ref, v_ref)
        if step < 2:
            logits = model.step(tokens, positions).clone()
        else:   # the third token goes through the captured graph
            captured = model.capture(3)
            for cache, saved in zip(model.k_cache + model.v_cache, saved_caches):
                cache.copy_(saved)   # capture warm-ups wrote position 0 slots: restore the context
            captured.tokens.copy_(tokens)
            captured.positions.copy_(positions)
            logits = captured.replay().clone()
        assert rel(logits, expected) < 1e-2, step
        assert torch.equal(logits.argmax(-1), expected.argmax(-1))
        tokens = expected.argmax(-1)
        positions = positions + 1
        saved_caches = [cache.clone() for cache in model.k_cache + model.v_cache]
    assert model.weight_bytes > 0


def test_packed_head_and_greedy_pick():
    """A head-quantised model: the head is one more packed matvec over this rank's rows of the code
    stream; the greedy step returns the arg-max of those logits (smallest token on a tie)."""
    torch.manual_seed(4)
    config = SMALL
    blocks = [quantised_block(config, 20 + i) for i in range(config.layers)]
    embedding = torch.randn(config.vocab, config.hidden, device="cuda").half()
    final_norm = (torch.rand(config.hidden, device="cuda") + 0.5).half()
    head_weight = (torch.randn(config.vocab, config.hidden, device="cuda") * 0.05).half()
    head_q = mk.int(4, group=128)(head_weight.float())
    dense = build_model(config, blocks, embedding, final_norm, head_q.w.half())
    packed = build_model(config, blocks, embedding, final_norm, head_q)
    assert packed.packed_head is not None and packed.head is None
    tokens = torch.tensor([3, 500, 77, 9], device="cuda")
    positions = torch.zeros(4, dtype=torch.int32, device="cuda")
    expected = dense.step(tokens, positions).float()
    logits = packed.step(tokens, positions).float()
    assert rel(logits, expected) < 2e-3
    picked = packed.step(tokens, positions, greedy=True)
    assert picked.dtype == torch.int64 and torch.equal(picked, logits.argmax(-1))
    # the key orders like the fp16 value, negative maxima included; a tie keeps the smallest index
    rows = torch.tensor([[-3.0, -1.5, -7.0, -1.5], [0.0, -0.0, -2.0, -1.0], [5.0, 65504.0, 2.0, 65504.0]], device="cuda").half()
    keys = kernels.argmax_keys(rows, torch.empty(3, dtype=torch.int64, device="cuda"), offset=10)
    assert kernels.tokens_of_keys(keys).tolist() == [11, 10, 11]
    assert (keys[2] ^ (1 << 63)) > (keys[1] ^ (1 << 63)) > (keys[0] ^ (1 << 63))


def test_decoder_refuses_positions_outside_the_cache():
    """The host check of an eager step; no out-of-range position ever reaches a kernel here."""
    config = SMALL
    model = tp.TensorParallelDecoder(config, rank=0, world=1, device=torch.device("cuda"), max_batch=2, capacity=16)
    tokens = torch.tensor([1, 2], device="cuda")
    for bad in ([0, 16], [-1, 3]):
        with pytest.raises(ValueError, match="leave the cache"):
            model.step(tokens, torch.tensor(bad, dtype=torch.int32, device="cuda"))
    assert kernels.decode_status() == 0


@pytest.mark.parametrize("world", [2, 4])
def test_shards_sum_to_the_full_projection(world):
    config = tp.DecoderConfig(layers=1, hidden=512, q_heads=8, kv_heads=4, head_dim=128, intermediate=1024, vocab=512)
    block = quantised_block(config, 42)
    device = torch.device("cuda")
    full = tp.shard_block(block, config, 0, 1, device)
    torch.manual_seed(5)
    x = torch.randn(4, config.hidden, device="cuda").half()
    wide_q = torch.randn(4, config.q_heads * config.head_dim, device="cuda").half()
    wide_i = torch.randn(4, config.intermediate, device="cuda").half()
    out = lambda shard: torch.empty(4, shard.out_rows, device="cuda", dtype=torch.float16)
    qkv_full, gu_full = full["qkv"](x, out(full["qkv"])), full["gate_up"](x, out(full["gate_up"]))
    o_full, down_full = full["o"](wide_q, out(full["o"])), full["down"](wide_i, out(full["down"]))
    q_rows, kv_rows = config.q_heads * config.head_dim, config.kv_heads * config.head_dim
    o_sum, down_sum = torch.zeros_like(o_full, dtype=torch.float32), torch.zeros_like(down_full, dtype=torch.float32)
    for rank in range(world):
        shards = tp.shard_block(block, config, rank, world, device)
        qkv = shards["qkv"](x, out(shards["qkv"]))
        rq, rk = tp.rows_of(rank, world, q_rows), tp.rows_of(rank, world, kv_rows)
        expected = torch.cat((qkv_full[:, rq], qkv_full[:, q_rows:][:, rk], qkv_full[:, q_rows + kv_rows:][:, rk]), 1)
        assert torch.equal(qkv, expected)   # same rows, same arithmetic: bit-identical
        gu = shards["gate_up"](x, out(shards["gate_up"]))
        ri = tp.rows_of(rank, world, config.intermediate)
        assert torch.equal(gu, torch.cat((gu_full[:, ri], gu_full[:, config.intermediate:][:, ri]), 1))
        share_q, share_i = q_rows // world, config.intermediate // world
        o_sum += shards["o"](wide_q[:, rank * share_q:(rank + 1) * share_q].contiguous(), out(shards["o"])).float()
        down_sum += shards["down"](wide_i[:, rank * share_i:(rank + 1) * share_i].contiguous(), out(shards["down"])).float()
    assert rel(o_sum, o_full) < 2e-3 and rel(down_sum, down_full) < 2e-3


# ---------------------------------------------------------------- the peer-memory reduction on one GPU
class LocalExchange:
    """``world`` exchange buffers on one device, as the ranks of one node would map them."""

    def __init__(self, world, rows, width):
        import ctypes

        from mlkit_b200 import _native

        self.lib, self.world, self.rows, self.width = _native.library(), world, rows, width
        size = self.lib.mkb_peer_buffer_bytes(rows, width, world)
        self.buffers = []
        for _ in range(world):
            pointer = ctypes.c_void_p()
            _native.check(self.lib.mkb_peer_alloc(size, ctypes.byref(pointer)), "peer_alloc")
            self.buffers.append(pointer.value)
        self.peers = torch.tensor(self.buffers, dtype=torch.int64, device="cuda")

    def reduce(self, rank, partial, residual, weight, eps=1e-5):
        """One reduction as rank ``rank`` issues it; returns (reduced, normed); ``residual`` is updated."""
        from mlkit_b200 import _native

        normed, reduced = torch.empty_like(partial), torch.empty_like(partial)
        _native.check(self.lib.mkb_peer_reduce_add_rmsnorm(
            partial.data_ptr(), self.peers.data_ptr(), self.buffers[rank], residual.data_ptr(), weight.data_ptr(),
            normed.data_ptr(), reduced.data_ptr(), partial.shape[0], self.width, self.rows, self.world, rank, eps,
            torch.cuda.current_stream().cuda_stream), "peer_reduce_add_rmsnorm")
        return reduced, normed

    def status(self, rank):
        import ctypes

        from mlkit_b200 import _native

        value = ctypes.c_int(-1)
        _native.check(self.lib.mkb_peer_status(self.buffers[rank], ctypes.byref(value)), "peer_status")
        return value.value

    def limit(self, rank, polls):
        from mlkit_b200 import _native

        _native.check(self.lib.mkb_peer_set_poll_limit(self.buffers[rank], polls), "peer_set_poll_limit")

    def split(self, rank, parts):
        from mlkit_b200 import _native

        _native.check(self.lib.mkb_peer_set_split(self.buffers[rank], parts), "peer_set_split")

    def close(self):
        torch.cuda.synchronize()
        for buffer in self.buffers:
            self.lib.mkb_peer_free(buffer)


def reference_add_rmsnorm(total16, residual, weight, eps=1e-5):
    """fp16 sum added to the residual (one rounding), then the norm with the operator's rounding points."""
    updated = (residual.float() + total16.float()).half()
    inverse = torch.rsqrt(updated.float().pow(2).mean(-1, keepdim=True) + eps)
    return updated, ((updated.float() * inverse).half().float() * weight.float()).half()


@pytest.mark.parametrize("rows_in", [1, 8])
def test_peer_reduction_of_one_rank_equals_add_rmsnorm(rows_in):
    """world = 1: the kernel pushes to and waits on its own buffer only.  Five reductions, eager and
    replayed from a CUDA graph, walk both slot parities and the persistent per-row counters; sum,
    residual and norm must equal ``mkb_add_rmsnorm`` on the same data bit for bit."""
    torch.manual_seed(rows_in)
    width = 1024
    exchange = LocalExchange(1, 8, width)
    weight = (torch.rand(width, device="cuda") + 0.5).half()
    residual, expected_residual = torch.zeros(rows_in, width, device="cuda").half(), torch.zeros(rows_in, width, device="cuda").half()
    for _ in range(3):
        partial = torch.randn(rows_in, width, device="cuda").half()
        reduced, normed = exchange.reduce(0, partial, residual, weight)
        expected_normed = torch.empty_like(partial)
        kernels.add_rmsnorm(expected_residual, partial, weight, expected_normed, 1e-5)
        assert torch.equal(reduced, partial) and torch.equal(residual, expected_residual)
        assert torch.equal(normed, expected_normed)
    partial = torch.randn(rows_in, width, device="cuda").half()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            reduced, normed = exchange.reduce(0, partial, residual, weight)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        graph.replay()
        expected_normed = torch.empty_like(partial)
        kernels.add_rmsnorm(expected_residual, partial, weight, expected_normed, 1e-5)
        torch.cuda.synchronize()
        assert torch.equal(reduced, partial) and torch.equal(residual, expected_residual)
        assert torch.equal(normed, expected_normed)
    assert exchange.status(0) == 0
    exchange.close()


@pytest.mark.parametrize("rows_in", [1, 8])
def test_peer_reduction_of_two_ranks_in_turn(rows_in):
    """Two ranks' buffers on one GPU, the ranks' kernels issued one after the other (kernels that wait
    on one another must not share a GPU).  Rank 1 goes first with a poll limit of a thousand: it
    delivers its partial to both buffers, its own wait for rank 0 runs out and its result is void.
    Rank 0 then finds both partials and must produce the fp16 sum in rank order, the updated residual
    and the norm.  Three rounds use both slot parities."""
    torch.manual_seed(10 + rows_in)
    width = 2048
    exchange = LocalExchange(2, 8, width)
    exchange.limit(1, 1000)
    weight = (torch.rand(width, device="cuda") + 0.5).half()
    residual = torch.randn(rows_in, width, device="cuda").half()
    expected_residual = residual.clone()
    scratch_residual = torch.zeros_like(residual)
    for _ in range(3):
        partials = [torch.randn(rows_in, width, device="cuda").half() for _ in range(2)]
        exchange.reduce(1, partials[1], scratch_residual, weight)
        reduced, normed = exchange.reduce(0, partials[0], residual, weight)
        total16 = (partials[0].float() + partials[1].float()).half()
        expected_residual, expected_normed = reference_add_rmsnorm(total16, expected_residual, weight)
        assert torch.equal(reduced, total16)
        assert torch.equal(residual, expected_residual)
        assert rel(normed, expected_normed) < 1e-3 and (normed.float() - expected_normed.float()).abs().max() < 0.02
    assert exchange.status(0) == 0 and exchange.status(1) == 1
    exchange.close()


def test_peer_reduction_wait_runs_out_without_hanging():
    """A flag that nothing sets: with a poll limit of a thousand the kernel gives up, sets the status
    word and finishes; the next call skips its wait altogether."""
    width = 512
    exchange = LocalExchange(2, 8, width)
    exchange.limit(0, 1000)
    weight = torch.ones(width, device="cuda").half()
    partial = torch.ones(2, width, device="cuda").half()
    residual = torch.zeros(2, width, device="cuda").half()
    assert exchange.status(0) == 0
    exchange.reduce(0, partial, residual, weight)
    torch.cuda.synchronize()
    assert exchange.status(0) == 1
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    exchange.limit(0, 20_000_000)   # would be seconds of polling if the wait were not skipped
    start.record()
    exchange.reduce(0, partial, residual, weight)
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 50 and exchange.status(0) == 1
    exchange.close()


@pytest.mark.parametrize("parts", [2, 4])
@pytest.mark.parametrize("rows_in", [1, 8])
def test_peer_reduction_with_a_row_split_over_several_ctas(rows_in, parts):
    """Wide worlds split a row over several CTAs (each pushes its slice; the slices' sums of squares meet
    through the rank's own header).  Forced here on two ranks run in turn, eager and from a CUDA graph: sum
    and residual are bit-equal to the one-CTA result, the norm agrees to the last bits (its sum of squares
    is added in another order), and a width the split does not divide falls back to fewer CTAs."""
    torch.manual_seed(40 + rows_in + parts)
    for width in (8192, 2056):
        exchange = LocalExchange(2, 8, width)
        exchange.limit(1, 1000)
        for rank in (0, 1):
            exchange.split(rank, parts)
        weight = (torch.rand(width, device="cuda") + 0.5).half()
        residual = torch.randn(rows_in, width, device="cuda").half()
        expected_residual, scratch_residual = residual.clone(), torch.zeros_like(residual)
        for _ in range(3):
            partials = [torch.randn(rows_in, width, device="cuda").half() for _ in range(2)]
            exchange.reduce(1, partials[1], scratch_residual, weight)
            reduced, normed = exchange.reduce(0, partials[0], residual, weight)
            total16 = (partials[0].float() + partials[1].float()).half()
            expected_residual, expected_normed = reference_add_rmsnorm(total16, expected_residual, weight)
            assert torch.equal(reduced, total16) and torch.equal(residual, expected_residual)
            assert rel(normed, expected_normed) < 1e-3 and (normed.float() - expected_normed.float()).abs().max() < 0.02
        assert exchange.status(0) == 0 and exchange.status(1) == 1
        exchange.close()
    # one rank alone, replayed from a graph: the per-CTA counters and both parities
    width = 4096
    exchange = LocalExchange(1, 8, width)
    exchange.split(0, parts)
    weight = (torch.rand(width, device="cuda") + 0.5).half()
    residual, expected_residual = torch.zeros(rows_in, width, device="cuda").half(), torch.zeros(rows_in, width, device="cuda").half()
    partial = torch.randn(rows_in, width, device="cuda").half()
    exchange.reduce(0, partial, residual, weight)
    expected_residual, _ = reference_add_rmsnorm(partial, expected_residual, weight)
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            reduced, normed = exchange.reduce(0, partial, residual, weight)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        expected_residual, expected_normed = reference_add_rmsnorm(partial, expected_residual, weight)
        assert torch.equal(reduced, partial) and torch.equal(residual, expected_residual)
        assert rel(normed, expected_normed) < 1e-3
    assert exchange.status(0) == 0
    exchange.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def two_rank_step(rank, world, peer_exchange):
    """Body of one rank of the 2-GPU tests (run by tests/two_rank_worker.py under torch.distributed.run).
    Returns a report dict; nothing is raised here, so no rank leaves the other one waiting."""
    import torch.distributed as dist

    config = SMALL
    report = {"rank": rank, "problems": []}
    with torch.cuda.device(rank):
        blocks = [quantised_block(config, 10 + i) for i in range(config.layers)]   # same seeds on every rank
        generator = torch.Generator(device="cuda").manual_seed(3)
        embedding = torch.randn(config.vocab, config.hidden, device="cuda", generator=generator).half()
        final_norm = (torch.rand(config.hidden, device="cuda", generator=generator) + 0.5).half()
        head = (torch.randn(config.vocab, config.hidden, device="cuda", generator=generator) * 0.05).half()
        model = tp.TensorParallelDecoder(config, rank=rank, world=world, device=torch.device("cuda", rank),
                                         max_batch=4, capacity=64)
        ones = torch.ones(config.hidden, device="cuda")
        for block in blocks:
            model.add_block(tp.shard_block(block, config, rank, world, torch.device("cuda", rank)), ones, ones)
        model.set_head(embedding, final_norm, head)
        tokens = torch.tensor([3, 500, 77], device="cuda")
        positions = torch.zeros(3, dtype=torch.int32, device="cuda")
        if peer_exchange:
            # the same step with the library all-reduce first: the peer-memory reduction adds the same
            # fp16 partials in fp32 and rounds once, so the two may differ by an fp16 rounding only
            through_nccl = model.step(tokens, positions).float().cpu()
            model.enable_peer_exchange()
        logits = model.step(tokens, positions).float().cpu()
        if peer_exchange:
            again = model.step(tokens, positions).float().cpu()       # the other parity of the slots
            if not torch.equal(logits, again):
                report["problems"].append("two steps on the same inputs differ")
            if matvec.relative_l2(logits.numpy(), through_nccl.numpy()) >= 2e-3:
                report["problems"].append("peer-memory reduction differs from the library all-reduce")
            captured = model.capture(3)                                # and inside a CUDA graph
            captured.tokens.copy_(tokens)
            captured.positions.copy_(positions)
            dist.barrier()
            replayed = captured.replay().float().cpu()
            if matvec.relative_l2(replayed.numpy(), logits.numpy()) >= 2e-3:
                report["problems"].append("graph replay differs from the eager step")
            if model.exchange.status() != 0:
                report["problems"].append("a bounded wait expired")
        if rank == 0:
            k_ref = [torch.zeros(4, config.kv_heads, 64, config.head_dim, device="cuda") for _ in blocks]
            v_ref = [torch.zeros(4, config.kv_heads, 64, config.head_dim, device="cuda") for _ in blocks]
            expected = dense_reference_step(config, blocks, embedding, final_norm, head, tokens, positions, k_ref, v_ref)
            report["error"] = float(matvec.relative_l2(logits.numpy(), expected.cpu().numpy()))
    return report


def _run_two_ranks(peer_exchange):
    """Two ranks under torch.distributed.run, as bench.py is launched; every rank prints one JSON report."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    worker = Path(__file__).with_name("two_rank_worker.py")
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), str(worker)] + (["--peer"] if peer_exchange else [])
    environment = dict(os.environ, NCCL_NVLS_ENABLE="0")
    finished = subprocess.run(command, capture_output=True, text=True, timeout=240, env=environment)
    import re

    reports = [json.loads(found) for found in re.findall(r"REPORT (\{.*?\})(?=\s|REPORT|$)", finished.stdout)]
    assert finished.returncode == 0 and len(reports) == 2, finished.stdout[-2000:] + finished.stderr[-2000:]
    for report in reports:
        assert report["problems"] == [], report
        if report["rank"] == 0:
            assert report["error"] < 1e-2


def test_two_gpu_decode_with_peer_memory_reduction():
    """The one-shot peer-memory all-reduce (mkb_peer_push + mkb_peer_add_rmsnorm) in place of NCCL."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_two_ranks(peer_exchange=True)


def test_two_gpu_decode_matches_dense_reference():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_two_ranks(peer_exchange=False)
