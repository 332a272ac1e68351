"""Tensor-parallel plumbing on CPU: two gloo ranks shard a layer, compute their parts with the numpy
oracle and exchange them; the result must equal the unsharded oracle product."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import matvec
from tests import helpers


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from mlkit_b200 import tp

        rows, width, bits, group = 64, 512, 4, 128
        layer = helpers.make_layer(rows, width, bits, group, seed=5)
        x = helpers.activations(3, width, seed=6)
        full = matvec.reconstruct_then_matmul(x, layer["packed"], layer["scales16"], layer["values"], group, bits,
                                              (rows, width))
        packed, scales = torch.from_numpy(layer["packed"]), torch.from_numpy(layer["scales16"])

        # row parallel: each rank owns a slice of the reduction axis; one all-reduce sums the partials
        part_packed, part_scales = tp.shard_columns(packed, scales, rank, world, width, bits, group)
        share = width // world
        partial = matvec.reconstruct_then_matmul(x[:, rank * share:(rank + 1) * share], part_packed.numpy(),
                                                 part_scales.numpy(), layer["values"], group, bits, (rows, share))
        reduced = torch.from_numpy(partial.astype(np.float32))
        dist.all_reduce(reduced)
        assert matvec.relative_l2(reduced.numpy(), full) < 1e-6

        # column parallel: each rank owns output rows; an all-gather assembles them
        own = tp.rows_of(rank, world, rows)
        part_packed, part_scales = tp.shard_rows(packed, scales, own, width, bits)
        mine = matvec.reconstruct_then_matmul(x, part_packed.numpy(), part_scales.numpy(), layer["values"], group,
                                              bits, (rows // world, width))
        pieces = [torch.empty(3, rows // world) for _ in range(world)]
        dist.all_gather(pieces, torch.from_numpy(mine.astype(np.float32)))
        assert matvec.relative_l2(torch.cat(pieces, 1).numpy(), full) < 1e-6

        # greedy pick over vocabulary shards: every rank contributes 8 bytes per sequence (the sortable
        # key of its best logit and the complement of its token id); the unsigned maximum wins
        logits = torch.tensor([[0.5, -2.0, 3.0, 3.0, -1.0, 2.5, 3.0, 0.0], [-4.0, -1.0, -3.0, -2.0, -1.0, -6.0, -7.0, -8.0]])
        share = logits.shape[1] // world
        local = logits[:, rank * share:(rank + 1) * share].half()
        bits = local.view(torch.int16).to(torch.int64) & 0xFFFF
        key = torch.where(bits >= 0x8000, ~bits & 0xFFFF, bits | 0x8000)          # the kernel's map of fp16 to unsigned
        words = (key << 32) | (0xFFFFFFFF - (torch.arange(share) + rank * share))
        best = tp.best_keys(words.t())   # this rank's best word per sequence
        gathered = [torch.empty_like(best) for _ in range(world)]
        dist.all_gather(gathered, best)
        winners = 0xFFFFFFFF - (tp.best_keys(torch.stack(gathered)) & 0xFFFFFFFF)
        assert winners.tolist() == [2, 1]   # ties keep the smallest token; negative maxima order correctly

        # a rank that fails between steps is seen by the others through the store, not through a hang
        store = dist.distributed_c10d._get_default_store()
        store.set(f"alive{rank}", "1")
        dist.barrier()
        assert all(store.get(f"alive{r}") == b"1" for r in range(world))
        dist.destroy_process_group()
    except Exception as error:  # noqa: BLE001
        failures.put(f"rank {rank}: {error!r}")
        raise


def test_two_ranks_shard_and_exchange():
    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_worker, args=(rank, 2, port, failures)) for rank in range(2)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=120)
    assert failures.empty(), failures.get()
    assert all(worker.exitcode == 0 for worker in workers)


def test_config_validation():
    from mlkit_b200 import tp

    tp.LLAMA3_70B.validate(8)
    tp.LLAMA3_70B.validate(1)
    tp.LLAMA3_8B.validate(8)
    with pytest.raises(ValueError, match="divide"):
        tp.LLAMA3_70B.validate(3)
    odd = tp.DecoderConfig(layers=1, hidden=256, q_heads=4, kv_heads=4, head_dim=32, intermediate=320, vocab=64)
    with pytest.raises(ValueError, match="splits a scale group"):
        odd.validate(4)
