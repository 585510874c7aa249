"""Host-side logic of the batch-sharded multi-GPU path, run as two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from matmulfreellm_b200.sharding import gather_batch, generate_sharded, shard_batch, shard_range


def test_shard_range_covers_batch_once():
    for n in (0, 1, 5, 8, 13, 256):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


class _EchoModel:
    """Stand-in for HGRNBitForCausalLM.generate: appends (sequence's first token + step) so that the gathered
    result shows which rank produced which rows."""

    def generate(self, ids, max_new_tokens=1):
        extra = torch.stack([ids[:, 0] + s for s in range(max_new_tokens)], 1)
        return torch.cat([ids, extra], 1)


def _worker(rank, world, port, n_total):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(n_total * 3).view(n_total, 3)
        mine = shard_batch(full, rank, world)
        back = gather_batch(mine * 2, n_total)
        assert torch.equal(back, full * 2)
        out = generate_sharded(_EchoModel(), full, max_new_tokens=2)
        want = torch.cat([full, full[:, :1], full[:, :1] + 1], 1)
        assert torch.equal(out, want)
        if n_total >= 2:                         # every rank then holds less than the whole batch
            with pytest.raises(ValueError):
                gather_batch(full, n_total)      # passing the whole batch is rejected before any collective
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_total", [8, 5, 1])
def test_two_rank_gather_and_generate(n_total):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, n_total), nprocs=2, join=True)


def test_single_process_passthrough():
    t = torch.arange(6).view(3, 2)
    assert gather_batch(t, 3) is t
    assert torch.equal(generate_sharded(_EchoModel(), t, 1), torch.cat([t, t[:, :1]], 1))
