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


class _EosModel:
    """Stand-in for generate(..., eos_token_id=e): sequence b (identified by its first token) emits eos at step
    first_token % 7, is padded with eos afterwards, and the result ends where the last LOCAL sequence finished —
    so two ranks return different widths."""

    def generate(self, ids, max_new_tokens=1, eos_token_id=None):
        stop = ids[:, 0] % 7
        steps = torch.arange(max_new_tokens).expand(ids.shape[0], max_new_tokens)
        toks = torch.where(steps >= stop[:, None], torch.full_like(steps, eos_token_id), 1000 + steps)
        n = min(int(stop.max().item()) + 1, max_new_tokens)
        return torch.cat([ids, toks[:, :n]], 1)


def _eos_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 0's sequences stop at steps 0..2, rank 1's at steps 3..6 -> local widths 3+3 and 3+7
        full = torch.tensor([[0, 9, 9], [1, 9, 9], [2, 9, 9], [3, 9, 9], [5, 9, 9], [6, 9, 9]])
        out = generate_sharded(_EosModel(), full, max_new_tokens=12, eos_token_id=77)
        want = _EosModel().generate(full, max_new_tokens=12, eos_token_id=77)       # the whole batch on one rank
        assert out.shape == want.shape == (6, 3 + 7) and torch.equal(out, want)
        # a sequence that never stops within the budget: full width, finished rows padded with eos
        full2 = torch.tensor([[0, 9, 9], [1, 9, 9], [6, 9, 9], [2, 9, 9]])
        out2 = generate_sharded(_EosModel(), full2, max_new_tokens=4, eos_token_id=77)
        want2 = _EosModel().generate(full2, max_new_tokens=4, eos_token_id=77)
        assert out2.shape == (4, 7) and torch.equal(out2, want2)
    finally:
        dist.destroy_process_group()


def test_two_rank_generate_with_eos_finishing_at_different_steps():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_eos_worker, args=(2, port), nprocs=2, join=True)


def test_single_process_passthrough():
    t = torch.arange(6).view(3, 2)
    assert gather_batch(t, 3) is t
    assert torch.equal(generate_sharded(_EchoModel(), t, 1), torch.cat([t, t[:, :1]], 1))


# ------------------------------------------------------------------------------------------------------------
# sequence (T) sharding of the recurrence: one (decay, final state) exchange per scan
# ------------------------------------------------------------------------------------------------------------
def _cpu_scan(gate_is_log):
    """h_t = f_t * h_{t-1} + x_t in fp32, as the oracle's naive recurrence; stands in for the CUDA scan kernel."""
    def scan(x, g, h0):
        f = g.float().exp() if gate_is_log else g.float()
        h = torch.zeros(x.shape[0], x.shape[-1]) if h0 is None else h0.float().clone()
        o = torch.empty(x.shape, dtype=torch.float32)
        for t in range(x.shape[1]):
            h = f[:, t] * h + x[:, t].float()
            o[:, t] = h
        return o.to(x.dtype), h
    return scan


def _seq_case(gate_is_log, T=53):
    g = torch.Generator().manual_seed(11)
    x = torch.randn(2, T, 8, generator=g)
    gate = torch.nn.functional.logsigmoid(torch.randn(2, T, 8, generator=g) + 1.0)
    return x, (gate if gate_is_log else gate.exp()), torch.randn(2, 8, generator=g)


def _seq_worker(rank, world, port, gate_is_log):
    from matmulfreellm_b200.seq_sharding import hgrn_scan_seq_sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, gate, h0 = _seq_case(gate_is_log)
        scan = _cpu_scan(gate_is_log)
        o_ref, h_ref = scan(x, gate, h0)
        lo, hi = shard_range(x.shape[1], rank, world)            # ragged slices: 53 positions over 2 or 3 ranks
        o, last = hgrn_scan_seq_sharded(x[:, lo:hi].contiguous(), gate[:, lo:hi].contiguous(), h0, gate_is_log,
                                        local_scan=scan)
        assert torch.allclose(o, o_ref[:, lo:hi], rtol=1e-5, atol=1e-5)
        assert torch.allclose(last, h_ref, rtol=1e-5, atol=1e-5)     # the whole sequence's final state, on every rank
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,gate_is_log", [(2, True), (3, True), (2, False)])
def test_sequence_sharded_scan_matches_whole_scan(world, gate_is_log):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_seq_worker, args=(world, port, gate_is_log), nprocs=world, join=True)


def test_fold_carries_and_single_process():
    from matmulfreellm_b200.seq_sharding import fold_carries, hgrn_scan_seq_sharded, slice_decay
    x, gate, h0 = _seq_case(True)
    scan = _cpu_scan(True)
    o_ref, h_ref = scan(x, gate, h0)
    # three slices folded by hand
    cuts = [(0, 20), (20, 21), (21, 53)]
    decay = torch.stack([slice_decay(gate[:, a:b], True) for a, b in cuts])
    final = torch.stack([scan(x[:, a:b], gate[:, a:b], h0 if i == 0 else None)[1] for i, (a, b) in enumerate(cuts)])
    carry, last = fold_carries(decay, final)
    assert torch.allclose(last, h_ref, rtol=1e-5, atol=1e-5)
    assert torch.count_nonzero(carry[0]) == 0
    assert torch.allclose(carry[2], scan(x[:, :21], gate[:, :21], h0)[1], rtol=1e-5, atol=1e-5)
    # without a process group the call is the plain scan
    o, last = hgrn_scan_seq_sharded(x, gate, h0, True, local_scan=scan)
    assert torch.equal(o, o_ref) and torch.equal(last, h_ref)
