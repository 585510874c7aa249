"""Sequence (time) sharding of the HGRN recurrence across the GPUs of one box.

    h_t = f_t * h_{t-1} + x_t          (mmfreelm/ops/hgrn/recurrent_fuse.py:32-68, chunk.py:28-60)

is linear in the incoming state: over a slice of time steps it acts as  h_out = A * h_in + H  with
A = prod f_t  and  H = the slice's final state from a zero start.  A long sequence split contiguously along T over
the ranks therefore needs ONE exchange per scan: every rank reduces its slice to (A, H) [B, D] fp32, one
all_gather moves the 2 * B * D * 4 bytes per rank, every rank folds the pairs of the ranks before it into its own
incoming state and runs its slice again from that state.  Rank 0 knows its incoming state from the start, so its
first pass is already final.  Everything else on the path (BitLinear, the row-wise kernels) is per token and shards
along T with no exchange at all.

Cost on ranks > 0: two scans (the first one's output is discarded) plus one read of the gate for A, about 2.5 times
the bytes of an unsharded scan, for 1/world of the sequence.
The reference has no counterpart (its sequence length is bound to one GPU); this is the exchange a context-parallel
prompt pass would use, kept as an op-level building block: the model classes do not call it.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

LocalScan = Callable[[torch.Tensor, torch.Tensor, Optional[torch.Tensor]], Tuple[torch.Tensor, torch.Tensor]]


def _cuda_scan(gate_is_log: bool) -> LocalScan:
    from . import kernels

    def scan(x, g, h0):
        return kernels.hgrn_scan(x, g, h0, True, gate_is_log=gate_is_log, state_dtype=torch.float32)

    return scan


def slice_decay(g: torch.Tensor, gate_is_log: bool) -> torch.Tensor:
    """A = prod_t f_t over the slice, fp32 [..., D]; g is the forget gate [..., T, D] or its logarithm."""
    if gate_is_log:
        return g.float().sum(dim=-2).exp()
    return g.float().prod(dim=-2)


def fold_carries(decay: torch.Tensor, final: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """decay, final: [W, ..., D] — the (A, H) pair of every rank in time order, rank 0's H already containing the
    sequence's initial state.  Returns (carry_in [W, ..., D], state after the last rank [..., D]); carry_in[0] is
    zero because rank 0 starts from the initial state itself."""
    carry = torch.zeros_like(final)
    h = final[0]
    for r in range(1, decay.shape[0]):
        carry[r] = h
        h = decay[r] * h + final[r]
    return carry, h


@torch.no_grad()
def hgrn_scan_seq_sharded(x: torch.Tensor, g: torch.Tensor, initial_state: Optional[torch.Tensor] = None,
                          gate_is_log: bool = True, group: Optional[dist.ProcessGroup] = None,
                          local_scan: Optional[LocalScan] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x, g: this rank's contiguous time slice [B, T_local, D] of sequences split along T in rank order (slices may
    differ in length).  `initial_state` [B, D] is the state before the first position; only rank 0 reads it.
    Returns (o for the local slice, state after the whole sequence — identical on every rank).

    `local_scan(x, g, h0) -> (o, h_end)` defaults to the CUDA scan kernel; tests inject a CPU scan to check the
    exchange logic over gloo."""
    scan = local_scan or _cuda_scan(gate_is_log)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    h0 = initial_state.float() if (initial_state is not None and rank == 0) else None
    o, h_end = scan(x, g, h0)                       # rank 0: final; other ranks: H of the slice from a zero state
    if world == 1:
        return o, h_end.float()
    pair = torch.stack([slice_decay(g, gate_is_log), h_end.float()]).contiguous()      # [2, B, D]
    every = pair.new_empty((world * 2,) + tuple(pair.shape[1:]))      # concatenated along dim 0 (gloo accepts no other form)
    dist.all_gather_into_tensor(every, pair, group=group)
    every = every.view((world, 2) + tuple(pair.shape[1:]))
    carry, last = fold_carries(every[:, 0], every[:, 1])
    if rank > 0:
        o, _ = scan(x, g, carry[rank].contiguous())
    return o, last


def _self_check() -> None:
    """Run under torch.distributed.run on N GPUs: a sequence sharded along T over the ranks and stitched with one
    NCCL all_gather per scan equals the same scan on one GPU (fp32 state within 1e-4, bf16 outputs within 1e-2)."""
    import json
    import os

    from .sharding import shard_range
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(5)
    B, T, D = 3, 1000 * world + 37, 256
    x = torch.randn(B, T, D, generator=gen).to(torch.bfloat16).to(dev)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, D, generator=gen) + 2.0).to(dev)
    h0 = torch.randn(B, D, generator=gen).to(dev)
    lo, hi = shard_range(T, rank, world)
    o_loc, last = hgrn_scan_seq_sharded(x[:, lo:hi].contiguous(), g[:, lo:hi].contiguous(), h0, True)
    o_ref, last_ref = _cuda_scan(True)(x, g, h0)
    so, sh = o_ref.float().abs().max().item(), last_ref.abs().max().item()
    err_o = (o_loc.float() - o_ref[:, lo:hi].float()).abs().max().item() / so
    err_h = (last - last_ref).abs().max().item() / sh
    flag = torch.tensor([1 if (err_o <= 1e-2 and err_h <= 1e-4) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "T-sharded scan == single-GPU scan", "world": world, "shape": [B, T, D],
                          "max_rel_err_o": err_o, "max_rel_err_state": err_h, "ok": bool(flag.item())}))
    dist.destroy_process_group()
    if not flag.item():
        raise SystemExit(1)


if __name__ == "__main__":
    _self_check()
