"""Batch sharding of independent sequences across the GPUs of one box.

Sequences never interact on this path (per-token statistics, per-sequence recurrent state, input-independent
weight scales), so every rank holds a full replica of the packed weights and runs its contiguous slice of
the batch with no collective on the data path.  NCCL (or gloo in CPU tests) is used once, to gather the
generated tokens or logits.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_items: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) slice of `n_items` for `rank`; the first n_items % world ranks get one extra."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_range(t.shape[0], rank, world)
    return t[lo:hi]


def gather_batch(local: torch.Tensor, n_total: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather the ranks' batch slices (dim 0) back into the full batch, on every rank.

    Shards may be ragged (n_total not divisible by the world size): each rank pads its slice to the largest
    shard, one all_gather_into_tensor moves the data, and the padding is dropped."""
    if not dist.is_available() or not dist.is_initialized():
        if local.shape[0] != n_total:
            raise ValueError("no process group: the local shard must be the whole batch")
        return local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, hi = shard_range(n_total, rank, world)
    if local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, expected {hi - lo}")
    width = -(-n_total // world)
    padded = local
    if local.shape[0] != width:
        padded = local.new_zeros((width,) + tuple(local.shape[1:]))
        padded[: local.shape[0]] = local
    out = local.new_empty((world * width,) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    pieces = []
    for r in range(world):
        rlo, rhi = shard_range(n_total, r, world)
        pieces.append(out[r * width: r * width + (rhi - rlo)])
    return torch.cat(pieces, dim=0)


@torch.no_grad()
def generate_sharded(model, input_ids: torch.Tensor, max_new_tokens: int, group: Optional[dist.ProcessGroup] = None,
                     **generate_kwargs) -> torch.Tensor:
    """Generate for the full batch `input_ids` [B, T] (identical on every rank): each rank decodes its slice with
    `model.generate`, then one gather returns [B, T + new] on every rank.  Ranks whose slice is empty (B < world)
    only take part in the gather.

    With `eos_token_id`, `generate` ends a slice where its last sequence finished, so the ranks' results differ in
    width.  A collective needs equal element counts on every rank: each slice is padded with eos to
    T + max_new_tokens before the gather, and the gathered batch is cut where a single-GPU `generate` of the whole
    batch would have stopped (one past the step at which the last sequence emitted eos, if every sequence did)."""
    B, T = input_ids.shape
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    eos = generate_kwargs.get("eos_token_id")
    mine = shard_batch(input_ids, rank, world)
    full_width = T + max_new_tokens
    if mine.shape[0]:
        out = model.generate(mine, max_new_tokens=max_new_tokens, **generate_kwargs)
        if out.shape[1] < full_width:
            if eos is None:
                raise RuntimeError(f"generate returned {out.shape[1]} positions, expected {full_width}")
            pad = out.new_full((out.shape[0], full_width - out.shape[1]), int(eos))
            out = torch.cat([out, pad], dim=1)
    else:
        out = input_ids.new_empty((0, full_width))
    full = gather_batch(out, B, group)
    if eos is not None and B and max_new_tokens:
        hit = full[:, T:] == int(eos)
        if bool(hit.any(dim=1).all()):
            steps = torch.arange(max_new_tokens, device=full.device).expand_as(hit)
            first = torch.where(hit, steps, torch.full_like(steps, max_new_tokens)).min(dim=1).values
            full = full[:, : T + int(first.max().item()) + 1]
    return full


def _self_check() -> None:
    """`python -m torch.distributed.run --nproc-per-node N -m matmulfreellm_b200.sharding`: a small random-init model,
    a ragged batch sharded over the N GPUs and gathered with NCCL, compared on every rank with the same batch decoded
    on that rank alone.  Prints one JSON line on rank 0."""
    import json
    import os

    from .models import HGRNBitConfig, HGRNBitForCausalLM
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if "RANK" in os.environ:
        dist.init_process_group("nccl", device_id=device)
    world = dist.get_world_size() if dist.is_initialized() else 1
    torch.manual_seed(0)                                   # same weights on every rank
    cfg = HGRNBitConfig(vocab_size=32000, hidden_size=256, num_hidden_layers=2, intermediate_size=704)
    model = HGRNBitForCausalLM(cfg).eval().to(device)
    model.pack_weights()
    model = model.bfloat16()
    B = 2 * world + 1                                      # ragged: one rank gets an extra sequence
    ids = torch.randint(0, 32000, (B, 12), generator=torch.Generator().manual_seed(1)).to(device)
    sharded = generate_sharded(model, ids, 16)
    alone = model.generate(ids, max_new_tokens=16)
    ok = torch.tensor([int(torch.equal(sharded, alone))], device=device)
    if dist.is_initialized():
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if (dist.get_rank() if dist.is_initialized() else 0) == 0:
        print(json.dumps({"check": "generate_sharded == single-GPU generate", "world": world, "batch": B,
                          "shape": list(sharded.shape), "ok": bool(ok.item())}), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()
    if not ok.item():
        raise SystemExit(1)


if __name__ == "__main__":
    _self_check()
