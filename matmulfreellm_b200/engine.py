"""Decode-step execution: one cached single-token forward plus arg-max, captured once in a CUDA graph and
replayed per generated token, so that the ~50 us of weight streaming a step needs is not buried under
host-side launch overhead."""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _lib, kernels
from .models.utils import RecurrentCache
from .ops.fusedbitnet import BitLinear


class GreedyDecoder:
    """Greedy decoding for a fixed batch size with device-resident state.

    `prefill(prompt)` runs the prompt once and seeds the static cache and the first token; each `step()`
    replays the captured graph: it reads `self.ids` [B,1], advances every layer's recurrent state in place,
    writes the next token to `self.next` [B] and feeds it back into `self.ids`.
    """

    def __init__(self, model, batch_size: int, use_graph: bool = True):
        self.model, self.B = model, batch_size
        dev = next(model.parameters()).device
        self.device = dev
        self.ids = torch.zeros(batch_size, 1, dtype=torch.int64, device=dev)
        self.next = torch.zeros(batch_size, dtype=torch.int64, device=dev)
        self.cache = RecurrentCache.from_legacy_cache(
            [layer.attn.init_state(batch_size) for layer in model.model.layers])
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_step = 0
        self._use_graph = use_graph

    def _step_eager(self):
        out = self.model(input_ids=self.ids, past_key_values=self.cache, use_cache=True)
        nxt = kernels.argmax_rows(out.logits[:, -1])
        self.next.copy_(nxt)
        self.ids.copy_(nxt[:, None])

    def _capture(self):
        saved = [tuple(s.clone() for s in layer) for layer in self.cache.states]
        saved_ids = self.ids.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                     # warm-up outside capture (allocator, lazy packing)
                self._step_eager()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        before = _lib.launch_count
        with torch.cuda.graph(graph):
            self._step_eager()
        self.kernels_per_step = _lib.launch_count - before
        self.graph = graph
        for layer, keep in zip(self.cache.states, saved):   # undo the warm-up steps' effect on the state
            for dst, src in zip(layer, keep):
                dst.copy_(src)
        self.ids.copy_(saved_ids)

    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt [B, T]; returns the first generated token [B] (also left in self.ids / self.next)."""
        if prompt_ids.shape[0] != self.B:
            raise ValueError(f"decoder was built for batch {self.B}, got {prompt_ids.shape[0]}")
        out = self.model(input_ids=prompt_ids, use_cache=True, last_token_only=True)
        for layer, new in zip(self.cache.states, out.past_key_values):
            for dst, src in zip(layer, new):
                dst.copy_(src)
        nxt = kernels.argmax_rows(out.logits[:, -1])
        self.next.copy_(nxt)
        self.ids.copy_(nxt[:, None])
        return self.next

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Consume self.ids, produce the next token in self.next (and feed it back). Returns self.next."""
        if not self._use_graph:
            before = _lib.launch_count
            self._step_eager()
            self.kernels_per_step = _lib.launch_count - before
        else:
            if self.graph is None:
                self._capture()
            self.graph.replay()
        return self.next

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        toks = torch.empty(self.B, max_new_tokens, dtype=torch.int64, device=self.device)
        self.prefill(prompt_ids)
        for t in range(max_new_tokens):
            toks[:, t].copy_(self.next)
            if t + 1 < max_new_tokens:
                self.step()
        return torch.cat([prompt_ids, toks], dim=1)


def bitlinear_modules(model) -> List[BitLinear]:
    """Every BitLinear of the model in execution order."""
    return [m for m in model.modules() if isinstance(m, BitLinear)]


class WeightStreamProbe:
    """Runs the BitLinear contraction of every layer of `model` once, back to back, for M token rows with
    pre-quantised activations — i.e. exactly the weight-streaming kernels of one decode step and nothing
    else — so their device time can be measured with CUDA events."""

    def __init__(self, model, M: int, out_dtype: torch.dtype):
        self.items = []
        dev = next(model.parameters()).device
        g = torch.Generator(device=dev).manual_seed(0)
        self.packed_bytes = 0
        for m in bitlinear_modules(model):
            pw = m.packed()
            x = torch.randn(M, pw.K, generator=g, device=dev, dtype=torch.float32).to(out_dtype)
            q, dq, rs = kernels.act_quant(x, None, 1e-6)
            out = torch.empty(M, pw.N, dtype=out_dtype, device=dev)
            self.items.append((q, dq, rs, pw, out))
            self.packed_bytes += pw.packed.numel()
        self.out_dtype = out_dtype
        self.launches = len(self.items)

    def run(self):
        for q, dq, rs, pw, out in self.items:
            kernels.bitlinear(q, dq, rs, pw, self.out_dtype, out=out)
