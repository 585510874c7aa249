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
    writes the next token to `self.next` [B], which is the same buffer as `self.ids`.
    """

    def __init__(self, model, batch_size: int, use_graph: bool = True):
        self.model, self.B = model, batch_size
        dev = next(model.parameters()).device
        self.device = dev
        # `next` [B] and `ids` [B,1] are two views of one buffer: the arg-max of a step writes the next step's input
        self.next = torch.zeros(batch_size, dtype=torch.int64, device=dev)
        self.ids = self.next.view(batch_size, 1)
        self.cache = RecurrentCache.from_legacy_cache(
            [layer.attn.init_state(batch_size) for layer in model.model.layers])
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_step = 0
        self.last_logits: Optional[torch.Tensor] = None
        self._use_graph = use_graph
        # prompt passes of a repeated length are replayed from a graph as well: an eager pass is about 200 launches
        # through Python (about 19 us of host time each), which is more than the GPU needs for a short prompt
        self._prompt_seen: dict = {}       # prompt length -> times seen
        self._prompt_graphs: dict = {}     # prompt length -> (graph, static ids buffer), at most PROMPT_GRAPHS entries
        self._host_graphs: dict = {}       # (ids_host ptr, out_host ptr) -> (graph with the two copies, the buffers)

    def _step_eager(self):
        out = self.model(input_ids=self.ids, past_key_values=self.cache, use_cache=True)
        # [B, V] logits of the step; inside the captured graph this is a fixed buffer that every replay rewrites, so a
        # caller that samples instead of taking the arg-max reads it after step() and overwrites self.next
        self.last_logits = out.logits[:, -1]
        kernels.argmax_rows(self.last_logits, out=self.next)

    def _capture(self, ids_host: Optional[torch.Tensor] = None, out_host: Optional[torch.Tensor] = None):
        """Capture one decode step.  With pinned host buffers the copy of the input ids to the device and of the new
        tokens back are nodes of the same graph (returned, not stored in self.graph)."""
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
        # capture on the warm-up stream: its split-K workspace already exists (and is zero), so no fill of a
        # fresh workspace is recorded into the graph
        with torch.cuda.graph(graph, stream=side):
            if ids_host is not None:
                self.ids.copy_(ids_host, non_blocking=True)
            self._step_eager()
            if out_host is not None:
                out_host.copy_(self.next, non_blocking=True)
        self.kernels_per_step = _lib.launch_count - before
        if ids_host is None and out_host is None:
            self.graph = graph
        for layer, keep in zip(self.cache.states, saved):   # undo the warm-up steps' effect on the state
            for dst, src in zip(layer, keep):
                dst.copy_(src)
        self.ids.copy_(saved_ids)
        return graph

    PROMPT_GRAPH_MAX_TOKENS = 8192   # larger prompts are bound by the GPU, and their graphs would pin gigabytes
    PROMPT_GRAPHS = 4

    def _prefill_eager(self, prompt_ids: torch.Tensor) -> None:
        out = self.model(input_ids=prompt_ids, use_cache=True, last_token_only=True)
        for layer, new in zip(self.cache.states, out.past_key_values):
            for dst, src in zip(layer, new):
                dst.copy_(src)
        kernels.argmax_rows(out.logits[:, -1], out=self.next)

    def _capture_prompt(self, T: int):
        ids = torch.zeros(self.B, T, dtype=torch.int64, device=self.device)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._prefill_eager(ids)               # warm-up outside capture (allocator, workspace of this stream)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            self._prefill_eager(ids)
        if len(self._prompt_graphs) >= self.PROMPT_GRAPHS:
            self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
        self._prompt_graphs[T] = (graph, ids)
        return graph, ids

    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt [B, T]; returns the first generated token [B] (also left in self.ids / self.next).  The
        pass overwrites the recurrent state (a prompt starts from the zero state).  From the second prompt of the same
        length on, the pass is replayed from a CUDA graph."""
        if prompt_ids.shape[0] != self.B:
            raise ValueError(f"decoder was built for batch {self.B}, got {prompt_ids.shape[0]}")
        T = prompt_ids.shape[1]
        if self._use_graph and self.B * T <= self.PROMPT_GRAPH_MAX_TOKENS:
            entry = self._prompt_graphs.get(T)
            seen = self._prompt_seen.get(T, 0)
            self._prompt_seen[T] = seen + 1
            if entry is None and seen >= 1:
                entry = self._capture_prompt(T)
            if entry is not None:
                graph, ids = entry
                ids.copy_(prompt_ids)
                graph.replay()
                return self.next
        self._prefill_eager(prompt_ids)
        return self.next

    @torch.no_grad()
    def seed(self, past_key_values, last_logits: torch.Tensor) -> torch.Tensor:
        """Take over after a prompt pass made elsewhere (e.g. one with a padding mask): copy its recurrent states
        into the static cache and pick the first token from its last-position logits [B, V]."""
        for layer, new in zip(self.cache.states, past_key_values):
            for dst, src in zip(layer, new):
                dst.copy_(src)
        kernels.argmax_rows(last_logits, out=self.next)
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
    def step_host(self, ids_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """One decode step driven from the host: the token ids [B, 1] are read from `ids_host`, the new tokens [B] are
        written to `out_host` (both int64 in pinned memory).  The two copies and the step's kernels are one CUDA graph
        launch; the call returns once it is enqueued — synchronise the stream before reading `out_host`."""
        if not (ids_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("step_host needs pinned host buffers")
        if ids_host.shape != self.ids.shape or out_host.shape != self.next.shape or ids_host.dtype != torch.int64 \
                or out_host.dtype != torch.int64:
            raise ValueError(f"step_host needs int64 buffers of shape {tuple(self.ids.shape)} and {tuple(self.next.shape)}")
        if not self._use_graph:
            self.ids.copy_(ids_host, non_blocking=True)
            self.step()
            out_host.copy_(self.next, non_blocking=True)
            return
        key = (ids_host.data_ptr(), out_host.data_ptr())
        entry = self._host_graphs.get(key)
        if entry is None:
            entry = (self._capture(ids_host, out_host), ids_host, out_host)   # the graph keeps pointing at these buffers
            self._host_graphs = {key: entry}
        entry[0].replay()

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        toks = torch.empty(self.B, max_new_tokens, dtype=torch.int64, device=self.device)
        self.prefill(prompt_ids)
        for t in range(max_new_tokens):
            toks[:, t].copy_(self.next)
            if t + 1 < max_new_tokens:
                self.step()
        return torch.cat([prompt_ids, toks], dim=1)


class FusedRunner:
    """The HGRNBit forward as a chain of fused kernels: per block four BitLinear contractions, each fed int8
    codes by one fused row-wise kernel, plus the gated recurrence scan — eight launches per block.

    Mathematically this is HGRNBitBlock.forward / HGRNBitAttention.forward / HGRNBitMLP.forward of the module
    path with the same rounding points; the i/f/g projections, which share their input row, run as one
    grouped contraction.  Built lazily from a model; rebuilt when a weight is repacked."""

    def __init__(self, lm):
        self.lm = lm
        model = lm.model
        cfg = lm.config
        self.h = cfg.hidden_size
        self.eps = cfg.rms_norm_eps
        self.layers = []
        for blk in model.layers:
            at, mlp = blk.attn, blk.mlp
            if at.input_dim != self.h:
                raise NotImplementedError("fused path needs expand_ratio == 1")
            self.layers.append(dict(
                attn_norm_w=self._w32(blk.attn_norm.weight),
                ifg=kernels.stack_packed([at.i_proj.packed(), at.f_proj.packed(), at.g_proj.packed()]),
                ifg_nw=[at.i_proj.norm_weight_f32(), at.f_proj.norm_weight_f32(), at.g_proj.norm_weight_f32()],
                gnorm_w=self._w32(at.g_norm.weight), gnorm_eps=at.g_norm.eps,
                o=at.o_proj.packed(), o_nw=at.o_proj.norm_weight_f32(),
                mlp_norm_w=self._w32(blk.mlp_norm.weight),
                gate=mlp.gate_proj.packed(), gate_nw=mlp.gate_proj.norm_weight_f32(),
                down=mlp.down_proj.packed(), down_nw=mlp.down_proj.norm_weight_f32(),
                eps_bl=at.i_proj.NORM_EPS,
            ))
        self.final_norm_w = self._w32(model.norm.weight)
        self.head = lm.lm_head.packed()
        self.head_nw = lm.lm_head.norm_weight_f32()
        self.head_eps = lm.lm_head.NORM_EPS
        self.dtype = model.embeddings.weight.dtype
        # per-layer lower bounds of the forget gates depend on parameters only: evaluated once (in the parameter
        # dtype, with the reference's op sequence) instead of on every forward
        with torch.no_grad():
            lbs = model.layer_lower_bounds()
        self.lower_bounds = None if lbs is None else [lbs[i].contiguous() for i in range(lbs.shape[0])]
        self.key = self.fingerprint(lm)

    @staticmethod
    def _w32(w):
        return None if w is None else w.detach().float().contiguous()

    @staticmethod
    def fingerprint(lm):
        """Changes whenever a parameter is replaced, cast or modified in place.  Walking the module tree costs about
        2 ms per call on a 24-block model, so the (parameter dict, name) slots are listed once per model object and
        only looked up afterwards; a replaced parameter is still seen, because the slot is read anew."""
        slots = lm.__dict__.get("_fused_param_slots")
        if slots is None:
            slots = [(m._parameters, n) for m in lm.modules() for n in m._parameters]
            object.__setattr__(lm, "_fused_param_slots", slots)
        out = []
        for d, n in slots:
            p = d.get(n)
            if p is not None:
                out.append((p.data_ptr(), p._version, p.dtype))
        return tuple(out)

    @torch.no_grad()
    def forward(self, input_ids, inputs_embeds, states, last_only: bool, want_logits: bool = True,
                want_hidden: bool = False, attention_mask=None):
        """states: list of fp32 [B, ..., h]-shaped tensors advanced in place.  attention_mask: optional [B, T], zero at
        (left-)padding positions — their input to the recurrence is dropped, as the reference's attention layer does
        (layers/hgrn_bit.py:119-120), for a prompt inside the scan and for a single decode token inside the step kernel.
        Returns (logits | None, hidden | None)."""
        model = self.lm.model
        if inputs_embeds is None:
            x = kernels.embedding(model.embeddings.weight, input_ids)
        else:
            x = inputs_embeds.to(self.dtype)
        B, T, h = x.shape
        M = B * T
        x = x.reshape(M, h)
        lbs = self.lower_bounds
        mask = None
        if attention_mask is not None:
            mask = (attention_mask.to(x.device) != 0).to(torch.uint8).contiguous()
        stream, z = x, None                      # residual stream, last block's MLP output
        for i, L in enumerate(self.layers):
            if i == 0:
                q, dq, rs, _, _ = kernels.prenorm_quant(x, None, L["attn_norm_w"], self.eps, L["ifg_nw"], L["eps_bl"], False)
            else:   # the reference adds residual + mlp output as a tensor op, then normalises the rounded sum
                q, dq, rs, stream, _ = kernels.prenorm_quant(z, stream, L["attn_norm_w"], self.eps, L["ifg_nw"], L["eps_bl"],
                                                             True, want_residual_out=True)
            ifg = kernels.bitlinear(q, dq, rs, L["ifg"], self.dtype).view(B, T, 3 * h)
            lb = lbs[i] if (lbs is not None and i > 0) else None
            if T == 1:   # decode: gates, state update, gate-norm and o_proj's prologue in one kernel
                q, dq, rs = kernels.decode_mix(ifg.view(M, 3 * h), lb, states[i].view(B, h), L["gnorm_w"], L["gnorm_eps"],
                                               L["o_nw"], L["eps_bl"], mask=None if mask is None else mask.view(B))
            else:
                o = kernels.hgrn_gated(ifg[:, :, :h], ifg[:, :, h:2 * h], lb, states[i].view(B, h), mask=mask)
                q, dq, rs = kernels.gatenorm_quant(ifg.view(M, 3 * h)[:, 2 * h:], o.view(M, h), L["gnorm_w"], L["gnorm_eps"],
                                                   L["o_nw"], L["eps_bl"])
            attn_out = kernels.bitlinear(q, dq, rs, L["o"], self.dtype)
            q, dq, rs, stream, _ = kernels.prenorm_quant(attn_out, stream, L["mlp_norm_w"], self.eps, [L["gate_nw"]], L["eps_bl"],
                                                         False, want_residual_out=True)
            gu = kernels.bitlinear(q, dq, rs, L["gate"], self.dtype)
            q, dq, rs = kernels.swiglu_quant(gu, L["down_nw"], L["eps_bl"])
            z = kernels.bitlinear(q, dq, rs, L["down"], self.dtype)
        if z is None:                             # no blocks: final norm of the embeddings
            z_rows, s_rows, round_first = stream, None, False
        else:
            z_rows, s_rows, round_first = z, stream, True
        if last_only:                             # only the last position of every sequence feeds lm_head
            z_rows = z_rows.view(B, T, h)[:, -1]
            s_rows = None if s_rows is None else s_rows.view(B, T, h)[:, -1]
        Tn = 1 if last_only else T
        q, dq, rs, _, hidden = kernels.prenorm_quant(z_rows, s_rows, self.final_norm_w, self.eps,
                                                     [self.head_nw] if want_logits else [], self.head_eps, round_first,
                                                     want_y=want_hidden)
        logits = kernels.bitlinear(q, dq, rs, self.head, self.dtype).view(B, Tn, -1) if want_logits else None
        return logits, (hidden.view(B, Tn, h) if hidden is not None else None)


def fused_runner(lm) -> FusedRunner:
    """The model's cached FusedRunner, rebuilt if any parameter changed since it was made."""
    r = getattr(lm, "_fused_runner", None)
    if r is None or r.key != FusedRunner.fingerprint(lm):
        r = FusedRunner(lm)
        object.__setattr__(lm, "_fused_runner", r)
    return r


def bitlinear_modules(model) -> List[BitLinear]:
    """Every BitLinear of the model in execution order."""
    return [m for m in model.modules() if isinstance(m, BitLinear)]


class WeightStreamProbe:
    """Exactly the BitLinear contractions of one decode step (the grouped i/f/g projection, o, gate, down of
    every block, then lm_head), with pre-quantised activations and nothing else, replayed from a CUDA graph so
    that their device time can be measured with CUDA events."""

    def __init__(self, lm, M: int, out_dtype: torch.dtype, use_graph: bool = True):
        self._use_graph = use_graph
        runner = fused_runner(lm)
        dev = next(lm.parameters()).device
        g = torch.Generator(device=dev).manual_seed(0)
        self.items = []
        self.packed_bytes = 0
        pws = []
        for L in runner.layers:
            pws += [L["ifg"], L["o"], L["gate"], L["down"]]
        pws.append(runner.head)
        for pw in pws:
            x = torch.randn(M, pw.K, generator=g, device=dev, dtype=torch.float32).to(out_dtype)
            q, dq, rs = kernels.act_quant(x, None, 1e-6)
            if pw.groups > 1:
                q, dq, rs = q.repeat(pw.groups, 1), dq.repeat(pw.groups), rs.repeat(pw.groups)
            out = torch.empty(M, pw.N, dtype=out_dtype, device=dev)
            self.items.append((q, dq, rs, pw, out))
            self.packed_bytes += pw.packed.numel()
        self.out_dtype = out_dtype
        self.launches = len(self.items)
        self.graph = None

    def run_eager(self):
        for q, dq, rs, pw, out in self.items:
            kernels.bitlinear(q, dq, rs, pw, self.out_dtype, out=out)

    def run(self):
        if not self._use_graph:
            return self.run_eager()
        if self.graph is None:
            side = torch.cuda.Stream(device=self.items[0][0].device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):          # the capture reuses this stream's (zeroed) workspace
                self.run_eager()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                self.run_eager()
            self.graph = graph
        self.graph.replay()
