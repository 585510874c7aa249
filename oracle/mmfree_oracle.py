"""CPU oracle for the MatMul-free LM inference hot path.  TEST INFRASTRUCTURE, NOT PRODUCT.

This module restates, in plain PyTorch-on-CPU and numpy, the algorithm of the reference
project (ridgerchu/matmulfreellm, package `mmfreelm`) for the path the CUDA library
replaces.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
it, and only as the checker; nothing under matmulfreellm_b200/ imports it.

Pinning: tests/test_oracle_golden.py checks every function here against fixtures under
tests/golden/ that were produced by running the reference's own pure-PyTorch functions
(activation_quant, weight_quant, rms_norm_ref, naive_recurrent_hgrn and the HGRNBit model with
its GPU-only leaves swapped for those functions) — see tests/golden/make_golden.py.

Two restatements of BitLinear live here:
  * the FLOAT path (`bitlinear_ref`) follows the reference line by line;
  * the INTEGER path (`ternary_codes`, `act_codes`, `bitlinear_int`) is the same arithmetic
    with the quantised values kept as integer codes.  It fixes the order of the few fp32
    operations involved (documented per function) so that a GPU kernel can match the codes
    bit for bit; sums of squares and of |w| are accumulated in fp64 so their value does not
    depend on summation order.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

TILE_ROWS, TILE_K = 128, 64


# ------------------------------------------------------------------------------------------
# float restatements (reference line by line)
# ------------------------------------------------------------------------------------------
def activation_quant(x: torch.Tensor) -> torch.Tensor:
    """mmfreelm/ops/fusedbitnet.py:15-29 — per-token absmax fake quantisation to int8."""
    scale = 127.0 / x.abs().max(dim=-1, keepdim=True).values.clamp(min=1e-5)
    return (x * scale).round().clamp(-128, 127) / scale


def weight_quant(w: torch.Tensor) -> torch.Tensor:
    """mmfreelm/ops/fusedbitnet.py:32-46 — per-tensor absmean fake quantisation to {-1,0,1}/scale."""
    scale = 1.0 / w.abs().mean().clamp(min=1e-5)
    return (w * scale).round().clamp(-1, 1) / scale


def rms_norm_ref(x, weight, bias=None, residual=None, eps=1e-6, prenorm=False):
    """mmfreelm/modules/layernorm.py:73-87 (identical copy at modules/fused_norm_gate.py:37-51).

    With a residual the reference's Triton kernel (layernorm.py:139-145) normalises the fp32
    sum and rounds only the stored residual_out; for fp32 tensors both readings agree. The
    kernel's reading is restated here because that is what runs on a GPU.
    """
    dtype = x.dtype
    xf = x.float()
    res_out = None
    if residual is not None:
        xf = xf + residual.float()
        res_out = xf.to(residual.dtype)
    rstd = 1 / torch.sqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    out = xf * rstd * weight.float() if weight is not None else xf * rstd
    if bias is not None:
        out = out + bias.float()
    out = out.to(dtype)
    if not prenorm:
        return out
    return out, (res_out if res_out is not None else x)


def swish_gate_norm_ref(x, o, weight, eps=1e-6):
    """mmfreelm/modules/fused_norm_gate.py:101-131 — y = rmsnorm(x)*w * o * sigmoid(o), fp32 math."""
    xf, of = x.float(), o.float()
    rstd = 1 / torch.sqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    y = xf * rstd * weight.float()
    return (y * of * torch.sigmoid(of)).to(x.dtype)


def swiglu_ref(x, y):
    """mmfreelm/modules/activations.py:115-119 — float(x)*float(y)/(1+exp(-float(x))) cast back."""
    xf, yf = x.float(), y.float()
    return (xf * yf / (1.0 + torch.exp(-xf))).to(x.dtype)


def bitlinear_ref(x, norm_weight, weight, eps=1e-8):
    """mmfreelm/ops/fusedbitnet.py:558-581 — BitLinear.forward: norm -> act quant -> weight quant -> F.linear.

    eps: 1e-8 for BitLinear (its RMSNorm module, fusedbitnet.py:556); FusedBitLinear's fused
    call uses 1e-6 (default of layer_norm_linear_quant_fn, fusedbitnet.py:520, not overridden
    at :603-610).  weight_quant is evaluated on every call, as in the reference (:456, :577).
    """
    x_norm = rms_norm_ref(x, norm_weight, eps=eps)
    # the straight-through form of :576-577 is kept: x + (q(x) - x) is not bitwise q(x) in fp32
    x_quant = x_norm + (activation_quant(x_norm) - x_norm)
    w_quant = weight + (weight_quant(weight) - weight)
    return F.linear(x_quant, w_quant)


def naive_recurrent_hgrn(x, g, initial_state=None, output_final_state=False):
    """mmfreelm/ops/hgrn/naive.py:8-31 — h_t = g_t*h_{t-1} + x_t, g in the linear domain, fp32 state.

    x, g: [B, H, T, D].  Returns (o in x.dtype, fp32 final state or None)."""
    dtype = x.dtype
    xf, gf = x.float(), g.float()
    B, H, T, D = xf.shape
    h = torch.zeros(B, H, D, dtype=torch.float32)
    if initial_state is not None:
        h = h + initial_state.detach().float().reshape(B, H, D)
    o = torch.empty_like(xf)
    for t in range(T):
        h = gf[:, :, t] * h + xf[:, :, t]
        o[:, :, t] = h
    return o.to(dtype), (h if output_final_state else None)


def chunk_hgrn_ref(x, g_log, initial_state=None, output_final_state=False):
    """mmfreelm/ops/hgrn/chunk.py:49-116, :287-296 — same recurrence with a LOG forget gate:
    h_t = exp(g_t)*h_{t-1} + x_t, i.e. naive_recurrent_hgrn(x, exp(g))."""
    return naive_recurrent_hgrn(x, torch.exp(g_log.float()), initial_state, output_final_state)


# ------------------------------------------------------------------------------------------
# integer restatement (bit-exact contract with the CUDA kernels)
# ------------------------------------------------------------------------------------------
def absmean(w: torch.Tensor) -> np.float32:
    """clamp(mean|w|, 1e-5): |w| summed in fp64, divided in fp64, rounded once to fp32."""
    wn = w.detach().float().numpy()
    m = np.float32(np.sum(np.abs(wn), dtype=np.float64) / wn.size)
    return np.maximum(m, np.float32(1e-5))


def ternary_codes(w: torch.Tensor) -> Tuple[np.ndarray, np.float32]:
    """weight_quant as codes: clamp(rint(w * (1/mean)), -1, 1) with fp32 `1/mean` and fp32 product."""
    wn = w.detach().float().numpy()
    mean = absmean(w)
    scale = np.float32(1.0) / mean
    codes = np.clip(np.rint(wn * scale), -1, 1).astype(np.int8)
    return codes, mean


def pack_ternary(codes: np.ndarray) -> np.ndarray:
    """The 2-bit tile-major layout the CUDA library stores (uint32 words).

    tile t (128 rows), chunk c (64 columns), row r -> 4 words at ((t*KC + c)*128 + r)*4;
    word q covers columns c*64 + q*16 + j, j in 0..15, at bit field f = j//4 + 4*(j%4);
    field value = code + 1; rows beyond N hold code 0."""
    N, K = codes.shape
    assert K % TILE_K == 0
    tiles, KC = -(-N // TILE_ROWS), K // TILE_K
    padded = np.zeros((tiles * TILE_ROWS, K), dtype=np.int64)
    padded[:N] = codes
    fields = (padded + 1).reshape(tiles, TILE_ROWS, KC, 4, 16)           # [t, r, c, q, j]
    j = np.arange(16)
    shift = 2 * (j // 4 + 4 * (j % 4))
    words = np.sum(fields << shift, axis=-1).astype(np.uint32)             # [t, r, c, q]
    return np.ascontiguousarray(words.transpose(0, 2, 1, 3)).reshape(-1)   # [t, c, r, q]


def act_codes(x: torch.Tensor, norm_weight: Optional[torch.Tensor], eps: float, use_norm: bool = True):
    """RMSNorm + activation_quant as codes.  x: [M,K] (any float dtype; widened exactly to fp32).

    rstd = 1/sqrt(float32(sum_fp64(x^2)/K) + eps)    (fp32 add, sqrt, divide)
    y    = (x*rstd)*w                                 (two fp32 products, in this order)
    a    = max(max|y|, 1e-5);  s = 127/a              (fp32 divide)
    q    = clamp(rint(y*s), -128, 127);  dq = a/127;  rowsum = sum(q)
    Returns (q int8 [M,K], dq float32 [M], rowsum int32 [M])."""
    xn = x.detach().float().numpy()
    M, K = xn.shape
    if use_norm:
        ss = np.sum(xn.astype(np.float64) ** 2, axis=-1)
        mean = (ss / K).astype(np.float32)
        rstd = np.float32(1.0) / np.sqrt(mean + np.float32(eps))
        y = xn * rstd[:, None]
        if norm_weight is not None:
            y = y * norm_weight.detach().float().numpy()[None, :]
    else:
        y = xn
    a = np.maximum(np.abs(y).max(axis=-1), np.float32(1e-5)).astype(np.float32)
    s = np.float32(127.0) / a
    q = np.clip(np.rint(y * s[:, None]), -128, 127).astype(np.int8)
    dq = (a / np.float32(127.0)).astype(np.float32)
    return q, dq, q.astype(np.int32).sum(axis=-1).astype(np.int32)


def bitlinear_acc(q: np.ndarray, codes: np.ndarray) -> np.ndarray:
    """int32 accumulators q[M,K] . codes[N,K]^T (exact; |acc| <= 127*K < 2^24 so fp32 BLAS is exact too)."""
    acc = q.astype(np.float32) @ codes.astype(np.float32).T
    return np.rint(acc).astype(np.int32)


def bitlinear_int(x: torch.Tensor, norm_weight, codes: np.ndarray, mean: np.float32, eps: float,
                  out_dtype: torch.dtype = torch.float32, use_norm: bool = True):
    """Integer BitLinear: out = float32(acc) * (dq * mean), rounded to out_dtype.  Returns (out, acc, q, dq)."""
    shape = x.shape
    q, dq, _ = act_codes(x.reshape(-1, shape[-1]), norm_weight, eps, use_norm)
    acc = bitlinear_acc(q, codes)
    out = acc.astype(np.float32) * (dq * np.float32(mean))[:, None]
    out_t = torch.from_numpy(out).to(out_dtype).reshape(*shape[:-1], codes.shape[0])
    return out_t, acc, q, dq


# ------------------------------------------------------------------------------------------
# HGRNBit model (mmfreelm/models/hgrn_bit/modeling_hgrn_bit.py, mmfreelm/layers/hgrn_bit.py)
# ------------------------------------------------------------------------------------------
@dataclass
class OracleConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    num_hidden_layers: int = 24
    intermediate_size: Optional[int] = None
    hidden_ratio: int = 4
    rms_norm_eps: float = 1e-6
    use_lower_bound: bool = True

    def __post_init__(self):
        if self.intermediate_size is None:  # modeling_hgrn_bit.py:45-47
            i = int(self.hidden_size * self.hidden_ratio * 2 / 3)
            self.intermediate_size = 256 * ((i + 255) // 256)


def random_weights(cfg: OracleConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded fp32 state dict with the reference's key names: projections, lm_head and embeddings
    N(0, 0.02); norm weights 1; lower_bounds 0."""
    g = torch.Generator().manual_seed(seed)
    h, I, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers

    def n(*shape):
        return torch.randn(*shape, generator=g) * 0.02

    sd = {"model.embeddings.weight": n(V, h), "model.lower_bounds": torch.zeros(L, h)}
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "attn_norm.weight"] = torch.ones(h)
        for name in ("i_proj", "f_proj", "g_proj", "o_proj"):
            sd[p + f"attn.{name}.weight"] = n(h, h)
            sd[p + f"attn.{name}.norm.weight"] = torch.ones(h)
        sd[p + "attn.g_norm.weight"] = torch.ones(h)
        sd[p + "mlp_norm.weight"] = torch.ones(h)
        sd[p + "mlp.gate_proj.weight"] = n(2 * I, h)
        sd[p + "mlp.gate_proj.norm.weight"] = torch.ones(h)
        sd[p + "mlp.down_proj.weight"] = n(h, I)
        sd[p + "mlp.down_proj.norm.weight"] = torch.ones(I)
    sd["model.norm.weight"] = torch.ones(h)
    sd["lm_head.weight"] = n(V, h)
    sd["lm_head.norm.weight"] = torch.ones(h)
    return sd


class OracleHGRNBit:
    """HGRNBitForCausalLM forward + greedy decoding on CPU.

    dtype: activation dtype (float32 or bfloat16); every tensor the reference materialises is
        rounded to it at the same point (torch CPU ops compute in fp32 and round once).
    linear: 'int'   — BitLinear through the integer restatement, weights ternarised ONCE from the
                      fp32 latent (this is what the CUDA path implements);
            'float' — BitLinear.forward as the reference runs it (weight_quant on every call,
                      fp32 F.linear); used to pin against the reference and as the CPU baseline.
    The recurrent state is kept in fp32 in both modes (naive_recurrent_hgrn, naive.py:16,29).

    Quantisation makes the model discontinuous: an input perturbation of one fp32 ulp can move an
    activation across a rounding tie and change one int8 code, which shifts that token's outputs by about
    dq*mean|w| (~5e-4 here).  Two correct implementations therefore agree per op to fp32 accuracy but
    only to ~1e-3 on logits after a few layers.
    """
    def __init__(self, cfg: OracleConfig, weights: Dict[str, torch.Tensor], dtype=torch.float32, linear="int",
                 bitlinear_eps: float = 1e-6):
        # bitlinear_eps: 1e-6 is what FusedBitLinear.forward uses on a GPU (default eps of
        # layer_norm_linear_quant_fn, fusedbitnet.py:520, not overridden at :603-610); 1e-8 is what
        # BitLinear.forward uses through its RMSNorm module (fusedbitnet.py:556) — the only variant of
        # the reference that runs on a CPU, hence the one the golden fixtures were made with.
        self.cfg, self.dtype, self.linear = cfg, dtype, linear
        self.BITLINEAR_EPS = bitlinear_eps
        self.w = {k: v.detach().float() for k, v in weights.items()}
        self._codes: Dict[str, Tuple[np.ndarray, np.float32]] = {}
        lb = self.w["model.lower_bounds"].to(dtype)
        if lb.shape[0]:
            lb = lb.softmax(0)                   # modeling_hgrn_bit.py:231-233
            lb = lb.cumsum(0) - lb[0]
        self.lower_bounds = lb

    # -- leaves -------------------------------------------------------------------------
    def _bl(self, x: torch.Tensor, name: str) -> torch.Tensor:
        nw = self.w[name + ".norm.weight"]
        if self.linear == "float":
            return bitlinear_ref(x.float(), nw, self.w[name + ".weight"], eps=self.BITLINEAR_EPS).to(self.dtype)
        if name not in self._codes:
            self._codes[name] = ternary_codes(self.w[name + ".weight"])
        codes, mean = self._codes[name]
        return bitlinear_int(x, nw, codes, mean, self.BITLINEAR_EPS, out_dtype=self.dtype)[0]

    # -- forward ------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, states: Optional[List[torch.Tensor]] = None,
                last_only: bool = False):
        """input_ids [B,T] -> (logits [B,T,V] (or [B,1,V] if last_only), states: L x fp32 [B,1,h])."""
        cfg, dt = self.cfg, self.dtype
        B, T = input_ids.shape
        h = self.w["model.embeddings.weight"].to(dt)[input_ids]
        if states is None:
            states = [torch.zeros(B, 1, cfg.hidden_size) for _ in range(cfg.num_hidden_layers)]
        new_states = []
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            residual = h
            x = rms_norm_ref(h, self.w[p + "attn_norm.weight"], eps=cfg.rms_norm_eps)          # block :98
            # HGRNBitAttention.forward, layers/hgrn_bit.py:110-140
            ii = self._bl(x, p + "attn.i_proj")
            f = self._bl(x, p + "attn.f_proj").sigmoid()
            if cfg.use_lower_bound and i > 0:
                lb = self.lower_bounds[i]
                f = lb + (1 - lb) * f
            ii = swiglu_ref(ii, 1 - f)
            o, st = naive_recurrent_hgrn(ii.unsqueeze(1), f.unsqueeze(1), states[i], True)     # [B,1,T,h]
            new_states.append(st)
            o = swish_gate_norm_ref(self._bl(x, p + "attn.g_proj"), o.squeeze(1), self.w[p + "attn.g_norm.weight"],
                                    eps=cfg.rms_norm_eps)
            o = self._bl(o, p + "attn.o_proj")
            # block :107-109
            h2, residual = rms_norm_ref(o, self.w[p + "mlp_norm.weight"], residual=residual, eps=cfg.rms_norm_eps,
                                        prenorm=True)
            y = self._bl(h2, p + "mlp.gate_proj")                                              # MLP :55-59
            gate, y = y.chunk(2, -1)
            z = self._bl(swiglu_ref(gate, y), p + "mlp.down_proj")
            h = residual + z
        h = rms_norm_ref(h, self.w["model.norm.weight"], eps=cfg.rms_norm_eps)
        if last_only:
            h = h[:, -1:]
        logits = self._bl(h, "lm_head")
        return logits, new_states

    def greedy(self, input_ids: torch.Tensor, steps: int):
        """Prefill, then `steps` greedy tokens. Returns (tokens [B,steps], per-step top-2 logit margins [B,steps])."""
        logits, states = self.forward(input_ids, last_only=True)
        toks, margins = [], []
        for _ in range(steps):
            last = logits[:, -1].float()
            top2 = last.topk(2, dim=-1).values
            margins.append(top2[:, 0] - top2[:, 1])
            nxt = last.argmax(-1)
            toks.append(nxt)
            logits, states = self.forward(nxt[:, None], states, last_only=True)
        return torch.stack(toks, 1), torch.stack(margins, 1)


# ------------------------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ------------------------------------------------------------------------------------------
def bitlinear_case(M: int, K: int, N: int, seed: int = 0, dtype=torch.bfloat16):
    """x ~ N(0,1) with K//100 outlier channels scaled x20, cast to `dtype`; latent w ~ 0.02*N(0,1) fp32; norm weight 1."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    cols = torch.randperm(K, generator=g)[: K // 100]
    x[:, cols] *= 20
    w = torch.randn(N, K, generator=g) * 0.02
    return x.to(dtype), w, torch.ones(K)


def hgrn_case(B: int, T: int, D: int, seed: int = 0, dtype=torch.bfloat16):
    """g_log = logsigmoid(N(0,1)) fp32; x = (1-exp(g_log))*silu(N(0,1)) cast to `dtype`. Shapes [B,1,T,D]."""
    g = torch.Generator().manual_seed(seed)
    g_log = F.logsigmoid(torch.randn(B, 1, T, D, generator=g))
    x = ((1 - torch.exp(g_log)) * F.silu(torch.randn(B, 1, T, D, generator=g))).to(dtype)
    return x, g_log

def nucleus_ref(logits, temperature: float, top_p: float):
    """What the reference's `model.generate(do_sample=True, top_p=..., temperature=...)` (generate.py:11) asks of
    transformers before it draws: TemperatureLogitsWarper (logits / temperature) then TopPLogitsWarper (keep the most
    probable tokens up to and including the one at which the kept mass reaches top_p, i.e. drop a token when the mass
    of the strictly more probable ones is already >= top_p; at least one token stays).  Tokens exactly as probable as
    the least probable kept one are all kept.  Returns (kept bool [M,V], unnormalised fp64 weights [M,V] of the
    tempered softmax, boundary margin [M]: distance of top_p from the nearest cumulative-mass step, relative to the
    total mass).  Pinned against transformers' own warpers in tests/test_oracle_golden.py."""
    z = np.asarray(logits, dtype=np.float32) * np.float32(1.0 / temperature)
    p = np.exp((z - z.max(-1, keepdims=True)).astype(np.float32)).astype(np.float64)
    kept = np.zeros(p.shape, dtype=bool)
    margin = np.zeros(p.shape[0])
    for m in range(p.shape[0]):
        row = p[m]
        total = row.sum()
        order = np.argsort(-row, kind="stable")
        csum = np.cumsum(row[order])
        want = min(top_p, 1.0) * total
        k = int(np.searchsorted(csum, want, side="left"))          # first position with csum >= want
        k = min(k, len(row) - 1)
        kept[m] = row >= row[order[k]]
        margin[m] = (np.abs(csum[:-1] - want).min() / total) if top_p < 1.0 and len(row) > 1 else np.inf
    return kept, p, margin


def sample_top_p_ref(logits, temperature: float, top_p: float, uniforms):
    """Nucleus sampling with caller-supplied uniform numbers: the kept set and weights of `nucleus_ref`, then a draw
    by inverse CDF in token order — the first kept token whose running kept mass exceeds u * kept mass (the
    multinomial draw of transformers' sampling loop, made deterministic by taking the uniform number as an input).
    Returns (tokens int64 [M], margin [M]) where margin is the distance of u * kept mass to the nearest CDF step and
    of top_p to the nearest nucleus step, relative to the total mass (rows with a tiny margin are ill-conditioned)."""
    kept_all, p, nucleus = nucleus_ref(logits, temperature, top_p)
    out = np.zeros(p.shape[0], dtype=np.int64)
    margin = np.zeros(p.shape[0])
    for m in range(p.shape[0]):
        row, kept = p[m], kept_all[m]
        total = row.sum()
        c = np.cumsum(np.where(kept, row, 0.0))
        target = float(uniforms[m]) * c[-1]
        idx = int(np.searchsorted(c, target, side="right"))        # first index with c > target
        idx = min(idx, len(row) - 1)
        while not kept[idx]:
            idx += 1
        out[m] = idx
        margin[m] = min(np.abs(c[kept] - target).min() / total, nucleus[m])
    return out, margin


def greedy_parity(oracle: "OracleHGRNBit", ids: torch.Tensor, steps: int, decoder, prompt_logits) -> dict:
    """Greedy decoding of a device implementation against this oracle, with the allowance for divergence MEASURED in
    the same run instead of assumed.

    `decoder` is any object with `prefill(ids_on_device) -> first tokens`, `step() -> next tokens` (feeding its own
    arg-max back through `decoder.ids` [B,1]), and after a step `decoder.last_logits` [B,V]; `prompt_logits(ids)`
    returns the device implementation's logits [B,V] for the last prompt position.

    1. The oracle decodes freely: tokens, logits and top-2 margin of every step.
    2. Teacher-forced pass: the decoder is fed the ORACLE's tokens; err[b,t] = max over the vocabulary of the logit
       difference at that step.  Rows with err 0 are bit-identical to the oracle's.
    3. Free-running pass: the decoder feeds itself.  Until a sequence first differs from the oracle, its computation
       is the teacher-forced one, so at the first differing step t* the two arg-maxes can only disagree if
       margin[b,t*] <= 2*err[b,t*]; a sequence that differs anywhere else has a wrong token.  After t* the sequence
       follows another path and is not compared further.
    Returns a dict: `explained` (every first difference satisfies the inequality), `violations` (list of (b, t*, margin,
    err)), `identical_fraction` (over all B*steps tokens), `identical_sequences`, `err_median`, `err_max` (over rows),
    `exact_rows` (fraction of rows with err == 0), `min_margin`."""
    B = ids.shape[0]
    dev = decoder.ids.device
    logits, states = oracle.forward(ids, last_only=True)
    ref_tokens, ref_logits, margins = [], [], []
    for _ in range(steps):
        last = logits[:, -1].float()
        top2 = last.topk(2, dim=-1).values
        margins.append(top2[:, 0] - top2[:, 1])
        ref_logits.append(last)
        nxt = last.argmax(-1)
        ref_tokens.append(nxt)
        logits, states = oracle.forward(nxt[:, None], states, last_only=True)
    ref_tokens, margins = torch.stack(ref_tokens, 1), torch.stack(margins, 1)

    err = torch.zeros(B, steps)
    decoder.prefill(ids.to(dev))
    err[:, 0] = (prompt_logits(ids).float().cpu() - ref_logits[0]).abs().amax(-1)
    for t in range(steps - 1):
        decoder.ids.copy_(ref_tokens[:, t:t + 1].to(dev))
        decoder.step()
        err[:, t + 1] = (decoder.last_logits.float().cpu() - ref_logits[t + 1]).abs().amax(-1)

    toks = [decoder.prefill(ids.to(dev)).clone().cpu()]
    for _ in range(steps - 1):
        toks.append(decoder.step().clone().cpu())
    toks = torch.stack(toks, 1)
    same = toks == ref_tokens
    violations, full = [], 0
    for b in range(B):
        if bool(same[b].all()):
            full += 1
            continue
        t = int(torch.nonzero(~same[b])[0])
        if not float(margins[b, t]) <= 2.0 * float(err[b, t]):
            violations.append((b, t, float(margins[b, t]), float(err[b, t])))
    return {"explained": not violations, "violations": violations, "identical_fraction": same.float().mean().item(),
            "identical_sequences": full, "err_median": err.median().item(), "err_max": err.max().item(),
            "exact_rows": (err == 0).float().mean().item(), "min_margin": margins.min().item()}
