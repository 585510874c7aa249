"""Tensor-level wrappers around the C ABI: shape/dtype checks, output allocation, stream.

PyTorch is used here for device memory and streams only; all arithmetic happens in
libmmfree_b200.so.  Every function requires CUDA tensors and raises otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import ctypes

import torch

from . import _lib
from ._lib import BF16, F16, F32, KERNEL_AUTO, KERNEL_GEMV, KERNEL_MMA, KERNEL_STREAM, TILE_K, TILE_ROWS  # noqa: F401

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


def _code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; expected float32, bfloat16 or float16") from None


# torch.cuda.current_stream() costs about 13 us of host time per call (device-index resolution, a Stream object);
# the raw handle is available directly, and a prompt pass makes several hundred launches
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _need_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("matmulfreellm_b200 kernels take CUDA tensors only (no CPU fallback exists)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    # the C entry points launch on the CURRENT device and `_stream()` is the current device's stream: tensors of
    # another GPU would be handed to a kernel running on this one (a fault, or with peer access silently the wrong GPU)
    cur = _raw_device() if _raw_device is not None else torch.cuda.current_device()
    if dev.index is not None and dev.index != cur:
        raise RuntimeError(f"tensors live on cuda:{dev.index} but the current device is cuda:{cur}; wrap the call in "
                           f"`with torch.cuda.device({dev.index}):` (the library launches on the current device)")
    _lib.require_device(cur)
    return dev


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------------------
# packed ternary weights
# ------------------------------------------------------------------------------------------
@dataclass
class PackedWeight:
    """2-bit packed ternary weight of one BitLinear (or of `groups` BitLinears stacked along N)."""
    packed: torch.Tensor   # uint8, tile-major layout (see include/mmfree_b200.h)
    scale: torch.Tensor    # float32 [groups]: mean|w| of each group
    N: int                 # total output features (all groups)
    K: int
    groups: int = 1
    slabs: Optional[torch.Tensor] = None   # uint8, the same codes in slab-major order (read by the decode kernel)

    @property
    def device(self) -> torch.device:
        return self.packed.device


def absmean(w: torch.Tensor) -> torch.Tensor:
    """clamp(mean|w|, 1e-5) as a float32[1] tensor (fp64 accumulation, deterministic)."""
    _need_cuda(w)
    if w.dtype != torch.float32 or not w.is_contiguous():
        raise TypeError("absmean expects a contiguous float32 tensor (the fp32 latent weight)")
    partials = torch.empty(_lib.ABSMEAN_PARTIALS, dtype=torch.float64, device=w.device)
    out = torch.empty(1, dtype=torch.float32, device=w.device)
    _lib.call("mmf_absmean_f32", w.data_ptr(), w.numel(), partials.data_ptr(), out.data_ptr(), _stream())
    return out


def ensure_slabs(pw: PackedWeight) -> PackedWeight:
    """Attach the slab-major copy of the packed codes that the mma.sync decode experiment streams (one contiguous piece per
    16 output rows).  Only available inside `_lib.experiments_library()`; made on first use."""
    if pw.slabs is None or pw.slabs.device != pw.packed.device:
        _need_cuda(pw.packed)
        slabs = torch.empty_like(pw.packed)
        _lib.call("mmf_repack_slabs", pw.packed.data_ptr(), pw.N, pw.K, slabs.data_ptr(), _stream())
        pw.slabs = slabs
    return pw


def pack_weight(w: torch.Tensor) -> PackedWeight:
    """Absmean-ternarise an fp32 latent weight [N,K] and pack it (offline step)."""
    _need_cuda(w)
    if w.dim() != 2:
        raise ValueError("weight must be [N, K]")
    w = w.detach()
    if w.dtype != torch.float32:
        w = w.float()
    w = w.contiguous()
    N, K = w.shape
    if K % TILE_K:
        raise ValueError(f"in_features must be a multiple of {TILE_K}, got {K}")
    mean = absmean(w)
    nbytes = _lib.load().mmf_packed_bytes(N, K)
    packed = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    _lib.call("mmf_pack_ternary", w.data_ptr(), N, K, mean.data_ptr(), packed.data_ptr(), _stream())
    return PackedWeight(packed, mean, N, K, 1)


def stack_packed(parts: Sequence[PackedWeight]) -> PackedWeight:
    """Stack BitLinears that share their input along N so they run as one grouped launch."""
    K = parts[0].K
    n = parts[0].N
    for p in parts:
        if p.K != K or p.N != n or p.groups != 1:
            raise ValueError("grouped BitLinears need identical [N,K]")
    if n % TILE_ROWS:
        raise ValueError(f"grouped BitLinears need out_features % {TILE_ROWS} == 0")
    # the layout is tile-major at the top level, so stacking along N is concatenation
    return PackedWeight(torch.cat([p.packed for p in parts]), torch.cat([p.scale for p in parts]), n * len(parts), K,
                        len(parts))


def unpack_codes(pw: PackedWeight) -> torch.Tensor:
    """int8 ternary codes [N,K] recovered from the packed buffer."""
    codes = torch.empty(pw.N, pw.K, dtype=torch.int8, device=pw.device)
    _lib.call("mmf_unpack_ternary", pw.packed.data_ptr(), pw.N, pw.K, codes.data_ptr(), _stream())
    return codes


# ------------------------------------------------------------------------------------------
# BitLinear
# ------------------------------------------------------------------------------------------
def act_quant(x: torch.Tensor, norm_weight: Optional[torch.Tensor], eps: float, use_norm: bool = True,
              out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None):
    """RMSNorm + per-row int8 absmax quantisation of x [M,K] -> (codes int8, dq fp32[M], rowsum int32[M])."""
    _need_cuda(x, norm_weight)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be [M,K] with unit inner stride")
    M, K = x.shape
    if norm_weight is not None:
        if norm_weight.dtype != torch.float32 or norm_weight.shape != (K,) or not norm_weight.is_contiguous():
            raise TypeError("norm weight must be contiguous float32 [K]")
    if out is None:
        q = torch.empty(M, K, dtype=torch.int8, device=x.device)
        dq = torch.empty(M, dtype=torch.float32, device=x.device)
        rs = torch.empty(M, dtype=torch.int32, device=x.device)
    else:
        q, dq, rs = out
    if M == 0:
        return q, dq, rs
    _lib.call("mmf_act_quant", x.data_ptr(), _code(x.dtype), x.stride(0), _ptr(norm_weight), int(use_norm), float(eps),
              q.data_ptr(), dq.data_ptr(), rs.data_ptr(), M, K, _stream())
    return q, dq, rs


_ws_cache: dict = {}     # (device index, raw stream handle) -> current workspace of that stream
_ws_retired: list = []   # workspaces that were outgrown: never freed, because a captured CUDA graph may still point at them
_ws_bytes: dict = {}     # (M, N, K) -> mmf_bitlinear_workspace_bytes, a pure function of the shape


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised split-K workspace, one per (device, stream); kernels leave it zeroed.

    A captured CUDA graph (decode step, prompt pass) bakes in the address of the workspace it was captured with, so a
    workspace is never released once handed out: when a later call on the same stream needs a larger one, the old
    buffer is retired (kept alive) and a new one takes its place for new launches."""
    key = (device.index, _stream())
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _ws_retired.append(ws)
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


def _rezero_workspaces() -> None:
    """After a failed launch or a device-side time-out partial sums may be left behind: clear every workspace in place
    (their addresses stay valid for captured graphs)."""
    for ws in list(_ws_cache.values()) + _ws_retired:
        with torch.cuda.device(ws.device):
            ws.zero_()


def check_status() -> None:
    """Synchronise and raise if any BitLinear kernel reported a device-side wait that gave up (status word
    at the start of the split-K workspace).  Costs a device sync; meant for tests and debugging."""
    failed = ctypes.c_int(0)
    _lib.call("mmf_hgrn_status", ctypes.addressof(failed))
    if failed.value:
        raise _lib.MMFreeError("mmf_hgrn_scan", -7, "a scan kernel gave up waiting for a TMA stage")
    for ws in list(_ws_cache.values()) + _ws_retired:
        torch.cuda.synchronize(ws.device)
        status = int(ws[:4].view(torch.int32).item())
        if status != 0:
            _rezero_workspaces()
            raise _lib.MMFreeError("mmf_bitlinear", -7, f"device-side wait timed out (status word {status})")


def bitlinear(q: torch.Tensor, dq: torch.Tensor, rowsum: torch.Tensor, pw: PackedWeight, out_dtype: torch.dtype,
              kernel: int = KERNEL_AUTO, return_acc: bool = False, out: Optional[torch.Tensor] = None):
    """Integer BitLinear contraction + dequantising epilogue.

    q/dq/rowsum are [groups*M, K] / [groups*M] / [groups*M] (group-major) as produced by act_quant.
    Returns out [M, N] (and the raw int32 accumulators when return_acc).
    """
    _need_cuda(q, dq, rowsum, pw.packed)
    G = pw.groups
    if q.dtype != torch.int8 or q.dim() != 2 or not q.is_contiguous() or q.shape[1] != pw.K or q.shape[0] % G:
        raise ValueError("q must be contiguous int8 [groups*M, K]")
    M = q.shape[0] // G
    if dq.numel() != G * M or rowsum.numel() != G * M or dq.dtype != torch.float32 or rowsum.dtype != torch.int32:
        raise ValueError("dq / rowsum must be float32 / int32 [groups*M]")
    if out is None:
        out = torch.empty(M, pw.N, dtype=out_dtype, device=q.device)
    elif out.shape != (M, pw.N) or out.stride(1) != 1 or out.dtype != out_dtype:
        raise ValueError("bad `out` tensor")
    acc = torch.empty(M, pw.N, dtype=torch.int32, device=q.device) if return_acc else None
    if M == 0:
        return (out, acc) if return_acc else out
    nbytes = _ws_bytes.get((M, pw.N, pw.K))
    if nbytes is None:
        nbytes = _ws_bytes[(M, pw.N, pw.K)] = _lib.load().mmf_bitlinear_workspace_bytes(M, pw.N, pw.K)
    ws = _workspace(q.device, nbytes)
    try:
        if kernel == KERNEL_STREAM:       # the mma.sync decode experiment: exists in the experiments build only
            ensure_slabs(pw)
            _lib.call("mmf_bitlinear_decode", q.data_ptr(), dq.data_ptr(), rowsum.data_ptr(), pw.slabs.data_ptr(),
                      pw.scale.data_ptr(), G, out.data_ptr(), _code(out_dtype), out.stride(0), _ptr(acc), M, pw.N, pw.K,
                      ws.data_ptr(), _stream())
        else:
            _lib.call("mmf_bitlinear", q.data_ptr(), dq.data_ptr(), rowsum.data_ptr(), pw.packed.data_ptr(),
                      pw.scale.data_ptr(), G, out.data_ptr(), _code(out_dtype), out.stride(0), _ptr(acc), M, pw.N, pw.K,
                      ws.data_ptr(), ws.numel(), kernel, _stream())
    except _lib.MMFreeError:
        _rezero_workspaces()  # a failed launch may have left partial sums behind
        raise
    return (out, acc) if return_acc else out


# ------------------------------------------------------------------------------------------
# HGRN recurrence
# ------------------------------------------------------------------------------------------
def hgrn_scan(x: torch.Tensor, g: torch.Tensor, initial_state: Optional[torch.Tensor], output_final_state: bool,
              gate_is_log: bool, state_dtype: Optional[torch.dtype] = None, final_state_out: Optional[torch.Tensor] = None):
    """x, g: [..., T, D] contiguous; leading dims are independent sequences. Returns (o, final_state|None)."""
    _need_cuda(x, g, initial_state)
    if x.shape != g.shape or x.dim() < 2:
        raise ValueError("x and g must have the same shape [..., T, D]")
    x = x.contiguous()
    g = g.contiguous()
    *lead, T, D = x.shape
    B = 1
    for s in lead:
        B *= s
    sdt = state_dtype or (initial_state.dtype if initial_state is not None else torch.float32)
    h0 = None
    if initial_state is not None:
        if initial_state.numel() != B * D:
            raise ValueError("initial_state must hold one value per (sequence, channel)")
        h0 = initial_state.detach().to(sdt).contiguous()
    ht = None
    if output_final_state:
        ht = final_state_out if final_state_out is not None else torch.empty(*lead, D, dtype=sdt, device=x.device)
    o = torch.empty_like(x)
    nbytes = _lib.load().mmf_hgrn_workspace_bytes(B, T, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device) if nbytes else None
    _lib.call("mmf_hgrn_scan", x.data_ptr(), _code(x.dtype), g.data_ptr(), _code(g.dtype), _ptr(h0), _ptr(ht),
              _code(sdt), o.data_ptr(), B, T, D, int(gate_is_log), _ptr(ws), nbytes, _stream())
    return o, ht


def hgrn_gated(i_raw: torch.Tensor, f_raw: torch.Tensor, lower_bound: Optional[torch.Tensor], state: torch.Tensor,
               out: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated recurrence from the raw i/f projections: i_raw, f_raw are [B,T,D] views with unit inner stride
    and a common row stride (e.g. column slabs of one [B,T,3D] tensor); `state` fp32 [B,D] is advanced in
    place; returns o [B,T,D].  `mask`: optional uint8 [B,T], 0 at padding positions (their input is dropped)."""
    _need_cuda(i_raw, f_raw, state, lower_bound)
    B, T, D = i_raw.shape
    ld = i_raw.stride(1)
    if (i_raw.stride(2) != 1 or f_raw.stride(2) != 1 or f_raw.stride(1) != ld or i_raw.stride(0) != T * ld
            or f_raw.stride(0) != T * ld or f_raw.shape != i_raw.shape or f_raw.dtype != i_raw.dtype):
        raise ValueError("i_raw / f_raw must be [B,T,D] slabs of one row-major tensor")
    if state.dtype != torch.float32 or state.numel() != B * D or not state.is_contiguous():
        raise ValueError("state must be contiguous float32 with B*D elements")
    if lower_bound is not None and (lower_bound.dtype != i_raw.dtype or lower_bound.numel() != D
                                    or not lower_bound.is_contiguous()):
        raise ValueError("lower_bound must be contiguous [D] in the activation dtype")
    o = out if out is not None else torch.empty(B, T, D, dtype=i_raw.dtype, device=i_raw.device)
    nbytes = _lib.load().mmf_hgrn_workspace_bytes(B, T, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=i_raw.device) if nbytes else None
    if mask is not None and (mask.dtype != torch.uint8 or mask.shape != (B, T) or not mask.is_contiguous() or not mask.is_cuda):
        raise ValueError("mask must be a contiguous uint8 CUDA tensor [B, T]")
    _lib.call("mmf_hgrn_gated_masked", i_raw.data_ptr(), f_raw.data_ptr(), ld, _code(i_raw.dtype), _ptr(lower_bound),
              _ptr(mask), state.data_ptr(), o.data_ptr(), B, T, D, _ptr(ws), nbytes, _stream())
    return o


# ------------------------------------------------------------------------------------------
# fused producers of BitLinear inputs
# ------------------------------------------------------------------------------------------
def _codes_buffers(G: int, M: int, D: int, device):
    return (torch.empty(G * M, D, dtype=torch.int8, device=device), torch.empty(G * M, dtype=torch.float32, device=device),
            torch.empty(G * M, dtype=torch.int32, device=device))


def prenorm_quant(x: torch.Tensor, residual: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps_norm: float,
                  bl_norm_ws: Sequence[Optional[torch.Tensor]], eps_bl: float, round_sum_first: bool,
                  want_residual_out: bool = False, want_y: bool = False):
    """[x + residual] -> RMSNorm -> len(bl_norm_ws) (0, 1 or 3) BitLinear prologues.  x / residual: [M,D] with unit
    inner stride (rows may be strided).  Returns (q, dq, rowsum, residual_out | None, y | None)."""
    _need_cuda(x, residual, norm_w)
    M, D = x.shape
    G = len(bl_norm_ws)
    q = dq = rs = None
    if G:
        q, dq, rs = _codes_buffers(G, M, D, x.device)
    res_out = torch.empty(M, D, dtype=x.dtype, device=x.device) if want_residual_out else None
    y = torch.empty(M, D, dtype=x.dtype, device=x.device) if want_y else None
    nws = list(bl_norm_ws) + [None] * (3 - G)
    if M:
        _lib.call("mmf_prenorm_quant", x.data_ptr(), x.stride(0), _ptr(residual), residual.stride(0) if residual is not None else 0,
                  _code(x.dtype), int(round_sum_first), _ptr(norm_w), float(eps_norm), _ptr(res_out), _ptr(y), G,
                  _ptr(nws[0]), _ptr(nws[1]), _ptr(nws[2]), float(eps_bl), _ptr(q), _ptr(dq), _ptr(rs), M, D, _stream())
    return q, dq, rs, res_out, y


def gatenorm_quant(g: torch.Tensor, o: torch.Tensor, gnorm_w: Optional[torch.Tensor], eps_g: float,
                   bl_norm_w: Optional[torch.Tensor], eps_bl: float):
    """rmsnorm(g)*w*o*sigmoid(o) -> BitLinear prologue.  g, o: [M,D], unit inner stride, rows may be strided."""
    _need_cuda(g, o, gnorm_w, bl_norm_w)
    M, D = g.shape
    q, dq, rs = _codes_buffers(1, M, D, g.device)
    if M:
        _lib.call("mmf_gatenorm_quant", g.data_ptr(), g.stride(0), o.data_ptr(), o.stride(0), _code(g.dtype), _ptr(gnorm_w),
                  float(eps_g), _ptr(bl_norm_w), float(eps_bl), q.data_ptr(), dq.data_ptr(), rs.data_ptr(), M, D, _stream())
    return q, dq, rs


def decode_mix(ifg: torch.Tensor, lower_bound: Optional[torch.Tensor], state: torch.Tensor,
               gnorm_w: Optional[torch.Tensor], eps_g: float, bl_norm_w: Optional[torch.Tensor], eps_bl: float,
               mask: Optional[torch.Tensor] = None):
    """One decode step of the token mixer: ifg [M, 3D] = i | f | g projections of the new token of M sequences;
    `state` fp32 [M, D] is advanced in place; returns o_proj's input codes (q, dq, rowsum).  `mask`: optional uint8 [M],
    0 where the new token is padding (its input to the recurrence is dropped)."""
    _need_cuda(ifg, state, lower_bound, gnorm_w, bl_norm_w, mask)
    if mask is not None and (mask.dtype != torch.uint8 or mask.numel() != ifg.shape[0] or not mask.is_contiguous()):
        raise ValueError("mask must be a contiguous uint8 tensor with one entry per row")
    M, D3 = ifg.shape
    D = D3 // 3
    if ifg.stride(1) != 1 or state.dtype != torch.float32 or state.numel() != M * D or not state.is_contiguous():
        raise ValueError("ifg must be [M, 3D] with unit inner stride and state contiguous float32 [M, D]")
    if lower_bound is not None and (lower_bound.dtype != ifg.dtype or lower_bound.numel() != D or not lower_bound.is_contiguous()):
        raise ValueError("lower_bound must be contiguous [D] in the activation dtype")
    q, dq, rs = _codes_buffers(1, M, D, ifg.device)
    if M:
        _lib.call("mmf_decode_mix_masked", ifg.data_ptr(), ifg.stride(0), _code(ifg.dtype), _ptr(lower_bound), _ptr(mask),
                  state.data_ptr(), _ptr(gnorm_w), float(eps_g), _ptr(bl_norm_w), float(eps_bl), q.data_ptr(), dq.data_ptr(),
                  rs.data_ptr(), M, D, _stream())
    return q, dq, rs


def swiglu_quant(gate_up: torch.Tensor, bl_norm_w: Optional[torch.Tensor], eps_bl: float):
    """silu(gate)*up for gate_up = [gate | up] ([M, 2D], contiguous) -> BitLinear prologue."""
    _need_cuda(gate_up, bl_norm_w)
    M, D2 = gate_up.shape
    D = D2 // 2
    if gate_up.stride(1) != 1:
        raise ValueError("gate_up must have unit inner stride")
    q, dq, rs = _codes_buffers(1, M, D, gate_up.device)
    if M:
        es = gate_up.element_size()
        _lib.call("mmf_swiglu_quant", gate_up.data_ptr(), gate_up.data_ptr() + D * es, gate_up.stride(0), _code(gate_up.dtype),
                  _ptr(bl_norm_w), float(eps_bl), q.data_ptr(), dq.data_ptr(), rs.data_ptr(), M, D, _stream())
    return q, dq, rs


# ------------------------------------------------------------------------------------------
# norms / activations / sampling helpers
# ------------------------------------------------------------------------------------------
def _as_rows(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1]).contiguous()


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, residual: Optional[torch.Tensor] = None,
            prenorm: bool = False, residual_in_fp32: bool = False):
    """RMSNorm with the optional fused residual add; mirrors rms_norm_fn's return convention."""
    _need_cuda(x, weight, residual)
    shape = x.shape
    x2 = _as_rows(x)
    M, D = x2.shape
    w = None if weight is None else weight.detach().float().contiguous()
    res2 = None
    res_dtype = x.dtype
    if residual is not None:
        if residual.shape != shape:
            raise AssertionError("residual must have the shape of x")
        res2 = _as_rows(residual)
        res_dtype = residual.dtype
    elif residual_in_fp32:
        res_dtype = torch.float32
    if res_dtype not in (x.dtype, torch.float32):
        raise TypeError("residual dtype must equal x dtype or be float32")
    y = torch.empty_like(x2)
    need_res_out = residual is not None or res_dtype != x.dtype
    res_out = torch.empty(M, D, dtype=res_dtype, device=x.device) if need_res_out else None
    _lib.call("mmf_rmsnorm", x2.data_ptr(), _code(x.dtype), _ptr(res2), _code(res_dtype), _ptr(w), float(eps),
              y.data_ptr(), _ptr(res_out), M, D, _stream())
    y = y.reshape(shape)
    if not prenorm:
        return y
    return y, (res_out.reshape(shape) if res_out is not None else x)


def rmsnorm_swishgate(x: torch.Tensor, o: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    _need_cuda(x, o, weight)
    if x.shape != o.shape or x.dtype != o.dtype:
        raise ValueError("x and o must agree in shape and dtype")
    shape = x.shape
    x2, o2 = _as_rows(x), _as_rows(o)
    w = None if weight is None else weight.detach().float().contiguous()
    y = torch.empty_like(x2)
    _lib.call("mmf_rmsnorm_swishgate", x2.data_ptr(), o2.data_ptr(), _code(x.dtype), _ptr(w), float(eps), y.data_ptr(),
              x2.shape[0], x2.shape[1], _stream())
    return y.reshape(shape)


def swiglu(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x * sigmoid(x) * y; x and y may be strided views (e.g. the halves of a chunk(2, -1))."""
    _need_cuda(x, y)
    if x.shape != y.shape or x.dtype != y.dtype:
        raise ValueError("x and y must agree in shape and dtype")
    shape = x.shape
    D = shape[-1]

    def rows(t):
        if t.stride(-1) != 1:
            return t.contiguous().view(-1, D)
        if t.dim() == 1:
            return t.view(1, D)
        # leading dims collapse into one row index when they are uniformly strided (true for chunk() views)
        if all(t.stride(i) == t.stride(i + 1) * t.shape[i + 1] for i in range(t.dim() - 2)):
            return t.as_strided((t.numel() // D, D), (t.stride(-2), 1))
        return t.contiguous().view(-1, D)

    x2, y2 = rows(x), rows(y)
    out = torch.empty(x2.shape[0], D, dtype=x.dtype, device=x.device)
    _lib.call("mmf_swiglu", x2.data_ptr(), x2.stride(0), y2.data_ptr(), y2.stride(0), out.data_ptr(), out.stride(0),
              _code(x.dtype), x2.shape[0], D, _stream())
    return out.view(shape)


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of the maximum of every row; `out`: optional contiguous int64 tensor with one element per row."""
    _need_cuda(logits)
    l2 = logits.reshape(-1, logits.shape[-1])
    if l2.stride(1) != 1:
        l2 = l2.contiguous()
    if out is None:
        idx = torch.empty(l2.shape[0], dtype=torch.int64, device=logits.device)
    else:
        if out.dtype != torch.int64 or out.numel() != l2.shape[0] or not out.is_contiguous() or out.device != logits.device:
            raise ValueError("bad `out` tensor")
        idx = out
    if l2.shape[0]:
        _lib.call("mmf_argmax_rows", l2.data_ptr(), _code(l2.dtype), l2.stride(0), l2.shape[0], l2.shape[1],
                  idx.data_ptr(), _stream())
    return idx if out is not None else idx.reshape(logits.shape[:-1])


def sample_top_p(logits: torch.Tensor, temperature: float, top_p: float, uniforms: torch.Tensor) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) restricted to its top-p nucleus, using the caller's uniform
    numbers (float32 in [0, 1), one per row): deterministic for given inputs.  Returns int64 indices."""
    _need_cuda(logits, uniforms)
    l2 = logits.reshape(-1, logits.shape[-1])
    if l2.stride(1) != 1:
        l2 = l2.contiguous()
    if uniforms.dtype != torch.float32 or uniforms.numel() != l2.shape[0] or not uniforms.is_contiguous():
        raise ValueError("uniforms must be contiguous float32 with one value per row")
    idx = torch.empty(l2.shape[0], dtype=torch.int64, device=logits.device)
    if l2.shape[0]:
        _lib.call("mmf_sample_top_p", l2.data_ptr(), _code(l2.dtype), l2.stride(0), float(temperature), float(top_p),
                  uniforms.data_ptr(), idx.data_ptr(), l2.shape[0], l2.shape[1], _stream())
    return idx.reshape(logits.shape[:-1])


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    _need_cuda(table, ids)
    if ids.dtype != torch.int64:
        ids = ids.long()
    flat = ids.reshape(-1).contiguous()
    table = table.contiguous()
    out = torch.empty(flat.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _lib.call("mmf_embedding", table.data_ptr(), _code(table.dtype), table.shape[0], table.shape[1], flat.data_ptr(),
              out.data_ptr(), flat.numel(), _stream())
    return out.reshape(*ids.shape, table.shape[1])


def int8_mma_peak_tops(n_tokens: int = 256, iters: int = 200000) -> float:
    """Measured int8 tensor-pipe peak (TOP/s) of the current GPU: bare tcgen05.mma kind::i8 loop. Synchronises."""
    import ctypes
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.require_device(torch.cuda.current_device())
    tops = ctypes.c_double(0.0)
    torch.cuda.synchronize()
    _lib.call("mmf_int8_mma_peak", n_tokens, iters, status.data_ptr(), ctypes.addressof(tops))
    return tops.value


def sync_probe(iters: int = 2000):
    """Synchronisation costs of the current GPU in microseconds: (grid barrier among one resident CTA per SM, one-way
    flag hand-over between two CTAs, per-kernel time of a dependent chain with programmatic dependent launch, the same
    without).  Synchronises."""
    scratch = torch.zeros(256, dtype=torch.int32, device="cuda")
    _lib.require_device(torch.cuda.current_device())
    vals = [ctypes.c_double(0.0) for _ in range(4)]
    torch.cuda.synchronize()
    _lib.call("mmf_sync_probe", iters, scratch.data_ptr(), *[ctypes.addressof(v) for v in vals])
    return tuple(v.value for v in vals)
