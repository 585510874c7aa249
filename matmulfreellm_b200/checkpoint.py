"""Packed checkpoints: an HGRNBit model as it is served — 2-bit packed ternary weights plus one fp32 scale per
BitLinear, the BitLinear / block norm weights, the embedding table and the lower bounds — in one file.

The reference keeps (and ships) the fp16 latent weights and re-ternarises them on every forward
(mmfreelm/ops/fusedbitnet.py:456); a packed file is 1/8 of that for the BitLinear weights and needs no
ternarisation at load time.  Format: an uncompressed `.npz` with

    config.json                     the HGRNBitConfig as JSON (uint8 bytes)
    manifest.json                   {"format": 1, "dtype": "...", "bitlinear": {name: [N, K]}, "tensors": {name: dtype}}
    <name>.packed   uint8           tile-major 2-bit codes of BitLinear `name` (layout: include/mmfree_b200.h)
    <name>.scale    float32 [1]     mean|w| of its latent weight
    <name>.norm     float32 [K]     its RMSNorm weight
    <other>         raw             every other parameter (embeddings, norms, lower bounds); bfloat16 as uint16 bits

`save_packed(model, path)` writes it from a model whose weights are packed; `load_packed(path, device)` builds the
model on `device` without ever materialising a latent weight: each BitLinear keeps an empty `weight` and serves its
packed buffer.  A loaded model can run forward / generate; it cannot be re-packed, fine-tuned or moved to another
device (load it there instead)."""
from __future__ import annotations

import io
import json
from typing import Dict

import numpy as np
import torch
from torch import nn

from . import kernels
from .models.hgrn_bit.configuration_hgrn_bit import HGRNBitConfig
from .ops.fusedbitnet import BitLinear

FORMAT_VERSION = 1
_NP_OF = {torch.float32: np.float32, torch.float16: np.float16, torch.int64: np.int64}


def _to_numpy(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), "bfloat16"
    return t.numpy(), str(t.dtype).replace("torch.", "")


def _from_numpy(a: np.ndarray, dtype: str) -> torch.Tensor:
    if dtype == "bfloat16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


def save_packed(model, path: str) -> Dict[str, int]:
    """Write `model` (HGRNBitForCausalLM with packed weights) to `path`.  Returns {"bytes": file size, "bitlinear": count}."""
    arrays: Dict[str, np.ndarray] = {}
    bitlinear: Dict[str, list] = {}
    tensors: Dict[str, str] = {}
    skip = set()
    for name, m in model.named_modules():
        if isinstance(m, BitLinear):
            pw = m.packed()
            if pw.groups != 1:
                raise ValueError("grouped packed weights are a run-time view; save the per-module weights")
            arrays[f"{name}.packed"] = pw.packed.detach().cpu().numpy()
            arrays[f"{name}.scale"] = pw.scale.detach().cpu().numpy()
            arrays[f"{name}.norm"] = m.norm_weight_f32().detach().cpu().numpy()
            bitlinear[name] = [int(pw.N), int(pw.K)]
            skip.add(f"{name}.weight")
            skip.add(f"{name}.norm.weight")
            if m.bias is not None:
                raise ValueError("BitLinear with bias is not part of the packed format")
    dtype = None
    for name, p in model.named_parameters():
        if name in skip:
            continue
        arrays[name], tensors[name] = _to_numpy(p)
        if name.endswith("embeddings.weight"):
            dtype = tensors[name]
    manifest = {"format": FORMAT_VERSION, "dtype": dtype or "float32", "bitlinear": bitlinear, "tensors": tensors}
    arrays["config.json"] = np.frombuffer(model.config.to_json_string().encode(), dtype=np.uint8)
    arrays["manifest.json"] = np.frombuffer(json.dumps(manifest).encode(), dtype=np.uint8)
    buf = io.BytesIO()
    np.savez(buf, **arrays)
    data = buf.getvalue()
    with open(path, "wb") as f:
        f.write(data)
    return {"bytes": len(data), "bitlinear": len(bitlinear)}


def read_packed(path: str):
    """(config dict, manifest dict, arrays) of a packed checkpoint, without building a model (host only)."""
    z = np.load(path, allow_pickle=False)
    cfg = json.loads(bytes(z["config.json"]).decode())
    manifest = json.loads(bytes(z["manifest.json"]).decode())
    if manifest.get("format") != FORMAT_VERSION:
        raise ValueError(f"packed checkpoint format {manifest.get('format')} (this library reads {FORMAT_VERSION})")
    return cfg, manifest, z


def load_packed(path: str, device="cuda"):
    """Build HGRNBitForCausalLM on `device` from a packed checkpoint."""
    from .models.hgrn_bit.modeling_hgrn_bit import HGRNBitForCausalLM
    cfg_dict, manifest, z = read_packed(path)
    cfg_dict = {k: v for k, v in cfg_dict.items() if k not in ("transformers_version", "architectures", "model_type")}
    config = HGRNBitConfig(**cfg_dict)
    device = torch.device(device)
    dtype = getattr(torch, manifest["dtype"])
    # build the skeleton on the meta device: no latent weight is ever allocated
    with torch.device("meta"):
        model = HGRNBitForCausalLM(config)
    model = model.to_empty(device=device).eval()
    modules = dict(model.named_modules())
    with torch.no_grad():
        for name, (N, K) in manifest["bitlinear"].items():
            m = modules[name]
            if (m.out_features, m.in_features) != (N, K):
                raise ValueError(f"{name}: checkpoint has [{N}, {K}], the config builds [{m.out_features}, {m.in_features}]")
            m.weight = nn.Parameter(torch.empty(0, device=device, dtype=dtype), requires_grad=False)
            m._packed = kernels.PackedWeight(torch.from_numpy(z[f"{name}.packed"].copy()).to(device),
                                             torch.from_numpy(z[f"{name}.scale"].copy()).to(device), N, K, 1)
            m._packed_from = None
            m.norm.weight = nn.Parameter(torch.from_numpy(z[f"{name}.norm"].copy()).to(device=device, dtype=dtype),
                                         requires_grad=False)
        params = dict(model.named_parameters())
        for name, dt in manifest["tensors"].items():
            src = _from_numpy(z[name], dt).to(device)
            p = params[name]
            if p.shape != src.shape:
                raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} != model shape {tuple(p.shape)}")
            p.data = src.to(dtype if p.is_floating_point() else p.dtype)
    return model
