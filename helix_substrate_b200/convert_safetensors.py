"""Write a model whose linears are HelixLinear as ONE HuggingFace checkpoint:
``model.safetensors`` with {module}.codebook / .indices / .sidecar_positions /
.sidecar_values / .bias (+ .group_scales / .group_offsets) next to the dense
tensors, and ``config.json`` carrying the quantization_config that makes
``from_pretrained`` rebuild the HelixLinear shells (key layout of the reference's
tools/convert_to_hf.py:75-101,212-222)."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict

import torch
import torch.nn as nn

from .helix_linear import HelixLinear


def hxq_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """Persistent tensors only; the empty ``weight`` stubs of HelixLinear are left out."""
    helix = {n for n, m in model.named_modules() if isinstance(m, HelixLinear)}
    out = {}
    for k, v in model.state_dict().items():
        if k.endswith(".weight") and k[:-7] in helix:
            continue
        out[k] = v.detach().to("cpu").contiguous()
    return out


def save_hxq_checkpoint(model: nn.Module, out_dir, quant_method: str = "hxq") -> Path:
    from safetensors.torch import save_file
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    sd = hxq_state_dict(model)
    seen, uniq = {}, {}
    for k, v in sd.items():  # tied tensors are stored once
        key = (v.data_ptr(), v.numel(), v.dtype)
        if v.numel() and key in seen:
            continue
        seen[key] = k
        uniq[k] = v
    save_file(uniq, str(out_dir / "model.safetensors"), metadata={"format": "pt"})
    mods = {n: m for n, m in model.named_modules() if isinstance(m, HelixLinear)}
    dense = sum(m.memory_savings()["dense_bytes"] for m in mods.values())
    comp = sum(m.memory_savings()["compressed_bytes"] for m in mods.values())
    gsz = {m.group_size for m in mods.values()}
    qc = {"quant_method": quant_method, "bits": 8, "n_clusters": 256, "compressed_modules": sorted(mods),
          "compression_ratio": round(dense / max(1, comp), 2), "n_svd_routed": sum(m.has_svd for m in mods.values())}
    if gsz and gsz != {0}:
        qc["group_size"] = max(gsz)
    cfg = model.config.to_dict() if hasattr(model, "config") else {}
    cfg["quantization_config"] = qc
    (out_dir / "config.json").write_text(json.dumps(cfg, indent=2, default=str))
    return out_dir
