"""ONE HuggingFace checkpoint out of an HXQ model: ``model.safetensors`` with
{module}.codebook / .indices / .sidecar_positions / .sidecar_values / .bias
(+ .group_scales / .group_offsets) next to the dense tensors, and ``config.json``
carrying the quantization_config that makes ``from_pretrained`` rebuild the
HelixLinear shells (key layout of the reference's tools/convert_to_hf.py:75-101,212-222).

Two sources: a live model whose linears are HelixLinear (``save_hxq_checkpoint``), or a
directory of ``*.cdnav3`` tensor folders and exact ``*.npy`` tensors as CDNAv3Writer
leaves it (``convert_cdnav3_to_safetensors`` / ``convert_model``, the reference's
helix_substrate/convert_safetensors.py:156-353), the second with the reference tool's
completeness gate: every tensor of the original dense checkpoint must be present or
replaced by its compressed parts, or the conversion fails
(tools/convert_to_hf.py:131-190)."""

from __future__ import annotations

import json
import shutil
import time
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np

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


# --------------------------------------------------------------------------- from a .cdnav3 directory

_TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "special_tokens_map.json",
                    "added_tokens.json", "generation_config.json", "vocab.json", "merges.txt")
_PART_SUFFIXES = (".codebook", ".indices", ".sidecar_positions", ".sidecar_values", ".group_scales", ".group_offsets")


def _module_of(tensor_name: str) -> str:
    return tensor_name[:-len(".weight")] if tensor_name.endswith(".weight") else tensor_name


def _read_cdnav3_tensor(tensor_dir: Path) -> Optional[Dict[str, torch.Tensor]]:
    """The parts of one ``*.cdnav3`` folder under their checkpoint keys; None for folders that hold
    no scalar-codebook tensor (no meta, or storage_mode "exact")."""
    meta_path = tensor_dir / "meta.json"
    if not meta_path.exists():
        return None
    meta = json.loads(meta_path.read_text())
    if meta.get("storage_mode") == "exact":
        return None
    if int(meta.get("vector_dim", 1)) != 1 or meta.get("index_dtype", "uint8") != "uint8":
        raise NotImplementedError(f"{tensor_dir.name}: only scalar codebooks with uint8 indices are on this path")
    rows, cols = (int(v) for v in meta["shape"])
    mod = _module_of(meta["tensor_name"])
    idx = np.fromfile(tensor_dir / "indices.bin", dtype=np.uint8)
    if idx.size != rows * cols:
        raise ValueError(f"{tensor_dir.name}: indices.bin holds {idx.size} entries, meta.json says {rows} x {cols}")
    out = {f"{mod}.codebook": torch.from_numpy(np.load(tensor_dir / "codebook.npy").astype(np.float32)),
           f"{mod}.indices": torch.from_numpy(idx.reshape(rows, cols).copy())}
    sc = tensor_dir / "sidecar.npz"
    if sc.exists():
        with np.load(sc) as z:
            out[f"{mod}.sidecar_positions"] = torch.from_numpy(z["positions"].astype(np.int64))
            out[f"{mod}.sidecar_values"] = torch.from_numpy(z["values"].astype(np.float32))
    if (tensor_dir / "group_scales.npy").exists():
        out[f"{mod}.group_scales"] = torch.from_numpy(np.load(tensor_dir / "group_scales.npy").astype(np.float32))
        out[f"{mod}.group_offsets"] = torch.from_numpy(np.load(tensor_dir / "group_offsets.npy").astype(np.float32))
    out["__module__"] = mod
    out["__group_size__"] = int(meta.get("group_size", 0))
    return out


def _original_shards(model_dir: Path) -> List[Path]:
    return sorted(Path(model_dir).glob("model*.safetensors"))


def convert_cdnav3_to_safetensors(cdnav3_dir, output_path, original_model_path=None) -> dict:
    """Every ``*.cdnav3`` folder and exact ``*.npy`` tensor of ``cdnav3_dir`` into one safetensors
    file.  ``original_model_path``: the dense checkpoint (a file, or a directory of shards) the
    tensors the writer skipped are copied from in their native dtype - and against which the
    result is checked: a tensor of the dense model that is neither present nor replaced by a
    compressed module's parts raises RuntimeError.  Returns the conversion statistics."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    cdnav3_dir, output_path = Path(cdnav3_dir), Path(output_path)
    tensors: Dict[str, torch.Tensor] = {}
    modules: List[str] = []
    group_sizes = set()
    for d in sorted(cdnav3_dir.glob("*.cdnav3")):
        if not d.is_dir():
            continue
        parts = _read_cdnav3_tensor(d)
        if parts is None:
            continue
        modules.append(parts.pop("__module__"))
        group_sizes.add(parts.pop("__group_size__"))
        tensors.update(parts)
    n_exact = 0
    for meta_path in sorted(cdnav3_dir.glob("*.npy.meta.json")):
        name = json.loads(meta_path.read_text()).get("tensor_name", "")
        npy = meta_path.with_name(meta_path.name[:-len(".meta.json")])
        if name and npy.exists():
            tensors[name] = torch.from_numpy(np.load(npy))      # native dtype (fp16 from this writer)
            n_exact += 1
    n_copied, n_dense = 0, 0
    if original_model_path is not None:
        src = Path(original_model_path)
        shards = _original_shards(src) if src.is_dir() else [src]
        replaced = {m + ".weight" for m in modules}
        missing = []
        for shard in shards:
            with safe_open(str(shard), framework="pt") as f:
                for k in f.keys():
                    n_dense += 1
                    if k in tensors or k in replaced:
                        continue
                    tensors[k] = f.get_tensor(k)
                    n_copied += 1
        # completeness gate: what the dense model has, the checkpoint has - as itself, with the dense
        # tensor's shape, or as the parts of a compressed module whose index matrix has that shape
        # (a stale folder from another model, or an exact tensor of the wrong size, stops here)
        for shard in shards:
            with safe_open(str(shard), framework="pt") as f:
                for k in f.keys():
                    shape = tuple(f.get_slice(k).get_shape())
                    if k in tensors:
                        if tuple(tensors[k].shape) != shape:
                            missing.append(f"{k}: shape {tuple(tensors[k].shape)} != dense {shape}")
                        continue
                    m = _module_of(k)
                    idx = tensors.get(f"{m}.indices")
                    if k not in replaced or idx is None or f"{m}.codebook" not in tensors:
                        missing.append(f"{k}: absent")
                    elif int(np.prod(shape)) != idx.numel() or shape[-1] != idx.shape[-1]:
                        missing.append(f"{k}: compressed as {tuple(idx.shape)}, dense {shape}")
        if missing:
            raise RuntimeError(f"completeness gate: {len(missing)} tensors of the dense model are not accounted for, "
                               f"e.g. {sorted(missing)[:5]}")
    for m in modules:   # every compressed module is whole
        idx, cb = tensors[f"{m}.indices"], tensors[f"{m}.codebook"]
        if idx.dtype != torch.uint8 or idx.ndim != 2 or cb.ndim != 1 or cb.numel() > 256:
            raise RuntimeError(f"{m}: malformed codebook / indices")
        if (f"{m}.sidecar_positions" in tensors) != (f"{m}.sidecar_values" in tensors):
            raise RuntimeError(f"{m}: sidecar positions and values must come together")
        if f"{m}.sidecar_positions" in tensors:
            pos = tensors[f"{m}.sidecar_positions"]
            if pos.numel() and (int(pos.max()) >= idx.numel() or bool((pos[1:] <= pos[:-1]).any())):
                raise RuntimeError(f"{m}: sidecar positions must be ascending and inside the matrix")
    output_path.parent.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(output_path), metadata={"format": "pt"})
    size = output_path.stat().st_size
    gs = {g for g in group_sizes if g}
    return {"n_compressed": len(modules), "n_exact": n_exact, "n_from_original": n_copied, "n_dense_tensors": n_dense,
            "n_total_keys": len(tensors), "output_bytes": size, "output_mb": round(size / 2 ** 20, 1),
            "compressed_modules": modules, "group_size": max(gs) if gs else 0}


def write_quantization_config(model_config_path, output_config_path, compressed_modules, manifest=None,
                              quant_method: str = "cdna_v3", group_size: int = 0) -> None:
    """config.json of the dense model + the quantization_config from_pretrained dispatches on
    (helix_substrate/convert_safetensors.py:241-270; "group_size" is this build's extension)."""
    model_config_path = Path(model_config_path)
    cfg = json.loads(model_config_path.read_text()) if model_config_path.exists() else {}
    qc = {"quant_method": quant_method, "bits": 8, "n_clusters": 256, "compressed_modules": list(compressed_modules)}
    if manifest:
        qc["compression_ratio"] = manifest.get("compression_ratio", 4.0)
        qc["n_svd_routed"] = manifest.get("n_svd_routed", 0)
    if group_size:
        qc["group_size"] = int(group_size)
    cfg["quantization_config"] = qc
    output_config_path = Path(output_config_path)
    output_config_path.parent.mkdir(parents=True, exist_ok=True)
    output_config_path.write_text(json.dumps(cfg, indent=2) + "\n")


def convert_model(cdnav3_dir, model_dir, output_dir) -> dict:
    """CDNA v3 directory + the dense model's directory (config, tokenizer, skipped tensors) -> a
    directory ``from_pretrained`` loads: model.safetensors, config.json with the
    quantization_config, tokenizer files, the manifest and a conversion receipt."""
    cdnav3_dir, model_dir, output_dir = Path(cdnav3_dir), Path(model_dir), Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    t0 = time.time()
    original = model_dir if _original_shards(model_dir) else None
    stats = convert_cdnav3_to_safetensors(cdnav3_dir, output_dir / "model.safetensors", original)
    manifest = {}
    if (cdnav3_dir / "manifest.json").exists():
        manifest = json.loads((cdnav3_dir / "manifest.json").read_text())
        shutil.copy2(cdnav3_dir / "manifest.json", output_dir / "cdnav3_manifest.json")
    write_quantization_config(model_dir / "config.json", output_dir / "config.json", stats["compressed_modules"],
                              manifest, group_size=stats["group_size"])
    for name in _TOKENIZER_FILES:
        if (model_dir / name).exists():
            shutil.copy2(model_dir / name, output_dir / name)
    stats["wall_time_s"] = round(time.time() - t0, 2)
    stats["output_dir"] = str(output_dir)
    (output_dir / "conversion_receipt.json").write_text(json.dumps(stats, indent=2) + "\n")
    return stats


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="CDNA v3 directory -> HuggingFace checkpoint of HelixLinear parts")
    ap.add_argument("--cdnav3-dir", required=True)
    ap.add_argument("--model-dir", required=True, help="the dense model's directory (config.json, tokenizer, model*.safetensors)")
    ap.add_argument("--output-dir", required=True)
    a = ap.parse_args(argv)
    stats = convert_model(a.cdnav3_dir, a.model_dir, a.output_dir)
    print(json.dumps({k: v for k, v in stats.items() if k != "compressed_modules"}, indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
