"""HuggingFace quantizer registration for HXQ / CDNA-v3 checkpoints.

``config.json["quantization_config"]["quant_method"]`` in {"cdna_v3", "helix",
"hxq"} makes ``AutoModelForCausalLM.from_pretrained`` build HelixLinear shells
for the listed modules, let the checkpoint loader fill their buffers
({module}.codebook / .indices / .sidecar_positions / .sidecar_values / .bias and,
for the group-affine extension, .group_scales / .group_offsets), then derive the
sidecar CSR.  Same names, config keys and lifecycle as the reference
(helix_substrate/hf_quantizer.py:86-669); the modules it creates run on the
sm_100a kernels.

One deliberate difference: rotary ``inv_freq`` is recomputed only when it was
left on the meta device or holds non-finite garbage, and theta is read from
``config.rope_parameters`` (transformers 5) before ``config.rope_theta``
(transformers 4) - the reference always recomputes with ``rope_theta`` and a
10000 default, which silently changes Qwen2's theta of 1e6 under transformers 5.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional, Union

import torch
import torch.nn as nn

logger = logging.getLogger(__name__)

try:
    from transformers.utils.quantization_config import QuantizationConfigMixin
    from transformers.quantizers.auto import register_quantization_config, register_quantizer
    from transformers.quantizers.base import HfQuantizer
    HAS_HF_QUANTIZER_API = True
except ImportError:  # usable without transformers: plain classes, no registration
    HAS_HF_QUANTIZER_API = False
    QuantizationConfigMixin = object
    HfQuantizer = object

    def register_quantization_config(name):
        return lambda cls: cls

    def register_quantizer(name):
        return lambda cls: cls

_HELIX_BUFFER_SUFFIXES = (
    ".codebook", ".indices", ".sidecar_positions", ".sidecar_values", ".svd_U", ".svd_s", ".svd_Vt",
    ".channel_scales", ".group_scales", ".group_offsets", ".codebook_f16", ".weight", ".bias",
)
_OPTIONAL_SUFFIXES = (
    ".codebook_f16", "._sidecar_vq_vals", "._sidecar_rows", "._sidecar_cols", "._sidecar_deltas",
    "._csr_rowptr", "._csr_cols", ".svd_U", ".svd_s", ".svd_Vt", ".bias", ".channel_scales",
    ".group_scales", ".group_offsets", ".sidecar_positions", ".sidecar_values", ".weight",
)


class _QuantMethodShim:
    """String that also has ``.value`` (newer transformers treat quant_method as an enum)."""

    def __init__(self, name: str):
        self.value = name

    def __str__(self) -> str:
        return self.value

    def __repr__(self) -> str:
        return f"_QuantMethodShim({self.value!r})"

    def __eq__(self, other: object) -> bool:
        return self.value == getattr(other, "value", other)

    def __hash__(self) -> int:
        return hash(self.value)


@register_quantization_config("cdna_v3")
class CDNAv3Config(QuantizationConfigMixin):
    """quantization_config block of an HXQ checkpoint (hf_quantizer.py:86-171)."""

    def __init__(self, bits: int = 8, n_clusters: int = 256, compressed_modules: Optional[List[str]] = None,
                 compression_ratio: float = 4.0, n_svd_routed: int = 0,
                 modules_to_not_convert: Optional[List[str]] = None,
                 module_k_map: Optional[Dict[str, int]] = None, vector_dim: int = 1,
                 module_vector_dim_map: Optional[Dict[str, int]] = None, index_packing: Optional[str] = None,
                 codebook_size: Optional[int] = None, sidecar_enabled: bool = True,
                 exact_patterns: Optional[List[str]] = None, group_size: int = 0, **kwargs):
        self.quant_method = _QuantMethodShim("cdna_v3")
        self.bits = bits
        self.n_clusters = codebook_size if codebook_size is not None else n_clusters
        self.compressed_modules = compressed_modules or []
        self.compression_ratio = compression_ratio
        self.n_svd_routed = n_svd_routed
        self.modules_to_not_convert = modules_to_not_convert or []
        self.sidecar_enabled = sidecar_enabled
        self.exact_patterns = exact_patterns or []
        self.module_k_map = module_k_map or {}
        self.vector_dim = vector_dim
        self.module_vector_dim_map = module_vector_dim_map or {}
        self.index_packing = index_packing
        self.group_size = group_size

    def to_dict(self) -> dict:
        d = {"quant_method": "cdna_v3", "bits": self.bits, "n_clusters": self.n_clusters,
             "compressed_modules": self.compressed_modules, "compression_ratio": self.compression_ratio,
             "n_svd_routed": self.n_svd_routed}
        if self.module_k_map:
            d["module_k_map"] = self.module_k_map
        if self.vector_dim > 1:
            d["vector_dim"] = self.vector_dim
        if self.module_vector_dim_map:
            d["module_vector_dim_map"] = self.module_vector_dim_map
        if self.group_size:
            d["group_size"] = self.group_size
        return d

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any], return_unused_kwargs: bool = False,
                  **kwargs) -> Union["CDNAv3Config", tuple]:
        d = dict(config_dict)
        d.pop("quant_method", None)
        d.update(kwargs)
        obj = cls(**d)
        return (obj, {}) if return_unused_kwargs else obj


def _replace_with_helix_linear(model: nn.Module, compressed_modules: set,
                               compute_dtype: torch.dtype = torch.float32,
                               module_k_map: Optional[Dict[str, int]] = None, n_clusters_default: int = 256,
                               vector_dim_default: int = 1,
                               module_vector_dim_map: Optional[Dict[str, int]] = None,
                               index_packing: Optional[str] = None, group_size: int = 0) -> tuple:
    """Swap every listed nn.Linear for a HelixLinear shell; listed nn.Embedding
    modules get codebook/indices buffers and are densified after loading."""
    from .helix_linear import HelixLinear
    k_map, vd_map = module_k_map or {}, module_vector_dim_map or {}
    done, embeddings, n = set(), set(), 0
    for name, mod in list(model.named_modules()):
        if name not in compressed_modules or id(mod) in done:
            continue
        if isinstance(mod, nn.Embedding):
            mod.register_buffer("codebook", torch.zeros(k_map.get(name, n_clusters_default)))
            mod.register_buffer("indices", torch.zeros(mod.num_embeddings, mod.embedding_dim, dtype=torch.uint8))
            embeddings.add(name)
        elif isinstance(mod, nn.Linear):
            shell = HelixLinear.from_quantized_config(
                mod.in_features, mod.out_features, tensor_name=f"{name}.weight", compute_dtype=compute_dtype,
                n_clusters=k_map.get(name, n_clusters_default), vector_dim=vd_map.get(name, vector_dim_default),
                index_packing=None, group_size=group_size)
            parent = model
            *head, leaf = name.split(".")
            for part in head:
                parent = getattr(parent, part)
            setattr(parent, leaf, shell)
        else:
            continue
        done.add(id(mod))
        n += 1
    return n, embeddings


def _rope_theta(config) -> float:
    rp = getattr(config, "rope_parameters", None)
    if isinstance(rp, dict) and "rope_theta" in rp:
        return float(rp["rope_theta"])
    return float(getattr(config, "rope_theta", 10000.0))


@register_quantizer("cdna_v3")
class HelixHfQuantizer(HfQuantizer if HAS_HF_QUANTIZER_API else object):
    """shells before loading -> loader fills buffers -> derived buffers after."""

    requires_calibration = False
    required_packages = ["helix_substrate"]
    requires_parameters_quantization = True

    def __init__(self, quantization_config: CDNAv3Config, **kwargs):
        if HAS_HF_QUANTIZER_API:
            super().__init__(quantization_config, **kwargs)
        self.quantization_config = quantization_config
        self._compressed_embeddings: set = set()
        self._aliased_prefixes: set = set()

    def validate_environment(self, *args, **kwargs):
        from . import helix_linear  # noqa: F401

    def update_dtype(self, dtype):
        return torch.float32 if dtype is None else dtype

    update_torch_dtype = update_dtype

    # ---- transformers 4.x parameter hooks (absent from 5.x's base class; harmless there)
    def check_quantized_param(self, model, param_value, param_name, state_dict, **kwargs) -> bool:
        from .helix_linear import HelixLinear
        if not param_name.endswith(_HELIX_BUFFER_SUFFIXES) or "." not in param_name:
            return False
        try:
            return isinstance(model.get_submodule(param_name.rsplit(".", 1)[0]), HelixLinear)
        except (AttributeError, ValueError):
            return False

    def create_quantized_param(self, model, param_value, param_name, target_device, *args, **kwargs) -> None:
        mod_path, buf = param_name.rsplit(".", 1)
        mod = model.get_submodule(mod_path)
        if buf == "weight":
            mod.weight = param_value.to(target_device)
        else:
            mod.register_buffer(buf, param_value.to(target_device))

    # ---- transformers 5.x: nothing is quantised on the fly, tensors load as stored
    def param_needs_quantization(self, model, param_name: str, **kwargs) -> bool:
        return False

    def _process_model_before_weight_loading(self, model: nn.Module, **kwargs) -> None:
        cfg = self.quantization_config
        compressed = set(cfg.compressed_modules)
        if not compressed:
            logger.warning("CDNAv3Config.compressed_modules is empty - nothing becomes HelixLinear")
            return
        k_map = dict(cfg.module_k_map or {})
        tied = getattr(model, "all_tied_weights_keys", None) or {}
        if isinstance(tied, dict):  # shared blocks: the alias path needs a shell as well
            for tgt, src in tied.items():
                if src.endswith(".weight") and tgt.endswith(".weight") and src[:-7] in compressed:
                    compressed.add(tgt[:-7])
                    if src[:-7] in k_map:
                        k_map.setdefault(tgt[:-7], k_map[src[:-7]])
        n, self._compressed_embeddings = _replace_with_helix_linear(
            model, compressed, module_k_map=k_map, n_clusters_default=cfg.n_clusters,
            vector_dim_default=getattr(cfg, "vector_dim", 1),
            module_vector_dim_map=dict(getattr(cfg, "module_vector_dim_map", None) or {}),
            index_packing=getattr(cfg, "index_packing", None), group_size=getattr(cfg, "group_size", 0))
        logger.info("HXQ: %d modules replaced (%d embeddings)", n, len(self._compressed_embeddings))
        seen: dict = {}

        def walk(mod, prefix=""):
            for cname, child in mod._modules.items():
                if child is None:
                    continue
                full = f"{prefix}.{cname}" if prefix else cname
                if id(child) in seen:
                    self._aliased_prefixes.add(full)
                else:
                    seen[id(child)] = full
                    walk(child, full)
        walk(model)

    def _process_model_after_weight_loading(self, model: nn.Module, **kwargs) -> None:
        from .helix_linear import HelixLinear
        tied = getattr(model, "all_tied_weights_keys", None) or {}
        if isinstance(tied, dict):
            for tgt, src in tied.items():
                if not (src.endswith(".weight") and tgt.endswith(".weight")):
                    continue
                try:
                    s_mod, t_mod = model.get_submodule(src[:-7]), model.get_submodule(tgt[:-7])
                except (AttributeError, ValueError):
                    continue
                if (isinstance(s_mod, HelixLinear) and isinstance(t_mod, HelixLinear) and s_mod is not t_mod
                        and not bool(t_mod.codebook.abs().sum())):
                    for b in ("codebook", "indices", "sidecar_positions", "sidecar_values", "svd_U", "svd_s",
                              "svd_Vt", "bias", "channel_scales", "group_scales", "group_offsets"):
                        t_mod.register_buffer(b, getattr(s_mod, b, None))
        n = 0
        for mod in model.modules():
            if isinstance(mod, HelixLinear):
                mod._recompute_derived()
                n += 1
        logger.info("HXQ: finalised %d HelixLinear modules", n)

        config = getattr(model, "config", None)
        for name, mod in model.named_modules():
            inv = getattr(mod, "inv_freq", None)
            if not isinstance(inv, torch.Tensor) or inv.numel() == 0:
                continue
            if inv.is_meta or not bool(torch.isfinite(inv).all()):
                dim = inv.shape[0] * 2
                theta = _rope_theta(config) if config is not None else 10000.0
                new = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
                mod.inv_freq = new if inv.is_meta else new.to(inv.device)
                logger.info("HXQ: recomputed inv_freq for %s (theta=%g)", name, theta)

        for name, mod in model.named_modules():
            if name in self._compressed_embeddings and isinstance(mod, nn.Embedding):
                cb, idx = getattr(mod, "codebook", None), getattr(mod, "indices", None)
                if cb is None or idx is None:
                    logger.warning("HXQ: %s has no codebook/indices", name)
                    continue
                with torch.no_grad():
                    mod.weight.copy_(cb[idx.long()])
                del mod.codebook, mod.indices

    def _is_under_alias(self, key: str) -> bool:
        return any(key.startswith(p + ".") for p in self._aliased_prefixes)

    def _drop_optional(self, keys: list, keep: set) -> list:
        compressed = set(self.quantization_config.compressed_modules)
        out = []
        for k in keys:
            if self._is_under_alias(k):
                continue
            if k.endswith(_OPTIONAL_SUFFIXES) and k.rsplit(".", 1)[0] in compressed and k not in keep:
                continue
            out.append(k)
        return out

    def update_missing_keys(self, model, missing_keys: list, prefix: str = "") -> list:
        return self._drop_optional(list(missing_keys), set())

    def update_expected_keys(self, model, expected_keys: list, loaded_keys: list) -> list:
        return self._drop_optional(list(expected_keys), set(loaded_keys))

    @property
    def is_trainable(self) -> bool:
        return False

    def is_serializable(self, safe_serialization=None) -> bool:
        return True


def _register_aliases() -> None:
    if not HAS_HF_QUANTIZER_API:
        return
    for alias in ("helix", "hxq"):
        try:
            register_quantization_config(alias)(CDNAv3Config)
            register_quantizer(alias)(HelixHfQuantizer)
        except Exception:  # already registered
            pass
    try:
        from transformers.quantizers.auto import AUTO_QUANTIZER_MAPPING, AUTO_QUANTIZATION_CONFIG_MAPPING
        for alias in ("cdna_v3", "helix", "hxq"):
            AUTO_QUANTIZATION_CONFIG_MAPPING[alias] = CDNAv3Config
            AUTO_QUANTIZER_MAPPING[alias] = HelixHfQuantizer
    except ImportError:
        pass


_register_aliases()
