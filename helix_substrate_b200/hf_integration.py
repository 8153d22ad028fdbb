"""Import-compatible names of the reference's older HF integration module
(helix_substrate/hf_integration.py:55-103).  Registration lives in
hf_quantizer; this module only keeps ``HelixQuantizationConfig`` and
``HelixHfQuantizer`` importable from their old location."""

from __future__ import annotations

from typing import Optional

from .hf_quantizer import CDNAv3Config, HelixHfQuantizer, HAS_HF_QUANTIZER_API  # noqa: F401

HF_AVAILABLE = HAS_HF_QUANTIZER_API

_DEFAULT_EXACT = ["embed_tokens", "embed_positions", "wte", "wpe", "lm_head", "layernorm", "layer_norm",
                  "norm", "backbone.embedding"]


class HelixQuantizationConfig(CDNAv3Config):
    """Older config spelling: ``codebook_size`` instead of ``n_clusters``."""

    def __init__(self, codebook_size: int = 256, sidecar_enabled: bool = True,
                 exact_patterns: Optional[list] = None, compressed_modules: Optional[list] = None,
                 modules_to_not_convert: Optional[list] = None, **kwargs):
        if codebook_size < 2 or codebook_size > 65536:
            raise ValueError(f"codebook_size must be 2-65536, got {codebook_size}")
        super().__init__(codebook_size=codebook_size, sidecar_enabled=sidecar_enabled,
                         exact_patterns=exact_patterns or list(_DEFAULT_EXACT),
                         compressed_modules=compressed_modules, modules_to_not_convert=modules_to_not_convert,
                         **kwargs)
        self.codebook_size = codebook_size
