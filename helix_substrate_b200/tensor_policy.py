"""Per-tensor compression policy: the subset of the reference's TensorPolicy /
TensorClass (helix_substrate/tensor_policy.py:30-262) that the codebook +
sidecar path reads, plus ``group_size`` for the group-affine extension."""

from __future__ import annotations

import re
from dataclasses import dataclass
from enum import Enum
from typing import Optional, Tuple


class TensorClass(Enum):
    EMBEDDING = "embedding"
    ATTENTION_QK = "attention_qk"
    ATTENTION_VO = "attention_vo"
    FFN = "ffn"
    NORM = "norm"
    LM_HEAD = "lm_head"
    UNKNOWN = "unknown"


@dataclass(frozen=True)
class TensorPolicy:
    tensor_class: TensorClass
    storage_mode: str  # "exact" | "codebook" | "codebook+sidecar"
    n_clusters: int = 256
    percentile: float = 99.9
    use_kmeans: bool = True
    sidecar_enabled: bool = True
    block_rows: int = 16
    max_corrections: int = 512
    vector_dim: int = 1
    svd_residual_rank: int = 0
    group_size: int = 0  # > 0: least-squares per-group scale/offset on top of the codebook


_PATTERNS = [
    (re.compile(r"(self_attn\.[qk]_proj|attn_[qk])\.weight$"), TensorClass.ATTENTION_QK),
    (re.compile(r"(self_attn\.[vo]_proj|attn_v|attn_output)\.weight$"), TensorClass.ATTENTION_VO),
    (re.compile(r"(mlp\.(gate|up|down)_proj|ffn_(gate|up|down)|mixer\.(in|out|B|C)_proj)\.weight$"), TensorClass.FFN),
    (re.compile(r"norm\w*\.weight$"), TensorClass.NORM),
    (re.compile(r"(embed_tokens|token_embd)\.weight$"), TensorClass.EMBEDDING),
    (re.compile(r"(lm_head|^output)\.weight$"), TensorClass.LM_HEAD),
]


def classify_tensor(name: str, shape: Optional[Tuple[int, ...]] = None) -> TensorClass:
    if shape is not None and len(shape) == 1:
        return TensorClass.NORM
    for pat, tc in _PATTERNS:
        if pat.search(name):
            return tc
    return TensorClass.UNKNOWN


def _cs(tc, percentile, block_rows=16, max_corrections=512):
    return TensorPolicy(tc, "codebook+sidecar", 256, percentile, True, True, block_rows, max_corrections)


_DEFAULTS = {
    TensorClass.NORM: TensorPolicy(TensorClass.NORM, "exact", 0, 100.0, False, False, 0, 0),
    TensorClass.EMBEDDING: TensorPolicy(TensorClass.EMBEDDING, "exact", 0, 100.0, False, False, 0, 0),
    TensorClass.ATTENTION_QK: _cs(TensorClass.ATTENTION_QK, 99.95),
    TensorClass.ATTENTION_VO: _cs(TensorClass.ATTENTION_VO, 99.9),
    TensorClass.FFN: _cs(TensorClass.FFN, 99.9),
    TensorClass.LM_HEAD: _cs(TensorClass.LM_HEAD, 99.9),
    TensorClass.UNKNOWN: _cs(TensorClass.UNKNOWN, 99.9, 32, 256),
}


def get_default_policy(tc: TensorClass) -> TensorPolicy:
    return _DEFAULTS[tc]


def get_policy(name: str, shape: Optional[Tuple[int, ...]] = None) -> TensorPolicy:
    return get_default_policy(classify_tensor(name, shape))
