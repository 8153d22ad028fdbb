"""``import helix_substrate`` drop-in: the reference's package name, served by
helix_substrate_b200.  Every submodule of the compressed-linear path resolves
under both of the reference's spellings (``helix_substrate.cdnav3_reader`` as its
code imports it, ``helix_substrate.hxq_reader_v3`` as the file is named), and the
HuggingFace quantizer is registered on import, as the reference does
(helix_substrate/__init__.py:27-36)."""

import importlib
import sys

import helix_substrate_b200 as _impl

__version__ = _impl.__version__

_SUBMODULES = (
    "helix_linear", "helix_affine_linear", "triton_vq_matmul", "triton_affine_group_matmul", "triton_affine_matmul",
    "cdnav3_reader", "cdnav3_writer", "hxq_reader_v3", "hxq_writer_v3", "generate_sidecars_v3",
    "tensor_policy", "hf_quantizer", "hf_integration", "hxq_writer_gpu", "tp", "packed",
)
for _name in _SUBMODULES:
    _mod = importlib.import_module(f"helix_substrate_b200.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod

from helix_substrate_b200.tensor_policy import classify_tensor, TensorPolicy, TensorClass  # noqa: E402,F401
from helix_substrate_b200.cdnav3_writer import CDNAv3Writer  # noqa: E402,F401
from helix_substrate_b200.cdnav3_reader import CDNAv3Reader  # noqa: E402,F401
from helix_substrate_b200.helix_linear import HelixLinear  # noqa: E402,F401
from helix_substrate_b200.hf_quantizer import CDNAv3Config, HelixHfQuantizer  # noqa: E402,F401
