"""B200-native HXQ compressed-linear forward path (helix-substrate drop-in).

uint8 indices into a 256-entry fp32 codebook, optional per-group affine, sparse
outlier sidecar; hand-written sm_100a kernels behind a C ABI (libhxq_b200.so)."""

__version__ = "0.1.0"

from .helix_linear import (  # noqa: F401
    HelixLinear, HelixLinearStats, load_helix_linear_from_cdnav3, load_cdna_factors, swap_to_helix,
    swap_summary, freeze_sidecar_phase, set_cuda_graph_mode, pre_step_kurtosis_all,
)
from .helix_affine_linear import HelixAffineLinear, quantize_linear_to_affine, swap_to_affine  # noqa: F401
from .packed import HxqWeight  # noqa: F401
