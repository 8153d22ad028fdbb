"""The writer under the reference's on-disk module name (hxq_writer_v3.py)."""
from .cdnav3_writer import CDNAv3Writer, _safe_name, _cosine  # noqa: F401
