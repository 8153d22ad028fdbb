"""The reader under the reference's on-disk module name (hxq_reader_v3.py)."""
from .cdnav3_reader import CDNAv3Reader  # noqa: F401
