"""Checkpoint formats: EXL3 trellis codec, safetensors scan, TP splitting, MXFP4."""
from . import exl3, mxfp4, tp, checkpoint, safetensors_io  # noqa: F401
