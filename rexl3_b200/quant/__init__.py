"""EXL3 quantizer and pack I/O."""
from .quantize import load_pack, quantize_dense, quantize_linear, random_fp_weights, write_pack  # noqa: F401
from .trellis import encode_tiles  # noqa: F401
