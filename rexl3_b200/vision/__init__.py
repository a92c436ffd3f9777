"""CPU image preprocessing for vision-language prompts (resize rule, PIL-exact bicubic, normalisation, patch layout, 2-D position ids)."""
from .preprocess import (ImageInputs, bicubic_resize_u8, patch_position_ids, patchify, preprocess_image, preprocess_video, smart_resize)  # noqa: F401
