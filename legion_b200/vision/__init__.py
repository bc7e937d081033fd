"""Images in prompts: decoding and preprocessing (``preprocess``), the vision tower that turns an image's patches
into input rows of the language model (``tower``), where those rows sit in a sequence and the rotary positions they
take (``media``), and the row cache keyed by image hash (``cache``).

Reference counterparts: ``src/vision/{mod,preprocess,qwen3vl,gemma4v,gpu}.rs``, ``src/cuda/vision.cu`` (tower),
``src/engine/lm/vision.rs`` and ``src/model/core/media.rs`` (image tokens, multi-section rotary positions, prefix
key). The tower here runs on PyTorch tensor operations: it is a prompt-time encoder of plain, bias-carrying GEMMs
and unmasked attention over a few thousand patches, not part of the decode loop."""
from .cache import RowCache
from .media import SeqMedia, VisionRuntime, expand_image_tokens, mrope_positions
from .preprocess import Preprocessed, VisionHparams, decode_image, preprocess
from .tower import VisionConfig, VisionTower, random_vision_weights

__all__ = ["RowCache", "SeqMedia", "VisionRuntime", "expand_image_tokens", "mrope_positions", "Preprocessed",
           "VisionHparams", "decode_image", "preprocess", "VisionConfig", "VisionTower", "random_vision_weights"]
