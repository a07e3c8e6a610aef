"""Image input: preprocessing, a CLIP-style vision transformer with a projector into the language model's embedding
space, and the prompt builder that splices image tokens into a text prompt."""
from .encoder import ImagePreprocessor, VisionConfig, VisionEncoder, convert_vision_tower, load_vision_encoder  # noqa: F401
from .prompt import MultimodalPrompt  # noqa: F401
