"""Model family: hybrid Gated-DeltaNet + gated-attention decoder, MTP head, drafter, NVFP4 format, safetensors IO."""
from .config import HybridConfig  # noqa: F401
