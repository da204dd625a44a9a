"""Parameter-name mapping between the native and the HuggingFace layouts (reference:
ironcore/checkpointing/weight_mapping.py:35-330)."""

from ironcore_b200.checkpoint.hf_interop import _ALIASES as ARCHITECTURE_ALIASES  # noqa: F401
from ironcore_b200.checkpoint.hf_interop import Architecture, WeightMapper, detect_architecture  # noqa: F401

get_architecture = detect_architecture
