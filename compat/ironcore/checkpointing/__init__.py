"""Native and HuggingFace checkpoints (reference: ironcore/checkpointing/{native,hf_interop,weight_mapping}.py)."""

from ironcore_b200.checkpoint import HFConfigManager, load_checkpoint, save_checkpoint  # noqa: F401
from ironcore_b200.checkpoint.hf_interop import Architecture, detect_architecture  # noqa: F401

from .hf_interop import (detect_checkpoint_format, export_to_huggingface, load_from_huggingface,  # noqa: F401
                         load_hf_config, load_hf_state_dict)
from .weight_mapping import WeightMapper  # noqa: F401

get_architecture = detect_architecture
