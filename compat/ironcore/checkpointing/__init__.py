"""Native and HuggingFace checkpoints (reference: ironcore/checkpointing/{native,hf_interop,weight_mapping}.py)."""

from ironcore_b200.checkpoint import HFConfigManager, load_checkpoint, save_checkpoint  # noqa: F401
from ironcore_b200.checkpoint.hf_interop import (Architecture, detect_architecture,  # noqa: F401
                                                 detect_checkpoint_format, export_to_huggingface,
                                                 load_from_huggingface)

from .weight_mapping import WeightMapper  # noqa: F401

get_architecture = detect_architecture
load_hf_config = HFConfigManager.load_hf_config
