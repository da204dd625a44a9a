"""Native and HuggingFace checkpoints (reference: ironcore/checkpointing/{native,hf_interop,weight_mapping}.py)."""

from ironcore_b200.checkpoint import HFConfigManager, load_checkpoint, save_checkpoint  # noqa: F401
from ironcore_b200.checkpoint.hf_interop import (Architecture, WeightMapper, export_to_huggingface,  # noqa: F401
                                                 load_from_huggingface)
