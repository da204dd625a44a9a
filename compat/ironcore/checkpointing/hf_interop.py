"""HuggingFace import / export (reference: ironcore/checkpointing/hf_interop.py:47-620)."""

from ironcore_b200.checkpoint.hf_interop import (detect_checkpoint_format, export_to_huggingface,  # noqa: F401
                                                 generate_hf_config, load_from_huggingface, read_hf_state_dict)
from ironcore_b200.checkpoint.native import HFConfigManager

load_hf_state_dict = read_hf_state_dict
load_hf_config = HFConfigManager.load_hf_config
_generate_hf_config = generate_hf_config
