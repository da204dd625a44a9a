"""ironcore_b200 — a Blackwell (B200, sm_100a) native LLM training and rollout framework.

Public surface mirrors the capabilities of the IronCore reference project
(``ironcore train/preprocess`` CLI, hierarchical YAML config groups, one unified
transformer covering GPT-2 / Llama / Gemma / Qwen / Phi shapes, DP / TP+SP / EP /
FSDP / ZeRO-1 layouts, Adam and Muon, GRPO rollouts on a paged KV cache, native and
HuggingFace-interoperable checkpoints) with the hot paths written as sm_100a CUDA
kernels (tcgen05 + TMEM + TMA) loaded from an in-tree shared library.
"""

__version__ = "0.1.0"
