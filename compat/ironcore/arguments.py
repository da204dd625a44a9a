"""Placeholder module of the reference (ironcore/arguments.py is empty there as well): flag parsing lives in
``ironcore.config`` (``load_trainer_config``, ``build_arg_parser``)."""

from ironcore_b200.config import build_arg_parser, load_trainer_config  # noqa: F401
