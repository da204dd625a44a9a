"""``ironcore``: the public names of haanjack/ironcore served by :mod:`ironcore_b200`.

A user of the reference can keep ``import ironcore`` / ``from ironcore.trainer import Trainer`` /
``from ironcore.parallel.parallel_states import get_tensor_model_parallel_rank`` and the ``ironcore``
console script. A module here is a re-export where the native object already has the reference's signature, and
a thin adapter (constructor arguments, ``[b, s, d]`` call conventions, argument order) where it does not; the
work is always done by ``ironcore_b200``. Each docstring names the reference file it mirrors.
(Reference: ironcore/__init__.py:11-20.)"""

from ironcore_b200.global_vars import (get_config, get_logger, get_timer, get_tokenizer,  # noqa: F401
                                       set_global_states)

__all__ = ["get_config", "get_tokenizer", "set_global_states", "get_logger", "get_timer"]
