"""Process and parallelism set-up (reference: ironcore/parallel/parallel.py:24-117).
``initialize_parallelism(config, model)`` returns the model prepared for data parallelism: the FSDP wrapper
with ``parallel.use_fsdp``, else the model itself (gradient reduction across data-parallel ranks is done by
the flat-buffer optimizer engine, not by a DistributedDataParallel wrapper)."""

from ironcore_b200.parallel.mesh import initialize_process  # noqa: F401


def initialize_parallelism(config, model):
    if config.parallel.use_fsdp:
        from ironcore_b200.parallel.fsdp import FullyShardedModel

        return model if isinstance(model, FullyShardedModel) else FullyShardedModel(model, config)
    return model


__all__ = ["initialize_process", "initialize_parallelism"]
