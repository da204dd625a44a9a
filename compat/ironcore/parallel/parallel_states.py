"""Process-group getters under the reference's names (ironcore/parallel/parallel_states.py:27-150).
``get_*_group_rank`` of the reference is the rank inside the group: ``get_*_rank`` here."""

from ironcore_b200.parallel.mesh import (destroy_model_parallel, get_data_parallel_group,  # noqa: F401
                                         get_data_parallel_rank, get_data_parallel_world_size,
                                         get_expert_data_parallel_group, get_expert_model_parallel_group,
                                         get_expert_model_parallel_rank, get_expert_model_parallel_world_size,
                                         get_tensor_model_parallel_group, get_tensor_model_parallel_rank,
                                         get_tensor_model_parallel_src_rank, get_tensor_model_parallel_world_size,
                                         model_parallel_is_initialized, sequence_parallel_enabled)
from ironcore_b200.parallel import mesh as _mesh


def initialize_model_parallel(tensor_model_parallel_size: int = 1, timeout_in_minutes: float = 10.0, *, timeout=None,
                              **kwargs):
    """The reference's signature (ironcore/parallel/parallel_states.py:27-30): the second positional argument is the
    process-group timeout in minutes (its own scripts also spell it ``timeout=``); expert parallelism and sequence
    parallelism are keyword arguments here."""
    minutes = timeout if timeout is not None else timeout_in_minutes
    return _mesh.initialize_model_parallel(tensor_model_parallel_size, timeout_in_minutes=float(minutes), **kwargs)


get_tensor_model_parallel_group_rank = get_tensor_model_parallel_rank
get_data_parallel_group_rank = get_data_parallel_rank
