"""Process-group getters under the reference's names (ironcore/parallel/parallel_states.py:27-150).
``get_*_group_rank`` of the reference is the rank inside the group: ``get_*_rank`` here."""

from ironcore_b200.parallel.mesh import (destroy_model_parallel, get_data_parallel_group,  # noqa: F401
                                         get_data_parallel_rank, get_data_parallel_world_size,
                                         get_expert_data_parallel_group, get_expert_model_parallel_group,
                                         get_expert_model_parallel_rank, get_expert_model_parallel_world_size,
                                         get_tensor_model_parallel_group, get_tensor_model_parallel_rank,
                                         get_tensor_model_parallel_src_rank, get_tensor_model_parallel_world_size,
                                         initialize_model_parallel, model_parallel_is_initialized,
                                         sequence_parallel_enabled)

get_tensor_model_parallel_group_rank = get_tensor_model_parallel_rank
get_data_parallel_group_rank = get_data_parallel_rank
