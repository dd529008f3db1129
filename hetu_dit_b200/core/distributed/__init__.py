from .parallel_state import (PROCESS_GROUP, ParallelGroups, destroy_model_parallel, get_cfg_group,
                             get_classifier_free_guidance_rank, get_classifier_free_guidance_world_size,
                             get_data_parallel_rank, get_data_parallel_world_size, get_dp_group, get_parallel_groups,
                             get_pipeline_parallel_rank, get_pipeline_parallel_world_size, get_pp_group,
                             get_ring_parallel_rank, get_ring_parallel_world_size, get_sequence_parallel_rank,
                             get_sequence_parallel_world_size, get_sp_group, get_tensor_model_parallel_rank,
                             get_tensor_model_parallel_world_size, get_tp_group, get_ulysses_parallel_rank,
                             get_ulysses_parallel_world_size, get_world_group, get_world_group_rank,
                             get_world_group_world_size, init_distributed_environment, initialize_model_parallel,
                             is_pipeline_first_stage, is_pipeline_last_stage, model_parallel_is_initialized,
                             set_seq_parallel_pg)
from .peer import PeerGroup, PeerHeap
from .runtime_state import (DiTRuntimeState, ModelGeometry, get_runtime_state, initialize_runtime_state,
                            reset_runtime_state, runtime_state_is_initialized)
from .utils import RankGenerator, generate_masked_orthogonal_rank_groups
