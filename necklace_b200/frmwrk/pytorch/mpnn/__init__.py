"""Tensor-parallel ("mp") building blocks."""
from .initialize import (destroy_model_parallel, get_data_parallel_group, get_data_parallel_rank,
                         get_data_parallel_world_size, get_model_parallel_group,
                         get_model_parallel_rank, get_model_parallel_src_rank,
                         get_model_parallel_world_size, initialize_model_parallel,
                         model_parallel_is_initialized)
from .layers import (ColumnParallelLinear, ParallelEmbedding, RowParallelLinear,
                     VocabParallelEmbedding)
from .mappings import (copy_to_model_parallel_region, gather_from_model_parallel_region,
                       reduce_from_model_parallel_region, scatter_to_model_parallel_region)
from .checkpointing import (checkpoint, get_cuda_rng_tracker, model_parallel_cuda_manual_seed,
                            partition_activations_in_checkpoint)
from .cross_entropy import vocab_parallel_cross_entropy
from .data import broadcast_data
from .grads import clip_grad_norm
from .utils import VocabUtility, divide, split_tensor_along_last_dim
