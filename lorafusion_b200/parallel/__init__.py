"""Parallel runtimes: process-group layouts, the 1F1B pipeline, symmetric-memory collectives
fused into kernels (data and tensor parallel) and host-side failure detection.

Names follow the reference where it has a counterpart
(``lorafusion/pipeline_parallel/pipe_module.py:98-154``,
``lorafusion/pipeline_parallel/multi_lora_schedule.py``).
"""

from .health import HealthMonitor, PeerFailure
from .layout import ParallelLayout, ParallelState, initialize_parallel_state
from .pipeline import (EMPTY_BATCH_MAGIC_TOKEN, PipeModel, PipelineMicrobatch, PipelineRuntime, PipelineStats,
                       even_layer_partition, get_pipeline_stage_layer_indices,
                       multi_lora_get_forward_backward_func)

__all__ = [
    "HealthMonitor", "PeerFailure", "ParallelLayout", "ParallelState", "initialize_parallel_state",
    "EMPTY_BATCH_MAGIC_TOKEN", "PipeModel", "PipelineMicrobatch", "PipelineRuntime", "PipelineStats",
    "even_layer_partition", "get_pipeline_stage_layer_indices", "multi_lora_get_forward_backward_func",
]
