"""Simulators: the event-driven 1F1B pipeline timing simulator with schedule generators
(``benchmarks_paper/imbalance_simulator`` in the reference) and the analytic performance /
memory predictor with measured B200 profiles (``lorafusion/simulator/mono.py``)."""

from .pipeline_sim import (PipelineTimeline, check_forward_backward_constraints, compare_schedules,
                           evaluate_schedule_pipeline_parallelism, find_overlaps, generate_data,
                           generate_mlora_schedule, generate_naive_schedule, generate_sorted_schedule,
                           simulate_1f1b, solve_schedule_order)
from .predictor import (CONFIG_DIR, HardwareSpec, LoRALLMPredictor, LoRALLMProfileResult, LoRALLMProfiler,
                        SimulationConfiguration, SimulationResult, best_configurations, calibrate_profile,
                        load_b200_profile, optimization_configuration_generator, synthesize_profile)

config_dir = CONFIG_DIR  # the name the reference's predictor imports

__all__ = [
    "PipelineTimeline", "check_forward_backward_constraints", "compare_schedules",
    "evaluate_schedule_pipeline_parallelism", "find_overlaps", "generate_data", "generate_mlora_schedule",
    "generate_naive_schedule", "generate_sorted_schedule", "simulate_1f1b", "solve_schedule_order", "CONFIG_DIR", "config_dir",
    "HardwareSpec", "LoRALLMPredictor", "LoRALLMProfileResult", "LoRALLMProfiler", "SimulationConfiguration",
    "SimulationResult", "best_configurations", "calibrate_profile", "load_b200_profile",
    "optimization_configuration_generator", "synthesize_profile",
]
