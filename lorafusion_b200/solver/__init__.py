"""Multi-adapter microbatch scheduling: adapter grouping, bin packing (first-fit-decreasing and an
exact branch-and-bound in C++), the cross-group merge pass, the bubble-lemma verifier with no-op
insertion, and schedule files.  Counterpart of ``lorafusion/solver/proposed_solver.py``."""

from .schedule import (AdapterGroupStepInfo, MicroBatchInfo, apply_merge_pass_for_adapter_group_step_infos,
                       bubble_lemma_violations, flatten_schedule, greedy_pack_decide_bins, group_adapters,
                       load_schedule, packing_data_to_microbatches_micro_milp,
                       packing_data_to_microbatches_micro_milp_with_multiprocessing, save_schedule,
                       schedule_name, schedule_statistics, solve_micro_milp_lexicographic,
                       verify_correctness_of_schedule)

__all__ = [
    "AdapterGroupStepInfo", "MicroBatchInfo", "apply_merge_pass_for_adapter_group_step_infos",
    "bubble_lemma_violations", "flatten_schedule", "greedy_pack_decide_bins", "group_adapters", "load_schedule",
    "packing_data_to_microbatches_micro_milp", "packing_data_to_microbatches_micro_milp_with_multiprocessing",
    "save_schedule", "schedule_name", "schedule_statistics", "solve_micro_milp_lexicographic",
    "verify_correctness_of_schedule",
]
