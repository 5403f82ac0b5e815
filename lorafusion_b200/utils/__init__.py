"""Utilities: benchmarking harness and timers, numerical test helpers, logging, SVG charts."""

from .benchmark import benchmark, create_profiler_context, set_warmup_and_number, tabulate_2d_benchmark_results
from .common import create_packed_dummy_inputs
from .testing import assert_close, assert_close_two_rounds, verbose_allclose

__all__ = ["benchmark", "create_profiler_context", "set_warmup_and_number", "tabulate_2d_benchmark_results",
           "assert_close", "assert_close_two_rounds", "verbose_allclose", "create_packed_dummy_inputs"]
