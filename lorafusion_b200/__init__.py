"""lorafusion_b200: a Blackwell-native (sm_100a) multi-LoRA fine-tuning framework.

Sub-packages
------------
``ops``        hand-written tcgen05/TMA kernels and their autograd wrappers, CPU oracles
``models``     decoder models (Llama / Qwen2 shapes), adapter containers, PEFT-format I/O
``parallel``   process-group layout, DP / TP / PP runtimes, symmetric-memory collectives
``solver``     multi-adapter microbatch packing (C++ core) and schedule verification
``simulator``  pipeline timing simulator and analytic performance / memory predictor
``train``      configuration dataclasses, synthetic data providers, training loops
``utils``      benchmarking, testing, logging, timers
"""

__version__ = "0.1.0"
