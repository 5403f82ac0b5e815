"""Analytic performance / memory predictor and GPU layer profiler.

Counterpart of ``lorafusion/simulator/mono.py`` (+ ``object.py`` and the YAML profiles under
``lorafusion/simulator/configs``): a *profile* holds per-layer forward and forward+backward
times at several token counts plus per-token memory figures; the *predictor* interpolates
them and combines them with a collective cost model into step time and peak memory of a
(dp, tp, pp, microbatch tokens, recomputed layers) configuration; the *enumerator* lists
feasible configurations.  Differences from the reference: tensor parallelism is a real term
(the reference only carries an ``embedding_tp_size`` and would raise on its
``"all-reduce"`` / ``"allreduce"`` mismatch, ``mono.py:1092,1502``); LoRA parameters are
counted once per adapter (``mono.py:1593-1597`` double counts); a roofline-based profile can
be synthesised without a GPU from the measured peaks of the machine.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Iterable, Optional, Sequence

import numpy as np
import yaml

from ..models.config import AdapterSpec, ModelConfig, get_model_config

TOKEN_GRID = (512, 1024, 2048, 4096, 8192, 16384)


@dataclass
class HardwareSpec:
    name: str = "B200"
    bf16_tflops: float = 1375.8          # sustained cuBLAS bf16, measured
    hbm_gbs: float = 6546.2              # measured copy bandwidth
    nvlink_gbs: float = 770.0            # measured peer copy bandwidth per direction
    allreduce_bus_gbs: float = 725.0     # measured 8-rank all-reduce bus bandwidth
    collective_latency_us: float = 12.0
    p2p_latency_us: float = 6.0
    memory_gb: float = 180.0
    gemm_efficiency: float = 0.85        # fraction of bf16_tflops the fused GEMMs reach
    # A layer split over tp ranks does not run tp times faster: the per-rank GEMMs are narrower and
    # carry the copy / reduce warps.  FLOP-weighted roofline fractions of the fused all-gather->GEMM
    # and GEMM->reduce-scatter kernels measured on 2 and 4 GPUs, relative to the single-GPU GEMMs;
    # 8 is extrapolated.
    tp_efficiency: dict = field(default_factory=lambda: {1: 1.0, 2: 0.92, 4: 0.82, 8: 0.7})

    @classmethod
    def from_measured_peaks(cls, path: str | Path) -> "HardwareSpec":
        p = Path(path)
        if not p.exists():
            return cls()
        d = json.loads(p.read_text())
        return cls(name=d.get("chip", "B200"), bf16_tflops=d.get("bf16_tflops_sustained", 1375.8),
                   hbm_gbs=d.get("hbm_gbs", 6546.2))


@dataclass
class LoRALLMProfileResult:
    """Measured (or synthesised) single-GPU profile of one model with LoRA adapters."""

    model: str
    num_layers: int
    hidden_size: int
    params_per_layer: int
    lora_params_per_layer_per_adapter: int
    embedding_params: int
    weight_bytes_per_param: float                 # 2 for bf16, ~0.53 for NF4 + absmax
    saved_bytes_per_token_per_layer: int          # kept for backward without recomputation
    checkpoint_bytes_per_token_per_layer: int     # kept with recomputation (layer input only)
    peak_intermediate_bytes_per_token: int
    head_intermediate_bytes_per_token: int
    tokens: list = field(default_factory=lambda: list(TOKEN_GRID))
    layer_fwd_ms: list = field(default_factory=list)
    layer_fwd_bwd_ms: list = field(default_factory=list)
    head_fwd_bwd_ms: list = field(default_factory=list)   # embedding + final norm + lm_head + loss

    def save(self, path: str | Path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(yaml.safe_dump(asdict(self), sort_keys=False))

    @classmethod
    def load(cls, path: str | Path) -> "LoRALLMProfileResult":
        return cls(**yaml.safe_load(Path(path).read_text()))

    # ---- interpolation -------------------------------------------------------------
    def _interp(self, ys: Sequence[float], tokens: float) -> float:
        xs = np.asarray(self.tokens, dtype=np.float64)
        ys = np.asarray(ys, dtype=np.float64)
        if tokens <= xs[0]:
            return float(ys[0] * tokens / xs[0])
        if tokens >= xs[-1]:
            return float(ys[-1] * tokens / xs[-1])
        return float(np.interp(tokens, xs, ys))

    def layer_fwd(self, tokens: float) -> float:
        return self._interp(self.layer_fwd_ms, tokens)

    def layer_fwd_bwd(self, tokens: float) -> float:
        return self._interp(self.layer_fwd_bwd_ms, tokens)

    def head_fwd_bwd(self, tokens: float) -> float:
        return self._interp(self.head_fwd_bwd_ms, tokens)


def synthesize_profile(cfg: ModelConfig | str, hw: Optional[HardwareSpec] = None, *, lora_rank: int = 16,
                       quantized: bool = False, mean_seq_len: int = 1024) -> LoRALLMProfileResult:
    """Roofline estimate of a profile: GEMM FLOPs at ``gemm_efficiency`` of the measured bf16
    peak plus memory-bound elementwise traffic at the measured HBM bandwidth."""
    cfg = get_model_config(cfg) if isinstance(cfg, str) else cfg
    hw = hw or HardwareSpec()
    h, i = cfg.hidden_size, cfg.intermediate_size
    ppl = cfg.layer_param_count()
    lora = lora_rank * (3 * h + cfg.qkv_size + cfg.q_size + h + 2 * h + 2 * i + i + h)
    fwd, fwd_bwd, head = [], [], []
    for t in TOKEN_GRID:
        gemm = 2.0 * ppl * t
        attn = 2.0 * 2 * t * min(mean_seq_len, t) * cfg.q_size / 2
        elt_bytes = t * (12 * h + 3 * cfg.qkv_size + 8 * i) * 2
        f = (gemm + attn) / (hw.bf16_tflops * 1e12 * hw.gemm_efficiency) + elt_bytes / (hw.hbm_gbs * 1e9)
        fwd.append(f * 1e3)
        fwd_bwd.append(f * 1e3 * 2.15)   # dX GEMMs equal the forward; attention backward is ~2.5x
        head.append((3 * 2.0 * cfg.vocab_size * h * t) / (hw.bf16_tflops * 1e12 * hw.gemm_efficiency) * 1e3)
    saved = (cfg.qkv_size + cfg.q_size + h + 2 * i) * 2 + cfg.num_heads * 4
    return LoRALLMProfileResult(
        model=cfg.name, num_layers=cfg.num_layers, hidden_size=h, params_per_layer=ppl,
        lora_params_per_layer_per_adapter=lora, embedding_params=cfg.vocab_size * h,
        weight_bytes_per_param=(0.5 + 4.0 / 64 / 4 + 1.0 / 64) if quantized else 2.0,
        saved_bytes_per_token_per_layer=saved, checkpoint_bytes_per_token_per_layer=h * 2,
        peak_intermediate_bytes_per_token=(3 * h + cfg.qkv_size + cfg.q_size + 5 * i) * 2,
        head_intermediate_bytes_per_token=h * 6, layer_fwd_ms=fwd, layer_fwd_bwd_ms=fwd_bwd,
        head_fwd_bwd_ms=head)


def calibrate_profile(profile: LoRALLMProfileResult, *, layer_fwd_bwd_ms: dict, head_fwd_bwd_ms: dict,
                      fwd_share: float = 0.32) -> LoRALLMProfileResult:
    """Rescale a synthesised profile so that it passes through measured points.

    ``layer_fwd_bwd_ms`` / ``head_fwd_bwd_ms`` map a token count to a measured time.  Every grid
    point takes the measured/synthetic ratio of the nearest measured token count (in log space);
    the forward time is set to ``fwd_share`` of forward+backward (the share seen in kernel
    traces of this framework: the backward holds the dX GEMMs, the LoRA gradient GEMMs and the
    2.5x heavier attention backward)."""
    import copy

    out = copy.deepcopy(profile)

    def ratios(measured: dict, synth: Sequence[float]) -> list:
        pts = sorted(measured)
        res = []
        for t in out.tokens:
            near = min(pts, key=lambda m: abs(math.log(m) - math.log(t)))
            res.append(measured[near] / profile._interp(synth, near))
        return res

    r_layer = ratios(layer_fwd_bwd_ms, profile.layer_fwd_bwd_ms)
    r_head = ratios(head_fwd_bwd_ms, profile.head_fwd_bwd_ms)
    out.layer_fwd_bwd_ms = [v * r for v, r in zip(profile.layer_fwd_bwd_ms, r_layer)]
    out.layer_fwd_ms = [v * fwd_share for v in out.layer_fwd_bwd_ms]
    out.head_fwd_bwd_ms = [v * r for v, r in zip(profile.head_fwd_bwd_ms, r_head)]
    return out


CONFIG_DIR = Path(__file__).resolve().parent / "configs"


def load_b200_profile(model: str) -> LoRALLMProfileResult:
    """Profile of ``model`` measured on B200 with this framework (``simulator/configs/*.yaml``,
    the counterpart of the reference's ``lorafusion/simulator/configs/*.yaml`` for H100)."""
    return LoRALLMProfileResult.load(CONFIG_DIR / f"{model}.yaml")


# ----------------------------------------------------------------------------------------
# collective cost model
# ----------------------------------------------------------------------------------------
def collective_time_ms(kind: str, nbytes: float, n: int, hw: HardwareSpec) -> float:
    """Alpha-beta model on a full-bandwidth NVSwitch domain.  ``kind`` is one of
    ``allreduce``, ``allgather``, ``reducescatter``, ``p2p`` (hyphens are accepted)."""
    kind = kind.replace("-", "").replace("_", "").lower()
    if n <= 1 and kind != "p2p":
        return 0.0
    lat = hw.collective_latency_us * 1e-3
    if kind == "allreduce":
        return lat + 2.0 * (n - 1) / n * nbytes / (hw.allreduce_bus_gbs * 1e9) * 1e3
    if kind in ("allgather", "reducescatter"):
        return lat + (n - 1) / n * nbytes / (hw.nvlink_gbs * 1e9) * 1e3
    if kind == "p2p":
        return hw.p2p_latency_us * 1e-3 + nbytes / (hw.nvlink_gbs * 1e9) * 1e3
    raise ValueError(f"unknown collective '{kind}'")


def overlap_time(compute_ms: float, comm_ms: float, overlap: float = 0.8) -> float:
    """Time of a compute phase with a communication phase of which ``overlap`` can hide."""
    hidden = min(comm_ms * overlap, compute_ms)
    return compute_ms + comm_ms - hidden


# ----------------------------------------------------------------------------------------
# predictor
# ----------------------------------------------------------------------------------------
@dataclass
class SimulationConfiguration:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    microbatch_tokens: int = 16384
    microbatches_per_step: int = 4            # per DP replica
    recompute_layers: Optional[int] = None    # None = all
    num_adapters: int = 4
    fused_tp_collectives: bool = True         # AG->GEMM / GEMM->RS overlapped inside the kernels
    zero3_base: bool = False                  # shard the frozen base over dp and gather per layer

    @property
    def world(self) -> int:
        return self.dp * self.tp * self.pp


@dataclass
class SimulationResult:
    step_ms: float
    tokens_per_s: float
    peak_memory_gb: float
    fits: bool
    stage_ms: list
    bubble_fraction: float
    breakdown: dict


class LoRALLMPredictor:
    def __init__(self, profile: LoRALLMProfileResult, hw: Optional[HardwareSpec] = None):
        self.p = profile
        self.hw = hw or HardwareSpec()

    def _layers_of_stage(self, s: int, pp: int) -> int:
        base, extra = divmod(self.p.num_layers, pp)
        return base + (1 if s < extra else 0)

    def stage_time_ms(self, c: SimulationConfiguration, s: int) -> tuple:
        p, hw = self.p, self.hw
        t = c.microbatch_tokens
        n_layers = self._layers_of_stage(s, c.pp)
        n_re = n_layers if c.recompute_layers is None else min(n_layers, c.recompute_layers)
        eff = hw.tp_efficiency.get(c.tp, min(hw.tp_efficiency.values()))
        fwd = p.layer_fwd(t) / c.tp / eff
        fb = p.layer_fwd_bwd(t) / c.tp / eff
        tp_comm = 0.0
        if c.tp > 1:
            act = t * p.hidden_size * 2
            per_layer = 4 * collective_time_ms("allgather", act, c.tp, hw) + \
                4 * collective_time_ms("reducescatter", act, c.tp, hw)
            tp_comm = per_layer
        z3 = 0.0
        if c.zero3_base and c.dp > 1:
            z3 = 2 * collective_time_ms("allgather", p.params_per_layer * p.weight_bytes_per_param / c.tp, c.dp, hw)
        layer = overlap_time(fb, tp_comm + z3, 0.9 if c.fused_tp_collectives else 0.0)
        total = n_layers * layer + n_re * fwd
        if s == c.pp - 1:
            total += p.head_fwd_bwd(t)
        return total, dict(layers=n_layers, recomputed=n_re, layer_ms=layer, tp_comm_ms=tp_comm)

    def memory_gb(self, c: SimulationConfiguration, s: int) -> float:
        p = self.p
        n_layers = self._layers_of_stage(s, c.pp)
        n_re = n_layers if c.recompute_layers is None else min(n_layers, c.recompute_layers)
        shard = c.tp * (c.dp if c.zero3_base else 1)
        weights = n_layers * p.params_per_layer * p.weight_bytes_per_param / shard
        if c.zero3_base:
            weights += 2 * p.params_per_layer * p.weight_bytes_per_param / c.tp
        if s == 0 or s == c.pp - 1:
            weights += p.embedding_params * 2
        lora = n_layers * p.lora_params_per_layer_per_adapter * c.num_adapters * 18 / c.tp
        inflight = c.pp - s
        t = c.microbatch_tokens
        acts = inflight * t * (n_re * p.checkpoint_bytes_per_token_per_layer +
                               (n_layers - n_re) * p.saved_bytes_per_token_per_layer / c.tp)
        peak = t * (p.peak_intermediate_bytes_per_token / c.tp + p.saved_bytes_per_token_per_layer / c.tp)
        if s == c.pp - 1:
            peak += min(t, 2048) * 2 * 2 * (p.embedding_params // p.hidden_size)
        return (weights + lora + acts + peak) / 1e9

    def estimate(self, c: SimulationConfiguration) -> SimulationResult:
        stages = [self.stage_time_ms(c, s) for s in range(c.pp)]
        stage_ms = [x[0] for x in stages]
        slow = max(stage_ms)
        m = c.microbatches_per_step
        p2p = collective_time_ms("p2p", c.microbatch_tokens * self.p.hidden_size * 2 / c.tp, 2, self.hw) if c.pp > 1 else 0.0
        step = (m + c.pp - 1) * slow + (2 * (c.pp - 1)) * p2p * 0.2 if c.pp > 1 else m * slow
        lora_bytes = self.p.num_layers / c.pp * self.p.lora_params_per_layer_per_adapter * c.num_adapters * 4 / c.tp
        dp_sync = collective_time_ms("allreduce", lora_bytes, c.dp, self.hw)
        step += dp_sync
        tokens = c.dp * m * c.microbatch_tokens
        mem = max(self.memory_gb(c, s) for s in range(c.pp))
        bubble = (c.pp - 1) / (m + c.pp - 1) if c.pp > 1 else 0.0
        return SimulationResult(step, tokens / (step / 1e3), mem, mem <= self.hw.memory_gb * 0.95, stage_ms,
                                bubble, dict(dp_sync_ms=dp_sync, p2p_ms=p2p, stages=[x[1] for x in stages]))


def optimization_configuration_generator(world: int, num_layers: int, *, microbatch_tokens: Sequence[int] = (4096, 8192, 16384),
                                         microbatches: Sequence[int] = (1, 2, 4, 8, 16)) -> Iterable[SimulationConfiguration]:
    """Enumerate power-of-two (dp, tp, pp) factorizations of ``world`` with a few microbatch
    settings and recomputation levels."""
    p2 = [1 << k for k in range(int(math.log2(world)) + 1)]
    for tp in p2:
        for pp in p2:
            if tp * pp > world or world % (tp * pp) or pp > num_layers:
                continue
            dp = world // (tp * pp)
            for t in microbatch_tokens:
                for m in microbatches:
                    if pp > 1 and m < pp:
                        continue
                    for re in (None, 0, num_layers // pp // 2):
                        yield SimulationConfiguration(dp=dp, tp=tp, pp=pp, microbatch_tokens=t,
                                                      microbatches_per_step=m, recompute_layers=re)


def best_configurations(predictor: LoRALLMPredictor, world: int, top: int = 5, **kw) -> list:
    scored = []
    for c in optimization_configuration_generator(world, predictor.p.num_layers, **kw):
        r = predictor.estimate(c)
        if r.fits:
            scored.append((r.tokens_per_s, c, r))
    scored.sort(key=lambda x: -x[0])
    return scored[:top]


# ----------------------------------------------------------------------------------------
# GPU profiler
# ----------------------------------------------------------------------------------------
class LoRALLMProfiler:
    """Measures a profile on the current GPU with 1- and 2-layer truncated models (per-layer
    time is the difference, as in ``mono.py:515-978``)."""

    def __init__(self, cfg: ModelConfig | str, adapters: Optional[Sequence[AdapterSpec]] = None, *,
                 quantize: bool = False, device: str = "cuda", tokens: Sequence[int] = TOKEN_GRID,
                 seq_len: int = 1024):
        self.cfg = get_model_config(cfg) if isinstance(cfg, str) else cfg
        self.adapters = list(adapters) if adapters else [AdapterSpec("lora_0", r=16, dropout=0.1)]
        self.quantize, self.device, self.tokens, self.seq_len = quantize, device, list(tokens), seq_len

    def _time_model(self, n_layers: int, tokens: int, backward: bool, iters: int = 3) -> float:
        import torch

        from ..models.decoder import DecoderStage
        from ..train.data import MicroBatchSpec, build_packed_batch

        stage = DecoderStage(self.cfg.with_layers(n_layers), self.adapters, self.device, quantize=self.quantize,
                             recompute=False, init_b_std=0.01, with_optimizer_state=False)
        n_seq = max(1, tokens // self.seq_len)
        lens = [tokens // n_seq] * n_seq
        batch = build_packed_batch(MicroBatchSpec([(0, lens)]), self.adapters, self.cfg.vocab_size, self.device)
        times = []
        for it in range(iters + 3):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if backward:
                stage.forward_backward(batch)
            else:
                stage.forward(batch)
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        del stage
        torch.cuda.empty_cache()
        return float(np.median(times))

    def profile(self) -> LoRALLMProfileResult:
        base = synthesize_profile(self.cfg, quantized=self.quantize, lora_rank=self.adapters[0].r,
                                  mean_seq_len=self.seq_len)
        fwd, fb, head = [], [], []
        for t in self.tokens:
            f1, f2 = self._time_model(1, t, False), self._time_model(2, t, False)
            b1, b2 = self._time_model(1, t, True), self._time_model(2, t, True)
            fwd.append(max(f2 - f1, 1e-3))
            fb.append(max(b2 - b1, 1e-3))
            head.append(max(b1 - (b2 - b1), 1e-3))
        base.tokens, base.layer_fwd_ms, base.layer_fwd_bwd_ms, base.head_fwd_bwd_ms = list(self.tokens), fwd, fb, head
        return base
