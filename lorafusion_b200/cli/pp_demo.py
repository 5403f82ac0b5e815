"""Pipeline partitioning demo on ONE GPU: split a model into stages, run them back to back and
check that the chained stages reproduce the unpartitioned model (loss and LoRA gradients).

    python -m lorafusion_b200.cli.pp_demo --model small --stages 4

Counterpart of ``lorafusion/pipeline_parallel/demo.py`` (four ``PipeModel`` stages executed
sequentially on one device).  The stages here are the same :class:`DecoderStage` objects the
multi-GPU runtime drives; activations and their gradients are handed over as plain tensors.
"""

from __future__ import annotations

import argparse
import json

import torch

from ..models.config import AdapterSpec, get_model_config
from ..models.decoder import DecoderStage
from ..ops import _native
from ..parallel.pipeline import PipeModel
from ..train.data import MicroBatchSpec, build_packed_batch


def run(model: str = "small", stages: int = 4, device: str = "cuda:0", seed: int = 0) -> dict:
    cfg = get_model_config(model)
    adapters = [AdapterSpec("lora_0", r=16, dropout=0.1), AdapterSpec("lora_1", r=8, dropout=0.0)]
    kw = dict(init_b_std=0.01, seed=seed, recompute=True, with_optimizer_state=False)
    whole = DecoderStage(cfg, adapters, device, **kw)
    parts = [PipeModel.from_model(whole, stage_idx=s, num_stages=stages, **kw) for s in range(stages)]
    batch = build_packed_batch(MicroBatchSpec([(0, [300, 84]), (1, [128, 200])]), adapters, cfg.vocab_size,
                               device, seed=seed)
    loss_whole = float(whole.forward_backward(batch))
    # forward through the chain, keeping what each stage saved
    h, saved = None, []
    for st in parts:
        h, sv = st.forward(batch, h)
        saved.append(sv)
    loss, dh = parts[-1].loss_and_grad(h, batch)
    for st, sv in zip(reversed(parts), reversed(saved)):
        dh = st.backward(sv, dh, batch)
    torch.cuda.synchronize()
    _native.check_device_errors()
    # LoRA gradients of stage s must equal the whole model's gradients of the same layers
    worst = 0.0
    for st in parts:
        for (layer, proj), v in st.arena.views.items():
            ref = whole.arena.views[(layer, proj)].stack
            for got, exp in ((v.stack.da, ref.da), (v.stack.db, ref.db)):
                scale = float(exp.abs().max()) + 1e-12
                worst = max(worst, float((got - exp).abs().max()) / scale)
    return {"model": cfg.name, "stages": stages, "layers_per_stage": [p.layer_end - p.layer_start for p in parts],
            "loss_whole": loss_whole, "loss_chained": float(loss), "max_rel_grad_diff": worst}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="small")
    ap.add_argument("--stages", type=int, default=4)
    args = ap.parse_args(argv)
    res = run(args.model, args.stages)
    print(json.dumps(res))
    if abs(res["loss_whole"] - res["loss_chained"]) > 1e-3 * abs(res["loss_whole"]) or res["max_rel_grad_diff"] > 2e-2:
        raise SystemExit("chained stages disagree with the unpartitioned model")
    return res


if __name__ == "__main__":
    main()
