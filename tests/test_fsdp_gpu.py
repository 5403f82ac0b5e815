"""ZeRO-3 style baseline stage (base weights sharded, gathered per layer): identical results to
the replicated stage, on one GPU (a single shard) and on two real ranks."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_BODY = r"""
import torch
from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.models.decoder import DecoderStage
from lorafusion_b200.models.fsdp_decoder import FsdpDecoderStage
from lorafusion_b200.train.data import MicroBatchSpec, build_packed_batch
from lorafusion_b200.ops import _native


def compare(dev, group, world):
    cfg = get_model_config("tiny")
    adapters = [AdapterSpec("lora_0", r=16, lora_alpha=32, dropout=0.1), AdapterSpec("lora_1", r=8, lora_alpha=16)]
    batch = build_packed_batch(MicroBatchSpec([(0, [100, 37, 200]), (1, [129, 64])]), adapters, cfg.vocab_size, dev, seed=5)
    for quantize in (False, True):
        for recompute in (False, True):
            kw = dict(quantize=quantize, init_b_std=0.02, seed=3, recompute=recompute)
            full = DecoderStage(cfg, adapters, dev, **kw)
            sharded = FsdpDecoderStage(cfg, adapters, dev, group, **kw)
            assert sharded.base_weight_bytes() <= full.base_weight_bytes() // world + 4 * 4 * 256
            for _ in range(2):   # two microbatches: the gather buffers are reused
                l1 = full.forward_backward(batch)
                l2 = sharded.forward_backward(batch)
            torch.cuda.synchronize()
            _native.check_device_errors()
            assert float(l1) == float(l2), (quantize, recompute, float(l1), float(l2))
            assert torch.equal(full.arena.grad, sharded.arena.grad), (quantize, recompute)
            layers = len(full.layers)
            # forward + backward gather every layer once each per microbatch
            assert sharded.gathered_bytes == 2 * 2 * sum(s.total for s in sharded._sharded), sharded.gathered_bytes
            assert all(lw.qkv is None for lw in sharded.layers) and layers == len(sharded._sharded)
"""


def test_single_shard_equals_replicated_stage():
    ns = {}
    exec(_BODY, ns)
    ns["compare"]("cuda", None, 1)


_CHILD = _BODY + r"""
import os, torch.distributed as dist
os.environ["NCCL_NVLS_ENABLE"] = "0"
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
compare(dev, dist.group.WORLD, world)
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_gather_their_shards(tmp_path):
    script = tmp_path / "child_fsdp.py"
    script.write_text(_CHILD)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                   PYTHONPATH=os.pathsep.join([os.getcwd(), os.environ.get("PYTHONPATH", "")]))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-3000:]}"
