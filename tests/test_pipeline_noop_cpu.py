"""No-op microbatches as pipeline slots, the run-time bubble-lemma assertion and the per-slot
health check of the pipeline runtime (gloo CPU ranks, no GPU needed).

A toy stage keeps one weight chain PER ADAPTER, recomputes its forward inside the backward
(like activation recomputation does) and takes an SGD step whenever the manager says an
adapter finished a global batch.  If a microbatch of global batch ``g + 1`` went forward
before the step of batch ``g``, its backward would recompute with other weights than its
forward used and the final weights would differ from the single-process run."""

import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lorafusion_b200.parallel.layout import ParallelLayout, ParallelState, initialize_parallel_state
from lorafusion_b200.parallel.pipeline import (BubbleLemmaError, PipelineMicrobatch, PipelineRuntime,
                                               check_bubble_lemma, even_layer_partition)
from lorafusion_b200.solver import schedule as S
from lorafusion_b200.train.manager import MultiLoRAManager

HIDDEN, LR, PP = 8, 0.05, 4
N_ADAPTERS, N_LAYERS = 2, 8


class AdapterToyStage:
    def __init__(self, layer_range, is_first, is_last):
        g = torch.Generator().manual_seed(7)
        allw = [[torch.randn(HIDDEN, HIDDEN, generator=g) * 0.4 for _ in range(N_LAYERS)] for _ in range(N_ADAPTERS)]
        s, e = layer_range
        self.w = {a: [w.clone().requires_grad_(True) for w in allw[a][s:e]] for a in range(N_ADAPTERS)}
        self.is_first, self.is_last = is_first, is_last

    def _chain(self, x, batch):
        outs = []
        for a, s, e in batch.segs:
            h = x[s:e]
            for w in self.w[a]:
                h = torch.tanh(h @ w)
            outs.append(h)
        return torch.cat(outs)

    def forward(self, batch, h_in):
        x = (batch.x if self.is_first else h_in).detach()
        with torch.no_grad():
            h = self._chain(x, batch)
        return h, x

    def loss_and_grad(self, out, batch):
        return (out ** 2).sum(), 2 * out

    def backward(self, saved, dh, batch):
        x = saved.clone().requires_grad_(True)
        self._chain(x, batch).backward(dh)  # recomputed with the weights of NOW
        return None if self.is_first else x.grad

    def step(self, adapter, num_microbatches):
        with torch.no_grad():
            for w in self.w[adapter]:
                w -= LR * w.grad / num_microbatches
                w.grad = None


def _schedule():
    """Two adapters, three global batches each, one microbatch per (adapter, batch): without
    no-ops consecutive global batches of an adapter are two slots apart, far less than PP."""
    data = [[[4, 4] for _ in range(3)] for _ in range(N_ADAPTERS)]
    steps = []
    for g in range(3):
        for a in range(N_ADAPTERS):
            mb = S.MicroBatchInfo({(a, g, k): 4 for k in range(2)}, 1024, 1)
            steps.append(S.AdapterGroupStepInfo.from_micro_batch_infos_list([mb]))
    ok, msgs, fixed = S.verify_correctness_of_schedule(data, steps, PP, add_bubble=True)
    assert ok, msgs
    flat = S.flatten_schedule(fixed)
    assert any(m.is_empty_marker for m in flat)
    return flat


def _pipeline_microbatches(flat):
    g = torch.Generator().manual_seed(11)
    out = []
    for mbi in flat:
        if mbi.is_empty_marker:
            out.append(PipelineMicrobatch(None, 0, is_empty=True))
            continue
        segs, rows = [], 0
        for a, lens in mbi.segments():
            segs.append((a, rows, rows + sum(lens)))
            rows += sum(lens)
        info = SimpleNamespace(micro_batch_info=mbi, allow_empty_micro_batch_info=False, microbatch_idx=None)
        batch = SimpleNamespace(x=torch.randn(rows, HIDDEN, generator=g), segs=segs, info=info, num_real_tokens=rows)
        out.append(PipelineMicrobatch(batch, rows))
    return out


def _manager(stage, pp):
    from lorafusion_b200.models.config import AdapterSpec

    mgr = MultiLoRAManager([AdapterSpec(f"a{i}") for i in range(N_ADAPTERS)], pp, 1024, [2] * N_ADAPTERS)
    mgr.register_step_fn(stage.step)
    return mgr


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, drop_noops, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        state = initialize_parallel_state(ParallelLayout(world, dp=1, pp=world, tp=1))
        fwd_g, bwd_g = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
        stage = AdapterToyStage(even_layer_partition(N_LAYERS, world)[rank], rank == 0, rank == world - 1)
        mgr = _manager(stage, world)
        rt = PipelineRuntime(stage, state, hidden_size=HIDDEN, dtype=torch.float32, device="cpu", manager=mgr,
                             fwd_group=fwd_g, bwd_group=bwd_g)
        mbs = _pipeline_microbatches(_schedule())
        if drop_noops:
            mbs = [m for m in mbs if not m.is_empty]
        try:
            rt.run(mbs)
            res = ("ok", {a: [w.detach().clone() for w in ws] for a, ws in stage.w.items()}, dict(mgr.steps_taken),
                   list(rt.executed_ops))
        except BubbleLemmaError as e:
            res = ("lemma", str(e), None, None)
        out_q.put((rank, res))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _run_ranks(drop_noops):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, PP, port, drop_noops, q)) for r in range(PP)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=180) for _ in range(PP))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return results


def _single_process_reference():
    stage = AdapterToyStage((0, N_LAYERS), True, True)
    mgr = _manager(stage, 1)
    state = ParallelState(ParallelLayout(1, dp=1, pp=1, tp=1), 0, 0, 0, 0)
    rt = PipelineRuntime(stage, state, hidden_size=HIDDEN, dtype=torch.float32, device="cpu", manager=mgr)
    rt.run(_pipeline_microbatches(_schedule()))
    return stage, mgr


def test_noop_slots_keep_weights_identical_to_single_process():
    ref, ref_mgr = _single_process_reference()
    assert ref_mgr.steps_taken == {0: 3, 1: 3}
    results = _run_ranks(drop_noops=False)
    parts = even_layer_partition(N_LAYERS, PP)
    n_slots = len(_schedule())
    for r, (s, e) in enumerate(parts):
        kind, weights, steps, ops = results[r]
        assert kind == "ok" and steps == {0: 3, 1: 3}
        # every slot, empty or not, has exactly one forward and one backward position
        assert sorted(i for k, i, _ in ops if k == "F") == list(range(n_slots))
        assert sorted(i for k, i, _ in ops if k == "B") == list(range(n_slots))
        assert any(empty for _, _, empty in ops)
        for a in range(N_ADAPTERS):
            for got, want in zip(weights[a], ref.w[a][s:e]):
                assert torch.allclose(got, want.detach(), rtol=1e-5, atol=1e-6)


def test_order_without_the_noops_is_refused_on_every_stage():
    results = _run_ranks(drop_noops=True)
    for r in range(PP):
        assert results[r][0] == "lemma" and "bubble lemma" in results[r][1]


def test_solver_schedules_satisfy_the_lemma_with_noops_and_not_without():
    import random

    rng = random.Random(5)
    with_noops = violating_when_filtered = 0
    for trial in range(12):
        n_adapters = rng.choice([1, 2, 3])
        data = [[[rng.choice([64, 128, 256, 512, 1024]) for _ in range(rng.choice([2, 4]))] for _ in range(3)]
                for _ in range(n_adapters)]
        groups = S.group_adapters(data, 2048, num_stages=PP)
        packed = S.packing_data_to_microbatches_micro_milp(data, groups, 2048, PP, time_limit=0.05, use_exact=False,
                                                           num_workers=1)
        merged = S.apply_merge_pass_for_adapter_group_step_infos(packed, PP)
        ok, msgs, fixed = S.verify_correctness_of_schedule(data, merged, PP, add_bubble=True)
        assert ok, msgs
        flat = S.flatten_schedule(fixed)
        mbs = [PipelineMicrobatch(None, 0, is_empty=True) if m.is_empty_marker else
               PipelineMicrobatch(SimpleNamespace(info=SimpleNamespace(micro_batch_info=m)), m.padded_total_tokens)
               for m in flat]
        check_bubble_lemma(mbs, PP)  # the order the runtime executes: no violation
        if any(m.is_empty for m in mbs):
            with_noops += 1
            try:
                check_bubble_lemma([m for m in mbs if not m.is_empty], PP)
            except BubbleLemmaError:
                violating_when_filtered += 1
    assert with_noops > 0 and violating_when_filtered == with_noops


def test_peer_failure_is_noticed_between_microbatch_slots():
    """Rank 1 leaves a failure note while rank 0 is in the middle of a schedule: rank 0 raises
    at its next slot instead of finishing the schedule (single process, in-memory store)."""
    from lorafusion_b200.parallel.health import HealthMonitor, PeerFailure

    store = dist.HashStore()
    mine = HealthMonitor(store, 0, 2, timeout=60.0)
    peer = HealthMonitor(store, 1, 2, timeout=60.0)
    mine.beat()
    peer.beat()

    class Stage(AdapterToyStage):
        calls = 0

        def forward(self, batch, h_in):
            Stage.calls += 1
            if Stage.calls == 2:
                peer.report_failure("RuntimeError: boom")
            return super().forward(batch, h_in)

    stage = Stage((0, N_LAYERS), True, True)
    state = ParallelState(ParallelLayout(1, dp=1, pp=1, tp=1), 0, 0, 0, 0)
    rt = PipelineRuntime(stage, state, hidden_size=HIDDEN, dtype=torch.float32, device="cpu",
                         manager=_manager(stage, 1), health=mine)
    with pytest.raises(PeerFailure) as err:
        rt.run(_pipeline_microbatches(_schedule()))
    assert err.value.ranks == [1] and "boom" in str(err.value)
    # the second forward ran; the check in front of its backward slot raised
    assert [op[0] for op in rt.executed_ops] == ["F", "B", "F"] and Stage.calls == 2
    assert store.get("lf_health/prog/0") == b"4"
