"""Pipeline runtime on gloo CPU ranks with a toy stage, pipeline simulator invariants, layout
arithmetic and the multi-LoRA manager (no GPU needed)."""

import os
import socket
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lorafusion_b200.parallel.layout import ParallelLayout, initialize_parallel_state
from lorafusion_b200.parallel.pipeline import (PipelineMicrobatch, PipelineRuntime, even_layer_partition,
                                               get_pipeline_stage_layer_indices)
from lorafusion_b200.simulator import pipeline_sim as ps
from lorafusion_b200.train.manager import MultiLoRAManager

HIDDEN = 16


class ToyStage:
    """tanh(x W) layers with autograd; first stage reads the batch, last stage has an MSE-like loss."""

    def __init__(self, weights, is_first, is_last):
        self.w = [w.clone().requires_grad_(True) for w in weights]
        self.is_first, self.is_last = is_first, is_last

    def forward(self, batch, h_in):
        x = batch.x if self.is_first else h_in.detach().requires_grad_(True)
        h = x
        for w in self.w:
            h = torch.tanh(h @ w)
        return h, (x, h)

    def loss_and_grad(self, out, batch):
        leaf = out.detach().requires_grad_(True)
        loss = (leaf ** 2).sum()
        loss.backward()
        return loss.detach(), leaf.grad

    def backward(self, saved, dh, batch):
        x, h = saved
        h.backward(dh)
        return None if self.is_first else x.grad


def _weights(n_layers):
    g = torch.Generator().manual_seed(0)
    return [torch.randn(HIDDEN, HIDDEN, generator=g) * 0.3 for _ in range(n_layers)]


def _batches():
    g = torch.Generator().manual_seed(1)
    toks = [8, 24, 0, 16, 8, 32]  # 0 = empty no-op microbatch
    return [PipelineMicrobatch(SimpleNamespace(x=torch.randn(t, HIDDEN, generator=g), info=None,
                                               num_real_tokens=t), t, is_empty=(t == 0)) for t in toks]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_layers, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layout = ParallelLayout(world, dp=1, pp=world, tp=1)
    state = initialize_parallel_state(layout)
    fwd_g, bwd_g = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
    s, e = even_layer_partition(n_layers, world)[rank]
    stage = ToyStage(_weights(n_layers)[s:e], rank == 0, rank == world - 1)
    rt = PipelineRuntime(stage, state, hidden_size=HIDDEN, dtype=torch.float32, device="cpu",
                         fwd_group=fwd_g, bwd_group=bwd_g)
    stats = rt.run(_batches())
    out_q.put((rank, [w.grad.clone() for w in stage.w], float(stats.loss_sum) if rank == world - 1 else None))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_1f1b_matches_single_process(world):
    n_layers = 6
    ref = ToyStage(_weights(n_layers), True, True)
    ref_loss = 0.0
    for mb in _batches():
        if mb.is_empty:
            continue
        out, saved = ref.forward(mb.batch, None)
        loss, dh = ref.loss_and_grad(out, mb.batch)
        ref.backward(saved, dh, mb.batch)
        ref_loss += float(loss)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_layers, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        r, grads, loss = q.get(timeout=120)
        results[r] = (grads, loss)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    parts = even_layer_partition(n_layers, world)
    for r, (s, e) in enumerate(parts):
        for g, w in zip(results[r][0], ref.w[s:e]):
            assert torch.allclose(g, w.grad, rtol=1e-5, atol=1e-6)
    assert abs(results[world - 1][1] - ref_loss) < 1e-3 * abs(ref_loss)


def test_layer_partition_and_layout():
    assert even_layer_partition(80, 4) == [(0, 20), (20, 40), (40, 60), (60, 80)]
    assert even_layer_partition(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert get_pipeline_stage_layer_indices(10, 4, 2) == [6, 7]
    lay = ParallelLayout.parse("tp4pp2", 8)
    assert (lay.dp, lay.pp, lay.tp) == (1, 2, 4)
    assert lay.tp_group_ranks(5) == [4, 5, 6, 7] and lay.pp_group_ranks(5) == [1, 5]
    lay = ParallelLayout.parse("pp4", 8)
    assert (lay.dp, lay.pp, lay.tp) == (2, 4, 1)
    assert lay.coords(5) == (2, 1, 0) and lay.dp_group_ranks(5) == [4, 5]
    assert sorted(r for g in lay.all_groups("pp") for r in g) == list(range(8))
    with pytest.raises(ValueError):
        ParallelLayout(8, dp=3, pp=2, tp=1)


def test_simulator_invariants_and_balanced_pipeline():
    rng = np.random.default_rng(0)
    fwd = rng.uniform(0.5, 2.0, (12, 4))
    bwd = 2 * fwd
    tl = ps.simulate_1f1b(fwd, bwd)
    assert not ps.find_overlaps(tl) and not ps.check_forward_backward_constraints(tl)
    assert 0.0 <= tl.bubble_ratio < 1.0
    # perfectly balanced: makespan = (M + S - 1) * (f + b), bubble = (S-1)/(M+S-1)
    M, S = 16, 4
    tl = ps.simulate_1f1b(np.ones((M, S)), 2 * np.ones((M, S)))
    assert abs(tl.total_time - (M + S - 1) * 3.0) < 1e-9
    assert abs(tl.bubble_ratio - (S - 1) / (M + S - 1)) < 1e-9
    assert tl.adjusted_bubble_ratio() < 1e-9


def test_solver_schedule_beats_naive_in_simulation():
    data = ps.generate_data(4, 4, 8, median=[256, 512, 1024, 2048], sigma=[0.5, 0.6, 0.7, 0.8], seed=3)
    res = ps.compare_schedules(data, 8192, 4, time_limit=0.2)
    assert set(res) == {"naive", "sorted", "mlora", "solver"}
    assert res["solver"]["tokens_per_time"] >= 0.99 * res["naive"]["tokens_per_time"]
    assert res["solver"]["microbatches"] <= res["naive"]["microbatches"] + 3 * 4


def test_manager_inflight_order_and_steps():
    from lorafusion_b200.models.config import AdapterSpec

    stepped = []
    mgr = MultiLoRAManager([AdapterSpec("a"), AdapterSpec("b")], 2, 4096, [4, 2], dp_size=1)
    mgr.register_step_fn(lambda a, n: stepped.append((a, n)))

    def info(counts):
        mbi = SimpleNamespace(adapter_num_samples_pairs=counts)
        return SimpleNamespace(micro_batch_info=mbi, allow_empty_micro_batch_info=False, microbatch_idx=None)

    i0, i1 = info({0: 2, 1: 2}), info({0: 2})
    mgr.add_batch_info(i0)
    mgr.add_batch_info(i1)
    with pytest.raises(ValueError):
        mgr.add_batch_info(info({0: 1}))  # more in flight than pipeline stages
    mgr.mark_forward_pass_started()
    assert mgr.get_current_batch_info() is i1
    mgr.mark_backward_pass_started()
    assert mgr.get_current_batch_info() is i0
    assert mgr.pop_oldest_batch_info() is i0
    assert mgr.maybe_reduce_grad_and_optimizer_step() == [1] and stepped == [(1, 1)]
    assert mgr.pop_oldest_batch_info() is i1
    assert mgr.maybe_reduce_grad_and_optimizer_step() == [0] and stepped[-1] == (0, 2)
    assert mgr.adapter_sample_counts == {0: 0, 1: 0} and i1.microbatch_idx == 1


def test_latency_minimising_order_search():
    """Exact search on small instances is a lower bound for every other order; the local search
    on larger ones never loses to the sorted or the given order; precedence pairs are kept."""
    import itertools
    import random

    from lorafusion_b200.simulator.pipeline_sim import (evaluate_schedule_pipeline_parallelism,
                                                        solve_schedule_order)

    rng = random.Random(3)
    toks = [rng.choice([1024, 2048, 4096, 8192, 12000]) for _ in range(6)]
    sol = solve_schedule_order(toks, 3)
    assert sol.method == "exact" and sorted(sol.order) == list(range(6))
    brute = min(evaluate_schedule_pipeline_parallelism([toks[i] for i in p], 3).total_time
                for p in itertools.permutations(range(6)))
    assert sol.total_time == pytest.approx(brute)
    # precedence: 5 before 0 and 0 before 3
    solp = solve_schedule_order(toks, 3, precedence=[(5, 0), (0, 3)])
    assert solp.order.index(5) < solp.order.index(0) < solp.order.index(3)
    assert solp.total_time >= sol.total_time - 1e-9
    big = [rng.choice([1024, 2048, 4096, 8192, 16384]) for _ in range(30)]
    solb = solve_schedule_order(big, 4, time_limit=0.3)
    assert solb.method == "local-search" and sorted(solb.order) == list(range(30))
    for ref in (big, sorted(big), sorted(big, reverse=True)):
        assert solb.total_time <= evaluate_schedule_pipeline_parallelism(ref, 4).total_time + 1e-9
    with pytest.raises(ValueError):
        solve_schedule_order(toks, 3, precedence=[(0, 1), (1, 0)])
