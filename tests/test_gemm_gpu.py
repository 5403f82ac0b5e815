"""GPU numerics of the tcgen05 GEMM family and the LoRA kernel building blocks against
plain fp32 PyTorch."""

import pytest
import torch

from lorafusion_b200.utils.testing import assert_close_two_rounds

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(
        torch.bfloat16)


def _f32mm(a, b):
    torch.backends.cuda.matmul.allow_tf32 = False
    return a.float() @ b.float()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 520, 200),
                                   (1024, 1024, 1024), (4097, 384, 4096)])
def test_gemm_nt(M, N, K):
    from lorafusion_b200.ops.gemm import gemm_nt

    a, b = _rand(M, K, seed=1), _rand(N, K, scale=0.05, seed=2)
    bias = _rand(N, seed=3)
    out = gemm_nt(a, b, bias=bias)
    ref = _f32mm(a, b.t()) + bias.float()
    assert_close_two_rounds(out, ref, msg=f"gemm_nt {M}x{N}x{K}")


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 520, 200),
                                   (2048, 1024, 4096)])
def test_gemm_nn(M, N, K):
    from lorafusion_b200.ops.gemm import gemm_nn

    a, b = _rand(M, K, seed=4), _rand(K, N, scale=0.05, seed=5)
    out = gemm_nn(a, b)
    assert_close_two_rounds(out, _f32mm(a, b), msg=f"gemm_nn {M}x{N}x{K}")


def _adapters(n, N, K, R=64, ranks=(16, 16, 32, 64), seed=10):
    a_all = torch.zeros(n, R, K, device="cuda", dtype=torch.bfloat16)
    b_all = torch.zeros(n, N, R, device="cuda", dtype=torch.bfloat16)
    for i in range(n):
        r = ranks[i % len(ranks)]
        a_all[i, :r] = _rand(r, K, scale=0.02, seed=seed + i)
        b_all[i, :, :r] = _rand(N, r, scale=0.02, seed=seed + 100 + i)
    return a_all, b_all


def _tile_adapters(seg_adapters, seg_tiles):
    ids = []
    for a, nt in zip(seg_adapters, seg_tiles):
        ids += [a] * nt
    return torch.tensor(ids, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("p", [0.0, 0.1])
def test_lora_linear_blocks(p):
    """All six building blocks on a 4-adapter packed batch, with and without dropout."""
    from lorafusion_b200.ops import lora_kernels as lk
    from lorafusion_b200.ops.philox import keep_mask

    N, K, n = 768, 1024, 4
    seg_adapters, seg_tiles = [2, 0, -1, 3, 1], [2, 1, 1, 3, 2]
    M = 128 * sum(seg_tiles)
    tile_adapter = _tile_adapters(seg_adapters, seg_tiles)
    alphas = torch.tensor([2.0, 1.0, 0.5, 0.25], device="cuda")
    x, w = _rand(M, K, seed=20), _rand(N, K, scale=0.03, seed=21)
    dy = _rand(M, N, seed=22)
    a_all, b_all = _adapters(n, N, K)
    drop = lk.DropoutSpec(seed=1234, stream_id=7, p=p)

    # ---- fp32 oracle ----
    keep = keep_mask(M, K, p, 1234, 7).cuda()
    inv = 1.0 / (1.0 - p)
    xh = torch.where(keep, x.float() * inv, torch.zeros((), device="cuda")).to(torch.bfloat16)
    row_adapter = tile_adapter.repeat_interleave(128).long()
    s_ref = torch.zeros(M, 64, device="cuda")
    ds_ref = torch.zeros(M, 64, device="cuda")
    for a in range(n):
        rows = row_adapter == a
        s_ref[rows] = alphas[a] * _f32mm(xh[rows], a_all[a].t())
        ds_ref[rows] = alphas[a] * _f32mm(dy[rows], b_all[a])

    s = lk.lora_down(x, a_all, tile_adapter=tile_adapter, adapter_scale=alphas, dropout=drop)
    assert_close_two_rounds(s, s_ref, msg="lora_down")
    ds = lk.lora_ds(dy, b_all, tile_adapter=tile_adapter, adapter_scale=alphas)
    assert_close_two_rounds(ds, ds_ref, msg="lora_ds")

    y = lk.base_lora_fwd(x, w, s, b_all, tile_adapter=tile_adapter)
    y_ref = _f32mm(x, w.t())
    dx_ref = _f32mm(dy, w)
    for a in range(n):
        rows = row_adapter == a
        y_ref[rows] += _f32mm(s[rows], b_all[a].t())
        dx_ref[rows] += torch.where(keep[rows], _f32mm(ds[rows], a_all[a]) * inv,
                                    torch.zeros((), device="cuda"))
    assert_close_two_rounds(y, y_ref, msg="base_lora_fwd")
    dx = lk.base_lora_dx(dy, w, ds, a_all, tile_adapter=tile_adapter, dropout=drop)
    assert_close_two_rounds(dx, dx_ref, msg="base_lora_dx")

    segs, start = [], 0
    for a, nt in zip(seg_adapters, seg_tiles):
        segs.append((a, start, start + 128 * nt))
        start += 128 * nt
    table = lk.SegmentTable(segs, torch.device("cuda"))
    da_all = torch.zeros(n, 64, K, device="cuda")
    db_all = torch.zeros(n, N, 64, device="cuda")
    for _ in range(2):  # accumulate twice: checks the += semantics
        lk.lora_db(dy, s, table, db_all)
        lk.lora_da(x, ds, table, da_all, dropout=drop)
    for a in range(n):
        rows = row_adapter == a
        assert_close_two_rounds(db_all[a], 2 * _f32mm(dy[rows].t(), s[rows]), rtol=1e-3,
                                atol=1e-2, msg=f"lora_db[{a}]")
        assert_close_two_rounds(da_all[a], 2 * _f32mm(ds[rows].t(), xh[rows]), rtol=1e-3,
                                atol=1e-2, msg=f"lora_da[{a}]")


@pytest.mark.parametrize("mixed_p", [False, True])
def test_gradient_kernels_split_long_segments_into_chunks(mixed_p):
    """Two long segments and few feature tiles: the work list is cut into token chunks that write
    partial sums, folded in a fixed order.  Same results as fp32 math, and bitwise the same from
    run to run."""
    from lorafusion_b200.ops import lora_kernels as lk
    from lorafusion_b200.ops.philox import keep_mask

    N, K, n, R = 256, 384, 2, 64
    segs = [(1, 0, 3072), (0, 3072, 5248)]          # 5 feature tiles at most -> 10 work items uncut
    M = 5248
    x, dy = _rand(M, K, seed=40), _rand(M, N, seed=41)
    s, ds = _rand(M, R, scale=0.1, seed=42), _rand(M, R, scale=0.1, seed=43)
    table = lk.SegmentTable(segs, torch.device("cuda"), total_rows=M)
    plan = table.split_plan(K)
    assert plan is not None and len(plan[1]) > 2 and plan[1] == sorted(plan[1], reverse=True)
    ps = [0.1, 0.2] if mixed_p else [0.1, 0.1]
    if mixed_p:
        from lorafusion_b200.ops.philox import dropout_threshold
        drop = lk.DropoutSpec(seed=77, stream_id=3, p=0.0,
                              adapter_thresh16=torch.tensor([dropout_threshold(q) for q in ps], dtype=torch.int32,
                                                            device="cuda"),
                              adapter_inv_keep=torch.tensor([1 / (1 - q) for q in ps], device="cuda"))
    else:
        drop = lk.DropoutSpec(seed=77, stream_id=3, p=0.1)
    outs = []
    for _ in range(2):
        da_all = torch.zeros(n, R, K, device="cuda")
        db_all = torch.zeros(n, N, R, device="cuda")
        lk.lora_db(dy, s, table, db_all)
        lk.lora_da(x, ds, table, da_all, dropout=drop)
        outs.append((da_all, db_all))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    da_all, db_all = outs[0]
    for a, r0, r1 in segs:
        keep = keep_mask(M, K, ps[a], 77, 3).cuda()[r0:r1]
        xh = torch.where(keep, x[r0:r1].float() / (1 - ps[a]), torch.zeros((), device="cuda")).to(torch.bfloat16)
        assert_close_two_rounds(db_all[a], _f32mm(dy[r0:r1].t(), s[r0:r1]), rtol=1e-3, atol=2e-2, msg=f"split lora_db[{a}]")
        assert_close_two_rounds(da_all[a], _f32mm(ds[r0:r1].t(), xh), rtol=1e-3, atol=2e-2, msg=f"split lora_da[{a}]")


@pytest.mark.parametrize("N", [768, 64])
def test_pair_dx_dropout_walks_many_tiles_per_pair(N):
    """The CTA-pair dX kernel with dropout puts the LoRA slab of the NEXT tile into the other
    accumulator in the middle of the current main loop and masks it in place.  With four pairs and
    twenty tiles every pair runs that hand-over several times; adapters differ inside a pair, one
    has no dropout, one row tile has no adapter, and the last pair is half empty.  ``N = 64`` is
    the single-main-block edge (the next slab is issued before the main product)."""
    from lorafusion_b200.ops import lora_kernels as lk
    from lorafusion_b200.ops import _native as nv
    from lorafusion_b200.ops.gemm import launch_gemm
    from lorafusion_b200.ops.philox import dropout_threshold, keep_mask

    K, n, R = 1024, 4, 64
    seg_adapters, seg_tiles = [2, 0, -1, 3, 1], [2, 1, 1, 3, 2]
    M = 128 * sum(seg_tiles)
    tile_adapter = _tile_adapters(seg_adapters, seg_tiles)
    ps = [0.1, 0.0, 0.2, 0.3]
    dy, w = _rand(M, N, seed=50), _rand(N, K, scale=0.03, seed=51)
    ds = _rand(M, R, scale=0.1, seed=52)
    a_all, _ = _adapters(n, N, K)
    drop = lk.DropoutSpec(seed=99, stream_id=5, p=0.0,
                          adapter_thresh16=torch.tensor([dropout_threshold(q) for q in ps], dtype=torch.int32,
                                                        device="cuda"),
                          adapter_inv_keep=torch.tensor([1 / (1 - q) for q in ps], device="cuda"))
    out = torch.full((M, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    launch_gemm(pair=True, a=dy, b=w, out=out, M=M, N=K, K=N, b_mn=True, b2_mn=True, bn=256, nacc=2,
                epi=nv.EPI_BF16_DROPMIX, a2=ds, b2=a_all.reshape(n * R, K), K2=R, b2_adapter_rows=R,
                tile_adapter=tile_adapter, max_ctas=8, **drop.kwargs())
    ref = _f32mm(dy, w)
    row_adapter = tile_adapter.repeat_interleave(128).long()
    for a in range(n):
        rows = row_adapter == a
        keep = keep_mask(M, K, ps[a], 99, 5).cuda()[rows]
        ref[rows] += torch.where(keep, _f32mm(ds[rows], a_all[a]) / (1 - ps[a]), torch.zeros((), device="cuda"))
    assert_close_two_rounds(out, ref, msg=f"pair dx dropout, contraction {N}")


def test_dropout_keep_fraction():
    from lorafusion_b200.ops.philox import keep_mask

    m = keep_mask(512, 1024, 0.1, seed=0)
    assert abs(float(m.float().mean()) - 0.9) < 5e-3


@pytest.mark.parametrize("double_quant", [False, True])
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_nf4_mainloop_gemm_matches_dequantize_then_gemm(double_quant, p):
    """The kernels that expand NF4 inside the main loop (forward, dX, dropout-mixed dX) against
    the same ops on the weight dequantised by plain PyTorch; the LoRA slab rides along."""
    from lorafusion_b200.ops import lora_kernels as lk
    from lorafusion_b200.ops import nf4
    from lorafusion_b200.ops.philox import keep_mask

    N, K, n = 768, 1024, 4
    seg_adapters, seg_tiles = [2, 0, -1, 3, 1], [2, 1, 1, 3, 2]
    M = 128 * sum(seg_tiles)
    tile_adapter = _tile_adapters(seg_adapters, seg_tiles)
    x, w = _rand(M, K, seed=30), _rand(N, K, scale=0.03, seed=31)
    dy = _rand(M, N, seed=32)
    a_all, b_all = _adapters(n, N, K)
    s, ds = _rand(M, 64, scale=0.1, seed=33), _rand(M, 64, scale=0.1, seed=34)
    bias = _rand(N, seed=35)
    qw = nf4.quantize_nf4(w, double_quant=double_quant)
    wd = nf4.dequantize_nf4_reference(qw)  # bf16, torch
    drop = lk.DropoutSpec(seed=99, stream_id=3, p=p)
    keep = keep_mask(M, K, p, 99, 3).cuda()
    row_adapter = tile_adapter.repeat_interleave(128).long()

    y = lk.base_lora_fwd(x, qw, s, b_all, tile_adapter=tile_adapter, bias=bias)
    dx = lk.base_lora_dx(dy, qw, ds, a_all, tile_adapter=tile_adapter, dropout=drop)
    dx_plain = lk.base_lora_dx(dy, qw, None, None, tile_adapter=None)

    y_ref = _f32mm(x, wd.t()) + bias.float()
    dx_ref = _f32mm(dy, wd)
    assert_close_two_rounds(dx_plain, dx_ref, msg="nf4 dX (no adapters)")
    inv = 1.0 / (1.0 - p)
    for a in range(n):
        rows = row_adapter == a
        y_ref[rows] += _f32mm(s[rows], b_all[a].t())
        dx_ref[rows] += torch.where(keep[rows], _f32mm(ds[rows], a_all[a]) * inv,
                                    torch.zeros((), device="cuda"))
    assert_close_two_rounds(y, y_ref, msg="nf4 forward")
    assert_close_two_rounds(dx, dx_ref, msg="nf4 dX")
    # same tiles, same arithmetic: identical to dequantise-to-scratch followed by the bf16 kernel
    from lorafusion_b200.ops import gemm as gemm_mod

    wd_native = nf4.dequantize_nf4(qw)
    was = gemm_mod._PAIR
    gemm_mod.set_pair_kernels(False)  # same single-CTA template for both
    try:
        y2 = lk.base_lora_fwd(x, wd_native, s, b_all, tile_adapter=tile_adapter, bias=bias)
    finally:
        gemm_mod.set_pair_kernels(was)
    assert torch.equal(y, y2)
