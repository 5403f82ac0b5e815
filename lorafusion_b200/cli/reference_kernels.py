"""The reference's own Triton kernels, imported unmodified and composed the way the reference
composes them, as a same-GPU baseline for ``cli/bench_kernels.py``.

What runs here is the reference's code, not this framework's: ``seeded_dropout`` (K1),
``fused_lora_xw_sb`` (K4), ``fused_lora_dyw_dsa`` (K6), ``fused_lora_dys_dyb`` (K8) and the
three ``fused_multi_lora_*`` kernels (K9-K11) from ``lorafusion/ops/triton_ops/*.py``, with
cuBLAS for ``S = dropout(X) A^T`` and ``dA = dS^T dropout(X)`` exactly as
``lorafusion/ops/lora_v1.py:87-166`` and ``lorafusion/ops/multi_lora.py:470-600`` do.  Three
things of the environment are supplied from here, none of them an edit of the reference:

* the package is looked for in ``<repository>/baseline/_ref`` (an unmodified copy of the
  reference's ``lorafusion`` directory) or wherever ``--reference-path`` /
  ``LORAFUSION_REFERENCE_PATH`` points;
* ``lorafusion.utils.benchmark`` imports ``mypy_extensions`` for two type aliases; a stand-in
  module with those two names is registered when the real one is not installed;
* the reference's tile table has no entry for this GPU (``triton_ops/config.py:136-146``
  raises), so its H100 tile configurations are passed explicitly through the ``config=``
  argument every kernel wrapper has.  The TMA variants are not used: they call
  ``tl._experimental_descriptor_*``, which the installed Triton no longer has.

Nothing in the training path imports this module.
"""

from __future__ import annotations

import importlib
import os
import sys
import types
from pathlib import Path
from typing import Optional

import torch

_REPO_ROOT = Path(__file__).resolve().parents[2]
_ref = None  # cache of the imported reference modules


class ReferenceUnavailable(RuntimeError):
    pass


def _install_mypy_extensions_stand_in() -> None:
    try:
        import mypy_extensions  # noqa: F401
        return
    except ImportError:
        pass
    mod = types.ModuleType("mypy_extensions")

    def _arg(type_=None, name=None):  # the two helpers only build type annotations
        return type_

    mod.DefaultNamedArg = _arg
    mod.NamedArg = _arg
    sys.modules["mypy_extensions"] = mod


def load_reference(path: Optional[str] = None) -> types.SimpleNamespace:
    """Import the reference's kernel modules; raises :class:`ReferenceUnavailable` with the
    reason when that is not possible."""
    global _ref
    if _ref is not None:
        return _ref
    root = Path(path or os.environ.get("LORAFUSION_REFERENCE_PATH") or _REPO_ROOT / "baseline" / "_ref")
    if not (root / "lorafusion" / "ops" / "triton_ops" / "fused_lora_xw_sb.py").exists():
        raise ReferenceUnavailable(f"no copy of the reference's lorafusion package under {root}")
    _install_mypy_extensions_stand_in()
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    try:
        ops = "lorafusion.ops.triton_ops."
        mods = {name: importlib.import_module(ops + name) for name in (
            "config", "dropout", "fused_lora_xw_sb", "fused_lora_dyw_dsa", "fused_lora_dys_dyb",
            "fused_multi_lora_xw_sb", "fused_multi_lora_dyw_dsa", "fused_multi_lora_dys_dyb")}
    except Exception as e:  # noqa: BLE001 - any import problem of foreign code is reported as such
        raise ReferenceUnavailable(f"importing the reference kernels failed: {type(e).__name__}: {e}") from e
    cfg = mods["config"]
    h100 = cfg.H100_CONFIG  # the tile table the reference ships for its best-supported GPU
    _ref = types.SimpleNamespace(mods=mods, h100=h100, block_m=int(h100.fused_multi_lora_block_size_m))
    return _ref


# ---------------------------------------------------------------------------------------------
# single adapter: lorafusion/ops/lora_v1.py:87-166
# ---------------------------------------------------------------------------------------------
def ref_lora_forward(x, w, a, b, alpha: float, p: float, seed: int = 0):
    """Returns ``(y, saved)``: K1 dropout (stores the mask and the masked copy of x), cuBLAS
    ``S``, K4 fused ``x W^T + alpha S B^T``."""
    R = load_reference()
    m = R.mods
    mask, xh = None, x
    if p > 0:
        xh, mask = m["dropout"].seeded_dropout(x=x, p=p, seed=seed, store_mask=True)
    s = xh @ a.T
    y = m["fused_lora_xw_sb"].fused_lora_xw_sb(x=x, w=w, s=s, b=b, alpha=alpha, bias=None,
                                                config=R.h100.fused_lora_xw_sb)
    return y, (xh, mask, s)


def ref_lora_backward(dy, w, a, b, alpha: float, p: float, saved):
    """K8 (dB and dS in one pass, fp32 atomics), cuBLAS ``dA``, K6 fused dX.  Returns
    ``(dx, da, db)``."""
    R = load_reference()
    m = R.mods
    xh, mask, s = saved
    db, ds = m["fused_lora_dys_dyb"].fused_lora_dys_dyb(dy=dy, b=b, s=s, alpha=alpha,
                                                         config=R.h100.fused_lora_dys_dyb)
    da = ds.T @ xh
    dx = m["fused_lora_dyw_dsa"].fused_lora_dyw_dsa(dy=dy, w=w, ds=ds, a=a, dropout_p=p, dropout_mask=mask,
                                                     config=R.h100.fused_lora_dyw_dsa)
    return dx, da, db


# ---------------------------------------------------------------------------------------------
# several adapters in one microbatch: lorafusion/ops/multi_lora.py:348-600
# ---------------------------------------------------------------------------------------------
def ref_multi_batch_info(seq_lens, ranks, alphas, dropout_ps, dtype=torch.bfloat16, device="cuda"):
    """The per-128-row-block tables the reference builds on the host
    (``prepare_multi_lora_batch_info``, ``multi_lora.py:385-432``): ``(rank, valid rows, first
    block of the segment)`` per block, and alpha / dropout p per block in the compute dtype."""
    bm = load_reference().block_m
    padded = [((n + bm - 1) // bm) * bm for n in seq_lens]
    rows, alpha_rows, p_rows, blk = [], [], [], 0
    for n, pad, r, al, p in zip(seq_lens, padded, ranks, alphas, dropout_ps):
        start = blk
        for i in range(pad // bm):
            rows.append((r, min(bm, n - i * bm), start))
            alpha_rows.append(al)
            p_rows.append(p)
            blk += 1
    return dict(
        seq_len_list=list(seq_lens), padded_seq_len_list=padded,
        block_to_lookup_table=torch.tensor(rows, dtype=torch.int32, device=device),
        block_to_alpha=torch.tensor(alpha_rows, dtype=dtype, device=device),
        block_to_dropout_p=torch.tensor(p_rows, dtype=dtype, device=device),
        max_r=max(ranks), same_p=dropout_ps[0] if len(set(dropout_ps)) == 1 else None)


def ref_multi_lora_forward(x, w, a_list, b_list, info, seed: int = 0):
    """K1, cuBLAS ``X cat(A)^T`` (every token times every adapter's rank, as the reference does),
    pointer tables, K9.  ``info["same_p"]`` must be set (one dropout rate for all adapters)."""
    R = load_reference()
    m = R.mods
    p = info["same_p"]
    if p is None:
        raise ValueError("this baseline covers adapters that share one dropout rate")
    mask, xh = None, x
    if p > 0:
        xh, mask = m["dropout"].seeded_dropout(x=x, p=p, seed=seed, store_mask=True)
    full_s = x @ torch.cat(a_list, dim=0).T
    s_list, cm, cr = [], 0, 0
    for pad, a in zip(info["padded_seq_len_list"], a_list):
        s_list.append(full_s[cm:cm + pad, cr:cr + a.shape[0]])
        cm += pad
        cr += a.shape[0]
    mx = m["fused_multi_lora_xw_sb"]
    s_ptrs, b_ptrs, _, _ = mx.construct_s_and_b_ptrs_list(raw_s_list=s_list, raw_b_list=b_list, block_size_m=R.block_m)
    y = mx.fused_multi_lora_xw_sb(
        x=xh, w=w, s_ptrs_list=s_ptrs, b_ptrs_list=b_ptrs, block_to_lookup_table=info["block_to_lookup_table"],
        block_to_alpha=info["block_to_alpha"], max_r=info["max_r"], total_r=full_s.shape[1], bias=None,
        block_size_m=R.block_m, config=R.h100.fused_multi_lora_xw_sb)
    return y, (xh, mask, s_list, s_ptrs, b_ptrs)


def ref_multi_lora_backward(dy, w, a_list, b_list, info, saved):
    """K11 (per-adapter fp32 atomics), per-adapter cuBLAS ``dA``, K10.  Returns
    ``(dx, da_list, db_list)``."""
    R = load_reference()
    m = R.mods
    xh, mask, s_list, s_ptrs, b_ptrs = saved
    total_r = sum(b.shape[1] for b in b_list)
    db_list, ds_list = m["fused_multi_lora_dys_dyb"].fused_multi_lora_dys_dyb(
        dy=dy, s_ptrs_list=s_ptrs, b_ptrs_list=b_ptrs, raw_s_list=s_list, raw_b_list=b_list,
        block_to_lookup_table=info["block_to_lookup_table"], block_to_alpha=info["block_to_alpha"],
        max_r=info["max_r"], total_r=total_r, block_size_m=R.block_m, config=R.h100.fused_multi_lora_dys_dyb)
    da_list, cm = [], 0
    for pad, ds in zip(info["padded_seq_len_list"], ds_list):
        da_list.append(ds.T @ xh[cm:cm + pad])
        cm += pad
    dx = m["fused_multi_lora_dyw_dsa"].fused_multi_lora_dyw_dsa(
        dy=dy, w=w, raw_ds_list=ds_list, raw_a_list=a_list, block_to_dropout_p=info["block_to_dropout_p"],
        block_to_lookup_table=info["block_to_lookup_table"], max_r=info["max_r"], enable_dropout=mask is not None,
        dropout_mask=mask, block_size_m=R.block_m, config=R.h100.fused_multi_lora_dyw_dsa)
    return dx, da_list, db_list


# ---------------------------------------------------------------------------------------------
# fp32 oracle for the checks (``lorafusion/ops/lora_torch_ref.py:6-48`` semantics, with the mask
# the reference kernel itself drew)
# ---------------------------------------------------------------------------------------------
def check_single(x, w, a, b, dy, alpha: float, p: float) -> dict:
    """Run the reference path once and compare every output with fp32 math that uses the
    kernel's own dropout mask.  Returns the largest absolute errors."""
    y, saved = ref_lora_forward(x, w, a, b, alpha, p)
    dx, da, db = ref_lora_backward(dy, w, a, b, alpha, p, saved)
    xh, mask, s = saved
    xf, wf, af, bf, dyf = (t.float() for t in (x, w, a, b, dy))
    xhf = xf if mask is None else xf * mask.float() / (1 - p)
    sf = (xhf @ af.T).to(torch.bfloat16).float()
    y_ref = xf @ wf.T + (sf @ bf.T) * alpha
    ds_ref = ((dyf @ bf) * alpha).to(torch.bfloat16).float()
    dsa = ds_ref @ af
    dx_ref = dyf @ wf + (dsa if mask is None else dsa * mask.float() / (1 - p))
    out = {"y": float((y.float() - y_ref).abs().max()), "dx": float((dx.float() - dx_ref).abs().max()),
           "da": float((da.float() - ds_ref.T @ xhf).abs().max()),
           "db": float((db.float() - (dyf.T @ sf) * alpha).abs().max()),
           "y_scale": float(y_ref.abs().max()), "dx_scale": float(dx_ref.abs().max())}
    return out
