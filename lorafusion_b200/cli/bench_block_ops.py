"""Benchmark of the non-GEMM kernels of a decoder block: attention forward / backward and
the token-wise kernels (RMSNorm, SwiGLU), each against its roofline.

    python -m lorafusion_b200.cli.bench_block_ops --model llama-3.1-70b --tokens 16384 --seq-len 4096

Attention is reported in TFLOP/s of the causal algorithmic work (``4 * d * sum(len^2) / 2``
forward, 2.5x that backward, per head); the token-wise kernels in GB/s of the bytes they
must move.  The reference takes these ops from FlashAttention-2 and Liger
(``lorafusion/patch/patch_transformers.py:150-159``, ``lorafusion/utils/module.py:40-69``).
"""

from __future__ import annotations

import argparse
import json

import torch

from ..models.config import get_model_config
from ..ops import _native, elementwise as ew
from ..ops.attention import attention_backward, attention_forward, build_attn_tiles
from ..utils.benchmark import benchmark


def run(args):
    cfg = get_model_config(args.model)
    dev = torch.device("cuda")
    torch.manual_seed(0)
    T, H, I = args.tokens, cfg.hidden_size, cfg.intermediate_size
    hq, hkv, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    n_seq = max(1, T // args.seq_len)
    lens = [args.seq_len] * n_seq
    if sum(lens) < T:
        lens.append(T - sum(lens))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    tiles = build_attn_tiles(cu, dev)
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device=dev).to(torch.bfloat16)
    kw = dict(warmup=args.warmup, number=args.number, flush=True)
    out, lse = attention_forward(qkv, tiles, hq, hkv)
    d_out = torch.randn_like(out)
    results = []

    def rec(name, seconds, flops=None, nbytes=None):
        row = {"kernel": name, "ms": seconds * 1e3}
        if flops is not None:
            row["tflops"] = flops / seconds / 1e12
        if nbytes is not None:
            row["gbs"] = nbytes / seconds / 1e9
        results.append(row)
        print(json.dumps(row))

    if args.profile_only in (None, "attention"):
        causal_flops = sum(4.0 * d * ln * ln / 2 for ln in lens) * hq
        t = benchmark(lambda: attention_forward(qkv, tiles, hq, hkv), **kw)
        rec("attention_fwd", t, flops=causal_flops)
        t = benchmark(lambda: attention_backward(qkv, out, d_out, lse, tiles, hq, hkv), **kw)
        rec("attention_bwd", t, flops=2.5 * causal_flops)
    if args.profile_only in (None, "tokenwise"):
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        res = torch.randn_like(x)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        t = benchmark(lambda: ew.rmsnorm_fwd(x, w, 1e-5, res=res), **kw)
        rec("rmsnorm_fwd(+residual)", t, nbytes=4 * T * H * 2)
        y, h, rstd = ew.rmsnorm_fwd(x, w, 1e-5, res=res)
        t = benchmark(lambda: ew.rmsnorm_bwd(x, h, w, rstd, dres=res), **kw)
        rec("rmsnorm_bwd(+residual grad)", t, nbytes=4 * T * H * 2)
        gu = torch.randn(T, 2 * I, device=dev).to(torch.bfloat16)
        t = benchmark(lambda: ew.swiglu_fwd(gu), **kw)
        rec("swiglu_fwd", t, nbytes=3 * T * I * 2)
        dact = torch.randn(T, I, device=dev).to(torch.bfloat16)
        t = benchmark(lambda: ew.swiglu_bwd(dact, gu), **kw)
        rec("swiglu_bwd", t, nbytes=5 * T * I * 2)
    _native.check_device_errors()
    return results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="llama-3.1-70b")
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--number", type=int, default=20)
    ap.add_argument("--profile-only", default=None, choices=["attention", "tokenwise"])
    run(ap.parse_args(argv))


if __name__ == "__main__":
    main()
