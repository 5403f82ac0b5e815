"""The allocation-free attention backward, called through its exported C symbol.

``lf_attn_bwd_noalloc`` is meant for processes that must not create device memory at the
point of the call (fixed memory partitions, callbacks of another runtime, frozen
allocators): its temporary buffer is a fixed array inside the library.  The test drives the
raw symbol with ctypes exactly as such a caller would -- passing only buffers that already
exist -- and checks, on two calls in a row (the second one reuses the array with the first
call's contents still in it), that it returns the same gradients as ``lf_attn_bwd``, and that
the amount of free device memory is the same after the call as before it.
It also checks that an oversized problem is refused instead of overrunning the array.
"""

import ctypes as C

import pytest
import torch

from lorafusion_b200.utils.testing import assert_close

pytestmark = pytest.mark.gpu

MAX_DELTA = 1 << 20
TOO_LARGE = -40


def _symbol():
    from lorafusion_b200.ops import _native as nv

    lib = nv.cuda_lib()
    fn = lib.lf_attn_bwd_noalloc
    VP, LL, I, F = C.c_void_p, C.c_longlong, C.c_int, C.c_float
    fn.argtypes = [VP, VP, VP, VP, LL, LL, I, I, I, I, I, VP, I, LL, VP, F, VP, VP]
    fn.restype = C.c_int
    return fn


def _case(lens, Hq, Hkv, seed):
    from lorafusion_b200.ops import attention as att

    g = torch.Generator(device="cuda").manual_seed(seed)
    M = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    qkv = torch.randn(M, (Hq + 2 * Hkv) * 128, generator=g, device="cuda").to(torch.bfloat16)
    d_out = torch.randn(M, Hq * 128, generator=g, device="cuda").to(torch.bfloat16)
    tiles = att.build_attn_tiles(cu, "cuda")
    out, lse = att.attention_forward(qkv, tiles, Hq, Hkv)
    expected = att.attention_backward(qkv, out, d_out, lse, tiles, Hq, Hkv)
    return qkv, out, d_out, lse, tiles, expected


def test_noalloc_matches_regular_entry_point_twice():
    from lorafusion_b200.ops import _native as nv

    fn = _symbol()
    scale = 1.0 / (128 ** 0.5)
    for call, (lens, Hq, Hkv) in enumerate([([300, 129, 64], 4, 2), ([200, 520], 8, 2)]):
        qkv, out, d_out, lse, tiles, expected = _case(lens, Hq, Hkv, seed=40 + call)
        M = qkv.shape[0]
        dqkv = torch.empty_like(qkv)  # the caller's own, pre-existing output buffer
        k0, v0 = Hq * 128, (Hq + Hkv) * 128
        err_ptr, stream_ptr = nv.err_word("cuda").data_ptr(), nv.current_stream_ptr()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(qkv.data_ptr(), out.data_ptr(), d_out.data_ptr(), dqkv.data_ptr(), M, qkv.stride(0), 0, k0, v0,
                Hq, Hkv, tiles.tiles.data_ptr(), tiles.num_tiles, out.stride(0), lse.data_ptr(), scale,
                err_ptr, stream_ptr)
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # the driver reports free memory of the whole device: nothing was taken by the call
        # (the first call may only have loaded the kernels' module, which happens before it
        # in this process because the regular entry point ran the same kernels above)
        assert free_after == free_before, f"call {call}: free device memory changed by {free_before - free_after} bytes"
        assert_close(dqkv, expected, msg=f"no-alloc attention backward, call {call}")


def test_noalloc_rejects_problems_beyond_its_scratch():
    fn = _symbol()
    Hq, M = 64, MAX_DELTA // 64 + 128
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = fn(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), M, 10240, 0, 8192, 9216, Hq,
            8, dummy.data_ptr(), 1, 8192, dummy.data_ptr(), 0.1, dummy.data_ptr(), None)
    assert rc == TOO_LARGE
