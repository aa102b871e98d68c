"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at call time (a fixed, pre-sized
memory budget; a thread that must not take the allocator lock or provoke cudaMalloc's implicit
synchronisation; a C program without PyTorch's allocator). `nplm_fa_bwd_noalloc` keeps its scratch
in a static device array inside the library. This test checks it against the regular entry point
(`nplm_fa_bwd`, scratch supplied by the caller) on two consecutive calls — the second call sees the
scratch contents the first one left behind — and checks that an oversized request is refused.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -20


def _entry():
    from nanoplm_b200.ops._lib import lib
    handle = lib("attention")
    fn = handle.nplm_fa_bwd_noalloc
    fn.restype = c_int
    err = handle.nplm_fa_bwd_noalloc_strerror
    err.restype = ctypes.c_char_p
    return fn, err


def _case(seed, lens, H=4, D=64):
    from nanoplm_b200.ops import kernels as k
    g = torch.Generator(device="cuda").manual_seed(seed)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    qkv = (torch.randn(T, 3 * H * D, device="cuda", generator=g)).to(torch.bfloat16)
    dout = (torch.randn(T, H * D, device="cuda", generator=g)).to(torch.bfloat16)
    ss, se = k.seq_bounds(cu_t, T)
    return qkv, dout, ss, se, T


def _call_noalloc(fn, qkv, out, dout, lse, ss, se, T, H, D, window, scale):
    from nanoplm_b200.ops._lib import status_word, stream_ptr
    dqkv = torch.empty_like(qkv)
    rc = fn(c_void_p(qkv.data_ptr()), c_void_p(out.data_ptr()), c_void_p(dout.data_ptr()),
            c_void_p(lse.data_ptr()), c_void_p(dqkv.data_ptr()), c_void_p(ss.data_ptr()),
            c_void_p(se.data_ptr()), c_int(T), c_int(H), c_int(D), c_int(window), c_float(scale),
            c_void_p(status_word(qkv.device).data_ptr()), stream_ptr())
    return rc, dqkv


def test_noalloc_attention_backward_matches_regular_entry_twice(cuda_status):
    from nanoplm_b200.ops import kernels as k
    fn, err = _entry()
    H, D, scale = 4, 64, 0.125
    cases = [(_case(1, [50, 200, 6, 300, 77]), -1), (_case(2, [128, 31, 400]), 64)]
    for (qkv, dout, ss, se, T), window in cases:          # two calls in a row share the scratch
        out, lse = k.fa_fwd(qkv, ss, se, H, D, window, scale)
        ref = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale)
        rc, got = _call_noalloc(fn, qkv, out, dout, lse, ss, se, T, H, D, window, scale)
        assert rc == 0, err(rc).decode()
        torch.cuda.synchronize()
        a, b = got.float(), ref.float()
        scale_ref = max(1.0, b.abs().max().item())
        assert torch.allclose(a, b, rtol=3e-2, atol=3e-2 * scale_ref), (a - b).abs().max().item()


def test_noalloc_rejects_problems_beyond_the_static_scratch():
    fn, err = _entry()
    H, D = 16, 64
    T = (4 << 20) // (H * D) + 128                        # one tile past the dq limit
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = c_void_p(dummy.data_ptr())
    rc = fn(p, p, p, p, p, p, p, c_int(T), c_int(H), c_int(D), c_int(-1), c_float(0.125), p,
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == TOO_LARGE
    assert b"too large" in err(rc)
