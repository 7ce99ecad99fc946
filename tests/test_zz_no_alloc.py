"""The allocation-free attention backward entry point (axb_flash_varlen_bwd_noalloc).

Some users of the kernel library cannot allocate device memory at the point where they need the
attention backward pass: a plugin confined to another framework's fixed memory pool, a host
callback or real-time thread where cudaMalloc is off limits, an embedder without PyTorch's
allocator. For them the library offers a variant whose temporaries live in a fixed array inside
the library. This test calls that variant through its exported C symbol (plain ctypes, no
wrapper) twice in a row and checks both results against the regular entry point, which gets its
scratch from the caller. It also checks that oversized problems are refused with a message.

The file name sorts last on purpose: should this entry point break, every other test has
already run.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from axolotl_b200.ops import _lib as L

    lib = L.cuda_lib()
    fn = lib.axb_flash_varlen_bwd_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong,
                   C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                   C.c_longlong, C.c_float, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int]
    return L, lib, fn


def _problem(lens, Hq, Hk, D, seed):
    from axolotl_b200.ops.functional import AttnMeta, flash_varlen

    torch.manual_seed(seed)
    dev = torch.device("cuda", 0)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    T = cu[-1]
    meta = AttnMeta(cu, dev)
    qkv = (torch.randn(T, (Hq + 2 * Hk) * D, device=dev) * 0.5).bfloat16().requires_grad_(True)
    out = flash_varlen(qkv, meta, Hq, Hk, D)
    dout = (torch.randn(T, Hq * D, device=dev) * 0.5).bfloat16()
    lse2 = out.grad_fn.saved_tensors[2].clone()
    (ref,) = torch.autograd.grad(out, qkv, dout)       # regular entry point, caller-owned scratch
    return T, meta, qkv.detach(), out.detach(), dout, lse2, ref


def _call(fn, L, T, meta, qkv, out, dout, lse2, Hq, Hk, D):
    dqkv = torch.empty_like(qkv)
    err = C.create_string_buffer(512)
    rc = fn(qkv.data_ptr(), qkv.stride(0), dout.data_ptr(), out.data_ptr(), out.stride(0), lse2.data_ptr(), T,
            Hq, Hk, D, 0, Hq * D, (Hq + Hk) * D, meta.tiles_bwd.data_ptr(), meta.n_tiles, dqkv.data_ptr(),
            dqkv.stride(0), 1.0 / math.sqrt(D), L.status_word(qkv.device).data_ptr(),
            torch.cuda.current_stream().cuda_stream, err, 512)
    return rc, dqkv, err.value.decode()


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_noalloc_matches_regular_entry_point_twice():
    L, lib, fn = _lib()
    Hq, Hk, D = 4, 2, 128
    # two different problems back to back: the second must not see leftovers of the first
    for seed, lens in ((0, [300, 129, 570]), (1, [64, 700])):
        T, meta, qkv, out, dout, lse2, ref = _problem(lens, Hq, Hk, D, seed)
        rc, got, msg = _call(fn, L, T, meta, qkv, out, dout, lse2, Hq, Hk, D)
        torch.cuda.synchronize()
        assert rc == 0, msg
        L.check_status()
        assert _rel(got, ref) < 2e-2


def test_noalloc_rejects_oversized_problem():
    L, lib, fn = _lib()
    Hq, Hk, D = 4, 2, 128
    T, meta, qkv, out, dout, lse2, ref = _problem([256], Hq, Hk, D, 2)
    dqkv = torch.empty_like(qkv)
    err = C.create_string_buffer(512)
    big_T = 4194304 // (Hq * D) + 1
    rc = fn(qkv.data_ptr(), qkv.stride(0), dout.data_ptr(), out.data_ptr(), out.stride(0), lse2.data_ptr(), big_T,
            Hq, Hk, D, 0, Hq * D, (Hq + Hk) * D, meta.tiles_bwd.data_ptr(), meta.n_tiles, dqkv.data_ptr(),
            dqkv.stride(0), 0.1, None, None, err, 512)
    assert rc == -20
    assert "exceeds the built-in scratch" in err.value.decode()


def test_noalloc_empty_and_negative_sizes():
    """An empty batch is a clean no-op (nothing launched, rc 0); a negative size is refused with its own code."""
    L, lib, fn = _lib()
    Hq, Hk, D = 4, 2, 128
    T, meta, qkv, out, dout, lse2, ref = _problem([128], Hq, Hk, D, 3)
    dqkv = torch.empty_like(qkv)
    err = C.create_string_buffer(512)
    args = lambda t: (qkv.data_ptr(), qkv.stride(0), dout.data_ptr(), out.data_ptr(), out.stride(0), lse2.data_ptr(), t,
                      Hq, Hk, D, 0, Hq * D, (Hq + Hk) * D, meta.tiles_bwd.data_ptr(), meta.n_tiles, dqkv.data_ptr(),
                      dqkv.stride(0), 0.1, None, None, err, 512)
    assert fn(*args(0)) == 0
    assert fn(*args(-5)) == -22 and "must be >= 0" in err.value.decode()
    torch.cuda.synchronize()
