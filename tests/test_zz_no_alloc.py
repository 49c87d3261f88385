"""The allocation-free C entry point (``cb200_rmsnorm_rope_bwd_noalloc``) against the regular operator.

Some users of this library are called from another runtime's execute callback, or run in a process that gave all
device memory to its own pool, and therefore cannot let an operator allocate scratch on every call. For them the
library exports one C function that keeps its scratch in a fixed array inside the library image. This test calls
that function through its exported symbol with raw device pointers, twice in a row with different data (the
shared scratch still holds the first call's partial sums when the second one starts), and checks both results
against ``torch.ops.cosmos_b200.rmsnorm_rope_bwd`` - bit for bit, because both run the same kernels with the same row
grouping - and against a plain PyTorch fp32 evaluation of the same backward within the tolerance of the kernel tests. It also checks that an over-sized problem is refused with a
message instead of being launched. This file is named to be collected last.
"""

import ctypes

import pytest
import torch

from cosmos_predict25_b200.ops import native, ref

pytestmark = pytest.mark.gpu

MAX_ROWS = 4194304


def _entry():
    native.load()  # torch libraries first, then the same shared object through ctypes
    lib = ctypes.CDLL(native.lib_path())
    fn = lib.cb200_rmsnorm_rope_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                           ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    bad = ((a - b).abs() > atol + rtol * b.abs()).float().mean().item()
    assert bad < 1e-4, f"{bad * 100:.3f}% of elements out of tolerance (max err {(a - b).abs().max().item():.4g})"


@pytest.mark.parametrize("HD,use_rope", [(128, True), (64, False)])
def test_no_alloc_entry_point_matches_operator_twice(HD, use_rope):
    fn = _entry()
    ops = native.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev)
    B, S, H = 2, 1111, 3
    for call, seed in enumerate((21, 22)):  # two calls in a row on the shared scratch
        torch.manual_seed(seed)
        x = torch.randn(B, S, H, HD, device=dev).bfloat16()
        dy = torch.randn(B, S, H, HD, device=dev).bfloat16() * (1 + call)
        w = (1 + 0.1 * torch.randn(HD, device=dev)).float().contiguous()
        cos = sin = angles = None
        if use_rope:
            ang = torch.rand(S, HD // 2, device=dev) * 40
            cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
            angles = torch.cat([ang, ang], dim=-1)      # rotate-half pairs (i, i + HD/2) share one angle
        _, rstd = ops.rmsnorm_rope_fwd(x, w, cos, sin, 1e-6)
        want_dx, want_dw = ops.rmsnorm_rope_bwd(dy, x, w, rstd, cos, sin)
        dx = torch.empty_like(x)
        dw = torch.empty(HD, device=dev, dtype=torch.float32)
        err = ctypes.create_string_buffer(256)
        rc = fn(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(cos), _ptr(sin), _ptr(dx), _ptr(dw), B * S * H, S, H, HD,
                ctypes.c_void_p(stream.cuda_stream), err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert torch.equal(dx, want_dx) and torch.equal(dw, want_dw)
        # fp32 oracle: autograd through the PyTorch definition of the forward
        xr, wr = x.float().requires_grad_(True), w.clone().requires_grad_(True)
        ref.rmsnorm_rope(xr, wr, angles, 1e-6).backward(dy.float())
        _close(dx, xr.grad, 3e-2, 3e-2)
        _close(dw, wr.grad, 0.3, 3e-2)


def test_no_alloc_entry_point_rejects_oversized_problem():
    fn = _entry()
    dev = torch.device("cuda", torch.cuda.current_device())
    tiny = torch.zeros(256, device=dev)
    err = ctypes.create_string_buffer(256)
    rc = fn(_ptr(tiny), _ptr(tiny), _ptr(tiny), _ptr(tiny), None, None, _ptr(tiny), _ptr(tiny), MAX_ROWS + 1, 1, 1, 128,
            ctypes.c_void_p(0), err, 256)
    assert rc == -1 and b"exceed" in err.value
    rc = fn(_ptr(tiny), _ptr(tiny), _ptr(tiny), _ptr(tiny), None, None, _ptr(tiny), _ptr(tiny), 16, 4, 4, 96,
            ctypes.c_void_p(0), err, 256)
    assert rc == -2
    torch.cuda.synchronize()
