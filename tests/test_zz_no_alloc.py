"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the device; it compares two
calls in a row against the ordinary entry point, whose scratch the caller provides."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


def _lib():
    from mindspore_b200 import _native
    lib = _native.cuda()
    assert lib is not None, "native CUDA library is not loaded"
    fn = lib.msb_rmsnorm_bwd_static
    fn.restype = _I
    fn.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _P]
    ref = lib.msb_rmsnorm_bwd
    ref.restype = _I
    ref.argtypes = [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _P]
    err = lib.msb_last_error
    err.restype = ctypes.c_char_p
    return fn, ref, err


def _case(rows, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x = mk(rows, H).bfloat16()
    dy = mk(rows, H).bfloat16()
    dres = mk(rows, H).bfloat16()
    w = (1 + 0.1 * mk(H)).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    return x, dy, dres, w, rstd


def test_static_scratch_matches_regular_entry_point_twice():
    fn, ref, err = _lib()
    from mindspore_b200 import _native
    lib_scratch = _native.cuda().msb_norm_bwd_scratch_elems
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two calls in a row, the second with a smaller H so that stale scratch beyond H and within H both matter
    for rows, H, seed, fp32, acc in ((777, 4096, 1, 1, 1), (300, 1024, 2, 0, 0)):
        x, dy, dres, w, rstd = _case(rows, H, seed)
        dt = torch.float32 if fp32 else torch.bfloat16
        dw_a = torch.ones(H, device="cuda", dtype=dt)
        dw_b = dw_a.clone()
        dx_a = torch.empty_like(x)
        dx_b = torch.empty_like(x)
        # the ordinary entry point reduces in two stages: its scratch is one partial row of H floats per CTA
        lib_scratch.restype = _L
        scratch = torch.empty(int(lib_scratch(H, 0)), device="cuda", dtype=torch.float32)
        rc = ref(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx_a.data_ptr(),
                 scratch.data_ptr(), dw_a.data_ptr(), fp32, acc, rows, H, stream)
        assert rc == 0, err()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx_b.data_ptr(),
                dw_b.data_ptr(), fp32, acc, rows, H, stream)
        assert rc == 0, err()
        torch.cuda.synchronize()
        assert torch.equal(dx_a, dx_b)
        # the weight gradient is summed with float atomics, whose order differs from launch to launch
        torch.testing.assert_close(dw_b.float(), dw_a.float(), rtol=2e-2, atol=2e-2 * dw_a.float().abs().max().item())
        # and against plain PyTorch fp32
        xl = x.float().requires_grad_(True)
        wl = w.float().requires_grad_(True)
        (xl * torch.rsqrt(xl.pow(2).mean(-1, keepdim=True) + 1e-5) * wl).backward(dy.float())
        expect = wl.grad + (1.0 if acc else 0.0)
        scale = expect.abs().max().item()
        assert (dw_b.float() - expect).abs().max().item() <= 2e-2 * scale
        assert (dx_b.float() - (xl.grad + dres.float())).abs().max().item() <= \
            2e-2 * (xl.grad + dres.float()).abs().max().item()


def test_static_scratch_rejects_sizes_beyond_its_limit():
    fn, _, err = _lib()
    rc = fn(None, None, None, None, None, None, None, 0, 0, 0, 16384 + 8, None)
    assert rc == 3
    assert b"exceeds" in err()
    rc = fn(None, None, None, None, None, None, None, 0, 0, 0, 12, None)
    assert rc == 1
