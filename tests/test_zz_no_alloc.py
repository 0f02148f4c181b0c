"""The allocation-free entry point, called through its exported C symbol.

`ttb_rmsnorm_bwd_noalloc` is for hosts that cannot get device memory at call time (a C program without a tensor
allocator, a process that handed its memory to another pool, a loop where cudaMalloc's device synchronisation is not
acceptable).  It must give the same dx / dw as the regular entry point, which takes its workspace from the caller.
Two calls in a row are checked because all calls share one built-in scratch array that keeps the previous contents.
This file sorts last on purpose: a failure here must not hide the result of any other test under `-x`."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    ref = b.abs().max().item()
    assert torch.allclose(a, b, rtol=tol, atol=tol * max(ref, 1e-6)), (a - b).abs().max().item()


def test_noalloc_entry_point_matches_regular_one():
    from torchturbo_b200 import kernels as K

    assert K.available()
    lib = C.CDLL(str(K.lib_path()))
    fn = lib.ttb_rmsnorm_bwd_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong,
                   C.c_int, C.c_int, C.c_void_p]
    lib.ttb_noalloc_strerror.restype = C.c_char_p
    torch.manual_seed(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # (rows, width, residual gradient given, (1 + w) variant): later calls reuse the scratch the earlier ones filled; the
    # list covers the documented maximum width, the smallest width, fewer rows than scratch blocks and both options
    for T, H, with_dres, one_plus_w in [(300, 2048, True, False), (77, 4096, True, False), (5, 8192, False, True),
                                        (3, 8, False, False), (1000, 8192, True, True)]:
        x = torch.randn(T, H, device="cuda").bfloat16()
        dy = torch.randn(T, H, device="cuda").bfloat16()
        dres = torch.randn(T, H, device="cuda").bfloat16() if with_dres else None
        w = torch.randn(H, device="cuda").bfloat16()
        _, rstd, _ = K.rmsnorm_fwd(x, w, 1e-6, one_plus_w=one_plus_w)
        dx_ref, dw_ref = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres, one_plus_w=one_plus_w)
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if with_dres else None,
                dx.data_ptr(), dw.data_ptr(), T, H, int(one_plus_w), stream)
        assert rc == 0, lib.ttb_noalloc_strerror(rc).decode()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        _close(dx, dx_ref)
        _close(dw, dw_ref)
    # every error class has its own range and its own text
    texts = {lib.ttb_noalloc_strerror(c) for c in (901, 100000 + 700, 110000 + 700, 200000 + 101)}
    assert len(texts) == 4 and all(b"unknown" not in t for t in texts)
    # sizes beyond the built-in scratch are refused with a readable message, and nothing runs
    rc = fn(0, 0, 0, 0, 0, 0, 0, 4, 8192 + 8, 0, stream)
    assert rc == 901 and b"8192" in lib.ttb_noalloc_strerror(rc)
    assert fn(0, 0, 0, 0, 0, 0, 0, 4, 100, 0, stream) == 901
