"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users drive these kernels from C / C++ in processes that cannot call cudaMalloc at that point (HBM already
handed out in full, or a section where cudaMalloc's device-wide synchronisation is not acceptable); for them the
library keeps the weight-gradient scratch in a static device array. This test calls the C symbol with raw device
pointers twice in a row (the second call re-uses the scratch that the first one left behind, once overwriting and once
accumulating into dw) and checks both results against the regular entry point and against the same gradients
written as plain fp32 PyTorch expressions, then checks that an over-long row is refused with a message instead of being run. The file name sorts last so that a run that stops at the first failure
has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _lib():
    from paddleformers_b200.ops import _build

    assert _build.load_extension(required=True)
    lib = ctypes.CDLL(_build.ext_path())
    fn = lib.pfb_rms_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p,
                                          ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, dy, x, w, rstd, dres, dx, dw, accumulate):
    err = ctypes.create_string_buffer(256)
    T, H = x.shape
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if dres is not None else None,
            dx.data_ptr(), dw.data_ptr(), T, H, dy.stride(0), int(accumulate), torch.cuda.current_stream().cuda_stream,
            err, len(err))
    return rc, err.value.decode()


def test_noalloc_rms_norm_bwd_matches_regular_entry_point():
    fn = _lib()
    ops = torch.ops.pfb200
    torch.manual_seed(0)
    dw_acc = None
    for call, (T, H, with_res, accumulate) in enumerate([(333, 4096, False, False), (1000, 2048, True, True)]):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
        dres = torch.randn(T, H, device="cuda", dtype=torch.bfloat16) if with_res else None
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        # regular entry point (caller-provided scratch)
        scratch = torch.empty(int(ops.rms_norm_bwd_scratch_rows()) * H, device="cuda", dtype=torch.float32)
        start = torch.randn(H, device="cuda") if accumulate else torch.zeros(H, device="cuda")
        dw_ref = start.clone()
        dx_ref = ops.rms_norm_bwd(dy, x, w, rstd, dres, dw_ref, accumulate, scratch)
        # allocation-free entry point
        dx = torch.empty_like(x)
        dw = start.clone()
        free_before = torch.cuda.mem_get_info()[0]
        rc, msg = _call(fn, dy, x, w, rstd, dres, dx, dw, accumulate)
        torch.cuda.synchronize()
        assert rc == 0, msg
        if call > 0:  # the very first call may load the module lazily; later calls must not take device memory
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert _rel_err(dx, dx_ref) < 1e-2
        assert _rel_err(dw, dw_ref) < 2e-2
        # fp32 oracle: y = x * rstd * w  =>  dx = rstd * (g - xhat * mean(g * xhat)) with g = dy * w, dw = sum_t dy * xhat
        xf, dyf, wf = x.float(), dy.float(), w.float()
        xhat = xf * rstd[:, None]
        g = dyf * wf
        dx_o = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
        if dres is not None:
            dx_o = dx_o + dres.float()
        dw_o = start + (dyf * xhat).sum(0)
        assert _rel_err(dx, dx_o) < 1e-2
        assert _rel_err(dw, dw_o) < 2e-2


def test_noalloc_rejects_rows_beyond_the_static_scratch():
    fn = _lib()
    T, H = 4, 8192 + 8
    x = torch.zeros(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(T, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.zeros(H, device="cuda")
    rc, msg = _call(fn, x, x, w, rstd, None, dx, dw, False)
    assert rc == -1 and "exceeds" in msg and "8192" in msg
