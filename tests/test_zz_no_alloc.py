"""The allocation-free read backward (``sihc_read_bwd_static``) against ``sihc_read_bwd``.

Some hosts cannot hand this library a scratch buffer: they planned all device
memory at start-up, or they run on a thread that must never call cudaMalloc.
For them the library carries a fixed 16 MiB scratch array of its own.  This test
calls that entry point directly through the C ABI, twice in a row on different
inputs (the second call finds the first call's partial sums still in the array),
and checks both results against the ordinary entry point, which gets a freshly
allocated workspace.  It also checks that a case too large for the fixed array is
refused with SIHC_ERR_CAPACITY instead of being launched.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
CELLS = {2: (1, 2), 4: (2, 2), 8: (2, 4), 16: (4, 4)}


def _run(lib, _lib, static, x, gs, alpha, dtype_code, wcode):
    b, h, w, c = x.shape
    e, _, s = alpha.shape
    kh, kw = CELLS[s]
    g = h // kh
    dx = torch.empty_like(x)
    dalpha = torch.empty(e, c, s, device=x.device, dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    ptrs = _lib.ptr_array([None if t is None else t.data_ptr() for t in gs])
    if static:
        rc = lib.sihc_read_bwd_static(x.data_ptr(), ptrs, alpha.data_ptr(), dx.data_ptr(), dalpha.data_ptr(),
                                      e, b, g, kh, kw, c, dtype_code, wcode, stream)
    else:
        nbytes = lib.sihc_wgrad_workspace_bytes(e, b, g, kh, kw, c, dtype_code)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
        rc = lib.sihc_read_bwd(x.data_ptr(), ptrs, alpha.data_ptr(), dx.data_ptr(), dalpha.data_ptr(),
                               ws.data_ptr(), ws.numel(), e, b, g, kh, kw, c, dtype_code, wcode, stream)
    torch.cuda.synchronize()
    return rc, dx, dalpha


@pytest.mark.parametrize("dtype,events,slots", [(torch.bfloat16, 1, 4), (torch.float32, 1, 4), (torch.bfloat16, 3, 4),
                                                (torch.bfloat16, 1, 8)])
def test_static_scratch_matches_workspace_entry_point_twice(dtype, events, slots):
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
    kh, kw = CELLS[slots]
    b, g, c = 24, 16, 768                      # 6144 tokens -> 192 partial-sum blocks
    torch.manual_seed(2024)
    for call in range(2):                      # the second call reuses the array the first one filled
        x = torch.randn(b, g * kh, g * kw, c, device=DEV).to(dtype) * (1.0 + call)
        alpha = (1.0 / slots + 0.05 * torch.randn(events, c, slots, device=DEV)).to(dtype)
        gs = [torch.randn(b, g * g, c, device=DEV).to(dtype) for _ in range(events)]
        if events > 1 and call == 1:
            gs[1] = None                       # an unused read output on the second call
        rc_s, dx_s, da_s = _run(lib, _lib, True, x, gs, alpha, code, code)
        rc_w, dx_w, da_w = _run(lib, _lib, False, x, gs, alpha, code, code)
        assert rc_s == 0, lib.sihc_status_string(rc_s)
        assert rc_w == 0, lib.sihc_status_string(rc_w)
        # Both entry points run the same kernels with the same fixed summation order; only the address of
        # the partial sums differs.  The results must therefore be identical bit for bit.
        assert torch.equal(dx_s, dx_w)
        assert torch.equal(da_s, da_w)
        if events > 1 and call == 1:
            assert torch.count_nonzero(da_s[1]) == 0


def test_static_scratch_refuses_oversized_case_without_launching():
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    # 24 events x 16 slots x 1152 channels over 2^20 tokens needs hundreds of MB of partial sums.
    need = lib.sihc_wgrad_workspace_bytes(24, 4096, 16, 4, 4, 1152, _lib.BF16)
    assert need > 16 * 1024 * 1024
    dummy = torch.zeros(64, device=DEV)
    before = _lib.launch_count()
    ptrs = _lib.ptr_array([dummy.data_ptr()] * 24)
    rc = lib.sihc_read_bwd_static(dummy.data_ptr(), ptrs, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                  24, 4096, 16, 4, 4, 1152, _lib.BF16, _lib.BF16,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == -8                                             # SIHC_ERR_CAPACITY
    assert b"capacity" in lib.sihc_status_string(rc)
    assert _lib.launch_count() == before
    torch.cuda.synchronize()
