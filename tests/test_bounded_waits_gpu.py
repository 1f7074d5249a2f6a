"""The give-up paths of the kernels' bounded waits.

Every spin inside the kernels (the quantizer's grid barrier, the GEMM's mbarrier waits) ends after a
time limit, records a code and lets the kernel drain and return.  `nvfp4_test_hooks` shortens the
limit to a millisecond and makes one arrival never come (a count that nothing completes), so the
wait runs out; the tests check that the launch RETURNS, that the documented word carries the code,
and that the next normal call is bit-exact after the documented clean-up.  Nothing here faults,
traps or spins without a limit."""
import ctypes

import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

LIMIT_NS = 1_000_000          # 1 ms


@pytest.fixture()
def L():
    from nvfp4_sm120_b200 import _lib
    lib = _lib.lib()
    yield lib
    lib.nvfp4_test_hooks(0, 0, 0)


def _fused(L, x, ws):
    from nvfp4_sm120_b200.tensor import swizzled_scale_dims
    rows, cols = x.shape
    sm, sk = swizzled_scale_dims(rows, cols)
    qd = torch.zeros(rows, cols // 2, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(sm, sk, dtype=torch.uint8, device="cuda")
    pts = torch.zeros((), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    if ws is None:
        code = L.nvfp4_quantize_static_bf16(x.data_ptr(), rows, cols, cols, 0, 0, None, 0, 0, qd.data_ptr(),
                                            sc.data_ptr(), pts.data_ptr(), stream)
    else:
        code = L.nvfp4_quantize_fused_bf16(x.data_ptr(), rows, cols, cols, 0, 0, None, 0, 0, qd.data_ptr(),
                                           sc.data_ptr(), pts.data_ptr(), ws.data_ptr(), 64, stream)
    assert code == 0
    torch.cuda.synchronize()                      # the launch returns, with or without the give-up
    return qd, sc, pts


def _static_status(L, clear):
    out = ctypes.c_int32(-77)
    assert L.nvfp4_quantize_static_status(ctypes.byref(out), int(clear), torch.cuda.current_stream().cuda_stream) == 0
    return out.value


def test_quantizer_grid_barrier_gives_up_reports_and_recovers(L):
    x = O.synthetic_tensor(2048, 2048, 41).cuda()           # 148 CTAs take part in the barrier
    ws = torch.zeros(16, dtype=torch.int32, device="cuda")
    want = _fused(L, x, ws)
    assert int(ws[4]) == 0
    L.nvfp4_test_hooks(LIMIT_NS, 1, 0)                      # the barrier waits for one CTA too many
    _fused(L, x, ws)
    L.nvfp4_test_hooks(0, 0, 0)
    assert int(ws[4]) == 1                                  # documented: word 4 = 1, the grid barrier gave up
    ws.zero_()                                              # documented clean-up before the next use
    got = _fused(L, x, ws)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert int(ws[4]) == 0


def test_static_entry_point_reports_a_give_up(L):
    x = O.synthetic_tensor(1024, 4096, 42).cuda()
    ws = torch.zeros(16, dtype=torch.int32, device="cuda")
    want = _fused(L, x, ws)
    assert _static_status(L, clear=True) in (0, 1, 2)       # whatever earlier tests left is cleared here
    _fused(L, x, None)
    assert _static_status(L, clear=False) == 0
    L.nvfp4_test_hooks(LIMIT_NS, 1, 0)
    _fused(L, x, None)
    L.nvfp4_test_hooks(0, 0, 0)
    _fused(L, x, None)                                      # a later good call does not hide the word
    assert _static_status(L, clear=True) == 1
    assert _static_status(L, clear=False) == 0
    got = _fused(L, x, None)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert L.nvfp4_quantize_static_status(None, 0, None) == -1


@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_wait_gives_up_reports_and_recovers(L, mode):
    """mode 1: one-CTA kernel, mode 2: persistent pair kernel.  The scale-factor warps never announce
    K slice 0; every role leaves its loop through a bounded wait, tensor memory is freed, the status
    word carries the code of the first wait that gave up, and the next launch is exact."""
    import nvfp4_sm120_b200 as Q
    m, n, k = 512, 768, 2048
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 43).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 44).cuda())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def run():
        d = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        code = L.nvfp4_gemm(qa.qdata.data_ptr(), qa.scale.data_ptr(), qa.per_tensor_scale.data_ptr(),
                            qb.qdata.data_ptr(), qb.scale.data_ptr(), qb.per_tensor_scale.data_ptr(),
                            d.data_ptr(), 1, m, n, k, n, status.data_ptr(), stream)
        assert code == 0
        torch.cuda.synchronize()
        return d

    try:
        L.nvfp4_gemm_set_mode(mode)
        want = run()
        assert int(status) == 0
        L.nvfp4_test_hooks(LIMIT_NS, 0, 1)
        run()
        L.nvfp4_test_hooks(0, 0, 0)
        assert int(status) in (1, 2, 3, 4)                   # producer / MMA / epilogue / scale wait gave up
        status.zero_()
        got = run()
        assert int(status) == 0
        assert torch.equal(got, want)
    finally:
        L.nvfp4_test_hooks(0, 0, 0)
        L.nvfp4_gemm_set_mode(0)
