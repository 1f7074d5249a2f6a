"""The no-allocation quantizer entry point (scratch inside the library) against the entry point that
takes a caller workspace.  It exists for callers that cannot allocate device memory at the call site
(FFI bindings inside a runtime that owns all of HBM, callbacks that must avoid cudaMalloc's implicit
synchronisation).  Collected last on purpose: a run that stops at the first failure has then already
run every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, x, mode, rht, signs, seed, with_ws):
    from nvfp4_sm120_b200.tensor import swizzled_scale_dims
    rows, cols = x.shape
    sm, sk = swizzled_scale_dims(rows, cols)
    qd = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sc = torch.full((sm, sk), 0xAA, dtype=torch.uint8, device=x.device)
    pts = torch.zeros((), dtype=torch.float32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    sp = signs.data_ptr() if rht else None
    if with_ws:
        ws = torch.zeros(16, dtype=torch.int32, device=x.device)
        code = fn(x.data_ptr(), rows, cols, cols, mode, rht, sp, seed, 0, qd.data_ptr(), sc.data_ptr(),
                  pts.data_ptr(), ws.data_ptr(), 64, stream)
    else:
        code = fn(x.data_ptr(), rows, cols, cols, mode, rht, sp, seed, 0, qd.data_ptr(), sc.data_ptr(),
                  pts.data_ptr(), stream)
    assert code == 0
    torch.cuda.synchronize()
    return qd, sc, pts


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    from nvfp4_sm120_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(5)
    signs = torch.tensor([1, -1, 1, 1, -1, -1, 1, -1, 1, 1, -1, 1, -1, 1, 1, -1], dtype=torch.float32, device="cuda")
    # two calls in a row on the same stream, different inputs and modes: the second one runs on the
    # scratch the first one left behind
    cases = [(torch.randn(1024, 2048, device="cuda", dtype=torch.bfloat16, generator=g), 0, 0, 0),
             (torch.randn(520, 4096, device="cuda", dtype=torch.bfloat16, generator=g) * 7, 1, 1, 11)]
    got = [_call(L.nvfp4_quantize_static_bf16, x, mode, rht, signs, seed, False) for (x, mode, rht, seed) in cases]
    want = [_call(L.nvfp4_quantize_fused_bf16, x, mode, rht, signs, seed, True) for (x, mode, rht, seed) in cases]
    for (gq, gs, gp), (wq, ws_, wp) in zip(got, want):
        assert torch.equal(gq, wq)          # bit-exact: same kernel, only the scratch lives elsewhere
        assert torch.equal(gs, ws_)
        assert torch.equal(gp, wp)


def test_static_scratch_entry_point_rejects_oversize_and_bad_shapes():
    from nvfp4_sm120_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(16, 32, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    args = (0, 0, None, 0, 0, out.data_ptr(), out.data_ptr(), None, None)
    assert L.nvfp4_quantize_static_bf16(x.data_ptr(), 2 ** 31, 16, 16, *args) == -8        # NVFP4_E_LIMIT
    assert L.nvfp4_quantize_static_bf16(x.data_ptr(), 16, 24, 24, *args) == -2             # cols % 16
