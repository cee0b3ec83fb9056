"""The allocation-free batch-norm forward (mb_bn_fwd_train_noalloc) against the regular entry
point, through the C ABI.

Some hosts of this library cannot allocate while a step is running: MONeT executes a schedule
solved for a fixed memory budget, and a pool that owns the whole device leaves nothing for a
kernel that wants extra scratch at run time.  For them the statistics scratch lives in an
8 MiB array inside the library.  The array is shared by every call and keeps the previous
call's contents, so the test makes two calls in a row on different data and expects each to
match the workspace-taking entry point exactly (same kernels, same partial-sum layout).

Collected last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(cuda, shape, seed, nhwc):
    from monet_b200 import _lib
    api = _lib.lib()
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g).to(cuda) * 2 + 0.5
    if nhwc:
        x = x.contiguous(memory_format=torch.channels_last)
    Cc = shape[1]
    gamma = (torch.rand(Cc, generator=g) + 0.5).to(cuda)
    beta = torch.randn(Cc, generator=g).to(cuda)
    d = _lib.BnDesc(shape[0], Cc, shape[2] * shape[3], _lib.MB_NHWC if nhwc else _lib.MB_NCHW, 1e-5, 0.1)
    stream = torch.cuda.current_stream().cuda_stream
    out = {}
    for name in ("regular", "noalloc"):
        y = torch.empty_like(x)
        mean = torch.empty(Cc, device=cuda)
        invstd = torch.empty(Cc, device=cuda)
        rm, rv = torch.zeros(Cc, device=cuda), torch.ones(Cc, device=cuda)
        if name == "regular":
            ws = torch.empty(api.mb_bn_workspace_bytes(C.byref(d)), dtype=torch.uint8, device=cuda)
            rc = api.mb_bn_fwd_train(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), rm.data_ptr(),
                                     rv.data_ptr(), y.data_ptr(), mean.data_ptr(), invstd.data_ptr(),
                                     C.byref(d), ws.data_ptr(), ws.numel(), stream)
        else:
            rc = api.mb_bn_fwd_train_noalloc(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                             rm.data_ptr(), rv.data_ptr(), y.data_ptr(),
                                             mean.data_ptr(), invstd.data_ptr(), C.byref(d), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        out[name] = (y, mean, invstd, rm, rv)
    return out


@pytest.mark.parametrize("nhwc", [True, False])
def test_noalloc_matches_regular_on_two_calls_in_a_row(cuda, nhwc):
    # two different shapes and data sets back to back: the second call sees the first one's
    # leftovers in the shared array and must not be affected by them
    for shape, seed in (((16, 256, 28, 28), 1), ((8, 64, 56, 56), 2)):
        out = _run_both(cuda, shape, seed, nhwc)
        for a, b in zip(out["regular"], out["noalloc"]):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
        y, mean, invstd = out["noalloc"][:3]
        assert torch.isfinite(y).all() and torch.isfinite(mean).all() and (invstd > 0).all()


def test_noalloc_rejects_shapes_beyond_the_built_in_scratch(cuda):
    from monet_b200 import _lib
    api = _lib.lib()
    # (2*S + 2) * C floats of scratch: 600 000 channels need 9.6 MB even with one chunk
    d = _lib.BnDesc(1, 600000, 2, _lib.MB_NHWC, 1e-5, 0.1)
    assert api.mb_bn_workspace_bytes(C.byref(d)) > 8 * 2 ** 20
    t = torch.empty(16, device=cuda)
    rc = api.mb_bn_fwd_train_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), None, None,
                                     t.data_ptr(), t.data_ptr(), t.data_ptr(), C.byref(d), None)
    assert rc == 3
    assert "scratch" in _lib.last_error() and "mb_bn_fwd_train" in _lib.last_error()


def _call_noalloc(api, _lib, x, gamma, beta, nhwc, stream):
    Cc = x.shape[1]
    d = _lib.BnDesc(x.shape[0], Cc, x.shape[2] * x.shape[3], _lib.MB_NHWC if nhwc else _lib.MB_NCHW, 1e-5, 0.1)
    y = torch.empty_like(x)
    mean = torch.empty(Cc, device=x.device)
    invstd = torch.empty(Cc, device=x.device)
    rc = api.mb_bn_fwd_train_noalloc(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), None, None,
                                     y.data_ptr(), mean.data_ptr(), invstd.data_ptr(), C.byref(d), stream)
    assert rc == 0, _lib.last_error()
    return y, mean, invstd


def test_noalloc_calls_queued_back_to_back_allocate_nothing_and_match_the_oracle(cuda):
    """The documented safe pattern: calls queued on ONE stream with no host synchronisation in
    between (the second call's kernels reuse the array the first call's are still using, in
    stream order).  Outputs are compared with the CPU oracle, and the device's free memory
    (cudaMemGetInfo) and torch's allocator must be unchanged across the calls: every buffer
    the test passes was allocated before them."""
    from monet_b200 import _lib
    from oracle import lm_ops_oracle as oracle
    api = _lib.lib()
    g = torch.Generator().manual_seed(9)
    cases = []
    for shape in ((16, 256, 28, 28), (8, 64, 56, 56), (4, 96, 7, 7)):
        x = (torch.randn(shape, generator=g) * 1.5 - 0.3).to(cuda).contiguous(memory_format=torch.channels_last)
        gamma = (torch.rand(shape[1], generator=g) + 0.5).to(cuda)
        beta = torch.randn(shape[1], generator=g).to(cuda)
        cases.append((x, gamma, beta))
    stream = torch.cuda.current_stream().cuda_stream
    # first call on the device resolves the array's address; outputs pre-allocated below
    _call_noalloc(api, _lib, *cases[0], True, stream)
    torch.cuda.synchronize()
    outs = [(torch.empty_like(x), torch.empty(x.shape[1], device=cuda), torch.empty(x.shape[1], device=cuda))
            for x, _, _ in cases]
    descs = [_lib.BnDesc(x.shape[0], x.shape[1], x.shape[2] * x.shape[3], _lib.MB_NHWC, 1e-5, 0.1) for x, _, _ in cases]
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for (x, gamma, beta), (y, mean, invstd), d in zip(cases, outs, descs):        # no sync in between
        rc = api.mb_bn_fwd_train_noalloc(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), None, None,
                                         y.data_ptr(), mean.data_ptr(), invstd.data_ptr(), C.byref(d), stream)
        assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    for (x, gamma, beta), (y, mean, invstd) in zip(cases, outs):
        Cc = x.shape[1]
        o_y, o_mean, o_invstd, _, _ = oracle.bn_forward_train(x.cpu().contiguous(), gamma.cpu(), beta.cpu(),
                                                              torch.zeros(Cc), torch.ones(Cc))
        assert torch.allclose(y.cpu(), o_y, rtol=1e-5, atol=1e-5)
        assert torch.allclose(mean.cpu(), o_mean, rtol=1e-5, atol=1e-6)
        assert torch.allclose(invstd.cpu(), o_invstd, rtol=1e-5, atol=1e-6)
