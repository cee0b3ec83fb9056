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
