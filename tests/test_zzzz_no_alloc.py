"""The allocation-free batch-norm entry point, called the way an embedder would call it: straight through
the exported C symbol of the shared library, with nothing but input and output buffers.

Some hosts of this library cannot let it allocate on the GPU -- all device memory belongs to their own
pool, or they sit in a loop where cudaMalloc's device-wide synchronisation is not acceptable. For them
`rb_bn_fwd_train_noalloc` keeps its per-channel scratch inside the library image. This test checks that
it agrees with the regular entry point (which takes a caller-provided scratch buffer) on two consecutive
calls with different data -- the second call must not see leftovers of the first in the shared scratch --
and that a channel count beyond the built-in maximum is refused with the documented code.

The file name sorts last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from rembrandt_b200 import _native

MAX_CHANNELS = 4096
E_TOO_MANY = -20


def _lib():
    _native.cuda()  # builds the library if needed
    lib = C.CDLL(str(_native.cuda_lib_path()))
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    lib.rb_bn_fwd_train_noalloc.argtypes = [vp, i64, i32, i32, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp]
    lib.rb_bn_fwd_train_noalloc.restype = i32
    lib.rb_bn_fwd_train.argtypes = [vp, i64, i32, i32, vp, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, vp]
    lib.rb_bn_fwd_train.restype = i32
    lib.rb_bn_noalloc_strerror.argtypes = [i32]
    lib.rb_bn_noalloc_strerror.restype = C.c_char_p
    return lib


def _run_both(lib, rows, channels, seed, with_residual):
    # a stream of our own: the entry point's last argument is the stream it must order its clear and kernels on
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        outs = _run_both_on_current_stream(lib, rows, channels, seed, with_residual)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return outs


def _run_both_on_current_stream(lib, rows, channels, seed, with_residual):
    torch.manual_seed(seed)
    dev = "cuda"
    x = (torch.randn(rows, channels, device=dev) * 1.7 + 0.3).bfloat16()
    res = torch.randn(rows, channels, device=dev).bfloat16() if with_residual else None
    gamma = torch.rand(channels, device=dev) + 0.5
    beta = torch.randn(channels, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for which in ("noalloc", "regular"):
        y = torch.full((rows, channels), float("nan"), device=dev, dtype=torch.bfloat16)
        mean = torch.empty(channels, device=dev)
        istd = torch.empty(channels, device=dev)
        rm = torch.zeros(channels, device=dev)
        rv = torch.ones(channels, device=dev)
        rp = res.data_ptr() if res is not None else None
        if which == "noalloc":
            rc = lib.rb_bn_fwd_train_noalloc(x.data_ptr(), rows, channels, channels, 1e-5, 0.1, mean.data_ptr(),
                                             istd.data_ptr(), rm.data_ptr(), rv.data_ptr(), gamma.data_ptr(),
                                             beta.data_ptr(), rp, y.data_ptr(), 1, stream)
        else:
            sums = torch.zeros(2 * channels, device=dev)
            rc = lib.rb_bn_fwd_train(x.data_ptr(), rows, channels, channels, sums.data_ptr(), 1e-5, 0.1,
                                     mean.data_ptr(), istd.data_ptr(), rm.data_ptr(), rv.data_ptr(), gamma.data_ptr(),
                                     beta.data_ptr(), rp, y.data_ptr(), 1, 0, None, stream)
        assert rc == 0, lib.rb_bn_noalloc_strerror(rc)
        torch.cuda.synchronize()
        outs.append((y.float(), mean, istd, rm, rv))
    return outs


def _assert_close(a, b, what):
    scale = float(b.abs().max().clamp_min(1e-6))
    err = float((a - b).abs().max())
    assert not torch.isnan(a).any(), f"{what}: NaN (unwritten output)"
    assert err <= 2e-2 * scale, f"{what}: max err {err:.4g} vs scale {scale:.4g}"


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row():
    lib = _lib()
    # first call: wide tensor; second call: fewer channels and other data, reusing the same built-in scratch
    for rows, channels, seed, with_res in ((1000, 256, 1, False), (777, 64, 2, True)):
        got, ref = _run_both(lib, rows, channels, seed, with_res)
        for g, r, name in zip(got, ref, ("y", "mean", "istd", "running mean", "running var")):
            _assert_close(g, r, f"{name} (C={channels})")


def test_noalloc_rejects_more_channels_than_the_built_in_scratch_holds():
    lib = _lib()
    rc = lib.rb_bn_fwd_train_noalloc(None, 8, MAX_CHANNELS + 8, MAX_CHANNELS + 8, 1e-5, 0.1, None, None, None, None,
                                     None, None, None, None, 0, None)
    assert rc == E_TOO_MANY
    assert b"4096" in lib.rb_bn_noalloc_strerror(rc)
