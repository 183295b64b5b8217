"""The allocation-free column-statistics entry point, h3s_column_stats_static.

It exists for hosts that may not allocate device memory at the moment they
need the K mean / V scale (a serving process with a frozen pool, a plug-in
running inside another framework's operator).  The scratch it accumulates in
is an array inside the library, shared by every call on the device, so the
thing to prove is that a call's result does not depend on what the previous
call left there: two calls in a row, on different shapes and data, must each
match h3s_column_stats (which gets a fresh scratch buffer from the caller).

Collected last on purpose: a run that stops at the first failure has then
already exercised every other test.  Needs a B200.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(heads, sequence, seed, dtype):
    gen = torch.Generator().manual_seed(seed)
    k = (torch.randn((1, heads, sequence, 128), generator=gen) + 0.25).to(dtype).cuda()
    v = (torch.randn((1, heads, sequence, 128), generator=gen) * (1 + seed)).to(dtype).cuda()
    return k, v


def _call_static(lib, k, v, k_mean, v_scale):
    """Straight through the C ABI: raw pointers, strides in elements, the current stream."""
    from h3_optimizations_b200 import _native

    heads, sequence = k.shape[1], k.shape[2]
    status = lib.h3s_column_stats_static(
        ctypes.c_void_p(k.data_ptr()), k.stride(1), k.stride(2),
        ctypes.c_void_p(v.data_ptr()), v.stride(1), v.stride(2),
        _native.dtype_code(k.dtype), heads, sequence, 448.0,
        ctypes.c_void_p(k_mean.data_ptr()), ctypes.c_void_p(v_scale.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert status == 0, lib.h3s_last_error().decode()


def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch(native_lib):
    from h3_optimizations_b200 import ops

    # a large first problem, then a smaller one with other data: if the shared
    # scratch were not cleared, the second result would carry the first one's sums
    for heads, sequence, seed, dtype in ((5, 1500, 1, torch.bfloat16), (2, 333, 2, torch.float32)):
        k, v = _inputs(heads, sequence, seed, dtype)
        want_mean, want_scale = ops.column_stats(k, v)
        got_mean = torch.full((1, heads, 128), float("nan"), dtype=torch.float32, device="cuda")
        got_scale = torch.full_like(got_mean, float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        _call_static(native_lib, k, v, got_mean, got_scale)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # device memory in use is the same before and after: the call allocated nothing, not
        # through torch's pool (the ABI knows nothing of it) and not from the driver either
        assert free_after == free_before, "the call changed the device's free memory by %d bytes" % (free_before - free_after)
        # the V scale is a maximum: order independent, so identical
        assert torch.equal(got_scale, want_scale)
        # the K mean is an FP64 sum gathered with atomics whose order varies from
        # launch to launch; after rounding the two agree to the last place or so
        assert torch.allclose(got_mean, want_mean, rtol=1e-6, atol=1e-7)
        # and both are right, not merely equal
        assert torch.allclose(got_mean.cpu(), k.float().mean(dim=-2).cpu(), rtol=0, atol=4e-3)


def test_sizes_beyond_the_built_in_scratch_are_refused(native_lib):
    status = native_lib.h3s_column_stats_static(None, 0, 0, None, 0, 0, 1, 65, 128, 448.0, None, None, None)
    assert status == -1
    message = native_lib.h3s_last_error().decode()
    assert "65 heads exceed the 64" in message and "h3s_column_stats" in message
