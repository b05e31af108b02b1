"""rewb200_linear_noalloc against rewb200_linear, through the C ABI.

The no-allocation entry point exists for hosts that cannot call cudaMalloc
(their own allocator owns the device heap, or they are inside a section that
must not synchronise the device).  It keeps split-K partial sums in a fixed
array inside the library, shared by every call, so this test makes two calls
in a row with different inputs and checks each against the allocating entry
point: the second result must not be polluted by what the first left behind.
Collected last so that a failure here cannot hide another test's result.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _case(api, lib, seed, M, K, N, with_bias):
    from oracle import orc
    from rew_b200 import _lib
    rng = np.random.default_rng(seed)
    xh = orc.bf16_round(rng.normal(size=(M, K)).astype(np.float32))
    wh = orc.bf16_round(rng.normal(0, 0.05, size=(K, N)).astype(np.float32))
    bh = rng.normal(0, 0.1, size=(N,)).astype(np.float32) if with_bias else None
    x = api.Tensor.from_host(xh, _lib.BF16)
    w = api.Tensor.from_host(wh, _lib.BF16)
    b = api.Tensor.from_host(bh) if with_bias else None
    want = api.Linear(w, b).forward(x).to_host()
    # and the CPU restatement of Linear.forward on the same bf16-rounded operands
    want_orc = orc.linear(xh, wh, bh if with_bias else np.zeros(N, np.float32))
    y = api.Tensor.from_host(np.full((M, N), 7.0, np.float32), _lib.BF16)  # caller-owned output, pre-filled
    ptr = lambda t: C.c_void_p(lib.rewb200_buffer_device_ptr(t._h)) if t is not None else None
    _lib.check(lib.rewb200_linear_noalloc(0, ptr(x), ptr(w), ptr(b), ptr(y), M, K, N))
    got = y.to_host()
    assert np.isfinite(got).all()
    assert rel_l2(got, want) < 5e-3  # the tolerance of the bf16 Linear tests
    assert rel_l2(got, want_orc) < 5e-3
    return got


@pytest.mark.parametrize("linear", ["tc", "mma"])
def test_noalloc_linear_matches_allocating_linear_twice_in_a_row(linear):
    """Either GEMM that can stand behind the entry point writes its split-K slabs into the shared array."""
    from rew_b200 import _lib, api
    _lib.init()
    lib = _lib.lib()
    api.set_option("linear", linear)
    try:
        _twice(api, lib)
    finally:
        api.set_option("linear", "tc")


def _twice(api, lib):
    first = _case(api, lib, 1, 32, 4096, 1024, True)     # split-K > 1: several slabs of the shared array
    second = _case(api, lib, 2, 5, 1024, 4096, False)    # other shape, other data, stale slabs behind it
    again = _case(api, lib, 1, 32, 4096, 1024, True)     # and the first case once more
    assert np.array_equal(first, again)                    # deterministic: no atomics, fixed summation order
    assert second.shape == (5, 4096)


def test_noalloc_linear_rejects_sizes_beyond_the_fixed_scratch():
    from rew_b200 import _lib, api
    from rew_b200._lib import RewB200Error
    _lib.init()
    lib = _lib.lib()
    one = api.Tensor.from_host(np.zeros((8, 8), np.float32), _lib.BF16)
    p = C.c_void_p(lib.rewb200_buffer_device_ptr(one._h))
    with pytest.raises(RewB200Error, match="exceeds the fixed scratch"):
        _lib.check(lib.rewb200_linear_noalloc(0, p, p, None, p, 32, 8, 128 * 1024))
    with pytest.raises(RewB200Error, match="M <= 32"):
        _lib.check(lib.rewb200_linear_noalloc(0, p, p, None, p, 33, 8, 8))
