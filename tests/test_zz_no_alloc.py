"""The allocation-free mHC pre entry point against the regular one.

Collected last on purpose (file name), so a run that stops at the first failure
has already run every other test.  Passes alone in a fresh process and after
the rest of the suite: it depends on no state left by other tests.
"""
import numpy as np
import pytest

import cases
from _gpu import bits, lib
from _oracle import P

pytestmark = pytest.mark.gpu


def regular(c, rows, d, n):
    y = np.empty((rows, d), np.float32); yn = np.empty((rows, d), np.float32)
    post = np.empty((rows, n), np.float32); comb = np.empty((rows, n, n), np.float32)
    rc = lib().apus_cuda_hc_pre(P(c["x4"]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]), 1e-6, 1e-6, 20,
                                P(c["norm_w"]), 1e-6, P(y), P(yn), P(post), P(comb), rows)
    assert rc == 0, lib().apus_cuda_last_error()
    lib().apus_cuda_forget(P(c["fn"]))
    return y, yn, post, comb


def no_alloc(c, rows, d, n):
    """Inputs and outputs are caller-owned device tensors; the entry point
    itself must allocate nothing."""
    import torch
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    x4, fn, scale, base, nw = t(c["x4"]), t(c["fn"]), t(c["scale"]), t(c["base"]), t(c["norm_w"])
    y = torch.empty(rows, d, device=dev); yn = torch.empty(rows, d, device=dev)
    post = torch.empty(rows, n, device=dev); comb = torch.empty(rows, n, n, device=dev)
    torch.cuda.synchronize()
    rc = lib().apus_cuda_hc_pre_noalloc_dev(x4.data_ptr(), d, n, fn.data_ptr(), scale.data_ptr(),
                                            base.data_ptr(), 1e-6, 1e-6, 20, nw.data_ptr(), 1e-6,
                                            y.data_ptr(), yn.data_ptr(), post.data_ptr(), comb.data_ptr(),
                                            rows, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib().apus_cuda_last_error()
    torch.cuda.synchronize()
    return tuple(v.cpu().numpy() for v in (y, yn, post, comb))


def test_no_alloc_matches_regular_twice_in_a_row():
    n = 4
    # two calls in a row with different sizes: the second must not see anything
    # the first left in the shared scratch
    for seed, rows, d in ((701, 7, 256), (702, 3, 4096)):
        c = cases.mhc_case(seed, rows, d)
        want = regular(c, rows, d, n)
        got = no_alloc(c, rows, d, n)
        for g, w in zip(got, want):      # same kernels, same order: identical bits
            assert np.array_equal(bits(g), bits(w))


@pytest.mark.parametrize("rows", [255, 256])
def test_no_alloc_at_the_row_limit_and_free_memory_unchanged(rows):
    """The largest calls the fixed scratch admits (an odd row count exercises the tail of
    the two-tokens-per-CTA kernel), bit for bit against the regular entry point; and a
    warmed-up call leaves the device's free memory where it was: nothing was allocated."""
    import torch
    n, d = 4, 128
    c = cases.mhc_case(703, rows, d)
    want = regular(c, rows, d, n)
    got = no_alloc(c, rows, d, n)                 # warm-up: resolves the scratch address on this device
    for g, w in zip(got, want):
        assert np.array_equal(bits(g), bits(w))
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    x4, fn, scale, base, nw = t(c["x4"]), t(c["fn"]), t(c["scale"]), t(c["base"]), t(c["norm_w"])
    y = torch.empty(rows, d, device=dev); yn = torch.empty(rows, d, device=dev)
    post = torch.empty(rows, n, device=dev); comb = torch.empty(rows, n, n, device=dev)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    rc = lib().apus_cuda_hc_pre_noalloc_dev(x4.data_ptr(), d, n, fn.data_ptr(), scale.data_ptr(), base.data_ptr(), 1e-6,
                                            1e-6, 20, nw.data_ptr(), 1e-6, y.data_ptr(), yn.data_ptr(), post.data_ptr(),
                                            comb.data_ptr(), rows, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib().apus_cuda_last_error()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free device memory moved by {free0 - free1} bytes across the call"
    assert np.array_equal(bits(y.cpu().numpy()), bits(want[0]))


def test_no_alloc_rejects_oversize():
    import torch
    d, n, rows = 64, 4, 257
    z = torch.zeros(rows * n * d, device="cuda")
    rc = lib().apus_cuda_hc_pre_noalloc_dev(z.data_ptr(), d, n, z.data_ptr(), z.data_ptr(), z.data_ptr(),
                                            1e-6, 1e-6, 20, None, 1e-6, z.data_ptr(), None, z.data_ptr(),
                                            z.data_ptr(), rows, None)
    assert rc != 0
    assert b"exceed the fixed scratch" in lib().apus_cuda_last_error()
