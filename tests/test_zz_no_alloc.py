"""The allocation-free entry point oc_moment_accum_static, called straight through the C ABI.

It exists for hosts that must not allocate device memory when they call into the library
(a call made under another runtime's stream capture or memory pool, or a process whose
device footprint is frozen after start-up): its scratch is a fixed array inside the library
instead of a buffer from the caller.  The test feeds the same chunks to it and to the
regular entry point (which gets a torch-allocated scratch) twice in a row and compares H and
C; the second call also proves that what the first call left in the shared array does no
harm.  This file sorts last on purpose, so a run that stops at the first failure has already
run every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _accumulate(lib, name, xq, xf, h, c, n_before, status, scratch=None):
    from onecompression_b200._lib import ptr, stream_handle

    t, d = xq.shape
    a_old, a_new = n_before / (n_before + t), 2.0 / (n_before + t)
    if name == "oc_moment_accum":
        rc = lib.oc_moment_accum(ptr(xq), ptr(xf), ptr(scratch), t, d, xq.stride(0), ptr(h), ptr(c), d,
                                 a_old, a_new, 0, 0, 0, 0, ptr(status), stream_handle())
    else:
        rc = lib.oc_moment_accum_static(ptr(xq), ptr(xf), t, d, xq.stride(0), ptr(h), ptr(c), d,
                                        a_old, a_new, 0, 0, 0, ptr(status), stream_handle())
    return rc


def test_static_scratch_entry_point_matches_regular_one():
    from onecompression_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(21)
    d, t = 512, 3000
    chunks = []
    for _ in range(2):
        xf = torch.randn(t, d, generator=g).half()
        xq = (xf.float() * (1 + 0.03 * torch.randn(t, d, generator=g))).half()
        chunks.append((xq.to(dev), xf.to(dev)))

    out = {}
    for name in ("oc_moment_accum", "oc_moment_accum_static"):
        h = torch.zeros(d, d, device=dev)
        c = torch.zeros(d, d, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        scratch = torch.empty(2 * t * d, dtype=torch.float16, device=dev)
        n = 0
        for xq, xf in chunks:                      # two calls in a row
            assert _accumulate(lib, name, xq, xf, h, c, n, status, scratch) == 0, lib.oc_last_error()
            n += xq.shape[0]
        assert lib.oc_mirror_upper(h.data_ptr(), d, d, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        out[name] = (h.cpu().double(), c.cpu().double())

    h0, c0 = out["oc_moment_accum"]
    h1, c1 = out["oc_moment_accum_static"]
    assert ((h1 - h0).norm() / h0.norm()).item() < 1e-5      # tolerance of the moment tests for H
    assert ((c1 - c0).norm() / c0.norm()).item() < 1e-4      # ... and for C
    # and both agree with float64
    xq = torch.cat([a.cpu() for a, _ in chunks]).double()
    xf = torch.cat([b.cpu() for _, b in chunks]).double()
    want_c = (2.0 / xq.shape[0]) * ((xf - xq).t() @ xq)
    assert ((c1 - want_c).norm() / want_c.norm()).item() < 1e-4


def test_static_scratch_rejects_oversized_call():
    from onecompression_b200 import _lib

    lib = _lib.load()
    cap = lib.oc_moment_static_capacity()
    assert cap == 16 * 1024 * 1024
    dev = torch.device("cuda:0")
    d = 64
    x = torch.zeros(8, d, dtype=torch.float16, device=dev)
    h = torch.zeros(d, d, device=dev)
    c = torch.zeros(d, d, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # claim more tokens than the scratch holds: refused before anything is launched
    rc = lib.oc_moment_accum_static(x.data_ptr(), x.data_ptr(), cap // d + 1, d, d, h.data_ptr(),
                                    c.data_ptr(), d, 0.0, 1.0, 0, 0, 0, status.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    assert b"built-in scratch" in lib.oc_last_error()
