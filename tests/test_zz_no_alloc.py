# SPDX-License-Identifier: Apache-2.0
"""The allocation-free kinetic-energy entry point, called through its exported C symbol.

Some callers of the native library cannot obtain device memory at call time (a host loop that must not take allocator
locks, an application that owns the whole device memory pool, a raw-pointer plugin ABI).  For them the library exports
``nva_kinetic_energy_noalloc``, whose double-precision accumulator is a fixed device array inside the library image.
The test loads the shared library with ``ctypes``, passes raw device pointers, and checks two consecutive calls (the
second with fewer systems and different data, so stale sums of the first call would show) against the regular operator.
This file sorts last so that a failure here cannot hide the results of other tests."""
import ctypes

import pytest
import torch

from nvalchemi_toolkit_b200.ops import _native

pytestmark = pytest.mark.gpu


def _call(lib, vel, mass, bidx, m):
    out = torch.full((m,), float("nan"), device=vel.device)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.nva_kinetic_energy_noalloc(ctypes.c_void_p(vel.data_ptr()), ctypes.c_void_p(mass.data_ptr()),
                                        ctypes.c_void_p(bidx.data_ptr()), ctypes.c_int64(vel.shape[0]), ctypes.c_int(m),
                                        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream))
    return rc, out


def test_noalloc_kinetic_energy_matches_operator_twice():
    assert _native.available()
    lib = ctypes.CDLL(_native.LIB_PATH)
    lib.nva_kinetic_energy_noalloc.restype = ctypes.c_int
    lib.nva_noalloc_last_error.restype = ctypes.c_char_p
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    for m, n in ((7, 5000), (3, 1234)):
        sizes = torch.randint(1, 2 * n // m, (m,), generator=g, device=dev)
        bidx = torch.repeat_interleave(torch.arange(m, device=dev, dtype=torch.int32), sizes)
        na = bidx.numel()
        vel = torch.randn(na, 3, device=dev, generator=g)
        mass = torch.rand(na, device=dev, generator=g) * 50 + 1
        ref = torch.ops.nvalchemi.compute_kinetic_energy(vel, mass, bidx, m)
        rc, out = _call(lib, vel, mass, bidx, m)
        torch.cuda.synchronize()
        assert rc == 0, lib.nva_noalloc_last_error()
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
        # independent statement of the same sum in float64 PyTorch
        ke64 = 0.5 * mass.double() * vel.double().pow(2).sum(-1)
        ref64 = torch.zeros(m, dtype=torch.float64, device=dev).index_add_(0, bidx.long(), ke64)
        assert torch.allclose(out.double(), ref64, rtol=1e-5, atol=1e-6)
    # atoms labelled with a system outside [0, m) are ignored (nothing is written outside the slots of this call)
    bad = bidx.clone()
    bad[::7] = m + 3
    bad[1::11] = 70000
    bad[2::13] = -5
    keep = (bad >= 0) & (bad < m)
    rc, out = _call(lib, vel, mass, bad, m)
    torch.cuda.synchronize()
    assert rc == 0, lib.nva_noalloc_last_error()
    ref64 = torch.zeros(m, dtype=torch.float64, device=dev).index_add_(0, bad[keep].long(), ke64[keep])
    assert torch.allclose(out.double(), ref64, rtol=1e-5, atol=1e-6)
    # sizes beyond the fixed accumulator are refused with a message and leave the output untouched
    rc, out = _call(lib, vel, mass, bidx, 65537)
    assert rc == 1 and b"NVA_NOALLOC_MAX_SYSTEMS" in lib.nva_noalloc_last_error()
    assert torch.isnan(out).all()
