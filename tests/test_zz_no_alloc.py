"""The allocation-free SRW forward entry point, called through its exported C
symbol, against the ordinary entry point that takes scratch from the caller.

Who needs it: embedders that cannot allocate device memory at the point of the
call (a server whose memory pool owns the whole GPU, a latency-critical thread
where cudaMalloc's device-wide synchronisation is unacceptable, a sandbox that
forbids the allocator).  The scratch tile lives in the library image instead.

This file is named so that pytest collects it last.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


class DsbGate(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("sharpness", ctypes.c_float), ("act_threshold", ctypes.c_float),
                ("act_cutoff", ctypes.c_float), ("epsilon", ctypes.c_float),
                ("max_intensity", ctypes.c_float), ("clip_max", ctypes.c_float),
                ("dead_threshold", ctypes.c_float)]


def _lib():
    from dawn_srw_b200.ops import build
    if not build.PLAIN_SO_PATH.exists():
        build.build()
    lib = ctypes.CDLL(str(build.PLAIN_SO_PATH))
    lib.dsb_srw_forward_static_last_error.restype = ctypes.c_char_p
    lib.dsb_srw_forward_static_capacity.restype = ctypes.c_ulonglong
    lib.dsb_srw_forward_static_bytes_needed.restype = ctypes.c_ulonglong
    return lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _ll(v):
    return ctypes.c_longlong(v)


def _problem(T, U, r, D, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    nz = torch.nn.functional.normalize
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    h, x = rn(T, r).bfloat16(), rn(T, D).bfloat16()
    emb, read, write = (nz(rn(U, d), dim=-1).bfloat16() for d in (r, D, D))
    s = h.float() @ emb.float().t()
    mu, sd = s.mean(-1), s.std(-1, unbiased=False) + 1e-8
    return h, emb, x, read, write, (mu + 0.2 * sd).contiguous(), (1.0 / sd).contiguous()


def _run(lib, static, prob, gate, status):
    h, emb, x, read, write, tau, isd = prob
    T, D, U, r = x.shape[0], x.shape[1], emb.shape[0], emb.shape[1]
    dev = x.device
    raw = torch.full((T, D), float("nan"), device=dev)
    den = torch.full((T,), float("nan"), device=dev)
    common = [_ptr(h), _ll(h.stride(0)), _ptr(emb), _ll(emb.stride(0)), _ptr(x), _ll(x.stride(0)),
              _ptr(read), _ll(read.stride(0)), _ptr(write), _ll(write.stride(0)),
              ctypes.c_int(T), ctypes.c_int(U), ctypes.c_int(r), ctypes.c_int(D), _ptr(tau), _ptr(isd)]
    tail = [_ptr(raw), _ll(raw.stride(0)), _ptr(den), ctypes.c_void_p(0), ctypes.c_void_p(0),
            ctypes.byref(gate), _ptr(status), ctypes.c_void_p(0)]     # stream 0 = torch's default stream
    if static:
        rc = lib.dsb_srw_forward_static(*common, *tail)
    else:
        Up = (U + 7) // 8 * 8
        scratch = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)   # the caller's allocation
        rc = lib.dsb_srw_forward(*common, _ptr(scratch), _ll(Up), *tail)
    torch.cuda.synchronize()
    return rc, raw, den


def test_static_scratch_entry_point_matches_the_allocating_one():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _lib()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gate = DsbGate(1, 500.0, 0.5, 0.01, 1e-4, 10.0, 10.0, 0.01)          # z * Phi(z) gate
    assert lib.dsb_srw_forward_static_capacity() == 64 << 20
    # two calls in a row with different shapes: the second must not be disturbed
    # by what the first left in the shared buffer
    for seed, (T, U, r, D) in enumerate([(384, 2600, 128, 384), (200, 1580, 64, 256)]):
        prob = _problem(T, U, r, D, seed, dev)
        rc_a, raw_a, den_a = _run(lib, False, prob, gate, status)
        rc_s, raw_s, den_s = _run(lib, True, prob, gate, status)
        # the contract in the name: once warm, a static call takes no device memory, neither
        # from the driver nor from torch's allocator (its outputs are allocated before the
        # measurement, exactly like the caller's own buffers would be)
        raw2 = torch.empty_like(raw_s)
        den2 = torch.empty_like(den_s)
        import gc
        gc.collect()                                  # earlier temporaries are gone before the baseline
        torch.cuda.synchronize()
        free0, alloc0 = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev)
        peak0 = torch.cuda.max_memory_allocated(dev)
        h, emb, x, read, write, tau, isd = prob
        for _ in range(2):
            rc = lib.dsb_srw_forward_static(
                _ptr(h), _ll(h.stride(0)), _ptr(emb), _ll(emb.stride(0)), _ptr(x), _ll(x.stride(0)),
                _ptr(read), _ll(read.stride(0)), _ptr(write), _ll(write.stride(0)), ctypes.c_int(T),
                ctypes.c_int(U), ctypes.c_int(r), ctypes.c_int(D), _ptr(tau), _ptr(isd), _ptr(raw2),
                _ll(raw2.stride(0)), _ptr(den2), ctypes.c_void_p(0), ctypes.c_void_p(0),
                ctypes.byref(gate), _ptr(status), ctypes.c_void_p(0))
            assert rc == 0
        torch.cuda.synchronize()
        # nothing was taken from the driver, and torch's allocator saw no request either (its
        # high-water mark did not move; the current figure may only have gone down)
        assert torch.cuda.mem_get_info(dev)[0] == free0
        assert torch.cuda.memory_allocated(dev) <= alloc0
        assert torch.cuda.max_memory_allocated(dev) == peak0
        assert torch.equal(raw2, raw_s)
        assert rc_a == 0 and rc_s == 0, lib.dsb_srw_forward_static_last_error()
        assert int(status.item()) == 0
        assert torch.isfinite(raw_s).all() and torch.isfinite(den_s).all()
        rel = ((raw_s - raw_a).norm() / (raw_a.norm() + 1e-12)).item()
        assert rel < 1e-5, rel
        assert torch.allclose(den_s, den_a, rtol=1e-4, atol=1e-5)
        # and both agree with plain fp32 math on the same bf16 inputs
        h, emb, x, read, write, tau, isd = prob
        z = ((h.float() @ emb.float().t()) - tau[:, None]) * isd[:, None]
        gte = torch.where(z > 0, z * 0.5 * (1 + torch.erf(z * 0.7071067811865476)), torch.zeros_like(z))
        ref = (gte * (x.float() @ read.float().t())) @ write.float()
        assert ((raw_s - ref).norm() / ref.norm()).item() < 6e-3
        assert torch.allclose(den_s, gte.sum(-1), rtol=1e-3, atol=1e-3)


def test_static_scratch_entry_point_refuses_oversized_problems():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _lib()
    T, U = 8192, 100000                              # 1.6 GB of scratch: far beyond 64 MiB
    assert lib.dsb_srw_forward_static_bytes_needed(T, U) > lib.dsb_srw_forward_static_capacity()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gate = DsbGate(1, 500.0, 0.5, 0.01, 1e-4, 10.0, 10.0, 0.01)
    null = ctypes.c_void_p(0)
    rc = lib.dsb_srw_forward_static(null, _ll(8), null, _ll(8), null, _ll(8), null, _ll(8), null, _ll(8),
                                    ctypes.c_int(T), ctypes.c_int(U), ctypes.c_int(64), ctypes.c_int(64),
                                    null, null, null, _ll(64), null, null, null, ctypes.byref(gate),
                                    _ptr(status), null)
    assert rc == 501
    msg = lib.dsb_srw_forward_static_last_error().decode()
    assert "needs" in msg and "static" in msg
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_static_scratch_entry_point_at_exactly_its_capacity():
    """T = 4096 tokens x U = 8192 units needs exactly the 64 MiB the library
    holds: accepted and correct; eight more (padded) units are refused."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _lib()
    T, U, r, D = 4096, 8192, 64, 128
    assert lib.dsb_srw_forward_static_bytes_needed(T, U) == lib.dsb_srw_forward_static_capacity()
    assert lib.dsb_srw_forward_static_bytes_needed(T, U + 1) > lib.dsb_srw_forward_static_capacity()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gate = DsbGate(1, 500.0, 0.5, 0.01, 1e-4, 10.0, 10.0, 0.01)
    prob = _problem(T, U, r, D, 5, dev)
    rc_a, raw_a, den_a = _run(lib, False, prob, gate, status)
    rc_s, raw_s, den_s = _run(lib, True, prob, gate, status)
    assert rc_a == 0 and rc_s == 0, lib.dsb_srw_forward_static_last_error()
    assert int(status.item()) == 0
    assert ((raw_s - raw_a).norm() / (raw_a.norm() + 1e-12)).item() < 1e-5
    assert torch.allclose(den_s, den_a, rtol=1e-4, atol=1e-5)
    null = ctypes.c_void_p(0)
    rc = lib.dsb_srw_forward_static(null, _ll(8), null, _ll(8), null, _ll(8), null, _ll(8), null, _ll(8),
                                    ctypes.c_int(T), ctypes.c_int(U + 1), ctypes.c_int(r),
                                    ctypes.c_int(D), null, null, null, _ll(D), null, null, null,
                                    ctypes.byref(gate), _ptr(status), null)
    assert rc == 501
