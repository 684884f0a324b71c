"""The allocation-free norm backward (`zb_norm_bwd_noalloc`, csrc/norm/norm_noalloc.h) must give
what the regular entry point gives.  It serves callers that cannot allocate device memory while
they run (allocator callbacks, threads barred from the allocator lock, guests in a process whose
memory someone else budgets): its scratch is an 8 MiB array compiled into the library.

The symbol is called through ctypes exactly as a C caller would, twice in a row, because every
call reuses the same scratch array and the second call must not be disturbed by what the first
left there.  This file sorts last on purpose so a run that stops at the first failure has
already executed every other test.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


@pytest.mark.parametrize("ln", [False, True])
def test_noalloc_matches_regular_entry_point(ln):
    from zorse_b200.ops import sm100 as k

    lib = k.lib()
    fn = lib.zb_norm_bwd_noalloc
    fn.restype = c_int
    g = torch.Generator().manual_seed(3)
    for (T, H), gdt in (((333, 4096), torch.float32), ((64, 1024), torch.bfloat16)):   # two calls in a row, different shapes
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        dy = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        dres = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(H, generator=g) * 0.1 + 1).to(torch.bfloat16).cuda()
        b = (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16).cuda() if ln else None
        _, stats = k.norm_fwd(x, w, b, 1e-5, ln)
        dw_ref = torch.ones(H, dtype=gdt, device="cuda")
        db_ref = torch.ones(H, dtype=gdt, device="cuda") if ln else None
        # the regular entry point this one is a variant of (zb_norm_bwd = version 1 of the wrapper)
        dx_ref = k.norm_bwd(dy, x, w, stats, dres, dw_ref, db_ref, ln, version=1)
        dw = torch.ones(H, dtype=gdt, device="cuda")
        db = torch.ones(H, dtype=gdt, device="cuda") if ln else None
        dx = torch.empty_like(x)
        assert lib.zb_norm_bwd_noalloc_init() == 0     # start-up call: resolves the scratch address on this device
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]     # the driver's view: a cudaMalloc inside the call would show here
        stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = fn(_ptr(dy), _ptr(x), _ptr(w), _ptr(stats), _ptr(dres), _ptr(dx), _ptr(dw), _ptr(db), c_int(T), c_int(H),
                c_int(int(ln)), c_int(int(gdt == torch.float32)), c_int(1), stream)
        assert rc == 0, lib.zb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(dx, dx_ref)
        tol = 1e-3 if gdt == torch.float32 else 6e-2
        assert (dw.float() - dw_ref.float()).abs().max().item() <= tol * max(1.0, dw_ref.float().abs().max().item())
        if ln:
            assert (db.float() - db_ref.float()).abs().max().item() <= tol * max(1.0, db_ref.float().abs().max().item())


def test_noalloc_rejects_oversized_hidden():
    from zorse_b200.ops import sm100 as k

    lib = k.lib()
    fn = lib.zb_norm_bwd_noalloc
    fn.restype = c_int
    z = c_void_p(0)
    rc = fn(z, z, z, z, z, z, z, z, c_int(4), c_int(16384), c_int(0), c_int(1), c_int(1), z)
    assert rc == -1 and b"exceeds the built-in scratch" in lib.zb_last_error()
