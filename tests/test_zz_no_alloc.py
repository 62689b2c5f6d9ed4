"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory when they call in (memory-planned
regions, plugins inside another runtime, latency-critical loops), so ``cb_rmsnorm_bwd_noalloc``
keeps its scratch inside the library.  This checks that it returns what the ordinary entry point
``cb_rmsnorm_bwd`` returns, twice in a row (the second call reuses the scratch the first one
dirtied), and that it refuses sizes beyond its built-in scratch.  The file name sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from chronicals_b200.csrc import build
    path = build.build()
    lib = ctypes.CDLL(path)
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.cb_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, F, I, P]
    lib.cb_rmsnorm_bwd_noalloc.restype = I
    lib.cb_rmsnorm_bwd_noalloc_max_n.restype = I
    lib.cb_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, P, I, I, F, I, P]
    lib.cb_rmsnorm_bwd.restype = I
    lib.cb_rmsnorm_bwd_blocks.argtypes = [I, I]
    lib.cb_rmsnorm_bwd_blocks.restype = I
    return lib


def _case(M, N, seed):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
    h = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).to(dev)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6).contiguous()
    return dy, h, w, res, rstd


@pytest.mark.parametrize("M,N", [(1000, 896), (77, 5120)])
def test_noalloc_matches_regular_entry_point_twice(M, N):
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                                  # second call sees the first call's leftovers
        dy, h, w, res, rstd = _case(M, N, seed=call)
        dx_ref, dw_ref = torch.empty_like(h), torch.empty_like(w)
        blocks = lib.cb_rmsnorm_bwd_blocks(M, N)
        part = torch.empty(blocks * N, dtype=torch.float32, device="cuda")
        rc = lib.cb_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), res.data_ptr(),
                                dx_ref.data_ptr(), dw_ref.data_ptr(), part.data_ptr(), M, N, 0.0, 0, stream)
        assert rc == 0
        dx, dw = torch.empty_like(h), torch.empty_like(w)
        rc = lib.cb_rmsnorm_bwd_noalloc(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), res.data_ptr(),
                                        dx.data_ptr(), dw.data_ptr(), M, N, 0.0, 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref), "dx does not depend on the scratch and must match bit for bit"
        err = (dw.float() - dw_ref.float()).abs().max().item()
        mag = dw_ref.float().abs().max().item()
        assert err <= 2e-2 + 2e-2 * mag, (err, mag)        # same tolerance as the other kernel tests


def test_noalloc_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    n_max = lib.cb_rmsnorm_bwd_noalloc_max_n()
    assert n_max == 8192
    N = n_max + 8
    t = torch.zeros(2, N, dtype=torch.bfloat16, device="cuda")
    r = torch.ones(2, dtype=torch.float32, device="cuda")
    rc = lib.cb_rmsnorm_bwd_noalloc(t.data_ptr(), t.data_ptr(), t[0].data_ptr(), r.data_ptr(), None, t.data_ptr(),
                                    None, 2, N, 0.0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -2
