"""The allocation-free LRU backward entry point against the regular one.

Some hosts of this library cannot give it a workspace: an XLA custom call sees
only the buffers the compiler planned, a replayed CUDA graph cannot grow one,
and a latency-critical acting loop must stay away from cudaMalloc.  For them
``mxk_linrec_c64_bwd_noalloc`` keeps its B*D partial sums in a fixed array
inside the library.  This file is named to be collected last, and the test
calls the entry point twice in a row because every call reuses that array.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def test_noalloc_matches_workspace_variant_twice():
    from memorax_b200 import _lib, ops
    lib = _lib.lib
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (bsz, steps, dim) in enumerate([(8, 37, 96), (5, 64, 130)]):
        gen = torch.Generator().manual_seed(100 + call)
        cplx = lambda *s: torch.complex(torch.randn(*s, generator=gen), torch.randn(*s, generator=gen)).cuda()
        lam = (cplx(dim) * 0.4).contiguous()
        bu, gh, h0, gh_last = cplx(bsz, steps, dim), cplx(bsz, steps, dim), cplx(bsz, dim), cplx(bsz, dim)
        done = (torch.rand(bsz, steps, generator=gen) < 0.05).to(torch.uint8).cuda()
        h, _ = ops.linrec_fwd(lam, bu, h0, None, done, want_decay=False)
        gb_ref, ga_ref, gh0_ref = ops.linrec_bwd(lam, h, h0, done, gh, gh_last)   # caller-provided workspace

        gb, ga, gh0 = torch.empty_like(h), torch.empty_like(lam), torch.empty_like(h0)
        st = lib.mxk_linrec_c64_bwd_noalloc(_p(lam), _p(h), _p(h0), _p(done), _p(gh), _p(gh_last), _p(gb), _p(ga),
                                            _p(gh0), bsz, steps, dim, 0, stream)
        assert st == 0, _lib.status_string(st)
        torch.cuda.synchronize()
        # same kernels, same reduction order: the two paths agree to fp32 round-off (1e-5 of max-abs)
        for got, ref in ((gb, gb_ref), (ga, ga_ref), (gh0, gh0_ref)):
            scale = float(ref.abs().max())
            assert float((got - ref).abs().max()) <= 1e-5 * scale


def test_noalloc_at_the_scratch_limit_against_oracle_and_workspace_variant():
    """B * D exactly at the limit (1024 x 512, the LRU benchmark's batch x width): every partial-sum
    slot of the built-in array is in use.  Checked against the regular entry point and, on a few
    sequences, against the fp64 oracle; one element more is rejected."""
    from memorax_b200 import _lib, ops
    from oracle import memoroid_oracle as mo
    lib = _lib.lib
    bsz, steps, dim = 1024, 4, 512
    assert bsz * dim == lib.mxk_linrec_noalloc_max_elements()
    gen = torch.Generator().manual_seed(7)
    cplx = lambda *s: torch.complex(torch.randn(*s, generator=gen), torch.randn(*s, generator=gen))
    lam = (cplx(dim) * 0.4).cuda()
    bu, gh = cplx(bsz, steps, dim).cuda(), cplx(bsz, steps, dim).cuda()
    done = (torch.rand(bsz, steps, generator=gen) < 0.1).to(torch.uint8).cuda()
    h, _ = ops.linrec_fwd(lam, bu, None, None, done, want_decay=False)
    gb_ref, ga_ref, _ = ops.linrec_bwd(lam, h, None, done, gh, None, need_gh0=False)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        gb, ga = torch.empty_like(h), torch.empty_like(lam)
        st = lib.mxk_linrec_c64_bwd_noalloc(_p(lam), _p(h), None, _p(done), _p(gh), None, _p(gb), _p(ga), None,
                                            bsz, steps, dim, 0, stream)
        assert st == 0, _lib.status_string(st)
        torch.cuda.synchronize()
        assert float((gb - gb_ref).abs().max()) <= 1e-5 * float(gb_ref.abs().max())
        assert float((ga - ga_ref).abs().max()) <= 1e-5 * float(ga_ref.abs().max())
    # fp64 oracle (JAX cotangent convention) on the whole problem: T = 4 keeps it cheap
    lam_l = lam.cpu().to(torch.complex128).requires_grad_()
    bu_l = bu.cpu().to(torch.complex128).requires_grad_()
    h_ref, _ = mo.linrec_seq(lam_l, bu_l, torch.zeros(bsz, dim, dtype=torch.complex128), done.cpu().double())
    (h_ref * gh.cpu().to(torch.complex128)).sum().real.backward()
    ga_o, gb_o = mo.jax_cotangent(lam_l.grad), mo.jax_cotangent(bu_l.grad)
    assert float((ga.cpu() - ga_o).abs().max()) <= 1e-4 * float(ga_o.abs().max())
    assert float((gb.cpu() - gb_o).abs().max()) <= 1e-5 * float(gb_o.abs().max())
    st = lib.mxk_linrec_c64_bwd_noalloc(_p(lam), _p(h), None, _p(done), _p(gh), None, _p(gb), _p(ga), None,
                                        bsz + 1, steps, dim, 0, stream)
    assert st == -6


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    from memorax_b200 import _lib
    lib = _lib.lib
    limit = lib.mxk_linrec_noalloc_max_elements()
    assert limit == 524288
    x = torch.zeros(16, dtype=torch.complex64, device="cuda")
    st = lib.mxk_linrec_c64_bwd_noalloc(_p(x), _p(x), None, None, _p(x), None, _p(x), _p(x), None,
                                        1024, 4, 1024, 0, None)
    assert st == -6 and "scratch" in _lib.status_string(st)
