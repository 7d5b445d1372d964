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


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    from memorax_b200 import _lib
    lib = _lib.lib
    limit = lib.mxk_linrec_noalloc_max_elements()
    assert limit == 524288
    x = torch.zeros(16, dtype=torch.complex64, device="cuda")
    st = lib.mxk_linrec_c64_bwd_noalloc(_p(x), _p(x), None, None, _p(x), None, _p(x), _p(x), None,
                                        1024, 4, 1024, 0, None)
    assert st == -6 and "scratch" in _lib.status_string(st)
