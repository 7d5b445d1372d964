"""Independent pin of the gated delta rule: the CUDA kernels against the
`flash-linear-attention` package (fla 0.5.1, Triton) used as a black box.

The reference has no delta-rule cell, so no reference vectors exist for this
op; the fp64 oracle follows the published recurrence, and this test checks the
same kernels against a second, unrelated implementation of that recurrence.
Nothing of fla is copied or shipped: it is imported here only.

Conventions bridged in this file:
  * fla's gate `g` is log(alpha); its state is (d_k, d_v), ours (d_v, d_k);
    its default query scale 1/sqrt(d_k) is switched off (scale = 1).
  * Episode resets: fla has none.  A sequence is cut at every done step and
    the pieces are passed as one packed variable-length batch (`cu_seqlens`);
    a piece that starts at a done step starts from a zero state, a piece that
    starts a row without done[b, 0] starts from that row's carried state.
If Triton cannot run on the box the test is skipped with the captured reason.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _fla():
    try:
        from fla.ops.gated_delta_rule import chunk_gated_delta_rule
        return chunk_gated_delta_rule
    except Exception as exc:   # missing package or Triton import failure
        pytest.skip(f"fla unavailable: {type(exc).__name__}: {exc}")


def _segments(done):
    """Start offsets (in the packed (B*T) axis) of the pieces and, per piece, the batch row it
    continues from its carried state (-1 = fresh state)."""
    bsz, steps = done.shape
    starts, carry_row = [], []
    for b in range(bsz):
        for t in range(steps):
            if t == 0 or done[b, t]:
                starts.append(b * steps + t)
                carry_row.append(b if (t == 0 and not done[b, 0]) else -1)
    return starts + [bsz * steps], carry_row


@pytest.mark.parametrize("shape,p_done,zero_state", [((2, 256, 2), 0.0, True), ((3, 192, 2), 0.02, False),
                                                     ((2, 512, 4), 0.005, True)])
def test_gdelta_matches_fla(shape, p_done, zero_state):
    chunk_gated_delta_rule = _fla()
    from memorax_b200 import ops
    bsz, steps, heads = shape
    dim = 128
    gen = torch.Generator().manual_seed(1000 + steps)
    mk = lambda *s: torch.randn(*s, generator=gen)
    nrm = lambda x: x / x.norm(dim=-1, keepdim=True)
    q, k = nrm(mk(bsz, steps, heads, dim)).bfloat16().cuda(), nrm(mk(bsz, steps, heads, dim)).bfloat16().cuda()
    v, d_o = mk(bsz, steps, heads, dim).bfloat16().cuda(), mk(bsz, steps, heads, dim).bfloat16().cuda()
    beta = torch.sigmoid(mk(bsz, steps, heads)).cuda()
    alpha = torch.exp(-torch.nn.functional.softplus(mk(bsz, steps, heads))).cuda()
    s0 = (torch.zeros(bsz, heads, dim, dim) if zero_state else mk(bsz, heads, dim, dim) * 0.3).cuda()
    done = torch.rand(bsz, steps, generator=gen) < p_done
    if p_done > 0:
        done[0, 0] = True
        done[-1, 70:72] = True

    # ---- this library
    o, s_last, states = ops.gdelta_fwd(q, k, v, alpha, beta, s0, done.cuda(), save_states=True, check=True)
    dq, dk, dv, dalpha, dbeta, ds0 = ops.gdelta_bwd(q, k, v, alpha, beta, d_o, states, done.cuda(), None, check=True)

    # ---- fla on the packed pieces
    cu, carry_row = _segments(done)
    pack = lambda x: x.reshape(1, bsz * steps, *x.shape[2:]).detach().clone().requires_grad_()
    fq, fk, fv, fb = pack(q), pack(k), pack(v), pack(beta)
    fg = pack(torch.log(alpha))
    h0 = torch.zeros(len(carry_row), heads, dim, dim, device="cuda")
    s0_leaf = s0.clone().requires_grad_()
    rows = [r for r in carry_row if r >= 0]
    if rows:
        idx = torch.tensor([i for i, r in enumerate(carry_row) if r >= 0], device="cuda")
        h0 = h0.index_put((idx,), s0_leaf[torch.tensor(rows, device="cuda")].transpose(-1, -2))
    try:
        fo, fh = chunk_gated_delta_rule(fq, fk, fv, fg, fb, scale=1.0, initial_state=h0, output_final_state=True,
                                        cu_seqlens=torch.tensor(cu, dtype=torch.long, device="cuda"))
        (fo.float() * pack(d_o).detach().float()).sum().backward()
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"fla could not run on this box: {type(exc).__name__}: {str(exc)[:200]}")
    # the final state of a row is the final state of its last piece
    last_piece = [max(i for i, st in enumerate(cu[:-1]) if st < (b + 1) * steps) for b in range(bsz)]
    f_last = fh[torch.tensor(last_piece, device="cuda")].transpose(-1, -2)

    unpack = lambda x: x.reshape(bsz, steps, *x.shape[2:])
    f_dalpha = unpack(fg.grad) / alpha
    f_dalpha = torch.where(done.cuda()[:, :, None], torch.zeros_like(f_dalpha), f_dalpha)
    pairs = [("o", o, unpack(fo)), ("s_last", s_last, f_last), ("dq", dq, unpack(fq.grad)), ("dk", dk, unpack(fk.grad)),
             ("dv", dv, unpack(fv.grad)), ("dalpha", dalpha, f_dalpha), ("dbeta", dbeta, unpack(fb.grad))]
    if not zero_state:
        pairs.append(("ds0", ds0, s0_leaf.grad))
    for name, got, ref in pairs:
        ref = ref.detach().float()
        scale = max(1.0, float(ref.abs().max()))
        err = float((got.float() - ref).abs().max())
        # both sides round to bf16 internally: 2e-2 of the tensor's scale covers either one against fp64
        assert err <= 4e-2 * scale, f"{name}: {err:.4f} vs scale {scale:.3f}"
