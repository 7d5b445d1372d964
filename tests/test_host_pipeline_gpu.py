"""The pinned-host entry (copy-in, kernels, copy-out overlapped slice by slice)
returns exactly what a single device-side call returns."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_direct_call():
    from memorax_b200 import ops
    from memorax_b200.host import HostPipeline
    g = torch.Generator().manual_seed(0)
    B, T, H, D = 10, 96, 2, 64
    mk = lambda *s: torch.randn(*s, generator=g)
    host = dict(q=(mk(B, T, H, D) / 8).bfloat16(), k=(mk(B, T, H, D) / 8).bfloat16(), v=(mk(B, T, H, D) / 8).bfloat16(),
                s0=mk(B, H, D, D) * 0.1, z0=mk(B, H, D).abs() * 0.1, done=(torch.rand(B, T, generator=g) < 0.03).to(torch.uint8))
    host = {k: v.pin_memory() for k, v in host.items()}

    def step(x):
        o, s_last, z_last, _ = ops.linattn_fwd(x["q"], x["k"], x["v"], x["s0"], x["z0"], x["done"])
        return o, s_last, z_last

    ref = step({k: v.cuda() for k, v in host.items()})
    outs = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in ref]
    for slices in (1, 3, 4):
        for o in outs:
            o.zero_()
        HostPipeline(step, B, torch.device("cuda", 0), slices=slices).run(host, outs)
        torch.cuda.synchronize()
        for got, want in zip(outs, ref):
            assert torch.equal(got, want.cpu()), slices


def test_host_pipeline_graph_replay_tracks_buffer_contents():
    """graph=True captures the schedule once; later calls replay it and must see the
    host buffers' CURRENT contents."""
    from memorax_b200 import ops
    from memorax_b200.host import HostPipeline
    g = torch.Generator().manual_seed(1)
    B, T, H, D = 12, 130, 2, 128
    mk = lambda *s: torch.randn(*s, generator=g)
    nrm = lambda x: x / x.norm(dim=-1, keepdim=True)

    def fresh():
        return dict(q=nrm(mk(B, T, H, D)).bfloat16(), k=nrm(mk(B, T, H, D)).bfloat16(), v=mk(B, T, H, D).bfloat16(),
                    alpha=torch.sigmoid(mk(B, T, H) + 2), beta=torch.sigmoid(mk(B, T, H)),
                    done=(torch.rand(B, T, generator=g) < 0.02).to(torch.uint8))

    def step(x):
        o, s_last, _ = ops.gdelta_fwd(x["q"], x["k"], x["v"], x["alpha"], x["beta"], None, x["done"])
        return o, s_last

    host = {k: v.pin_memory() for k, v in fresh().items()}
    ref = step({k: v.cuda() for k, v in host.items()})
    outs = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in ref]
    pipe = HostPipeline(step, B, torch.device("cuda", 0), slices=3, graph=True)
    for trial in range(3):
        if trial:
            for k, v in fresh().items():
                host[k].copy_(v)          # same pinned buffers, new contents
            ref = step({k: v.cuda() for k, v in host.items()})
        for o in outs:
            o.zero_()
        pipe.run(host, outs)
        torch.cuda.synchronize()
        for got, want in zip(outs, ref):
            assert torch.equal(got, want.cpu()), trial
    assert len(pipe._graphs) == 1


def test_host_pipeline_overlapping_calls():
    """overlap_calls=2: calls stream (copy-in of call i+1 under the copy-out of call i); every call must
    still deliver exactly the single-call results into its own output buffers."""
    from memorax_b200 import ops
    from memorax_b200.host import HostPipeline
    g = torch.Generator().manual_seed(2)
    B, T, H, D = 9, 200, 2, 64
    mk = lambda *s: torch.randn(*s, generator=g)

    def fresh():
        d = dict(q=(mk(B, T, H, D) / 8).bfloat16(), k=(mk(B, T, H, D) / 8).bfloat16(), v=(mk(B, T, H, D) / 8).bfloat16(),
                 s0=mk(B, H, D, D) * 0.1, z0=mk(B, H, D).abs() * 0.1, done=(torch.rand(B, T, generator=g) < 0.02).to(torch.uint8))
        return {k: v.pin_memory() for k, v in d.items()}

    def step(x):
        o, s_last, z_last, _ = ops.linattn_fwd(x["q"], x["k"], x["v"], x["s0"], x["z0"], x["done"])
        return o, s_last, z_last

    calls = [fresh() for _ in range(5)]
    refs = [step({k: v.cuda() for k, v in c.items()}) for c in calls]
    outs = [[torch.zeros(r.shape, dtype=r.dtype).pin_memory() for r in ref] for ref in refs]
    pipe = HostPipeline(step, B, torch.device("cuda", 0), slices=3, overlap_calls=2)
    for c, o in zip(calls, outs):
        pipe.run(c, o)
    pipe.wait()
    for i, (ref, out) in enumerate(zip(refs, outs)):
        for got, want in zip(out, ref):
            assert torch.equal(got, want.cpu()), i
    assert pipe.inputs_consumed is not None and pipe.inputs_consumed.query()


def test_host_pipeline_restages_on_new_shapes_and_copies_unsliced_inputs_whole():
    """The pipeline owns the device copies of its inputs: a later call with other shapes gets new staging buffers,
    and an input whose leading dimension is not the batch (here the time-invariant decay) is copied whole once."""
    from memorax_b200 import ops
    from memorax_b200.host import HostPipeline
    g = torch.Generator().manual_seed(3)
    B, D = 8, 96

    def make(T):
        d = dict(lam=(torch.rand(D, generator=g) * 0.9).to(torch.complex64),
                 bu=torch.complex(torch.randn(B, T, D, generator=g), torch.randn(B, T, D, generator=g)),
                 done=(torch.rand(B, T, generator=g) < 0.05).to(torch.uint8))
        return {k: v.pin_memory() for k, v in d.items()}

    def step(x):
        h, _ = ops.linrec_fwd(x["lam"], x["bu"], None, None, x["done"], want_decay=False)
        return (h,)

    for overlap in (1, 2):
        pipe = HostPipeline(step, B, torch.device("cuda", 0), slices=2, overlap_calls=overlap)
        calls = [make(T) for T in (40, 40, 72, 40)]
        refs = [step({k: v.cuda() for k, v in c.items()})[0].cpu() for c in calls]
        outs = [[torch.zeros(r.shape, dtype=r.dtype).pin_memory()] for r in refs]
        for c, o in zip(calls, outs):
            pipe.run(c, o)
        pipe.wait()
        for i, (ref, out) in enumerate(zip(refs, outs)):
            assert torch.equal(out[0], ref), (overlap, i)
