"""CPU-only checks of the boundary and the host logic: the C-ABI library loads
and exports every symbol the header declares (no compute calls), argument
validation happens before any launch, the benchmark's CPU arm runs, and two
gloo ranks agree on the shard bookkeeping the multi-GPU benchmark uses."""
import json
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from memorax_b200.build import build_library
    build_library()
    from memorax_b200 import _lib
    return _lib


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "mxk.h")).read()
    declared = set(re.findall(r"\b(mxk_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(lib.lib, name), f"{name} declared in mxk.h but not exported"
    assert declared == set(lib.SIGNATURES), declared ^ set(lib.SIGNATURES)


def test_status_strings_and_validation_without_a_gpu(lib):
    assert lib.lib.mxk_abi_version() >= 3
    assert lib.status_string(0) == "ok"
    for code in (-1, -2, -3, -4, -5, -6):
        assert lib.status_string(code) != "unknown mxk status"
    L = lib.lib
    # every entry point rejects bad arguments on the host, before touching CUDA
    assert L.mxk_linrec_f32_fwd(None, 0, None, None, None, None, None, None, 1, 1, 1, None) == -1
    assert L.mxk_linrec_c64_bwd(None, 1, None, None, None, None, None, None, None, None, None, 0, 1, 1, 1, 0, None) == -1
    assert L.mxk_loglinrec_f32_fwd(None, None, None, None, None, None, None, None, 1, 1, 1, None) == -1
    assert L.mxk_linattn_bf16_fwd(*([None] * 11), 1, 1, 1, 64, 1e-6, 1, None) == -1
    assert L.mxk_gdelta_bf16_fwd(*([None] * 11), 0, None, 1, 1, 1, 128, None) == -1
    assert L.mxk_gdelta_bf16_bwd(*([None] * 17), 1, 1, 1, 128, None) == -1
    import ctypes
    buf = (ctypes.c_char * 256)()
    p = ctypes.addressof(buf) & ~15
    assert L.mxk_linattn_bf16_fwd(p, p, p, None, None, None, p, None, None, None, None, 1, 1, 1, 128, 1e-6, 1, None) == -4
    assert L.mxk_linattn_bf16_fwd(p, p, p, None, None, None, p, None, None, None, None, 1, 1, 1, 12, 1e-6, 1, None) == -4
    assert L.mxk_linattn_chunk_states_bytes(2, 65, 3, 32) == 2 * 3 * 2 * 9 * 64 * 16 and L.mxk_linattn_chunk_states_bytes(1, 1, 1, 12) == 0
    assert L.mxk_linattn_bf16_fwd(p, p, p, None, None, None, p, None, None, None, None, 0, 1, 1, 64, 1e-6, 1, None) == -2
    assert L.mxk_gdelta_bf16_fwd(p, p, p, p, p, None, None, p + 2, None, None, p, 1 << 20, None, 1, 1, 1, 128, None) == -3
    assert L.mxk_gdelta_bf16_fwd(p, p, p, p, p, None, None, p, None, None, None, 0, None, 1, 1, 1, 128, None) == -5
    assert L.mxk_gdelta_bf16_fwd(p, p, p, p, p, None, None, p, None, None, p, 16, None, 1, 1, 1, 128, None) == -5
    assert L.mxk_gdelta_workspace_bytes(2, 65, 3, 64) == 2 * 3 * 2 * 8192
    assert L.mxk_linrec_c64_bwd_noalloc(p, p, None, None, p, None, p, p, None, 1 << 12, 1, 1 << 12, 0, None) == -6
    assert L.mxk_linattn_chunk_states_bytes(2, 65, 3, 64) == 2 * 3 * 2 * 9 * 64 * 16
    assert L.mxk_gdelta_chunk_states_bytes(2, 65, 3, 128) == 2 * 3 * 2 * (16 + 8) * 128 * 16
    assert L.mxk_linrec_bwd_workspace_bytes(1, 1, 4, 9, 8) == 4 * 8 * 8
    # the last-state-only recurrences: missing pointers, bad dimensions, misaligned buffers, unsupported group width
    assert L.mxk_linrec_f32_last(None, 0, None, None, None, None, 1, 1, 1, None) == -1
    assert L.mxk_linrec_c64_last(p, 1, p, None, None, p, 0, 1, 1, None) == -2
    assert L.mxk_linrec_c64_last(p, 1, p + 4, None, None, p, 1, 1, 1, None) == -3
    assert L.mxk_linrec_f32_grouped_last(None, None, None, None, None, 1, 1, 128, 1, None) == -1
    assert L.mxk_linrec_f32_grouped_last(p, p, None, None, p, 1, 1, 100, 1, None) == -4


def test_missing_library_fails_loudly(tmp_path):
    code = ("import os; os.environ['MXK_LIBRARY'] = %r\n"
            "try:\n    import memorax_b200._lib\nexcept ImportError as e:\n    print('raised', 'no fallback' in str(e))\n"
            % str(tmp_path / "nope.so"))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert "raised True" in out.stdout, out.stdout + out.stderr


def test_ops_refuse_cpu_tensors(lib):
    import torch
    from memorax_b200 import ops
    with pytest.raises(ValueError):
        ops.linrec_fwd(torch.zeros(2, 3, 4), torch.zeros(2, 3, 4))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--workload", "c1", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port"


def _gloo_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    w = bench.LinRecC1(batch=4)
    x = w.host_inputs(seed_offset=1000 * rank)          # the per-rank seeding of the GPU arm
    h = w.cpu_step(x)
    # ranks own disjoint sequences: different data, same shapes; timing is the max over ranks
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    chk = torch.tensor([float(x["b"].sum())])
    gathered = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(gathered, chk)
    q.put((rank, float(t), [float(g) for g in gathered], tuple(h.shape), w.tokens()))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_independent_sequences():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, 29571, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in res] == [2.0, 2.0]                # max over ranks
    assert res[0][2] == res[1][2] and res[0][2][0] != res[0][2][1]   # disjoint per-rank inputs
    assert res[0][3] == res[1][3] == (4, 128, 256) and res[0][4] * 2 == 2 * 4 * 128


def _bucket_worker(rank, world, port, q):
    """One rank of the gradient all-reduce test: the trainer's bucketing and hooks on a CPU model over gloo."""
    import torch
    import torch.distributed as dist
    from torch import nn
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from memorax_b200 import blocks

    class Net(nn.Module):                       # three top-level blocks -> three buckets
        def __init__(self):
            super().__init__()
            self.embed, self.mid, self.head = nn.Linear(6, 16), nn.Linear(16, 16), nn.Linear(16, 1)

        def forward(self, obs, done):
            return self.head(torch.tanh(self.mid(torch.tanh(self.embed(obs))))).squeeze(-1)

    torch.manual_seed(0)                        # same parameters on both ranks
    model = Net().to(torch.bfloat16)
    calls = []
    blocks.ops.adam_step = lambda flat, grad, m, v, step, *a, **k: calls.append(grad.clone())   # no device kernel on CPU
    trainer = blocks.FlatAdamTrainer(model, world_size=world)
    g = torch.Generator().manual_seed(10 + rank)     # different data per rank
    obs = torch.randn(4, 5, 6, generator=g).bfloat16()
    target = torch.randn(4, 5, generator=g)
    trainer.step(obs, None, target)
    reduced = calls[0].float()
    # what the sum over ranks must be: each rank's local gradient, gathered and added
    model.zero_grad()
    trainer.flat_grad.zero_()
    (0.5 * (model(obs, None).float() - target).square().mean()).backward()   # hooks fire again; ignore their handles
    for hdl in trainer._handles:
        hdl.wait()
    q.put((rank, [tuple(b) for b in trainer.buckets], len(calls), reduced.tolist()))
    dist.destroy_process_group()


def test_gradient_buckets_are_reduced_under_backward_on_two_gloo_ranks():
    """The c5 trainer cuts the flat gradient into one bucket per top-level block and launches each bucket's
    all-reduce from a gradient hook; two gloo ranks with different data must end up with the same, summed
    gradient, every bucket reduced exactly once and the buckets tiling the buffer."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_bucket_worker, args=(r, 2, 29581, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    (_, buckets0, ncalls0, grad0), (_, buckets1, ncalls1, grad1) = res
    assert buckets0 == buckets1 and len(buckets0) == 3 and ncalls0 == ncalls1 == 1
    assert buckets0[0][0] == 0 and all(a[1] == b[0] for a, b in zip(buckets0, buckets0[1:]))
    assert sum(n for _, _, n in buckets0) == 6           # 3 x (weight, bias)
    assert grad0 == grad1 and any(abs(x) > 0 for x in grad0)   # identical after the all-reduce, and not all zero
