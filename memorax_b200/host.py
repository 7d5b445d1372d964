"""Host-buffer entry to the ops: pinned host tensors in, pinned host tensors out.

A caller that keeps its batch in host memory (the reference's CPU-environment
setups do: docs/source/guides/sharp_bits.md:3-9) pays PCIe both ways.  Every op
here is independent per sequence, so the batch is cut into slices that flow
through three streams -- host-to-device copy, kernels, device-to-host copy --
and the two copy directions and the kernels overlap.

With ``graph=True`` the whole three-stream schedule of one call is captured into a
CUDA graph the first time a given set of host buffers is seen and replayed
afterwards, so that a step costs one launch on the host however many slices it has
(the usual pattern: the caller refills the same pinned staging buffers every step).

With ``overlap_calls=N`` (eager mode) consecutive calls stream: the copy-in of call
i+1 no longer waits for the copy-out of call i (host inputs have no producer on the
device), so both copy engines stay busy across calls; at most N calls are in flight on the device and the
host blocks once it is two calls further ahead (its lead, and with it the device memory held by calls not yet
copied out, stays bounded).
The caller then must not rewrite a host input buffer before ``inputs_consumed`` (an
event recorded after the last copy-in of the latest call) has completed."""
from __future__ import annotations

import torch


class HostPipeline:
    """``run(host_inputs, host_outputs)`` applies ``step`` (a function from a dict
    of device tensors to a tuple of device tensors) slice by slice.

    Tensors whose leading dimension equals ``batch`` are sliced; anything else is
    copied whole with the first slice.  ``slices=1`` degenerates to copy, run,
    copy on one stream each (for steps that are not separable over the batch).

    In the eager modes the device copies of the inputs live in staging buffers owned by the pipeline (one set per
    call that may be in flight) and a call's device outputs are kept until its copy-out has completed, so nothing
    is allocated per call for the inputs and the allocator tracks no cross-stream uses.  The device tensors that
    ``run`` returns are therefore only valid until ``overlap_calls`` further calls have been issued.

    ``graph=True``: ``step`` must then be capturable (no host synchronisation, no
    data-dependent host control flow) and the host tensors must stay alive and in
    place for as long as the pipeline is used with them."""

    def __init__(self, step, batch, device, slices=4, graph=False, overlap_calls=1):
        if graph and overlap_calls > 1:
            raise ValueError("overlap_calls applies to the eager mode: replayed graphs run back to back")
        self.step, self.batch, self.device = step, batch, device
        self.slices = max(1, min(slices, batch))
        self.graph = graph
        self.overlap_calls = max(1, int(overlap_calls))
        self._finished = []          # completion events of the calls still in flight, oldest first
        self._pending = []           # (copy-out event, device outputs) of slices whose copy-out may still be running
        self._issued = []            # completion events of the calls the host has issued and not yet waited for
        self._in_bufs = {}           # staging set -> {input name: device buffer}
        self._calls = 0
        self.inputs_consumed = None
        self._graphs = {}
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.s_capture = torch.cuda.Stream(device=device) if graph else None

    def _bounds(self, i):
        per = -(-self.batch // self.slices)
        return i * per, min(self.batch, (i + 1) * per)

    def run(self, host_inputs, host_outputs):
        if not self.graph:
            return self._enqueue(host_inputs, host_outputs, capturing=False)
        key = (tuple((n, t.data_ptr(), tuple(t.shape), t.dtype) for n, t in host_inputs.items()),
               tuple((t.data_ptr(), tuple(t.shape), t.dtype) for t in host_outputs))
        entry = self._graphs.get(key)
        if entry is None:
            # once eagerly (lazy initialisation, allocator warm-up), then capture
            self._enqueue(host_inputs, host_outputs, capturing=False)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.s_capture):
                keep = self._enqueue(host_inputs, host_outputs, capturing=True)
            entry = self._graphs[key] = (g, keep, host_inputs, host_outputs)
        entry[0].replay()
        return entry[1]

    def _staging(self, slot, host_inputs):
        """Device copies of the inputs live in staging buffers that belong to the pipeline (one set per call that
        may be in flight), so that a call allocates nothing for them and the allocator never has to track
        cross-stream uses; they are (re)allocated when a call brings tensors of another shape."""
        bufs = self._in_bufs.setdefault(slot, {})
        fresh = False
        for name, t in host_inputs.items():
            b = bufs.get(name)
            if b is None or b.shape != t.shape or b.dtype != t.dtype:
                if b is not None:   # still in use by earlier calls on the copy and kernel streams
                    b.record_stream(self.s_in)
                    b.record_stream(self.s_run)
                bufs[name] = torch.empty(t.shape, dtype=t.dtype, device=self.device)
                fresh = True
        if fresh:   # the new blocks' earlier life on the caller's stream comes first
            born = torch.cuda.Event()
            born.record(torch.cuda.current_stream(self.device))
            self.s_in.wait_event(born)
        return bufs

    def _release_finished(self):
        """Drops the device tensors of calls whose copy-out has completed (they are kept until then instead of
        being handed to the allocator with cross-stream use records, which makes every later allocation poll events)."""
        while self._pending and self._pending[0][0].query():
            self._pending.pop(0)

    def _enqueue(self, host_inputs, host_outputs, capturing):
        main = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(main)
        streaming = self.overlap_calls > 1 and not capturing
        # kernels and copy-out always follow the caller's stream (weights or other device state the step
        # reads); the copy-in does too unless calls may overlap, in which case it only waits for the call
        # `overlap_calls` back, which bounds the device buffers in flight
        for s in ((self.s_run, self.s_out) if streaming else (self.s_in, self.s_run, self.s_out)):
            s.wait_event(start)
        if streaming and len(self._finished) >= self.overlap_calls:
            self.s_in.wait_event(self._finished[-self.overlap_calls])
            del self._finished[:-self.overlap_calls]
        if streaming and len(self._issued) > self.overlap_calls + 2:
            # the host stays at most two calls ahead of what the device may have in flight: an unbounded lead would
            # keep every call's device outputs alive at once (the allocator then grows by a cudaMalloc per tensor
            # and call) without making anything faster
            self._issued.pop(0).synchronize()
        staged = None
        if not capturing:
            self._release_finished()
            # staging set i % overlap_calls: its previous user is the call the copy-in has just been made to wait for
            staged = self._staging(self._calls % self.overlap_calls, host_inputs)
            self._calls += 1
        keep = []
        shared = {}
        for i in range(self.slices):
            lo, hi = self._bounds(i)
            if lo >= hi:
                break
            with torch.cuda.stream(self.s_in):
                x = {}
                for name, t in host_inputs.items():
                    sliced = t.dim() > 0 and t.shape[0] == self.batch
                    if capturing:   # a captured schedule owns its tensors (the graph's pool; kept alive in `keep`)
                        if sliced:
                            x[name] = t[lo:hi].to(self.device, non_blocking=True)
                        else:
                            if name not in shared:
                                shared[name] = t.to(self.device, non_blocking=True)
                            x[name] = shared[name]
                    elif sliced:
                        x[name] = staged[name][lo:hi]
                        x[name].copy_(t[lo:hi], non_blocking=True)
                    else:
                        if name not in shared:
                            shared[name] = staged[name]
                            shared[name].copy_(t, non_blocking=True)
                        x[name] = shared[name]
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            self.s_run.wait_event(ready)
            with torch.cuda.stream(self.s_run):
                outs = self.step(x)
                done = torch.cuda.Event()
                done.record(self.s_run)
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                for dst, src in zip(host_outputs, outs):
                    if dst.dim() > 0 and dst.shape[0] == self.batch and src.shape[0] == hi - lo:
                        dst[lo:hi].copy_(src, non_blocking=True)
                    else:
                        dst.copy_(src, non_blocking=True)
                if not capturing:   # this slice's device outputs go back to the allocator once they have been copied out
                    copied = torch.cuda.Event()
                    copied.record(self.s_out)
                    self._pending.append((copied, outs))
            keep.append((x, outs))
        finished = torch.cuda.Event()
        finished.record(self.s_out)
        if streaming:
            # the caller's stream is NOT made to wait here (that would serialise the next call's kernels
            # behind this call's copy-out); call wait() before reading the host outputs
            self._finished.append(finished)
            self._issued.append(finished)
            self.inputs_consumed = ready
        else:
            main.wait_event(finished)
        return keep

    def join(self):
        """Makes the caller's current stream wait (on the device) for every call issued so far."""
        main = torch.cuda.current_stream(self.device)
        for ev in self._finished:
            main.wait_event(ev)

    def wait(self):
        """Blocks the host until every call issued so far has delivered its host outputs."""
        for ev in self._finished:
            ev.synchronize()
        self._finished.clear()
        self._issued.clear()
        torch.cuda.current_stream(self.device).synchronize()
        self._release_finished()
