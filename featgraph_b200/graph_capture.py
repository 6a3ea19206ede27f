"""A fixed sequence of library calls replayed as ONE CUDA graph.

On a small graph (the reference's own test and benchmark sizes: thousands of rows) a call's kernels last a
few microseconds each, and what a training step pays is the launches: up to four kernels per SpMM (hub rows,
long rows, the other rows, short rows, some on side streams with their fork and join events), one or more per
SDDMM, each behind a Python-to-C call.  The calls of a step are the same every iteration - same adjacency,
same buffers, only the buffers' contents change - so they can be recorded once and replayed with one launch.

Every device entry point of the library only enqueues work on the caller's stream (the side streams it uses are
forked from and joined back to that stream by events), allocates nothing and never synchronises, which is what
stream capture needs.  The host-buffer calls (``run_host``) are not for capture: they use pinned staging
and the library's own copy streams across calls.

    step = featgraph_b200.graph_capture.capture(lambda: (spmm.run([x]), sddmm.run([x, y])))
    for it in range(iters):
        x.copy_(...); y.copy_(...)      # new contents, same tensors
        h, scores = step.replay()       # the modules' output tensors, refreshed
"""
import torch


class CapturedCalls:
    """``fn`` is called ``warmup`` times directly (first calls create the library's per-device streams and
    set kernel attributes), then once under stream capture.  ``fn`` must only enqueue device work on the current
    stream - module ``run`` / ``compute`` calls, ``GraphOps`` calls, torch ops on preallocated tensors - and
    must not synchronise or read results back.  ``replay()`` enqueues the recorded work on the current stream
    and returns what ``fn`` returned during capture (the same tensors every time)."""

    def __init__(self, fn, device=None, warmup=2):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(self.device):
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(max(int(warmup), 1)):
                    fn()
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.result = fn()

    def replay(self):
        with torch.cuda.device(self.device):
            self.graph.replay()
        return self.result


def capture(fn, device=None, warmup=2):
    """Record the device work ``fn()`` enqueues into a CUDA graph; see ``CapturedCalls``."""
    return CapturedCalls(fn, device=device, warmup=warmup)
