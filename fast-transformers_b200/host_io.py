"""Steps whose inputs and results live in host memory: copies and kernels of neighbouring steps
overlap.

The causal product on config-sized inputs takes a quarter of a millisecond on the GPU, while
moving its four inputs in and its four results out takes milliseconds over PCIe.  PCIe is
full duplex, so a stream of such steps is fastest when step ``i+1``'s host->device copies,
step ``i``'s kernels and step ``i-1``'s device->host copies run at the same time.  This class
does exactly that with three CUDA streams and two sets of device input buffers; the compute
callback is ordinary package code (for example the autograd ``causal_dot_product``).

The reference has no counterpart: its kernels take device tensors and it leaves transfers to
the caller (``fast_transformers/causal_product/__init__.py:38-64``).
"""
import torch


class HostStepPipeline:
    """``run(host_inputs, host_outputs)`` enqueues one step: copy the pinned ``host_inputs`` to
    the device, call ``compute(*device_inputs)`` (which returns a tuple of device tensors), copy
    the results into the pinned ``host_outputs``.  Nothing blocks the host; call
    :meth:`synchronize` before reading ``host_outputs`` of the last step.  ``host_outputs`` of
    step ``i`` must not be read before step ``i``'s copies have finished, and are overwritten by
    the next step that is given the same buffers."""

    def __init__(self, compute, example_inputs, device=None, depth=2):
        self.compute = compute
        self.device = torch.device(device if device is not None else "cuda")
        self.depth = depth
        self.compute_stream = torch.cuda.current_stream(self.device)
        self.in_stream = torch.cuda.Stream(self.device)
        self.out_stream = torch.cuda.Stream(self.device)
        self.inputs = [[torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs]
                       for _ in range(depth)]
        self.in_ready = [torch.cuda.Event() for _ in range(depth)]
        self.in_free = [torch.cuda.Event() for _ in range(depth)]
        self.step = 0

    def run(self, host_inputs, host_outputs):
        b = self.step % self.depth
        if self.step >= self.depth:
            # the kernels that read this set of device inputs two steps ago have finished
            self.in_stream.wait_event(self.in_free[b])
        with torch.cuda.stream(self.in_stream):
            for d, h in zip(self.inputs[b], host_inputs):
                d.copy_(h, non_blocking=True)
            self.in_ready[b].record(self.in_stream)
        self.compute_stream.wait_event(self.in_ready[b])
        results = self.compute(*self.inputs[b])
        self.in_free[b].record(self.compute_stream)
        done = torch.cuda.Event()
        done.record(self.compute_stream)
        self.out_stream.wait_event(done)
        with torch.cuda.stream(self.out_stream):
            for h, d in zip(host_outputs, results):
                d.record_stream(self.out_stream)
                h.copy_(d, non_blocking=True)
        self.step += 1

    def synchronize(self):
        self.in_stream.synchronize()
        self.compute_stream.synchronize()
        self.out_stream.synchronize()
