"""CUDA-graph capture of a sequence of library calls.

A quantized network at a small batch is bound by launches, not by the GPU: a
ResNet-18 forward is about 130 kernels, each entered through one C-ABI call.
`Captured` records those calls once into a CUDA graph (torch.cuda.CUDAGraph:
torch provides the capture stream and keeps the buffers of the captured call
at fixed addresses) and replays them with one launch. Everything the library
does inside a call is stream-ordered (kernels, cudaMemsetAsync, the scratch
it takes from the stream-ordered pool), so a call can be captured as it is;
the one-time set-up of a kernel (attributes, the device status word) happens
in the warm-up calls before the capture.
"""
import torch


class Captured:
    """`fn(*inputs)` captured as a CUDA graph.

    inputs are copied into static tensors before every replay; the returned
    tensor is the graph's static output (valid until the next replay)."""

    def __init__(self, fn, *example_inputs, warmup=2):
        self.static_inputs = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_output = fn(*self.static_inputs)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        self.graph.replay()
        return self.static_output
