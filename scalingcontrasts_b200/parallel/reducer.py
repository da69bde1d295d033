"""``GradientReducer``: sums parameter gradients across the box with the multimem all-reduce, overlapped with backward.

Parameters are packed into buckets that live in the domain's symmetric heap. A post-accumulate hook copies each fresh
gradient into its slot of the bucket and re-points ``param.grad`` at that slot (the optimizer then reads the reduced
values in place); when a bucket's last gradient has arrived, the bucket's all-reduce is launched on a side stream while
autograd keeps running the rest of backward on the main stream. The scale (1 for the sum this loss needs, 1/world for an
average) and the bfloat16 <-> float32 handling are folded into the collective kernel: bfloat16 payloads are reduced in
float32 inside the switch and stored back as bfloat16.

The reducer uses its own control channel of the domain, so its rounds never mix with the loss step's barrier and
summands all-reduce that run on the main stream at the same time.

The reference has no gradient exchange for parameters (it has no model); its all-reduce moves only four floats per step
(scalingcontrasts.cu:309). This class is what puts its collective kernels to work in a training loop.
"""
from __future__ import annotations

from typing import Iterable, List

import torch

REDUCER_CHANNEL = 1


class _Bucket:
    def __init__(self, dtype: torch.dtype) -> None:
        self.dtype = dtype
        self.parameters: List[torch.nn.Parameter] = []
        self.views: List[torch.Tensor] = []
        self.offset = 0
        self.scalars = 0
        self.pending = 0
        self.done = torch.cuda.Event()
        self.launched = False


class GradientReducer:
    def __init__(self, parameters: Iterable[torch.nn.Parameter], domain, bucket_bytes: int = 32 << 20, scale: float = 1.0) -> None:
        self.domain, self.scale = domain, float(scale)
        self.enabled = domain is not None and getattr(domain, "members", 1) > 1 and hasattr(domain, "alloc")
        self.buckets: List[_Bucket] = []
        self._by_parameter = {}  # id(parameter) -> (bucket, view)
        self._handles = []
        if not self.enabled:
            return
        self.stream = torch.cuda.Stream(device=domain.device)
        self._ready = torch.cuda.Event()
        ordered = [p for p in parameters if p.requires_grad]
        ordered.reverse()  # gradients arrive roughly in reverse registration order
        for parameter in ordered:
            if parameter.dtype not in (torch.bfloat16, torch.float32):
                raise ValueError("the reducer handles bfloat16 and float32 parameters")
            size = parameter.numel() * parameter.element_size()
            bucket = self.buckets[-1] if self.buckets else None
            if bucket is None or bucket.dtype != parameter.dtype or (bucket.scalars * parameter.element_size() + size > bucket_bytes
                                                                   and bucket.parameters):
                bucket = _Bucket(parameter.dtype)
                self.buckets.append(bucket)
            bucket.parameters.append(parameter)
            per_vector = 16 // parameter.element_size()
            bucket.scalars += -(-parameter.numel() // per_vector) * per_vector
        for bucket in self.buckets:
            element = 2 if bucket.dtype == torch.bfloat16 else 4
            bucket.offset = domain.alloc(bucket.scalars * element)
            cursor = bucket.offset
            per_vector = 16 // element
            for parameter in bucket.parameters:
                view = domain.tensor(cursor, tuple(parameter.shape), parameter.dtype)
                bucket.views.append(view)
                cursor += -(-parameter.numel() // per_vector) * per_vector * element
                self._by_parameter[id(parameter)] = (bucket, view)
                self._handles.append(parameter.register_post_accumulate_grad_hook(self._on_gradient))
            domain.tensor(bucket.offset, (bucket.scalars,), bucket.dtype).zero_()
            bucket.pending = len(bucket.parameters)

    @staticmethod
    def heap_bytes(parameters: Iterable[torch.nn.Parameter]) -> int:
        """Symmetric heap the reducer takes for these parameters (with room for alignment)."""
        total = 0
        for parameter in parameters:
            if parameter.requires_grad:
                total += -(-parameter.numel() * parameter.element_size() // 16) * 16 + 256
        return total + 4096

    def landing_buffers(self, module: torch.nn.Module) -> dict:
        """Parameter name -> this reducer's bucket slot for it. A backward pass that writes a gradient straight into its
        slot (and hands autograd an alias of it) saves the copy the hook would otherwise make."""
        if not self.enabled:
            return {}
        return {name: self._by_parameter[id(parameter)][1] for name, parameter in module.named_parameters()
                if id(parameter) in self._by_parameter}

    def _on_gradient(self, parameter: torch.nn.Parameter) -> None:
        bucket, view = self._by_parameter[id(parameter)]
        if parameter.grad.data_ptr() != view.data_ptr():
            view.copy_(parameter.grad)
            parameter.grad = view
        bucket.pending -= 1
        if bucket.pending == 0:
            self._launch(bucket)

    def _launch(self, bucket: _Bucket) -> None:
        self._ready.record()
        self.stream.wait_event(self._ready)
        self.domain.all_reduce(bucket.scalars, self.stream, offset=bucket.offset, dtype=bucket.dtype, scale=self.scale,
                               channel=REDUCER_CHANNEL)
        bucket.done.record(self.stream)
        bucket.launched = True

    def wait(self) -> None:
        """Makes the current stream wait for every bucket's all-reduce and re-arms the buckets for the next backward."""
        if not self.enabled:
            return
        current = torch.cuda.current_stream()
        for bucket in self.buckets:
            if bucket.pending == 0 and not bucket.launched:
                self._launch(bucket)
            if bucket.launched:
                current.wait_event(bucket.done)
            bucket.pending = len(bucket.parameters)
            bucket.launched = False

    def launches_per_step(self) -> int:
        return len(self.buckets) if self.enabled else 0

    def remove(self) -> None:
        for handle in self._handles:
            handle.remove()
        self._handles = []
