"""Attention for host-resident Q, K, V: head groups streamed through the GPU.

Heads are independent on this path (Q/K are quantised per 128 tokens per head, V per head), so a caller
whose tensors live in pinned host memory does not have to wait for all of Q, K, V to arrive before the
first kernel starts: ``attention_host`` copies group g+1 in while group g is computed and group g-1 is
copied out, on a copy-in, a copy-out and two compute streams with two device buffers per tensor (the kernels
of consecutive groups overlap at their ragged last waves; the first group is one head).  The result equals
``attention(q.cuda(), k.cuda(), v.cuda())`` bit for bit.  The reference has no such helper (its callers keep
tensors on the device); the copies are ``ovc_copy_head_slice`` of libovc.so.
"""

import torch

from . import _lib, api


def _copy(lib, dst, dst_first, src, src_first, heads, to_device, stream):
    length, dst_heads = dst.shape[0], dst.shape[1]
    bytes_per_head = dst.shape[2] * dst.element_size()
    _lib.check(
        lib.ovc_copy_head_slice(dst.data_ptr(), dst_heads, dst_first, src.data_ptr(), src.shape[1], src_first, heads,
                                length, bytes_per_head, 1 if to_device else 0, stream.cuda_stream),
        "ovc_copy_head_slice",
    )


class HostAttention:
    """Reusable streams and device buffers for ``attention_host`` calls of one shape."""

    def __init__(self, length, heads, dtype, device, heads_per_group=4):
        if heads_per_group < 1:
            raise ValueError("heads_per_group must be positive")
        self.length, self.heads, self.dtype = length, heads, dtype
        self.device = torch.device(device)
        self.group = min(heads_per_group, heads)
        with torch.cuda.device(self.device):
            self.copy_in, self.copy_out = torch.cuda.Stream(), torch.cuda.Stream()
            # One compute stream per buffer slot: the kernels of consecutive groups may overlap, so that the next
            # group's CTAs fill the SMs that the previous group's last, partial wave leaves idle.
            self.compute = [torch.cuda.Stream(), torch.cuda.Stream()]
            shape = (length, self.group, 128)
            self.inputs = [[torch.empty(shape, dtype=dtype, device=self.device) for _ in range(3)] for _ in range(2)]
            self.landed = [torch.cuda.Event() for _ in range(2)]
            self.consumed = [torch.cuda.Event() for _ in range(2)]
            self.results = [None, None]
            self.stored = [torch.cuda.Event() for _ in range(2)]

    def __call__(self, q, k, v, out=None, **attention_options):
        for t in (q, k, v):
            if t.is_cuda or t.dtype != self.dtype or tuple(t.shape) != (self.length, self.heads, 128) or not t.is_contiguous():
                raise ValueError("attention_host expects contiguous host tensors [S,H,128] of the prepared shape and dtype")
            if not t.is_pinned():
                raise ValueError("attention_host expects pinned host memory (tensor.pin_memory())")
        if out is None:
            out = torch.empty((self.length, self.heads, 128), dtype=torch.bfloat16, pin_memory=True)
        elif out.is_cuda or not out.is_pinned() or out.dtype != torch.bfloat16 or tuple(out.shape) != tuple(q.shape) or not out.is_contiguous():
            raise ValueError("out must be a contiguous pinned bfloat16 host tensor of Q's shape")
        lib = _lib.load()
        caller = torch.cuda.current_stream(self.device)
        # Head groups in order.  The first group is a single head, so that the first kernel starts after one
        # head's copies instead of a whole group's (nothing overlaps that first copy); a remainder comes last.
        lead = 1 if self.group > 1 and self.heads > self.group else 0
        starts = ([0] if lead else []) + list(range(lead, self.heads, self.group))
        with torch.cuda.device(self.device):
            for stream in (self.copy_in, self.copy_out, *self.compute):
                stream.wait_stream(caller)
            for index, first in enumerate(starts):
                slot = index & 1
                count = 1 if (lead and index == 0) else min(self.group, self.heads - first)
                if index >= 2:
                    self.copy_in.wait_event(self.consumed[slot])  # the group that used this buffer has been computed
                for buffer, source in zip(self.inputs[slot], (q, k, v)):
                    # a last, smaller group goes into the leading heads of the buffer
                    _copy(lib, buffer, 0, source, first, count, True, self.copy_in)
                self.landed[slot].record(self.copy_in)
                compute = self.compute[slot]
                compute.wait_event(self.landed[slot])
                if index >= 2:
                    compute.wait_event(self.stored[slot])  # the result that lived in this slot has left
                with torch.cuda.stream(compute):
                    if count == self.group:
                        args = self.inputs[slot]
                    else:
                        args = [buffer[:, :count].contiguous() for buffer in self.inputs[slot]]
                    self.results[slot] = api.attention(*args, **attention_options)
                self.consumed[slot].record(compute)
                self.copy_out.wait_event(self.consumed[slot])
                _copy(lib, out, first, self.results[slot], 0, count, False, self.copy_out)
                self.stored[slot].record(self.copy_out)
            caller.wait_stream(self.copy_out)
            for compute in self.compute:
                caller.wait_stream(compute)
            caller.wait_stream(self.copy_in)
        return out


def attention_host(q, k, v, out=None, *, device="cuda", heads_per_group=4, **attention_options):
    """BF16/FP16 pinned host tensors [S,H,128] in, pinned BF16 host tensor out; work is ordered on the current
    stream of ``device`` (synchronise it before reading ``out``).  Keyword options are those of ``attention``."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    runner = HostAttention(q.shape[0], q.shape[1], q.dtype, device, heads_per_group)
    return runner(q, k, v, out, **attention_options)
