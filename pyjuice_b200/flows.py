"""One contiguous arena for every parameter-flow accumulator of a circuit.

Data-parallel EM sums the parameter flows of all ranks once per update (PyJuice:
``TensorCircuit.sync_param_flows``, model/tensorcircuit.py:1420-1471, one ``all_reduce`` per flow tensor plus one
for the scalar ``_cum_flow``).  Here the sum-layer flows, every input layer's flows and the running flow total live
in ONE fp32 buffer, so the synchronisation is a single NCCL all-reduce over NVLink with no host round trip:

    [ header: cum_flow split as (hi, lo) | sum-layer flows | input layer 0 flows | input layer 1 flows | ... ]

Segments start on 256-byte boundaries.  ``reduce_len`` lets the caller leave a tail out of the collective — the
replica accumulators of tied input vectors, once they have been folded into their source range.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

_ALIGN = 64            # floats (256 bytes)
_SPLIT = 4096.0        # cum_flow = hi * _SPLIT + lo keeps integers exact in fp32 up to 2^36


def _round_up(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


class _CastBack:
    """Work handle of a reduced-precision all-reduce: ``wait()`` orders the current stream after the collective and
    copies the result back into the fp32 arena."""

    def __init__(self, works, dst, low):
        self.works, self.dst, self.low = works, dst, low

    def wait(self):
        for w in self.works:
            w.wait()
        self.dst.copy_(self.low)


class _Works:
    """Several collectives waited for as one."""

    def __init__(self, works):
        self.works = works

    def wait(self):
        for w in self.works:
            w.wait()


def all_reduce_async(t: torch.Tensor, group=None, dtype: Optional[torch.dtype] = None):
    """Start the SUM all-reduce of a whole tensor (in ``dtype`` on the wire, if given); returns a handle with ``wait()``."""
    import torch.distributed as dist
    if dtype is None or dtype == t.dtype:
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=True)
    low = t.to(dtype)
    return _CastBack([dist.all_reduce(low, op=dist.ReduceOp.SUM, group=group, async_op=True)], t, low)


class FlowArena:
    def __init__(self, sizes: Sequence[int], device):
        self.sizes = [int(s) for s in sizes]
        self.offsets: List[int] = []
        off = _ALIGN                                   # header
        for s in self.sizes:
            self.offsets.append(off)
            off += _round_up(s)
        self.total = off
        self.buf = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.views = [self.buf[o:o + s] for o, s in zip(self.offsets, self.sizes)]

    def segment_end(self, i: int, length: Optional[int] = None) -> int:
        """Arena offset one past the first ``length`` floats of segment ``i`` (whole segment by default)."""
        return self.offsets[i] + (self.sizes[i] if length is None else int(length))

    def all_reduce(self, cum_flow, group=None, dtype: Optional[torch.dtype] = None,
                   reduce_len: Optional[int] = None, op=None) -> torch.Tensor:
        """Sum the first ``reduce_len`` floats of the arena (all of it by default) over the process group, the flow
        total riding in the header.  Returns a 2-element device tensor holding the summed flow total (see
        ``decode_total``).  ``dtype`` (e.g. bfloat16) reduces in lower
        precision and copies back, as the reference's ``sync_param_flows(dtype=...)`` does."""
        import torch.distributed as dist
        op = dist.ReduceOp.SUM if op is None else op
        n = self.total if reduce_len is None else int(reduce_len)
        if isinstance(cum_flow, torch.Tensor):          # device scalar (fp64): split on the device, no host sync
            t = cum_flow.to(self.buf.device, torch.float64).reshape(())
            hi = torch.floor(t / _SPLIT)
            self.buf[:2].copy_(torch.stack((hi, t - hi * _SPLIT)).to(torch.float32))
        else:
            hi = float(int(cum_flow // _SPLIT))
            head = torch.tensor([hi, float(cum_flow - hi * _SPLIT)], dtype=torch.float32)
            self.buf[:2].copy_(head, non_blocking=True)
        part = self.buf[:n]
        if dtype is not None and dtype != torch.float32:
            hdr = self.buf[:_ALIGN].clone()            # the header stays fp32: reduce it separately
            low = part.to(dtype)
            dist.all_reduce(low, op=op, group=group)
            part.copy_(low)
            dist.all_reduce(hdr, op=op, group=group)
            self.buf[:_ALIGN].copy_(hdr)
        else:
            dist.all_reduce(part, op=op, group=group)
        return self.buf[:2].clone()                    # decoded lazily with `decode_total` (no host sync here)

    def write_total(self, cum_flow) -> None:
        """Put the running flow total into the header as (hi, lo), without a host sync for device scalars."""
        if isinstance(cum_flow, torch.Tensor):
            t = cum_flow.to(self.buf.device, torch.float64).reshape(())
            hi = torch.floor(t / _SPLIT)
            self.buf[:2].copy_(torch.stack((hi, t - hi * _SPLIT)).to(torch.float32))
        else:
            hi = float(int(cum_flow // _SPLIT))
            self.buf[:2].copy_(torch.tensor([hi, float(cum_flow - hi * _SPLIT)], dtype=torch.float32), non_blocking=True)

    def all_reduce_range_async(self, begin: int, end: int, group=None, dtype: Optional[torch.dtype] = None):
        """Start the SUM all-reduce of arena[begin:end] and return a handle with ``wait()``: the collective runs on the
        backend's own stream after the work already enqueued on the current stream, and later kernels on the
        current stream overlap with it until ``wait()`` is called.  With ``dtype`` (e.g. bfloat16) the range is
        reduced in that precision and copied back by ``wait()`` — half the bytes on the wire, as the reference's
        ``sync_param_flows(dtype=...)`` (model/tensorcircuit.py:1456-1460); the header (the flow total) always
        travels in fp32."""
        import torch.distributed as dist
        part = self.buf[begin:end]
        if dtype is None or dtype == torch.float32:
            return dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group, async_op=True)
        works = []
        lo = begin
        if begin < _ALIGN:                              # the range starts inside the header: keep that part fp32
            head = self.buf[begin:min(end, _ALIGN)]
            works.append(dist.all_reduce(head, op=dist.ReduceOp.SUM, group=group, async_op=True))
            lo = min(end, _ALIGN)
        body = self.buf[lo:end]
        low = body.to(dtype)
        works.append(dist.all_reduce(low, op=dist.ReduceOp.SUM, group=group, async_op=True))
        return _CastBack(works, body, low)

    @staticmethod
    def decode_total(head: torch.Tensor) -> float:
        hi, lo = head.tolist()
        return hi * _SPLIT + lo
