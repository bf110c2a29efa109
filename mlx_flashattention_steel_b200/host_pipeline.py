"""Attention for callers whose tensors live in host memory.

`flash_attention_from_host` takes q, k, v in (ideally pinned) host memory, runs
`flash_attention` on the device and leaves the result in host memory.  The batch is cut
into chunks that travel through a small ring of CUDA streams, so the host->device copy
of chunk i+1, the kernel of chunk i and the device->host copy of chunk i-1 overlap; a
step then costs about max(copy in, copy out, compute) instead of their sum.  Batches are
independent in attention, so chunking changes no result.

The reference has no counterpart (MLX arrays live in unified memory on Apple silicon);
on a discrete GPU this is the shape its callers' data path takes.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .attention import flash_attention


class HostPipeline:
    """Reusable device staging buffers and streams for repeated calls of one shape."""

    def __init__(self, q_shape, kv_shape, dtype, device, chunk: int = 1, depth: int = 3, want_lse: bool = True):
        B = q_shape[0]
        self.chunk = max(1, min(chunk, B))
        self.depth = max(1, depth)
        self.device = torch.device(device)
        self.want_lse = want_lse
        c = self.chunk
        self.streams = [torch.cuda.Stream(device=self.device) for _ in range(self.depth)]
        self.dq = [torch.empty((c,) + tuple(q_shape[1:]), dtype=dtype, device=self.device) for _ in range(self.depth)]
        self.dk = [torch.empty((c,) + tuple(kv_shape[1:]), dtype=dtype, device=self.device) for _ in range(self.depth)]
        self.dv = [torch.empty((c,) + tuple(kv_shape[1:]), dtype=dtype, device=self.device) for _ in range(self.depth)]

    def run(self, q, k, v, out, lse=None, **kw):
        B = q.shape[0]
        cur = torch.cuda.current_stream(self.device)
        for s in self.streams:
            s.wait_stream(cur)
        for i, b0 in enumerate(range(0, B, self.chunk)):
            b1 = min(B, b0 + self.chunk)
            n = b1 - b0
            slot = i % self.depth
            st = self.streams[slot]
            with torch.cuda.stream(st):
                dq, dk, dv = self.dq[slot][:n], self.dk[slot][:n], self.dv[slot][:n]
                dq.copy_(q[b0:b1], non_blocking=True)
                dk.copy_(k[b0:b1], non_blocking=True)
                dv.copy_(v[b0:b1], non_blocking=True)
                if self.want_lse and lse is not None:
                    o, l = flash_attention(dq, dk, dv, return_lse=True, stream=st, **kw)
                    lse[b0:b1].copy_(l, non_blocking=True)
                else:
                    o = flash_attention(dq, dk, dv, stream=st, **kw)
                out[b0:b1].copy_(o, non_blocking=True)
                # the staging buffers of this slot are reused `depth` chunks later on the same stream,
                # so stream order alone keeps the copies and the kernel from overtaking each other
        for s in self.streams:
            cur.wait_stream(s)
        return out, lse


def flash_attention_from_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                              lse: Optional[torch.Tensor] = None, device="cuda", chunk: int = 1, depth: int = 3,
                              pipeline: Optional[HostPipeline] = None, return_lse: bool = False,
                              **kw) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q [B,Hq,N,D], k/v [B,Hkv,S,D] in host memory -> (out, lse) in host memory.

    Keyword arguments of `flash_attention` (scale, causal, softcap, window_size) pass through.  Pinned
    inputs and outputs are needed for the copies to be asynchronous; pageable tensors still work, only
    slower.  The call returns once the work is queued; synchronise the current stream (or the device)
    before reading `out`."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("flash_attention_from_host expects host tensors; call flash_attention for device tensors")
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    if return_lse and lse is None:
        lse = torch.empty(q.shape[:3], dtype=torch.float32, pin_memory=True)
    if pipeline is None:
        pipeline = HostPipeline(q.shape, k.shape, q.dtype, device, chunk=chunk, depth=depth, want_lse=return_lse)
    return pipeline.run(q, k, v, out, lse if return_lse else None, **kw)
