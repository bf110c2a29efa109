"""Attention for callers whose tensors live in host memory.

`flash_attention_from_host` takes q, k, v in (ideally pinned) host memory, runs
`flash_attention` on the device and leaves the result in host memory.  The batch is cut
into pieces that travel through three streams (copies in, kernels, copies out) tied by
events, so the host->device copy of piece i+1, the kernel of piece i and the device->host
copy of piece i-1 overlap; a step then costs about max(copy in, copy out, compute) instead
of their sum.  Batches are
independent in attention, so chunking changes no result.

The reference has no counterpart (MLX arrays live in unified memory on Apple silicon);
on a discrete GPU this is the shape its callers' data path takes.
"""
from __future__ import annotations

from typing import Optional, Tuple

import math

import torch

from .attention import _fwd_raw


class HostPipeline:
    """Reusable device staging buffers, streams and events for repeated calls of one shape.

    Three streams, one per role: host->device copies, kernels, device->host copies.  A piece's input slot is free as
    soon as its kernel has run and its output slot as soon as its copy out has finished, so the inbound copies never
    wait for outbound ones and the PCIe link stays busy in both directions.

    The slots' events outlive a call, so calls can follow one another without draining the pipeline: with
    ``join=False`` a call returns with its last pieces still in flight and the next call's first copies in overlap
    its copies out; `join()` (or a later call with ``join=True``) makes the current stream wait for all of them.  A
    stream of requests then costs max(copy in, copy out, compute) per request, with no fill and drain between them."""

    def __init__(self, q_shape, kv_shape, dtype, device, chunk: int = 1, depth: int = 3, want_lse: bool = True,
                 head_chunk: int = 0):
        """chunk: batches per piece; head_chunk: kv heads per piece (0 = all of them).  A piece is a
        (batch range, kv-head range) block with its group of query heads -- the unit that is independent in
        attention -- so smaller pieces shorten the pipeline's fill and drain without changing any result."""
        B, Hq, Hkv = q_shape[0], q_shape[1], kv_shape[1]
        self.chunk = max(1, min(chunk, B))
        self.head_chunk = Hkv if head_chunk <= 0 else max(1, min(head_chunk, Hkv))
        self.group = Hq // Hkv
        self.depth = max(1, depth)
        self.device = torch.device(device)
        self.want_lse = want_lse
        c, hc, g = self.chunk, self.head_chunk, self.group
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=self.device) for _ in range(3))
        mk = lambda shape, dt: [torch.empty(shape, dtype=dt, device=self.device) for _ in range(self.depth)]
        self.dq = mk((c, hc * g) + tuple(q_shape[2:]), dtype)
        self.dk = mk((c, hc) + tuple(kv_shape[2:]), dtype)
        self.dv = mk((c, hc) + tuple(kv_shape[2:]), dtype)
        self.do = mk((c, hc * g) + tuple(q_shape[2:]), dtype)
        self.dl = mk((c, hc * g, q_shape[2]), torch.float32) if want_lse else None
        # per slot: the last kernel that read its inputs, the last copy out that read its outputs
        self._ran = [None] * self.depth
        self._copied = [None] * self.depth
        self._next_slot = 0

    def join(self):
        """Makes the current stream wait for everything this pipeline has queued."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)

    def run(self, q, k, v, out, lse=None, scale=None, causal=False, softcap=0.0, window_size=None, copies_only=False,
            join=True):
        """copies_only: a measuring aid -- the same copies through the same streams and events with the kernel launch
        left out (what comes back is whatever the staging buffers held); it shows what the host link alone allows.
        join: make the current stream wait for this call's work before returning (see the class docstring)."""
        B, Hkv, g, D = q.shape[0], k.shape[1], self.group, q.shape[3]
        if scale is None:
            scale = 1.0 / math.sqrt(D)
        window_left = -1 if window_size is None else int(window_size[0])
        want_lse = self.want_lse and lse is not None
        cur = torch.cuda.current_stream(self.device)
        # work queued on the current stream before this call comes first (it may have produced the host tensors)
        started = cur.record_event()
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(started)
        pieces = [(b0, min(B, b0 + self.chunk), h0, min(Hkv, h0 + self.head_chunk))
                  for b0 in range(0, B, self.chunk) for h0 in range(0, Hkv, self.head_chunk)]
        for b0, b1, h0, h1 in pieces:
            n, nh = b1 - b0, h1 - h0
            slot = self._next_slot
            self._next_slot = (slot + 1) % self.depth
            dq, dk, dv = self.dq[slot][:n, :nh * g], self.dk[slot][:n, :nh], self.dv[slot][:n, :nh]
            do = self.do[slot][:n, :nh * g]
            dl = self.dl[slot][:n, :nh * g] if want_lse else None
            with torch.cuda.stream(self.s_in):
                if self._ran[slot] is not None:
                    self.s_in.wait_event(self._ran[slot])              # the slot's last kernel has read its inputs
                dq.copy_(q[b0:b1, h0 * g:h1 * g], non_blocking=True)
                dk.copy_(k[b0:b1, h0:h1], non_blocking=True)
                dv.copy_(v[b0:b1, h0:h1], non_blocking=True)
                landed = self.s_in.record_event()
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(landed)
                if self._copied[slot] is not None:
                    self.s_run.wait_event(self._copied[slot])          # the slot's last outputs have left it
                # a ragged last piece is a strided view of its slot: let the launch allocate its outputs then
                full = do.is_contiguous() and (dl is None or dl.is_contiguous())
                if copies_only:
                    o, l, full = do, dl, True
                else:
                    o, l = _fwd_raw(dq, dk, dv, float(scale), bool(causal), float(softcap), window_left, want_lse, self.s_run,
                                    out=do if full else None, lse=dl if full else None)
                self._ran[slot] = self.s_run.record_event()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self._ran[slot])
                if not full:
                    o.record_stream(self.s_out)
                    if l is not None:
                        l.record_stream(self.s_out)
                if want_lse:
                    lse[b0:b1, h0 * g:h1 * g].copy_(l, non_blocking=True)
                out[b0:b1, h0 * g:h1 * g].copy_(o, non_blocking=True)
                self._copied[slot] = self.s_out.record_event()
        if join:
            self.join()
        return out, lse


def flash_attention_from_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                              lse: Optional[torch.Tensor] = None, device="cuda", chunk: int = 1, depth: int = 3,
                              head_chunk: int = 0, pipeline: Optional[HostPipeline] = None, return_lse: bool = False,
                              join: bool = True, **kw) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q [B,Hq,N,D], k/v [B,Hkv,S,D] in host memory -> (out, lse) in host memory.

    Keyword arguments of `flash_attention` (scale, causal, softcap, window_size) pass through.  Pinned
    inputs and outputs are needed for the copies to be asynchronous; pageable tensors still work, only
    slower.  The call returns once the work is queued; synchronise the current stream (or the device)
    before reading `out`.  With a reusable `pipeline` and ``join=False`` consecutive calls overlap (the next call's
    copies in run beside this call's copies out); call ``pipeline.join()`` before synchronising."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("flash_attention_from_host expects host tensors; call flash_attention for device tensors")
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    if return_lse and lse is None:
        lse = torch.empty(q.shape[:3], dtype=torch.float32, pin_memory=True)
    if pipeline is None:
        pipeline = HostPipeline(q.shape, k.shape, q.dtype, device, chunk=chunk, depth=depth, want_lse=return_lse, head_chunk=head_chunk)
    return pipeline.run(q, k, v, out, lse if return_lse else None, join=join, **kw)
