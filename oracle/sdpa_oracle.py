"""CPU restatement of the reference's SDPA fallback formulas.  TEST INFRASTRUCTURE ONLY.

Parity status: **parity unpinned at the bit level.**  The arithmetic of the
reference's CPU path lives in MLX (``mx.fast.scaled_dot_product_attention``,
``mx.softmax``, ``mx.dequantize``; requirement ``mlx>=0.18.0``, developed on
0.31.0), which is not vendored in the reference and not installable here, and the
reference ships no golden vectors.  What is pinned: the mathematical definition
each reference test states as its own oracle (cited per function) and analytic
known-answer cases (tests/test_oracle.py).  Parity with the CUDA kernels is
therefore defined by tolerance: 2e-2 max-abs for f16/bf16, 1e-5 for f32, bit-exact
for the page gather.

Every function computes in float64 unless ``faithful=True``, which rounds where the
reference formulas round (scores in the input dtype, probabilities cast to the
input dtype before ``A @ V``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

LOG2E = 1.4426950408889634


def _visible(N: int, S: int, causal: bool, window_left: int, rows: slice) -> Optional[torch.Tensor]:
    """Boolean [rows, S] visibility mask, or None when everything is visible.

    Causal: additive ``-inf`` on ``triu(k = S - N + 1)`` i.e. key ``j`` visible to
    row ``i`` iff ``j <= i + (S - N)`` (mlx_mfa/attention.py:2066-2072;
    tests/test_attention.py:32-39).  Window: ``k_idx >= q_idx - left`` with
    ``q_idx = arange(S - N, S)``, no right bound unless causal
    (mlx_mfa/attention.py:293-305; tests/test_attention.py:4829-4845)."""
    if not causal and window_left < 0:
        return None
    qi = torch.arange(N)[rows].unsqueeze(1) + (S - N)
    kj = torch.arange(S).unsqueeze(0)
    vis = torch.ones((qi.shape[0], S), dtype=torch.bool)
    if causal:
        vis &= kj <= qi
    if window_left >= 0:
        vis &= kj >= qi - window_left
    return vis


def sdpa(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    causal: bool = False,
    softcap: float = 0.0,
    window_left: int = -1,
    faithful: bool = False,
    row_block: int = 1024,
    alibi_slopes: Optional[torch.Tensor] = None,
    block_mask: Optional[torch.Tensor] = None,
    block: Tuple[int, int] = (32, 16),
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Dense attention.  q [B,Hq,N,D], k/v [B,Hkv,S,D] (CPU tensors, any float dtype).

    Returns (O, L_steel, L_fallback): O float64 (or q.dtype when faithful);
    L_steel = log2(e) * logsumexp(s) (kernel convention, csrc/mfa_steel_fwd.cpp:630,
    1208-1221); L_fallback = log2(sum_j 2^{s_j}) (mlx_mfa/attention.py:2096-2110).

    Follows _fallback_sdpa (mlx_mfa/attention.py:2058-2076) and _softcap_sdpa_ref
    (mlx_mfa/attention.py:1731-1771: scale, tanh cap, then mask, softmax in f32,
    probabilities cast to q.dtype before A @ V).  GQA: query head h reads kv head
    h // (Hq/Hkv) (csrc/mfa_steel_fwd.cpp:545), as the tests do with mx.repeat
    (tests/test_attention.py:458-460).  Rows with no visible key give O = 0,
    L = -inf.  alibi_slopes [Hq]: slope[h] * (j - (i + S - N)) is added after the
    cap and before the mask (_alibi_sdpa_ref, mlx_mfa/attention.py:1774-1822, with
    the kernel's query position i + qL_off, csrc/mfa_steel_fwd.cpp:951-970; the two
    differ by a per-row constant, which the softmax cancels).  block_mask bool
    [ceil(N/BQ), ceil(S/BK)] with block = (BQ, BK): element (i, j) is visible only if
    block_mask[i // BQ, j // BK] (_sparse_fallback_sdpa / _block_mask_to_float_bias,
    mlx_mfa/attention.py:1399-1432).
    """
    B, Hq, N, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    g = Hq // Hkv
    cdt = q.dtype if faithful else torch.float64
    sdt = torch.float32 if faithful else torch.float64
    kk = k.repeat_interleave(g, dim=1).to(cdt)
    vv = v.repeat_interleave(g, dim=1).to(cdt)
    qq = q.to(cdt)
    O = torch.zeros((B, Hq, N, D), dtype=cdt)
    L1 = torch.full((B, Hq, N), float("-inf"), dtype=torch.float64)
    L2 = torch.full((B, Hq, N), float("-inf"), dtype=torch.float64)
    if S == 0:
        return O, L1, L2
    for r0 in range(0, N, row_block):
        rows = slice(r0, min(N, r0 + row_block))
        s = torch.matmul(qq[:, :, rows], kk.transpose(-1, -2)) * scale
        if softcap > 0:
            s = torch.tanh(s / softcap) * softcap
        s = s.to(sdt)
        if alibi_slopes is not None:
            qpos = torch.arange(rows.start, rows.stop, dtype=sdt)[:, None] + (S - N)
            kpos = torch.arange(S, dtype=sdt)[None, :]
            s = s + alibi_slopes.to(sdt)[None, :, None, None] * (kpos - qpos)[None, None]
        vis = _visible(N, S, causal, window_left, rows)
        if block_mask is not None:
            cells = block_mask.bool().repeat_interleave(block[0], dim=0)[:N].repeat_interleave(block[1], dim=1)[:, :S]
            cells = cells[rows]
            vis = cells if vis is None else (vis & cells)
        if vis is not None:
            s = s.masked_fill(~vis, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        a = torch.where(den > 0, e / den, torch.zeros_like(e))
        O[:, :, rows] = torch.matmul(a.to(cdt), vv)
        s64 = s.to(torch.float64)
        m64 = m.to(torch.float64)
        lse_nat = (m64 + torch.log(torch.exp(s64 - m64).sum(-1, keepdim=True))).squeeze(-1)
        L1[:, :, rows] = lse_nat * LOG2E
        L2[:, :, rows] = (m64 + torch.log2(torch.exp2(s64 - m64).sum(-1, keepdim=True))).squeeze(-1)
    return O, L1, L2


def varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_q: Sequence[int],
    cu_k: Sequence[int],
    scale: Optional[float] = None,
    causal: bool = False,
    faithful: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packed sequences: slice, attend, concatenate — _varlen_split_concat
    (mlx_mfa/attention.py:2365-2390; tests/test_attention.py:2254-2272).
    Returns (O [1,H,total_q,D], L_steel [1,H,total_q])."""
    outs, ls = [], []
    for i in range(len(cu_q) - 1):
        o, l1, _ = sdpa(q[:, :, cu_q[i]:cu_q[i + 1]], k[:, :, cu_k[i]:cu_k[i + 1]],
                        v[:, :, cu_k[i]:cu_k[i + 1]], scale, causal, faithful=faithful)
        outs.append(o)
        ls.append(l1)
    return torch.cat(outs, dim=2), torch.cat(ls, dim=2)


def paged_gather(pool: np.ndarray, block_table: np.ndarray, seq_lens: np.ndarray, max_kv_len: int) -> np.ndarray:
    """pool [P,bs,H,D] -> [B,H,max_kv_len,D]; the loop of MFAPagedKVGather::eval_cpu
    (csrc/mfa_paged_gather.cpp:89-129) vectorised per page: zero-filled output,
    tokens beyond seq_lens[b] and pages with a negative table entry stay zero."""
    P, bs, H, D = pool.shape
    B = block_table.shape[0]
    out = np.zeros((B, H, max_kv_len, D), dtype=pool.dtype)
    for b in range(B):
        n = int(seq_lens[b])
        for lb in range((n + bs - 1) // bs):
            phys = int(block_table[b, lb])
            if phys < 0:
                continue
            t0 = lb * bs
            cnt = min(bs, n - t0)
            out[b, :, t0:t0 + cnt, :] = pool[phys, :cnt].transpose(1, 0, 2)
    return out


def dequant(data: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Per-token-per-head symmetric dequantisation to the query dtype:
    ``float(x) * float(scale)`` rounded to ``dtype`` — mx.dequantize(..., dtype=q.dtype)
    with one zero-bias group spanning D (mlx_mfa/integrations/mlx_lm.py:97-110)."""
    return (data.to(torch.float32) * scale.to(torch.float32).unsqueeze(-1)).to(dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset=0, interleaved: bool = True,
         rotary_dim: Optional[int] = None) -> torch.Tensor:
    """Rotary embedding of x [B,H,N,D] in float64 (mlx_mfa/attention.py:2128-2210): row n of batch b uses table row
    offset[b] + n; interleaved pairs (2i, 2i+1) or halves (i, i + rot/2); out[a] = x[a]cos - x[b]sin,
    out[b] = x[a]sin + x[b]cos; elements beyond rotary_dim pass through."""
    B, H, N, D = x.shape
    rot = D if rotary_dim is None else rotary_dim
    xd = x.to(torch.float64)
    out = xd.clone()
    offs = [int(offset)] * B if isinstance(offset, int) else [int(o) for o in offset]
    for b in range(B):
        c = cos[offs[b]:offs[b] + N].to(torch.float64)[None]          # [1, N, rot/2]
        s_ = sin[offs[b]:offs[b] + N].to(torch.float64)[None]
        if interleaved:
            a, bb = xd[b, :, :, 0:rot:2], xd[b, :, :, 1:rot:2]
            out[b, :, :, 0:rot:2] = a * c - bb * s_
            out[b, :, :, 1:rot:2] = a * s_ + bb * c
        else:
            a, bb = xd[b, :, :, :rot // 2], xd[b, :, :, rot // 2:rot]
            out[b, :, :, :rot // 2] = a * c - bb * s_
            out[b, :, :, rot // 2:rot] = a * s_ + bb * c
    return out


def quantise_kv(x: torch.Tensor, kind: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-(token, head) symmetric quantisation of rows [..., D] to int8 or fp8-e4m3, the inverse of `dequant`:
    scale = f16(max|x| / qmax) (1 where that is zero), q = round-to-nearest-even(x / float(scale)) clamped to
    +-qmax (qmax 127 / 448).  float32 arithmetic throughout, so a device kernel can match it bit for bit.  The
    reference has no 8-bit pool (its quantised caches are MLX affine tuples, mlx_mfa/integrations/mlx_lm.py:97-110);
    this is the format this build defines for its decode kernel."""
    qmax = 127.0 if kind == "int8" else 448.0
    xf = x.to(torch.float32)
    sc = (xf.abs().amax(dim=-1) / qmax).to(torch.float16)
    sc = torch.where(sc == 0, torch.ones_like(sc), sc)
    y = xf / sc.to(torch.float32).unsqueeze(-1)
    if kind == "int8":
        return y.round().clamp(-127, 127).to(torch.int8), sc
    return y.clamp(-448, 448).to(torch.float8_e4m3fn), sc


def kv_append(k_pool: torch.Tensor, v_pool: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
              slot_mapping: Sequence[int], k_scale: Optional[torch.Tensor] = None,
              v_scale: Optional[torch.Tensor] = None) -> None:
    """In-place scatter of new tokens [T, Hkv, D] into pools [P, bs, Hkv, D]: token t goes to page
    slot // bs, offset slot % bs (negative slots are skipped) -- the end state of the splice loop of
    PagedKVCache.append (mlx_mfa/attention.py:2642-2711).  8-bit pools are quantised with `quantise_kv`
    and their scales written to k_scale / v_scale [P, bs, Hkv]."""
    P, bs, H, D = k_pool.shape
    for pool, new, scale in ((k_pool, k_new, k_scale), (v_pool, v_new, v_scale)):
        quant = pool.dtype in (torch.int8, torch.float8_e4m3fn)
        for t, slot in enumerate(slot_mapping):
            slot = int(slot)
            if slot < 0 or slot >= P * bs:
                continue
            page, offs = divmod(slot, bs)
            if quant:
                qx, sc = quantise_kv(new[t], "int8" if pool.dtype == torch.int8 else "e4m3")
                pool[page, offs] = qx
                scale[page, offs] = sc
            else:
                pool[page, offs] = new[t].to(torch.float32).to(pool.dtype)


def paged_attention(
    q: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    scale: Optional[float] = None,
    causal: bool = False,
    softcap: float = 0.0,
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Paged attention as the reference's CPU route does it: gather pages, slice each
    sequence to its exact length, attend per sequence, concatenate
    (mlx_mfa/attention.py:2950-2989).  Quantized pools are dequantised to q.dtype
    first.  Returns (O float64 [B,Hq,Nq,D], L_steel [B,Hq,Nq])."""
    B = q.shape[0]
    if k_scale is not None:
        k_pool = dequant(k_pool, k_scale, q.dtype)
        v_pool = dequant(v_pool, v_scale, q.dtype)
    lens = seq_lens.numpy()
    table = block_table.numpy()
    outs, ls = [], []
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            outs.append(torch.zeros((1,) + tuple(q.shape[1:]), dtype=torch.float64))
            ls.append(torch.full((1,) + tuple(q.shape[1:3]), float("-inf"), dtype=torch.float64))
            continue
        kb = paged_gather(k_pool.view(torch.int16).numpy() if k_pool.element_size() == 2 else k_pool.numpy(),
                          table[b:b + 1], lens[b:b + 1], n)
        vb = paged_gather(v_pool.view(torch.int16).numpy() if v_pool.element_size() == 2 else v_pool.numpy(),
                          table[b:b + 1], lens[b:b + 1], n)
        kt, vt = torch.from_numpy(kb), torch.from_numpy(vb)
        if k_pool.element_size() == 2:
            kt, vt = kt.view(k_pool.dtype), vt.view(v_pool.dtype)
        o, l1, _ = sdpa(q[b:b + 1], kt, vt, scale, causal, softcap)
        outs.append(o)
        ls.append(l1)
    return torch.cat(outs, dim=0), torch.cat(ls, dim=0)


def backward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dout: torch.Tensor,
    scale: Optional[float] = None,
    causal: bool = False,
    cu_q: Optional[Sequence[int]] = None,
    cu_k: Optional[Sequence[int]] = None,
    softcap: float = 0.0,
    window_left: int = -1,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """dQ, dK, dV by autograd in float64 through the formulas above — what the
    reference tests do with mx.grad(reference_sdpa) (tests/test_attention.py:191-207,
    4362-4368).  With cu_q/cu_k the sequences are packed (varlen).  softcap and window_left follow the
    reference's differentiable SDPA fallbacks (mlx_mfa/attention.py:1976-1992 window mask, 2020-2027 and
    1758-1768 tanh cap before the mask)."""
    q64 = q.detach().to(torch.float64).requires_grad_(True)
    k64 = k.detach().to(torch.float64).requires_grad_(True)
    v64 = v.detach().to(torch.float64).requires_grad_(True)
    B, Hq, N, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    g = Hq // k.shape[1]

    def attend(qs, ks, vs):
        n, s_len = qs.shape[2], ks.shape[2]
        kk = ks.repeat_interleave(g, dim=1)
        vv = vs.repeat_interleave(g, dim=1)
        s = torch.matmul(qs, kk.transpose(-1, -2)) * scale
        if softcap > 0:
            s = torch.tanh(s / softcap) * softcap
        vis = _visible(n, s_len, causal, window_left, slice(0, n))
        if vis is not None:
            s = s.masked_fill(~vis, float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1), vv)

    if cu_q is None:
        o = attend(q64, k64, v64)
    else:
        parts = [attend(q64[:, :, cu_q[i]:cu_q[i + 1]], k64[:, :, cu_k[i]:cu_k[i + 1]],
                        v64[:, :, cu_k[i]:cu_k[i + 1]]) for i in range(len(cu_q) - 1)]
        o = torch.cat(parts, dim=2)
    o.backward(dout.to(torch.float64))
    return q64.grad, k64.grad, v64.grad
