"""Writes tests/golden/sdpa_golden.npz: small seeded inputs and the float64 outputs
of the CPU oracle.  The reference ships no golden vectors and its CPU arithmetic
(MLX) cannot run here, so these vectors pin the oracle against itself over time and
give the GPU tests fixed inputs; they are not outputs of the reference.

Usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import sdpa_oracle as orc  # noqa: E402


def main():
    out = {}
    g = torch.Generator().manual_seed(1234)
    q = torch.randn((2, 4, 37, 64), generator=g)
    k = torch.randn((2, 2, 40, 64), generator=g)
    v = torch.randn((2, 2, 40, 64), generator=g)
    O, L, _ = orc.sdpa(q, k, v, causal=True)
    out.update(dense_causal_gqa_q=q.numpy(), dense_causal_gqa_k=k.numpy(), dense_causal_gqa_v=v.numpy(),
               dense_causal_gqa_o=O.numpy(), dense_causal_gqa_lse=L.numpy())
    q = torch.randn((1, 2, 70, 128), generator=g)
    k = torch.randn((1, 2, 70, 128), generator=g)
    v = torch.randn((1, 2, 70, 128), generator=g)
    O, L, _ = orc.sdpa(q, k, v, causal=True, softcap=30.0, window_left=17)
    out.update(softcap_window_q=q.numpy(), softcap_window_k=k.numpy(), softcap_window_v=v.numpy(),
               softcap_window_o=O.numpy(), softcap_window_lse=L.numpy(),
               softcap_window_softcap=np.float64(30.0), softcap_window_window_left=np.int64(17))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sdpa_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path))


if __name__ == "__main__":
    main()
