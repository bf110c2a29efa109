"""Two-GPU test (skipped on a one-GPU box): a long decode sequence whose pages are split across
two ranks, each running the paged decode kernel on its part, combined over NCCL; the result must
match the one-GPU kernel on the whole sequence and the CPU oracle."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, payload, ret):
    import torch.distributed as dist

    import mlx_flashattention_steel_b200 as fa
    from mlx_flashattention_steel_b200 import parallel as par

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        q, kq, vq, ks, vs, table, seq_len = payload
        n_pages = (seq_len + 15) // 16
        lo, hi, ntok = par.split_pages(n_pages, world, rank, 16, seq_len)
        # this rank's part of the page list, renumbered from 0; the pools hold only its own pages
        pages = table[0, lo:hi].long()
        k_loc, v_loc = kq[pages].to(dev), vq[pages].to(dev)
        ks_loc, vs_loc = ks[pages].to(dev), vs[pages].to(dev)
        tbl = torch.arange(hi - lo, dtype=torch.int32, device=dev).unsqueeze(0)
        lens = torch.tensor([ntok], dtype=torch.int32, device=dev)
        O, L = par.decode_long_sequence(q.to(dev), k_loc, v_loc, tbl, lens, k_scale=ks_loc, v_scale=vs_loc)
        torch.cuda.synchronize()
        if rank == 0:
            ret.put((O.cpu(), L.cpu()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_long_sequence_split_across_two_gpus(dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import mlx_flashattention_steel_b200 as fa
    from oracle import sdpa_oracle as orc

    from .util import make_paged, randn, run_ranks

    seq_len = 20000
    pg = make_paged(1, 8, 128, 16, [seq_len], torch.bfloat16, 700, quant="int8")
    q = randn((1, 32, 1, 128), torch.bfloat16, 701)
    payload = (q, pg["k"], pg["v"], pg["k_scale"], pg["v_scale"], pg["block_table"], seq_len)
    O, L = run_ranks(_worker, 2, (payload,), timeout=300)
    one, lone = fa.flash_attention_paged(q.to(dev), pg["k"].to(dev), pg["v"].to(dev), pg["block_table"].to(dev),
                                         pg["seq_lens"].to(dev), k_scale=pg["k_scale"].to(dev),
                                         v_scale=pg["v_scale"].to(dev), return_lse=True)
    assert float((O.float() - one.cpu().float()).abs().max()) <= 2e-2
    assert float((L - lone.cpu()).abs().max()) <= 2e-2
    ref, lref = orc.paged_attention(q, pg["k"], pg["v"], pg["block_table"], pg["seq_lens"], k_scale=pg["k_scale"],
                                    v_scale=pg["v_scale"])
    assert float((O.double() - ref).abs().max()) <= 2e-2
    assert float((L.double() - lref).abs().max()) <= 2e-2
