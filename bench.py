#!/usr/bin/env python
"""Headline benchmark: causal GQA prefill attention TFLOP/s (causal-adjusted) on B200,
with the paged int8-KV decode GB/s reported beside it.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

N = 1 workload ("config 2"): B=4, Hq=32, Hkv=8, N=S=8192, D=128, bf16, causal,
softcap=50, return_lse; synthetic N(0,1) inputs from a fixed seed.  With N > 1 (one
process per GPU under torchrun) every rank runs its own batch of 4 — (batch, kv-head)
shards need no collective — so scaling is weak and `value` is the sum over ranks.
Beside that headline the line carries, at every N: `strong` (the ONE fixed config-2
batch dealt out as 32 (batch, kv-head) units, 32/N per rank), `decode` (config 4 with
its 128 sequences sharded by batch, each rank with its own pool), `decode_long` (one
256k-token int8 sequence whose pages are split across the ranks, partials combined
over NCCL) and `e2e.copy_ceiling_gbs` (the end-to-end pipeline with the kernel left out).

One "step" = one forward over the batch.  `value` is timed with CUDA events on the
launching stream with inputs resident in HBM (inputs are 403 MB > the 126 MB L2, so no
explicit flush is needed); `e2e` is the same step through the public Python API with
pinned host buffers, host->device and device->host copies inside the timed region.
`--impl reference` times the CPU restatement of the reference's SDPA fallback (the
reference's own CPU arithmetic lives in MLX, which cannot be installed here).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "prefill attn TFLOP/s (causal-adj)"
C2 = dict(B=4, Hq=32, Hkv=8, N=8192, S=8192, D=128, softcap=50.0)
C4 = dict(B=128, Hq=32, Hkv=8, D=128, block_size=16, lo=512, hi=32768)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tf=p["bf16_tflops"], tf_sustained=p.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


def causal_pairs(N, S):
    off = S - N
    return sum(min(S, i + off + 1) for i in range(N)) if N != S else N * (N + 1) // 2


def prefill_flops(cfg, batch=None):
    b = cfg["B"] if batch is None else batch
    return 4.0 * b * cfg["Hq"] * cfg["D"] * causal_pairs(cfg["N"], cfg["S"])


class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs: NVML queries (read-only) from a
    thread every ~2 ms; nvidia-smi at 100 ms when NVML cannot be loaded."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index):
        self.index = index
        self.rows = []          # (wall time, sm MHz, power W, reasons bit mask)
        self.proc = None
        self.nvml = None
        self.stop_flag = False
        self.max_mhz = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, h

    def start(self):
        try:
            self.nvml, self.handle = self._nvml_handle()
            self.max_mhz = float(self.nvml.nvmlDeviceGetMaxClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                watts = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                try:
                    mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.rows.append((time.time(), mhz, watts, mask))
            except Exception:
                break
            time.sleep(0.002)

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inv = {v: k for k, v in self.BITS.items()}
        for line in self.proc.stdout:
            r = [x.strip() for x in line.split(",")]
            if len(r) < 9:
                continue
            mask = 0
            for nme, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    mask |= inv[nme]
            self.max_mhz = float(r[2])
            self.rows.append((time.time(), float(r[1]), float(r[3]), mask))

    def stop(self, t0, t1):
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML, no nvidia-smi"]}
        if self.nvml is not None:
            self.stop_flag = True
            self.t.join(timeout=1.0)
            source, slack = "nvml", 0.0
        else:
            time.sleep(0.15)
            self.proc.terminate()
            source, slack = "nvidia-smi", 0.15
        rows = [r for r in self.rows if t0 - slack <= r[0] <= t1 + slack] or list(self.rows)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mask = 0
        for r in rows:
            mask |= r[3]
        return {"sm_mhz": statistics.median(r[1] for r in rows), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(v for k, v in self.BITS.items() if mask & k), "samples": len(rows),
                "power_w_max": max(r[2] for r in rows), "source": source}


def make_prefill_inputs(cfg, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    B, Hq, Hkv, N, S, D = (cfg[k] for k in ("B", "Hq", "Hkv", "N", "S", "D"))
    # generated on the device for speed; the distribution (N(0,1), bf16) is what the config names
    gd = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn((B, Hq, N, D), generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn((B, Hkv, S, D), generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, D), generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
    del g
    return q, k, v


def cpu_prefill_sample(cfg, seed, repeats=1):
    """Times the oracle (CPU restatement of the reference's softcap SDPA fallback) on one
    (batch, kv-group) slice of the workload: 1 batch x Hq/Hkv query heads x 1 kv head."""
    from oracle import sdpa_oracle as orc

    g = cfg["Hq"] // cfg["Hkv"]
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn((1, g, cfg["N"], cfg["D"]), generator=gen)
    k = torch.randn((1, 1, cfg["S"], cfg["D"]), generator=gen)
    v = torch.randn((1, 1, cfg["S"], cfg["D"]), generator=gen)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.sdpa(q, k, v, causal=True, softcap=cfg["softcap"], faithful=True, row_block=512)
        best = min(best, time.perf_counter() - t0)
    flops = 4.0 * g * cfg["D"] * causal_pairs(cfg["N"], cfg["S"])
    return flops / best / 1e12, best, f"1 batch x 1 kv-head group ({g} q-heads) of the workload = 1/{cfg['B'] * cfg['Hkv']} of a step, float32, torch CPU"


def run_reference(args, rank, world):
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = dict(C2)
    for _ in range(max(args.warmup, 0)):
        cpu_prefill_sample(dict(cfg, N=1024, S=1024), 0)
    vals, secs = [], []
    sample = ""
    for i in range(args.steps):
        tf, s, sample = cpu_prefill_sample(cfg, 2 + i)
        vals.append(tf)
        secs.append(s)
    val = statistics.median(vals)
    g = cfg["Hq"] // cfg["Hkv"]
    slice_ms = statistics.median(secs) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": slice_ms,
        "ms_per_step_full_equiv": slice_ms * cfg["B"] * cfg["Hkv"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (wider than the reference's own bf16 CPU path: the restatement computes in float32)",
        "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's SDPA fallback (MLX itself is not installable here); "
                "each step times one (batch, kv-group) slice = 1/32 of the workload: ms_per_step is that slice's own time, "
                "ms_per_step_full_equiv the same scaled to the whole batch; value (TFLOP/s) is scale-free",
    }
    print(json.dumps(line), flush=True)


def workload_config(n):
    return {"workload": "config 2: GQA causal prefill fwd B=4 Hq=32 Hkv=8 N=S=8192 D=128 bf16 softcap=50 return_lse",
            "global_batch": C2["B"] * n, "seq_len": C2["N"], "parallelism": f"(batch,kv-head) shards, dp{n}, no collective",
            "l2": "inputs (403 MB) exceed L2 (126 MB); no explicit flush"}


def dram_traffic_ratio(key):
    """DRAM bytes per algorithmic byte of the ncu capture named `key` (measured on a small case of the same kernel);
    None when the table is missing."""
    try:
        t = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))[key]
        return float(t["dram_bytes"]) / float(t["algorithmic_bytes"])
    except (OSError, KeyError, ValueError):
        return None


def bench_decode(device, steps, warmup, pk, batch=None, rank=0, world=1, dist=None):
    """Config 4: paged int8-KV decode, B=128, seq_lens ~ U[512, 32768], page 16.  With world > 1 the 128 sequences are
    sharded by batch: rank r owns a subset of them, balanced by KV length, with a pool of its own (no collective on the
    data path); the total is all ranks' bytes over the slowest rank's time."""
    import numpy as np

    import mlx_flashattention_steel_b200 as fa
    from mlx_flashattention_steel_b200 import parallel as par

    cfg = dict(C4)
    if batch:
        cfg["B"] = batch
    rng = np.random.default_rng(4)
    all_lens = rng.integers(cfg["lo"], cfg["hi"] + 1, size=cfg["B"]).astype(np.int32)
    # sequences are dealt out by KV length (the cost of a decode step), not by position: the slowest rank sets the time
    mine = par.shard_by_load(all_lens, world)[rank]
    lens = all_lens[np.asarray(mine, dtype=np.int64)]
    nb = len(mine)
    bs, Hkv, D = cfg["block_size"], cfg["Hkv"], cfg["D"]
    pages_per = (lens + bs - 1) // bs
    P = int(pages_per.sum()) + 8
    perm = rng.permutation(P)
    max_blocks = int(pages_per.max())
    table = -np.ones((nb, max_blocks), dtype=np.int32)
    pos = 0
    for b in range(nb):
        n = int(pages_per[b])
        table[b, :n] = perm[pos:pos + n]
        pos += n
    gd = torch.Generator(device=device).manual_seed(4 + rank)
    pools = {}
    for name in ("k", "v"):
        qx = torch.empty((P, bs, Hkv, D), dtype=torch.int8, device=device)
        sc = torch.empty((P, bs, Hkv), dtype=torch.float16, device=device)
        step_p = 8192
        for p0 in range(0, P, step_p):
            x = torch.randn((min(step_p, P - p0), bs, Hkv, D), generator=gd, device=device)
            s = (x.abs().amax(dim=-1) / 127.0).to(torch.float16)
            qx[p0:p0 + x.shape[0]] = (x / s.float().unsqueeze(-1)).round().clamp(-127, 127).to(torch.int8)
            sc[p0:p0 + x.shape[0]] = s
        pools[name] = (qx, sc)
    q = torch.randn((nb, cfg["Hq"], 1, D), generator=gd, device=device).to(torch.bfloat16)
    table_t = torch.from_numpy(table).to(device)
    lens_t = torch.from_numpy(lens).to(device)
    max_len = int(lens.max())
    tokens = int(lens.sum())
    bytes_alg = tokens * Hkv * (2 * D + 4)

    def step():
        return fa.flash_attention_paged(q, pools["k"][0], pools["v"][0], table_t, lens_t, causal=True, block_size=bs,
                                        k_scale=pools["k"][1], v_scale=pools["v"][1], max_kv_len=max_len)

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    gbs = bytes_alg / (ms * 1e-3) / 1e9
    ms_max, bytes_total, per_rank = ms, bytes_alg, [gbs]
    if dist is not None:
        t = torch.tensor([ms, float(bytes_alg)], device=device, dtype=torch.float64)
        allt = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        ms_max = max(float(x[0]) for x in allt)
        bytes_total = sum(float(x[1]) for x in allt)
        per_rank = [float(x[1]) / (float(x[0]) * 1e-3) / 1e9 for x in allt]
    total_gbs = bytes_total / (ms_max * 1e-3) / 1e9
    ratio = dram_traffic_ratio("decode_paged_config4_small")
    return {"metric": "paged-decode KV GB/s", "value": total_gbs, "unit": "GB/s", "ms_per_step": ms_max,
            "workload": f"config 4: B={cfg['B']} Hq=32 Hkv=8 D=128 page 16 seq_lens~U[512,32768] int8 KV + f16 scales, bf16 q"
                        + (f"; sequences sharded by batch over {world} GPUs (balanced by KV length), one pool per GPU" if world > 1 else ""),
            "n_gpus": world, "per_gpu_gbs": per_rank, "tokens": tokens if world == 1 else None,
            "algorithmic_bytes": bytes_total,
            # per GPU: rank 0's own launch against the measured copy bandwidth of one GPU
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                         # the ncu capture was taken at B=24; DRAM traffic grows with the tokens processed
                         "traffic": bytes_alg * ratio if ratio else None, "peak_source": pk["src"]},
            "gpu_launches": steps * 2}


def bench_strong(device, rank, world, dist, steps, warmup):
    """Strong scaling of config 2: ONE fixed batch (same seed on every rank), dealt out as 32 (batch, kv-head) units;
    each rank attends its 32 / world units as views of the full tensors, no collective.  Time = slowest rank."""
    import mlx_flashattention_steel_b200 as fa
    from mlx_flashattention_steel_b200 import parallel as par

    cfg = dict(C2)
    q, k, v = make_prefill_inputs(cfg, device, seed=2)
    g = cfg["Hq"] // cfg["Hkv"]
    blocks = par.shard_blocks(cfg["B"], cfg["Hkv"], world, rank)

    def step():
        for b, h0, h1 in blocks:
            fa.flash_attention(q[b:b + 1, h0 * g:h1 * g], k[b:b + 1, h0:h1], v[b:b + 1, h0:h1], causal=True,
                               softcap=cfg["softcap"], return_lse=True)

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    units = sum(h1 - h0 for _, h0, h1 in blocks)
    return {"scaling": "strong", "workload": "the one config-2 batch (B=4, 32 (batch, kv-head) units) split over the GPUs",
            "units_per_gpu": units, "launches_per_step_per_gpu": len(blocks), "ms_per_step": ms,
            "value": prefill_flops(cfg) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}


def bench_decode_long(device, rank, world, dist, steps, warmup):
    """One 262144-token int8 sequence (Hq=32, Hkv=8, D=128, page 16) whose pages are split across the ranks: each rank
    runs the paged decode kernel on its pages (fp32 partials + lse in one packed buffer), one NCCL all-gather, one
    combine launch.  Reports the whole step and the local kernel alone, i.e. the share the exchange costs."""
    import mlx_flashattention_steel_b200 as fa
    from mlx_flashattention_steel_b200 import attention as fa_attn, parallel as par

    S, Hq, Hkv, D, bs = 262144, 32, 8, 128, 16
    n_pages = S // bs
    lo, hi, ntok = par.split_pages(n_pages, world, rank, bs, S)
    P = hi - lo
    gd = torch.Generator(device=device).manual_seed(40 + rank)
    kq = torch.randint(-127, 128, (P, bs, Hkv, D), generator=gd, device=device, dtype=torch.int8)
    vq = torch.randint(-127, 128, (P, bs, Hkv, D), generator=gd, device=device, dtype=torch.int8)
    ksc = (torch.rand((P, bs, Hkv), generator=gd, device=device) * 0.004 + 0.006).to(torch.float16)
    vsc = (torch.rand((P, bs, Hkv), generator=gd, device=device) * 0.004 + 0.006).to(torch.float16)
    q = torch.randn((1, Hq, 1, D), generator=torch.Generator(device=device).manual_seed(41), device=device).to(torch.bfloat16)
    tbl = torch.randperm(P, generator=gd, device=device).to(torch.int32).unsqueeze(0)
    lens = torch.tensor([ntok], dtype=torch.int32, device=device)

    def local():
        return fa_attn._decode_raw(q, kq, vq, ksc, vsc, tbl, lens, ntok, D ** -0.5, False, 0.0, bs, True, None, packed=True)

    def full():
        if dist is None:
            return fa.flash_attention_paged(q, kq, vq, tbl, lens, k_scale=ksc, v_scale=vsc, max_kv_len=ntok)
        return par.decode_long_sequence(q, kq, vq, tbl, lens, k_scale=ksc, v_scale=vsc, max_kv_len=ntok)

    res = {}
    for name, fn in (("step", full), ("local_kernel", local)):
        for _ in range(max(warmup, 3)):
            fn()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if dist is not None:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        res[name] = ms
    bytes_alg = S * Hkv * (2 * D + 4)
    return {"workload": "one 262144-token sequence, int8 KV + f16 scales, Hq=32 Hkv=8 D=128 page 16, pages split over the GPUs",
            "n_gpus": world, "ms_per_step": res["step"], "local_kernel_ms": res["local_kernel"],
            "exchange_share": max(0.0, 1.0 - res["local_kernel"] / res["step"]) if world > 1 else 0.0,
            "exchange": "NCCL all-gather of Hq*(D+4) fp32 per rank + one combine launch" if world > 1 else "none (one GPU)",
            "value": bytes_alg / (res["step"] * 1e-3) / 1e9, "unit": "GB/s"}


def _time_ms(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_extras(device, pk):
    """The other configs of the spec, measured the same way (device-resident inputs, CUDA events):
    config 1 (fp32 dense causal), config 3 (sliding window) and config 5 (packed varlen fwd+bwd)."""
    import numpy as np

    import mlx_flashattention_steel_b200 as fa

    out = {}
    gd = torch.Generator(device=device).manual_seed(11)
    mk = lambda shape, dt: torch.randn(shape, generator=gd, device=device).to(dt)
    # config 1: B=1 H=8 N=S=1024 D=128 float32 causal
    q, k, v = (mk((1, 8, 1024, 128), torch.float32) for _ in range(3))
    ms = _time_ms(lambda: fa.flash_attention(q, k, v, causal=True), 20, 5)
    fl = 4.0 * 8 * 128 * (1024 * 1025 // 2)
    out["config1_fp32_causal"] = {"ms": ms, "tflops": fl / ms / 1e9, "kernel": "fa_fwd_f32 (FFMA)"}
    # config 3: B=2 H=16 N=S=32768 D=128 fp16 window (512, 0), causal
    q, k, v = (mk((2, 16, 32768, 128), torch.float16) for _ in range(3))
    ms = _time_ms(lambda: fa.flash_attention(q, k, v, causal=True, window_size=(512, 0)), 10, 3)
    pairs = sum(min(i + 1, 513) for i in range(32768))
    fl = 4.0 * 2 * 16 * 128 * pairs
    byts = 4 * q.numel() * 2
    out["config3_window512_fp16"] = {"ms": ms, "tflops": fl / ms / 1e9, "frac_tensor_peak": fl / ms / 1e9 / pk["tf"],
                                     "gbs": byts / ms / 1e6, "frac_hbm_peak": byts / ms / 1e6 / pk["hbm"]}
    # the same shape through a block mask (32 x 16 cells): the causal sliding-window builder switches on the cells a
    # +-512 window around each query block's centre touches; FLOPs are counted over the active cells
    bm = fa.make_sliding_window_mask(32768, 512, 128, causal=True, device=device)
    ms = _time_ms(lambda: fa.flash_attention_sparse(q, k, v, bm, causal=True), 10, 3)
    fl = 4.0 * 2 * 16 * 128 * float(bm.sum().item()) * 32 * 16
    out["sparse_window_mask_fp16"] = {"ms": ms, "active_cells": float(bm.float().mean().item()),
                                      "tflops_active_cells": fl / ms / 1e9, "kernel": "fa_fwd_sm100_kernel<128, f16, features>"}
    del q, k, v
    # head_dim 256, the reference's largest kernel size (its own table: causal forward, N = 8192): B=2 H=16 bf16
    q, k, v = (mk((2, 16, 8192, 256), torch.bfloat16) for _ in range(3))
    ms = _time_ms(lambda: fa.flash_attention(q, k, v, causal=True), 10, 3)
    fl = 4.0 * 2 * 16 * 256 * (8192 * 8193 // 2)
    out["head_dim256_causal_bf16"] = {"ms": ms, "tflops": fl / ms / 1e9, "frac_tensor_peak": fl / ms / 1e9 / pk["tf"],
                                      "kernel": "fa_fwd_sm100_kernel<256> (one CTA per SM)"}
    del q, k, v
    # config 5: packed varlen, 65536 tokens, lengths ~ U{128..4096}, H=16 D=64 bf16 causal, fwd + bwd
    rng = np.random.default_rng(5)
    lens = []
    while sum(lens) < 65536:
        lens.append(int(rng.integers(128, 4097)))
    lens[-1] -= sum(lens) - 65536
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=device)
    q, k, v, do = (mk((1, 16, 65536, 64), torch.bfloat16) for _ in range(4))
    pairs = sum(L * (L + 1) // 2 for L in lens)
    fl_fwd = 4.0 * 16 * 64 * pairs
    ms_f = _time_ms(lambda: fa.flash_attention_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=True), 10, 3)

    def fb():
        qg, kg, vg = q.detach().requires_grad_(True), k.detach().requires_grad_(True), v.detach().requires_grad_(True)
        fa.flash_attention_varlen(qg, kg, vg, cu, cu, max(lens), max(lens), causal=True).backward(do)

    ms_fb = _time_ms(fb, 10, 3)
    out["config5_varlen_bf16_d64"] = {"num_seqs": len(lens), "fwd_ms": ms_f, "fwd_tflops": fl_fwd / ms_f / 1e9,
                                      "fwd_bwd_ms": ms_fb, "fwd_bwd_tflops": 3.5 * fl_fwd / ms_fb / 1e9,
                                      "frac_tensor_peak": 3.5 * fl_fwd / ms_fb / 1e9 / pk["tf"]}
    del q, k, v, do
    # backward at head_dim 128: config 2's shape (B=4, Hq=32, Hkv=8, N=S=8192, bf16, causal), without and with its
    # soft cap; 2.5 x the forward's causal-adjusted FLOPs (five GEMMs), whatever the kernels recompute
    from mlx_flashattention_steel_b200 import attention as fa_attn
    q, k, v, do = mk((4, 32, 8192, 128), torch.bfloat16), mk((4, 8, 8192, 128), torch.bfloat16), \
        mk((4, 8, 8192, 128), torch.bfloat16), mk((4, 32, 8192, 128), torch.bfloat16)
    fl = 2.5 * prefill_flops(C2)
    bwd = {}
    for name, cap in (("plain", 0.0), ("softcap50", 50.0)):
        o_, l_ = fa_attn._fwd_raw(q, k, v, 128 ** -0.5, True, cap, -1, True, None)
        ms = _time_ms(lambda: fa_attn._bwd_raw(q, k, v, o_, l_, do, 128 ** -0.5, True, None, softcap=cap), 5, 3)
        bwd[name] = {"ms": ms, "tflops": fl / ms / 1e9, "frac_tensor_peak": fl / ms / 1e9 / pk["tf"]}
        del o_, l_
    bwd["kernels"] = "bwd_dkv_sm100_kernel + bwd_dq_sm100_kernel (tcgen05; 7 GEMMs executed for the 5 counted)"
    out["bwd_d128_dense"] = bwd
    del q, k, v, do
    # KV-cache write path (the producer of config 4's pools): 262144 new tokens x 8 kv heads x 128, bf16 in,
    # int8 + f16 scales out, into randomly placed pages filled in token order (what a prefill append looks like).
    # Algorithmic bytes = tokens read + values and scales written.
    T, H, D, bs = 262144, 8, 128, 16
    P = T // bs
    kn, vn = mk((T, H, D), torch.bfloat16), mk((T, H, D), torch.bfloat16)
    pages = torch.randperm(P, generator=gd, device=device).to(torch.int64)
    slots = (pages[:, None] * bs + torch.arange(bs, device=device)[None, :]).reshape(-1).contiguous()
    kp = torch.zeros((P, bs, H, D), dtype=torch.int8, device=device)
    vp = torch.zeros_like(kp)
    ks = torch.ones((P, bs, H), dtype=torch.float16, device=device)
    vs = torch.ones_like(ks)
    ms = _time_ms(lambda: fa.kv_append(kn, vn, slots, kp, vp, ks, vs), 10, 3)
    byts = 2.0 * T * H * (D * 2 + D + 2)
    out["kv_append_int8"] = {"tokens": T, "ms": ms, "gbs": byts / ms / 1e6, "frac_hbm_peak": byts / ms / 1e6 / pk["hbm"],
                             "kernel": "kv_append_kernel<bf16, int8>"}
    return out


def profile_case(name, device, steps, warmup):
    """Profiling aids (not bench values): small cases of the other kernels, sized for an ncu capture -- inputs larger
    than L2, well under a GB on the device, a few launches."""
    import numpy as np

    import mlx_flashattention_steel_b200 as fa
    from mlx_flashattention_steel_b200 import attention as fa_attn

    gd = torch.Generator(device=device).manual_seed(21)
    mk = lambda shape, dt: torch.randn(shape, generator=gd, device=device).to(dt)
    if name == "c3":          # config 3 reduced: B=1, H=2, N=S=32768, fp16, causal, window (512, 0)
        q, k, v = (mk((1, 2, 32768, 128), torch.float16) for _ in range(3))
        fn = lambda: fa.flash_attention(q, k, v, causal=True, window_size=(512, 0))
    elif name == "c5":        # config 5 reduced: 16384 packed tokens, lengths ~ U[128, 4096], H=16, D=64, bf16, fwd + bwd
        rng = np.random.default_rng(5)
        lens = []
        while sum(lens) < 16384:
            lens.append(int(rng.integers(128, 4097)))
        lens[-1] -= sum(lens) - 16384
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=device)
        q, k, v, do = (mk((1, 16, 16384, 64), torch.bfloat16) for _ in range(4))

        def fn():
            qg, kg, vg = (x.detach().requires_grad_(True) for x in (q, k, v))
            fa.flash_attention_varlen(qg, kg, vg, cu, cu, max(lens), max(lens), causal=True).backward(do)
    elif name == "bwd128":    # config 2's shape reduced: B=2, Hq=16, Hkv=4, N=S=8192, bf16, causal, backward only
        q, k, v, do = mk((2, 16, 8192, 128), torch.bfloat16), mk((2, 4, 8192, 128), torch.bfloat16), \
            mk((2, 4, 8192, 128), torch.bfloat16), mk((2, 16, 8192, 128), torch.bfloat16)
        o_, l_ = fa_attn._fwd_raw(q, k, v, 128 ** -0.5, True, 0.0, -1, True, None)
        fn = lambda: fa_attn._bwd_raw(q, k, v, o_, l_, do, 128 ** -0.5, True, None)
    elif name == "d256":      # head_dim 256 forward: B=1, H=16, N=S=8192, bf16, causal (201 MB of q, k, v, o)
        q, k, v = (mk((1, 16, 8192, 256), torch.bfloat16) for _ in range(3))
        fn = lambda: fa.flash_attention(q, k, v, causal=True)
    else:
        raise SystemExit(f"unknown --case {name}")
    ms = _time_ms(fn, steps, warmup)
    print(json.dumps({"note": f"--case {name}: profiling case, not a bench value", "ms_per_step": ms,
                      "kernel_status": int(fa.kernel_status())}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the config-4 decode measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip configs 1, 3 and 5")
    ap.add_argument("--small", action="store_true", help="profiling aid: N=S=4096, B=2 (not a bench value)")
    ap.add_argument("--case", default="", choices=["", "c3", "c5", "bwd128", "d256"],
                    help="profiling aid: run one small case of another kernel and exit (not a bench value)")
    ap.add_argument("--only-decode", type=int, default=0, metavar="B",
                    help="profiling aid: run only the decode measurement with batch B (not a bench value)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import mlx_flashattention_steel_b200 as fa

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    pk = peaks()
    if args.only_decode:
        print(json.dumps(bench_decode(device, args.steps, args.warmup, pk, batch=args.only_decode)), flush=True)
        return
    if args.case:
        profile_case(args.case, device, args.steps, args.warmup)
        return
    cfg = dict(C2)
    if args.small:
        cfg.update(B=2, N=4096, S=4096)
    q, k, v = make_prefill_inputs(cfg, device, seed=2 + rank)
    flops = prefill_flops(cfg)
    warm = max(args.warmup, 3)

    def step():
        return fa.flash_attention(q, k, v, causal=True, softcap=cfg["softcap"], return_lse=True)

    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    torch.cuda.synchronize()
    t_wall0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    ms_total = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms_total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
        dist.barrier()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ms = ms_total / args.steps
    tf_rank = flops / (ms * 1e-3) / 1e12
    value = tf_rank * world

    if args.small:
        print(json.dumps({"note": "--small profiling case, not a bench value", "ms_per_step": ms, "tflops": tf_rank}), flush=True)
        return

    # ---- end to end through the public API with pinned host buffers ----
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    hl = torch.empty(q.shape[:3], dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = ho.numel() * ho.element_size() + hl.numel() * 4

    # the public host-memory entry point: per-batch chunks pipelined over three streams, so the
    # host->device copy, the kernel and the device->host copy of neighbouring chunks overlap
    pipe = fa.HostPipeline(hq.shape, hk.shape, hq.dtype, device, chunk=1, depth=3, want_lse=True)

    # Consecutive steps are a stream of requests.  With join=False step i + 1's copies in run beside step i's copies out
    # (every step still copies all of its inputs in and its result out; the pipeline is joined before the closing
    # event); with join=True every call drains before the next.  Overlapping wins while the host link has duplex
    # headroom (one or two GPUs here); with more GPUs sharing the host's memory system it can lose, so both are timed
    # and the faster one (by the slowest rank) is the figure reported; the other rides along in the same object.
    e2e_steps = max(3, min(args.steps, 10))

    def timed(step_fn):
        for _ in range(2):
            step_fn()
        pipe.join()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0.record()
        for _ in range(e2e_steps):
            step_fn()
        pipe.join()
        e1.record()
        torch.cuda.synchronize()
        ms_ = e0.elapsed_time(e1) / e2e_steps
        if dist is not None:
            t = torch.tensor([ms_], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_ = float(t.item())
        return ms_

    def e2e_step(join):
        return lambda: fa.flash_attention_from_host(hq, hk, hv, out=ho, lse=hl, pipeline=pipe, return_lse=True,
                                                    causal=True, softcap=cfg["softcap"], join=join)

    e2e_by_mode = {"overlapped calls": timed(e2e_step(False)), "joined calls": timed(e2e_step(True))}
    e2e_mode = min(e2e_by_mode, key=e2e_by_mode.get)
    e2e_ms = e2e_by_mode[e2e_mode]
    e2e_val = flops / (e2e_ms * 1e-3) / 1e12 * world

    # the same pipeline, in the same mode, with the kernel launch left out, all ranks at once: what the host link and
    # the host's memory allow for these copies (the ceiling the end-to-end figure is to be read against)
    copy_ms = timed(lambda: pipe.run(hq, hk, hv, ho, hl, causal=True, softcap=cfg["softcap"], copies_only=True,
                                     join=(e2e_mode == "joined calls")))
    copy_ceiling_gbs = (h2d + d2h) * world / (copy_ms * 1e-3) / 1e9
    del hq, hk, hv, ho, hl, pipe

    decode = None
    if not args.no_decode and not args.small:
        try:
            decode = bench_decode(device, max(args.steps, 10), warm, pk, rank=rank, world=world, dist=dist)
        except NotImplementedError as e:  # decode kernel not built for this shape
            decode = {"unavailable": str(e)}
    del q, k, v
    strong = bench_strong(device, rank, world, dist, max(3, min(args.steps, 10)), warm)
    decode_long = bench_decode_long(device, rank, world, dist, 20, warm)
    extras = None
    if rank == 0 and world == 1 and not args.no_extras:
        extras = bench_extras(device, pk)
    if dist is not None:
        dist.barrier()

    if rank == 0:
        traffic_ratio = dram_traffic_ratio("fwd_sm100_config2_small")
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            tf, secs, sample = cpu_prefill_sample(C2, 2)
            cpu = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample,
                   "seconds": secs}
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            # traffic: dram bytes of one launch; the ncu capture was taken on a smaller case of the same kernel and is
            # scaled by the algorithmic bytes (q + k + v + o + lse) of this launch
            "roofline": {"bound": "tensor", "achieved": tf_rank, "peak": pk["tf"], "unit": "TFLOP/s",
                         "frac": tf_rank / pk["tf"],
                         "traffic": (traffic_ratio * (h2d + d2h)) if traffic_ratio else None, "peak_source": pk["src"],
                         "frac_of_sustained": (tf_rank / pk["tf_sustained"]) if pk.get("tf_sustained") else None,
                         "flops_per_launch": flops},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "copy_ceiling_gbs": copy_ceiling_gbs, "copies_only_ms_per_step": copy_ms,
                    "achieved_copy_gbs": (h2d + d2h) * world / (e2e_ms * 1e-3) / 1e9,
                    "frac_of_copy_ceiling": copy_ms / e2e_ms, "mode": e2e_mode,
                    "ms_per_step_by_mode": e2e_by_mode},
            "gpu_launches": args.steps,
            "kernel_status": int(fa.kernel_status()),       # 0 = no bounded wait inside a tcgen05 kernel gave up
            "clocks": clocks,
            "decode": decode,
            "strong": strong,
            "decode_long": decode_long,
            "extras": extras,
        }
        if args.small:
            line["note"] = "--small profiling case, not a bench value"
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
