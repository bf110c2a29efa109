// Blackwell backward, head_dim 128, part 1 of 2: dQ.  tcgen05 MMAs with TMEM accumulators, TMA-staged tiles.
//
// The reference splits its backward into a dQ kernel and a dK/dV kernel (csrc/mfa_steel_bwd.cpp:284-745 and
// 765-1293; dispatch csrc/mfa_attention.cpp:732-930); so does this path for head_dim 128, where one kernel holding
// S^T, dP^T, dV, dK and dQ would need 640 TMEM columns.  Each kernel recomputes P from the forward's lse.  dQ needs
// no atomics this way: every query tile is owned by one CTA, so the result is bit-reproducible.
//
// One CTA = 128 query rows of one query head; it walks the 64-key tiles those rows can see (causal / window tiles
// outside the band are skipped whole).  Per key tile j, three GEMMs with M = 128 query rows:
//   S(j)  = Q . K(j)^T      (SS, N = 64, K = 128)  -> TMEM S buffer j % 3
//   dP(j) = dO . V(j)^T     (SS, N = 64, K = 128)  -> TMEM dP buffer j % 3
//   8 compute warps (thread = query row; the two warps of a lane quarter split the 64 key columns) form
//   P = 2^(s - L) and dS = P o (dP - delta) [x (1 - tanh^2) under a soft cap] and write dS back as a 16-bit A operand
//   over the dP columns they came from.  There are two such sets of 8 warps, one for the even tiles and one for the
//   odd ones: a warp's step is a chain of latencies (barrier, TMEM load, arithmetic, TMEM store, arrive), and with
//   one set the tensor pipe was active a third of the time
//   dQ   += dS(j) . K(j)    (A from TMEM, B = K(j) as an MN-major operand, N = 128)  -> TMEM dQ
// Issue order SD(0) SD(1) dQ(0) SD(2) dQ(1) ...: the S / dP MMAs of the next tile are queued while the compute warps
// work on this one.
// Warp 16 is the TMA producer (Q and dO once, K and V tiles into a four-stage ring), one thread of warp 17
// issues the MMAs.  dQ leaves TMEM once, scaled, through shared memory (TMA store for the dense layout).
// TMEM (all 512 columns): [0,128) S0 S1, [128,256) dP0 dP1, [256,384) dQ, [384,512) Q and dO as A operands.  No load uses cluster multicast; every mbarrier wait is
// bounded and a timeout raises this file's status word (read through b200fa_kernel_status).
#include "common.cuh"
#include "launch.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace b200fa {
// Device status word of this file's kernels: bit 0 = a bounded wait gave up.
static __device__ int g_kernel_status = 0;

namespace {

constexpr int HD = 128;
constexpr int BM = 128;            // query rows per CTA
constexpr int BN = 64;             // keys per tile
constexpr int kStages = 4;         // K / V ring: tiles j .. j + 2 are in use at once, one more is in flight
constexpr int kBufs = 2;           // S / dP buffers in TMEM
constexpr int kThreads = 576;      // warps 0-7 compute (even tiles), 8-15 compute (odd tiles), 16 producer, 17 MMA issue
constexpr int kProducerWarp = 16, kMmaWarp = 17;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t cS = 0, cDP = 128, cDQ = 256;
// Q and dO rows as 16-bit A operands (two elements per column), copied from shared memory once per CTA: the S / dP
// MMAs then read only K / V from shared memory, whose bandwidth is what an SS MMA of this shape saturates
constexpr uint32_t cQA = 384, cDOA = 448;

constexpr int kQBytes = BM * HD * 2;        // 32768: [2 d-halves][128 rows][128 B]
constexpr int kKVBytes = BN * HD * 2;       // 16384: [2 d-halves][64 rows][128 B]
constexpr int kStageBytes = 2 * kKVBytes;   // K then V
constexpr int kSmemTiles = 2 * kQBytes + kStages * kStageBytes;
constexpr int kSmemBytes = kSmemTiles + 256 + 1024;

enum Bar {
  BAR_Q = 0,
  BAR_KV_FULL = 1,          // + stage
  BAR_KV_EMPTY = 5,         // + stage: a compute warp has seen the dQ MMAs of the tile (the last readers of its K, V) complete
  BAR_SD_FULL = 9,          // + buffer: S and dP of a tile are complete
  BAR_DS_READY = 12,        // + buffer: count 8, the compute warps have written dS
  BAR_DQ_FINAL = 15,
  BAR_STAGED = 16,          // count 16: the compute warps have staged their dQ rows in shared memory
  BAR_QA_READY = 17,        // count 16: Q and dO sit in TMEM
  BAR_COUNT = 18
};

struct DqArgs {
  BwdParams p;
  int tma_store;
};

template <int DT> __device__ __forceinline__ uint32_t pack16q(float a, float b) {
  return DT == 0 ? Elem<__half>::pack(a, b) : Elem<__nv_bfloat16>::pack(a, b);
}

// CAP (soft cap) and WIN (left window) are compile-time variants: the plain kernel's loops carry neither.  FEAT: the
// ALiBi bias and / or a block mask (cells of 16, 32 or 64 keys), without CAP / WIN.
template <int DT, bool CAP, bool WIN, bool FEAT>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmDQ, const DqArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;
  unsigned char* sDO = sQ + kQBytes;
  unsigned char* sKV = sDO + kQBytes;                       // [stage][K | V]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

  const BwdParams& p = a.p;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;
  int batch = blockIdx.z;
  const int kvh = head / p.gqa;
  int N = p.N, S = p.S, q_begin = 0, k_begin = 0;
  if (p.cu_q != nullptr) {
    q_begin = p.cu_q[batch];
    N = p.cu_q[batch + 1] - q_begin;
    k_begin = p.cu_k[batch];
    S = p.cu_k[batch + 1] - k_begin;
    batch = 0;
  }
  const int q0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * BM;   // heavy (late) tiles first
  if (q0 >= N) return;
  const int off = S - N;
  int k_hi = S;
  if (p.causal) k_hi = min(S, q0 + BM + off);
  int k_lo = 0;
  if constexpr (WIN) k_lo = max(0, q0 + off - p.window_left);
  const int kt_begin = k_lo / BN;
  const int kt_end = k_hi > 0 ? (k_hi + BN - 1) / BN : 0;
  const int n_tiles = kt_end - kt_begin;

  if (n_tiles <= 0) {
    // no visible key for any row of this tile: dQ = 0
    if (warp < 4) {
      const int row = q0 + tid;
      if (row < N) {
        uint4* drow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dq) + batch * p.dq_bs + head * p.dq_hs +
                                               static_cast<int64_t>(q_begin + row) * p.dq_rs);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) drow[i] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }

  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };
  auto load_kv = [&](int j) {
    const int st = j % kStages;
    unsigned char* dst = sKV + st * kStageBytes;
    mbar_arrive_expect_tx(bar(BAR_KV_FULL + st), kStageBytes);
    const int row = k_begin + (kt_begin + j) * BN;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      tma_load_4d(smem_u32(dst + hf * (kKVBytes / 2)), &tmK, bar(BAR_KV_FULL + st), 64 * hf, row, kvh, batch);
      tma_load_4d(smem_u32(dst + kKVBytes + hf * (kKVBytes / 2)), &tmV, bar(BAR_KV_FULL + st), 64 * hf, row, kvh, batch);
    }
  };
  if (warp == kProducerWarp && lane == 0) {
    mbar_init(bar(BAR_Q), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(BAR_KV_FULL + s), 1);
      mbar_init(bar(BAR_KV_EMPTY + s), 1);
    }
    for (int b = 0; b < kBufs; ++b) {
      mbar_init(bar(BAR_SD_FULL + b), 1);
      mbar_init(bar(BAR_DS_READY + b), 8);
    }
    mbar_init(bar(BAR_DQ_FINAL), 1);
    mbar_init(bar(BAR_STAGED), 16);
    mbar_init(bar(BAR_QA_READY), 16);
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async();
    mbar_arrive_expect_tx(bar(BAR_Q), 2 * kQBytes);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      tma_load_4d(smem_u32(sQ + hf * (kQBytes / 2)), &tmQ, bar(BAR_Q), 64 * hf, q_begin + q0, head, batch);
      tma_load_4d(smem_u32(sDO + hf * (kQBytes / 2)), &tmDO, bar(BAR_Q), 64 * hf, q_begin + q0, head, batch);
    }
    for (int j = 0; j < kStages && j < n_tiles; ++j) load_kv(j);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp == kProducerWarp) {
    // ============================ producer ============================
    if (lane == 0) {
      for (int j = kStages; j < n_tiles; ++j) {
        // the stage's previous tile t = j - kStages is free when its dQ MMAs have completed; a compute warp says so
        // when it sees the commit that follows them (the one that carries S / dP of tile t + 2).  The producer is at
        // most one completion behind that barrier: the stage is released again only after tile j has been used
        if (!mbar_wait_bounded(bar(BAR_KV_EMPTY + j % kStages), ((j / kStages) & 1) ^ 1, s_abort)) break;
        load_kv(j);
      }
    }
  } else if (warp == kMmaWarp) {
    // ============================ MMA issue ============================
    if (lane == 0) {
      const uint32_t id_sd = instr_desc(DT, 0, BM, BN);          // S, dP: B K-major, N = 64
      const uint32_t id_dq = instr_desc(DT, 1, BM, HD);          // dQ: B = K MN-major, N = 128
      const uint64_t kd0 = smem_desc(smem_u32(sKV), 16, 1024);
      const uint64_t kmn0 = smem_desc(smem_u32(sKV), kKVBytes / 2, 1024);
      constexpr uint64_t kHalfK = (kKVBytes / 2) >> 4, kStageU = kStageBytes >> 4, kVOff = kKVBytes >> 4;
      bool ok = mbar_wait_bounded(bar(BAR_QA_READY), 0, s_abort);
      tc_fence_after();
      // S(j), dP(j) into buffer j & 1.  `landed`: the tile's K / V are known to have landed (the compute warps checked
      // before they handed over dS(j - 2)); the first two tiles wait here
      auto issue_sd = [&](int j, bool landed) -> bool {
        const int st = j % kStages, b = j % kBufs;
        if (!landed) {
          if (!mbar_wait_bounded(bar(BAR_KV_FULL + st), (j / kStages) & 1, s_abort)) return false;
          tc_fence_after();
        }
        const uint64_t kd = kd0 + static_cast<uint64_t>(st) * kStageU, vd = kd + kVOff;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ts(tmem + cS + 64 * b, tmem + cQA + k * 8, kd + (k >> 2) * kHalfK + (k & 3) * 2, id_sd, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ts(tmem + cDP + 64 * b, tmem + cDOA + k * 8, vd + (k >> 2) * kHalfK + (k & 3) * 2, id_sd, k > 0 ? 1u : 0u);
        return true;
      };
      for (int j = 0; j < kBufs && j < n_tiles && ok; ++j) {
        ok = issue_sd(j, false);
        if (ok) tc_commit(bar(BAR_SD_FULL + j));
      }
      // One wait and one commit per tile: dQ(j), then S / dP of tile j + 2 into the buffer whose dS those MMAs have
      // just read (the pipe runs in order), then one commit that both hands tile j + 2 to the compute warps and
      // releases tile j's K / V stage to the producer.
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % kStages, b = j % kBufs;
        if (!mbar_wait_bounded(bar(BAR_DS_READY + b), (j / kBufs) & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        const uint64_t kmn = kmn0 + static_cast<uint64_t>(st) * kStageU;
        // A = dS in TMEM: 16 keys = 8 columns; keys 0-31 of the tile at +0, 32-63 at +32 (where the two warps of a
        // row wrote them).  B = K rows = keys: 16 rows = 2048 B = 128 units.
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          mma_ts(tmem + cDQ, tmem + cDP + 64 * b + (k >> 1) * 32 + (k & 1) * 8, kmn + k * 128, id_dq,
                 (j > 0 || k > 0) ? 1u : 0u);
        if (j + kBufs < n_tiles) issue_sd(j + kBufs, true);
        tc_commit(bar(BAR_SD_FULL + b));
        if (j + 1 == n_tiles) tc_commit(bar(BAR_DQ_FINAL));
      }
    }
  } else {
    // ============================ compute warps 0-15 ============================
    const int wq = warp & 3, hf = (warp >> 2) & 1, set = warp >> 3;   // TMEM lane quarter, key-column half, tile parity
    const int rloc = wq * 32 + lane;
    const int row = q0 + rloc;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    // -L and -delta of this thread's row; rows beyond N or without any visible key get P = 0 (exp2 of -inf)
    float nL = -INFINITY, nD = 0.f;
    if (row < N) {
      const int64_t idx = batch * p.lse_bs + head * p.lse_hs + q_begin + row;
      const float L = p.lse[idx];
      nL = (L == -INFINITY) ? -INFINITY : -L;
      nD = -p.delta[idx];
    }
    const float cap_in = CAP ? p.scale / p.softcap : 0.f, cap_out = p.softcap * kLog2e;
    const bool precise_tanh = p.softcap >= kPreciseTanhMinCap;
    const float2 c2 = make_float2(p.scale_log2, p.scale_log2), nL2 = make_float2(nL, nL), nD2 = make_float2(nD, nD);
    const float alibi_l2 = (FEAT && p.alibi != nullptr) ? p.alibi[head] * kLog2e : 0.f;
    const bool masked_cells = FEAT && p.bmask != nullptr;
    const int cell_sh = masked_cells ? (p.bm_bk == 16 ? 4 : (p.bm_bk == 32 ? 5 : 6)) : 6;
    const uint8_t* mask_row = masked_cells ? p.bmask + static_cast<int64_t>(min(row, N - 1) / p.bm_bq) * p.bm_nk : nullptr;
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q), 0, s_abort));
    if (ok) {
      // this row's 128 bytes of d-half hf of Q (set 0) or dO (set 1) -> 32 TMEM columns of the A operand
      const uint32_t rowa = smem_u32(set == 0 ? sQ : sDO) + hf * (kQBytes / 2) + rloc * 128;
      uint32_t qr[32];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(qr[4 * c]), "=r"(qr[4 * c + 1]), "=r"(qr[4 * c + 2]), "=r"(qr[4 * c + 3])
                     : "r"(rowa + static_cast<uint32_t>((c ^ (rloc & 7)) << 4))
                     : "memory");
      tmem_st32(tmem + lane_base + (set == 0 ? cQA : cDOA) + hf * 32, qr);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_QA_READY));
    }
    for (int j = set; j < n_tiles && ok; j += 2) {
      const int b = j % kBufs;
      const int k0 = (kt_begin + j) * BN + hf * 32;            // first key of this thread's 32 columns
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_SD_FULL + b), (j / kBufs) & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      // the commit just seen followed dQ(j - 2): that tile's K / V stage can be refilled
      if (j >= kBufs && wq == 0 && hf == 0 && lane == 0) mbar_arrive(bar(BAR_KV_EMPTY + (j - kBufs) % kStages));
      // FEAT: bit c = mask cell c of this row under the 32 keys from k0 (two cells of 16 keys, else one); the bias of
      // key k0 for this row, in the log2 domain
      unsigned cells = 3u;
      float ab = 0.f;
      if constexpr (FEAT) {
        if (masked_cells) {
          const int cb0 = k0 >> cell_sh;
          cells = (cb0 < p.bm_nk && mask_row[cb0] != 0) ? 1u : 0u;
          if (cell_sh == 4) cells |= (cb0 + 1 < p.bm_nk && mask_row[cb0 + 1] != 0) ? 2u : 0u;
          else cells |= cells << 1;
        }
        ab = alibi_l2 * static_cast<float>(k0 - (row + off));
      }
      uint32_t rs[32], rd[32];
      tmem_ld32(tmem + lane_base + cS + 64 * b + hf * 32, rs);
      tmem_ld32(tmem + lane_base + cDP + 64 * b + hf * 32, rd);
      tc_wait_ld();
      // visible keys of this row, relative to k0: [lo_rel, hi_rel]
      const int hi_rel = (p.causal ? min(S - 1, row + off) : S - 1) - k0;
      const int lo_rel = WIN ? row + off - p.window_left - k0 : 0;
      const bool need_mask = __any_sync(0xffffffffu, hi_rel < 31 || (WIN && lo_rel > 0));
      uint32_t pd[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 sv = make_float2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1]));
        const float2 dv = make_float2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1]));
        float2 t, dcap;
        if constexpr (CAP) {
          const float2 th = make_float2(cap_tanh(sv.x * cap_in, precise_tanh), cap_tanh(sv.y * cap_in, precise_tanh));
          t = __ffma2_rn(th, make_float2(cap_out, cap_out), nL2);
          dcap = __ffma2_rn(make_float2(-th.x, -th.y), th, make_float2(1.f, 1.f));
        } else {
          t = __ffma2_rn(sv, c2, nL2);
        }
        if constexpr (FEAT) {
          t = __fadd2_rn(t, make_float2(fmaf(alibi_l2, static_cast<float>(i), ab), fmaf(alibi_l2, static_cast<float>(i + 1), ab)));
        }
        float2 pe = make_float2(fast_exp2(t.x), fast_exp2(t.y));
        if constexpr (FEAT) {
          if (!((cells >> (i >> 4)) & 1u)) pe = make_float2(0.f, 0.f);     // keys i, i + 1 share a 16-key cell
        }
        if (need_mask) {
          if (i > hi_rel || (WIN && i < lo_rel)) pe.x = 0.f;
          if (i + 1 > hi_rel || (WIN && i + 1 < lo_rel)) pe.y = 0.f;
        }
        float2 dsv = __fmul2_rn(pe, __fadd2_rn(dv, nD2));
        if constexpr (CAP) dsv = __fmul2_rn(dsv, dcap);
        pd[i >> 1] = pack16q<DT>(dsv.x, dsv.y);
      }
      // dS goes back as 16-bit pairs along the key index, inside the 32 columns this warp has just read
      tmem_st16(tmem + lane_base + cDP + 64 * b + hf * 32, pd);
      tc_wait_st();
      // the MMA thread issues S / dP of tile j + 2 right behind dQ(j) without a wait of its own: see that tile's
      // K / V land before handing over dS(j)
      if (j + kBufs < n_tiles) {
        const int jn = j + kBufs;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_KV_FULL + jn % kStages), (jn / kStages) & 1, s_abort))) { ok = false; break; }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_DS_READY + b));
    }

    // ---- epilogue: dQ * scale -> 16-bit, through shared memory (the Q / dO tiles are free: every MMA has completed) ----
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DQ_FINAL), 0, s_abort));
    if (ok) {
      tc_fence_after();
      // this warp's 32 of the 128 columns: d-half hf, 32-column half `set` of it; staged as [d-half][row][128 B],
      // 16-byte chunks swizzled by row
      {
        const int c = set;
        uint32_t o[32];
        tmem_ld32(tmem + lane_base + cDQ + hf * 64 + c * 32, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack16q<DT>(__uint_as_float(o[i]) * p.scale, __uint_as_float(o[i + 1]) * p.scale);
          v.y = pack16q<DT>(__uint_as_float(o[i + 2]) * p.scale, __uint_as_float(o[i + 3]) * p.scale);
          v.z = pack16q<DT>(__uint_as_float(o[i + 4]) * p.scale, __uint_as_float(o[i + 5]) * p.scale);
          v.w = pack16q<DT>(__uint_as_float(o[i + 6]) * p.scale, __uint_as_float(o[i + 7]) * p.scale);
          const int chunk = c * 4 + (i >> 3);
          if (a.tma_store) {
            *reinterpret_cast<uint4*>(sQ + hf * (kQBytes / 2) + rloc * 128 + ((chunk ^ (rloc & 7)) << 4)) = v;
          } else if (row < N) {
            uint16_t* drow = reinterpret_cast<uint16_t*>(p.dq) + batch * p.dq_bs + head * p.dq_hs +
                             static_cast<int64_t>(q_begin + row) * p.dq_rs;
            *reinterpret_cast<uint4*>(drow + hf * 64 + chunk * 8) = v;
          }
        }
      }
      if (a.tma_store) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_STAGED));
        if (tid == 0 && mbar_wait_bounded(bar(BAR_STAGED), 0, s_abort)) {
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2)
            tma_store_4d(&tmDQ, smem_u32(sQ + h2 * (kQBytes / 2)), 64 * h2, q0, head, batch);
          tma_store_commit();
          tma_store_wait<0>();
        }
      }
    }
  }

  // ---- teardown ----
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && *s_abort != 0) atomicOr(&g_kernel_status, 1);
}

bool make_map128(CUtensorMap* m, int dtype, const void* base, int rows, int H, int B, int64_t rs, int64_t hs, int64_t bs,
                 int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(rows), static_cast<uint64_t>(H),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(rs) * 2, static_cast<uint64_t>(hs) * 2, static_cast<uint64_t>(bs) * 2};
  const uint32_t box[4] = {64, static_cast<uint32_t>(box_rows), 1, 1};
  return encode_tmap(m, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims,
                     strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

// dQ for head_dim 128; p.delta must already hold delta.  Dense: nbatch = B, max_q = N.  Packed varlen: nbatch =
// number of sequences, max_q = the longest query sequence.
cudaError_t launch_bwd_dq_sm100(const BwdParams& p, int dtype, int nbatch, int max_q, cudaStream_t stream) {
  if (nbatch <= 0 || max_q <= 0) return cudaSuccess;
  CUtensorMap tmQ, tmK, tmV, tmDO, tmDQ;
  auto fix = [](int64_t s, int64_t fallback) { return s > 0 ? s : fallback; };   // size-1 dimensions only (see bwd_sm100_strides_ok)
  const int64_t q_hs = fix(p.q_hs, static_cast<int64_t>(p.N) * p.q_rs), q_bs = fix(p.q_bs, q_hs * p.Hq);
  const int64_t k_hs = fix(p.k_hs, static_cast<int64_t>(p.S) * p.k_rs), k_bs = fix(p.k_bs, k_hs * p.Hkv);
  const int64_t v_hs = fix(p.v_hs, static_cast<int64_t>(p.S) * p.v_rs), v_bs = fix(p.v_bs, v_hs * p.Hkv);
  const int64_t do_hs = static_cast<int64_t>(p.N) * HD, do_bs = do_hs * p.Hq;
  if (!make_map128(&tmQ, dtype, p.q, p.N, p.Hq, p.B, p.q_rs, q_hs, q_bs, BM) ||
      !make_map128(&tmK, dtype, p.k, p.S, p.Hkv, p.B, p.k_rs, k_hs, k_bs, BN) ||
      !make_map128(&tmV, dtype, p.v, p.S, p.Hkv, p.B, p.v_rs, v_hs, v_bs, BN) ||
      !make_map128(&tmDO, dtype, p.dout, p.N, p.Hq, p.B, HD, do_hs, do_bs, BM))
    return cudaErrorInvalidValue;
  DqArgs a;
  a.p = p;
  a.tma_store = (p.cu_q == nullptr && make_map128(&tmDQ, dtype, p.dq, p.N, p.Hq, p.B, p.dq_rs, fix(p.dq_hs, 1), fix(p.dq_bs, 1), BM)) ? 1 : 0;
  if (!a.tma_store) tmDQ = tmQ;
  dim3 grid((max_q + BM - 1) / BM, p.Hq, nbatch);
  auto launch = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    kern<<<grid, kThreads, kSmemBytes, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, a);
    return cudaGetLastError();
  };
  const bool cap = p.softcap > 0.f, win = p.window_left >= 0, feat = p.alibi != nullptr || p.bmask != nullptr;
  if (feat) return dtype == 0 ? launch(bwd_dq_sm100_kernel<0, false, false, true>) : launch(bwd_dq_sm100_kernel<1, false, false, true>);
  if (dtype == 0) {
    if (cap) return win ? launch(bwd_dq_sm100_kernel<0, true, true, false>) : launch(bwd_dq_sm100_kernel<0, true, false, false>);
    return win ? launch(bwd_dq_sm100_kernel<0, false, true, false>) : launch(bwd_dq_sm100_kernel<0, false, false, false>);
  }
  if (cap) return win ? launch(bwd_dq_sm100_kernel<1, true, true, false>) : launch(bwd_dq_sm100_kernel<1, true, false, false>);
  return win ? launch(bwd_dq_sm100_kernel<1, false, true, false>) : launch(bwd_dq_sm100_kernel<1, false, false, false>);
}

cudaError_t bwd_dq_sm100_read_clear_status(cudaStream_t stream, int* out) {
  const int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_kernel_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess && *out != 0)
    e = cudaMemcpyToSymbolAsync(g_kernel_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return e;
}

}  // namespace b200fa
