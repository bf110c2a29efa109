// Blackwell backward, head_dim 128, part 1 of 2: dQ.  tcgen05 MMAs with TMEM accumulators, TMA-staged tiles.
//
// The reference splits its backward into a dQ kernel and a dK/dV kernel (csrc/mfa_steel_bwd.cpp:284-745 and
// 765-1293; dispatch csrc/mfa_attention.cpp:732-930); so does this path for head_dim 128, where one kernel holding
// S^T, dP^T, dV, dK and dQ would need 640 TMEM columns.  Each kernel recomputes P from the forward's lse.  dQ needs
// no atomics this way: every query tile is owned by one CTA, so the result is bit-reproducible.
//
// One CTA = 128 query rows of one query head; it walks the 128-key tiles those rows can see (causal / window tiles
// outside the band are skipped whole).  Per key tile j, three GEMMs with M = 128 query rows, all of them N = 128
// (an N = 64 MMA of this shape takes 1.5x its share of the tensor pipe):
//   S(j)  = Q . K(j)^T      (A = Q in TMEM, B = K(j) K-major)   -> TMEM S
//   dP(j) = dO . V(j)^T     (A = dO in shared memory, B = V(j) K-major)  -> TMEM dP
//   dQ   += dS(j) . K(j)    (A = dS in TMEM, B = K(j) as an MN-major operand)  -> TMEM dQ
// S and dP have one buffer each, and 16 compute warps (thread = query row, a warp = 32 rows x 32 keys) work on a
// tile in two phases so that neither buffer is held long:
//   phase A  load S(j) into registers (S is free for tile j + 2 from here on: S_FREE), P' = 2^(s - L) [x (1 - tanh^2)]:
//            bound by the special-function unit
//   phase B  load dP(j) into registers (dP is free for tile j + 1: DP_FREE), dS = P' o (dP - delta), written as a
//            16-bit A operand into columns of its own (DS_READY)
// Each arrival releases one group of MMAs: dP(j+1) on DP_FREE(j), dQ(j) on DS_READY(j), S(j+2) on S_FREE(j+1).
// Nothing on the tensor pipe waits for the compute warps' arithmetic.  The three groups write disjoint accumulators
// and a tcgen05.commit tracks the MMAs of the thread that executes it, so each group has an issuing thread of its
// own (one lane of warps 17, 18, 19): in place a thread spends about 96 clocks per MMA it issues, waits included,
// against the pipe's 64, and three threads keep the pipe fed where one does not.
// Warp 16 is the TMA producer (Q and dO once; K tiles into a four-stage ring, V tiles into a two-stage ring).
// Q passes through the last K stage into TMEM (a 16-bit A operand); dO stays in
// shared memory (the dP MMAs are SS: TMEM has no room for it beside dS).  dQ leaves TMEM once, scaled, through
// shared memory (TMA store for the dense layout).
// TMEM (all 512 columns): [0,128) S, [128,256) dP, [256,384) dQ, [384,448) Q, [448,512) dS.  No load uses cluster
// multicast; every mbarrier wait is bounded and a timeout raises this file's status word (read through
// b200fa_kernel_status).
#include <type_traits>

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
constexpr int BN = 128;            // keys per tile
constexpr int kKStages = 4;        // K(j) is read by S(j) two tiles before dQ(j): three tiles in use, one in flight
constexpr int kVStages = 2;        // V(j) is read once, by dP(j)
constexpr int kThreads = 640;      // warps 0-15 compute, 16 producer, 17 / 18 / 19 MMA issue (dP / S / dQ)
constexpr int kProducerWarp = 16, kMmaWarp = 17, kMmaWarpS = 18, kMmaWarpQ = 19;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t cS = 0, cDP = 128, cDQ = 256;
// Q rows as a 16-bit A operand (two elements per column), copied from shared memory once per CTA; dS of the current
// tile, 16 keys per 8 columns
constexpr uint32_t cQA = 384, cDS = 448;

constexpr int kTileBytes = BN * HD * 2;     // 32768: [2 d-halves][128 rows][128 B]; Q and dO tiles have the same shape
constexpr int kSmemTiles = (kKStages + kVStages + 1) * kTileBytes;     // + dO
constexpr int kSmemBytes = kSmemTiles + 256 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory");

enum Bar {
  BAR_Q = 0,                // Q and dO have landed
  BAR_K_FULL = 1,           // + stage (4)
  BAR_V_FULL = 5,           // + stage (2)
  BAR_K_FREE = 7,           // + stage: a compute warp has seen dQ of the stage's tile complete
  BAR_V_FREE = 11,          // + stage: a compute warp has seen dP of the stage's tile complete
  BAR_S_FULL = 13,          // S of a tile is complete
  BAR_DP_FULL = 14,         // dP of a tile is complete
  BAR_DQ_DONE = 15,         // the dQ MMAs of a tile are complete: its dS columns and its K stage are free
  BAR_S_FREE = 16,          // count 16: the compute warps hold S in registers
  BAR_DP_FREE = 17,         // count 16: the compute warps hold dP in registers
  BAR_DS_READY = 18,        // count 16: the compute warps have written dS
  BAR_STAGED = 19,          // count 16: the compute warps have staged their dQ rows in shared memory
  BAR_QA_READY = 20,        // count 16: Q sits in TMEM
  BAR_COUNT = 21
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
  unsigned char* sK = smem;                                 // [stage] K tiles
  unsigned char* sV = sK + kKStages * kTileBytes;           // [stage] V tiles
  unsigned char* sDO = sV + kVStages * kTileBytes;          // dO, resident: the A operand of the dP MMAs
  unsigned char* sQ = sK + (kKStages - 1) * kTileBytes;     // Q passes through the last K stage
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
  auto load_k = [&](int j) {
    const int st = j % kKStages;
    unsigned char* dst = sK + st * kTileBytes;
    mbar_arrive_expect_tx(bar(BAR_K_FULL + st), kTileBytes);
    const int row = k_begin + (kt_begin + j) * BN;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
      tma_load_4d(smem_u32(dst + hf * (kTileBytes / 2)), &tmK, bar(BAR_K_FULL + st), 64 * hf, row, kvh, batch);
  };
  auto load_v = [&](int j) {
    const int st = j % kVStages;
    unsigned char* dst = sV + st * kTileBytes;
    mbar_arrive_expect_tx(bar(BAR_V_FULL + st), kTileBytes);
    const int row = k_begin + (kt_begin + j) * BN;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
      tma_load_4d(smem_u32(dst + hf * (kTileBytes / 2)), &tmV, bar(BAR_V_FULL + st), 64 * hf, row, kvh, batch);
  };
  if (warp == kProducerWarp && lane == 0) {
    mbar_init(bar(BAR_Q), 1);
    for (int st = 0; st < kKStages; ++st) mbar_init(bar(BAR_K_FULL + st), 1);
    for (int st = 0; st < kVStages; ++st) mbar_init(bar(BAR_V_FULL + st), 1);
    for (int st = 0; st < kKStages; ++st) mbar_init(bar(BAR_K_FREE + st), 1);
    for (int st = 0; st < kVStages; ++st) mbar_init(bar(BAR_V_FREE + st), 1);
    mbar_init(bar(BAR_S_FULL), 1);
    mbar_init(bar(BAR_DP_FULL), 1);
    mbar_init(bar(BAR_DQ_DONE), 1);
    mbar_init(bar(BAR_S_FREE), 16);
    mbar_init(bar(BAR_DP_FREE), 16);
    mbar_init(bar(BAR_DS_READY), 16);
    mbar_init(bar(BAR_STAGED), 16);
    mbar_init(bar(BAR_QA_READY), 16);
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async();
    mbar_arrive_expect_tx(bar(BAR_Q), 2 * kTileBytes);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      tma_load_4d(smem_u32(sQ + hf * (kTileBytes / 2)), &tmQ, bar(BAR_Q), 64 * hf, q_begin + q0, head, batch);
      tma_load_4d(smem_u32(sDO + hf * (kTileBytes / 2)), &tmDO, bar(BAR_Q), 64 * hf, q_begin + q0, head, batch);
    }
    for (int j = 0; j < kKStages - 1 && j < n_tiles; ++j) load_k(j);
    for (int j = 0; j < kVStages && j < n_tiles; ++j) load_v(j);
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
      // the stage Q came through joins the K ring once Q sits in TMEM
      bool ok = true;
      if (n_tiles > kKStages - 1) {
        ok = mbar_wait_bounded(bar(BAR_QA_READY), 0, s_abort);
        if (ok) load_k(kKStages - 1);
      }
      // In time order: V(e)'s stage is released in phase B of tile e, K(e - 1)'s in phase B of tile e (when dQ(e - 1)
      // is seen complete).  Each barrier's next completion needs the tile loaded here, so the producer is never
      // more than one completion behind.
      for (int e = 0; e < n_tiles && ok; ++e) {
        if (e + kVStages < n_tiles) {
          ok = mbar_wait_bounded(bar(BAR_V_FREE + e % kVStages), (e / kVStages) & 1, s_abort);
          if (!ok) break;
          load_v(e + kVStages);
        }
        if (e >= 1 && e - 1 + kKStages < n_tiles) {
          ok = mbar_wait_bounded(bar(BAR_K_FREE + (e - 1) % kKStages), ((e - 1) / kKStages) & 1, s_abort);
          if (!ok) break;
          load_k(e - 1 + kKStages);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ============================ MMA issue ============================
    if (lane == 0) {
      const uint32_t id_sd = instr_desc(DT, 0, BM, BN);          // S, dP: B K-major, N = 128 keys
      const uint32_t id_dq = instr_desc(DT, 1, BM, HD);          // dQ: B = K MN-major, N = 128 = head_dim
      const uint64_t kd0 = smem_desc(smem_u32(sK), 16, 1024);
      const uint64_t vd0 = smem_desc(smem_u32(sV), 16, 1024);
      const uint64_t dod = smem_desc(smem_u32(sDO), 16, 1024);
      const uint64_t kmn0 = smem_desc(smem_u32(sK), kTileBytes / 2, 1024);
      constexpr uint64_t kHalf = (kTileBytes / 2) >> 4, kTileU = kTileBytes >> 4;
      auto issue_dp = [&](int j) {
        const uint64_t vd = vd0 + static_cast<uint64_t>(j % kVStages) * kTileU;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ss(tmem + cDP, dod + (k >> 2) * kHalf + (k & 3) * 2, vd + (k >> 2) * kHalf + (k & 3) * 2, id_sd, k > 0 ? 1u : 0u);
        tc_commit(bar(BAR_DP_FULL));
      };
      // The first V tile is waited for here (BAR_Q, behind QA_READY, also covers dO); every later one by the compute
      // warps, before the arrival that lets its MMAs be issued.
      bool ok = mbar_wait_bounded(bar(BAR_QA_READY), 0, s_abort) && mbar_wait_bounded(bar(BAR_V_FULL + 0), 0, s_abort);
      if (ok) {
        tc_fence_after();
        issue_dp(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          // every warp holds dP(j) in registers (and has seen V(j + 1) land)
          if (!mbar_wait_bounded(bar(BAR_DP_FREE), j & 1, s_abort)) { ok = false; break; }
          tc_fence_after();
          issue_dp(j + 1);
        }
      }
    }
  } else if (warp == kMmaWarpQ) {
    // ============================ MMA issue: dQ ============================
    if (lane == 0) {
      const uint32_t id_dq = instr_desc(DT, 1, BM, HD);          // dQ: B = K MN-major, N = 128 = head_dim
      const uint64_t kmn0 = smem_desc(smem_u32(sK), kTileBytes / 2, 1024);
      constexpr uint64_t kTileU = kTileBytes >> 4;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (!mbar_wait_bounded(bar(BAR_DS_READY), j & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        const uint64_t kmn = kmn0 + static_cast<uint64_t>(j % kKStages) * kTileU;
        // A = dS in TMEM: 16 keys = 8 columns.  B = K rows = keys: 16 rows = 2048 B = 128 units.
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          mma_ts(tmem + cDQ, tmem + cDS + k * 8, kmn + k * 128, id_dq, (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(bar(BAR_DQ_DONE));
      }
    }
  } else if (warp == kMmaWarpS) {
    // ============================ MMA issue: S ============================
    // A second issuing thread: S(j + 2) depends on nothing the other thread issues (its buffer is freed by S_FREE,
    // its commit tracks its own MMAs), and its waits and issues overlap the other thread's.
    if (lane == 0) {
      const uint32_t id_sd = instr_desc(DT, 0, BM, BN);
      const uint64_t kd0 = smem_desc(smem_u32(sK), 16, 1024);
      constexpr uint64_t kHalf = (kTileBytes / 2) >> 4, kTileU = kTileBytes >> 4;
      auto issue_s = [&](int j) {
        const uint64_t kd = kd0 + static_cast<uint64_t>(j % kKStages) * kTileU;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ts(tmem + cS, tmem + cQA + k * 8, kd + (k >> 2) * kHalf + (k & 3) * 2, id_sd, k > 0 ? 1u : 0u);
        tc_commit(bar(BAR_S_FULL));
      };
      // the first two K tiles are waited for here, every later one by the compute warps before S_FREE
      bool ok = mbar_wait_bounded(bar(BAR_QA_READY), 0, s_abort) && mbar_wait_bounded(bar(BAR_K_FULL + 0), 0, s_abort);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 1; j < n_tiles && ok; ++j) {
        // every warp holds S(j - 1) in registers (and has seen K(j) land)
        if (!mbar_wait_bounded(bar(BAR_S_FREE), (j - 1) & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        issue_s(j);
      }
    }
  } else if (warp < 16) {
    // ============================ compute warps 0-15 ============================
    const int wq = warp & 3, cq = warp >> 2;          // TMEM lane quarter (rows), 32-key column quarter of a tile
    const int hf = cq & 1, set = cq >> 1;              // for the Q copy: d-half; warps of set 0 copy
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
    const SmallCap sc = CAP ? small_cap_consts(p.scale, p.softcap) : SmallCap{};
    const float2 c2 = make_float2(p.scale_log2, p.scale_log2), nL2 = make_float2(nL, nL), nD2 = make_float2(nD, nD);
    const float alibi_l2 = (FEAT && p.alibi != nullptr) ? p.alibi[head] * kLog2e : 0.f;
    const bool masked_cells = FEAT && p.bmask != nullptr;
    const int cell_sh = masked_cells ? (p.bm_bk == 16 ? 4 : (p.bm_bk == 32 ? 5 : 6)) : 6;
    const uint8_t* mask_row = masked_cells ? p.bmask + static_cast<int64_t>(min(row, N - 1) / p.bm_bq) * p.bm_nk : nullptr;
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q), 0, s_abort));
    if (ok) {
      if (set == 0) {
        // this row's 128 bytes of d-half hf of Q -> 32 TMEM columns of the A operand
        const uint32_t rowa = smem_u32(sQ) + hf * (kTileBytes / 2) + rloc * 128;
        uint32_t qr[32];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                       : "=r"(qr[4 * c]), "=r"(qr[4 * c + 1]), "=r"(qr[4 * c + 2]), "=r"(qr[4 * c + 3])
                       : "r"(rowa + static_cast<uint32_t>((c ^ (rloc & 7)) << 4))
                       : "memory");
        tmem_st32(tmem + lane_base + cQA + hf * 32, qr);
        tc_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_QA_READY));
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int k0 = (kt_begin + j) * BN + cq * 32;            // first key of this thread's 32 columns
      // ---------------- phase A: S -> P' ----------------
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_S_FULL), j & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      uint32_t rs[32];
      tmem_ld32(tmem + lane_base + cS + cq * 32, rs);
      tc_wait_ld();
      // S(j + 1) is issued when every warp holds S(j): see that tile's K land first
      if (j + 1 < n_tiles) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_K_FULL + (j + 1) % kKStages), ((j + 1) / kKStages) & 1, s_abort))) { ok = false; break; }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_S_FREE));
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
      // visible keys of this row, relative to k0: [lo_rel, hi_rel]
      const int hi_rel = (p.causal ? min(S - 1, row + off) : S - 1) - k0;
      const int lo_rel = WIN ? row + off - p.window_left - k0 : 0;
      const bool need_mask = __any_sync(0xffffffffu, hi_rel < 31 || (WIN && lo_rel > 0));
      float pr[32];                                            // P, times (1 - tanh^2) under a soft cap
      // soft cap: are all of this warp's scores small enough for the polynomial form (see small_cap_consts)?
      bool small_y = false;
      if constexpr (CAP) {
        float am = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) am = fmaxf(am, fabsf(__uint_as_float(rs[i])));
        small_y = __all_sync(0xffffffffu, am * cap_in <= sc.y3);
      }
      auto phase_a = [&](auto small_c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 sv = make_float2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1]));
          float2 t, dcap;
          if constexpr (CAP) {
            if constexpr (decltype(small_c)::value) {
              const float2 z = __fmul2_rn(sv, sv);
              t = __ffma2_rn(sv, __ffma2_rn(z, make_float2(sc.kb3, sc.kb3), make_float2(sc.kk, sc.kk)), nL2);
              dcap = __ffma2_rn(z, __ffma2_rn(z, make_float2(sc.e2, sc.e2), make_float2(sc.e1, sc.e1)), make_float2(1.f, 1.f));
            } else {
              const float2 th = make_float2(cap_tanh(sv.x * cap_in, precise_tanh), cap_tanh(sv.y * cap_in, precise_tanh));
              t = __ffma2_rn(th, make_float2(cap_out, cap_out), nL2);
              dcap = __ffma2_rn(make_float2(-th.x, -th.y), th, make_float2(1.f, 1.f));
            }
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
          if constexpr (CAP) pe = __fmul2_rn(pe, dcap);
          pr[i] = pe.x;
          pr[i + 1] = pe.y;
        }
      };
      if (CAP && small_y) phase_a(std::true_type{}); else phase_a(std::false_type{});
      // dP(j + 1) is issued on DP_FREE(j) without a wait of the MMA thread's own: see that tile's V land first.
      // Checked here, where it costs nothing: the exponentials above are still in flight
      if (j + 1 < n_tiles) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_V_FULL + (j + 1) % kVStages), ((j + 1) / kVStages) & 1, s_abort))) { ok = false; break; }
      }
      // ---------------- phase B: dP -> dS ----------------
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DP_FULL), j & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      // dP(j) is complete: V(j)'s stage can be refilled
      if (warp == 0 && lane == 0) mbar_arrive(bar(BAR_V_FREE + j % kVStages));
      uint32_t rd[32];
      tmem_ld32(tmem + lane_base + cDP + cq * 32, rd);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_DP_FREE));
      uint32_t pd[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 dv = make_float2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1]));
        const float2 dsv = __fmul2_rn(make_float2(pr[i], pr[i + 1]), __fadd2_rn(dv, nD2));
        pd[i >> 1] = pack16q<DT>(dsv.x, dsv.y);
      }
      // the dS columns still hold dS(j - 1) until dQ(j - 1) has read them; its completion also frees K(j - 1)'s stage
      if (j >= 1) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DQ_DONE), (j - 1) & 1, s_abort))) { ok = false; break; }
        tc_fence_after();
        if (warp == 0 && lane == 0) mbar_arrive(bar(BAR_K_FREE + (j - 1) % kKStages));
      }
      // dS as 16-bit pairs along the key index: this warp's 32 keys -> 16 columns
      tmem_st16(tmem + lane_base + cDS + cq * 16, pd);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_DS_READY));
    }

    // ---- epilogue: dQ * scale -> 16-bit, through shared memory ----
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DQ_DONE), (n_tiles - 1) & 1, s_abort));
    if (ok) {
      tc_fence_after();
      // this warp's 32 of the 128 columns: d-half dh, 32-column half c of it; staged as [d-half][row][128 B] in the
      // first K stage (every load has been consumed), 16-byte chunks swizzled by row
      {
        const int dh = cq >> 1, c = cq & 1;
        uint32_t o[32];
        tmem_ld32(tmem + lane_base + cDQ + dh * 64 + c * 32, o);
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
            *reinterpret_cast<uint4*>(sK + dh * (kTileBytes / 2) + rloc * 128 + ((chunk ^ (rloc & 7)) << 4)) = v;
          } else if (row < N) {
            uint16_t* drow = reinterpret_cast<uint16_t*>(p.dq) + batch * p.dq_bs + head * p.dq_hs +
                             static_cast<int64_t>(q_begin + row) * p.dq_rs;
            *reinterpret_cast<uint4*>(drow + dh * 64 + chunk * 8) = v;
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
            tma_store_4d(&tmDQ, smem_u32(sK + h2 * (kTileBytes / 2)), 64 * h2, q0, head, batch);
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
