// Blackwell backward, head_dim 128, part 2 of 2: dK and dV.  tcgen05 MMAs with every accumulator in TMEM.
//
// The counterpart of the reference's dK/dV kernel (csrc/mfa_steel_bwd.cpp:765-1293); dQ is computed by
// bwd_dq_sm100.cu.  One persistent CTA per SM takes work items from a global counter; an item is a tile of 128 keys of
// one kv head, for which the CTA walks the query heads of the GQA group and the 128-row query tiles that can see those
// keys.  Per query tile (128 queries), four GEMMs with M = 128 key rows, every MMA N = 128 (an N = 64 MMA of this
// shape takes 1.5x its share of the tensor pipe):
//   S^T  = K . Q^T      (SS, K = 128)                                   -> TMEM [0,128)
//   dP^T = V . dO^T     (SS, K = 128)                                   -> TMEM [128,256)
//   dV  += P^T . dO     (A from TMEM, B = dO as an MN-major operand)    -> TMEM [256,384)
//   dK  += dS^T . Q     (A from TMEM, B = Q MN-major)                   -> TMEM [384,512)
// All 512 TMEM columns are in use, so K and V stay in shared memory as A operands and S^T / dP^T have one buffer
// each.  16 compute warps (thread = key row, a warp = 32 keys x 32 queries) work in two phases:
//   phase A  S^T -> P^T = 2^(s - L), written back as a 16-bit A operand over the columns it came from (P_READY),
//            with P^T [x (1 - tanh^2) under a soft cap] kept in registers
//   phase B  dP^T -> dS^T = P^T o (dP^T - delta), written back the same way (DS_READY)
// and the MMA thread alternates two groups: on P_READY dV(t) S^T(t+1), on DS_READY dK(t) dP^T(t+1); each group runs
// on the tensor pipe while the compute warps are in the other phase.  Warp 16 is the TMA producer (K and V once per
// item; Q and dO double-buffered, with -L and -delta of the query rows staged beside them), one thread of warp 17
// issues the MMAs.  dK / dV leave TMEM once per item, through shared memory as whole rows.  No load uses cluster
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
constexpr int BK = 128;      // keys per item (TMEM lanes)
constexpr int BQ = 128;      // queries per step
constexpr int kThreads = 576;       // warps 0-15 compute, 16 producer, 17 MMA issue
constexpr int kProducerWarp = 16, kMmaWarp = 17;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t cST = 0, cDPT = 128, cDV = 256, cDK = 384;

constexpr int kTileBytes = 128 * HD * 2;                 // 32768: one [2 d-halves][128 rows][128 B] tile
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kQStages = 3;      // Q(t) is read by S^T(t) one group before P_READY(t - 1)'s dV and by dK(t) last: three in use
constexpr int kDOStages = 2;     // dO(t): dP^T(t), then dV(t)
constexpr int kStatBytes = 2 * 2 * BQ * 4;               // -L and -delta of a query tile, two slots
constexpr int kSmemTiles = (2 + kQStages + kDOStages) * kTileBytes;        // K, V, Q x3, dO x2 = 229376
constexpr int kSmemUsed = kSmemTiles + kStatBytes + 256;
// All of the 227 KB a CTA can have: the tiles need a 1024-byte boundary, so the dynamic window may start up to
// kSmemBytes - kSmemUsed bytes off one (checked at run time; a CTA that finds less room raises status bit 1)
constexpr int kSmemBytes = 227 * 1024;
static_assert(kSmemUsed <= kSmemBytes, "shared memory");

// BAR_KV lives for the whole kernel; the others are set up again for every work item
enum Bar {
  BAR_KV = 0,
  BAR_Q_FULL = 1,        // + stage (3)
  BAR_DO_FULL = 4,       // + stage (2)
  BAR_STAT_FULL = 6,     // + slot (2): -L and -delta of a query tile are written
  BAR_Q_EMPTY = 8,       // + stage: a compute warp has seen dK of the stage's tile complete (at the start of the next
                         //   tile's phase B; every warp has then finished the tile's phase B, so its stat slot is free too)
  BAR_DO_EMPTY = 11,     // + stage: a compute warp has seen dV of the stage's tile complete (start of the next phase A)
  BAR_ST_FULL = 13,      // S^T of a tile is complete (and dV of the tile before it)
  BAR_DPT_FULL = 14,     // dP^T of a tile is complete (and dK of the tile before it)
  BAR_P_READY = 15,      // count 16: P^T is written
  BAR_DS_READY = 16,     // count 16: dS^T is written
  BAR_ACC_DONE = 17,
  BAR_COUNT = 18
};

struct DkvArgs {
  BwdParams p;
  int gx, gy, total_items;      // work items: (key tile, kv head, batch | sequence), key tile fastest
  int* counter;                 // next work item (zeroed by the preprocess kernel)
};

__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void lds_v4u(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}
// The address of the L / delta rows must come from here, issued after the wait that makes the data visible, so that
// no (non-volatile) load moves above that wait or is merged with the same address of another tile.
__device__ __forceinline__ uint32_t opaque_u32(uint32_t x) {
  uint32_t y;
  asm volatile("mov.u32 %0, %1;\n" : "=r"(y) : "r"(x) : "memory");
  return y;
}
template <int DT> __device__ __forceinline__ uint32_t pack16k(float a, float b) {
  return DT == 0 ? Elem<__half>::pack(a, b) : Elem<__nv_bfloat16>::pack(a, b);
}

// CAP (soft cap) and WIN (left window) are compile-time variants: the plain kernel's loops carry neither.
// FEAT: the ALiBi bias slope[h] * (key - (query + S - N)) and / or a block mask (cells of mask_bq x mask_bk, mask_bq a
// multiple of 32 so that the 32 queries a thread handles per step share one cell), as the forward's feature
// instantiation applies them (csrc/mfa_steel_fwd.cpp:951-970, 230-262 in the reference).  Without CAP / WIN.
template <int DT, bool CAP, bool WIN, bool FEAT>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dkv_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const DkvArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;
  unsigned char* sV = sK + kTileBytes;
  unsigned char* sQ = sV + kTileBytes;                 // [3 stages][2 d-halves][128][128 B]
  unsigned char* sDO = sQ + kQStages * kTileBytes;     // [2 stages]
  float* sL = reinterpret_cast<float*>(smem + kSmemTiles);      // [2 slots][BQ]
  float* sDel = sL + 2 * BQ;                                    // [2 slots][BQ]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles + kStatBytes);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  // [2][8]: this item and the next one as {index or -1, key tile, kv head, batch, k_begin, S, q_begin, N}
  volatile int* s_work = reinterpret_cast<volatile int*>(s_tmem + 2);

  const BwdParams& p = a.p;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };
  if (smem + kSmemUsed > smem_raw + kSmemBytes) {          // CTA-uniform: the window starts too far off a 1024-byte boundary
    if (tid == 0) atomicOr(&g_kernel_status, 2);
    return;
  }

  // Next item that has keys (grid cells beyond a sequence's end are skipped), decoded into slot `sl` of s_work for
  // every role to read; index -1 when the list is exhausted.  Run by one thread.
  auto fetch_next = [&](int sl) -> int {
    volatile int* o = s_work + sl * 8;
    for (int tries = 0; tries < (1 << 24); ++tries) {
      const int idx = atomicAdd(a.counter, 1);
      if (idx >= a.total_items) break;
      const int kt = idx % a.gx, kvh_ = (idx / a.gx) % a.gy, z = idx / (a.gx * a.gy);
      int kb = 0, S_ = p.S, qb = 0, N_ = p.N;
      if (p.cu_k != nullptr) {
        kb = p.cu_k[z];
        S_ = p.cu_k[z + 1] - kb;
      }
      if (kt * BK >= S_) continue;
      if (p.cu_q != nullptr) {
        qb = p.cu_q[z];
        N_ = p.cu_q[z + 1] - qb;
      }
      o[1] = kt; o[2] = kvh_; o[3] = p.cu_q != nullptr ? 0 : z; o[4] = kb; o[5] = S_; o[6] = qb; o[7] = N_;
      o[0] = idx;
      return idx;
    }
    o[0] = -1;
    return -1;
  };
  if (warp == kProducerWarp && lane == 0) {
    mbar_init(bar(BAR_KV), 1);
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async();
    fetch_next(0);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  int kv_uses = 0;                                       // items so far that loaded K / V (phase of BAR_KV)

  for (int w = 0;; ++w) {
  volatile int* wk = s_work + (w & 1) * 8;
  if (wk[0] < 0 || *s_abort != 0) break;
  const int kvh = wk[2], bb = wk[3], k_begin = wk[4], S = wk[5], q_begin = wk[6], N = wk[7];
  const int n0 = wk[1] * BK;
  const int off = S - N;
  int m_begin = 0;
  if (p.causal) m_begin = max(0, n0 - off) / BQ;
  int m_end = (N + BQ - 1) / BQ;
  // a left window: the last row that still sees this tile's last key is i = key - off + window_left
  if constexpr (WIN) m_end = min(m_end, max(0, min(S, n0 + BK) - 1 - off + p.window_left) / BQ + 1);
  const int nm = max(0, m_end - m_begin);
  const int n_iter = nm * p.gqa;
  const uint32_t kv_par = kv_uses & 1;
  if (n_iter > 0) ++kv_uses;

  auto load_q = [&](int it) {
    const int st = it % kQStages;
    const int hq = kvh * p.gqa + it / nm, m = m_begin + it % nm;
    mbar_arrive_expect_tx(bar(BAR_Q_FULL + st), kTileBytes);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
      tma_load_4d(smem_u32(sQ + st * kTileBytes + hf * kHalfBytes), &tmQ, bar(BAR_Q_FULL + st), 64 * hf, q_begin + m * BQ, hq, bb);
  };
  auto load_do = [&](int it) {
    const int st = it % kDOStages;
    const int hq = kvh * p.gqa + it / nm, m = m_begin + it % nm;
    mbar_arrive_expect_tx(bar(BAR_DO_FULL + st), kTileBytes);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
      tma_load_4d(smem_u32(sDO + st * kTileBytes + hf * kHalfBytes), &tmDO, bar(BAR_DO_FULL + st), 64 * hf, q_begin + m * BQ, hq, bb);
  };
  if (warp == kProducerWarp && lane == 0) {
    if (w > 0)
      for (int i = BAR_Q_FULL; i < BAR_COUNT; ++i) mbar_inval(bar(i));    // nobody waits or arrives between items
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(bar(BAR_Q_FULL + s), 1);
      mbar_init(bar(BAR_Q_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BAR_DO_FULL + s), 1);
      mbar_init(bar(BAR_DO_EMPTY + s), 1);
      mbar_init(bar(BAR_STAT_FULL + s), 1);
    }
    mbar_init(bar(BAR_ST_FULL), 1);
    mbar_init(bar(BAR_DPT_FULL), 1);
    mbar_init(bar(BAR_P_READY), 16);        // one arrive per compute warp
    mbar_init(bar(BAR_DS_READY), 16);
    mbar_init(bar(BAR_ACC_DONE), 1);
    fence_barrier_init();
    fence_proxy_async();
    if (n_iter > 0) {
      mbar_arrive_expect_tx(bar(BAR_KV), 2 * kTileBytes);
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_4d(smem_u32(sK + hf * kHalfBytes), &tmK, bar(BAR_KV), 64 * hf, k_begin + n0, kvh, bb);
        tma_load_4d(smem_u32(sV + hf * kHalfBytes), &tmV, bar(BAR_KV), 64 * hf, k_begin + n0, kvh, bb);
      }
      load_q(0);
      load_do(0);
      if (n_iter > 1) {
        load_q(1);
        load_do(1);
      }
      if (n_iter > 2) load_q(2);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == kProducerWarp) {
    // ============================ producer ============================
    // -L and -delta of tile `it`'s 128 query rows -> registers (four rows per lane); rows beyond N (or without any
    // visible key) get L = +inf so that their P is exactly zero
    float Lr[4], dr[4];
    auto read_stats = [&](int it) {
      const int hq = kvh * p.gqa + it / nm, m = m_begin + it % nm;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = m * BQ + lane * 4 + i;
        Lr[i] = INFINITY;
        dr[i] = 0.f;
        if (row < N) {
          const int64_t idx = bb * p.lse_bs + hq * p.lse_hs + q_begin + row;
          Lr[i] = p.lse[idx];
          dr[i] = p.delta[idx];
          if (Lr[i] == -INFINITY) Lr[i] = INFINITY;
        }
      }
    };
    auto write_stats = [&](int it) {
      const int sl = it & 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sL[sl * BQ + lane * 4 + i] = -Lr[i];            // stored negated: the compute loop adds them
        sDel[sl * BQ + lane * 4 + i] = -dr[i];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_STAT_FULL + sl));
      __syncwarp();
    };
    for (int it = 0; it < 2 && it < n_iter; ++it) {
      read_stats(it);
      write_stats(it);
    }
    // Tile e's dO stage is released at the start of phase A of tile e + 1, its Q stage and stat slot at the start of
    // phase B of tile e + 1: dO(e + 2), then Q(e + 3) and the stats of tile e + 2, go there.  Each barrier's next
    // completion needs the tile loaded here, so the producer is never more than one completion behind.
    for (int e = 0; e + 2 < n_iter; ++e) {
      read_stats(e + 2);
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DO_EMPTY + (e & 1)), (e >> 1) & 1, s_abort))) break;
      if (lane == 0) load_do(e + 2);
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q_EMPTY + e % kQStages), (e / kQStages) & 1, s_abort))) break;
      if (lane == 0 && e + 3 < n_iter) load_q(e + 3);
      write_stats(e + 2);
    }
    // the next item, for every role to read after the end-of-item sync
    if (lane == 0) fetch_next((w + 1) & 1);
  } else if (warp == kMmaWarp) {
   if (lane == 0 && n_iter > 0) {
    // ============================ MMA issue ============================
    //   S^T(0) dP^T(0) | P_READY(t) -> dV(t) S^T(t+1) | DS_READY(t) -> dK(t) dP^T(t+1) | ...
    const uint32_t id_st = instr_desc(DT, 0, 128, BQ);     // S^T, dP^T: B K-major, N = 128 queries
    const uint32_t id_mn = instr_desc(DT, 1, 128, HD);     // dV, dK: B MN-major, N = 128 = head_dim
    const uint64_t kd = smem_desc(smem_u32(sK), 16, 1024), vd = smem_desc(smem_u32(sV), 16, 1024);
    const uint64_t qd0 = smem_desc(smem_u32(sQ), 16, 1024), dod0 = smem_desc(smem_u32(sDO), 16, 1024);
    const uint64_t qmn0 = smem_desc(smem_u32(sQ), kHalfBytes, 1024), domn0 = smem_desc(smem_u32(sDO), kHalfBytes, 1024);
    constexpr uint64_t kTileU = kTileBytes >> 4, kHalfU = kHalfBytes >> 4;
    bool ok = mbar_wait_bounded(bar(BAR_KV), kv_par, s_abort);
    // A = the K / V rows (K-major, two d-halves), B rows = the 128 queries of tile `it`
    auto issue_st = [&](int it) {
      const uint64_t qd = qd0 + (it % kQStages) * kTileU;
#pragma unroll
      for (int k = 0; k < HD / 16; ++k)
        mma_ss(tmem + cST, kd + (k >> 2) * kHalfU + (k & 3) * 2, qd + (k >> 2) * kHalfU + (k & 3) * 2, id_st, k > 0 ? 1u : 0u);
      tc_commit(bar(BAR_ST_FULL));
    };
    auto issue_dpt = [&](int it) {
      const uint64_t dod = dod0 + (it & 1) * kTileU;
#pragma unroll
      for (int k = 0; k < HD / 16; ++k)
        mma_ss(tmem + cDPT, vd + (k >> 2) * kHalfU + (k & 3) * 2, dod + (k >> 2) * kHalfU + (k & 3) * 2, id_st, k > 0 ? 1u : 0u);
      tc_commit(bar(BAR_DPT_FULL));
    };
    // the first Q and dO tiles are waited for here, every later one by the compute warps before the arrival that
    // lets its MMAs be issued
    if (ok) ok = mbar_wait_bounded(bar(BAR_Q_FULL), 0, s_abort);
    if (ok) {
      tc_fence_after();
      issue_st(0);
      ok = mbar_wait_bounded(bar(BAR_DO_FULL), 0, s_abort);
    }
    if (ok) {
      tc_fence_after();
      issue_dpt(0);
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint64_t qmn = qmn0 + (it % kQStages) * kTileU, domn = domn0 + (it & 1) * kTileU;
      // the compute warps vouch, before they arrive here, that the next tile's Q has landed (DS_READY: its dO)
      if (!mbar_wait_bounded(bar(BAR_P_READY), it & 1, s_abort)) { ok = false; break; }
      tc_fence_after();
      // A in TMEM: 8 columns per 16 queries; queries 32c .. 32c + 31 of the tile at column 32c (where warp column c
      // wrote them); B rows = queries, 16 rows = 128 units
#pragma unroll
      for (int k = 0; k < BQ / 16; ++k)
        mma_ts(tmem + cDV, tmem + cST + (k >> 1) * 32 + (k & 1) * 8, domn + k * 128, id_mn, (it > 0 || k > 0) ? 1u : 0u);
      // S^T(it + 1) overwrites the P^T those MMAs read: the pipe runs in order
      if (it + 1 < n_iter) issue_st(it + 1);
      if (!mbar_wait_bounded(bar(BAR_DS_READY), it & 1, s_abort)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < BQ / 16; ++k)
        mma_ts(tmem + cDK, tmem + cDPT + (k >> 1) * 32 + (k & 1) * 8, qmn + k * 128, id_mn, (it > 0 || k > 0) ? 1u : 0u);
      if (it + 1 < n_iter) issue_dpt(it + 1);
    }
    if (ok) tc_commit(bar(BAR_ACC_DONE));
   }
  } else {
    // ============================ compute warps 0-15 ============================
    const int wq = warp & 3, cq = warp >> 2;                 // TMEM lane quarter (keys), 32-query column quarter
    const int rloc = wq * 32 + lane;                         // key row inside the tile
    const int key = n0 + rloc;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    if (n_iter == 0) {
      // no query sees these keys: dK = dV = 0
      if (key < S) {
        const int64_t o = bb * p.dk_bs + kvh * p.dk_hs + static_cast<int64_t>(k_begin + key) * p.dk_rs + cq * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dk) + o)[i] = make_uint4(0u, 0u, 0u, 0u);
          reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dv) + o)[i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    } else {
    bool ok = true;
    const int q0l = cq * 32;                               // first query (inside the tile) of this warp's 32 columns
    const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
    const float cap_in = CAP ? p.scale / p.softcap : 0.f, cap_out = p.softcap * kLog2e;
    const bool precise_tanh = p.softcap >= kPreciseTanhMinCap;
    const SmallCap sc = CAP ? small_cap_consts(p.scale, p.softcap) : SmallCap{};
    const int wlo = WIN ? off - p.window_left : 0;         // window: key visible iff key >= qrow + wlo
    for (int it = 0; it < n_iter && ok; ++it) {
      const int sl = it & 1;
      const int m = m_begin + it % nm;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_STAT_FULL + sl), (it >> 1) & 1, s_abort))) { ok = false; break; }
      const uint32_t Ls = opaque_u32(smem_u32(sL + sl * BQ)), Ds = Ls + 2 * BQ * 4;
      const bool need_mask = (n0 + BK > S) || (p.causal && (n0 + BK - 1 > m * BQ + off)) ||
                             (WIN && (n0 < m * BQ + BQ - 1 + off - p.window_left));
      const float alibi_l2 = (FEAT && p.alibi != nullptr) ? p.alibi[kvh * p.gqa + it / nm] * kLog2e : 0.f;
      // FEAT: the mask cell of (these 32 queries, this key) and the bias of the first of them, in the log2 domain
      bool cell_on = true;
      float ab = 0.f;
      if constexpr (FEAT) {
        const int qrow0 = m * BQ + q0l;
        if (p.bmask != nullptr)
          cell_on = key < S && p.bmask[static_cast<int64_t>(min(qrow0, N - 1) / p.bm_bq) * p.bm_nk + key / p.bm_bk] != 0;
        ab = alibi_l2 * static_cast<float>(key - off - qrow0);
      }

      // ---------------- phase A: S^T -> P^T (TMEM, 16-bit) and P^T [x (1 - tanh^2)] (registers) ----------------
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_ST_FULL), it & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      // the commit just seen also followed dV(it - 1), the last reader of the other dO stage
      if (it >= 1 && warp == 0 && lane == 0) mbar_arrive(bar(BAR_DO_EMPTY + ((it - 1) & 1)));
      float pr[32];
      {
        uint32_t rs[32];
        tmem_ld32(tmem + lane_base + cST + q0l, rs);
        tc_wait_ld();
        uint32_t pp[16];
        // soft cap: are all of this warp's scores small enough for the polynomial form (see small_cap_consts)?
        bool small_y = false;
        if constexpr (CAP) {
          float am = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) am = fmaxf(am, fabsf(__uint_as_float(rs[i])));
          small_y = __all_sync(0xffffffffu, am * cap_in <= sc.y3);
        }
        auto phase_a = [&](auto masked, auto small_c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 nL = lds_f4(Ls + (q0l + i) * 4);      // -L of four queries
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              const float2 sv = make_float2(__uint_as_float(rs[i + e]), __uint_as_float(rs[i + e + 1]));
              const float2 nl = e == 0 ? make_float2(nL.x, nL.y) : make_float2(nL.z, nL.w);
              float2 t;
              [[maybe_unused]] float2 dcap;
              if constexpr (CAP) {
                if constexpr (decltype(small_c)::value) {
                  const float2 z = __fmul2_rn(sv, sv);
                  t = __ffma2_rn(sv, __ffma2_rn(z, make_float2(sc.kb3, sc.kb3), make_float2(sc.kk, sc.kk)), nl);
                  dcap = __ffma2_rn(z, __ffma2_rn(z, make_float2(sc.e2, sc.e2), make_float2(sc.e1, sc.e1)), make_float2(1.f, 1.f));
                } else {
                  const float2 th = make_float2(cap_tanh(sv.x * cap_in, precise_tanh), cap_tanh(sv.y * cap_in, precise_tanh));
                  t = __ffma2_rn(th, make_float2(cap_out, cap_out), nl);
                  dcap = __ffma2_rn(make_float2(-th.x, -th.y), th, make_float2(1.f, 1.f));
                }
              } else {
                t = __ffma2_rn(sv, c2, nl);
              }
              if constexpr (FEAT) {
                t = __fadd2_rn(t, make_float2(fmaf(-alibi_l2, static_cast<float>(i + e), ab), fmaf(-alibi_l2, static_cast<float>(i + e + 1), ab)));
              }
              float2 pe = make_float2(fast_exp2(t.x), fast_exp2(t.y));
              if constexpr (FEAT) {
                if (!cell_on) pe = make_float2(0.f, 0.f);
              }
              if constexpr (decltype(masked)::value) {
                const int qrow = m * BQ + q0l + i + e;
                const bool kin = key < S;
                if (!(kin && (!p.causal || key <= qrow + off) && (!WIN || key >= qrow + wlo))) pe.x = 0.f;
                if (!(kin && (!p.causal || key <= qrow + 1 + off) && (!WIN || key >= qrow + 1 + wlo))) pe.y = 0.f;
              }
              pp[(i + e) >> 1] = pack16k<DT>(pe.x, pe.y);
              if constexpr (CAP) pe = __fmul2_rn(pe, dcap);
              pr[i + e] = pe.x;
              pr[i + e + 1] = pe.y;
            }
          }
        };
        if (CAP && small_y) {
          if (need_mask) phase_a(std::true_type{}, std::true_type{}); else phase_a(std::false_type{}, std::true_type{});
        } else {
          if (need_mask) phase_a(std::true_type{}, std::false_type{}); else phase_a(std::false_type{}, std::false_type{});
        }
        // P^T goes back as 16-bit pairs along the query index, inside the 32 columns this warp has just read
        tmem_st16(tmem + lane_base + cST + q0l, pp);
        tc_wait_st();
      }
      // on behalf of the MMA thread: the next tile's Q has landed (its S^T follows this tile's dV)
      if (it + 1 < n_iter &&
          !__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q_FULL + (it + 1) % kQStages), ((it + 1) / kQStages) & 1, s_abort))) { ok = false; break; }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_P_READY));

      // ---------------- phase B: dP^T -> dS^T ----------------
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DPT_FULL), it & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      // the commit just seen also followed dK(it - 1), the last reader of that tile's Q stage; and every warp has
      // finished phase B(it - 1), the last reader of its stat slot
      if (it >= 1 && warp == 0 && lane == 0) mbar_arrive(bar(BAR_Q_EMPTY + (it - 1) % kQStages));
      // in two halves of 16 queries: fewer registers are live at once
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t rd[16];
        tmem_ld16(tmem + lane_base + cDPT + q0l + 16 * h, rd);
        tc_wait_ld();
        uint32_t pd[8];
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          const float4 nD = lds_f4(Ds + (q0l + 16 * h + i) * 4);      // -delta of four queries
          const float2 d0 = __fmul2_rn(make_float2(pr[16 * h + i], pr[16 * h + i + 1]),
                                       __fadd2_rn(make_float2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1])), make_float2(nD.x, nD.y)));
          const float2 d1 = __fmul2_rn(make_float2(pr[16 * h + i + 2], pr[16 * h + i + 3]),
                                       __fadd2_rn(make_float2(__uint_as_float(rd[i + 2]), __uint_as_float(rd[i + 3])), make_float2(nD.z, nD.w)));
          pd[i >> 1] = pack16k<DT>(d0.x, d0.y);
          pd[(i >> 1) + 1] = pack16k<DT>(d1.x, d1.y);
        }
        // dS^T of queries 16h .. 16h + 15 over columns 8h .. 8h + 7 of this warp's 32.  The second half's dP^T sits in
        // columns 16 .. 31, which this store does not touch
        tmem_st8(tmem + lane_base + cDPT + q0l + 8 * h, pd);
      }
      tc_wait_st();
      // on behalf of the MMA thread: the next tile's dO has landed (its dP^T follows this tile's dK)
      if (it + 1 < n_iter &&
          !__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DO_FULL + ((it + 1) & 1)), ((it + 1) >> 1) & 1, s_abort))) { ok = false; break; }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_DS_READY));
    }

    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_ACC_DONE), 0, s_abort));
    // dK, dV: rows = keys, this warp's 32 of the 128 columns.  The tiles go through shared memory (the Q stages,
    // which nothing reads any more: dK in stage 0, dV in stage 1) so that each store instruction writes whole
    // 128-byte rows.
    if (ok) {
      tc_fence_after();
      const int dh = cq >> 1, c = cq & 1;                // d-half, 32-column half of it
      uint32_t rk[32], rv[32];
      tmem_ld32(tmem + lane_base + cDK + cq * 32, rk);
      tmem_ld32(tmem + lane_base + cDV + cq * 32, rv);
      tc_wait_ld();
      const uint32_t srow = smem_u32(sQ) + dh * kHalfBytes + rloc * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 8 * j;
        const uint32_t o = static_cast<uint32_t>(((c * 4 + j) ^ (rloc & 7)) << 4);
        sts_v4(srow + o, pack16k<DT>(__uint_as_float(rk[i]) * p.scale, __uint_as_float(rk[i + 1]) * p.scale),
               pack16k<DT>(__uint_as_float(rk[i + 2]) * p.scale, __uint_as_float(rk[i + 3]) * p.scale),
               pack16k<DT>(__uint_as_float(rk[i + 4]) * p.scale, __uint_as_float(rk[i + 5]) * p.scale),
               pack16k<DT>(__uint_as_float(rk[i + 6]) * p.scale, __uint_as_float(rk[i + 7]) * p.scale));
        sts_v4(srow + kTileBytes + o, pack16k<DT>(__uint_as_float(rv[i]), __uint_as_float(rv[i + 1])),
               pack16k<DT>(__uint_as_float(rv[i + 2]), __uint_as_float(rv[i + 3])),
               pack16k<DT>(__uint_as_float(rv[i + 4]), __uint_as_float(rv[i + 5])),
               pack16k<DT>(__uint_as_float(rv[i + 6]), __uint_as_float(rv[i + 7])));
      }
    }
    // all sixteen compute warps pass here, whatever happened before (a named barrier has no time-out)
    asm volatile("bar.sync 1, 512;\n" ::: "memory");
    if (ok) {
      // 128 rows x 2 d-halves x 8 chunks of 16 bytes per tensor; a warp instruction covers four whole half-rows
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int i = r4 * 512 + tid;
        const int h = i >> 10, r = (i >> 3) & 127, c = i & 7;
        const uint32_t sa = smem_u32(sQ) + h * kHalfBytes + r * 128 + static_cast<uint32_t>((c ^ (r & 7)) << 4);
        uint4 vk, vv;
        lds_v4u(sa, vk.x, vk.y, vk.z, vk.w);
        lds_v4u(sa + kTileBytes, vv.x, vv.y, vv.z, vv.w);
        if (n0 + r < S) {
          const int64_t o = bb * p.dk_bs + kvh * p.dk_hs + static_cast<int64_t>(k_begin + n0 + r) * p.dk_rs + h * 64 + c * 8;
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dk) + o) = vk;
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dv) + o) = vv;
        }
      }
    }
    }  // n_iter > 0
  }

  // ---- end of the item: every MMA has completed (the compute warps saw ACC_DONE), the epilogue has read its staging
  // rows; the barriers may be set up again and the tiles refilled
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  }  // work items

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

bool make_map128k(CUtensorMap* m, int dtype, const void* base, int rows, int H, int B, int64_t rs, int64_t hs, int64_t bs) {
  const uint64_t dims[4] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(rows), static_cast<uint64_t>(H),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(rs) * 2, static_cast<uint64_t>(hs) * 2, static_cast<uint64_t>(bs) * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tmap(m, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims,
                     strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

bool bwd_split_sm100_supported(int dtype, int D) { return (dtype == 0 || dtype == 1) && D == HD && get_encode_tiled() != nullptr; }

// dK and dV for head_dim 128; p.delta must hold delta and *p.work_counter zero.
cudaError_t launch_bwd_dkv_sm100(const BwdParams& p, int dtype, int nbatch, int max_k, cudaStream_t stream) {
  if (nbatch <= 0 || max_k <= 0) return cudaSuccess;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  auto fix = [](int64_t s, int64_t fallback) { return s > 0 ? s : fallback; };   // size-1 dimensions only (see bwd_sm100_strides_ok)
  const int64_t q_hs = fix(p.q_hs, static_cast<int64_t>(p.N) * p.q_rs), q_bs = fix(p.q_bs, q_hs * p.Hq);
  const int64_t k_hs = fix(p.k_hs, static_cast<int64_t>(p.S) * p.k_rs), k_bs = fix(p.k_bs, k_hs * p.Hkv);
  const int64_t v_hs = fix(p.v_hs, static_cast<int64_t>(p.S) * p.v_rs), v_bs = fix(p.v_bs, v_hs * p.Hkv);
  const int64_t do_hs = static_cast<int64_t>(p.N) * HD, do_bs = do_hs * p.Hq;
  if (!make_map128k(&tmQ, dtype, p.q, p.N, p.Hq, p.B, p.q_rs, q_hs, q_bs) ||
      !make_map128k(&tmK, dtype, p.k, p.S, p.Hkv, p.B, p.k_rs, k_hs, k_bs) ||
      !make_map128k(&tmV, dtype, p.v, p.S, p.Hkv, p.B, p.v_rs, v_hs, v_bs) ||
      !make_map128k(&tmDO, dtype, p.dout, p.N, p.Hq, p.B, HD, do_hs, do_bs))
    return cudaErrorInvalidValue;
  DkvArgs a;
  a.p = p;
  a.gx = (max_k + BK - 1) / BK;
  a.gy = p.Hkv;
  const long long items = static_cast<long long>(a.gx) * a.gy * nbatch;
  if (items > 0x7fffffffLL || p.work_counter == nullptr) return cudaErrorInvalidValue;
  a.total_items = static_cast<int>(items);
  a.counter = p.work_counter;
  int dev = 0, sm_count = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      sm_count <= 0)
    sm_count = 148;
  dim3 grid(static_cast<unsigned>(items < sm_count ? items : sm_count), 1, 1);   // one persistent CTA per SM
  auto launch = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    kern<<<grid, kThreads, kSmemBytes, stream>>>(tmQ, tmK, tmV, tmDO, a);
    return cudaGetLastError();
  };
  const bool cap = p.softcap > 0.f, win = p.window_left >= 0, feat = p.alibi != nullptr || p.bmask != nullptr;
  if (feat) return dtype == 0 ? launch(bwd_dkv_sm100_kernel<0, false, false, true>) : launch(bwd_dkv_sm100_kernel<1, false, false, true>);
  if (dtype == 0) {
    if (cap) return win ? launch(bwd_dkv_sm100_kernel<0, true, true, false>) : launch(bwd_dkv_sm100_kernel<0, true, false, false>);
    return win ? launch(bwd_dkv_sm100_kernel<0, false, true, false>) : launch(bwd_dkv_sm100_kernel<0, false, false, false>);
  }
  if (cap) return win ? launch(bwd_dkv_sm100_kernel<1, true, true, false>) : launch(bwd_dkv_sm100_kernel<1, true, false, false>);
  return win ? launch(bwd_dkv_sm100_kernel<1, false, true, false>) : launch(bwd_dkv_sm100_kernel<1, false, false, false>);
}

cudaError_t bwd_dkv_sm100_read_clear_status(cudaStream_t stream, int* out) {
  const int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_kernel_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess && *out != 0)
    e = cudaMemcpyToSymbolAsync(g_kernel_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return e;
}

}  // namespace b200fa
