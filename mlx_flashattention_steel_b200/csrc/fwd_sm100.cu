// Blackwell forward kernel: tcgen05 MMAs with TMEM accumulators, TMA-staged tiles,
// warp-specialised roles.  Dense and packed-varlen layouts, 16-bit, D = 64, 128 or 256; any N, S; GQA;
// causal (lower-right), left window, softcap, lse.  What it computes is the reference forward
// (csrc/mfa_steel_fwd.cpp:801-1221); how is Blackwell's own:
//
//   warps 0-3  softmax: thread r owns query row r = TMEM lane r.  It pulls the row of
//              S out of TMEM (tcgen05.ld), applies scale / softcap / masks, keeps the
//              running max and sum, writes P (16-bit) back into the same TMEM columns
//              (tcgen05.st) and, rarely, rescales O in TMEM (only when the row max grew
//              by more than 2^8, so P stays small).
//   warp 4     producer: TMA tensor copies of the Q tile (once) and of K / V tiles into
//              two-stage rings, 128B-swizzled, completion on mbarriers.
//   warp 5     MMA issue (one thread): S(j) = Q.K(j)^T  (SS, M=128 N=64 K=16 x8) into one
//              of two S buffers, then O += P(j).V(j)  (A from TMEM, M=128 N=D K=16 x4).
//              Issue order S(0) S(1) PV(0) S(2) PV(1) ... keeps the tensor pipe busy while
//              the softmax warps work on the other buffer; tcgen05.commit signals the
//              mbarriers that free smem stages and publish S / O.
//
// TMEM (256 of 512 columns up to D = 128, so two CTAs share an SM and hide each other's softmax; D = 256 takes 384
// and one CTA per SM):
//   [0,64) S0 / P0   [64,128) S1 / P1   [128,128+D) O.
// Tiles above the causal diagonal or left of the window are skipped whole.
// Paged K / V (prefill-sized queries over a page pool; the role of the reference's paged STEEL forward,
// csrc/mfa_steel_fwd.cpp:2462-3121, host csrc/mfa_attention.cpp:1355-1552): the producer walks the block table and
// brings a 64-key tile in as four 16-token boxes, one per page or part of a page; holes in the table and units
// beyond the sequence read the pool's out-of-bounds rows, which TMA fills with zeros.  Nothing is gathered.
// No load here uses cluster multicast.  Every mbarrier wait is bounded; on a timeout the
// CTA raises its abort flag, frees its TMEM, sets bit 0 of this file's device status word
// (read through b200fa_kernel_status) and leaves; that launch's outputs are then undefined.
#include <cstdio>

#include "common.cuh"
#include "launch.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace b200fa {
// Device status word of this file's kernels: bit 0 = a bounded wait gave up.
static __device__ int g_kernel_status = 0;


namespace {

constexpr int BM = 128;      // query rows per CTA
constexpr int BN = 64;       // keys per tile
constexpr int kStages = 2;
constexpr int kThreads = 192;
// TMEM columns of one CTA: two 64-column S buffers + head_dim columns of O, rounded up to a power of two.  256 for
// head_dim <= 128 (two CTAs per SM), all 512 for head_dim 256 (one CTA per SM)
template <int HD> constexpr uint32_t tmem_cols() { return HD > 128 ? 512u : 256u; }
constexpr int kMaxListTiles = 1024;   // block-sparse instantiation: active key tiles of one query tile (16-bit indices)

// Sizes that depend on the head dim (64, 128 or 256).  Tiles are stored as 64-element (128-byte) wide halves,
// [half][row][128 B], each half one 128B-swizzle atom wide.
template <int HD> struct Cfg {
  static constexpr int kHalves = HD / 64;
  static constexpr int kQBytes = BM * HD * 2;          // 32768 (D=128) / 16384 (D=64)
  static constexpr int kKVBytes = BN * HD * 2;         // 16384 / 8192 per stage
  static constexpr int kSmemTiles = kQBytes + 2 * kStages * kKVBytes;
  static constexpr int kSmemBytes = kSmemTiles + 256 + 1024;   // + barriers + alignment slack
  static constexpr int kSmemBytesFeat = kSmemBytes + kMaxListTiles * 3;   // + the active-tile list and its flags
};

// barrier slots (uint64 each)
enum Bar {
  BAR_Q = 0,
  BAR_K_FULL = 1,            // +stage
  BAR_V_FULL = 5,
  BAR_PV_DONE = 7,           // +stage: P.V of a tile has completed -- O may be rescaled, the V stage is free again
  BAR_S_FULL = 9,            // +buffer: S of a tile is complete -- for the softmax warps, and the K stage is free again
  BAR_P_FULL = 11,           // +buffer
  BAR_Q_FREE = 13,           // persistent CTAs: the item's last S MMAs have read Q -- the next item's Q may land
  BAR_O_STAGED = 14,         // count 4: the softmax warps have written their O rows to shared memory
  BAR_O_FINAL = 15,          // committed once, after the last P.V: O is complete
  BAR_COUNT = 16
};

struct Sm100Args {
  FwdParams p;
  int tma_store;             // dense layout: O leaves through shared memory and TMA stores
  int gx, gy, total_items;   // persistent CTAs: items = (query tile, head, batch | sequence), query tile fastest
};

// max / min of 64 values as a 3-ary tree (depth 4) instead of a 63-deep dependent chain
__device__ __forceinline__ float tree_max64(const float (&x)[64]) {
  float a[22];
#pragma unroll
  for (int i = 0; i < 21; ++i) a[i] = max3(x[3 * i], x[3 * i + 1], x[3 * i + 2]);
  a[21] = x[63];
  float b[8];
#pragma unroll
  for (int i = 0; i < 7; ++i) b[i] = max3(a[3 * i], a[3 * i + 1], a[3 * i + 2]);
  b[7] = a[21];
  return max3(max3(b[0], b[1], b[2]), max3(b[3], b[4], b[5]), fmaxf(b[6], b[7]));
}
// max of |x| over 64 values (the absolute values fold into the max instruction's source modifiers)
__device__ __forceinline__ float tree_absmax64(const float (&x)[64]) {
  float a[22];
#pragma unroll
  for (int i = 0; i < 21; ++i) a[i] = max3(fabsf(x[3 * i]), fabsf(x[3 * i + 1]), fabsf(x[3 * i + 2]));
  a[21] = fabsf(x[63]);
  float b[8];
#pragma unroll
  for (int i = 0; i < 7; ++i) b[i] = max3(a[3 * i], a[3 * i + 1], a[3 * i + 2]);
  b[7] = a[21];
  return max3(max3(b[0], b[1], b[2]), max3(b[3], b[4], b[5]), fmaxf(b[6], b[7]));
}
__device__ __forceinline__ float tree_min64(const float (&x)[64]) {
  float a[22];
#pragma unroll
  for (int i = 0; i < 21; ++i) a[i] = min3(x[3 * i], x[3 * i + 1], x[3 * i + 2]);
  a[21] = x[63];
  float b[8];
#pragma unroll
  for (int i = 0; i < 7; ++i) b[i] = min3(a[3 * i], a[3 * i + 1], a[3 * i + 2]);
  b[7] = a[21];
  return min3(min3(b[0], b[1], b[2]), min3(b[3], b[4], b[5]), fminf(b[6], b[7]));
}

// Of every 4 key pairs a softmax thread handles, this many take exp2 on the FMA pipe (exp2_poly2) instead of
// the special-function unit.  0 by default: measured on config 2, shares of 25 % and 50 % were 5 % and 10 % slower
// (the polynomial costs about 20 FMA-pipe clocks per pair against 16 on the special-function unit, and the kernel
// is not bound by that unit alone).  Kept as a build-time switch for shapes where that balance differs.
#ifndef B200FA_EXP_POLY_PAIRS
#define B200FA_EXP_POLY_PAIRS 0
#endif
constexpr int kExpPolyPairs = B200FA_EXP_POLY_PAIRS;

// 2^t for two values without the special-function unit: n = round(t) by the 1.5*2^23 trick, 2^(t-n) by a cubic
// on [-0.5, 0.5] (relative error < 7.5e-5, far below the 16-bit rounding of P), n added into the exponent field.
__device__ __forceinline__ float2 exp2_poly2(float2 t) {
  const float2 magic = make_float2(12582912.f, 12582912.f), neg_magic = make_float2(-12582912.f, -12582912.f);
  const float2 tc = make_float2(fmaxf(t.x, -125.f), fmaxf(t.y, -125.f));
  const float2 tt = __fadd2_rn(tc, magic);
  const float2 nf = __fadd2_rn(tt, neg_magic);
  const float2 r = __ffma2_rn(nf, make_float2(-1.f, -1.f), tc);
  float2 q = __ffma2_rn(r, make_float2(0.0551716685f, 0.0551716685f), make_float2(0.2426111251f, 0.2426111251f));
  q = __ffma2_rn(r, q, make_float2(0.6932609677f, 0.6932609677f));
  q = __ffma2_rn(r, q, make_float2(0.9999280572f, 0.9999280572f));
  return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(tt.x) << 23)),
                     __int_as_float(__float_as_int(q.y) + (__float_as_int(tt.y) << 23)));
}
// exp2 of a pair; `pair` is the compile-time index of the pair inside the row
__device__ __forceinline__ float2 exp2_pair(float2 t, int pair) {
  if ((pair & 3) < kExpPolyPairs) return exp2_poly2(t);
  return make_float2(fast_exp2(t.x), fast_exp2(t.y));
}

// DT: 0 = float16, 1 = bfloat16 (a template parameter so that the inner loops convert once, not once per type)
template <int DT> __device__ __forceinline__ uint32_t pack16(float a, float b) {
  return DT == 0 ? Elem<__half>::pack(a, b) : Elem<__nv_bfloat16>::pack(a, b);
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------
// FEAT adds the ALiBi bias and the block mask (reference: mlx_mfa/attention.py:1079-1216 flash_attention_sparse,
// csrc/mfa_steel_fwd.cpp:230-262 the shader's per-tile mask test): a key tile is visited only if one of the mask
// cells under it is set, and partially set tiles are masked by element.  The plain instantiation compiles none of it.
// PERSIST: the CTA stays on its SM and walks items i = blockIdx.x, blockIdx.x + gridDim.x, ... (a query tile of one
// head each) instead of one item per CTA.  TMEM, the barriers and the rings live across items: every phase is counted
// in tiles (g) or items (itn) since the CTA started, the producer requests the next item's Q as soon as the last S
// MMAs of this one have read it and its K tiles as their stages free up, so set-up, launch gaps and load latency are
// paid once per SM instead of once per query tile -- what shapes with few key tiles per query tile (a sliding
// window, short packed sequences) spend a third of their time on otherwise.
// CAPM: 0 = no soft cap, 1 = a cap below kPreciseTanhMinCap (64), 2 = a larger one.  Only the large caps can push the
// bf16 path's upper bound of the row max out of the exponent range, and only for them is tanh.approx too coarse: the
// guard and the two-operation tanh are compiled into that instantiation alone, so the common caps (30, 50) keep the
// lean loop, and the instantiation without a cap carries no tanh code at all (the kernels are sensitive to the size of
// their unrolled loops: measured per variant on the same box).
template <int HD, int DT, bool FEAT, bool PERSIST, int CAPM>
__global__ void __launch_bounds__(kThreads, 2)
fa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                    const Sm100Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kHalves = Cfg<HD>::kHalves, kQBytes = Cfg<HD>::kQBytes, kKVBytes = Cfg<HD>::kKVBytes,
                kSmemTiles = Cfg<HD>::kSmemTiles;
  unsigned char* sQ = smem;
  unsigned char* sK = sQ + kQBytes;
  unsigned char* sV = sK + kStages * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_ntiles = reinterpret_cast<int*>(s_tmem + 2);
  uint16_t* s_list = reinterpret_cast<uint16_t*>(smem + kSmemTiles + 256);     // FEAT only
  unsigned char* s_flag = reinterpret_cast<unsigned char*>(s_list + kMaxListTiles);

  static_assert(!(FEAT && PERSIST), "the feature instantiation keeps per-CTA tile lists: one item per CTA");
  const FwdParams& p = a.p;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // geometry of the current item; the lambdas below read these by reference
  int head, batch, kvh, N, S, q_begin, k_begin, q0, off, kt_begin, kt_end, n_tiles;
  auto item_geometry = [&](int xt, int h, int z, int gx) {
    head = h;
    batch = z;
    kvh = head / p.gqa;
    N = p.N; S = p.S; q_begin = 0; k_begin = 0;
    if (p.cu_q != nullptr) {
      // packed varlen: z is the sequence; rows of the neighbouring sequences that a tile drags in
      // are masked (keys) or simply not stored (queries)
      q_begin = p.cu_q[batch];
      N = p.cu_q[batch + 1] - q_begin;
      k_begin = p.cu_k[batch];
      S = p.cu_k[batch + 1] - k_begin;
      batch = 0;
    } else if (p.kv_lens != nullptr) {
      S = min(max(p.kv_lens[batch], 0), p.S);          // this batch entry's own key count
    }
    q0 = (gx - 1 - xt) * BM;
    off = S - N;
    int k_hi = S;
    if (p.causal) k_hi = min(S, q0 + BM + off);
    int k_lo = 0;
    if (p.window_left >= 0) k_lo = max(0, q0 + off - p.window_left);
    kt_begin = k_lo / BN;
    kt_end = k_hi > 0 ? (k_hi + BN - 1) / BN : 0;
    n_tiles = kt_end - kt_begin;
  };
  const bool paged = p.block_table != nullptr;
  if constexpr (!PERSIST) {
    item_geometry(static_cast<int>(blockIdx.x), static_cast<int>(blockIdx.y), static_cast<int>(blockIdx.z),
                  static_cast<int>(gridDim.x));
    if (q0 >= N) return;
  }
  const bool sparse = FEAT && p.bmask != nullptr;
  if constexpr (FEAT) {
    if (sparse) {
      // every thread tests key tiles (all mask bytes of a tile are fetched at once: no short-circuit, so the loads
      // overlap), then warp 0 compacts the tiles that have a set cell under this query tile
      {
        const int rb0 = q0 / p.bm_bq, rb1 = (min(q0 + BM, N) - 1) / p.bm_bq;
        for (int kt = kt_begin + tid; kt < kt_end; kt += kThreads) {
          const int cb0 = (kt * BN) / p.bm_bk, cb1 = (min((kt + 1) * BN, S) - 1) / p.bm_bk;
          unsigned any = 0u;
          for (int rb = rb0; rb <= rb1; ++rb)
            for (int cb = cb0; cb <= cb1; ++cb) any |= p.bmask[rb * p.bm_nk + cb];
          s_flag[kt - kt_begin] = any != 0u ? 1 : 0;
        }
      }
      __syncthreads();
      if (warp == 0) {
        int count = 0;
        for (int base = kt_begin; base < kt_end; base += 32) {
          const int kt = base + lane;
          const bool on = kt < kt_end && s_flag[kt - kt_begin] != 0;
          const unsigned bal = __ballot_sync(0xffffffffu, on);
          if (on) s_list[count + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(kt);
          count += __popc(bal);
        }
        if (lane == 0) *s_ntiles = count;
      }
      __syncthreads();
      n_tiles = *s_ntiles;
    }
  }
  // j-th key tile this CTA visits
  auto tile_of = [&](int j) -> int {
    if constexpr (FEAT) return sparse ? static_cast<int>(s_list[j]) : kt_begin + j;
    return kt_begin + j;
  };

  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };

  // no visible key for any row of this tile: O = 0, lse = -inf
  auto zero_rows = [&]() {
    if (warp < 4) {
      const int row = q0 + tid;
      if (row < N) {
        uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.o) + batch * p.o_bs + head * p.o_hs +
                                               static_cast<int64_t>(q_begin + row) * p.o_rs);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) orow[i] = make_uint4(0u, 0u, 0u, 0u);
        if (p.lse != nullptr) p.lse[batch * p.lse_bs + head * p.lse_hs + q_begin + row] = -INFINITY;
      }
    }
  };
  if constexpr (!PERSIST) {
    if (n_tiles <= 0) {
      zero_rows();
      return;
    }
  }

  // Paged pools: first pool token of each 16-token unit of the j-th tile (a page is page_size / 16 units).  Units
  // whose table entry is missing, negative or beyond the pool, and units past the sequence's end, point at the first
  // row beyond the pool: TMA delivers zeros (and the full byte count) for it.
  struct UnitToks { int t[BN / 16]; };
  auto unit_toks = [&](int j) -> UnitToks {
    UnitToks u;
    const int upp = p.page_size >> 4;
    const int oob = p.num_pages * p.page_size;
    const int32_t* row = p.block_table + static_cast<int64_t>(batch) * p.max_blocks;
#pragma unroll
    for (int i = 0; i < BN / 16; ++i) {
      const int unit = tile_of(j) * (BN / 16) + i;
      const int blk = unit / upp;
      int page = -1;
      if (unit * 16 < S && blk < p.max_blocks) page = __ldg(row + blk);
      u.t[i] = (page >= 0 && page < p.num_pages) ? page * p.page_size + (unit % upp) * 16 : oob;
    }
    return u;
  };
  auto load_paged = [&](unsigned char* dst, const CUtensorMap* tm, uint32_t b, const UnitToks& u) {
#pragma unroll
    for (int i = 0; i < BN / 16; ++i)
#pragma unroll
      for (int hf = 0; hf < kHalves; ++hf)
        tma_load_4d(smem_u32(dst + hf * (kKVBytes / kHalves) + i * 2048), tm, b, 64 * hf, u.t[i], kvh, 0);
  };
  // The producer thread sets up the barriers and starts the first loads (Q and as many K / V tiles as there are
  // stages, all of which are empty) before the CTA-wide sync, so TMEM allocation and the sync hide under them.
  // st: ring stage = parity of the tile's running count since the CTA started
  auto load_k = [&](int j, int st, const UnitToks& u) {
    mbar_arrive_expect_tx(bar(BAR_K_FULL + st), kKVBytes);
    if (paged) {
      load_paged(sK + st * kKVBytes, &tmK, bar(BAR_K_FULL + st), u);
      return;
    }
#pragma unroll
    for (int hf = 0; hf < kHalves; ++hf)
      tma_load_4d(smem_u32(sK + st * kKVBytes + hf * (kKVBytes / kHalves)), &tmK, bar(BAR_K_FULL + st), 64 * hf,
                  k_begin + tile_of(j) * BN, kvh, batch);
  };
  auto load_v = [&](int j, int st, const UnitToks& u) {
    mbar_arrive_expect_tx(bar(BAR_V_FULL + st), kKVBytes);
    if (paged) {
      load_paged(sV + st * kKVBytes, &tmV, bar(BAR_V_FULL + st), u);
      return;
    }
#pragma unroll
    for (int hf = 0; hf < kHalves; ++hf)
      tma_load_4d(smem_u32(sV + st * kKVBytes + hf * (kKVBytes / kHalves)), &tmV, bar(BAR_V_FULL + st), 64 * hf,
                  k_begin + tile_of(j) * BN, kvh, batch);
  };
  if (warp == 4 && lane == 0) {
    mbar_init(bar(BAR_Q), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(BAR_K_FULL + s), 1);
      mbar_init(bar(BAR_V_FULL + s), 1);
      mbar_init(bar(BAR_PV_DONE + s), 1);
      mbar_init(bar(BAR_S_FULL + s), 1);
      mbar_init(bar(BAR_P_FULL + s), 4);     // one arrive per softmax warp
    }
    mbar_init(bar(BAR_O_STAGED), 4);
    mbar_init(bar(BAR_O_FINAL), 1);
    mbar_init(bar(BAR_Q_FREE), 1);
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async();
    if constexpr (!PERSIST) {
      mbar_arrive_expect_tx(bar(BAR_Q), kQBytes);
#pragma unroll
      for (int hf = 0; hf < kHalves; ++hf)
        tma_load_4d(smem_u32(sQ + hf * (kQBytes / kHalves)), &tmQ, bar(BAR_Q), 64 * hf, q_begin + q0, head, batch);
      for (int j = 0; j < kStages && j < n_tiles; ++j) {
        UnitToks u = {};
        if (paged) u = unit_toks(j);
        load_k(j, j & 1, u);
        load_v(j, j & 1, u);
      }
    }
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(s_tmem), tmem_cols<HD>());
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tS0 = tmem, tO = tmem + 128;   // S buffers at +0 and +64, O (HD columns) at +128

  // Persistent CTAs: the O tile leaves through the V stages (free once the item's last P.V has completed) and a TMA
  // store that the producer thread issues: it is the one that needs those stages next, and the softmax warps move on at
  // once.  One item per CTA: through the Q buffer, stored by the first softmax thread.
  auto store_o = [&](uint32_t parity, int q0_, int head_, int batch_) {
    if (mbar_wait_bounded(bar(BAR_O_STAGED), parity, s_abort)) {
#pragma unroll
      for (int hf = 0; hf < kHalves; ++hf)
        tma_store_4d(&tmO, smem_u32(sV + hf * (kQBytes / kHalves)), 64 * hf, q0_, head_, batch_);
      tma_store_commit();
      tma_store_wait_read<0>();        // the copies have left shared memory; the kernel's end makes them visible
    }
  };

  int g0 = 0, itn = 0;       // key tiles and items this CTA has been through: every barrier phase counts from them
  int prev_q0 = 0, prev_head = 0, prev_batch = 0;
  const int n_items = PERSIST ? a.total_items : 1;
  for (int it = PERSIST ? static_cast<int>(blockIdx.x) : 0; it < n_items; it += PERSIST ? static_cast<int>(gridDim.x) : 1) {
  if constexpr (PERSIST) {
    item_geometry(it % a.gx, (it / a.gx) % a.gy, it / (a.gx * a.gy), a.gx);
    if (q0 >= N) continue;
    if (n_tiles <= 0) {
      zero_rows();
      continue;
    }
  }

  if (warp == 4) {
    // ============================ producer ============================
    if (lane == 0) {
      bool okp = true;
      if constexpr (PERSIST) {
        // Q of this item may land once the previous item's S MMAs have read theirs
        if (itn > 0) okp = mbar_wait_bounded(bar(BAR_Q_FREE), (itn - 1) & 1, s_abort);
        if (okp) {
          mbar_arrive_expect_tx(bar(BAR_Q), kQBytes);
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf)
            tma_load_4d(smem_u32(sQ + hf * (kQBytes / kHalves)), &tmQ, bar(BAR_Q), 64 * hf, q_begin + q0, head, batch);
        }
      }
      // paged: the table entries of a tile are fetched one tile ahead, so that their latency passes under the wait
      // for the stage
      constexpr int j_first = PERSIST ? 0 : kStages;     // one item per CTA: the first tiles were requested before the sync
      UnitToks u_next = {};
      if (paged && j_first < n_tiles) u_next = unit_toks(j_first);
      for (int j = j_first; j < n_tiles && okp; ++j) {
        const int g = g0 + j, st = g & 1;
        const uint32_t par = ((g >> 1) & 1) ^ 1;
        const UnitToks u = u_next;
        if (paged && j + 1 < n_tiles) u_next = unit_toks(j + 1);
        // K(g) and V(g) reuse the stage of tile g-2: wait until its S MMAs, then its PV MMAs, have read it.  These
        // are the barriers the softmax warps wait on too: every commit costs the MMA thread a bubble, so one commit
        // serves both readers.  Neither can be more than one completion ahead of this thread: S(g) needs K(g) and
        // P.V(g) needs V(g), which are loaded below.
        if (g >= kStages && !mbar_wait_bounded(bar(BAR_S_FULL + st), par, s_abort)) break;
        load_k(j, st, u);
        if (g >= kStages && !mbar_wait_bounded(bar(BAR_PV_DONE + st), par, s_abort)) break;
        if constexpr (PERSIST) {
          // the V stages hold the previous item's staged O tile until its store has read them
          if (j == 0 && itn > 0 && a.tma_store) store_o((itn - 1) & 1, prev_q0, prev_head, prev_batch);
        }
        load_v(j, st, u);
      }
    }
  } else if (warp == 5) {
    // ============================ MMA issue ============================
    if (lane == 0) {
      const uint32_t idesc_qk = instr_desc(DT, 0, BM, BN);
      const uint32_t idesc_pv = instr_desc(DT, 1, BM, HD);
      // Descriptors differ only in their start-address field (low word); build the bases once so that
      // the issue loop is a handful of integer adds per MMA.
      const uint64_t qd = smem_desc(smem_u32(sQ), 16, 1024);
      const uint64_t kd0 = smem_desc(smem_u32(sK), 16, 1024);
      const uint64_t vd0 = smem_desc(smem_u32(sV), kKVBytes / kHalves, 1024);
      constexpr uint64_t kHalfQ = (kQBytes / kHalves) >> 4, kHalfK = (kKVBytes / kHalves) >> 4, kStageKV = kKVBytes >> 4;
      bool ok = mbar_wait_bounded(bar(BAR_Q), itn & 1, s_abort);
      auto issue_s = [&](int j) -> bool {
        const int g = g0 + j, st = g & 1;
        if (!mbar_wait_bounded(bar(BAR_K_FULL + st), (g >> 1) & 1, s_abort)) return false;
        tc_fence_after();
        const uint64_t kd = kd0 + static_cast<uint64_t>(st) * kStageKV;
        const uint32_t d_tmem = tS0 + st * 64;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          // K-major operands: 64-wide halves of [rows][128 B]; a k-step of 16 elements is 32 B (2 units) inside the swizzle row
          mma_ss(d_tmem, qd + (k >> 2) * kHalfQ + (k & 3) * 2, kd + (k >> 2) * kHalfK + (k & 3) * 2, idesc_qk,
                 k > 0 ? 1u : 0u);
        }
        tc_commit(bar(BAR_S_FULL + st));        // for the softmax warps and for the producer
        if constexpr (PERSIST) {
          if (j + 1 == n_tiles) tc_commit(bar(BAR_Q_FREE));   // nothing of this item reads Q any more
        }
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = g0 + j, st = g & 1;
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        // V landed long ago; wait for it first so that nothing but the MMA issue follows the arrival of P
        if (!mbar_wait_bounded(bar(BAR_V_FULL + st), (g >> 1) & 1, s_abort)) { ok = false; break; }
        if (!mbar_wait_bounded(bar(BAR_P_FULL + st), (g >> 1) & 1, s_abort)) { ok = false; break; }
        tc_fence_after();
        const uint64_t vd = vd0 + static_cast<uint64_t>(st) * kStageKV;
        const uint32_t a_tmem = tS0 + st * 64;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // B = V, MN-major: [half][key][64 d]; 8-key groups 1024 B apart, d-halves kKVBytes/2 apart;
          // a k-step is 16 keys = 2048 B (128 units).  A = P in TMEM: 16 16-bit values = 8 columns per k-step.
          mma_ts(tO, a_tmem + k * 8, vd + k * 128, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar(BAR_PV_DONE + st));       // for the softmax warps' rescale and for the producer
        if (j + 1 == n_tiles) tc_commit(bar(BAR_O_FINAL));
      }
    }
  } else {
    // ============================ softmax (warps 0-3) ============================
    const int row = q0 + tid;                         // query row of this thread
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    constexpr bool BIGCAP = CAPM == 2;
    constexpr bool use_cap = CAPM != 0;
    const float cap_in = use_cap ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;

    // softcap on: t = x * (kk + kb3 z + kb5 z^2 + kb7 z^3), z = x^2, is cap*log2(e)*tanh(x*scale/cap) to degree 7
    const float kk = cap_in * cap_out;                // scale * log2(e)
    const float c2 = cap_in * cap_in;
    const float kb3 = kk * (-1.f / 3.f) * c2, kb5 = kk * (2.f / 15.f) * c2 * c2, kb7 = kk * (-17.f / 315.f) * c2 * c2 * c2;
    // largest |y| for which the degree-3 / degree-5 polynomial is within 1e-3 / cap of tanh(y)
    const float y_deg3 = use_cap ? fminf(0.5f, powf(1e-3f * 7.5f / p.softcap, 0.2f)) : 0.f;
    const float y_deg5 = use_cap ? fminf(0.5f, powf(1e-3f * (315.f / 17.f) / p.softcap, 1.f / 7.f)) : 0.f;
    // ... and the degree-7 one within 2e-3 / cap (0.497 at cap 50); beyond it tanh itself is evaluated
    const float y_deg7 = BIGCAP ? fminf(0.5f, powf(2e-3f * (2835.f / 62.f) / p.softcap, 1.f / 9.f)) : 0.5f;
    constexpr bool precise_tanh = BIGCAP;
    const bool monotone = p.scale > 0.f;              // lets the row max be taken on the raw dot products
    const float alibi_l2 = (FEAT && p.alibi != nullptr) ? p.alibi[head] * kLog2e : 0.f;

    // FEAT: bit c = mask cell c of this row's block row under the key tile starting at k0
    // (cells are 16, 32 or 64 keys wide: shifts, and the row's mask line, are worked out once)
    const int cell_sh = (FEAT && sparse) ? (p.bm_bk == 16 ? 4 : (p.bm_bk == 32 ? 5 : 6)) : 6;
    const int ncell = BN >> cell_sh;
    const unsigned full_cells = (1u << ncell) - 1u;
    const uint8_t* mask_row = (FEAT && sparse) ? p.bmask + static_cast<int64_t>(min(row, N - 1) / p.bm_bq) * p.bm_nk : nullptr;
    auto row_cells = [&](int k0) -> unsigned {
      const int cb0 = k0 >> cell_sh;
      unsigned c4 = 0u;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c < ncell && cb0 + c < p.bm_nk && mask_row[cb0 + c] != 0) c4 |= 1u << c;
      return c4;
    };
    unsigned cells_next = 0xffffffffu;
    if constexpr (FEAT) {
      if (sparse) cells_next = row_cells(tile_of(0) * BN);
    }

    for (int j = 0; j < n_tiles; ++j) {
      const int g = g0 + j, st = g & 1;
      const int k0 = tile_of(j) * BN;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_S_FULL + st), (g >> 1) & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld32(tS0 + lane_base + st * 64, r0);
      tmem_ld32(tS0 + lane_base + st * 64 + 32, r1);
      tc_wait_ld();
      float x[BN];                                     // raw q.k of this row
#pragma unroll
      for (int i = 0; i < 32; ++i) { x[i] = __uint_as_float(r0[i]); x[32 + i] = __uint_as_float(r1[i]); }

      unsigned cells = 0xffffffffu;                   // FEAT: set mask cells of this row under the tile
      bool cells_partial = false;
      if constexpr (FEAT) {
        if (sparse) {
          // fetched one tile ahead, so that the mask bytes' latency hides under the previous tile's work
          cells = cells_next;
          cells_partial = __any_sync(0xffffffffu, cells != full_cells);
          if (j + 1 < n_tiles) cells_next = row_cells(tile_of(j + 1) * BN);
        }
      }
      const bool need_mask = (k0 + BN > S) || (p.causal && (k0 + BN - 1 > q0 + off)) ||
                             (p.window_left >= 0 && (k0 < q0 + BM - 1 + off - p.window_left)) || cells_partial;
      const bool fast = !need_mask && monotone && !(FEAT && p.alibi != nullptr);
      // mode 0: t = x*scale_log2 - m ; 1: softcap by polynomial ; 2: softcap by tanh.approx ; 3: general (masked tile)
      int mode = 3;
      unsigned deg = 2;                                // mode 1 only: 0, 1, 2 = polynomial of degree 3, 5, 7
      float m_tile;
      if (fast) {
        // scale and softcap are increasing in x, so the tile max is f(max x): one pass of 3-input max
        if (!use_cap) {
          mode = 0;
          m_tile = tree_max64(x) * p.scale_log2;
        } else {
          // cap*tanh(y), y = x*scale/cap: the odd Taylor polynomial of tanh runs on the FMA pipe and leaves the
          // special-function unit to exp2.  Its degree (3, 5 or 7) is the lowest whose truncation error, times
          // cap, stays below 1e-3 (2e-3 for degree 7) for the largest |y| among the warp's rows; above that range
          // (|y| = 0.5 at most) tanh itself is evaluated.
          // bf16: one tree over |x| serves both the range check and the reference max -- f(max|x|) is an upper
          // bound of the row max, at most 2*cap*log2(e)*|y| binades above it.  That is harmless while the bound
          // stays inside the exponent range P is computed in (ex2.approx.ftz flushes below 2^-126): up to 96
          // binades it is used as it stands (softcap 50 never exceeds 72); beyond, the warp takes the exact max with
          // a second tree, as fp16 always does (its P would underflow much earlier).
          float xmax, ax;
          if (DT == 1) {
            ax = tree_absmax64(x);
            xmax = ax;
          } else {
            xmax = tree_max64(x);
            ax = fmaxf(xmax, -tree_min64(x));
          }
          const float ay = ax * cap_in;
          // one warp-wide OR carries both answers: the highest polynomial level any row needs (one-hot in bits 0-3) and
          // whether any row's bound leaves the exponent range (bit 4)
          unsigned lvl;
          if constexpr (BIGCAP) {
            const unsigned code = (ay <= y_deg3 ? 1u : (ay <= y_deg5 ? 2u : (ay <= y_deg7 ? 4u : 8u))) |
                                  ((DT == 1 && 2.f * cap_out * ay > 96.f) ? 16u : 0u);
            const unsigned all = __reduce_or_sync(0xffffffffu, code);
            lvl = (all & 8u) ? 3u : ((all & 4u) ? 2u : ((all & 2u) ? 1u : 0u));
            if (DT == 1 && (all & 16u)) xmax = tree_max64(x);
          } else {
            // caps below 64: the bound is at most 2 * 64 * log2(e) * 0.5 = 92 binades above the row max, inside the range
            lvl = __reduce_max_sync(0xffffffffu, ay <= y_deg3 ? 0u : (ay <= y_deg5 ? 1u : (ay <= y_deg7 ? 2u : 3u)));
          }
          if (lvl < 3u) {
            mode = 1;
            deg = lvl;
            const float z = xmax * xmax;
            const float q = lvl == 0u ? fmaf(z, kb3, kk) : (lvl == 1u ? fmaf(z, fmaf(z, kb5, kb3), kk) : fmaf(z, fmaf(z, fmaf(z, kb7, kb5), kb3), kk));
            m_tile = xmax * q;
          } else {
            mode = 2;
            if (DT == 1) xmax = tree_max64(x);          // scores may saturate here: take the exact max
            m_tile = cap_out * cap_tanh(xmax * cap_in, precise_tanh);
          }
        }
      } else {
        // without softcap or bias a masked tile keeps the raw dot products: the mask writes -inf, the max is taken
        // on them and mode 0 folds the scale into the exponent's FMA as on an unmasked tile
        const bool raw = !use_cap && monotone && !(FEAT && p.alibi != nullptr);
        if (use_cap) {
          if (precise_tanh) {
#pragma unroll
            for (int i = 0; i < BN; ++i) x[i] = cap_out * tanh_exp(x[i] * cap_in);
          } else {
#pragma unroll
            for (int i = 0; i < BN; ++i) x[i] = cap_out * fast_tanh(x[i] * cap_in);
          }
        } else if (!raw) {
#pragma unroll
          for (int i = 0; i < BN; ++i) x[i] *= p.scale_log2;
        }
        if constexpr (FEAT) {
          if (p.alibi != nullptr) {
            // slope * (key - query position), in the log2 domain like the scores
            const float base = alibi_l2 * static_cast<float>(k0 - (row + off));
#pragma unroll
            for (int i = 0; i < BN; ++i) x[i] += fmaf(alibi_l2, static_cast<float>(i), base);
          }
        }
        if (need_mask) {
          // first / last visible column of this row in tile coordinates; a tile usually crosses only one of the
          // two edges (the diagonal or the end of the keys on the right, the window on the left)
          const int hi_rel = (p.causal ? min(S - 1, row + off) : S - 1) - k0;
          const int lo_rel = (p.window_left >= 0 ? row + off - p.window_left : 0) - k0;
          const bool cut_hi = (k0 + BN > S) || (p.causal && (k0 + BN - 1 > q0 + off));
          const bool cut_lo = p.window_left >= 0 && (k0 < q0 + BM - 1 + off - p.window_left);
          if (cut_hi) {
#pragma unroll
            for (int i = 0; i < BN; ++i)
              if (i > hi_rel) x[i] = -INFINITY;
          }
          if (cut_lo) {
#pragma unroll
            for (int i = 0; i < BN; ++i)
              if (i < lo_rel) x[i] = -INFINITY;
          }
          if constexpr (FEAT) {
            if (cells_partial) {
#pragma unroll
              for (int i = 0; i < BN; ++i)
                if (!((cells >> (i >> cell_sh)) & 1u)) x[i] = -INFINITY;
            }
          }
        }
        m_tile = tree_max64(x);
        if (raw) {
          mode = 0;
          m_tile *= p.scale_log2;                      // -inf (a fully masked row) stays -inf: the scale is positive
        }
      }

      // lazy rescale: keep the old reference max unless the row max grew by more than 2^8
      const bool need = m_tile > m_used + 8.f;
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = fmaxf(m_used, m_tile);
        const float corr = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);
        l_run *= corr;
        if (j > 0) {
          // O is being accumulated by PV(j-1): wait for it, then scale this row in TMEM
          // P.V(j-1): completion (j-1)>>1 of its stage's barrier; the next one there needs this tile's successor's P
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1, s_abort))) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + lane_base + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st32(tO + lane_base + c * 32, o);
          }
        }
        m_used = m_new;
      }
      const float msub = (m_used == -INFINITY) ? 0.f : m_used;
      const float2 nm2 = make_float2(-msub, -msub);
      float2 lsum2 = make_float2(0.f, 0.f);
      uint32_t pk[32];
      if (mode == 0) {
        const float2 k2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int i = 0; i < BN; i += 2) {
          const float2 t = __ffma2_rn(make_float2(x[i], x[i + 1]), k2, nm2);
          const float2 e = exp2_pair(t, i >> 1);
          lsum2 = __fadd2_rn(lsum2, e);
          pk[i >> 1] = pack16<DT>(e.x, e.y);
        }
      } else if (mode == 1) {
        const float2 kk2 = make_float2(kk, kk), b32 = make_float2(kb3, kb3), b52 = make_float2(kb5, kb5),
                     b72 = make_float2(kb7, kb7);
        if (deg == 0u) {
#pragma unroll
          for (int i = 0; i < BN; i += 2) {
            const float2 xv = make_float2(x[i], x[i + 1]);
            const float2 q = __ffma2_rn(__fmul2_rn(xv, xv), b32, kk2);
            const float2 t = __ffma2_rn(xv, q, nm2);
            const float2 e = exp2_pair(t, i >> 1);
            lsum2 = __fadd2_rn(lsum2, e);
            pk[i >> 1] = pack16<DT>(e.x, e.y);
          }
        } else if (deg == 1u) {
#pragma unroll
          for (int i = 0; i < BN; i += 2) {
            const float2 xv = make_float2(x[i], x[i + 1]);
            const float2 z = __fmul2_rn(xv, xv);
            const float2 q = __ffma2_rn(z, __ffma2_rn(z, b52, b32), kk2);
            const float2 t = __ffma2_rn(xv, q, nm2);
            const float2 e = exp2_pair(t, i >> 1);
            lsum2 = __fadd2_rn(lsum2, e);
            pk[i >> 1] = pack16<DT>(e.x, e.y);
          }
        } else {
#pragma unroll
          for (int i = 0; i < BN; i += 2) {
            const float2 xv = make_float2(x[i], x[i + 1]);
            const float2 z = __fmul2_rn(xv, xv);
            const float2 q = __ffma2_rn(z, __ffma2_rn(z, __ffma2_rn(z, b72, b52), b32), kk2);
            const float2 t = __ffma2_rn(xv, q, nm2);
            const float2 e = exp2_pair(t, i >> 1);
            lsum2 = __fadd2_rn(lsum2, e);
            pk[i >> 1] = pack16<DT>(e.x, e.y);
          }
        }
      } else if (mode == 2) {
        if (precise_tanh) {
#pragma unroll
          for (int i = 0; i < BN; i += 2) {
            const float2 e = make_float2(fast_exp2(fmaf(cap_out, tanh_exp(x[i] * cap_in), -msub)),
                                         fast_exp2(fmaf(cap_out, tanh_exp(x[i + 1] * cap_in), -msub)));
            lsum2 = __fadd2_rn(lsum2, e);
            pk[i >> 1] = pack16<DT>(e.x, e.y);
          }
        } else {
#pragma unroll
          for (int i = 0; i < BN; i += 2) {
            const float2 e = make_float2(fast_exp2(fmaf(cap_out, fast_tanh(x[i] * cap_in), -msub)),
                                         fast_exp2(fmaf(cap_out, fast_tanh(x[i + 1] * cap_in), -msub)));
            lsum2 = __fadd2_rn(lsum2, e);
            pk[i >> 1] = pack16<DT>(e.x, e.y);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < BN; i += 2) {
          const float2 e = make_float2(fast_exp2(x[i] - msub), fast_exp2(x[i + 1] - msub));
          lsum2 = __fadd2_rn(lsum2, e);
          pk[i >> 1] = pack16<DT>(e.x, e.y);
        }
      }
      l_run += lsum2.x + lsum2.y;
      // P(j) overwrites the first 32 columns of S(j): lane = row, column c = keys (2c, 2c+1)
      tmem_st32(tS0 + lane_base + st * 64, pk);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_P_FULL + st));
    }

    // ---- epilogue: O / l -> global, lse ----
    // O is complete when the barrier committed after the last P.V fires.  It is used once per CTA, so its parity
    // cannot alias: PV_DONE would not do here, because a warp may reach this point two completions ahead of it
    // (S(n-1) complete only implies PV(n-3)) or after both have happened, and a parity wait is only sound within one
    // phase of the barrier.
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_O_FINAL), itn & 1, s_abort));
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      if (a.tma_store) {
        // Stage the tile in the Q buffer (free: every S MMA has completed; persistent CTAs, whose next Q may already
        // be landing there, use the V stages: every P.V has completed) as two 64-wide 128B-swizzled halves and
        // let TMA write it: full-line stores instead of 32 rows x 16 bytes per instruction; rows beyond N are
        // clipped by the tensor map.
        unsigned char* stage = PERSIST ? sV : sQ;
        const int r = tid;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + lane_base + c * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack16<DT>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            v.y = pack16<DT>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            v.z = pack16<DT>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            v.w = pack16<DT>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            const int chunk = c * 4 + (i >> 3);              // 16-byte chunk of the row: half = chunk / 8
            unsigned char* dst = stage + (chunk >> 3) * (kQBytes / kHalves) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = v;
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_O_STAGED));          // persistent CTAs: the producer thread issues the store
        if constexpr (!PERSIST) {
          if (tid == 0 && mbar_wait_bounded(bar(BAR_O_STAGED), 0, s_abort)) {
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf)
              tma_store_4d(&tmO, smem_u32(sQ + hf * (kQBytes / kHalves)), 64 * hf, q0, head, batch);
            tma_store_commit();
            tma_store_wait<0>();
          }
        }
      } else {
        uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + batch * p.o_bs + head * p.o_hs +
                         static_cast<int64_t>(q_begin + row) * p.o_rs;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + lane_base + c * 32, o);
          tc_wait_ld();
          if (row < N) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack16<DT>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              v.y = pack16<DT>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              v.z = pack16<DT>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              v.w = pack16<DT>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
            }
          }
        }
      }
      if (p.lse != nullptr && row < N)
        p.lse[batch * p.lse_bs + head * p.lse_hs + q_begin + row] = l_run > 0.f ? m_used + log2f(l_run) : -INFINITY;
    }
  }

  prev_q0 = q0; prev_head = head; prev_batch = batch;
  g0 += n_tiles;
  ++itn;
  if (*s_abort != 0) break;
  }  // items

  if constexpr (PERSIST) {
    // the last item's O tile
    if (warp == 4 && lane == 0 && itn > 0 && a.tma_store && *s_abort == 0) store_o((itn - 1) & 1, prev_q0, prev_head, prev_batch);
  }

  // ---- teardown: everyone meets, then the allocating warp frees TMEM ----
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, tmem_cols<HD>());
  }
  if (tid == 0 && *s_abort != 0) atomicOr(&g_kernel_status, 1);
}

bool make_map(CUtensorMap* m, int dtype, const void* base, int D, int rows, int H, int B, int64_t rs, int64_t hs,
              int64_t bs, int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(rows), static_cast<uint64_t>(H),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(rs) * 2, static_cast<uint64_t>(hs) * 2, static_cast<uint64_t>(bs) * 2};
  const uint32_t box[4] = {64, static_cast<uint32_t>(box_rows), 1, 1};
  return encode_tmap(m, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims,
                     strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

bool fwd_sm100_supported(const FwdParams& p, int dtype, int D) {
  if (!(dtype == 0 || dtype == 1) || !(D == 64 || D == 128 || D == 256)) return false;
  // head_dim 256: one CTA per SM (192 KB of tiles, 384 TMEM columns); no bias / block-mask instantiation
  if (D == 256 && (p.alibi != nullptr || p.bmask != nullptr)) return false;
  if (p.N <= 0 || p.S <= 0 || p.B <= 0) return false;
  // A broadcast (stride 0) batch or head dimension of extent > 1 cannot be described to TMA, whose strides must be
  // positive; such views run the portable kernel, which indexes with the caller's strides as they are.
  if ((p.B > 1 && (p.q_bs == 0 || p.k_bs == 0 || p.v_bs == 0 || p.o_bs == 0)) ||
      (p.Hq > 1 && (p.q_hs == 0 || p.o_hs == 0)) || (p.Hkv > 1 && (p.k_hs == 0 || p.v_hs == 0)))
    return false;
  if (p.block_table != nullptr) {
    // paged K / V: dense queries only, pages of a multiple of 16 tokens, no bias / block mask
    if (p.cu_q != nullptr || p.alibi != nullptr || p.bmask != nullptr) return false;
    if (p.page_size < 16 || p.page_size % 16 != 0 || p.num_pages <= 0 || p.max_blocks <= 0) return false;
    if (static_cast<int64_t>(p.num_pages) * p.page_size >= (1LL << 31)) return false;
  }
  if (p.kv_lens != nullptr && p.cu_q != nullptr) return false;
  if (p.bmask != nullptr) {
    // mask cells must tile the 64-key tiles, and the active-tile list holds 16-bit indices of at most kMaxListTiles
    if (!(p.bm_bk == 16 || p.bm_bk == 32 || p.bm_bk == 64) || p.bm_bq <= 0) return false;
    if ((p.S + BN - 1) / BN > kMaxListTiles) return false;
  }
  return get_encode_tiled() != nullptr;
}

// Persistent CTAs pay off where set-up, launch gaps and the first loads' latency are a visible part of a CTA's life
// and the items are many and short: packed sequences (config 5's forward: 0.889 -> 0.837 ms; ten unmasked key tiles per
// query tile: +6 %).  They do not for a sliding window (config 3: -2.5 %: its query tiles are bounded by the fill and
// drain of the S -> softmax -> P.V pipeline, which a persistent CTA pays per item just the same) and they lose where
// items are long and uneven (config 2: 2.23 -> 2.74 ms with the static deal), which keep one CTA per item and the
// hardware scheduler's balancing.  `mode`: 0 = choose, 1 = persistent, 2 = one item per CTA (descriptor flags).
static bool want_persistent(const FwdParams& p, int nbatch, int max_q, int sm_count, int mode) {
  if (mode != 0) return mode == 1;
  const long long items = static_cast<long long>((max_q + BM - 1) / BM) * p.Hq * nbatch;
  return p.cu_q != nullptr && p.window_left < 0 && items >= 8LL * 2 * sm_count && max_q <= 64 * BM;
}

template <int HD, int DT, bool FEAT>
static cudaError_t launch_hd(const FwdParams& p, int nbatch, int max_q, cudaStream_t stream) {
  constexpr int dtype = DT;
  CUtensorMap tmQ, tmK, tmV, tmO;
  // TMA: a size-1 dimension still needs a legal stride (extents > 1 have positive strides: fwd_sm100_supported)
  auto fix = [](int64_t s, int64_t fallback) { return s > 0 ? s : fallback; };
  const int64_t q_hs = fix(p.q_hs, static_cast<int64_t>(p.N) * p.q_rs), q_bs = fix(p.q_bs, q_hs * p.Hq);
  const int64_t k_hs = fix(p.k_hs, static_cast<int64_t>(p.S) * p.k_rs), k_bs = fix(p.k_bs, k_hs * p.Hkv);
  const int64_t v_hs = fix(p.v_hs, static_cast<int64_t>(p.S) * p.v_rs), v_bs = fix(p.v_bs, v_hs * p.Hkv);
  if (!make_map(&tmQ, dtype, p.q, HD, p.N, p.Hq, p.B, p.q_rs, q_hs, q_bs, BM)) return cudaErrorInvalidValue;
  if (p.block_table != nullptr) {
    // pools [num_pages, page_size, Hkv, D] seen as [1][Hkv][num_pages * page_size tokens][D]; boxes of 16 tokens
    const int tokens = p.num_pages * p.page_size;
    const int64_t tok_stride = static_cast<int64_t>(p.Hkv) * HD;
    if (!make_map(&tmK, dtype, p.k, HD, tokens, p.Hkv, 1, tok_stride, HD, tok_stride * tokens, 16) ||
        !make_map(&tmV, dtype, p.v, HD, tokens, p.Hkv, 1, tok_stride, HD, tok_stride * tokens, 16))
      return cudaErrorInvalidValue;
  } else if (!make_map(&tmK, dtype, p.k, HD, p.S, p.Hkv, p.B, p.k_rs, k_hs, k_bs, BN) ||
             !make_map(&tmV, dtype, p.v, HD, p.S, p.Hkv, p.B, p.v_rs, v_hs, v_bs, BN)) {
    return cudaErrorInvalidValue;
  }
  Sm100Args a;
  a.p = p;
  // dense outputs go out by TMA; packed sequences share rows of one tensor, so their tiles are stored row by row
  const int64_t o_hs = fix(p.o_hs, static_cast<int64_t>(p.N) * p.o_rs), o_bs = fix(p.o_bs, o_hs * p.Hq);
  a.tma_store = (p.cu_q == nullptr && make_map(&tmO, dtype, p.o, HD, p.N, p.Hq, p.B, p.o_rs, o_hs, o_bs, BM)) ? 1 : 0;
  if (!a.tma_store) tmO = tmQ;
  constexpr int smem_bytes = FEAT ? Cfg<HD>::kSmemBytesFeat : Cfg<HD>::kSmemBytes;
  dim3 grid((max_q + BM - 1) / BM, p.Hq, nbatch);
  a.gx = static_cast<int>(grid.x);
  a.gy = static_cast<int>(grid.y);
  const int capm = p.softcap >= kPreciseTanhMinCap ? 2 : (p.softcap > 0.f ? 1 : 0);
  const long long items = static_cast<long long>(grid.x) * grid.y * grid.z;
  a.total_items = static_cast<int>(items < 0x7fffffffLL ? items : 0x7fffffffLL);
  if constexpr (!FEAT && HD <= 128) {
    int dev = 0, sm_count = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sm_count <= 0)
      sm_count = 148;
    if (items < 0x7fffffffLL && want_persistent(p, nbatch, max_q, sm_count, a.p.persist_mode)) {
      const int ctas = static_cast<int>(items < 2LL * sm_count ? items : 2LL * sm_count);     // two CTAs per SM
      auto launch_p = [&](auto kern) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        kern<<<ctas, kThreads, smem_bytes, stream>>>(tmQ, tmK, tmV, tmO, a);
        return cudaGetLastError();
      };
      return capm == 2 ? launch_p(fa_fwd_sm100_kernel<HD, DT, false, true, 2>)
                       : (capm == 1 ? launch_p(fa_fwd_sm100_kernel<HD, DT, false, true, 1>) : launch_p(fa_fwd_sm100_kernel<HD, DT, false, true, 0>));
    }
  }
  auto launch_1 = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<grid, kThreads, smem_bytes, stream>>>(tmQ, tmK, tmV, tmO, a);
    return cudaGetLastError();
  };
  return capm == 2 ? launch_1(fa_fwd_sm100_kernel<HD, DT, FEAT, false, 2>)
                   : (capm == 1 ? launch_1(fa_fwd_sm100_kernel<HD, DT, FEAT, false, 1>) : launch_1(fa_fwd_sm100_kernel<HD, DT, FEAT, false, 0>));
}

// Dense: nbatch = B, max_q = N.  Packed varlen (p.cu_q set, B == 1, N/S = total tokens): nbatch = number of
// sequences, max_q = longest query sequence.
cudaError_t launch_fwd_sm100(const FwdParams& p, int dtype, int D, int nbatch, int max_q, cudaStream_t stream) {
  if (nbatch <= 0 || max_q <= 0) return cudaSuccess;
  if (p.alibi != nullptr || p.bmask != nullptr) {
    if (D == 64)
      return dtype == 0 ? launch_hd<64, 0, true>(p, nbatch, max_q, stream) : launch_hd<64, 1, true>(p, nbatch, max_q, stream);
    return dtype == 0 ? launch_hd<128, 0, true>(p, nbatch, max_q, stream) : launch_hd<128, 1, true>(p, nbatch, max_q, stream);
  }
  if (D == 64)
    return dtype == 0 ? launch_hd<64, 0, false>(p, nbatch, max_q, stream) : launch_hd<64, 1, false>(p, nbatch, max_q, stream);
  if (D == 256)
    return dtype == 0 ? launch_hd<256, 0, false>(p, nbatch, max_q, stream) : launch_hd<256, 1, false>(p, nbatch, max_q, stream);
  return dtype == 0 ? launch_hd<128, 0, false>(p, nbatch, max_q, stream) : launch_hd<128, 1, false>(p, nbatch, max_q, stream);
}

cudaError_t fwd_sm100_read_clear_status(cudaStream_t stream, int* out) {
  const int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_kernel_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess && *out != 0)
    e = cudaMemcpyToSymbolAsync(g_kernel_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return e;
}

}  // namespace b200fa
