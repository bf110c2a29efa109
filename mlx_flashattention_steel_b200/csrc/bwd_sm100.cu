// Blackwell backward main kernel (head_dim 64, 16-bit): tcgen05 MMAs with every accumulator in TMEM.
// Same mathematics as bwd_mma.cu (reference: csrc/mfa_steel_bwd.cpp:284-745, 765-1293); the preprocess
// (delta, dQ accumulator reset) and the final dQ conversion are shared with it.
//
// One CTA owns a tile of 128 keys of one kv head and walks the query heads of the GQA group and the
// 128-row query tiles that can see those keys.  Per query tile, five GEMMs, all M = 128:
//   S^T  = K . Q^T      (SS, N = 128 queries, K = 64)      -> TMEM [  0,128)
//   dP^T = V . dO^T     (SS)                                -> TMEM [128,256)
//   8 compute warps (thread = key row, two warps per 32 rows splitting the query columns) turn these into
//   P^T = 2^(scale*log2e*S^T - L) and dS^T = P^T o (dP^T - delta), written back as 16-bit A operands over
//   the columns they came from, and dS also to shared memory as a [query][key] tile
//   dV  += P^T . dO     (A from TMEM, B = dO as an MN-major operand, N = 64)   -> TMEM [256,320)
//   dK  += dS^T . Q     (A from TMEM, B = Q MN-major)                          -> TMEM [320,384)
//   dQ   = dS . K       (SS: A = dS tile, B = K MN-major)                      -> TMEM [384,448)
// dQ is read out of TMEM by the compute warps while the next tile's S^T / dP^T are being computed and
// added to the fp32 accumulator with vector red.global.add; dK / dV leave TMEM once, at the end.
// Warp 8 is the TMA producer (K, V once; Q, dO double-buffered; L and delta staged with them), warp 9
// issues the MMAs.  No load uses cluster multicast; every mbarrier wait is bounded.
#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace b200fa {

namespace {

constexpr int BK = 128;      // keys per CTA (TMEM lanes)
constexpr int BQ = 128;      // queries per step
constexpr int HD = 64;
constexpr int kThreads = 320;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t cST = 0, cDPT = 128, cDV = 256, cDK = 320, cDQ = 384;

constexpr int kTileBytes = 128 * HD * 2;                 // 16384: one [128 rows][64] tile
constexpr int kDSBytes = BQ * BK * 2;                    // 32768: dS as two 64-key halves [half][query][128 B]
constexpr int kStatBytes = 2 * 2 * BQ * 4;               // L and delta, two stages
constexpr int kSmemTiles = 2 * kTileBytes + 4 * kTileBytes + kDSBytes;   // K, V, Q x2, dO x2, dS = 131072
constexpr int kSmemBytes = kSmemTiles + kStatBytes + 256 + 1024;

enum Bar { BAR_KV = 0, BAR_Q_FULL = 1, BAR_Q_EMPTY = 3, BAR_ST_DONE = 5, BAR_PD_READY = 6, BAR_DQ_DONE = 7, BAR_COUNT = 8 };

struct BwdArgs {
  BwdParams p;
  int dtype;
};

__device__ __forceinline__ uint32_t pack16b(int dtype, float a, float b) {
  return dtype == 0 ? Elem<__half>::pack(a, b) : Elem<__nv_bfloat16>::pack(a, b);
}

__global__ void __launch_bounds__(kThreads, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;
  unsigned char* sV = sK + kTileBytes;
  unsigned char* sQ = sV + kTileBytes;                 // [2][128][128 B]
  unsigned char* sDO = sQ + 2 * kTileBytes;            // [2][128][128 B]
  unsigned char* sDS = sDO + 2 * kTileBytes;           // [2 halves][128 queries][128 B]
  float* sL = reinterpret_cast<float*>(smem + kSmemTiles);      // [2][BQ]
  float* sDel = sL + 2 * BQ;                                    // [2][BQ]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles + kStatBytes);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

  const BwdParams& p = a.p;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  int bb = blockIdx.z;
  int q_begin = 0, k_begin = 0, N = p.N, S = p.S;
  if (p.cu_q != nullptr) {
    q_begin = p.cu_q[bb];
    N = p.cu_q[bb + 1] - q_begin;
    k_begin = p.cu_k[bb];
    S = p.cu_k[bb + 1] - k_begin;
    bb = 0;
  }
  const int n0 = blockIdx.x * BK;
  if (n0 >= S) return;
  const int off = S - N;
  int m_begin = 0;
  if (p.causal) m_begin = max(0, n0 - off) / BQ;
  const int m_end = (N + BQ - 1) / BQ;
  const int nm = max(0, m_end - m_begin);
  const int n_iter = nm * p.gqa;

  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };

  if (n_iter == 0) {
    // no query sees these keys: dK = dV = 0
    if (warp < 8) {
      const int key = n0 + (warp & 3) * 32 + lane, hf = warp >> 2;
      if (key < S) {
        const int64_t o = bb * p.dk_bs + kvh * p.dk_hs + static_cast<int64_t>(k_begin + key) * p.dk_rs + hf * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dk) + o)[i] = make_uint4(0u, 0u, 0u, 0u);
          reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dv) + o)[i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    return;
  }

  if (tid == 0) {
    mbar_init(bar(BAR_KV), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BAR_Q_FULL + s), 1);
      mbar_init(bar(BAR_Q_EMPTY + s), 1);
    }
    mbar_init(bar(BAR_ST_DONE), 1);
    mbar_init(bar(BAR_PD_READY), 8);      // one arrive per compute warp
    mbar_init(bar(BAR_DQ_DONE), 1);
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp == 8) {
    // ============================ producer ============================
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(BAR_KV), 2 * kTileBytes);
      tma_load_4d(smem_u32(sK), &tmK, bar(BAR_KV), 0, k_begin + n0, kvh, bb);
      tma_load_4d(smem_u32(sV), &tmV, bar(BAR_KV), 0, k_begin + n0, kvh, bb);
    }
    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1;
      const int hq = kvh * p.gqa + it / nm, m = m_begin + it % nm;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q_EMPTY + st), ((it >> 1) & 1) ^ 1, s_abort))) break;
      // -L and -delta of the 128 query rows ride with the Q tile; rows beyond N (or without any visible key)
      // get L = +inf so that their P is exactly zero
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ql = lane * 4 + i;
        const int row = m * BQ + ql;
        float L = INFINITY, dl = 0.f;
        if (row < N) {
          const int64_t idx = bb * p.lse_bs + hq * p.lse_hs + q_begin + row;
          L = p.lse[idx];
          dl = p.delta[idx];
          if (L == -INFINITY) L = INFINITY;
        }
        sL[st * BQ + ql] = -L;            // stored negated: the compute loop adds them
        sDel[st * BQ + ql] = -dl;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(bar(BAR_Q_FULL + st), 2 * kTileBytes);
        tma_load_4d(smem_u32(sQ + st * kTileBytes), &tmQ, bar(BAR_Q_FULL + st), 0, q_begin + m * BQ, hq, bb);
        tma_load_4d(smem_u32(sDO + st * kTileBytes), &tmDO, bar(BAR_Q_FULL + st), 0, q_begin + m * BQ, hq, bb);
      }
      __syncwarp();
    }
  } else if (warp == 9) {
    // ============================ MMA issue ============================
    const bool leader = lane == 0;
    const uint32_t id_st = instr_desc(a.dtype, 0, 128, BQ);     // S^T, dP^T: B K-major, N = 128
    const uint32_t id_mn = instr_desc(a.dtype, 1, 128, HD);     // dV, dK, dQ: B MN-major, N = 64
    const uint64_t kd = smem_desc(smem_u32(sK), 16, 1024), vd = smem_desc(smem_u32(sV), 16, 1024);
    const uint64_t kmn = smem_desc(smem_u32(sK), kTileBytes, 1024);
    const uint64_t dsd = smem_desc(smem_u32(sDS), 16, 1024);
    constexpr uint64_t kTileU = kTileBytes >> 4;
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_KV), 0, s_abort));
    auto issue_stdp = [&](int it) -> bool {
      const int st = it & 1;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q_FULL + st), (it >> 1) & 1, s_abort))) return false;
      tc_fence_after();
      const uint64_t qd = smem_desc(smem_u32(sQ), 16, 1024) + st * kTileU;
      const uint64_t dod = smem_desc(smem_u32(sDO), 16, 1024) + st * kTileU;
#pragma unroll
      for (int k = 0; k < HD / 16; ++k)
        if (leader) mma_ss(tmem + cST, kd + k * 2, qd + k * 2, id_st, k > 0 ? 1u : 0u);
#pragma unroll
      for (int k = 0; k < HD / 16; ++k)
        if (leader) mma_ss(tmem + cDPT, vd + k * 2, dod + k * 2, id_st, k > 0 ? 1u : 0u);
      if (leader) tc_commit(bar(BAR_ST_DONE));
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_stdp(0);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it & 1;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_PD_READY), it & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      const uint64_t qmn = smem_desc(smem_u32(sQ), kTileBytes, 1024) + st * kTileU;
      const uint64_t domn = smem_desc(smem_u32(sDO), kTileBytes, 1024) + st * kTileU;
      // dV += P^T.dO and dK += dS^T.Q: A in TMEM (8 columns per 16 queries; queries 0-63 at +0, 64-127 at +64,
      // where the two column halves were written), B rows = queries, 16 rows = 128 units
#pragma unroll
      for (int k = 0; k < BQ / 16; ++k)
        if (leader) mma_ts(tmem + cDV, tmem + cST + (k >> 2) * 64 + (k & 3) * 8, domn + k * 128, id_mn, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
      for (int k = 0; k < BQ / 16; ++k)
        if (leader) mma_ts(tmem + cDK, tmem + cDPT + (k >> 2) * 64 + (k & 3) * 8, qmn + k * 128, id_mn, (it > 0 || k > 0) ? 1u : 0u);
      if (leader) tc_commit(bar(BAR_Q_EMPTY + st));
      // dQ = dS.K: A = dS [query][key] in two 64-key halves, B = K rows = keys
#pragma unroll
      for (int k = 0; k < BK / 16; ++k)
        if (leader) mma_ss(tmem + cDQ, dsd + (k >> 2) * (static_cast<uint64_t>(kDSBytes / 2) >> 4) + (k & 3) * 2, kmn + k * 128,
                           id_mn, k > 0 ? 1u : 0u);
      if (leader) tc_commit(bar(BAR_DQ_DONE));
      __syncwarp();
      if (it + 1 < n_iter) ok = issue_stdp(it + 1);
    }
  } else {
    // ============================ compute warps 0-7 ============================
    const int wq = warp & 3, hf = warp >> 2;                 // TMEM lane quarter, column half
    const int rloc = wq * 32 + lane;                         // key row (S^T, dK, dV) or query row (dQ) inside the tile
    const int key = n0 + rloc;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    bool ok = true;

    auto flush_dq = [&](int it_done) {
      // dQ tile of iteration it_done: rows = queries, this warp's 32 of the 64 columns -> fp32 accumulator
      const int hq = kvh * p.gqa + it_done / nm, m = m_begin + it_done % nm;
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + cDQ + hf * 32, r);
      tc_wait_ld();
      const int row = m * BQ + rloc;
      if (row < N) {
        float* acc = p.dq_acc + ((static_cast<int64_t>(bb) * p.Hq + hq) * p.N + q_begin + row) * HD + hf * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          atomicAdd(reinterpret_cast<float4*>(acc + i), make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                    __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])));
      }
    };

    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1;
      const int m = m_begin + it % nm;
      if (it > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DQ_DONE), (it - 1) & 1, s_abort))) { ok = false; break; }
        tc_fence_after();
        flush_dq(it - 1);
      }
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_Q_FULL + st), (it >> 1) & 1, s_abort))) { ok = false; break; }
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_ST_DONE), it & 1, s_abort))) { ok = false; break; }
      tc_fence_after();
      const float* Ls = sL + st * BQ;
      const float* Ds = sDel + st * BQ;
      const bool need_mask = (n0 + BK > S) || (p.causal && (n0 + BK - 1 > m * BQ + off));
      // dS[query][this key] lives at ds_col + query * 128 + ((key chunk ^ (query & 7)) << 4); the eight swizzled
      // chunk offsets are fixed per thread, and the query offsets are compile-time constants of the unrolled loop
      unsigned char* ds_col = sDS + (rloc >> 6) * (kDSBytes / 2) + (rloc & 7) * 2;
      const int kchunk = (rloc & 63) >> 3;
      unsigned char* ds_sw[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) ds_sw[r] = ds_col + ((kchunk ^ r) << 4);
      const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
      auto run_tile = [&](auto masked) {
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        const int col0 = hf * 64 + c * 32;                 // first query column of this chunk
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem + lane_base + cST + col0, rs);
        tmem_ld32(tmem + lane_base + cDPT + col0, rd);
        tc_wait_ld();
        uint32_t pp[16], pd[16];
        const int rowoff = col0 * 128;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 nL = *reinterpret_cast<const float4*>(Ls + col0 + i);      // -L of four queries
          const float4 nD = *reinterpret_cast<const float4*>(Ds + col0 + i);      // -delta
#pragma unroll
          for (int e = 0; e < 4; e += 2) {
            const float2 sv = make_float2(__uint_as_float(rs[i + e]), __uint_as_float(rs[i + e + 1]));
            const float2 dv = make_float2(__uint_as_float(rd[i + e]), __uint_as_float(rd[i + e + 1]));
            const float2 nl = e == 0 ? make_float2(nL.x, nL.y) : make_float2(nL.z, nL.w);
            const float2 nd = e == 0 ? make_float2(nD.x, nD.y) : make_float2(nD.z, nD.w);
            const float2 t = __ffma2_rn(sv, c2, nl);
            float2 pe = make_float2(fast_exp2(t.x), fast_exp2(t.y));
            if constexpr (decltype(masked)::value) {
              const int qrow = m * BQ + col0 + i + e;
              const bool kin = key < S;
              if (!(kin && (!p.causal || key <= qrow + off))) pe.x = 0.f;
              if (!(kin && (!p.causal || key <= qrow + 1 + off))) pe.y = 0.f;
            }
            const float2 dsv = __fmul2_rn(pe, __fadd2_rn(dv, nd));
            pp[(i + e) >> 1] = pack16b(a.dtype, pe.x, pe.y);
            const uint32_t dpk = pack16b(a.dtype, dsv.x, dsv.y);
            pd[(i + e) >> 1] = dpk;
            const int ql = i + e;                          // query inside the chunk; (col0 + ql) & 7 == ql & 7
            *reinterpret_cast<uint16_t*>(ds_sw[ql & 7] + rowoff + ql * 128) = static_cast<uint16_t>(dpk & 0xffffu);
            *reinterpret_cast<uint16_t*>(ds_sw[(ql + 1) & 7] + rowoff + (ql + 1) * 128) = static_cast<uint16_t>(dpk >> 16);
          }
        }
        // P^T and dS^T overwrite the columns they came from: 16-bit pairs along the query index
        // (inside this warp's own 64 columns, whose contents it has already loaded: the other warp of these
        // rows may still be reading its half)
        tmem_st16(tmem + lane_base + cST + hf * 64 + c * 16, pp);
        tmem_st16(tmem + lane_base + cDPT + hf * 64 + c * 16, pd);
      }
      };
      if (need_mask) run_tile(std::true_type{}); else run_tile(std::false_type{});
      tc_wait_st();
      fence_proxy_async();          // the dS tile was written with ordinary stores and is read by the MMA
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_PD_READY));
    }

    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar(BAR_DQ_DONE), (n_iter - 1) & 1, s_abort));
    if (ok) {
      tc_fence_after();
      flush_dq(n_iter - 1);
      // dK, dV: rows = keys, this warp's 32 of the 64 columns
      if (true) {
        uint32_t rk[32], rv[32];
        tmem_ld32(tmem + lane_base + cDK + hf * 32, rk);
        tmem_ld32(tmem + lane_base + cDV + hf * 32, rv);
        tc_wait_ld();
        if (key < S) {
          const int64_t o = bb * p.dk_bs + kvh * p.dk_hs + static_cast<int64_t>(k_begin + key) * p.dk_rs + hf * 32;
          uint16_t* dkp = reinterpret_cast<uint16_t*>(p.dk) + o;
          uint16_t* dvp = reinterpret_cast<uint16_t*>(p.dv) + o;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 vk, vv;
            vk.x = pack16b(a.dtype, __uint_as_float(rk[i]) * p.scale, __uint_as_float(rk[i + 1]) * p.scale);
            vk.y = pack16b(a.dtype, __uint_as_float(rk[i + 2]) * p.scale, __uint_as_float(rk[i + 3]) * p.scale);
            vk.z = pack16b(a.dtype, __uint_as_float(rk[i + 4]) * p.scale, __uint_as_float(rk[i + 5]) * p.scale);
            vk.w = pack16b(a.dtype, __uint_as_float(rk[i + 6]) * p.scale, __uint_as_float(rk[i + 7]) * p.scale);
            vv.x = pack16b(a.dtype, __uint_as_float(rv[i]), __uint_as_float(rv[i + 1]));
            vv.y = pack16b(a.dtype, __uint_as_float(rv[i + 2]), __uint_as_float(rv[i + 3]));
            vv.z = pack16b(a.dtype, __uint_as_float(rv[i + 4]), __uint_as_float(rv[i + 5]));
            vv.w = pack16b(a.dtype, __uint_as_float(rv[i + 6]), __uint_as_float(rv[i + 7]));
            *reinterpret_cast<uint4*>(dkp + i) = vk;
            *reinterpret_cast<uint4*>(dvp + i) = vv;
          }
        }
      }
    }
  }

  // ---- teardown ----
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

bool make_map64(CUtensorMap* m, int dtype, const void* base, int rows, int H, int B, int64_t rs, int64_t hs, int64_t bs) {
  const uint64_t dims[4] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(rows), static_cast<uint64_t>(H),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(rs) * 2, static_cast<uint64_t>(hs) * 2, static_cast<uint64_t>(bs) * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tmap(m, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims,
                     strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

bool bwd_sm100_supported(int dtype, int D) { return (dtype == 0 || dtype == 1) && D == HD && get_encode_tiled() != nullptr; }

// Main backward step only: p.delta and p.dq_acc must already hold delta and zeros.
cudaError_t launch_bwd_sm100_main(const BwdParams& p, int dtype, int nbatch, int max_k, cudaStream_t stream) {
  if (nbatch <= 0 || max_k <= 0) return cudaSuccess;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  auto fix = [](int64_t s, int64_t fallback) { return s > 0 ? s : fallback; };
  const int64_t q_hs = fix(p.q_hs, static_cast<int64_t>(p.N) * p.q_rs), q_bs = fix(p.q_bs, q_hs * p.Hq);
  const int64_t k_hs = fix(p.k_hs, static_cast<int64_t>(p.S) * p.k_rs), k_bs = fix(p.k_bs, k_hs * p.Hkv);
  const int64_t v_hs = fix(p.v_hs, static_cast<int64_t>(p.S) * p.v_rs), v_bs = fix(p.v_bs, v_hs * p.Hkv);
  const int64_t do_hs = static_cast<int64_t>(p.N) * HD, do_bs = do_hs * p.Hq;
  if (!make_map64(&tmQ, dtype, p.q, p.N, p.Hq, p.B, p.q_rs, q_hs, q_bs) ||
      !make_map64(&tmK, dtype, p.k, p.S, p.Hkv, p.B, p.k_rs, k_hs, k_bs) ||
      !make_map64(&tmV, dtype, p.v, p.S, p.Hkv, p.B, p.v_rs, v_hs, v_bs) ||
      !make_map64(&tmDO, dtype, p.dout, p.N, p.Hq, p.B, HD, do_hs, do_bs))
    return cudaErrorInvalidValue;
  BwdArgs a;
  a.p = p;
  a.dtype = dtype;
  cudaError_t e = cudaFuncSetAttribute(bwd_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((max_k + BK - 1) / BK, p.Hkv, nbatch);
  bwd_sm100_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmQ, tmK, tmV, tmDO, a);
  return cudaGetLastError();
}

}  // namespace b200fa
