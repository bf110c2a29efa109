// Portable 16-bit forward kernel: ldmatrix + mma.sync m16n8k16, cp.async double
// buffering, online softmax in registers.  Handles every shape the C-ABI admits
// (any N, S; D = 64 or 128; GQA; causal lower-right; left window; softcap;
// packed varlen) and is the fallback for shapes the tcgen05 kernel does not take.
//
// What it computes follows the reference forward (csrc/mfa_steel_fwd.cpp:801-1221):
// S = scale*Q.K^T -> softcap -> masks -> online softmax (base 2) -> O += P.V,
// O /= sum, L = max + log2(sum).
#include "common.cuh"
#include "launch.h"

namespace b200fa {

namespace {

constexpr int kBQ = 128;
constexpr int kBK = 64;
constexpr int kThreads = 256;

template <int ROWS, int D, typename T>
__device__ __forceinline__ void load_tile_async(T* s, const T* g, int64_t rs, int row0, int limit,
                                                int tid) {
  constexpr int CH = D / 8;
  const uint32_t sbase = smem_u32(s);
#pragma unroll
  for (int i = tid; i < ROWS * CH; i += kThreads) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    bool pred = gr < limit;
    const T* src = g + static_cast<int64_t>(pred ? gr : 0) * rs + c * 8;
    cp_async16(sbase + swz_off<D>(r, c * 8), src, pred);
  }
}

template <typename T, int D, bool VARLEN>
__global__ void __launch_bounds__(kThreads) fa_fwd_mma_kernel(const FwdParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + kBQ * D;
  T* sV = sK + 2 * kBK * D;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int head = blockIdx.y;
  const int kvh = head / p.gqa;
  int bb = blockIdx.z;
  int q_begin = 0, k_begin = 0, N = p.N, S = p.S;
  if (VARLEN) {
    q_begin = p.cu_q[bb];
    N = p.cu_q[bb + 1] - q_begin;
    k_begin = p.cu_k[bb];
    S = p.cu_k[bb + 1] - k_begin;
    bb = 0;
  }
  // heaviest (last) causal tiles are scheduled first
  const int q0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * kBQ;
  if (q0 >= N) return;
  const int off = S - N;

  int k_hi = S;
  if (p.causal) k_hi = min(S, q0 + kBQ + off);
  int k_lo = 0;
  if (p.window_left >= 0) k_lo = max(0, q0 + off - p.window_left);
  const int kt_begin = k_lo / kBK;
  const int kt_end = k_hi > 0 ? (k_hi + kBK - 1) / kBK : 0;

  const T* qg = reinterpret_cast<const T*>(p.q) + bb * p.q_bs + head * p.q_hs + q_begin * p.q_rs;
  const T* kg = reinterpret_cast<const T*>(p.k) + bb * p.k_bs + kvh * p.k_hs + k_begin * p.k_rs;
  const T* vg = reinterpret_cast<const T*>(p.v) + bb * p.v_bs + kvh * p.v_hs + k_begin * p.v_rs;
  T* og = reinterpret_cast<T*>(p.o) + bb * p.o_bs + head * p.o_hs + q_begin * p.o_rs;

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.f, 0.f};

  // Block-sparse mask: a key tile is visited only if one of its (query block, key block) cells is active; every
  // thread scans the same few bytes, so the decision is uniform across the CTA.  Bit 0 of the result: some cell
  // active; bit 1: all cells active (no per-element masking needed for this tile).
  auto tile_cells = [&](int kt) -> int {
    if (p.bmask == nullptr) return 3;
    const int rb0 = q0 / p.bm_bq, rb1 = (min(q0 + kBQ, N) - 1) / p.bm_bq;
    const int cb0 = (kt * kBK) / p.bm_bk, cb1 = (min((kt + 1) * kBK, S) - 1) / p.bm_bk;
    bool any = false, all = true;
    for (int rb = rb0; rb <= rb1; ++rb)
      for (int cb = cb0; cb <= cb1; ++cb) {
        const bool on = p.bmask[rb * p.bm_nk + cb] != 0;
        any = any || on;
        all = all && on;
      }
    return (any ? 1 : 0) | (all ? 2 : 0);
  };
  auto next_active = [&](int kt) -> int {
    while (kt < kt_end && !(tile_cells(kt) & 1)) ++kt;
    return kt;
  };

  load_tile_async<kBQ, D>(sQ, qg, p.q_rs, q0, N, tid);
  const int kt_first = next_active(kt_begin);
  if (kt_first < kt_end) {
    load_tile_async<kBK, D>(sK, kg, p.k_rs, kt_first * kBK, S, tid);
    load_tile_async<kBK, D>(sV, vg, p.v_rs, kt_first * kBK, S, tid);
  }
  cp_async_commit();

  const uint32_t sQ_u = smem_u32(sQ);
  const int row_a = warp * 16 + (lane & 15);       // ldmatrix row for A fragments
  const int col_a = (lane >> 4) * 8;
  const int r0 = q0 + warp * 16 + g;               // global query rows of this thread
  const int r1 = r0 + 8;
  const bool use_cap = p.softcap > 0.f;
  const float cap_in = use_cap ? p.scale / p.softcap : 0.f;
  const float cap_out = p.softcap * kLog2e;
  const bool precise_tanh = p.softcap >= kPreciseTanhMinCap;
  const float alibi_l2 = p.alibi != nullptr ? p.alibi[head] * kLog2e : 0.f;

  int stage = 0;
  for (int kt = kt_first; kt < kt_end; stage ^= 1) {
    const int kt_next = next_active(kt + 1);
    cp_async_wait<0>();
    __syncthreads();
    if (kt_next < kt_end) {
      load_tile_async<kBK, D>(sK + (stage ^ 1) * kBK * D, kg, p.k_rs, kt_next * kBK, S, tid);
      load_tile_async<kBK, D>(sV + (stage ^ 1) * kBK * D, vg, p.v_rs, kt_next * kBK, S, tid);
      cp_async_commit();
    }
    const uint32_t sK_u = smem_u32(sK + stage * kBK * D);
    const uint32_t sV_u = smem_u32(sV + stage * kBK * D);

    // ---- S = Q K^T ----
    float s[kBK / 8][4];
#pragma unroll
    for (int i = 0; i < kBK / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, sQ_u + swz_off<D>(row_a, kk * 16 + col_a));
#pragma unroll
      for (int nj = 0; nj < kBK / 16; ++nj) {
        uint32_t bfr[4];
        const int krow = nj * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int kcol = kk * 16 + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(bfr, sK_u + swz_off<D>(krow, kcol));
        mma16816<T>(s[2 * nj], a, bfr[0], bfr[1]);
        mma16816<T>(s[2 * nj + 1], a, bfr[2], bfr[3]);
      }
    }

    // ---- scale, softcap (before masks), masks ----
    const int k0 = kt * kBK;
    if (use_cap) {
#pragma unroll
      for (int i = 0; i < kBK / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] = cap_out * cap_tanh(s[i][e] * cap_in, precise_tanh);
    } else {
#pragma unroll
      for (int i = 0; i < kBK / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] *= p.scale_log2;
    }
    if (p.alibi != nullptr) {
      // ALiBi: slope * (key - query position), in the base-2 domain, after scale / softcap and before the masks
#pragma unroll
      for (int i = 0; i < kBK / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = k0 + i * 8 + 2 * t + (e & 1);
          const int row = (e < 2) ? r0 : r1;
          s[i][e] = fmaf(alibi_l2, static_cast<float>(col - (row + off)), s[i][e]);
        }
      }
    }
    const bool cells_partial = !(tile_cells(kt) & 2);
    const bool need_mask = (k0 + kBK > S) || (p.causal && (k0 + kBK - 1 > q0 + off)) ||
                           (p.window_left >= 0 && (k0 < q0 + kBQ - 1 + off - p.window_left)) || cells_partial;
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < kBK / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = k0 + i * 8 + 2 * t + (e & 1);
          const int row = (e < 2) ? r0 : r1;
          bool vis = col < S;
          if (p.causal) vis = vis && (col <= row + off);
          if (p.window_left >= 0) vis = vis && (col >= row + off - p.window_left);
          if (cells_partial && vis) vis = p.bmask[(min(row, N - 1) / p.bm_bq) * p.bm_nk + col / p.bm_bk] != 0;
          if (!vis) s[i][e] = -INFINITY;
        }
      }
    }

    // ---- online softmax ----
    float mx[2] = {row_max[0], row_max[1]};
#pragma unroll
    for (int i = 0; i < kBK / 8; ++i) {
      mx[0] = fmaxf(mx[0], fmaxf(s[i][0], s[i][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[i][2], s[i][3]));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float corr[2], msub[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      msub[h] = (mx[h] == -INFINITY) ? 0.f : mx[h];
      corr[h] = fast_exp2(row_max[h] - msub[h]);  // row_max = -inf -> 0
      row_max[h] = mx[h];
      row_sum[h] *= corr[h];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
#pragma unroll
    for (int i = 0; i < kBK / 8; ++i) {
      s[i][0] = fast_exp2(s[i][0] - msub[0]);
      s[i][1] = fast_exp2(s[i][1] - msub[0]);
      s[i][2] = fast_exp2(s[i][2] - msub[1]);
      s[i][3] = fast_exp2(s[i][3] - msub[1]);
      row_sum[0] += s[i][0] + s[i][1];
      row_sum[1] += s[i][2] + s[i][3];
    }

    // ---- O += P V ----
#pragma unroll
    for (int kb = 0; kb < kBK / 16; ++kb) {
      uint32_t a[4];
      a[0] = Elem<T>::pack(s[2 * kb][0], s[2 * kb][1]);
      a[1] = Elem<T>::pack(s[2 * kb][2], s[2 * kb][3]);
      a[2] = Elem<T>::pack(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      a[3] = Elem<T>::pack(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
      for (int dj = 0; dj < D / 16; ++dj) {
        uint32_t bfr[4];
        const int vrow = kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int vcol = dj * 16 + ((lane >> 4) << 3);
        ldmatrix_x4_trans(bfr, sV_u + swz_off<D>(vrow, vcol));
        mma16816<T>(o[2 * dj], a, bfr[0], bfr[1]);
        mma16816<T>(o[2 * dj + 1], a, bfr[2], bfr[3]);
      }
    }
    kt = kt_next;
  }
  cp_async_wait<0>();
  // A tile without any key tile never reached the loop's barrier: the Q rows this warp is about to reuse for its
  // output were requested by threads of every warp, and their copies must have landed first (CTA-uniform branch)
  if (kt_first >= kt_end) __syncthreads();

  // ---- epilogue ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
  }
  const float inv0 = row_sum[0] > 0.f ? 1.f / row_sum[0] : 0.f;
  const float inv1 = row_sum[1] > 0.f ? 1.f / row_sum[1] : 0.f;

  // Each warp stages its own 16 rows in the Q tile it alone reads.
  __syncwarp();
  {
    unsigned char* sO = reinterpret_cast<unsigned char*>(sQ);
    const int lr0 = warp * 16 + g, lr1 = lr0 + 8;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + 2 * t;
      uint32_t v0 = Elem<T>::pack(o[i][0] * inv0, o[i][1] * inv0);
      uint32_t v1 = Elem<T>::pack(o[i][2] * inv1, o[i][3] * inv1);
      *reinterpret_cast<uint32_t*>(sO + swz_off<D>(lr0, i * 8) + (col & 7) * 2) = v0;
      *reinterpret_cast<uint32_t*>(sO + swz_off<D>(lr1, i * 8) + (col & 7) * 2) = v1;
    }
    __syncwarp();
    constexpr int CH = D / 8;
#pragma unroll
    for (int i = lane; i < 16 * CH; i += 32) {
      const int r = i / CH, c = i % CH;
      const int lr = warp * 16 + r;
      const int gr = q0 + lr;
      if (gr < N) {
        uint4 val = *reinterpret_cast<const uint4*>(sO + swz_off<D>(lr, c * 8));
        *reinterpret_cast<uint4*>(og + static_cast<int64_t>(gr) * p.o_rs + c * 8) = val;
      }
    }
  }
  if (p.lse != nullptr && t == 0) {
    float* lg = p.lse + bb * p.lse_bs + head * p.lse_hs + q_begin;
    if (r0 < N) lg[r0] = row_sum[0] > 0.f ? row_max[0] + log2f(row_sum[0]) : -INFINITY;
    if (r1 < N) lg[r1] = row_sum[1] > 0.f ? row_max[1] + log2f(row_sum[1]) : -INFINITY;
  }
}

template <typename T, int D, bool VARLEN>
cudaError_t launch_one(const FwdParams& p, int nbatch, int max_q, cudaStream_t stream) {
  constexpr size_t smem = static_cast<size_t>(kBQ + 4 * kBK) * D * sizeof(T);
  auto kern = fa_fwd_mma_kernel<T, D, VARLEN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  dim3 grid((max_q + kBQ - 1) / kBQ, p.Hq, nbatch);
  kern<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_mma(const FwdParams& p, int dtype, int D, bool varlen, int nbatch, int max_q,
                           cudaStream_t stream) {
  if (max_q <= 0 || nbatch <= 0) return cudaSuccess;
#define B200FA_CASE(T_, D_)                                                   \
  return varlen ? launch_one<T_, D_, true>(p, nbatch, max_q, stream)          \
                : launch_one<T_, D_, false>(p, nbatch, max_q, stream)
  if (dtype == 0 && D == 64) { B200FA_CASE(__half, 64); }
  if (dtype == 0 && D == 128) { B200FA_CASE(__half, 128); }
  if (dtype == 1 && D == 64) { B200FA_CASE(__nv_bfloat16, 64); }
  if (dtype == 1 && D == 128) { B200FA_CASE(__nv_bfloat16, 128); }
  if (dtype == 0 && D == 256) { B200FA_CASE(__half, 256); }
  if (dtype == 1 && D == 256) { B200FA_CASE(__nv_bfloat16, 256); }
#undef B200FA_CASE
  return cudaErrorInvalidValue;
}

}  // namespace b200fa
