// Backward dQ / dK / dV, 16-bit, D = 64 or 128, dense and packed-varlen layouts.
//
// What it computes is the reference's STEEL backward (csrc/mfa_steel_bwd.cpp:284-745 dQ,
// 765-1293 dK/dV; host side csrc/bindings.cpp:120-163):
//   P = 2^(scale*log2e*S - L),  dP = dO.V^T,  dS = P o (dP - delta),  delta = sum_d dO o O
//   dV = P^T.dO,  dK = scale * dS^T.Q,  dQ = scale * dS.K
// With a soft cap the forward's score is cap*tanh(scale*S/cap): P uses the capped score and dS gains the factor
// 1 - tanh^2 (the reference differentiates its SDPA fallback for softcap and windows, mlx_mfa/attention.py:1976-1992,
// 2020-2027; here both run in the kernels).  A left window masks keys j < i + (S - N) - window_left.
// with P and dS rounded to the input dtype before their MMAs, as the reference does
// (csrc/mfa_steel_bwd.cpp:1100-1101, 1200-1201).
//
// Shape of the work: three launches.
//   1. bwd_preprocess: delta[b,h,i] and zero of the fp32 dQ accumulator.
//   2. bwd_main: one CTA per (key tile of 64, kv head, batch | sequence).  K and V tiles stay in shared
//      memory; the CTA walks the query heads of the GQA group and the query tiles that can see its keys
//      (causal tiles below the diagonal are skipped), keeps dK / dV in registers, and adds its dQ
//      contribution into the fp32 accumulator with vector red.global.add.  S^T = K.Q^T is computed
//      transposed so that P^T and dS^T leave the MMA already in A-operand layout for dV and dK; dS^T goes
//      through shared memory once for the dQ product.  ldmatrix + mma.sync m16n8k16, cp.async double buffer.
//   3. bwd_convert: dQ accumulator * scale -> dtype.
// Causal masks are lower-right aligned (key j visible to row i iff j <= i + S - N), per sequence.
#include "common.cuh"
#include "launch.h"

namespace b200fa {

namespace {

constexpr int kBM = 64;   // queries per step
constexpr int kBN = 64;   // keys per CTA
constexpr int kThreads = 256;

__host__ __device__ inline size_t bwd_align(size_t x) { return (x + 255) / 256 * 256; }

// ---------------------------------------------------------------------------
// 1. delta and dQ-accumulator reset.  One warp per (b, h, row).
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const BwdParams p, int total_rows) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (blockIdx.x == 0 && threadIdx.x == 0 && p.work_counter != nullptr) *p.work_counter = 0;
  if (warp >= total_rows) return;
  // warp index = (b*Hq + h)*N + i
  const int i = warp % p.N;
  const int h = (warp / p.N) % p.Hq;
  const int b = warp / (p.N * p.Hq);
  const T* o = reinterpret_cast<const T*>(p.o) + b * p.o_bs + h * p.o_hs + static_cast<int64_t>(i) * p.o_rs;
  const T* dout = reinterpret_cast<const T*>(p.dout) + (static_cast<int64_t>(b) * p.Hq + h) * p.N * D + static_cast<int64_t>(i) * D;
  float acc = 0.f;
  constexpr int PER = D / 32;     // 2 or 4 elements per lane
#pragma unroll
  for (int e = 0; e < PER; e += 2) {
    const uint32_t ow = *reinterpret_cast<const uint32_t*>(o + lane * PER + e);
    const uint32_t dw = *reinterpret_cast<const uint32_t*>(dout + lane * PER + e);
    const float2 of = Elem<T>::unpack(ow), df = Elem<T>::unpack(dw);
    acc = fmaf(of.x, df.x, acc);
    acc = fmaf(of.y, df.y, acc);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) p.delta[warp] = acc;
  if (p.dq_acc != nullptr) {          // the split head_dim-128 path has no accumulator
    float* dq = p.dq_acc + static_cast<int64_t>(warp) * D;
#pragma unroll
    for (int e = 0; e < PER; ++e) dq[lane + 32 * e] = 0.f;
  }
}

// The same with 16-byte accesses: D / 8 lanes per row, each with 8 elements of O and dO and 8 accumulator words to
// clear (one warp per row left every lane with 4 bytes per load and ran at 2.8 TB/s).  Needs 16-byte aligned rows.
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_preprocess_vec_kernel(const BwdParams p) {
  constexpr int LPR = D / 8;                                   // lanes per row: 8 or 16
  // grid = (rows of one head in blocks of 256 / LPR, Hq, B): no division by run-time values per thread
  const int h = blockIdx.y;
  const long long b = blockIdx.z;
  const unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t == 0 && h == 0 && b == 0 && p.work_counter != nullptr) *p.work_counter = 0;
  const int i = static_cast<int>(t / LPR);
  const int c = static_cast<int>(t % LPR);
  const bool live = i < p.N;                                   // whole rows share a warp: the shuffles below stay legal
  const long long row = (b * p.Hq + h) * p.N + i;
  float acc = 0.f;
  if (live) {
    const T* o = reinterpret_cast<const T*>(p.o) + b * p.o_bs + h * p.o_hs + static_cast<int64_t>(i) * p.o_rs + c * 8;
    const T* dout = reinterpret_cast<const T*>(p.dout) + row * D + c * 8;
    const uint4 ow = *reinterpret_cast<const uint4*>(o), dw = *reinterpret_cast<const uint4*>(dout);
    const uint32_t ou[4] = {ow.x, ow.y, ow.z, ow.w}, du[4] = {dw.x, dw.y, dw.z, dw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 of = Elem<T>::unpack(ou[e]), df = Elem<T>::unpack(du[e]);
      acc = fmaf(of.x, df.x, acc);
      acc = fmaf(of.y, df.y, acc);
    }
    if (p.dq_acc != nullptr) {        // the split head_dim-128 path has no accumulator
      float4* dq = reinterpret_cast<float4*>(p.dq_acc + row * D + c * 8);
      dq[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      dq[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int sft = LPR / 2; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
  if (live && c == 0) p.delta[row] = acc;
}

// ---------------------------------------------------------------------------
// 3. dQ accumulator -> dtype
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) bwd_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, float scale,
                                                          long long n_pairs) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_pairs; i += stride) {
    const float2 v = reinterpret_cast<const float2*>(acc)[i];
    reinterpret_cast<uint32_t*>(dq)[i] = Elem<T>::pack(v.x * scale, v.y * scale);
  }
}

// ---------------------------------------------------------------------------
// 2. main kernel
// ---------------------------------------------------------------------------
template <int ROWS, int D, typename T>
__device__ __forceinline__ void load_tile_async(T* s, const T* g, int64_t rs, int row0, int limit, int tid) {
  constexpr int CH = D / 8;
  const uint32_t sbase = smem_u32(s);
#pragma unroll
  for (int i = tid; i < ROWS * CH; i += kThreads) {
    const int r = i / CH, c = i % CH;
    const int gr = row0 + r;
    const bool pred = gr < limit;
    const T* src = g + static_cast<int64_t>(pred ? gr : 0) * rs + c * 8;
    cp_async16(sbase + swz_off<D>(r, c * 8), src, pred);
  }
}

template <typename T, int D, bool VARLEN>
__global__ void __launch_bounds__(kThreads) bwd_main_kernel(const BwdParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* sK = reinterpret_cast<T*>(smem_raw);            // [64][D]
  T* sV = sK + kBN * D;                              // [64][D]
  T* sQ = sV + kBN * D;                              // [2][64][D]
  T* sdO = sQ + 2 * kBM * D;                         // [2][64][D]
  T* sDS = sdO + 2 * kBM * D;                        // [64 keys][64 queries]
  float* sL = reinterpret_cast<float*>(sDS + kBN * kBM);   // [2][64]
  float* sDel = sL + 2 * kBM;                              // [2][64]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wk = warp & 3, wq = warp >> 2;           // key block (16 keys) and query half (32 queries) of this warp
  const int kvh = blockIdx.y;
  int bb = blockIdx.z;
  int q_begin = 0, k_begin = 0, N = p.N, S = p.S;
  if (VARLEN) {
    q_begin = p.cu_q[bb];
    N = p.cu_q[bb + 1] - q_begin;
    k_begin = p.cu_k[bb];
    S = p.cu_k[bb + 1] - k_begin;
    bb = 0;
  }
  const int n0 = blockIdx.x * kBN;
  if (n0 >= S) return;
  const int off = S - N;

  const T* kg = reinterpret_cast<const T*>(p.k) + bb * p.k_bs + kvh * p.k_hs + k_begin * p.k_rs;
  const T* vg = reinterpret_cast<const T*>(p.v) + bb * p.v_bs + kvh * p.v_hs + k_begin * p.v_rs;

  // query tiles that can see keys of this tile: rows i >= n0 - off
  int m_begin = 0;
  if (p.causal) m_begin = max(0, n0 - off) / kBM;
  int m_end = (N + kBM - 1) / kBM;
  // a left window: the last row that still sees this tile's last key is i = key - off + window_left
  if (p.window_left >= 0) m_end = min(m_end, max(0, min(S, n0 + kBN) - 1 - off + p.window_left) / kBM + 1);
  const int nm = max(0, m_end - m_begin);
  const int n_iter = nm * p.gqa;
  const bool use_cap = p.softcap > 0.f;
  const float cap_in = use_cap ? p.scale / p.softcap : 0.f, cap_out = p.softcap * kLog2e;
  const bool precise_tanh = p.softcap >= kPreciseTanhMinCap;

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }

  auto load_q_tile = [&](int it, int stage) {
    const int gi = it / nm, m = m_begin + it % nm;
    const int hq = kvh * p.gqa + gi;
    const T* qg = reinterpret_cast<const T*>(p.q) + bb * p.q_bs + hq * p.q_hs + q_begin * p.q_rs;
    const T* dog = reinterpret_cast<const T*>(p.dout) + (static_cast<int64_t>(bb) * p.Hq + hq) * p.N * D +
                   static_cast<int64_t>(q_begin) * D;
    load_tile_async<kBM, D>(sQ + stage * kBM * D, qg, p.q_rs, m * kBM, N, tid);
    load_tile_async<kBM, D>(sdO + stage * kBM * D, dog, D, m * kBM, N, tid);
    if (tid < kBM) {
      const int row = m * kBM + tid;
      const int64_t idx = bb * p.lse_bs + hq * p.lse_hs + q_begin + row;
      sL[stage * kBM + tid] = row < N ? p.lse[idx] : INFINITY;      // +inf -> P = 0 for rows beyond N
      sDel[stage * kBM + tid] = row < N ? p.delta[idx] : 0.f;
    }
  };

  load_tile_async<kBN, D>(sK, kg, p.k_rs, n0, S, tid);
  load_tile_async<kBN, D>(sV, vg, p.v_rs, n0, S, tid);
  if (n_iter > 0) load_q_tile(0, 0);
  cp_async_commit();

  const uint32_t sK_u = smem_u32(sK), sV_u = smem_u32(sV), sDS_u = smem_u32(sDS);
  const int kr0 = wk * 16;          // key rows of this warp inside the tile
  const int qc0 = wq * 32;          // query columns of this warp inside the tile

  for (int it = 0; it < n_iter; ++it) {
    const int stage = it & 1;
    const int gi = it / nm, m = m_begin + it % nm;
    const int hq = kvh * p.gqa + gi;
    cp_async_wait<0>();
    __syncthreads();
    if (it + 1 < n_iter) {
      load_q_tile(it + 1, stage ^ 1);
      cp_async_commit();
    }
    const uint32_t sQ_u = smem_u32(sQ + stage * kBM * D), sdO_u = smem_u32(sdO + stage * kBM * D);
    const float alibi_l2 = p.alibi != nullptr ? p.alibi[hq] * kLog2e : 0.f;      // the bias the forward added
    const float* Ls = sL + stage * kBM;
    const float* Ds = sDel + stage * kBM;

    // ---- S^T = K.Q^T and dP^T = V.dO^T : [16 keys] x [32 queries] per warp ----
    float st[4][4], dp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t ak[4], av[4];
      const int arow = kr0 + (lane & 15), acol = kk * 16 + ((lane >> 4) << 3);
      ldmatrix_x4(ak, sK_u + swz_off<D>(arow, acol));
      ldmatrix_x4(av, sV_u + swz_off<D>(arow, acol));
#pragma unroll
      for (int nj = 0; nj < 2; ++nj) {
        uint32_t bq[4], bo[4];
        const int brow = qc0 + nj * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int bcol = kk * 16 + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(bq, sQ_u + swz_off<D>(brow, bcol));
        ldmatrix_x4(bo, sdO_u + swz_off<D>(brow, bcol));
        mma16816<T>(st[2 * nj], ak, bq[0], bq[1]);
        mma16816<T>(st[2 * nj + 1], ak, bq[2], bq[3]);
        mma16816<T>(dp[2 * nj], av, bo[0], bo[1]);
        mma16816<T>(dp[2 * nj + 1], av, bo[2], bo[3]);
      }
    }

    // ---- P^T and dS^T in registers: element e of n-tile j is (key kr0+g+8*(e>>1), query qc0+8j+2t+(e&1)) ----
    uint32_t pa[2][4], da[2][4];       // A fragments (16 keys x 16 queries) for the two query k-blocks
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float pv[4], dsv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = n0 + kr0 + g + ((e >> 1) << 3);
        const int ql = qc0 + 8 * j + 2 * t + (e & 1);
        const int qrow = m * kBM + ql;
        bool vis = key < S;
        if (p.causal) vis = vis && (key <= qrow + off);
        if (p.window_left >= 0) vis = vis && (key >= qrow + off - p.window_left);
        if (p.bmask != nullptr && vis) vis = p.bmask[(min(qrow, N - 1) / p.bm_bq) * p.bm_nk + key / p.bm_bk] != 0;
        const float L = Ls[ql];
        float base = st[j][e] * p.scale_log2, dcap = 1.f;
        if (use_cap) {
          const float th = cap_tanh(st[j][e] * cap_in, precise_tanh);
          base = cap_out * th;
          dcap = fmaf(-th, th, 1.f);                     // d(cap * tanh(s / cap)) / ds
        }
        const float sc = fmaf(alibi_l2, static_cast<float>(key - (qrow + off)), base);
        const float pe = (vis && L != -INFINITY) ? fast_exp2(sc - L) : 0.f;
        pv[e] = pe;
        dsv[e] = pe * (dp[j][e] - Ds[ql]) * dcap;
      }
      // n-tile j of the C layout is half (j & 1) of k-block (j >> 1) of the A layout
      pa[j >> 1][(j & 1) * 2 + 0] = Elem<T>::pack(pv[0], pv[1]);
      pa[j >> 1][(j & 1) * 2 + 1] = Elem<T>::pack(pv[2], pv[3]);
      const uint32_t d01 = Elem<T>::pack(dsv[0], dsv[1]), d23 = Elem<T>::pack(dsv[2], dsv[3]);
      da[j >> 1][(j & 1) * 2 + 0] = d01;
      da[j >> 1][(j & 1) * 2 + 1] = d23;
      // dS^T tile in shared memory: [key][query]
      const int qcol = qc0 + 8 * j + 2 * t;
      *reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(sDS) + swz_off<kBM>(kr0 + g, qcol & ~7) + (qcol & 7) * 2) = d01;
      *reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(sDS) + swz_off<kBM>(kr0 + g + 8, qcol & ~7) + (qcol & 7) * 2) = d23;
    }

    // ---- dV += P^T.dO and dK += dS^T.Q : k = 32 queries of this warp ----
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
      for (int dj = 0; dj < D / 16; ++dj) {
        uint32_t bo[4], bq[4];
        const int brow = qc0 + kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int bcol = dj * 16 + ((lane >> 4) << 3);
        ldmatrix_x4_trans(bo, sdO_u + swz_off<D>(brow, bcol));
        ldmatrix_x4_trans(bq, sQ_u + swz_off<D>(brow, bcol));
        mma16816<T>(dv[2 * dj], pa[kb], bo[0], bo[1]);
        mma16816<T>(dv[2 * dj + 1], pa[kb], bo[2], bo[3]);
        mma16816<T>(dk[2 * dj], da[kb], bq[0], bq[1]);
        mma16816<T>(dk[2 * dj + 1], da[kb], bq[2], bq[3]);
      }
    }
    __syncthreads();     // dS^T tile complete

    // ---- dQ tile += dS.K : warp computes 16 queries x D/2 columns over all 64 keys ----
    {
      const int qr0 = (warp & 3) * 16;
      const int d0 = (warp >> 2) * (D / 2);
      float dq[D / 16][4];
#pragma unroll
      for (int i = 0; i < D / 16; ++i) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < kBN / 16; ++kk) {
        uint32_t a[4];
        const int arow = kk * 16 + (lane & 7) + ((lane >> 4) << 3);     // key row of the stored dS^T
        const int acol = qr0 + (((lane >> 3) & 1) << 3);                // query column
        ldmatrix_x4_trans(a, sDS_u + swz_off<kBM>(arow, acol));
#pragma unroll
        for (int dj = 0; dj < D / 32; ++dj) {
          uint32_t b[4];
          const int brow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int bcol = d0 + dj * 16 + ((lane >> 4) << 3);
          ldmatrix_x4_trans(b, sK_u + swz_off<D>(brow, bcol));
          mma16816<T>(dq[2 * dj], a, b[0], b[1]);
          mma16816<T>(dq[2 * dj + 1], a, b[2], b[3]);
        }
      }
      float* acc = p.dq_acc + ((static_cast<int64_t>(bb) * p.Hq + hq) * p.N + q_begin) * D;
      const int r0 = m * kBM + qr0 + g, r1 = r0 + 8;
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        const int col = d0 + 8 * i + 2 * t;
        if (r0 < N) atomicAdd(reinterpret_cast<float2*>(acc + static_cast<int64_t>(r0) * D + col), make_float2(dq[i][0], dq[i][1]));
        if (r1 < N) atomicAdd(reinterpret_cast<float2*>(acc + static_cast<int64_t>(r1) * D + col), make_float2(dq[i][2], dq[i][3]));
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- dK, dV: the two query-half warps of a key block add up through shared memory, then store ----
  float* red = reinterpret_cast<float*>(sQ);        // [64 keys][D] floats fits in the Q/dO buffers (2*2*64*D*2 bytes)
  T* dkg = reinterpret_cast<T*>(p.dk) + bb * p.dk_bs + kvh * p.dk_hs + static_cast<int64_t>(k_begin) * p.dk_rs;
  T* dvg = reinterpret_cast<T*>(p.dv) + bb * p.dk_bs + kvh * p.dk_hs + static_cast<int64_t>(k_begin) * p.dk_rs;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    float (&acc)[D / 8][4] = pass == 0 ? dk : dv;
    const float mul = pass == 0 ? p.scale : 1.f;
    if (wq == 1) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const int col = 8 * i + 2 * t;
        *reinterpret_cast<float2*>(red + (kr0 + g) * D + col) = make_float2(acc[i][0], acc[i][1]);
        *reinterpret_cast<float2*>(red + (kr0 + g + 8) * D + col) = make_float2(acc[i][2], acc[i][3]);
      }
    }
    __syncthreads();
    if (wq == 0) {
      T* outp = pass == 0 ? dkg : dvg;
      const int k0r = n0 + kr0 + g, k1r = k0r + 8;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const int col = 8 * i + 2 * t;
        const float2 o0 = *reinterpret_cast<const float2*>(red + (kr0 + g) * D + col);
        const float2 o1 = *reinterpret_cast<const float2*>(red + (kr0 + g + 8) * D + col);
        if (k0r < S)
          *reinterpret_cast<uint32_t*>(outp + static_cast<int64_t>(k0r) * p.dk_rs + col) =
              Elem<T>::pack((acc[i][0] + o0.x) * mul, (acc[i][1] + o0.y) * mul);
        if (k1r < S)
          *reinterpret_cast<uint32_t*>(outp + static_cast<int64_t>(k1r) * p.dk_rs + col) =
              Elem<T>::pack((acc[i][2] + o1.x) * mul, (acc[i][3] + o1.y) * mul);
      }
    }
    __syncthreads();
  }
}

template <typename T, int D>
cudaError_t launch_t(const BwdParams& p, int dtype, bool varlen, int nbatch, int max_q, int max_k, bool allow_sm100,
                     cudaStream_t stream) {
  const int total_rows = p.B * p.Hq * p.N;
  {
    const bool rows16 = reinterpret_cast<uintptr_t>(p.o) % 16 == 0 && reinterpret_cast<uintptr_t>(p.dout) % 16 == 0 &&
                        p.o_rs % 8 == 0 && p.o_hs % 8 == 0 && p.o_bs % 8 == 0;
    if (rows16 && p.Hq <= 65535 && p.B <= 65535) {
      const long long threads = static_cast<long long>(p.N) * (D / 8);
      const dim3 pgrid(static_cast<unsigned>((threads + 255) / 256), p.Hq, p.B);
      bwd_preprocess_vec_kernel<T, D><<<pgrid, 256, 0, stream>>>(p);
    } else {
      const int blocks = (total_rows + 7) / 8;
      bwd_preprocess_kernel<T, D><<<blocks, 256, 0, stream>>>(p, total_rows);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  constexpr size_t smem = (2 * kBN * D + 4 * kBM * D + kBN * kBM) * sizeof(T) + 4 * kBM * sizeof(float);
  dim3 grid((max_k + kBN - 1) / kBN, p.Hkv, nbatch);
  cudaError_t e;
  if (p.dq_acc == nullptr) {
    // head_dim 128 on tcgen05: dK / dV and dQ by a kernel each, no accumulator and no conversion pass
    e = launch_bwd_dkv_sm100(p, dtype, nbatch, max_k, stream);
    if (e != cudaSuccess) return e;
    return launch_bwd_dq_sm100(p, dtype, nbatch, max_q, stream);
  }
  if (allow_sm100 && bwd_sm100_supported(dtype, D) && bwd_sm100_strides_ok(p)) {
    e = launch_bwd_sm100_main(p, dtype, nbatch, max_k, stream);
    if (e != cudaSuccess) return e;
  } else if (varlen) {
    e = cudaFuncSetAttribute(bwd_main_kernel<T, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    if (grid.x > 0) bwd_main_kernel<T, D, true><<<grid, kThreads, smem, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(bwd_main_kernel<T, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    if (grid.x > 0) bwd_main_kernel<T, D, false><<<grid, kThreads, smem, stream>>>(p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const long long n_pairs = static_cast<long long>(total_rows) * D / 2;
  long long blocks = (n_pairs + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  bwd_convert_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p.dq_acc, reinterpret_cast<T*>(p.dq), p.scale, n_pairs);
  return cudaGetLastError();
}

}  // namespace

// delta, work counter and -- except on the split head_dim-128 path -- the fp32 dQ accumulator
size_t bwd_workspace_bytes(int B, int Hq, int N_total, int D, bool split) {
  const size_t rows = static_cast<size_t>(B) * Hq * N_total;
  return bwd_align(rows * sizeof(float)) + 256 + (split ? 0 : bwd_align(rows * D * sizeof(float)));
}

bool bwd_takes_split_path(const BwdParams& p, int dtype, int D, bool allow_sm100) {
  return allow_sm100 && bwd_split_sm100_supported(dtype, D) && bwd_sm100_strides_ok(p);
}

cudaError_t launch_bwd(const BwdParams& p_in, int dtype, int D, bool varlen, int nbatch, int max_q, int max_k,
                       void* workspace, bool allow_sm100, cudaStream_t stream) {
  BwdParams p = p_in;
  const size_t rows = static_cast<size_t>(p.B) * p.Hq * p.N;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  p.delta = reinterpret_cast<float*>(ws);
  p.work_counter = reinterpret_cast<int*>(ws + bwd_align(rows * sizeof(float)));
  p.dq_acc = bwd_takes_split_path(p, dtype, D, allow_sm100) ? nullptr
                                                            : reinterpret_cast<float*>(ws + bwd_align(rows * sizeof(float)) + 256);
  if (rows == 0) return cudaSuccess;
  if (dtype == 0 && D == 64) return launch_t<__half, 64>(p, dtype, varlen, nbatch, max_q, max_k, allow_sm100, stream);
  if (dtype == 0 && D == 128) return launch_t<__half, 128>(p, dtype, varlen, nbatch, max_q, max_k, allow_sm100, stream);
  if (dtype == 1 && D == 64) return launch_t<__nv_bfloat16, 64>(p, dtype, varlen, nbatch, max_q, max_k, allow_sm100, stream);
  if (dtype == 1 && D == 128) return launch_t<__nv_bfloat16, 128>(p, dtype, varlen, nbatch, max_q, max_k, allow_sm100, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200fa
