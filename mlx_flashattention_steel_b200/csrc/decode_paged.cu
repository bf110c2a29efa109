// Paged-KV decode: split-KV flash-decoding with the log-sum-exp combine inside the
// same launch.  Replaces the reference's gather + per-sequence two-kernel flash-decode
// route (mlx_mfa/attention.py:3008-3017; csrc/mfa_attention.cpp:150-288; kernels
// csrc/mfa_steel_fwd.cpp:1541-1991, 2008-2105) and its paged forward
// (csrc/mfa_steel_fwd.cpp:2462-3121).
//
// Shape of the work
//   * The pages of all sequences form one list of U units.  CTA c of G takes units
//     [c*U/G, (c+1)*U/G): equal bytes per CTA whatever the sequence lengths are.
//   * A CTA holds HPC kv heads (one consumer warp each) plus one producer warp.  The
//     producer looks pages up in block_table and brings each page in with ONE TMA
//     tensor copy per pool ([block_size tokens] x [HPC heads] x [row bytes], a
//     contiguous 16 KB of HBM for 8 int8 heads), 128B-swizzled by token, plus one
//     bulk copy per scale array, into a ring of stages guarded by mbarriers.
//   * A consumer warp computes S = Q.K^T (rows = the GQA group x query tokens, padded
//     to the 16 rows of mma.m16n8k16) and O^T += V^T.P^T for its head.  int8 / e4m3
//     values are widened to f16 in registers straight from the swizzled tile;
//     k_scale multiplies the scores, v_scale is folded into P.
//   * A CTA that covers a whole sequence writes the result; otherwise it writes a
//     partial (normalised O, base-2 lse) and bumps a counter; the CTA that brings the
//     counter to the number of parts combines them.  Nobody spins on anybody.
//
//   * Pages of 32, 64, ... tokens are walked as 16-token units (a unit is what one TMA box and one consumer step
//     cover).  Dense caches [B, Hkv, S, D] (the reference's flash-decode route for N <= 4, S >= 256 on plain
//     flash_attention calls, csrc/mfa_attention.cpp:150-288) run the same kernel: unit j of sequence b is its tokens
//     [16 j, 16 j + 16), addressed through a tensor map with the cache's own strides, and no table is read.
//   * head_dim 128 for every pool type; head_dim 64 for 16-bit pools and dense caches.
//
// Every mbarrier wait is bounded (tma.cuh); a timeout raises the error word at the
// start of the workspace and the CTA leaves.
#include <cuda_fp8.h>

#include <cstdio>
#include <type_traits>

#include <mutex>

#include "../../include/b200fa.h"
#include "common.cuh"
#include "decode.h"
#include "tma.cuh"

namespace b200fa {

namespace {

constexpr int kBS = 16;           // tokens per unit (one TMA box, one consumer step); a page is 1, 2, 4, ... units
constexpr int kMaxStages = 8;

enum KvKind { KV_F16 = 0, KV_BF16 = 1, KV_I8 = 2, KV_E4M3 = 3 };

struct DecodeLayout {          // workspace carve-up, in bytes from the workspace base
  size_t err;                  // int[4]: [0] error word
  size_t counters;             // int[B * HG]
  size_t page_start;           // int[B + 1]
  size_t part_lse;             // float[slots * Hq * Nq]
  size_t part_o;               // float[slots * Hq * Nq * D]
  size_t total;
  int slots;
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ __device__ inline DecodeLayout make_layout(int B, int Hq, int Nq, int HG, int G, int kD) {
  DecodeLayout L;
  L.err = 0;
  L.counters = 16;
  L.page_start = align_up(L.counters + sizeof(int) * static_cast<size_t>(B) * HG, 16);
  L.slots = G + B;
  L.part_lse = align_up(L.page_start + sizeof(int) * (static_cast<size_t>(B) + 1), 16);
  L.part_o = align_up(L.part_lse + sizeof(float) * static_cast<size_t>(L.slots) * Hq * Nq, 16);
  L.total = align_up(L.part_o + sizeof(float) * static_cast<size_t>(L.slots) * Hq * Nq * kD, 16);
  return L;
}

struct KernelArgs {
  DecodeParams p;
  DecodeLayout lay;
  int HG;            // head groups = Hkv / HPC
  int group;         // Hq / Hkv
  int rows;          // group * Nq (<= 8)
  int stages;
  int upp;              // 16-token units per page = block_size / 16
  int stage_kv_bytes;   // bytes of one K (or V) stage tile = HPC * kBS * row_bytes
  int scale_bytes;      // bytes of one scale page = kBS * Hkv * 2 (0 when not quantized)
  float q_prescale;     // folded into Q (8-bit pools) or applied to the scores (16-bit)
  float cap_log2;       // softcap * log2(e)
  float inv_cap;        // 1 / softcap
};

// ---------------------------------------------------------------------------
// plan: page prefix sums, counters and error word reset
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) decode_plan_kernel(const int32_t* __restrict__ seq_lens, int B,
                                                           int max_kv_len, int n_counters,
                                                           int* __restrict__ err, int* __restrict__ counters,
                                                           int* __restrict__ page_start) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { carry = 0; page_start[0] = 0; }
  if (tid < 4) err[tid] = 0;
  for (int i = tid; i < n_counters; i += blockDim.x) counters[i] = 0;
  __syncthreads();
  for (int base = 0; base < B; base += blockDim.x) {
    const int i = base + tid;
    int val = 0;
    if (i < B) {
      int len = seq_lens != nullptr ? seq_lens[i] : max_kv_len;
      len = len < 0 ? 0 : (len > max_kv_len ? max_kv_len : len);
      val = (len + kBS - 1) / kBS;
    }
    int x = val;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int incl = x + (warp > 0 ? warp_sums[warp - 1] : 0) + carry;
    if (i < B) page_start[i + 1] = incl;
    __syncthreads();
    if (tid == blockDim.x - 1) carry = incl;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_half(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
  return __half2float(__ushort_as_half(v));
}
// two biased bytes (x ^ 0x80) at byte positions given by `sel` -> half2 of the signed values
__device__ __forceinline__ uint32_t i8pair_to_h2(uint32_t biased, uint32_t sel) {
  const uint32_t magic = prmt(biased, 0x64646464u, sel);      // 0x64XX64YY = 1024 + u
  __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&magic), __floats2half2_rn(1152.f, 1152.f));
  return *reinterpret_cast<uint32_t*>(&h);
}
// the same without the subtraction: half2 of 1024 + (x + 128) = x + 1152.  Used for K, where the constant offset
// becomes 1152 * sum(q) in each score and is taken out of the fp32 accumulator after the eight MMAs of a tile.
__device__ __forceinline__ uint32_t i8pair_to_h2_biased(uint32_t biased, uint32_t sel) {
  return prmt(biased, 0x64646464u, sel);
}
__device__ __forceinline__ uint32_t e4m3pair_to_h2(uint32_t two_bytes) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_bytes & 0xffffu), __NV_E4M3);
  __half2 h = r;
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ float clamp_h(float x) { return fminf(fmaxf(x, -65504.f), 65504.f); }

// CTA index (of G) whose unit range [c*U/G, (c+1)*U/G) holds unit u
__device__ __forceinline__ int cta_of_unit(long long u, int G, long long U) {
  return static_cast<int>(((u + 1) * G - 1) / U);
}

// ---------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------
// CAP: soft cap on.  A template parameter so that the common launch without one carries no tanh code in its unrolled
// inner loops (with it compiled in, config 4 -- which has no soft cap -- ran 4 % slower).
template <int KV, int HPC, int kD, bool CAP>
__global__ void __launch_bounds__((HPC + 1) * 32, 1)
decode_paged_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const KernelArgs a) {
  constexpr bool kQuant = (KV == KV_I8 || KV == KV_E4M3);
  static_assert(kD == 128 || (kD == 64 && !kQuant), "head_dim 64 is built for 16-bit pools only");
  constexpr int kKS = kD / 16;                         // k-steps of S = Q.K^T, m-tiles of O^T
  constexpr int kRowBytes = kQuant ? kD : 2 * kD;      // bytes of one (token, head) row
  constexpr int kHalves = kRowBytes / 128;
  constexpr int kHeadBytes = kBS * kRowBytes;          // one head of one page in shared memory
  using MmaT = typename std::conditional<KV == KV_BF16, __nv_bfloat16, __half>::type;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve: [stages] K tiles, [stages] V tiles, [stages] k scales, [stages] v scales, barriers, misc
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const DecodeParams& p = a.p;
  const int NS = a.stages;
  unsigned char* sK = smem;
  unsigned char* sV = sK + static_cast<size_t>(NS) * a.stage_kv_bytes;
  unsigned char* sKs = sV + static_cast<size_t>(NS) * a.stage_kv_bytes;
  unsigned char* sVs = sKs + static_cast<size_t>(NS) * a.scale_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sVs + static_cast<size_t>(NS) * a.scale_bytes);  // full[NS], empty[NS]
  int* s_page = reinterpret_cast<int*>(bars + 2 * kMaxStages);
  volatile int* s_abort = s_page + kMaxStages;
  int* s_last = const_cast<int*>(s_abort) + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int hg = blockIdx.y;
  const int c = blockIdx.x;

  unsigned char* ws = reinterpret_cast<unsigned char*>(p.workspace);
  int* err = reinterpret_cast<int*>(ws + a.lay.err);
  int* counters = reinterpret_cast<int*>(ws + a.lay.counters);
  const int* page_start = reinterpret_cast<const int*>(ws + a.lay.page_start);
  float* part_lse = reinterpret_cast<float*>(ws + a.lay.part_lse);
  float* part_o = reinterpret_cast<float*>(ws + a.lay.part_o);

  const int rows = a.rows;
  const int HqNq = p.Hq * p.Nq;

  // Sequences of length zero have no unit: CTA 0 of each head group zero-fills them.
  if (c == 0) {
    for (int b = 0; b < p.B; ++b) {
      if (page_start[b + 1] != page_start[b]) continue;
      for (int i = tid; i < HPC * a.group * p.Nq * kD; i += blockDim.x) {
        const int d = i % kD;
        const int r = i / kD;                       // (head in cta, group, qi)
        const int qi = r % p.Nq;
        const int hq = (hg * HPC) * a.group + r / p.Nq;
        const size_t orow = (static_cast<size_t>(b) * p.Hq + hq) * p.Nq + qi;
        const size_t o = orow * kD + d;
        if (p.packed_f32) {
          float* pk = reinterpret_cast<float*>(p.out) + orow * (kD + 4);
          pk[d] = 0.f;
          if (d == 0) pk[kD] = -INFINITY;
        } else {
          if (p.q_dtype == 0) reinterpret_cast<__half*>(p.out)[o] = __float2half(0.f);
          else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16(0.f);
          if (p.lse != nullptr && d == 0) p.lse[orow] = -INFINITY;
        }
      }
    }
  }

  // With fewer units than CTAs only the first U CTAs work, one unit each, so that the
  // CTAs sharing a sequence are always consecutive.
  const long long U = page_start[p.B];
  const int G = U < static_cast<long long>(gridDim.x) ? static_cast<int>(U) : static_cast<int>(gridDim.x);
  if (c >= G) return;
  const long long lo = static_cast<long long>(c) * U / G;
  const long long hi = static_cast<long long>(c + 1) * U / G;
  if (lo >= hi) return;

  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);                 // full: producer arrive (+ tx bytes)
      mbar_init(smem_u32(&bars[kMaxStages + i]), HPC);  // empty: one arrive per consumer warp
    }
    *s_abort = 0;
    *s_last = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  // first sequence: largest b with page_start[b] <= lo
  int b_first;
  {
    int l = 0, r = p.B;   // invariant: page_start[l] <= lo < page_start[r]  (page_start[B] = U > lo)
    while (r - l > 1) {
      const int m = (l + r) >> 1;
      if (page_start[m] <= lo) l = m; else r = m;
    }
    b_first = l;
  }

  const uint32_t tx_bytes = 2u * a.stage_kv_bytes + 2u * a.scale_bytes;

  if (warp == HPC) {
    // ======================= producer warp =======================
    int stage = 0;
    uint32_t phase = 0;
    long long u = lo;
    int b = b_first;
    bool ok = true;
    while (u < hi && ok) {
      const int s0 = page_start[b], s1 = page_start[b + 1];
      if (s1 <= u) { ++b; continue; }
      const int j_lo = static_cast<int>(u - s0);
      const int j_hi = static_cast<int>((hi < s1 ? hi : s1) - s0);
      const int32_t* row = p.dense ? nullptr : p.block_table + static_cast<size_t>(b) * p.max_blocks;
      for (int j0 = j_lo; j0 < j_hi && ok; j0 += 32) {
        const int jj = j0 + lane;
        // first token of unit jj in the pool (paged: its page's tokens start at page * block_size) or in the
        // sequence (dense); -1 = no page
        int my_tok = -1;
        if (jj < j_hi) {
          if (p.dense) {
            my_tok = jj * kBS;
          } else {
            const int pg_id = row[jj / a.upp];
            if (pg_id >= p.num_pages) atomicOr(err, 2);              // table entry beyond the pool
            else if (pg_id >= 0) my_tok = pg_id * p.block_size + (jj % a.upp) * kBS;
          }
        }
        const int n = min(32, j_hi - j0);
        for (int i = 0; i < n; ++i) {
          const int page = __shfl_sync(0xffffffffu, my_tok, i);       // token offset of the unit, or -1
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bars[kMaxStages + stage]), phase ^ 1u, s_abort))) { ok = false; break; }
          if (lane == 0) {
            s_page[stage] = page;
            const uint32_t full = smem_u32(&bars[stage]);
            if (page >= 0) {
              mbar_arrive_expect_tx(full, tx_bytes);
              const int batch_coord = p.dense ? b : 0;
              tma_load_5d(smem_u32(sK + static_cast<size_t>(stage) * a.stage_kv_bytes), &tmK, full, 0, page, 0, hg * HPC, batch_coord);
              tma_load_5d(smem_u32(sV + static_cast<size_t>(stage) * a.stage_kv_bytes), &tmV, full, 0, page, 0, hg * HPC, batch_coord);
              if (kQuant) {
                const size_t soff = static_cast<size_t>(page / kBS) * a.scale_bytes;
                bulk_load(smem_u32(sKs + static_cast<size_t>(stage) * a.scale_bytes),
                          reinterpret_cast<const unsigned char*>(p.k_scale) + soff, a.scale_bytes, full);
                bulk_load(smem_u32(sVs + static_cast<size_t>(stage) * a.scale_bytes),
                          reinterpret_cast<const unsigned char*>(p.v_scale) + soff, a.scale_bytes, full);
              }
            } else {
              mbar_arrive(full);                  // hole in the table: consumers treat K = V = 0
            }
          }
          __syncwarp();
          if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
      }
      u = s0 + j_hi;
      if (u >= s1) ++b;
    }
    if (!ok && lane == 0) atomicOr(err, 1);
    return;
  }

  // ======================= consumer warps =======================
  const int kvh = hg * HPC + warp;
  const int qi_row = g / a.group;                // query token of fragment row g
  const int hq_row = kvh * a.group + g % a.group;
  const bool row_valid = g < rows;
  int stage = 0;
  uint32_t phase = 0;
  long long u = lo;
  int b = b_first;
  bool ok = true;

  while (u < hi && ok) {
    const int s0 = page_start[b], s1 = page_start[b + 1];
    if (s1 <= u) { ++b; continue; }
    const int j_lo = static_cast<int>(u - s0);
    const int j_hi = static_cast<int>((hi < s1 ? hi : s1) - s0);
    int len = p.seq_lens != nullptr ? p.seq_lens[b] : p.max_kv_len;
    len = len < 0 ? 0 : (len > p.max_kv_len ? p.max_kv_len : len);
    const int c_first = cta_of_unit(s0, G, U);
    const int c_last = cta_of_unit(static_cast<long long>(s1) - 1, G, U);
    const int n_parts = c_last - c_first + 1;

    // ---- Q fragments (A operand rows 0..7; rows 8..15 are zero padding) ----
    uint32_t qa[8][2];                 // kKS k-steps are used
    float q_bias = 0.f;          // int8 pools: 1152 * sum of the row's query values (see i8pair_to_h2_biased)
    {
      const size_t qoff = ((static_cast<size_t>(b) * p.Hq + hq_row) * p.Nq + qi_row) * kD;
      if constexpr (kQuant) {
        // lane t owns d in [32t, 32t+32): k-step s uses d = 32t + 4s + {0,1 | 2,3}
        float f[32];
        if (row_valid) {
          if (p.q_dtype == 0) {
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.q) + qoff + 32 * t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w = src[i];
              const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&ww[e]));
                f[i * 8 + e * 2] = v2.x; f[i * 8 + e * 2 + 1] = v2.y;
              }
            }
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + qoff + 32 * t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w = src[i];
              const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float2 v2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww[e]));
                f[i * 8 + e * 2] = v2.x; f[i * 8 + e * 2 + 1] = v2.y;
              }
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = 0.f;
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          qa[s][0] = pack_h2(clamp_h(f[4 * s] * a.q_prescale), clamp_h(f[4 * s + 1] * a.q_prescale));
          qa[s][1] = pack_h2(clamp_h(f[4 * s + 2] * a.q_prescale), clamp_h(f[4 * s + 3] * a.q_prescale));
        }
        if (KV == KV_I8) {
          // 1152 * (sum over the head dim of this row's f16 query values): the part of every score that comes from
          // the +1152 offset left inside the widened K values
          float qs = 0.f;
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            const float2 u = __half22float2(*reinterpret_cast<const __half2*>(&qa[s][0]));
            const float2 w = __half22float2(*reinterpret_cast<const __half2*>(&qa[s][1]));
            qs += (u.x + u.y) + (w.x + w.y);
          }
          qs += __shfl_xor_sync(0xffffffffu, qs, 1);
          qs += __shfl_xor_sync(0xffffffffu, qs, 2);
          q_bias = 1152.f * qs;
        }
      } else {
        // natural order: a0 = Q[g][16s + 2t, +1], a2 = Q[g][16s + 8 + 2t, +1]
        const uint32_t* src = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.q) + qoff);
#pragma unroll
        for (int s = 0; s < kKS; ++s) {
          qa[s][0] = row_valid ? src[8 * s + t] : 0u;
          qa[s][1] = row_valid ? src[8 * s + 4 + t] : 0u;
        }
      }
    }

    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;
    float vnorm = 1.f, vunnorm = 1.f;             // power-of-two normalisation of v_scale inside P
    bool first_page = true;
    const int causal_lim = p.causal ? (qi_row + len - p.Nq) : 0x7fffffff;   // last visible token of row g

    // Two pages per iteration: their loads, conversions and MMAs are independent, which gives the
    // scheduler twice the instruction-level parallelism, and one online-softmax step covers 32 tokens.
    for (int j = j_lo; j < j_hi; j += 2) {
      const int np = min(2, j_hi - j);
      int stg[2], pg[2];
      {
        int s2 = stage;
        uint32_t ph2 = phase;
        bool okw = true;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          stg[q] = s2;
          if (q < np && okw) {
            okw = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bars[s2]), ph2, s_abort));
            if (++s2 == NS) { s2 = 0; ph2 ^= 1u; }
          }
        }
        if (!okw) { ok = false; break; }
      }
      uint32_t kbase[2], vbase[2], ksb[2], vsb[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        pg[q] = q < np ? s_page[stg[q]] : -2;       // -1: hole in the table, -2: no second page
        kbase[q] = smem_u32(sK + static_cast<size_t>(stg[q]) * a.stage_kv_bytes) + warp * kHeadBytes;
        vbase[q] = smem_u32(sV + static_cast<size_t>(stg[q]) * a.stage_kv_bytes) + warp * kHeadBytes;
        ksb[q] = smem_u32(sKs + static_cast<size_t>(stg[q]) * a.scale_bytes) + kvh * 2;
        vsb[q] = smem_u32(sVs + static_cast<size_t>(stg[q]) * a.scale_bytes) + kvh * 2;
      }
      const int scale_stride = p.Hkv * 2;          // bytes between tokens in a scale page

      // ---- S = Q K^T : rows = query rows (8 real), cols = 16 tokens (two n-tiles) per page ----
      float sacc[2][2][4];
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int i = 0; i < 2; ++i) { sacc[q][i][0] = sacc[q][i][1] = sacc[q][i][2] = sacc[q][i][3] = 0.f; }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (pg[q] >= 0) {
          if constexpr (kQuant) {
#pragma unroll
            for (int jn = 0; jn < 2; ++jn) {
              const int tok = 8 * jn + g;                     // tok & 7 == g
              const uint32_t rowa = kbase[q] + tok * 128;
              const uint4 w0 = lds128(rowa + (((2 * t) ^ g) << 4));
              const uint4 w1 = lds128(rowa + (((2 * t + 1) ^ g) << 4));
              const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
              for (int s = 0; s < 8; ++s) {
                uint32_t b0, b1;
                if (KV == KV_I8) {
                  const uint32_t x = words[s] ^ 0x80808080u;
                  b0 = i8pair_to_h2_biased(x, 0x4140u);
                  b1 = i8pair_to_h2_biased(x, 0x4342u);
                } else {
                  b0 = e4m3pair_to_h2(words[s]);
                  b1 = e4m3pair_to_h2(words[s] >> 16);
                }
                const uint32_t afrag[4] = {qa[s][0], 0u, qa[s][1], 0u};
                mma16816<MmaT>(sacc[q][jn], afrag, b0, b1);
              }
            }
          } else {
#pragma unroll
            for (int s = 0; s < kKS; ++s) {
              uint32_t bfr[4];
              const int tok = (lane & 7) + ((lane >> 4) << 3);
              const int dcol = 16 * s + (((lane >> 3) & 1) << 3);
              const uint32_t addr = kbase[q] + (dcol >> 6) * (kBS * 128) + tok * 128 + ((((dcol & 63) >> 3) ^ (tok & 7)) << 4);
              ldmatrix_x4(bfr, addr);
              const uint32_t afrag[4] = {qa[s][0], 0u, qa[s][1], 0u};
              mma16816<MmaT>(sacc[q][0], afrag, bfr[0], bfr[1]);
              mma16816<MmaT>(sacc[q][1], afrag, bfr[2], bfr[3]);
            }
          }
        }
      }

      // ---- scale / softcap / masks: per page this lane holds tokens {2t, 2t+1, 8+2t, 9+2t} of row g ----
      float sc[2][4], vsc[2][4];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int tok0 = (j + q) * kBS;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = ((e >> 1) << 3) + 2 * t + (e & 1);
          float s = sacc[q][e >> 1][e & 1];
          vsc[q][e] = 1.f;
          if (kQuant) {
            float ksv = 1.f;
            if (pg[q] >= 0) {
              ksv = lds_half(ksb[q] + tok * scale_stride);
              vsc[q][e] = lds_half(vsb[q] + tok * scale_stride);
              if (KV == KV_I8) s -= q_bias;                 // the K values went into the MMA as x + 1152
            }
            s *= ksv;
          } else {
            s *= a.q_prescale;
          }
          if constexpr (CAP) s = a.cap_log2 * cap_tanh(s * a.inv_cap, a.inv_cap * kPreciseTanhMinCap <= 1.f);
          const int tg = tok0 + tok;
          sc[q][e] = (pg[q] != -2 && tg < len && tg <= causal_lim) ? s : -INFINITY;
          if (tg >= len) vsc[q][e] = 0.f;               // whatever the slot's scale holds (it may be a NaN pattern)
        }
      }
      if (kQuant && first_page) {
        // power of two near the first token's v scale keeps p * v_scale inside f16's normal range
        float v0 = (pg[0] >= 0) ? lds_half(vsb[0]) : 1.f;
        v0 = __shfl_sync(0xffffffffu, v0, 0);
        uint32_t bits = __float_as_uint(v0) & 0x7f800000u;
        if (bits == 0u || bits == 0x7f800000u) bits = 0x3f800000u;
        vunnorm = __uint_as_float(bits);
        vnorm = 1.f / vunnorm;
        first_page = false;
      }

      // ---- online softmax over the (up to) 32 tokens ----
      float mx = fmaxf(fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[0][2], sc[0][3])),
                       fmaxf(fmaxf(sc[1][0], sc[1][1]), fmaxf(sc[1][2], sc[1][3])));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float msub = (m_new == -INFINITY) ? 0.f : m_new;
      const bool grew = m_new > m_run;
      if (__any_sync(0xffffffffu, grew)) {
        const float corr = fast_exp2(m_run - msub);       // 1 when unchanged, 0 from -inf
        l_run *= corr;
        const float c0 = __shfl_sync(0xffffffffu, corr, (2 * t) * 4);
        const float c1 = __shfl_sync(0xffffffffu, corr, (2 * t + 1) * 4);
#pragma unroll
        for (int i = 0; i < kKS; ++i) {
          oacc[i][0] *= c0; oacc[i][1] *= c1; oacc[i][2] *= c0; oacc[i][3] *= c1;
        }
        m_run = m_new;
      }
      float pr[2][4];
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pr[q][e] = fast_exp2(sc[q][e] - msub);
          l_run += pr[q][e];
        }

      // ---- O^T += V^T P^T : rows = 16 head-dim values per m-tile, cols = query rows ----
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (pg[q] >= 0) {
          // Slots of the last page beyond the sequence's end hold whatever the pool's owner left there; their P is
          // zero, but 0 * NaN (or 0 * inf) would still poison the row, so their V values are cleared as they are
          // loaded.  amask[h]: tokens (2t, 2t+1) for h = 0, (2t+8, 2t+9) for h = 1, one 16-bit lane per token.
          const int tail_from = len - (j + q) * kBS;      // first token of this page that is beyond the sequence
          const bool tail = tail_from < kBS;              // warp-uniform
          uint32_t amask[2] = {0xffffffffu, 0xffffffffu};
          if (tail) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
              amask[h] = (2 * t + 8 * h < tail_from ? 0x0000ffffu : 0u) | (2 * t + 8 * h + 1 < tail_from ? 0xffff0000u : 0u);
          }
          uint32_t pb0, pb1;
          if (kQuant) {
            pb0 = pack_h2(pr[q][0] * vsc[q][0] * vnorm, pr[q][1] * vsc[q][1] * vnorm);
            pb1 = pack_h2(pr[q][2] * vsc[q][2] * vnorm, pr[q][3] * vsc[q][3] * vnorm);
          } else if (KV == KV_BF16) {
            pb0 = pack_bf2(pr[q][0], pr[q][1]);
            pb1 = pack_bf2(pr[q][2], pr[q][3]);
          } else {
            pb0 = pack_h2(pr[q][0], pr[q][1]);
            pb1 = pack_h2(pr[q][2], pr[q][3]);
          }
          if constexpr (kQuant) {
            // lane (g,t) reads word w = g + 8*jj (4 head-dim bytes) of token rows 2t, 2t+1, 2t+8, 2t+9
            const uint32_t rA = vbase[q] + (2 * t) * 128, rB = rA + 128, rC = rA + 8 * 128, rD = rC + 128;
            const int xa = (2 * t) & 7, xb = (2 * t + 1) & 7;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int w = g + 8 * jj;
              const int ch = w >> 2, wi = (w & 3) << 2;
              uint32_t A = lds32(rA + ((ch ^ xa) << 4) + wi);
              uint32_t Bw = lds32(rB + ((ch ^ xb) << 4) + wi);
              uint32_t Cw = lds32(rC + ((ch ^ xa) << 4) + wi);
              uint32_t Dw = lds32(rD + ((ch ^ xb) << 4) + wi);
              if (KV == KV_I8) { A ^= 0x80808080u; Bw ^= 0x80808080u; Cw ^= 0x80808080u; Dw ^= 0x80808080u; }
              const uint32_t ab[2] = {prmt(A, Bw, 0x5140u), prmt(A, Bw, 0x7362u)};   // [A0 B0 A1 B1], [A2 B2 A3 B3]
              const uint32_t cd[2] = {prmt(Cw, Dw, 0x5140u), prmt(Cw, Dw, 0x7362u)};
#pragma unroll
              for (int kp = 0; kp < 2; ++kp) {
                uint32_t af[4];
                if (KV == KV_I8) {
                  af[0] = i8pair_to_h2(ab[kp], 0x4140u);   // head-dim byte 2kp   , tokens 2t, 2t+1
                  af[1] = i8pair_to_h2(ab[kp], 0x4342u);   // head-dim byte 2kp+1 , tokens 2t, 2t+1
                  af[2] = i8pair_to_h2(cd[kp], 0x4140u);   // tokens 2t+8, 2t+9
                  af[3] = i8pair_to_h2(cd[kp], 0x4342u);
                } else {
                  af[0] = e4m3pair_to_h2(ab[kp]);
                  af[1] = e4m3pair_to_h2(ab[kp] >> 16);
                  af[2] = e4m3pair_to_h2(cd[kp]);
                  af[3] = e4m3pair_to_h2(cd[kp] >> 16);
                  if (tail) { af[0] &= amask[0]; af[1] &= amask[0]; af[2] &= amask[1]; af[3] &= amask[1]; }
                }
                mma16816<MmaT>(oacc[jj * 2 + kp], af, pb0, pb1);
              }
            }
          } else {
#pragma unroll
            for (int mt = 0; mt < kKS; ++mt) {
              uint32_t af[4];
              const int tok = (lane & 7) + ((lane >> 4) << 3);
              const int dcol = 16 * mt + (((lane >> 3) & 1) << 3);
              const uint32_t addr = vbase[q] + (dcol >> 6) * (kBS * 128) + tok * 128 + ((((dcol & 63) >> 3) ^ (tok & 7)) << 4);
              // after .trans: a0 = (d 0-7, tok 0-7), a1 = (d 8-15, tok 0-7), a2 = (d 0-7, tok 8-15), a3 = (d 8-15, tok 8-15)
              ldmatrix_x4_trans(af, addr);
              if (tail) { af[0] &= amask[0]; af[1] &= amask[0]; af[2] &= amask[1]; af[3] &= amask[1]; }
              mma16816<MmaT>(oacc[mt], af, pb0, pb1);
            }
          }
        }
      }

      __syncwarp();
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (q < np) {
          if (lane == 0) mbar_arrive(smem_u32(&bars[kMaxStages + stg[q]]));
          if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
      }
    }
    if (!ok) break;

    // ---- end of this CTA's part of sequence b ----
    float l_row = l_run;
    l_row += __shfl_xor_sync(0xffffffffu, l_row, 1);
    l_row += __shfl_xor_sync(0xffffffffu, l_row, 2);
    const float lse_row = l_row > 0.f ? m_run + log2f(l_row) : -INFINITY;
    const float inv_row = l_row > 0.f ? vunnorm / l_row : 0.f;
    // accumulator columns are query rows 2t and 2t+1
    const float inv0 = __shfl_sync(0xffffffffu, inv_row, (2 * t) * 4);
    const float inv1 = __shfl_sync(0xffffffffu, inv_row, (2 * t + 1) * 4);
    const int r0 = 2 * t, r1 = 2 * t + 1;
    const bool direct = (n_parts == 1);
    const int slot = c + b;

#pragma unroll
    for (int i = 0; i < kKS; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // head-dim index of accumulator register e of m-tile i
        int d;
        if (kQuant) d = 32 * (i >> 1) + 4 * g + 2 * (i & 1) + (e >> 1);
        else d = 16 * i + g + ((e >> 1) << 3);
        const int r = (e & 1) ? r1 : r0;
        if (r >= rows) continue;
        const float val = oacc[i][e] * ((e & 1) ? inv1 : inv0);
        const int hq = kvh * a.group + r % a.group;
        const int qi = r / a.group;
        if (direct) {
          const size_t orow = (static_cast<size_t>(b) * p.Hq + hq) * p.Nq + qi;
          const size_t o = orow * kD + d;
          if (p.packed_f32) reinterpret_cast<float*>(p.out)[orow * (kD + 4) + d] = val;
          else if (p.q_dtype == 0) reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(val);
          else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(val);
        } else {
          part_o[(static_cast<size_t>(slot) * HqNq + hq * p.Nq + qi) * kD + d] = val;
        }
      }
    }
    if (t == 0 && row_valid) {
      if (direct) {
        const size_t orow = (static_cast<size_t>(b) * p.Hq + hq_row) * p.Nq + qi_row;
        if (p.packed_f32) reinterpret_cast<float*>(p.out)[orow * (kD + 4) + kD] = lse_row;
        else if (p.lse != nullptr) p.lse[orow] = lse_row;
      } else {
        part_lse[static_cast<size_t>(slot) * HqNq + hq_row * p.Nq + qi_row] = lse_row;
      }
    }

    if (!direct) {
      __threadfence();
      named_bar_sync(1, HPC * 32);
      if (tid == 0) {
        const int old = atomicAdd(&counters[b * a.HG + hg], 1);
        *s_last = (old == n_parts - 1) ? 1 : 0;
      }
      named_bar_sync(1, HPC * 32);
      const bool last = *s_last != 0;
      if (last) {
        __threadfence();
        // combine: L = log2 sum_i 2^lse_i ; O = sum_i 2^(lse_i - L) O_i  (csrc/mfa_steel_fwd.cpp:2066-2101)
        for (int r = 0; r < rows; ++r) {
          const int hq = kvh * a.group + r % a.group;
          const int qi = r / a.group;
          const size_t rowi = static_cast<size_t>(hq) * p.Nq + qi;
          float mmax = -INFINITY;
          for (int i = 0; i < n_parts; ++i)
            mmax = fmaxf(mmax, __ldcg(&part_lse[static_cast<size_t>(c_first + i + b) * HqNq + rowi]));
          const float msb = (mmax == -INFINITY) ? 0.f : mmax;
          float wsum = 0.f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          const bool col_live = lane * 4 < kD;            // head_dim 64: the first 16 lanes carry the row
          for (int i = 0; i < n_parts; ++i) {
            const size_t sl = static_cast<size_t>(c_first + i + b);
            const float w = exp2f(__ldcg(&part_lse[sl * HqNq + rowi]) - msb);
            wsum += w;
            if (!col_live) continue;
            const float4 v4 = __ldcg(reinterpret_cast<const float4*>(&part_o[(sl * HqNq + rowi) * kD + lane * 4]));
            acc.x = fmaf(w, v4.x, acc.x); acc.y = fmaf(w, v4.y, acc.y);
            acc.z = fmaf(w, v4.z, acc.z); acc.w = fmaf(w, v4.w, acc.w);
          }
          const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
          const size_t orow = (static_cast<size_t>(b) * p.Hq + hq) * p.Nq + qi;
          const size_t o = orow * kD + lane * 4;
          if (p.packed_f32) {
            float* pk = reinterpret_cast<float*>(p.out) + orow * (kD + 4);
            if (col_live) *reinterpret_cast<float4*>(pk + lane * 4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
            if (lane == 0) pk[kD] = wsum > 0.f ? mmax + log2f(wsum) : -INFINITY;
          } else if (!col_live) {
          } else if (p.q_dtype == 0) {
            __half2 h0 = __floats2half2_rn(acc.x * inv, acc.y * inv), h1 = __floats2half2_rn(acc.z * inv, acc.w * inv);
            uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
            *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + o) = pk;
          } else {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), h1 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
            uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = pk;
          }
          if (!p.packed_f32 && p.lse != nullptr && lane == 0) p.lse[orow] = wsum > 0.f ? mmax + log2f(wsum) : -INFINITY;
        }
      }
      named_bar_sync(1, HPC * 32);   // s_last is reused by the next sequence
    }

    u = static_cast<long long>(s0) + j_hi;
    if (u >= s1) ++b;
  }
  if (!ok && lane == 0) atomicOr(err, 1);
}

// Combine of per-GPU partials: one warp per output row, lanes across the head dim.
__global__ void __launch_bounds__(256) combine_partials_kernel(const float* __restrict__ g, int R, long long rows, int D,
                                                               int out_dtype, void* __restrict__ out, float* __restrict__ lse) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int W = D + 4;
  float m = -INFINITY;
  for (int r = 0; r < R; ++r) m = fmaxf(m, g[(static_cast<long long>(r) * rows + row) * W + D]);
  const float ms = (m == -INFINITY) ? 0.f : m;
  float wsum = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool live = lane * 4 < D;
  for (int r = 0; r < R; ++r) {
    const float* src = g + (static_cast<long long>(r) * rows + row) * W;
    const float w = exp2f(src[D] - ms);
    wsum += w;
    if (live) {
      const float4 v = *reinterpret_cast<const float4*>(src + lane * 4);
      acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  if (live) {
    const long long o = row * D + lane * 4;
    uint2 pk;
    if (out_dtype == 0) {
      pk = make_uint2(pack_h2(acc.x * inv, acc.y * inv), pack_h2(acc.z * inv, acc.w * inv));
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + o) = pk;
    } else {
      pk = make_uint2(pack_bf2(acc.x * inv, acc.y * inv), pack_bf2(acc.z * inv, acc.w * inv));
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + o) = pk;
    }
  }
  if (lse != nullptr && lane == 0) lse[row] = wsum > 0.f ? m + log2f(wsum) : -INFINITY;
}

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int pick_hpc(int Hkv) {
  if (Hkv % 8 == 0) return 8;
  if (Hkv % 4 == 0) return 4;
  if (Hkv % 2 == 0) return 2;
  return 1;
}

int pick_grid_x(int Hkv, int num_splits) {
  const int hpc = pick_hpc(Hkv);
  const int hg = Hkv / hpc;
  int target = device_sm_count() * (8 / hpc);     // CTAs in flight over the whole grid
  int gx = (target + hg - 1) / hg;
  if (gx < 1) gx = 1;
  if (num_splits > 0 && gx > num_splits) gx = num_splits;
  return gx;
}

template <int KV, int HPC, int D>
cudaError_t launch_t(const CUtensorMap& tmK, const CUtensorMap& tmV, const KernelArgs& a, int gx, size_t smem,
                     cudaStream_t stream) {
  dim3 grid(gx, a.HG);
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    kern<<<grid, (HPC + 1) * 32, smem, stream>>>(tmK, tmV, a);
    return cudaGetLastError();
  };
  return a.inv_cap > 0.f ? go(decode_paged_kernel<KV, HPC, D, true>) : go(decode_paged_kernel<KV, HPC, D, false>);
}

template <int KV, int D>
cudaError_t launch_kv(int hpc, const CUtensorMap& tmK, const CUtensorMap& tmV, const KernelArgs& a, int gx,
                      size_t smem, cudaStream_t stream) {
  switch (hpc) {
    case 8: return launch_t<KV, 8, D>(tmK, tmV, a, gx, smem, stream);
    case 4: return launch_t<KV, 4, D>(tmK, tmV, a, gx, smem, stream);
    case 2: return launch_t<KV, 2, D>(tmK, tmV, a, gx, smem, stream);
    default: return launch_t<KV, 1, D>(tmK, tmV, a, gx, smem, stream);
  }
}

}  // namespace

cudaError_t launch_combine_partials(const float* gathered, int R, long long rows, int D, int out_dtype, void* out,
                                    float* lse, cudaStream_t stream) {
  if (R <= 0 || rows <= 0) return cudaSuccess;
  const long long blocks = (rows * 32 + 255) / 256;
  combine_partials_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(gathered, R, rows, D, out_dtype, out, lse);
  return cudaGetLastError();
}

size_t decode_workspace_bytes(int B, int Hq, int Hkv, int Nq, int D, int max_kv_len, int num_splits) {
  (void)max_kv_len;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Nq <= 0) return 16;
  const int hpc = pick_hpc(Hkv);
  return make_layout(B, Hq, Nq, Hkv / hpc, pick_grid_x(Hkv, num_splits), D).total;
}

cudaError_t launch_decode_paged(const DecodeParams& p, cudaStream_t stream, char* msg, size_t msg_len) {
  const bool quant = p.kv_dtype == 3 || p.kv_dtype == 4;
  const int hpc = pick_hpc(p.Hkv);
  const int HG = p.Hkv / hpc;
  const int gx = pick_grid_x(p.Hkv, p.num_splits);
  const int kD = p.D;
  const int row_bytes = quant ? kD : 2 * kD;
  if (!(kD == 128 || (kD == 64 && !quant))) {
    snprintf(msg, msg_len, "head_dim %d with kv_dtype %d (built: 128 for every pool type, 64 for 16-bit pools)", kD, p.kv_dtype);
    return cudaErrorNotSupported;
  }
  if (!p.dense && (p.block_size < kBS || p.block_size % kBS != 0)) {
    snprintf(msg, msg_len, "block_size %d: pages must hold a multiple of %d tokens", p.block_size, kBS);
    return cudaErrorNotSupported;
  }

  KernelArgs a;
  a.p = p;
  a.upp = p.dense ? 1 : p.block_size / kBS;
  a.lay = make_layout(p.B, p.Hq, p.Nq, HG, gx, kD);
  a.HG = HG;
  a.group = p.Hq / p.Hkv;
  a.rows = a.group * p.Nq;
  a.stage_kv_bytes = hpc * kBS * row_bytes;
  a.scale_bytes = quant ? kBS * p.Hkv * 2 : 0;
  const size_t per_stage = 2 * static_cast<size_t>(a.stage_kv_bytes) + 2 * static_cast<size_t>(a.scale_bytes);
  // several small CTAs share an SM when a CTA holds few heads
  const size_t budget = hpc == 8 ? 200 * 1024 : (hpc == 4 ? 100 * 1024 : (hpc == 2 ? 50 * 1024 : 26 * 1024));
  int stages = static_cast<int>(budget / per_stage);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) {
    snprintf(msg, msg_len, "Hkv=%d needs %zu bytes per stage; too large for the stage ring", p.Hkv, per_stage);
    return cudaErrorNotSupported;
  }
  a.stages = stages;
  const float sc = p.softcap > 0.f ? p.scale : p.scale * kLog2e;
  a.q_prescale = sc;
  a.cap_log2 = p.softcap * kLog2e;
  a.inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  const size_t smem = 1024 + static_cast<size_t>(stages) * per_stage + 2 * kMaxStages * 8 + kMaxStages * 4 + 64;

  // tensor maps, in bytes: (128 B, tokens, 128-byte halves of a row, heads, batch).  A pool is one "batch" of
  // num_pages * block_size tokens with the heads of a token side by side; a dense cache has its own strides.
  CUtensorMap tmK, tmV;
  const uint32_t box[5] = {128, kBS, static_cast<uint32_t>(row_bytes / 128), static_cast<uint32_t>(hpc), 1};
  bool maps_ok;
  if (p.dense) {
    const uint64_t dims[5] = {128, static_cast<uint64_t>(p.max_kv_len), static_cast<uint64_t>(row_bytes / 128),
                              static_cast<uint64_t>(p.Hkv), static_cast<uint64_t>(p.B)};
    auto strides_of = [&](int64_t bs, int64_t hs, int64_t rs, uint64_t (&st)[4]) {
      // a size-1 dimension still needs a legal stride
      const uint64_t row = static_cast<uint64_t>(rs) * 2;
      const uint64_t head = hs > 0 ? static_cast<uint64_t>(hs) * 2 : row * p.max_kv_len;
      st[0] = row; st[1] = 128; st[2] = head;
      st[3] = bs > 0 ? static_cast<uint64_t>(bs) * 2 : head * p.Hkv;
    };
    uint64_t ks[4], vs[4];
    strides_of(p.k_bs, p.k_hs, p.k_rs, ks);
    strides_of(p.v_bs, p.v_hs, p.v_rs, vs);
    maps_ok = encode_tmap(&tmK, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, p.k_pool, dims, ks, box, CU_TENSOR_MAP_SWIZZLE_128B) &&
              encode_tmap(&tmV, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, p.v_pool, dims, vs, box, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    const uint64_t tokens = static_cast<uint64_t>(p.num_pages) * p.block_size;
    const uint64_t dims[5] = {128, tokens, static_cast<uint64_t>(row_bytes / 128), static_cast<uint64_t>(p.Hkv), 1};
    const uint64_t strides[4] = {static_cast<uint64_t>(p.Hkv) * row_bytes, 128, static_cast<uint64_t>(row_bytes),
                                 tokens * p.Hkv * row_bytes};
    maps_ok = encode_tmap(&tmK, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, p.k_pool, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) &&
              encode_tmap(&tmV, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, p.v_pool, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (!maps_ok) {
    snprintf(msg, msg_len, "cuTensorMapEncodeTiled failed for the K / V tensors");
    return cudaErrorInvalidValue;
  }

  unsigned char* ws = reinterpret_cast<unsigned char*>(p.workspace);
  decode_plan_kernel<<<1, 1024, 0, stream>>>(p.seq_lens, p.B, p.max_kv_len, p.B * HG,
                                             reinterpret_cast<int*>(ws + a.lay.err),
                                             reinterpret_cast<int*>(ws + a.lay.counters),
                                             reinterpret_cast<int*>(ws + a.lay.page_start));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  switch (p.kv_dtype) {
    case 0: return kD == 64 ? launch_kv<KV_F16, 64>(hpc, tmK, tmV, a, gx, smem, stream)
                            : launch_kv<KV_F16, 128>(hpc, tmK, tmV, a, gx, smem, stream);
    case 1: return kD == 64 ? launch_kv<KV_BF16, 64>(hpc, tmK, tmV, a, gx, smem, stream)
                            : launch_kv<KV_BF16, 128>(hpc, tmK, tmV, a, gx, smem, stream);
    case 3: return launch_kv<KV_I8, 128>(hpc, tmK, tmV, a, gx, smem, stream);
    case 4: return launch_kv<KV_E4M3, 128>(hpc, tmK, tmV, a, gx, smem, stream);
    default: snprintf(msg, msg_len, "kv_dtype %d", p.kv_dtype); return cudaErrorNotSupported;
  }
}

}  // namespace b200fa

// ---------------------------------------------------------------------------
// Decode without a caller-supplied workspace
// ---------------------------------------------------------------------------
// Scratch for b200fa_decode_paged_static: the same carve-up the workspace variant
// uses (error word, per-sequence counters, page prefix sums, split partials), held in
// a fixed array that every GPU loading this library keeps until the process exits.
#define B200FA_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
static __device__ __align__(256) unsigned char g_decode_static_scratch[B200FA_STATIC_SCRATCH_BYTES];

namespace b200fa {
void set_last_error(const char* msg);

namespace {
// In host code the array's name is only a handle; the device address has to be asked
// for, once per device, while that device is current.
cudaError_t static_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess) return e;
    addr[dev] = p;
  }
  *out = addr[dev];
  return cudaSuccess;
}
}  // namespace
}  // namespace b200fa

extern "C" int32_t b200fa_decode_paged_static(const b200fa_desc* d, const void* q, const void* k_pool,
                                              const void* v_pool, const void* k_scale, const void* v_scale,
                                              const int32_t* block_table, const int32_t* seq_lens,
                                              int32_t num_pages, int32_t block_size, int32_t max_blocks,
                                              int32_t max_kv_len, void* out, float* lse, void* stream) {
  if (d == nullptr) {
    b200fa::set_last_error("descriptor is null");
    return B200FA_ERR_INVALID_ARG;
  }
  const size_t need = b200fa_decode_paged_workspace_bytes(d, max_kv_len);
  if (need > B200FA_STATIC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "b200fa_decode_paged_static: this problem needs %zu bytes of scratch, the built-in scratch holds %u; "
             "use b200fa_decode_paged with a workspace, or lower B / Hq*N",
             need, B200FA_STATIC_SCRATCH_BYTES);
    b200fa::set_last_error(msg);
    return B200FA_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  cudaError_t e = b200fa::static_scratch_address(&scratch);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "b200fa_decode_paged_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    b200fa::set_last_error(msg);
    return B200FA_ERR_CUDA;
  }
  // Same validation, planning and kernels as the workspace variant; the plan kernel
  // clears the counters and the error word at the start of every call.
  return b200fa_decode_paged(d, q, k_pool, v_pool, k_scale, v_scale, block_table, seq_lens, num_pages,
                             block_size, max_blocks, max_kv_len, out, lse, scratch,
                             B200FA_STATIC_SCRATCH_BYTES, stream);
}

// The static entry's error word sits at the start of the built-in scratch, whose address callers never see.
extern "C" int32_t b200fa_decode_paged_static_status(void* stream, int32_t* status_out) {
  if (status_out == nullptr) {
    b200fa::set_last_error("status_out is null");
    return B200FA_ERR_INVALID_ARG;
  }
  void* scratch = nullptr;
  cudaError_t e = b200fa::static_scratch_address(&scratch);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "b200fa_decode_paged_static_status: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    b200fa::set_last_error(msg);
    return B200FA_ERR_CUDA;
  }
  return b200fa_workspace_status(scratch, stream, status_out);
}
