// KV-cache write path: scatters new key / value tokens into the page pools, quantising on the way when the
// pool is 8-bit.  It does on the device, in one launch for any number of sequences, what the reference's
// PagedKVCache.append does block by block with array concatenations (mlx_mfa/attention.py:2642-2711), and it
// is the producer of the int8 / fp8 pool format the decode kernel reads.
//
// A (token, kv head) row of D values is handled by D/8 lanes (16-byte loads), K and V in the same launch
// (blockIdx.y); warps walk the rows with a grid stride.  A row is 128 or 256 bytes in and 64 to 256 bytes out,
// every access a contiguous segment: the kernel is bound by HBM (about 3 bytes moved per stored int8 value,
// 4 per 16-bit value).
//
// 8-bit pools (one symmetric group spanning D, zero bias):
//   scale = f16(max|x| / qmax)  (1 if that is zero),  q = round_to_nearest_even(x / float(scale)),
//   int8: qmax 127, clamped to [-127, 127];  e4m3: qmax 448, clamped, then rounded to e4m3.
// Division and roundings are IEEE, so the bytes match a float32 host computation exactly.
#include <cuda_fp8.h>

#include "common.cuh"
#include "launch.h"

namespace b200fa {

namespace {

constexpr int kWarpsPerBlock = 8;

// SrcT: __half or __nv_bfloat16.  POOL: 0 f16, 1 bf16, 3 int8, 4 e4m3 (the library's dtype codes).
// Each lane moves 8 values (one 16-byte load), so a row takes D/8 lanes and a warp handles 32/(D/8) rows per step;
// warps walk the rows with a grid stride, three steps in flight, from a grid of a few CTAs per SM.
template <typename SrcT, int POOL, int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
kv_append_kernel(const SrcT* __restrict__ k_new, const SrcT* __restrict__ v_new, int64_t token_stride, int64_t head_stride,
                 const int64_t* __restrict__ slots, void* __restrict__ k_pool, void* __restrict__ v_pool,
                 __half* __restrict__ k_scale, __half* __restrict__ v_scale, int T, int Hkv, int64_t total_slots) {
  // values per lane: 8 (one 16-byte load) for 16-bit pools, 16 for 8-bit pools, whose per-row work (row maximum over
  // the lanes, scale, reciprocal) and per-lane overhead then spread over twice the values and whose stores are 16 bytes
  constexpr int VPL = (POOL >= 3) ? 16 : 8;
  constexpr int LPR = D / VPL;           // lanes per row
  constexpr int RPW = 32 / LPR;          // rows per warp step
  const int lane = threadIdx.x & 31, sub = lane / LPR, l = lane % LPR;
  const bool is_v = blockIdx.y != 0;
  const SrcT* new_base = is_v ? v_new : k_new;
  void* pool = is_v ? v_pool : k_pool;
  __half* scale_out = is_v ? v_scale : k_scale;
  const int64_t rows = static_cast<int64_t>(T) * Hkv;
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;

  // one row per lane group; the rows of the next two steps are fetched before the current one is quantised and
  // stored.  The values are loaded whether or not the slot turns out to be writable: the source row exists for every
  // token, and a load that waited for the slot would put two memory latencies in series.
  struct Row {
    uint4 raw[VPL / 8];
    int64_t slot;
    int h;
    bool write;
  };
  // (token, head) of the row this lane group fetches next: advanced by one grid stride per fetch, so that the 64-bit
  // division happens once per thread and not once per row
  const int64_t step = n_warps * RPW;
  const int64_t first = warp_id * RPW + sub;
  const int step_t = static_cast<int>(step / Hkv), step_h = static_cast<int>(step % Hkv);
  int64_t f_row = first;
  int f_t = static_cast<int>(first / Hkv), f_h = static_cast<int>(first % Hkv);
  auto fetch = [&]() -> Row {
    Row r;
#pragma unroll
    for (int j = 0; j < VPL / 8; ++j) r.raw[j] = make_uint4(0u, 0u, 0u, 0u);
    r.slot = -1;
    r.h = f_h;
    const int t = f_t;
    if (f_row < rows) {
      r.slot = __ldg(slots + t);
#pragma unroll
      for (int j = 0; j < VPL / 8; ++j)
        r.raw[j] = __ldg(reinterpret_cast<const uint4*>(new_base + t * token_stride + r.h * head_stride + l * VPL + j * 8));
    }
    r.write = r.slot >= 0 && r.slot < total_slots;      // padding entries and slots outside the pool write nothing
    f_row += step;
    f_t += step_t;
    f_h += step_h;
    if (f_h >= Hkv) {
      f_h -= Hkv;
      ++f_t;
    }
    return r;
  };

  Row nxt = fetch(), nxt2 = fetch();                    // fetch() of a row past the end loads nothing
  for (int64_t r0 = warp_id * RPW; r0 < rows; r0 += step) {
    const Row cur = nxt;
    nxt = nxt2;
    nxt2 = fetch();
    const int64_t slot = cur.slot;
    const int h = cur.h;
    const bool write = cur.write;
    float x[VPL];
#pragma unroll
    for (int j = 0; j < VPL / 8; ++j) {
      const uint32_t w[4] = {cur.raw[j].x, cur.raw[j].y, cur.raw[j].z, cur.raw[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = Elem<SrcT>::unpack(w[i]);
        x[8 * j + 2 * i] = f.x;
        x[8 * j + 2 * i + 1] = f.y;
      }
    }
    const int64_t dst_row = slot * Hkv + h;             // pools are [page, offset, head, D]: row index = slot * Hkv + h

    if (POOL == 0 || POOL == 1) {
      // 16-bit pool: the same bits, or a conversion through float when the types differ
      uint4 o;
      if (POOL == 0) o = make_uint4(Elem<__half>::pack(x[0], x[1]), Elem<__half>::pack(x[2], x[3]), Elem<__half>::pack(x[4], x[5]), Elem<__half>::pack(x[6], x[7]));
      else o = make_uint4(Elem<__nv_bfloat16>::pack(x[0], x[1]), Elem<__nv_bfloat16>::pack(x[2], x[3]), Elem<__nv_bfloat16>::pack(x[4], x[5]), Elem<__nv_bfloat16>::pack(x[6], x[7]));
      if (write) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(pool) + dst_row * D + l * 8) = o;
      continue;
    }

    // 8-bit pool: row max over the row's lanes, scale, quantise
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // Correctly rounded quotients without the division routine: with r = rn(1/b), q0 = rn(a*r), the residual
    // e = a - b*q0 is exact in one fma and rn(q0 + e*r) is the IEEE quotient (the final step of a Newton division).
    auto div_rn = [](float a, float b, float rb) -> float {
      const float q0 = a * rb;
      return fmaf(fmaf(-q0, b, a), rb, q0);
    };
    const float qmax = POOL == 3 ? 127.f : 448.f;
    __half sc = __float2half_rn(div_rn(amax, qmax, __frcp_rn(qmax)));
    if (__half2float(sc) == 0.f) sc = __float2half_rn(1.f);
    const float scf = __half2float(sc);
    const float rcp = __frcp_rn(scf);
    uint32_t packed[VPL / 4];
    if (POOL == 3) {
      // the same Newton step on value pairs (packed f32x2 ops), round to nearest even, clamp to [-127, 127]
      // (saturating pack covers the top, one max the bottom), four values per pack pair
      const float2 rb2 = make_float2(rcp, rcp), nb2 = make_float2(-scf, -scf);
      int qi[VPL];
#pragma unroll
      for (int i = 0; i < VPL; i += 2) {
        const float2 a = make_float2(x[i], x[i + 1]);
        const float2 q0 = __fmul2_rn(a, rb2);
        const float2 y = __ffma2_rn(__ffma2_rn(q0, nb2, a), rb2, q0);
        // round to nearest even without the conversion unit: adding 1.5 * 2^23 leaves the integer in the low mantissa
        // bits (exact for |y| < 2^22; y is at most 127.5 here and is clamped from below first)
        const float2 r = __fadd2_rn(make_float2(fmaxf(y.x, -127.f), fmaxf(y.y, -127.f)), make_float2(12582912.f, 12582912.f));
        qi[i] = __float_as_int(r.x) - 0x4B400000;
        qi[i + 1] = __float_as_int(r.y) - 0x4B400000;
      }
#pragma unroll
      for (int w = 0; w < VPL / 4; ++w) {
        // cvt.pack d, a, b, c = (c << 16) | (sat8(a) << 8) | sat8(b): the upper pair first, then the lower pair on top
        uint32_t hi;
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(qi[4 * w + 3]), "r"(qi[4 * w + 2]), "r"(0));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(packed[w]) : "r"(qi[4 * w + 1]), "r"(qi[4 * w]), "r"(hi));
      }
    } else {
      uint32_t q[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const float y = div_rn(x[i], scf, rcp);
        q[i] = static_cast<uint32_t>(__nv_cvt_float_to_fp8(fminf(fmaxf(y, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3));
      }
#pragma unroll
      for (int w = 0; w < VPL / 4; ++w) packed[w] = q[4 * w] | (q[4 * w + 1] << 8) | (q[4 * w + 2] << 16) | (q[4 * w + 3] << 24);
    }
    if (write) {
      if constexpr (VPL == 16) {
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pool) + dst_row * D + l * 16) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      } else {
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(pool) + dst_row * D + l * 8) = make_uint2(packed[0], packed[1]);
      }
      if (l == 0) scale_out[dst_row] = sc;
    }
  }
}

template <typename SrcT, int POOL>
cudaError_t launch_d(int D, const void* k_new, const void* v_new, int64_t ts, int64_t hs, const int64_t* slots, void* k_pool,
                     void* v_pool, void* k_scale, void* v_scale, int T, int Hkv, int64_t total_slots, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(T) * Hkv;
  const int rpw = 32 / (D / (POOL >= 3 ? 16 : 8));
  // enough CTAs to cover the rows once, capped at 8 per SM on each of K and V (148 SMs): the rest is the grid stride
  const int64_t want = (rows + static_cast<int64_t>(kWarpsPerBlock) * rpw - 1) / (static_cast<int64_t>(kWarpsPerBlock) * rpw);
  dim3 grid(static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8), 2);
  if (D == 128)
    kv_append_kernel<SrcT, POOL, 128><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const SrcT*>(k_new), static_cast<const SrcT*>(v_new), ts, hs, slots, k_pool, v_pool,
        static_cast<__half*>(k_scale), static_cast<__half*>(v_scale), T, Hkv, total_slots);
  else
    kv_append_kernel<SrcT, POOL, 64><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const SrcT*>(k_new), static_cast<const SrcT*>(v_new), ts, hs, slots, k_pool, v_pool,
        static_cast<__half*>(k_scale), static_cast<__half*>(v_scale), T, Hkv, total_slots);
  return cudaGetLastError();
}

template <typename SrcT>
cudaError_t launch_pool(int pool_dtype, int D, const void* k_new, const void* v_new, int64_t ts, int64_t hs, const int64_t* slots,
                        void* k_pool, void* v_pool, void* k_scale, void* v_scale, int T, int Hkv, int64_t total_slots,
                        cudaStream_t stream) {
  switch (pool_dtype) {
    case 0: return launch_d<SrcT, 0>(D, k_new, v_new, ts, hs, slots, k_pool, v_pool, k_scale, v_scale, T, Hkv, total_slots, stream);
    case 1: return launch_d<SrcT, 1>(D, k_new, v_new, ts, hs, slots, k_pool, v_pool, k_scale, v_scale, T, Hkv, total_slots, stream);
    case 3: return launch_d<SrcT, 3>(D, k_new, v_new, ts, hs, slots, k_pool, v_pool, k_scale, v_scale, T, Hkv, total_slots, stream);
    case 4: return launch_d<SrcT, 4>(D, k_new, v_new, ts, hs, slots, k_pool, v_pool, k_scale, v_scale, T, Hkv, total_slots, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_kv_append(int src_dtype, int pool_dtype, int D, const void* k_new, const void* v_new, int64_t token_stride,
                             int64_t head_stride, const int64_t* slots, void* k_pool, void* v_pool, void* k_scale,
                             void* v_scale, int T, int Hkv, int64_t total_slots, cudaStream_t stream) {
  if (T <= 0 || Hkv <= 0) return cudaSuccess;
  if (src_dtype == 0)
    return launch_pool<__half>(pool_dtype, D, k_new, v_new, token_stride, head_stride, slots, k_pool, v_pool, k_scale, v_scale, T,
                               Hkv, total_slots, stream);
  return launch_pool<__nv_bfloat16>(pool_dtype, D, k_new, v_new, token_stride, head_stride, slots, k_pool, v_pool, k_scale,
                                    v_scale, T, Hkv, total_slots, stream);
}

}  // namespace b200fa
