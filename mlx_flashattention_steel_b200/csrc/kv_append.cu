// KV-cache write path: scatters new key / value tokens into the page pools, quantising on the way when the
// pool is 8-bit.  It does on the device, in one launch for any number of sequences, what the reference's
// PagedKVCache.append does block by block with array concatenations (mlx_mfa/attention.py:2642-2711), and it
// is the producer of the int8 / fp8 pool format the decode kernel reads.
//
// One warp per (token, kv head) row of D values, K and V in the same launch (blockIdx.y).  A row is 128 or 256
// bytes in and 64 to 256 bytes out, every access a full-warp contiguous segment: the kernel is bound by HBM
// (about 3 bytes moved per stored int8 value, 4 per 16-bit value).
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

// SRC: 0 f16, 1 bf16.  POOL: 0 f16, 1 bf16, 3 int8, 4 e4m3 (the library's dtype codes).  EPL: elements per lane (D / 32).
template <typename SrcT, int POOL, int EPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
kv_append_kernel(const SrcT* __restrict__ k_new, const SrcT* __restrict__ v_new, int64_t token_stride, int64_t head_stride,
                 const int64_t* __restrict__ slots, void* __restrict__ k_pool, void* __restrict__ v_pool,
                 __half* __restrict__ k_scale, __half* __restrict__ v_scale, int T, int Hkv, int64_t total_slots) {
  constexpr int D = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int64_t rowid = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (rowid >= static_cast<int64_t>(T) * Hkv) return;
  const int t = static_cast<int>(rowid / Hkv), h = static_cast<int>(rowid % Hkv);
  const int64_t slot = slots[t];
  if (slot < 0 || slot >= total_slots) return;          // padding entry (or a slot outside the pool): nothing is written
  const bool is_v = blockIdx.y != 0;
  const SrcT* src = (is_v ? v_new : k_new) + t * token_stride + h * head_stride + lane * EPL;
  // one 8-byte (D = 128) or 4-byte (D = 64) load per lane: the warp reads the row as one contiguous segment
  uint32_t raw[EPL / 2];
  if (EPL == 4) {
    const uint2 v = *reinterpret_cast<const uint2*>(src);
    raw[0] = v.x;
    raw[EPL / 2 - 1] = v.y;
  } else {
    raw[0] = *reinterpret_cast<const uint32_t*>(src);
  }
  float x[EPL];
#pragma unroll
  for (int i = 0; i < EPL / 2; ++i) {
    const float2 f = Elem<SrcT>::unpack(raw[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
  const int64_t dst_row = slot * Hkv + h;               // pools are [page, offset, head, D]: row index = slot * Hkv + h
  void* pool = is_v ? v_pool : k_pool;

  if (POOL == 0 || POOL == 1) {
    // 16-bit pool: copy (same type) or convert through float
    uint16_t outv[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      if (POOL == 0) { const __half hv = __float2half_rn(x[i]); outv[i] = *reinterpret_cast<const uint16_t*>(&hv); }
      else { const __nv_bfloat16 bv = __float2bfloat16_rn(x[i]); outv[i] = *reinterpret_cast<const uint16_t*>(&bv); }
    }
    uint16_t* dst = reinterpret_cast<uint16_t*>(pool) + dst_row * D + lane * EPL;
    if (EPL == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(outv[0] | (static_cast<uint32_t>(outv[1]) << 16), outv[2] | (static_cast<uint32_t>(outv[3 % EPL]) << 16));
    else *reinterpret_cast<uint32_t*>(dst) = outv[0] | (static_cast<uint32_t>(outv[1]) << 16);
    return;
  }

  // 8-bit pool: row max, scale, quantise
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float qmax = POOL == 3 ? 127.f : 448.f;
  __half sc = __float2half_rn(__fdiv_rn(amax, qmax));
  if (__half2float(sc) == 0.f) sc = __float2half_rn(1.f);
  const float scf = __half2float(sc);
  uint8_t q[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const float y = __fdiv_rn(x[i], scf);
    if (POOL == 3) {
      q[i] = static_cast<uint8_t>(static_cast<int8_t>(max(-127, min(127, __float2int_rn(y)))));
    } else {
      q[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(fminf(fmaxf(y, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3));
    }
  }
  uint8_t* dst = reinterpret_cast<uint8_t*>(pool) + dst_row * D + lane * EPL;
  if (EPL == 4) *reinterpret_cast<uint32_t*>(dst) = q[0] | (q[1] << 8) | (q[2 % EPL] << 16) | (static_cast<uint32_t>(q[3 % EPL]) << 24);
  else *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(q[0] | (q[1] << 8));
  if (lane == 0) (is_v ? v_scale : k_scale)[dst_row] = sc;
}

template <typename SrcT, int POOL>
cudaError_t launch_d(int D, const void* k_new, const void* v_new, int64_t ts, int64_t hs, const int64_t* slots, void* k_pool,
                     void* v_pool, void* k_scale, void* v_scale, int T, int Hkv, int64_t total_slots, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(T) * Hkv;
  dim3 grid(static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock), 2);
  if (D == 128)
    kv_append_kernel<SrcT, POOL, 4><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        static_cast<const SrcT*>(k_new), static_cast<const SrcT*>(v_new), ts, hs, slots, k_pool, v_pool,
        static_cast<__half*>(k_scale), static_cast<__half*>(v_scale), T, Hkv, total_slots);
  else
    kv_append_kernel<SrcT, POOL, 2><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
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
