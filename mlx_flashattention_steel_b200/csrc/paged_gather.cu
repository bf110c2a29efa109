// Page gather: pool [num_pages, block_size, H, D] -> out [B, H, max_kv_len, D].
// out[b,h,t,:] = pool[block_table[b, t / block_size], t % block_size, h, :] when
// t < seq_lens[b] and the table entry is non-negative, else zero.  A bit-exact
// copy with 64-bit offsets; same contract as the reference's paged_kv_gather
// (csrc/mfa_paged_gather.cpp:44-80 kernel, 89-129 CPU loop).
#include <cuda_fp8.h>

#include "common.cuh"
#include "launch.h"

namespace b200fa {

namespace {

// I: index type of the flattened chunk space (32-bit whenever it fits: the index is split by run-time divisors per chunk)
template <typename I>
__global__ void __launch_bounds__(256) paged_kv_gather_kernel(
    const uint4* __restrict__ pool, const int32_t* __restrict__ block_table,
    const int32_t* __restrict__ seq_lens, int H, int chunks_per_row /* D*elem_bytes/16 */,
    int block_size, int max_blocks, int max_kv_len, long long total_chunks, uint4* __restrict__ out) {
  const I stride = static_cast<I>(gridDim.x) * blockDim.x, total = static_cast<I>(total_chunks);
  for (I idx = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    // idx = ((b*H + h)*max_kv_len + t)*chunks_per_row + c
    const int c = static_cast<int>(idx % static_cast<I>(chunks_per_row));
    I rem = idx / static_cast<I>(chunks_per_row);
    const int t = static_cast<int>(rem % static_cast<I>(max_kv_len));
    rem /= static_cast<I>(max_kv_len);
    const int h = static_cast<int>(rem % static_cast<I>(H));
    const int b = static_cast<int>(rem / static_cast<I>(H));
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (t < seq_lens[b]) {
      const int page = block_table[static_cast<long long>(b) * max_blocks + t / block_size];
      if (page >= 0) {
        const long long src =
            ((static_cast<long long>(page) * block_size + (t % block_size)) * H + h) * chunks_per_row + c;
        val = pool[src];
      }
    }
    out[idx] = val;
  }
}

// Gather + dequantise: one thread per 16 pool bytes (16 values of one (token, head) row), written as 32 bytes of the
// 16-bit output.  value = T(float(x) * float(scale)): one rounding, to the output type, as the host definition has it.
template <typename T, bool E4M3>
__global__ void __launch_bounds__(256) paged_kv_gather_dequant_kernel(
    const uint4* __restrict__ pool, const __half* __restrict__ scale, const int32_t* __restrict__ block_table,
    const int32_t* __restrict__ seq_lens, int H, int chunks_per_row /* D / 16 */, int block_size, int max_blocks,
    int max_kv_len, long long total_chunks, uint4* __restrict__ out) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_chunks; idx += stride) {
    const int c = static_cast<int>(idx % chunks_per_row);
    long long rem = idx / chunks_per_row;
    const int t = static_cast<int>(rem % max_kv_len);
    rem /= max_kv_len;
    const int h = static_cast<int>(rem % H);
    const int b = static_cast<int>(rem / H);
    uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
    if (t < seq_lens[b]) {
      const int page = block_table[static_cast<long long>(b) * max_blocks + t / block_size];
      if (page >= 0) {
        const long long rowi = (static_cast<long long>(page) * block_size + (t % block_size)) * H + h;
        const uint4 raw = pool[rowi * chunks_per_row + c];
        const float sc = __half2float(scale[rowi]);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t byte = (w[i] >> (8 * e)) & 0xffu;
            if (E4M3) {
              const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
              f[e] = __half2float(__half(hr));
            } else {
              f[e] = static_cast<float>(static_cast<int>(static_cast<signed char>(byte)));
            }
          }
          o[2 * i] = Elem<T>::pack(f[0] * sc, f[1] * sc);
          o[2 * i + 1] = Elem<T>::pack(f[2] * sc, f[3] * sc);
        }
        lo = make_uint4(o[0], o[1], o[2], o[3]);
        hi = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
    out[2 * idx] = lo;
    out[2 * idx + 1] = hi;
  }
}

// The transpose of the gather, for gradients: grad_pool[page, t % bs, h, :] += grad[b, h, t, :] for t < seq_lens[b]
// and a non-negative table entry (the role of _scatter_to_pool, mlx_mfa/attention.py:2878-2940).  The pool-shaped
// output must start at zero; a page listed by several sequences (a shared prefix) accumulates all of them, which is
// why the adds are packed 16-bit atomics rather than stores.
template <typename T2>
__global__ void __launch_bounds__(256) paged_kv_scatter_add_kernel(
    const uint4* __restrict__ grad, const int32_t* __restrict__ block_table, const int32_t* __restrict__ seq_lens, int H,
    int chunks_per_row, int block_size, int max_blocks, int max_kv_len, long long total_chunks, T2* __restrict__ grad_pool) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_chunks; idx += stride) {
    const int c = static_cast<int>(idx % chunks_per_row);
    long long rem = idx / chunks_per_row;
    const int t = static_cast<int>(rem % max_kv_len);
    rem /= max_kv_len;
    const int h = static_cast<int>(rem % H);
    const int b = static_cast<int>(rem / H);
    if (t >= seq_lens[b]) continue;
    const int page = block_table[static_cast<long long>(b) * max_blocks + t / block_size];
    if (page < 0) continue;
    const uint4 v = grad[idx];
    const long long dst = (((static_cast<long long>(page) * block_size + (t % block_size)) * H + h) * chunks_per_row + c) * 4;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) atomicAdd(grad_pool + dst + i, *reinterpret_cast<const T2*>(&w[i]));
  }
}

}  // namespace

cudaError_t launch_paged_scatter_add(const void* grad, const int32_t* block_table, const int32_t* seq_lens, int B, int H,
                                     int D, int dtype, int block_size, int max_blocks, int max_kv_len, void* grad_pool,
                                     cudaStream_t stream) {
  const int cpr = D * 2 / 16;
  const long long total = static_cast<long long>(B) * H * max_kv_len * cpr;
  if (total == 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  const long long cap = 148LL * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == 0)
    paged_kv_scatter_add_kernel<__half2><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(grad), block_table, seq_lens, H, cpr, block_size, max_blocks, max_kv_len, total,
        reinterpret_cast<__half2*>(grad_pool));
  else
    paged_kv_scatter_add_kernel<__nv_bfloat162><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(grad), block_table, seq_lens, H, cpr, block_size, max_blocks, max_kv_len, total,
        reinterpret_cast<__nv_bfloat162*>(grad_pool));
  return cudaGetLastError();
}

cudaError_t launch_paged_gather_dequant(const void* pool, const void* scale, const int32_t* block_table,
                                        const int32_t* seq_lens, int B, int H, int D, int pool_dtype, int out_dtype,
                                        int block_size, int max_blocks, int max_kv_len, void* out, cudaStream_t stream) {
  const int cpr = D / 16;
  const long long total = static_cast<long long>(B) * H * max_kv_len * cpr;
  if (total == 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  const long long cap = 148LL * 32;
  if (blocks > cap) blocks = cap;
  const unsigned g = static_cast<unsigned>(blocks);
  const uint4* pl = reinterpret_cast<const uint4*>(pool);
  const __half* sc = reinterpret_cast<const __half*>(scale);
  uint4* o = reinterpret_cast<uint4*>(out);
  const bool e4 = pool_dtype == 4;
  if (out_dtype == 0) {
    if (e4) paged_kv_gather_dequant_kernel<__half, true><<<g, 256, 0, stream>>>(pl, sc, block_table, seq_lens, H, cpr, block_size, max_blocks, max_kv_len, total, o);
    else paged_kv_gather_dequant_kernel<__half, false><<<g, 256, 0, stream>>>(pl, sc, block_table, seq_lens, H, cpr, block_size, max_blocks, max_kv_len, total, o);
  } else {
    if (e4) paged_kv_gather_dequant_kernel<__nv_bfloat16, true><<<g, 256, 0, stream>>>(pl, sc, block_table, seq_lens, H, cpr, block_size, max_blocks, max_kv_len, total, o);
    else paged_kv_gather_dequant_kernel<__nv_bfloat16, false><<<g, 256, 0, stream>>>(pl, sc, block_table, seq_lens, H, cpr, block_size, max_blocks, max_kv_len, total, o);
  }
  return cudaGetLastError();
}

cudaError_t launch_paged_gather(const void* pool, const int32_t* block_table, const int32_t* seq_lens,
                                int B, int H, int D, int elem_bytes, int block_size, int max_blocks,
                                int max_kv_len, void* out, cudaStream_t stream) {
  const int cpr = D * elem_bytes / 16;
  const long long total = static_cast<long long>(B) * H * max_kv_len * cpr;
  if (total == 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  const long long cap = 148LL * 32;
  if (blocks > cap) blocks = cap;
  if (total < (1LL << 31))
    paged_kv_gather_kernel<uint32_t><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(pool), block_table, seq_lens, H, cpr, block_size, max_blocks,
        max_kv_len, total, reinterpret_cast<uint4*>(out));
  else
    paged_kv_gather_kernel<long long><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(pool), block_table, seq_lens, H, cpr, block_size, max_blocks,
        max_kv_len, total, reinterpret_cast<uint4*>(out));
  return cudaGetLastError();
}

}  // namespace b200fa
