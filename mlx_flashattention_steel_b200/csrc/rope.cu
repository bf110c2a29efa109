// Rotary position embedding as its own pass over Q or K ([B, H, N, D], 16-bit), in place or into a second
// tensor.  The reference rotates inside its Metal attention kernel (csrc/mfa_steel_fwd.cpp:704-734, 831-858) or
// with array ops (mlx_mfa/attention.py:2128-2210); here the rotation is a memory-bound pass of its own: at the
// prefill sizes this library is built for it moves < 100 MB against an attention that runs for milliseconds,
// and the attention kernels keep their TMA-fed operand path untouched.
//
//   interleaved (LLaMA):  pairs (2i, 2i+1);   split halves (GPT-NeoX): pairs (i, i + rot/2),  i < rot/2
//   out[a] = x[a]*cos[pos][i] - x[b]*sin[pos][i],   out[b] = x[a]*sin[pos][i] + x[b]*cos[pos][i]
//   pos = offset(batch) + row;  elements d >= rot pass through;  `inverse` flips the sign of sin (the transpose of
//   the rotation, which is what the backward pass applies to the gradients).
//
// One thread per 16-byte chunk (8 values); in split-half mode a thread owns a chunk of the first half and its
// partner chunk, so an in-place call never reads what another thread writes.  float32 arithmetic, one rounding.
#include "common.cuh"
#include "launch.h"

namespace b200fa {

namespace {

// I: index type of the flattened (batch, head, row, chunk) space: 32-bit whenever it fits, because the index is split by
// run-time divisors for every 16-byte chunk and a 64-bit division costs several times the rest of the work
template <typename T, typename I>
__global__ void __launch_bounds__(256)
rope_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ cosb, const float* __restrict__ sinb,
            const int* __restrict__ offsets, int offset, int B, int H, int N, int D, int rot, int interleaved, int inverse,
            int64_t x_bs, int64_t x_hs, int64_t x_rs, int64_t o_bs, int64_t o_hs, int64_t o_rs) {
  const int half = rot >> 1;
  // chunks a thread may own per row: all D/8 (interleaved); first-half chunks + pass-through chunks (split halves)
  const int rot_chunks = rot >> 3, half_chunks = half >> 3, tail_chunks = (D - rot) >> 3;
  const int per_row = interleaved ? (D >> 3) : (half_chunks + tail_chunks);
  const I total = static_cast<I>(B) * H * N * per_row;
  for (I idx = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<I>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % static_cast<I>(per_row));
    I r = idx / static_cast<I>(per_row);
    const int n = static_cast<int>(r % static_cast<I>(N));
    r /= static_cast<I>(N);
    const int h = static_cast<int>(r % static_cast<I>(H)), b = static_cast<int>(r / static_cast<I>(H));
    const T* xr = x + b * x_bs + h * x_hs + static_cast<int64_t>(n) * x_rs;
    T* orow = out + b * o_bs + h * o_hs + static_cast<int64_t>(n) * o_rs;
    const int pos = (offsets != nullptr ? offsets[b] : offset) + n;
    const float* cr = cosb + static_cast<int64_t>(pos) * half;
    const float* sr = sinb + static_cast<int64_t>(pos) * half;
    const float sgn = inverse ? -1.f : 1.f;

    if (interleaved) {
      const int d0 = c * 8;
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + d0);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t o[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 v = Elem<T>::unpack(w[p]);
        const int i = (d0 >> 1) + p;
        if (i < half) {
          const float cs = __ldg(cr + i), sn = sgn * __ldg(sr + i);
          o[p] = Elem<T>::pack(v.x * cs - v.y * sn, v.x * sn + v.y * cs);
        } else {
          o[p] = w[p];
        }
      }
      *reinterpret_cast<uint4*>(orow + d0) = make_uint4(o[0], o[1], o[2], o[3]);
    } else if (c < half_chunks) {
      const int d0 = c * 8;                                  // elements d0..d0+7 pair with d0+half..d0+half+7
      const uint4 ra = *reinterpret_cast<const uint4*>(xr + d0);
      const uint4 rb = *reinterpret_cast<const uint4*>(xr + d0 + half);
      const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w}, wb[4] = {rb.x, rb.y, rb.z, rb.w};
      uint32_t oa[4], ob[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 a = Elem<T>::unpack(wa[p]), bb = Elem<T>::unpack(wb[p]);
        const int i = d0 + 2 * p;
        const float c0 = __ldg(cr + i), s0 = sgn * __ldg(sr + i), c1 = __ldg(cr + i + 1), s1 = sgn * __ldg(sr + i + 1);
        oa[p] = Elem<T>::pack(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
        ob[p] = Elem<T>::pack(a.x * s0 + bb.x * c0, a.y * s1 + bb.y * c1);
      }
      *reinterpret_cast<uint4*>(orow + d0) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
      *reinterpret_cast<uint4*>(orow + d0 + half) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
    } else {
      const int d0 = (rot_chunks + (c - half_chunks)) * 8;   // pass-through chunk beyond rotary_dim
      if (out != x) *reinterpret_cast<uint4*>(orow + d0) = *reinterpret_cast<const uint4*>(xr + d0);
    }
  }
}

}  // namespace

cudaError_t launch_rope(int dtype, const void* x, void* out, const float* cosb, const float* sinb, const int* offsets,
                        int offset, int B, int H, int N, int D, int rot, int interleaved, int inverse, const int64_t* xs,
                        const int64_t* os, cudaStream_t stream) {
  const int per_row = interleaved ? D / 8 : (rot / 16 + (D - rot) / 8);
  const int64_t total = static_cast<int64_t>(B) * H * N * per_row;
  if (total <= 0) return cudaSuccess;
  const int64_t want = (total + 255) / 256;
  const unsigned grid = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
  const bool small = total < (1LL << 31);
#define B200FA_ROPE_LAUNCH(T, I)                                                                                         \
  rope_kernel<T, I><<<grid, 256, 0, stream>>>(static_cast<const T*>(x), static_cast<T*>(out), cosb, sinb, offsets, offset, B, \
                                              H, N, D, rot, interleaved, inverse, xs[0], xs[1], xs[2], os[0], os[1], os[2])
  if (dtype == 0) {
    if (small) B200FA_ROPE_LAUNCH(__half, uint32_t); else B200FA_ROPE_LAUNCH(__half, int64_t);
  } else {
    if (small) B200FA_ROPE_LAUNCH(__nv_bfloat16, uint32_t); else B200FA_ROPE_LAUNCH(__nv_bfloat16, int64_t);
  }
#undef B200FA_ROPE_LAUNCH
  return cudaGetLastError();
}

}  // namespace b200fa
