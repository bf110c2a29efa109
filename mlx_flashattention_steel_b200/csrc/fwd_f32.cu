// float32 forward kernel: FFMA on the CUDA cores with fp32 accumulation and
// precise exp2f/tanhf, for the <= 1e-5 parity bar that tf32 tensor-core inputs
// (10-bit mantissa) cannot meet.  Fills the role of the reference's fp32 forward
// (csrc/mfa_attention.cpp:85-129, generator csrc/mfa_shader_gen.cpp:105-303).
// Same masks, softcap order and lse convention as the 16-bit kernels.
#include "common.cuh"
#include "launch.h"

namespace b200fa {

namespace {

constexpr int kBQ = 64;
constexpr int kBK = 64;
constexpr int kThreads = 256;
constexpr int kPad = 4;  // floats; makes 16-byte reads of consecutive rows conflict-free

template <int D>
__device__ __forceinline__ void load_rows(float* s, const float* g, int64_t rs, int row0, int limit,
                                          int tid) {
  constexpr int CH = D / 4;
  for (int i = tid; i < 64 * CH; i += kThreads) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gr < limit) val = *reinterpret_cast<const float4*>(g + static_cast<int64_t>(gr) * rs + c * 4);
    *reinterpret_cast<float4*>(s + r * (D + kPad) + c * 4) = val;
  }
}

template <int D, bool VARLEN>
__global__ void __launch_bounds__(kThreads) fa_fwd_f32_kernel(const FwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LD = D + kPad;
  constexpr int LDP = kBK + kPad;
  float* sQ = reinterpret_cast<float*>(smem_raw);
  float* sK = sQ + kBQ * LD;
  float* sV = sK + kBK * LD;
  float* sP = sV + kBK * LD;

  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
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
  const int q0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * kBQ;
  if (q0 >= N) return;
  const int off = S - N;
  int k_hi = S;
  if (p.causal) k_hi = min(S, q0 + kBQ + off);
  int k_lo = 0;
  if (p.window_left >= 0) k_lo = max(0, q0 + off - p.window_left);
  const int kt_begin = k_lo / kBK;
  const int kt_end = k_hi > 0 ? (k_hi + kBK - 1) / kBK : 0;

  const float* qg = reinterpret_cast<const float*>(p.q) + bb * p.q_bs + head * p.q_hs + q_begin * p.q_rs;
  const float* kg = reinterpret_cast<const float*>(p.k) + bb * p.k_bs + kvh * p.k_hs + k_begin * p.k_rs;
  const float* vg = reinterpret_cast<const float*>(p.v) + bb * p.v_bs + kvh * p.v_hs + k_begin * p.v_rs;
  float* og = reinterpret_cast<float*>(p.o) + bb * p.o_bs + head * p.o_hs + q_begin * p.o_rs;

  constexpr int NC = D / 64;  // float4 output columns per thread
  float4 o[4][NC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) o[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
  float row_max[4], row_sum[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { row_max[i] = -INFINITY; row_sum[i] = 0.f; }

  load_rows<D>(sQ, qg, p.q_rs, q0, N, tid);

  const bool use_cap = p.softcap > 0.f;
  const float alibi = p.alibi != nullptr ? p.alibi[head] : 0.f;

  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int k0 = kt * kBK;
    __syncthreads();  // previous tile fully consumed
    load_rows<D>(sK, kg, p.k_rs, k0, S, tid);
    load_rows<D>(sV, vg, p.v_rs, k0, S, tid);
    __syncthreads();

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int d = 0; d < D; d += 4) {
      float4 q4[4], k4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) q4[i] = *reinterpret_cast<const float4*>(sQ + (ty + 16 * i) * LD + d);
#pragma unroll
      for (int j = 0; j < 4; ++j) k4[j] = *reinterpret_cast<const float4*>(sK + (tx + 16 * j) * LD + d);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(q4[i].x, k4[j].x, acc[i][j]);
          acc[i][j] = fmaf(q4[i].y, k4[j].y, acc[i][j]);
          acc[i][j] = fmaf(q4[i].z, k4[j].z, acc[i][j]);
          acc[i][j] = fmaf(q4[i].w, k4[j].w, acc[i][j]);
        }
    }

    // scale, softcap, masks; scores move to the base-2 domain
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = q0 + ty + 16 * i;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = k0 + tx + 16 * j;
        float sc = acc[i][j] * p.scale;
        if (use_cap) sc = tanhf(sc / p.softcap) * p.softcap;
        if (p.alibi != nullptr) sc = fmaf(alibi, static_cast<float>(col - (row + off)), sc);
        sc *= kLog2e;
        bool vis = col < S;
        if (p.causal) vis = vis && (col <= row + off);
        if (p.window_left >= 0) vis = vis && (col >= row + off - p.window_left);
        acc[i][j] = vis ? sc : -INFINITY;
      }
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float mx = fmaxf(fmaxf(acc[i][0], acc[i][1]), fmaxf(acc[i][2], acc[i][3]));
#pragma unroll
      for (int sft = 1; sft < 16; sft <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
      mx = fmaxf(mx, row_max[i]);
      const float msub = (mx == -INFINITY) ? 0.f : mx;
      const float corr = exp2f(row_max[i] - msub);
      row_max[i] = mx;
      row_sum[i] *= corr;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        o[i][c].x *= corr; o[i][c].y *= corr; o[i][c].z *= corr; o[i][c].w *= corr;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float pv = exp2f(acc[i][j] - msub);
        row_sum[i] += pv;
        sP[(ty + 16 * i) * LDP + tx + 16 * j] = pv;
      }
    }
    __syncthreads();

    // O += P V
#pragma unroll 2
    for (int key = 0; key < kBK; key += 4) {
      float4 p4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p4[i] = *reinterpret_cast<const float4*>(sP + (ty + 16 * i) * LDP + key);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        float4 v4[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c)
          v4[c] = *reinterpret_cast<const float4*>(sV + (key + kk) * LD + tx * 4 + 64 * c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float pv = kk == 0 ? p4[i].x : kk == 1 ? p4[i].y : kk == 2 ? p4[i].z : p4[i].w;
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            o[i][c].x = fmaf(pv, v4[c].x, o[i][c].x);
            o[i][c].y = fmaf(pv, v4[c].y, o[i][c].y);
            o[i][c].z = fmaf(pv, v4[c].z, o[i][c].z);
            o[i][c].w = fmaf(pv, v4[c].w, o[i][c].w);
          }
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float sum = row_sum[i];
#pragma unroll
    for (int sft = 1; sft < 16; sft <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sft);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    const int row = q0 + ty + 16 * i;
    if (row < N) {
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        float4 val = o[i][c];
        val.x *= inv; val.y *= inv; val.z *= inv; val.w *= inv;
        *reinterpret_cast<float4*>(og + static_cast<int64_t>(row) * p.o_rs + tx * 4 + 64 * c) = val;
      }
      if (p.lse != nullptr && tx == 0) {
        float* lg = p.lse + bb * p.lse_bs + head * p.lse_hs + q_begin;
        lg[row] = sum > 0.f ? row_max[i] + log2f(sum) : -INFINITY;
      }
    }
  }
}

template <int D, bool VARLEN>
cudaError_t launch_one(const FwdParams& p, int nbatch, int max_q, cudaStream_t stream) {
  constexpr size_t smem = (static_cast<size_t>(3) * 64 * (D + kPad) + 64 * (kBK + kPad)) * sizeof(float);
  auto kern = fa_fwd_f32_kernel<D, VARLEN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  dim3 grid((max_q + kBQ - 1) / kBQ, p.Hq, nbatch);
  kern<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_f32(const FwdParams& p, int D, bool varlen, int nbatch, int max_q,
                           cudaStream_t stream) {
  if (max_q <= 0 || nbatch <= 0) return cudaSuccess;
  if (D == 64) return varlen ? launch_one<64, true>(p, nbatch, max_q, stream)
                             : launch_one<64, false>(p, nbatch, max_q, stream);
  if (D == 128) return varlen ? launch_one<128, true>(p, nbatch, max_q, stream)
                              : launch_one<128, false>(p, nbatch, max_q, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200fa
