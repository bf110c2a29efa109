// Shared device helpers and kernel parameter blocks for libb200fa.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200fa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Parameter block shared by the forward kernels (dense and varlen).  Role of
// MFASteelParams (csrc/mfa_steel_fwd.hpp:25-54) in the reference.
struct FwdParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;            // may be null
  int64_t q_bs, q_hs, q_rs;
  int64_t k_bs, k_hs, k_rs;
  int64_t v_bs, v_hs, v_rs;
  int64_t o_bs, o_hs, o_rs;
  int64_t lse_bs, lse_hs;
  int B, Hq, Hkv, N, S;
  int gqa;               // Hq / Hkv
  float scale;           // multiplies q.k
  float scale_log2;      // scale * log2(e)
  float softcap;         // 0 = off
  int causal;
  int window_left;       // -1 = off
  const int* cu_q;       // varlen only
  const int* cu_k;
  const float* alibi;    // per q-head slopes, or null
  const unsigned char* bmask;  // block mask bytes [rows / bm_bq][bm_nk], or null
  int bm_bq, bm_bk, bm_nk;
  // Dense layout only (tcgen05 kernel): per-batch key counts (null = S for every batch entry), and a page pool in
  // place of dense k / v: k and v then point at pools [num_pages, page_size, Hkv, D] and the keys of batch entry b
  // are the tokens block_table[b][0 .. ] lists, kv_lens[b] of them.
  const int* kv_lens;
  const int* block_table;      // [B, max_blocks], -1 = no page; null = dense k / v
  int max_blocks, page_size, num_pages;
  int persist_mode;            // tcgen05 forward: 0 = the launcher chooses, 1 = persistent CTAs, 2 = one item per CTA
};

// Backward parameter block.  Role of MFASteelBackwardParams
// (csrc/mfa_steel_bwd.hpp:29-54).
struct BwdParams {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* dout;
  const float* lse;
  float* delta;          // workspace [B,Hq,N_pad]
  float* dq_acc;         // workspace fp32 [B,Hq,N,D]
  int* work_counter;     // workspace: next work item of the persistent backward kernel (reset by the preprocess kernel)
  void* dq;
  void* dk;
  void* dv;
  int64_t q_bs, q_hs, q_rs;
  int64_t k_bs, k_hs, k_rs;
  int64_t v_bs, v_hs, v_rs;
  int64_t o_bs, o_hs, o_rs;     // out and dout share a layout
  int64_t dq_bs, dq_hs, dq_rs;  // contiguous
  int64_t dk_bs, dk_hs, dk_rs;  // contiguous; dv shares it
  int64_t lse_bs, lse_hs;
  int B, Hq, Hkv, N, S;
  int gqa;
  float scale;
  float scale_log2;
  float softcap;         // 0 = off: the forward capped the scaled scores with cap * tanh(s / cap)
  int causal;
  int window_left;       // -1 = off
  const int* cu_q;
  const int* cu_k;
  const float* alibi;    // per q-head slopes, or null
  const unsigned char* bmask;  // block mask bytes [rows / bm_bq][bm_nk], or null
  int bm_bq, bm_bk, bm_nk;
};

// ---------------------------------------------------------------------------
// element type traits
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
};
template <> struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
};

// ---------------------------------------------------------------------------
// PTX wrappers (portable tensor-core path: ldmatrix + mma.sync m16n8k16)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                 uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4],
                                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// tanh of the soft cap.  tanh.approx is specified to a relative error of 2^-11; multiplied by cap * log2(e) that is
// an absolute error of the capped score, negligible for the caps models use (30, 50) and above the 2e-2 parity bar
// from cap ~ 70 on.  Caps of 64 and more therefore take 1 - 2 / (2^(2 y log2 e) + 1): two special-function operations,
// absolute error ~1e-7 (saturates cleanly: 2^x = inf gives 1, 2^x = 0 gives -1).
constexpr float kPreciseTanhMinCap = 64.f;
__device__ __forceinline__ float tanh_exp(float y) {
  const float e = fast_exp2(y * (2.f * kLog2e));
  return 1.f - __fdividef(2.f, e + 1.f);
}
__device__ __forceinline__ float cap_tanh(float y, bool precise) { return precise ? tanh_exp(y) : fast_tanh(y); }
// Backward kernels, soft cap, small scores.  With y = s * scale / cap and |y| <= y3 = min(0.3, (7.5e-3 / cap)^(1/5))
// the degree-3 truncation of tanh is within 1e-3 / cap of it, so the capped score in the log2 domain is
//   cap * log2(e) * tanh(y) ~ s * (kk + kb3 * z),  z = s^2, kk = scale * log2(e), kb3 = -kk * (scale / cap)^2 / 3
// and 1 - tanh^2(y) ~ 1 + z * (e1 + e2 * z), e1 = -(scale / cap)^2, e2 = (2 / 3) (scale / cap)^4 (the y^6 / 9 term is
// below 1e-5 there): six packed FMA-pipe operations per pair of scores and no special-function operation besides the
// two exponentials.  tanh.approx on every score instead doubles the load of the special-function unit (16 results per
// clock per SM), which is what bounds phase A of those kernels.
struct SmallCap {
  float y3, kk, kb3, e1, e2;
};
__device__ __forceinline__ SmallCap small_cap_consts(float scale, float softcap) {
  SmallCap c;
  const float ci = scale / softcap;
  c.y3 = fminf(0.3f, powf(7.5e-3f / softcap, 0.2f));
  c.kk = scale * kLog2e;
  c.kb3 = -c.kk * ci * ci * (1.f / 3.f);
  c.e1 = -ci * ci;
  c.e2 = (2.f / 3.f) * ci * ci * ci * ci;
  return c;
}

// Shared-memory tile of rows x DCOLS 16-bit elements, 16-byte chunks XOR-swizzled
// by the row so that ldmatrix reads of 8 consecutive rows are conflict-free.
template <int DCOLS>
__device__ __forceinline__ uint32_t swz_off(int row, int col /*multiple of 8*/) {
  int chunk = col >> 3;
  return static_cast<uint32_t>((row * DCOLS + ((chunk ^ (row & 7)) << 3)) * 2);
}

}  // namespace b200fa
