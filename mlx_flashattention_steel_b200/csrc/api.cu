// C-ABI of libb200fa.so: argument validation, kernel-family choice and launch.
// Host-side role of MFAttention::eval_gpu and friends in the reference
// (csrc/mfa_attention.cpp:47-409, 732-930, 1228-1305, 1355-1496) without their
// allocation: callers own outputs and workspace.
#include "../../include/b200fa.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "decode.h"
#include "launch.h"

namespace {

thread_local char g_err[512] = "";

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int32_t cuda_fail(cudaError_t e, const char* what) {
  return fail(B200FA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int elem_bytes(int dtype) {
  switch (dtype) {
    case B200FA_F16:
    case B200FA_BF16: return 2;
    case B200FA_F32: return 4;
    case B200FA_I8:
    case B200FA_E4M3: return 1;
    default: return 0;
  }
}

// Resolves strides (all-zero => contiguous [B,H,rows,D]) and checks them.
bool resolve_strides(const int64_t in[3], int H, int rows, int D, int eb, int64_t out[3]) {
  if (in[0] == 0 && in[1] == 0 && in[2] == 0) {
    out[2] = D;
    out[1] = static_cast<int64_t>(rows) * D;
    out[0] = static_cast<int64_t>(H) * rows * D;
    return true;
  }
  for (int i = 0; i < 3; ++i) {
    if (in[i] < 0) return false;
    if ((in[i] * eb) % 16 != 0) return false;
    out[i] = in[i];
  }
  return out[2] >= D;
}

int32_t check_common(const b200fa_desc* d, bool varlen) {
  if (d == nullptr) return fail(B200FA_ERR_INVALID_ARG, "descriptor is null");
  if (d->dtype != B200FA_F16 && d->dtype != B200FA_BF16 && d->dtype != B200FA_F32)
    return fail(B200FA_ERR_UNSUPPORTED, "dtype %d: expected f16, bf16 or f32", d->dtype);
  if (d->D != 64 && d->D != 128 && !(d->D == 256 && d->dtype != B200FA_F32))
    return fail(B200FA_ERR_UNSUPPORTED, "head_dim %d: this build has 64 and 128 (and 256 for the f16 / bf16 forward)", d->D);
  if (d->B < 0 || d->Hq <= 0 || d->Hkv <= 0 || d->N < 0 || d->S < 0)
    return fail(B200FA_ERR_INVALID_ARG, "negative or zero extent (B=%d Hq=%d Hkv=%d N=%d S=%d)", d->B,
                d->Hq, d->Hkv, d->N, d->S);
  if (d->Hq % d->Hkv != 0)
    return fail(B200FA_ERR_INVALID_ARG, "q_heads (%d) must be divisible by kv_heads (%d)", d->Hq, d->Hkv);
  if (varlen && d->B != 1) return fail(B200FA_ERR_INVALID_ARG, "varlen expects B == 1, got %d", d->B);
  if (!(d->scale == d->scale)) return fail(B200FA_ERR_INVALID_ARG, "scale is NaN");
  if (d->softcap < 0.f) return fail(B200FA_ERR_INVALID_ARG, "softcap must be >= 0");
  if (d->window_left < -1) return fail(B200FA_ERR_INVALID_ARG, "window_left must be >= -1");
  return B200FA_OK;
}

int32_t fill_fwd_params(const b200fa_desc* d, const void* q, const void* k, const void* v, void* out,
                        float* lse, b200fa::FwdParams* p) {
  const int eb = elem_bytes(d->dtype);
  int64_t qs[3], ks[3], vs[3], os[3];
  if (!resolve_strides(d->q_strides, d->Hq, d->N, d->D, eb, qs) ||
      !resolve_strides(d->k_strides, d->Hkv, d->S, d->D, eb, ks) ||
      !resolve_strides(d->v_strides, d->Hkv, d->S, d->D, eb, vs) ||
      !resolve_strides(d->o_strides, d->Hq, d->N, d->D, eb, os))
    return fail(B200FA_ERR_INVALID_ARG, "strides must be non-negative, 16-byte multiples, row stride >= D");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
    return fail(B200FA_ERR_INVALID_ARG, "q, k, v and out must be 16-byte aligned");
  memset(p, 0, sizeof(*p));
  p->q = q; p->k = k; p->v = v; p->o = out; p->lse = lse;
  p->q_bs = qs[0]; p->q_hs = qs[1]; p->q_rs = qs[2];
  p->k_bs = ks[0]; p->k_hs = ks[1]; p->k_rs = ks[2];
  p->v_bs = vs[0]; p->v_hs = vs[1]; p->v_rs = vs[2];
  p->o_bs = os[0]; p->o_hs = os[1]; p->o_rs = os[2];
  p->lse_hs = d->N;
  p->lse_bs = static_cast<int64_t>(d->Hq) * d->N;
  p->B = d->B; p->Hq = d->Hq; p->Hkv = d->Hkv; p->N = d->N; p->S = d->S;
  p->gqa = d->Hq / d->Hkv;
  p->scale = d->scale;
  p->scale_log2 = d->scale * b200fa::kLog2e;
  p->softcap = d->softcap;
  p->causal = d->causal ? 1 : 0;
  p->window_left = d->window_left;
  p->alibi = d->alibi_slopes;
  p->bmask = d->block_mask;
  p->bm_bq = d->mask_bq; p->bm_bk = d->mask_bk; p->bm_nk = d->mask_nk;
  p->kv_lens = d->kv_lens;
  p->persist_mode = (d->flags & B200FA_FLAG_FWD_PERSISTENT) ? 1 : ((d->flags & B200FA_FLAG_FWD_ONE_ITEM) ? 2 : 0);
  if (d->block_mask != nullptr) {
    if (d->mask_bq <= 0 || d->mask_bk <= 0 || static_cast<int64_t>(d->mask_nk) * d->mask_bk < d->S)
      return fail(B200FA_ERR_INVALID_ARG, "block_mask: block sizes must be positive and mask_nk * mask_bk cover S");
    if (d->dtype == B200FA_F32) return fail(B200FA_ERR_UNSUPPORTED, "block_mask takes f16 / bf16");
  }
  return B200FA_OK;
}

}  // namespace

namespace b200fa {
// Lets entry points defined in other .cu files fill the thread-local error string.
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
}  // namespace b200fa

extern "C" {

const char* b200fa_last_error(void) { return g_err; }
const char* b200fa_version(void) { return "b200fa 0.1 (sm_100a)"; }

int32_t b200fa_device_info(int32_t device, b200fa_device_info_t* out) {
  if (out == nullptr) return fail(B200FA_ERR_INVALID_ARG, "out is null");
  int dev = device;
  cudaError_t e;
  if (dev < 0) {
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
  memset(out, 0, sizeof(*out));
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->sm_count = prop.multiProcessorCount;
  out->smem_per_block_optin = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  out->has_tcgen05 = prop.major == 10 ? 1 : 0;
  strncpy(out->name, prop.name, sizeof(out->name) - 1);
  return B200FA_OK;
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
// Dense flash-decode route (the reference's use_flash_decode, csrc/mfa_attention.cpp:150-151: N <= 4, S >= 256,
// 16-bit, no block mask), further limited to what the split-KV decode kernel takes: at most 8 query rows per kv
// head, head_dim 64 / 128, no window and no ALiBi, contiguous q and out.
static bool dense_decode_route(const b200fa_desc* d) {
  if (d == nullptr || (d->dtype != B200FA_F16 && d->dtype != B200FA_BF16)) return false;
  if (d->flags & B200FA_FLAG_FORCE_MMA_SYNC) return false;
  if (!(d->N >= 1 && d->N <= 4 && d->S >= 256) || (d->D != 64 && d->D != 128)) return false;
  if (d->Hkv <= 0 || d->Hq % d->Hkv != 0 || (d->Hq / d->Hkv) * d->N > 8) return false;
  if (d->window_left >= 0 || d->alibi_slopes != nullptr || d->block_mask != nullptr) return false;
  if (d->causal && d->N > d->S) return false;
  auto contiguous = [&](const int64_t st[3]) {
    return (st[0] == 0 && st[1] == 0 && st[2] == 0) ||
           (st[2] == d->D && st[1] == static_cast<int64_t>(d->N) * d->D && (d->B == 1 || st[0] == static_cast<int64_t>(d->Hq) * d->N * d->D));
  };
  return contiguous(d->q_strides) && contiguous(d->o_strides);
}

size_t b200fa_fwd_workspace_bytes(const b200fa_desc* d) {
  if (!dense_decode_route(d)) return 0;
  return b200fa::decode_workspace_bytes(d->B, d->Hq, d->Hkv, d->N, d->D, d->S, d->num_splits);
}

int32_t b200fa_fwd(const b200fa_desc* d, const void* q, const void* k, const void* v, void* out,
                   float* lse, void* workspace, size_t workspace_bytes, void* stream) {
  int32_t st = check_common(d, false);
  if (st != B200FA_OK) return st;
  if (d->B == 0 || d->N == 0) return B200FA_OK;
  if (q == nullptr || out == nullptr) return fail(B200FA_ERR_INVALID_ARG, "q or out is null");
  if (d->S > 0 && (k == nullptr || v == nullptr)) return fail(B200FA_ERR_INVALID_ARG, "k or v is null");
  b200fa::FwdParams p;
  st = fill_fwd_params(d, q, d->S > 0 ? k : q, d->S > 0 ? v : q, out, lse, &p);
  if (st != B200FA_OK) return st;
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  // A few query rows against a long dense cache: split-KV decode over the cache in place (all SMs share the keys of
  // every head) instead of one 128-row tile per head.  Taken when the caller brought the workspace the query asked
  // for; without it the call runs the prefill kernel, which is correct for every shape.
  if (dense_decode_route(d) && workspace != nullptr && aligned16(workspace) &&
      workspace_bytes >= b200fa::decode_workspace_bytes(d->B, d->Hq, d->Hkv, d->N, d->D, d->S, d->num_splits) &&
      !(p.B > 1 && (p.k_bs == 0 || p.v_bs == 0)) && !(p.Hkv > 1 && (p.k_hs == 0 || p.v_hs == 0))) {
    b200fa::DecodeParams dp;
    memset(&dp, 0, sizeof(dp));
    dp.q = q; dp.k_pool = k; dp.v_pool = v; dp.out = out; dp.lse = lse; dp.workspace = workspace;
    dp.B = d->B; dp.Hq = d->Hq; dp.Hkv = d->Hkv; dp.Nq = d->N; dp.D = d->D;
    dp.num_pages = 0; dp.block_size = 16; dp.max_blocks = 0; dp.max_kv_len = d->S;
    dp.q_dtype = d->dtype; dp.kv_dtype = d->dtype;
    dp.scale = d->scale; dp.softcap = d->softcap; dp.causal = d->causal ? 1 : 0;
    dp.num_splits = d->num_splits;
    dp.dense = 1;
    dp.k_bs = p.k_bs; dp.k_hs = p.k_hs; dp.k_rs = p.k_rs;
    dp.v_bs = p.v_bs; dp.v_hs = p.v_hs; dp.v_rs = p.v_rs;
    char msg[256] = "";
    e = b200fa::launch_decode_paged(dp, cs, msg, sizeof(msg));
    if (e == cudaSuccess) return B200FA_OK;
    if (e != cudaErrorNotSupported) return fail(B200FA_ERR_CUDA, "dense decode launch: %s %s", cudaGetErrorString(e), msg);
    // not a shape the decode kernel takes after all: fall through to the prefill kernels
  }
  if (d->kv_lens != nullptr && (d->dtype == B200FA_F32 || !b200fa::fwd_sm100_supported(p, d->dtype, d->D)))
    return fail(B200FA_ERR_UNSUPPORTED, "kv_lens takes f16 / bf16 at head_dim 64 / 128 with positive batch and head strides");
  if (d->dtype == B200FA_F32) {
    e = b200fa::launch_fwd_f32(p, d->D, false, d->B, d->N, cs);
  } else if ((d->kv_lens != nullptr || !(d->flags & B200FA_FLAG_FORCE_MMA_SYNC)) && b200fa::fwd_sm100_supported(p, d->dtype, d->D)) {
    e = b200fa::launch_fwd_sm100(p, d->dtype, d->D, d->B, d->N, cs);
  } else {
    e = b200fa::launch_fwd_mma(p, d->dtype, d->D, false, d->B, d->N, cs);
  }
  if (e != cudaSuccess) return cuda_fail(e, "forward launch");
  return B200FA_OK;
}

int32_t b200fa_combine_partials(const float* gathered, int32_t R, int64_t rows, int32_t D, int32_t out_dtype,
                                void* out, float* lse, void* stream) {
  if (R < 0 || rows < 0 || D <= 0 || D % 4 != 0 || D > 128) return fail(B200FA_ERR_INVALID_ARG, "combine_partials: bad extent");
  if (out_dtype != B200FA_F16 && out_dtype != B200FA_BF16) return fail(B200FA_ERR_UNSUPPORTED, "combine_partials: f16 / bf16 output");
  if (R == 0 || rows == 0) return B200FA_OK;
  if (!gathered || !out) return fail(B200FA_ERR_INVALID_ARG, "combine_partials: null pointer");
  if (!aligned16(gathered) || (reinterpret_cast<uintptr_t>(out) & 7u)) return fail(B200FA_ERR_INVALID_ARG, "combine_partials: alignment");
  cudaError_t e = b200fa::launch_combine_partials(gathered, R, rows, D, out_dtype, out, lse, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "combine_partials launch");
  return B200FA_OK;
}

int32_t b200fa_fwd_paged(const b200fa_desc* d, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_table, const int32_t* seq_lens, int32_t num_pages, int32_t block_size,
                         int32_t max_blocks, int32_t max_kv_len, void* out, float* lse, void* stream) {
  int32_t st = check_common(d, false);
  if (st != B200FA_OK) return st;
  if (d->dtype != B200FA_F16 && d->dtype != B200FA_BF16) return fail(B200FA_ERR_UNSUPPORTED, "paged forward takes f16 / bf16");
  if (d->kv_dtype != d->dtype)
    return fail(B200FA_ERR_UNSUPPORTED, "paged forward reads 16-bit pools; dequantise 8-bit pools with b200fa_paged_kv_gather_dequant");
  if (d->D != 64 && d->D != 128) return fail(B200FA_ERR_UNSUPPORTED, "paged forward is built for head_dim 64 and 128");
  if (d->alibi_slopes != nullptr || d->block_mask != nullptr)
    return fail(B200FA_ERR_UNSUPPORTED, "alibi_slopes / block_mask are not supported in paged mode");
  if (block_size < 16 || block_size % 16 != 0)
    return fail(B200FA_ERR_UNSUPPORTED, "paged forward takes pages of a multiple of 16 tokens, got %d", block_size);
  if (num_pages <= 0 || max_blocks <= 0 || max_kv_len < 0) return fail(B200FA_ERR_INVALID_ARG, "bad extent");
  if (static_cast<int64_t>(num_pages) * block_size >= (1LL << 31)) return fail(B200FA_ERR_UNSUPPORTED, "pool of 2^31 tokens or more");
  if (static_cast<int64_t>(max_blocks) * block_size < max_kv_len)
    return fail(B200FA_ERR_INVALID_ARG, "max_kv_len %d exceeds max_blocks*block_size", max_kv_len);
  if (d->B == 0 || d->N == 0) return B200FA_OK;
  if (!q || !k_pool || !v_pool || !block_table || !seq_lens || !out) return fail(B200FA_ERR_INVALID_ARG, "null tensor pointer");
  b200fa_desc dd = *d;
  dd.S = max_kv_len;
  dd.k_strides[0] = dd.k_strides[1] = dd.k_strides[2] = 0;      // the pools are addressed through the table, not by strides
  dd.v_strides[0] = dd.v_strides[1] = dd.v_strides[2] = 0;
  b200fa::FwdParams p;
  st = fill_fwd_params(&dd, q, k_pool, v_pool, out, lse, &p);
  if (st != B200FA_OK) return st;
  p.kv_lens = seq_lens;
  p.block_table = block_table;
  p.max_blocks = max_blocks; p.page_size = block_size; p.num_pages = num_pages;
  if (!b200fa::fwd_sm100_supported(p, d->dtype, d->D))
    return fail(B200FA_ERR_UNSUPPORTED, "paged forward: shape or strides not taken by the tcgen05 kernel");
  cudaError_t e = b200fa::launch_fwd_sm100(p, d->dtype, d->D, d->B, d->N, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "paged forward launch");
  return B200FA_OK;
}

int32_t b200fa_paged_kv_gather_dequant(const void* pool, const void* scale, const int32_t* block_table,
                                       const int32_t* seq_lens, int32_t B, int32_t H, int32_t D, int32_t pool_dtype,
                                       int32_t out_dtype, int32_t block_size, int32_t max_blocks, int32_t max_kv_len,
                                       void* out, void* stream) {
  if (B < 0 || H <= 0 || D <= 0 || block_size <= 0 || max_blocks < 0 || max_kv_len < 0)
    return fail(B200FA_ERR_INVALID_ARG, "bad extent");
  if (pool_dtype != B200FA_I8 && pool_dtype != B200FA_E4M3) return fail(B200FA_ERR_UNSUPPORTED, "gather_dequant: pool must be int8 or e4m3");
  if (out_dtype != B200FA_F16 && out_dtype != B200FA_BF16) return fail(B200FA_ERR_UNSUPPORTED, "gather_dequant: output must be f16 or bf16");
  if (D % 16 != 0) return fail(B200FA_ERR_INVALID_ARG, "D must be a multiple of 16");
  if (B == 0 || max_kv_len == 0) return B200FA_OK;
  if (!pool || !scale || !block_table || !seq_lens || !out) return fail(B200FA_ERR_INVALID_ARG, "null pointer");
  if (!aligned16(pool) || !aligned16(out)) return fail(B200FA_ERR_INVALID_ARG, "pool/out must be 16-byte aligned");
  if (static_cast<int64_t>(max_blocks) * block_size < max_kv_len)
    return fail(B200FA_ERR_INVALID_ARG, "max_kv_len %d exceeds max_blocks*block_size", max_kv_len);
  cudaError_t e = b200fa::launch_paged_gather_dequant(pool, scale, block_table, seq_lens, B, H, D, pool_dtype, out_dtype,
                                                      block_size, max_blocks, max_kv_len, out,
                                                      reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "gather_dequant launch");
  return B200FA_OK;
}

size_t b200fa_fwd_varlen_workspace_bytes(const b200fa_desc* d, int32_t num_seqs, int32_t max_seqlen_q,
                                         int32_t max_seqlen_k) {
  (void)d; (void)num_seqs; (void)max_seqlen_q; (void)max_seqlen_k;
  return 0;
}

int32_t b200fa_fwd_varlen(const b200fa_desc* d, const void* q, const void* k, const void* v,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int32_t num_seqs,
                          int32_t max_seqlen_q, int32_t max_seqlen_k, void* out, float* lse,
                          void* workspace, size_t workspace_bytes, void* stream) {
  (void)workspace; (void)workspace_bytes; (void)max_seqlen_k;
  int32_t st = check_common(d, true);
  if (st != B200FA_OK) return st;
  if (num_seqs < 0 || max_seqlen_q < 0) return fail(B200FA_ERR_INVALID_ARG, "negative num_seqs/max_seqlen");
  if (num_seqs == 0 || d->N == 0 || max_seqlen_q == 0) return B200FA_OK;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || cu_seqlens_q == nullptr ||
      cu_seqlens_k == nullptr)
    return fail(B200FA_ERR_INVALID_ARG, "null tensor pointer");
  b200fa::FwdParams p;
  st = fill_fwd_params(d, q, k, v, out, lse, &p);
  if (st != B200FA_OK) return st;
  if (d->alibi_slopes != nullptr || d->block_mask != nullptr || d->kv_lens != nullptr)
    return fail(B200FA_ERR_UNSUPPORTED, "alibi_slopes / block_mask / kv_lens with packed sequences are not built");
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (d->dtype == B200FA_F32) {
    e = b200fa::launch_fwd_f32(p, d->D, true, num_seqs, max_seqlen_q, cs);
  } else if (!(d->flags & B200FA_FLAG_FORCE_MMA_SYNC) && b200fa::fwd_sm100_supported(p, d->dtype, d->D)) {
    e = b200fa::launch_fwd_sm100(p, d->dtype, d->D, num_seqs, max_seqlen_q, cs);
  } else {
    e = b200fa::launch_fwd_mma(p, d->dtype, d->D, true, num_seqs, max_seqlen_q, cs);
  }
  if (e != cudaSuccess) return cuda_fail(e, "varlen forward launch");
  return B200FA_OK;
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// Shape, stride and option fields of the backward parameter block (no workspace pointers yet).
static int32_t fill_bwd_params(const b200fa_desc* d, const void* q, const void* k, const void* v, const void* out,
                               const float* lse, const void* dout, void* dq, void* dk, void* dv, const int32_t* cu_q,
                               const int32_t* cu_k, b200fa::BwdParams* pp) {
  b200fa::FwdParams f;
  int32_t st = fill_fwd_params(d, q, k, v, const_cast<void*>(out), nullptr, &f);
  if (st != B200FA_OK) return st;
  b200fa::BwdParams& p = *pp;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k = k; p.v = v; p.o = out; p.dout = dout; p.lse = lse;
  p.dq = dq; p.dk = dk; p.dv = dv;
  p.q_bs = f.q_bs; p.q_hs = f.q_hs; p.q_rs = f.q_rs;
  p.k_bs = f.k_bs; p.k_hs = f.k_hs; p.k_rs = f.k_rs;
  p.v_bs = f.v_bs; p.v_hs = f.v_hs; p.v_rs = f.v_rs;
  p.o_bs = f.o_bs; p.o_hs = f.o_hs; p.o_rs = f.o_rs;
  p.dq_rs = d->D; p.dq_hs = static_cast<int64_t>(d->N) * d->D; p.dq_bs = p.dq_hs * d->Hq;
  p.dk_rs = d->D; p.dk_hs = static_cast<int64_t>(d->S) * d->D; p.dk_bs = p.dk_hs * d->Hkv;
  p.lse_hs = f.lse_hs; p.lse_bs = f.lse_bs;
  p.B = d->B; p.Hq = d->Hq; p.Hkv = d->Hkv; p.N = d->N; p.S = d->S;
  p.gqa = f.gqa; p.scale = d->scale; p.scale_log2 = f.scale_log2; p.causal = f.causal;
  p.softcap = d->softcap; p.window_left = d->window_left;
  p.cu_q = cu_q; p.cu_k = cu_k;
  p.alibi = d->alibi_slopes;
  p.bmask = d->block_mask;
  p.bm_bq = d->mask_bq; p.bm_bk = d->mask_bk; p.bm_nk = d->mask_nk;
  return B200FA_OK;
}

static bool bwd_allow_sm100(const b200fa_desc* d) { return !(d->flags & B200FA_FLAG_FORCE_MMA_SYNC); }

// The split head_dim-128 path keeps no fp32 dQ accumulator, which is most of the workspace.
static size_t bwd_need_bytes(const b200fa_desc* d) {
  b200fa::BwdParams p;
  if (d->dtype == B200FA_F32 || d->D == 256 ||
      fill_bwd_params(d, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &p) != B200FA_OK)
    return b200fa::bwd_workspace_bytes(d->B, d->Hq, d->N, d->D, false);
  return b200fa::bwd_workspace_bytes(d->B, d->Hq, d->N, d->D, b200fa::bwd_takes_split_path(p, d->dtype, d->D, bwd_allow_sm100(d)));
}

static int32_t bwd_common(const b200fa_desc* d, const void* q, const void* k, const void* v,
                          const void* out, const float* lse, const void* dout, void* dq, void* dk,
                          void* dv, const int32_t* cu_q, const int32_t* cu_k, int nbatch, int max_q,
                          int max_k, void* workspace, size_t workspace_bytes, void* stream) {
  const bool varlen = cu_q != nullptr;
  int32_t st = check_common(d, varlen);
  if (st != B200FA_OK) return st;
  if (d->dtype == B200FA_F32)
    return fail(B200FA_ERR_UNSUPPORTED, "backward is built for f16 and bf16 (the reference's STEEL backward, "
                                        "mlx_mfa/attention.py:2008-2012, takes the same)");
  if (d->kv_lens != nullptr) return fail(B200FA_ERR_UNSUPPORTED, "backward with kv_lens is not built");
  if (d->B == 0 || d->N == 0 || nbatch == 0) return B200FA_OK;
  if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv)
    return fail(B200FA_ERR_INVALID_ARG, "null tensor pointer");
  if (d->D == 256) return fail(B200FA_ERR_UNSUPPORTED, "backward for head_dim 256 is not built");
  const size_t need = bwd_need_bytes(d);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(B200FA_ERR_WORKSPACE, "backward needs %zu workspace bytes, got %zu", need, workspace_bytes);
  if (!aligned16(workspace)) return fail(B200FA_ERR_INVALID_ARG, "workspace must be 16-byte aligned");
  if (!aligned16(dout) || !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
    return fail(B200FA_ERR_INVALID_ARG, "dout, dq, dk, dv must be 16-byte aligned");
  if ((d->alibi_slopes != nullptr || d->block_mask != nullptr) && varlen)
    return fail(B200FA_ERR_UNSUPPORTED, "alibi_slopes / block_mask with packed sequences are not built");
  b200fa::BwdParams p;
  st = fill_bwd_params(d, q, k, v, out, lse, dout, dq, dk, dv, cu_q, cu_k, &p);
  if (st != B200FA_OK) return st;
  cudaError_t e = b200fa::launch_bwd(p, d->dtype, d->D, varlen, nbatch, max_q, max_k, workspace, bwd_allow_sm100(d),
                                     reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "backward launch");
  return B200FA_OK;
}

size_t b200fa_bwd_workspace_bytes(const b200fa_desc* d) {
  if (d == nullptr) return 0;
  return bwd_need_bytes(d);
}

int32_t b200fa_bwd(const b200fa_desc* d, const void* q, const void* k, const void* v, const void* out,
                   const float* lse, const void* dout, void* dq, void* dk, void* dv, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if (d == nullptr) return fail(B200FA_ERR_INVALID_ARG, "descriptor is null");
  return bwd_common(d, q, k, v, out, lse, dout, dq, dk, dv, nullptr, nullptr, d->B, d->N, d->S, workspace,
                    workspace_bytes, stream);
}

size_t b200fa_bwd_varlen_workspace_bytes(const b200fa_desc* d, int32_t num_seqs, int32_t max_seqlen_q,
                                         int32_t max_seqlen_k) {
  (void)num_seqs; (void)max_seqlen_q; (void)max_seqlen_k;
  if (d == nullptr) return 0;
  return bwd_need_bytes(d);
}

int32_t b200fa_bwd_varlen(const b200fa_desc* d, const void* q, const void* k, const void* v,
                          const void* out, const float* lse, const void* dout,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int32_t num_seqs,
                          int32_t max_seqlen_q, int32_t max_seqlen_k, void* dq, void* dk, void* dv,
                          void* workspace, size_t workspace_bytes, void* stream) {
  if (d == nullptr) return fail(B200FA_ERR_INVALID_ARG, "descriptor is null");
  if (cu_seqlens_q == nullptr || cu_seqlens_k == nullptr)
    return fail(B200FA_ERR_INVALID_ARG, "cu_seqlens is null");
  if (num_seqs < 0 || max_seqlen_q < 0 || max_seqlen_k < 0)
    return fail(B200FA_ERR_INVALID_ARG, "negative num_seqs/max_seqlen");
  return bwd_common(d, q, k, v, out, lse, dout, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, num_seqs,
                    max_seqlen_q, max_seqlen_k, workspace, workspace_bytes, stream);
}

// ---------------------------------------------------------------------------
// paged KV: gather and decode
// ---------------------------------------------------------------------------
int32_t b200fa_paged_kv_gather(const void* pool, const int32_t* block_table, const int32_t* seq_lens,
                               int32_t B, int32_t H, int32_t D, int32_t eb, int32_t block_size,
                               int32_t max_blocks, int32_t max_kv_len, void* out, void* stream) {
  if (B < 0 || H <= 0 || D <= 0 || block_size <= 0 || max_blocks < 0 || max_kv_len < 0)
    return fail(B200FA_ERR_INVALID_ARG, "bad extent");
  if (eb != 1 && eb != 2 && eb != 4) return fail(B200FA_ERR_INVALID_ARG, "elem_bytes must be 1, 2 or 4");
  if ((D * eb) % 16 != 0) return fail(B200FA_ERR_INVALID_ARG, "D*elem_bytes must be a multiple of 16");
  if (B == 0 || max_kv_len == 0) return B200FA_OK;
  if (!pool || !block_table || !seq_lens || !out) return fail(B200FA_ERR_INVALID_ARG, "null pointer");
  if (!aligned16(pool) || !aligned16(out)) return fail(B200FA_ERR_INVALID_ARG, "pool/out must be 16-byte aligned");
  if (static_cast<int64_t>(max_blocks) * block_size < max_kv_len)
    return fail(B200FA_ERR_INVALID_ARG, "max_kv_len %d exceeds max_blocks*block_size", max_kv_len);
  cudaError_t e = b200fa::launch_paged_gather(pool, block_table, seq_lens, B, H, D, eb, block_size,
                                              max_blocks, max_kv_len, out,
                                              reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "gather launch");
  return B200FA_OK;
}

int32_t b200fa_paged_kv_scatter_add(const void* grad, const int32_t* block_table, const int32_t* seq_lens, int32_t B,
                                    int32_t H, int32_t D, int32_t dtype, int32_t block_size, int32_t max_blocks,
                                    int32_t max_kv_len, void* grad_pool, void* stream) {
  if (B < 0 || H <= 0 || D <= 0 || block_size <= 0 || max_blocks < 0 || max_kv_len < 0)
    return fail(B200FA_ERR_INVALID_ARG, "bad extent");
  if (dtype != B200FA_F16 && dtype != B200FA_BF16) return fail(B200FA_ERR_UNSUPPORTED, "scatter_add: f16 / bf16 only");
  if (D % 8 != 0) return fail(B200FA_ERR_INVALID_ARG, "D must be a multiple of 8");
  if (B == 0 || max_kv_len == 0) return B200FA_OK;
  if (!grad || !block_table || !seq_lens || !grad_pool) return fail(B200FA_ERR_INVALID_ARG, "null pointer");
  if (!aligned16(grad) || !aligned16(grad_pool)) return fail(B200FA_ERR_INVALID_ARG, "grad/grad_pool must be 16-byte aligned");
  if (static_cast<int64_t>(max_blocks) * block_size < max_kv_len)
    return fail(B200FA_ERR_INVALID_ARG, "max_kv_len %d exceeds max_blocks*block_size", max_kv_len);
  cudaError_t e = b200fa::launch_paged_scatter_add(grad, block_table, seq_lens, B, H, D, dtype, block_size, max_blocks,
                                                   max_kv_len, grad_pool, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "scatter_add launch");
  return B200FA_OK;
}

int32_t b200fa_kv_append(int32_t src_dtype, int32_t pool_dtype, int32_t T, int32_t Hkv, int32_t D, int32_t block_size,
                         int64_t num_pages, const void* k_new, const void* v_new, int64_t token_stride,
                         int64_t head_stride, const int64_t* slot_mapping, void* k_pool, void* v_pool, void* k_scale,
                         void* v_scale, void* stream) {
  if (src_dtype != B200FA_F16 && src_dtype != B200FA_BF16)
    return fail(B200FA_ERR_UNSUPPORTED, "kv_append: new tokens must be f16 or bf16");
  if (pool_dtype != B200FA_F16 && pool_dtype != B200FA_BF16 && pool_dtype != B200FA_I8 && pool_dtype != B200FA_E4M3)
    return fail(B200FA_ERR_UNSUPPORTED, "kv_append: pool dtype %d not built", pool_dtype);
  if (D != 64 && D != 128) return fail(B200FA_ERR_UNSUPPORTED, "kv_append: head_dim %d not built (64, 128)", D);
  if (T < 0 || Hkv <= 0 || block_size <= 0 || num_pages < 0) return fail(B200FA_ERR_INVALID_ARG, "kv_append: bad extent");
  if (T == 0) return B200FA_OK;
  if (!k_new || !v_new || !slot_mapping || !k_pool || !v_pool) return fail(B200FA_ERR_INVALID_ARG, "kv_append: null pointer");
  const bool quant = pool_dtype == B200FA_I8 || pool_dtype == B200FA_E4M3;
  if (quant && (!k_scale || !v_scale)) return fail(B200FA_ERR_INVALID_ARG, "kv_append: 8-bit pools need k_scale and v_scale");
  // rows are read with 16-byte loads
  if (token_stride % 8 != 0 || head_stride % 8 != 0 || !aligned16(k_new) || !aligned16(v_new))
    return fail(B200FA_ERR_INVALID_ARG, "kv_append: k_new/v_new rows must be 16-byte aligned");
  if (!aligned16(k_pool) || !aligned16(v_pool)) return fail(B200FA_ERR_INVALID_ARG, "kv_append: pools must be 16-byte aligned");
  cudaError_t e = b200fa::launch_kv_append(src_dtype, pool_dtype, D, k_new, v_new, token_stride, head_stride, slot_mapping,
                                           k_pool, v_pool, k_scale, v_scale, T, Hkv, num_pages * block_size,
                                           reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "kv_append launch");
  return B200FA_OK;
}

int32_t b200fa_rope(int32_t dtype, int32_t B, int32_t H, int32_t N, int32_t D, int32_t rotary_dim, int32_t interleaved,
                    int32_t inverse, const void* x, const int64_t* x_strides, void* out, const int64_t* out_strides,
                    const float* cos_table, const float* sin_table, int32_t max_pos, const int32_t* offsets, int32_t offset,
                    void* stream) {
  if (dtype != B200FA_F16 && dtype != B200FA_BF16) return fail(B200FA_ERR_UNSUPPORTED, "rope: f16 / bf16 only");
  if (B < 0 || H <= 0 || N < 0 || D <= 0 || D % 8 != 0) return fail(B200FA_ERR_INVALID_ARG, "rope: bad extent (D must be a multiple of 8)");
  if (rotary_dim <= 0 || rotary_dim > D || rotary_dim % 2 != 0)
    return fail(B200FA_ERR_INVALID_ARG, "rope: rotary_dim %d must be even and in (0, D]", rotary_dim);
  if (!interleaved && rotary_dim % 16 != 0)
    return fail(B200FA_ERR_UNSUPPORTED, "rope: split-half mode needs rotary_dim to be a multiple of 16");
  if ((D - rotary_dim) % 8 != 0 && !interleaved) return fail(B200FA_ERR_UNSUPPORTED, "rope: D - rotary_dim must be a multiple of 8");
  if (B == 0 || N == 0) return B200FA_OK;
  if (!x || !out || !cos_table || !sin_table || !x_strides || !out_strides) return fail(B200FA_ERR_INVALID_ARG, "rope: null pointer");
  if (!aligned16(x) || !aligned16(out)) return fail(B200FA_ERR_INVALID_ARG, "rope: x and out must be 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    if (x_strides[i] % 8 != 0 || out_strides[i] % 8 != 0) return fail(B200FA_ERR_INVALID_ARG, "rope: strides must be multiples of 8 elements");
  if (offsets == nullptr && (offset < 0 || static_cast<int64_t>(offset) + N > max_pos))
    return fail(B200FA_ERR_INVALID_ARG, "rope: positions [%d, %d) exceed the table's %d rows", offset, offset + N, max_pos);
  cudaError_t e = b200fa::launch_rope(dtype, x, out, cos_table, sin_table, offsets, offset, B, H, N, D, rotary_dim,
                                      interleaved ? 1 : 0, inverse ? 1 : 0, x_strides, out_strides,
                                      reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "rope launch");
  return B200FA_OK;
}

int32_t b200fa_kernel_status(void* stream, int32_t* status_out) {
  if (status_out == nullptr) return fail(B200FA_ERR_INVALID_ARG, "status_out is null");
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  int a = 0, b = 0;
  int c = 0, dd = 0;
  cudaError_t e = b200fa::fwd_sm100_read_clear_status(cs, &a);
  if (e == cudaSuccess) e = b200fa::bwd_sm100_read_clear_status(cs, &b);
  if (e == cudaSuccess) e = b200fa::bwd_dkv_sm100_read_clear_status(cs, &c);
  if (e == cudaSuccess) e = b200fa::bwd_dq_sm100_read_clear_status(cs, &dd);
  if (e != cudaSuccess) return cuda_fail(e, "kernel status read");
  *status_out = a | b | c | dd;
  return B200FA_OK;
}

int32_t b200fa_workspace_status(const void* workspace, void* stream, int32_t* status_out) {
  if (workspace == nullptr || status_out == nullptr) return fail(B200FA_ERR_INVALID_ARG, "null pointer");
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  int32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, cs);
  if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
  if (e != cudaSuccess) return cuda_fail(e, "workspace status read");
  *status_out = word;
  return B200FA_OK;
}

static int32_t decode_check(const b200fa_desc* d) {
  if (d == nullptr) return fail(B200FA_ERR_INVALID_ARG, "descriptor is null");
  if (d->dtype != B200FA_F16 && d->dtype != B200FA_BF16)
    return fail(B200FA_ERR_UNSUPPORTED, "paged decode takes f16 or bf16 queries");
  if (d->D != 128 && d->D != 64) return fail(B200FA_ERR_UNSUPPORTED, "paged decode is built for head_dim 64 and 128");
  if (d->D == 64 && d->kv_dtype != d->dtype)
    return fail(B200FA_ERR_UNSUPPORTED, "paged decode at head_dim 64 takes 16-bit pools (8-bit pools: head_dim 128)");
  if (d->B < 0 || d->Hq <= 0 || d->Hkv <= 0 || d->N <= 0)
    return fail(B200FA_ERR_INVALID_ARG, "bad extent");
  if (d->Hq % d->Hkv != 0)
    return fail(B200FA_ERR_INVALID_ARG, "q_heads (%d) must be divisible by kv_heads (%d)", d->Hq, d->Hkv);
  if ((d->Hq / d->Hkv) * d->N > 8)
    return fail(B200FA_ERR_UNSUPPORTED, "paged decode takes (Hq/Hkv)*N <= 8 query rows per kv head");
  const int kv = d->kv_dtype;
  if (!(kv == d->dtype || kv == B200FA_I8 || kv == B200FA_E4M3))
    return fail(B200FA_ERR_UNSUPPORTED, "kv_dtype must equal dtype or be int8 / e4m3");
  if (d->window_left >= 0) return fail(B200FA_ERR_UNSUPPORTED, "window is not supported in paged mode");
  return B200FA_OK;
}

size_t b200fa_decode_paged_workspace_bytes(const b200fa_desc* d, int32_t max_kv_len) {
  if (d == nullptr) return 0;
  return b200fa::decode_workspace_bytes(d->B, d->Hq, d->Hkv, d->N, d->D, max_kv_len, d->num_splits);
}

int32_t b200fa_decode_paged(const b200fa_desc* d, const void* q, const void* k_pool, const void* v_pool,
                            const void* k_scale, const void* v_scale, const int32_t* block_table,
                            const int32_t* seq_lens, int32_t num_pages, int32_t block_size,
                            int32_t max_blocks, int32_t max_kv_len, void* out, float* lse,
                            void* workspace, size_t workspace_bytes, void* stream) {
  int32_t st = decode_check(d);
  if (st != B200FA_OK) return st;
  if (block_size < 16 || block_size % 16 != 0)
    return fail(B200FA_ERR_UNSUPPORTED, "paged decode takes pages of 16, 32, 48, 64, ... tokens (a multiple of 16), got %d", block_size);
  if (num_pages <= 0 || max_blocks <= 0 || max_kv_len < 0) return fail(B200FA_ERR_INVALID_ARG, "bad extent");
  if (d->B == 0) return B200FA_OK;
  if (!q || !k_pool || !v_pool || !block_table || !seq_lens || !out)
    return fail(B200FA_ERR_INVALID_ARG, "null tensor pointer");
  const bool quant = d->kv_dtype == B200FA_I8 || d->kv_dtype == B200FA_E4M3;
  if (quant && (!k_scale || !v_scale)) return fail(B200FA_ERR_INVALID_ARG, "quantized pools need k_scale and v_scale");
  if (!aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool) || !aligned16(out) ||
      (quant && (!aligned16(k_scale) || !aligned16(v_scale))))
    return fail(B200FA_ERR_INVALID_ARG, "tensors must be 16-byte aligned");
  if (static_cast<int64_t>(max_blocks) * block_size < max_kv_len)
    return fail(B200FA_ERR_INVALID_ARG, "max_kv_len %d exceeds max_blocks*block_size", max_kv_len);
  const size_t need = b200fa::decode_workspace_bytes(d->B, d->Hq, d->Hkv, d->N, d->D, max_kv_len, d->num_splits);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(B200FA_ERR_WORKSPACE, "decode needs %zu workspace bytes, got %zu", need, workspace_bytes);
  if (!aligned16(workspace)) return fail(B200FA_ERR_INVALID_ARG, "workspace must be 16-byte aligned");
  b200fa::DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.k_scale = k_scale; p.v_scale = v_scale;
  p.block_table = block_table; p.seq_lens = seq_lens; p.out = out; p.lse = lse;
  p.workspace = workspace;
  p.B = d->B; p.Hq = d->Hq; p.Hkv = d->Hkv; p.Nq = d->N; p.D = d->D;
  p.num_pages = num_pages; p.block_size = block_size; p.max_blocks = max_blocks; p.max_kv_len = max_kv_len;
  p.q_dtype = d->dtype; p.kv_dtype = d->kv_dtype;
  p.scale = d->scale; p.softcap = d->softcap; p.causal = d->causal ? 1 : 0;
  p.num_splits = d->num_splits;
  p.packed_f32 = (d->flags & B200FA_FLAG_PACKED_F32) ? 1 : 0;
  char msg[256] = "";
  cudaError_t e = b200fa::launch_decode_paged(p, reinterpret_cast<cudaStream_t>(stream), msg, sizeof(msg));
  if (e == cudaErrorNotSupported) return fail(B200FA_ERR_UNSUPPORTED, "decode: %s", msg);
  if (e != cudaSuccess) return fail(B200FA_ERR_CUDA, "decode launch: %s %s", cudaGetErrorString(e), msg);
  return B200FA_OK;
}

}  // extern "C"
