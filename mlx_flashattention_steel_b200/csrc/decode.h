// Parameters and launcher of the paged split-KV decode kernel.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200fa {

struct DecodeParams {
  const void* q;            // [B, Hq, Nq, D] contiguous, f16 or bf16
  const void* k_pool;       // [num_pages, block_size, Hkv, D] kv_dtype
  const void* v_pool;
  const void* k_scale;      // [num_pages, block_size, Hkv] f16 (8-bit pools)
  const void* v_scale;
  const int32_t* block_table;  // [B, max_blocks]; null = dense caches (see `dense`)
  const int32_t* seq_lens;     // [B]; null = every sequence holds max_kv_len tokens
  void* out;                // [B, Hq, Nq, D] q dtype
  float* lse;               // [B, Hq, Nq] or null
  void* workspace;
  int B, Hq, Hkv, Nq, D;
  int num_pages, block_size, max_blocks, max_kv_len;
  int q_dtype, kv_dtype;
  float scale, softcap;
  int causal;
  int num_splits;           // upper bound on CTAs per head group; 0 = one per SM
  // Dense caches: k_pool / v_pool are [B, Hkv, S, D] tensors with these strides (elements; D contiguous), S =
  // max_kv_len; "page" j of sequence b is its tokens [16 j, 16 j + 16), no table is read.
  int dense;
  int64_t k_bs, k_hs, k_rs, v_bs, v_hs, v_rs;
  // Partial results for a combine across GPUs: `out` is float [B * Hq * Nq][D + 4] -- the normalised row in fp32
  // with its base-2 lse at column D (columns D + 1 .. D + 3 pad the row to 16 bytes) -- and `lse` is ignored.
  int packed_f32;
};

// gathered: [R][rows][D + 4] packed partials (see DecodeParams::packed_f32) -> out [rows][D] (dtype 0 f16 / 1 bf16),
// lse [rows] (may be null): L = log2 sum_r 2^lse_r, O = sum_r 2^(lse_r - L) O_r.
cudaError_t launch_combine_partials(const float* gathered, int R, long long rows, int D, int out_dtype, void* out,
                                    float* lse, cudaStream_t stream);

size_t decode_workspace_bytes(int B, int Hq, int Hkv, int Nq, int D, int max_kv_len, int num_splits);
cudaError_t launch_decode_paged(const DecodeParams& p, cudaStream_t stream, char* msg, size_t msg_len);

}  // namespace b200fa
