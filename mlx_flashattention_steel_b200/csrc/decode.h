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
};

size_t decode_workspace_bytes(int B, int Hq, int Hkv, int Nq, int D, int max_kv_len, int num_splits);
cudaError_t launch_decode_paged(const DecodeParams& p, cudaStream_t stream, char* msg, size_t msg_len);

}  // namespace b200fa
