// Internal launcher declarations: one per kernel family.  The C-ABI layer
// (api.cu) validates arguments, picks a family and calls these.  This table of
// ahead-of-time template instances plays the role of the reference's run-time
// shader cache keyed by KernelKey (csrc/shader_cache.hpp:29-77).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200fa {

struct FwdParams;
struct BwdParams;

// dtype codes as in b200fa.h: 0 f16, 1 bf16, 2 f32.
cudaError_t launch_fwd_mma(const FwdParams& p, int dtype, int D, bool varlen, int nbatch, int max_q,
                           cudaStream_t stream);
cudaError_t launch_fwd_f32(const FwdParams& p, int D, bool varlen, int nbatch, int max_q,
                           cudaStream_t stream);

// tcgen05 / TMEM / TMA forward (dense and packed-varlen layouts, D = 64 or 128, 16-bit).
bool fwd_sm100_supported(const FwdParams& p, int dtype, int D);
cudaError_t launch_fwd_sm100(const FwdParams& p, int dtype, int D, int nbatch, int max_q, cudaStream_t stream);

// int8 / e4m3 pool + f16 scales -> f16 / bf16 dense [B, H, max_kv_len, D]
cudaError_t launch_paged_gather_dequant(const void* pool, const void* scale, const int32_t* block_table,
                                        const int32_t* seq_lens, int B, int H, int D, int pool_dtype, int out_dtype,
                                        int block_size, int max_blocks, int max_kv_len, void* out, cudaStream_t stream);
cudaError_t launch_paged_gather(const void* pool, const int32_t* block_table, const int32_t* seq_lens,
                                int B, int H, int D, int elem_bytes, int block_size, int max_blocks,
                                int max_kv_len, void* out, cudaStream_t stream);

// split: the head_dim-128 tcgen05 path (bwd_takes_split_path), which needs no dQ accumulator
size_t bwd_workspace_bytes(int B, int Hq, int N_total, int D, bool split);
bool bwd_takes_split_path(const BwdParams& p, int dtype, int D, bool allow_sm100);
// allow_sm100: let the tcgen05 kernels run where they exist (head_dim 64: one kernel plus the dQ conversion;
// head_dim 128: a dK/dV kernel and a dQ kernel); the preprocess is common to all.
cudaError_t launch_bwd(const BwdParams& p, int dtype, int D, bool varlen, int nbatch, int max_q,
                       int max_k, void* workspace, bool allow_sm100, cudaStream_t stream);
bool bwd_sm100_supported(int dtype, int D);
bool bwd_sm100_strides_ok(const BwdParams& p);
cudaError_t launch_bwd_sm100_main(const BwdParams& p, int dtype, int nbatch, int max_k, cudaStream_t stream);
// head_dim 128 (bwd_dkv_sm100.cu, bwd_dq_sm100.cu): p.delta filled, *p.work_counter zero
bool bwd_split_sm100_supported(int dtype, int D);
cudaError_t launch_bwd_dkv_sm100(const BwdParams& p, int dtype, int nbatch, int max_k, cudaStream_t stream);
cudaError_t launch_bwd_dq_sm100(const BwdParams& p, int dtype, int nbatch, int max_q, cudaStream_t stream);

// KV-cache write path (kv_append.cu): scatter T new tokens per kv head into the page pools; 8-bit pools are
// quantised per (token, head) with an f16 scale.  Strides in elements; slots[t] = page * block_size + offset.
cudaError_t launch_kv_append(int src_dtype, int pool_dtype, int D, const void* k_new, const void* v_new, int64_t token_stride,
                             int64_t head_stride, const int64_t* slots, void* k_pool, void* v_pool, void* k_scale,
                             void* v_scale, int T, int Hkv, int64_t total_slots, cudaStream_t stream);

// Transpose of the page gather for gradients (paged_gather.cu); grad_pool must be zero on entry.  dtype 0 f16, 1 bf16.
cudaError_t launch_paged_scatter_add(const void* grad, const int32_t* block_table, const int32_t* seq_lens, int B, int H,
                                     int D, int dtype, int block_size, int max_blocks, int max_kv_len, void* grad_pool,
                                     cudaStream_t stream);

// Rotary embedding pass (rope.cu).  xs / os: batch, head, row strides in elements; offsets (device, [B]) or one offset.
cudaError_t launch_rope(int dtype, const void* x, void* out, const float* cosb, const float* sinb, const int* offsets,
                        int offset, int B, int H, int N, int D, int rot, int interleaved, int inverse, const int64_t* xs,
                        const int64_t* os, cudaStream_t stream);

// Read (and clear when set) the device status word of the tcgen05 kernels of each file; they wait for `stream`.
cudaError_t fwd_sm100_read_clear_status(cudaStream_t stream, int* out);
cudaError_t bwd_sm100_read_clear_status(cudaStream_t stream, int* out);
cudaError_t bwd_dkv_sm100_read_clear_status(cudaStream_t stream, int* out);
cudaError_t bwd_dq_sm100_read_clear_status(cudaStream_t stream, int* out);

}  // namespace b200fa
