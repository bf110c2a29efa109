/*
 * b200fa.h — C-ABI of libb200fa.so: flash attention for NVIDIA B200 (sm_100a).
 *
 * This is the boundary that replaces the reference's nanobind module
 * `mlx_mfa._ext` (csrc/bindings.cpp) for the attention hot path.  Each entry
 * point names the reference binding it stands in for.
 *
 * Conventions
 *   - every function is extern "C", takes plain pointers and sizes, returns an
 *     int32 status (B200FA_OK == 0, negative on error) and never throws;
 *   - all tensor pointers are DEVICE pointers; the caller owns inputs, outputs
 *     and the workspace (query its size with the *_workspace_bytes functions);
 *     nothing here allocates device memory, except where an entry point's own
 *     comment says otherwise;
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous
 *     with respect to the host and no entry point synchronises;
 *   - layouts follow the reference: q [B,Hq,N,D], k/v [B,Hkv,S,D], out like q,
 *     lse [B,Hq,N] float32; the last (D) dimension is contiguous, the other
 *     strides are given in ELEMENTS in the descriptor;
 *   - lse is base-2: lse = log2(sum_j exp(s_j)), s_j the scaled (and
 *     soft-capped, masked) score — the convention of the reference kernels
 *     (csrc/mfa_steel_fwd.cpp:630, 1208-1221) that its backward consumes;
 *   - b200fa_last_error() returns a thread-local message for the last failure.
 */
#ifndef B200FA_H_
#define B200FA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define B200FA_OK                  0
#define B200FA_ERR_INVALID_ARG    -1   /* null pointer, bad shape/stride/alignment */
#define B200FA_ERR_UNSUPPORTED    -2   /* dtype / head_dim / option not built */
#define B200FA_ERR_WORKSPACE      -3   /* workspace missing or too small */
#define B200FA_ERR_CUDA           -4   /* a CUDA runtime call failed */
#define B200FA_ERR_DEVICE         -5   /* device is not sm_100 */

/* element types */
#define B200FA_F16   0
#define B200FA_BF16  1
#define B200FA_F32   2
#define B200FA_I8    3   /* KV pools only: int8 with per-token-per-head scale */
#define B200FA_E4M3  4   /* KV pools only: fp8 e4m3 with per-token-per-head scale */

/* flags */
#define B200FA_FLAG_FORCE_MMA_SYNC  1  /* use the portable mma.sync kernels even where a tcgen05 kernel exists */
#define B200FA_FLAG_FWD_PERSISTENT  8  /* tcgen05 forward: persistent CTAs (each walks many query tiles) whatever the shape */
#define B200FA_FLAG_FWD_ONE_ITEM   16  /* tcgen05 forward: one query tile per CTA whatever the shape; without either flag the
                                          launcher chooses (persistent for large packed-sequence launches) */
#define B200FA_FLAG_PACKED_F32      4  /* b200fa_decode_paged: `out` is float [B*Hq*N][D+4], the normalised row in fp32 with
                                          its base-2 lse at column D (columns D+1..D+3 pad the row to 16 bytes); `lse` is
                                          ignored.  The per-GPU partial of a sequence whose pages are spread over several
                                          GPUs, in the form b200fa_combine_partials takes. */

/*
 * Problem descriptor.  Plays the role of MFAttention::Params + MFASteelParams
 * (csrc/mfa_attention.hpp:30-41, csrc/mfa_steel_fwd.hpp:25-54).
 * For the varlen entry points B == 1, N == total_q, S == total_k.
 */
typedef struct b200fa_desc {
  int32_t dtype;        /* B200FA_F16 | B200FA_BF16 | B200FA_F32 (q, out, dout, grads) */
  int32_t kv_dtype;     /* == dtype, or B200FA_I8 / B200FA_E4M3 for decode pools */
  int32_t B, Hq, Hkv;   /* Hq % Hkv == 0 (GQA / MQA) */
  int32_t N, S, D;      /* query rows, key rows, head dim (64 or 128; 256 for the 16-bit forward) */
  int64_t q_strides[3]; /* batch, head, row — in elements; 0,0,0 => contiguous BHND */
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t o_strides[3];
  float   scale;        /* multiplies q.k^T; reference default 1/sqrt(D) */
  float   softcap;      /* 0 = off; s = cap*tanh(s/cap) before masking */
  int32_t causal;       /* lower-right aligned: key j visible to row i iff j <= i + (S-N) */
  int32_t window_left;  /* -1 = off; key j visible iff j >= i + (S-N) - window_left */
  int32_t num_splits;   /* decode: 0 = choose automatically */
  int32_t flags;
  const float* alibi_slopes; /* NULL = off; device float32 [Hq]: slope[h] * (j - (i + S - N)) is added to the scaled
                                (and soft-capped) score of row i, key j (csrc/mfa_steel_fwd.cpp:951-970).  Dense
                                layout only, forward and backward. */
  const uint8_t* block_mask; /* NULL = off; device bytes [ceil(N/mask_bq), mask_nk]: row i sees key j only if
                                block_mask[i / mask_bq][j / mask_bk] != 0 (flash_attention_sparse,
                                mlx_mfa/attention.py:1219-1311).  Key tiles without an active block are skipped.
                                Dense layout, 16-bit, forward and backward. */
  int32_t mask_bq, mask_bk, mask_nk;
  const int32_t* kv_lens;    /* NULL = off; device int32 [B]: batch entry b attends to its first kv_lens[b] keys only
                                (clamped to [0, S]; the causal alignment follows that count).  Dense forward, f16 /
                                bf16, head_dim 64 / 128.  The reference slices each sequence to its exact length on
                                the host and launches once per sequence (mlx_mfa/attention.py:2950-2989); this is the
                                same result from one launch. */
} b200fa_desc;

typedef struct b200fa_device_info_t {
  int32_t cc_major, cc_minor, sm_count;
  int32_t smem_per_block_optin;
  int64_t total_mem;
  int32_t has_tcgen05;          /* 1 when built for and running on sm_100 */
  char    name[128];
} b200fa_device_info_t;

/* Replaces get_device_info (csrc/bindings.cpp:165-216). `device` < 0 = current. */
int32_t b200fa_device_info(int32_t device, b200fa_device_info_t* out);

const char* b200fa_last_error(void);
const char* b200fa_version(void);

/*
 * Forward, dense layout.  Replaces mfa_attention_forward (csrc/bindings.cpp:21-35)
 * and mfa_forward_with_lse (csrc/bindings.cpp:38-57); host dispatch role of
 * MFAttention::eval_gpu (csrc/mfa_attention.cpp:47-409).  `lse` may be NULL.
 * The forward kernels need no scratch: both *_fwd*_workspace_bytes queries always return 0 (they exist so that a
 * binding can treat every operator alike) and the workspace arguments are ignored.
 */
size_t  b200fa_fwd_workspace_bytes(const b200fa_desc* d);
int32_t b200fa_fwd(const b200fa_desc* d, const void* q, const void* k, const void* v,
                   void* out, float* lse, void* workspace, size_t workspace_bytes,
                   void* stream);

/*
 * Forward, packed variable-length sequences.  Replaces
 * mfa_attention_varlen_forward (csrc/bindings.cpp:320-344) /
 * MFAVarlenAttention::eval_gpu (csrc/mfa_attention.cpp:1228-1305).
 * cu_seqlens_* are device int32 [num_seqs+1]; max_seqlen_* are host ints
 * (the reference front end passes them the same way, mlx_mfa/attention.py:2399-2400).
 */
size_t  b200fa_fwd_varlen_workspace_bytes(const b200fa_desc* d, int32_t num_seqs,
                                          int32_t max_seqlen_q, int32_t max_seqlen_k);
int32_t b200fa_fwd_varlen(const b200fa_desc* d, const void* q, const void* k, const void* v,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                          int32_t num_seqs, int32_t max_seqlen_q, int32_t max_seqlen_k,
                          void* out, float* lse, void* workspace, size_t workspace_bytes,
                          void* stream);

/*
 * Backward dQ/dK/dV, dense layout.  Replaces mfa_steel_backward
 * (csrc/bindings.cpp:120-163: delta = sum(dO*O) + MFASteelBwdDQ + MFASteelBwdDKV,
 * csrc/mfa_attention.cpp:732-930).  `lse` is the forward's base-2 lse.
 * dq like q; dk, dv like k, v ([B,Hkv,S,D], summed over the GQA group).
 */
size_t  b200fa_bwd_workspace_bytes(const b200fa_desc* d);
int32_t b200fa_bwd(const b200fa_desc* d, const void* q, const void* k, const void* v,
                   const void* out, const float* lse, const void* dout,
                   void* dq, void* dk, void* dv,
                   void* workspace, size_t workspace_bytes, void* stream);

/*
 * Backward, packed variable-length sequences, one launch sequence for all
 * sequences.  Replaces the per-sequence Python loop of _varlen_bwd
 * (mlx_mfa/attention.py:2492-2521).
 */
size_t  b200fa_bwd_varlen_workspace_bytes(const b200fa_desc* d, int32_t num_seqs,
                                          int32_t max_seqlen_q, int32_t max_seqlen_k);
int32_t b200fa_bwd_varlen(const b200fa_desc* d, const void* q, const void* k, const void* v,
                          const void* out, const float* lse, const void* dout,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                          int32_t num_seqs, int32_t max_seqlen_q, int32_t max_seqlen_k,
                          void* dq, void* dk, void* dv,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * Paged-KV attention for short queries (decode), split-KV with the
 * log-sum-exp combine done inside the same launch.  Replaces
 * mfa_paged_steel_forward (csrc/bindings.cpp:367-407) and the gather +
 * per-sequence flash-decode route of flash_attention_paged
 * (mlx_mfa/attention.py:3008-3017, csrc/mfa_attention.cpp:150-288).
 *   k_pool/v_pool  [num_pages, block_size, Hkv, D] in d->kv_dtype
 *   k_scale/v_scale [num_pages, block_size, Hkv] float16, required for
 *                  B200FA_I8 / B200FA_E4M3, NULL otherwise; a stored value x
 *                  stands for float(x) * scale (dense-dequant path of
 *                  mlx_mfa/integrations/mlx_lm.py:97-110 with one group per row)
 *   block_table    int32 [B, max_blocks], -1 = no page
 *   seq_lens       int32 [B]
 *   d->N is the number of query rows per sequence, with (Hq/Hkv) * N <= 8; d->S is ignored;
 *   causal is per-sequence lower-right aligned.
 * `num_pages` bounds the block_table entries (larger ones are treated as holes and reported through the error word).
 * Slots of a sequence's last page beyond seq_lens[b] may hold anything, NaN patterns included: they are masked
 * before they reach the arithmetic.  The workspace size depends on B, Hq, Hkv, N and num_splits only; max_kv_len is
 * taken by the query so that the signature can stay when that changes.
 */
size_t  b200fa_decode_paged_workspace_bytes(const b200fa_desc* d, int32_t max_kv_len);
int32_t b200fa_decode_paged(const b200fa_desc* d, const void* q,
                            const void* k_pool, const void* v_pool,
                            const void* k_scale, const void* v_scale,
                            const int32_t* block_table, const int32_t* seq_lens,
                            int32_t num_pages, int32_t block_size, int32_t max_blocks,
                            int32_t max_kv_len,
                            void* out, float* lse,
                            void* workspace, size_t workspace_bytes, void* stream);

/*
 * Merges R partial attention results over disjoint key ranges (one per GPU, gathered by the caller -- one NCCL
 * all-gather of the packed rows): gathered is float [R][rows][D+4] in the B200FA_FLAG_PACKED_F32 form,
 * out [rows][D] in out_dtype (f16 / bf16), lse float [rows] or NULL.  L = log2 sum_r 2^lse_r,
 * O = sum_r 2^(lse_r - L) O_r: the split combine of the reference's flash-decode reduce
 * (csrc/mfa_steel_fwd.cpp:2066-2101), applied across GPUs; the reference itself is single-device.  D a multiple of 4,
 * at most 128.
 */
int32_t b200fa_combine_partials(const float* gathered, int32_t R, int64_t rows, int32_t D, int32_t out_dtype,
                                void* out, float* lse, void* stream);

/*
 * Paged-KV attention for prefill-sized queries (chunked prefill over a page pool): the forward kernel reads K / V
 * through the block table, page by page; nothing is gathered.  Replaces mfa_paged_steel_forward
 * (csrc/bindings.cpp:367-407; MFAPagedSteelForward, csrc/mfa_attention.cpp:1355-1552; kernel
 * csrc/mfa_steel_fwd.cpp:2462-3121) for the shapes b200fa_decode_paged does not take.
 *   q [B, Hq, N, D] (strides from the descriptor), k_pool / v_pool [num_pages, block_size, Hkv, D] in d->dtype
 *   (16-bit pools; 8-bit pools go through b200fa_paged_kv_gather_dequant first), block_size a multiple of 16,
 *   block_table int32 [B, max_blocks] (-1 or an entry beyond the pool = a page of zeros), seq_lens int32 [B].
 * Sequence b attends to its first seq_lens[b] tokens (at most max_kv_len); causal is lower-right aligned per
 * sequence; softcap and window_left apply; d->S is ignored.  Slots of a sequence's last page beyond seq_lens[b] must
 * hold finite values (their probabilities are zero, but the tensor core multiplies them all the same).
 * No workspace.  head_dim 64 / 128, f16 / bf16.
 */
int32_t b200fa_fwd_paged(const b200fa_desc* d, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_table, const int32_t* seq_lens, int32_t num_pages, int32_t block_size,
                         int32_t max_blocks, int32_t max_kv_len, void* out, float* lse, void* stream);

/*
 * Page gather with dequantisation: out[b,h,t,:] = out_dtype(float(pool[page, t % block_size, h, :]) * scale[page,
 * t % block_size, h]) for t < seq_lens[b] and a valid table entry, else zero -- the dense-dequant path of
 * mlx_mfa/integrations/mlx_lm.py:97-110 (mx.dequantize(..., dtype=q.dtype)) fused with the gather of
 * csrc/mfa_paged_gather.cpp:44-80.  pool_dtype B200FA_I8 / B200FA_E4M3, out_dtype B200FA_F16 / B200FA_BF16,
 * scale float16 [num_pages, block_size, H]; D a multiple of 16.
 */
int32_t b200fa_paged_kv_gather_dequant(const void* pool, const void* scale, const int32_t* block_table,
                                       const int32_t* seq_lens, int32_t B, int32_t H, int32_t D, int32_t pool_dtype,
                                       int32_t out_dtype, int32_t block_size, int32_t max_blocks, int32_t max_kv_len,
                                       void* out, void* stream);

/*
 * Paged decode for callers that cannot give it a workspace.  Same arguments and
 * result as b200fa_decode_paged minus the workspace pair.  It has no counterpart in
 * the reference, whose primitives get their scratch from MLX's allocator.
 *
 * Who needs it: a serving engine that has handed all of its device memory to the KV
 * page pool at start-up and has no allocator left to ask at decode time; a host
 * binding (cgo, JNI, a plugin ABI) that only passes the operator its input and output
 * buffers; a latency-bound step that must not run into the device-wide stall a
 * cudaMalloc/cudaFree can cause.  The split-KV partials, counters and page prefix
 * sums live instead in a 16 MiB array inside the library's device image, which every
 * GPU that loads the library holds until the process exits.
 *
 * Limits and rules:
 *   - the problem must fit: b200fa_decode_paged_workspace_bytes(d, max_kv_len) <= 16 MiB
 *     (config-4-sized decode, B=128 Hq=32 D=128, needs 4.6 MB); larger problems get
 *     B200FA_ERR_WORKSPACE with an explanatory message and run nothing;
 *   - the first call on each device looks up the array's device address (a host-side
 *     query, no allocation); make that first call outside any stream capture;
 *   - all calls on a device share the one array: two calls whose kernels can overlap
 *     on the GPU (different streams, no ordering between them) race on it — serialise
 *     them, or give the second one its own workspace through b200fa_decode_paged;
 *   - what must start from zero (counters, error word) is cleared by the call itself;
 *     the rest of the array keeps the previous call's partials and is overwritten
 *     before it is read;
 *   - it calls no cudaMalloc, cudaFree or allocating library routine.
 */
int32_t b200fa_decode_paged_static(const b200fa_desc* d, const void* q,
                                   const void* k_pool, const void* v_pool,
                                   const void* k_scale, const void* v_scale,
                                   const int32_t* block_table, const int32_t* seq_lens,
                                   int32_t num_pages, int32_t block_size, int32_t max_blocks,
                                   int32_t max_kv_len,
                                   void* out, float* lse, void* stream);

/*
 * Error word of the last b200fa_decode_paged_static call on the current device (same bits as
 * b200fa_workspace_status: 0 = ok, bit 0 = a bounded wait inside the kernel gave up and the outputs are undefined,
 * bit 1 = a block_table entry pointed beyond num_pages and was treated as a hole).  The word lives at the start of
 * the built-in scratch, whose address a caller of the static entry never sees; this reads it.  Waits for `stream`.
 * Like the static entry itself it has no counterpart in the reference and allocates nothing.
 */
int32_t b200fa_decode_paged_static_status(void* stream, int32_t* status_out);

/*
 * Transpose of b200fa_paged_kv_gather, for the backward pass through a page pool: grad [B, H, max_kv_len, D]
 * (f16 / bf16, contiguous) is added into grad_pool [num_pages, block_size, H, D], which the caller zeroes first;
 * tokens beyond seq_lens[b] and negative table entries contribute nothing, a page listed by several sequences
 * receives the sum.  Replaces _scatter_to_pool (mlx_mfa/attention.py:2878-2940).
 */
int32_t b200fa_paged_kv_scatter_add(const void* grad, const int32_t* block_table, const int32_t* seq_lens, int32_t B,
                                    int32_t H, int32_t D, int32_t dtype, int32_t block_size, int32_t max_blocks,
                                    int32_t max_kv_len, void* grad_pool, void* stream);

/*
 * KV-cache write path.  Scatters T new tokens (k_new / v_new, element (t, h, d) at t*token_stride +
 * h*head_stride + d, f16 or bf16) into page pools laid out [num_pages, block_size, Hkv, D]; token t goes to
 * slot_mapping[t] = page * block_size + offset (device int64; negative or out-of-pool entries are skipped).
 * pool_dtype F16 / BF16 stores the values (converted if the types differ); I8 / E4M3 quantises each (token, head)
 * row with scale = f16(max|x| / qmax) (qmax 127 / 448, 1 when zero), q = rne(x / scale), and writes the scale
 * to k_scale / v_scale [num_pages, block_size, Hkv] (f16) -- the pool format b200fa_decode_paged reads.
 * One launch serves any number of sequences.  Replaces the per-block concatenations of PagedKVCache.append
 * (mlx_mfa/attention.py:2642-2711); the reference has no 8-bit pool, so the quantising mode has no counterpart.
 */
int32_t b200fa_kv_append(int32_t src_dtype, int32_t pool_dtype, int32_t T, int32_t Hkv, int32_t D, int32_t block_size,
                         int64_t num_pages, const void* k_new, const void* v_new, int64_t token_stride,
                         int64_t head_stride, const int64_t* slot_mapping, void* k_pool, void* v_pool, void* k_scale,
                         void* v_scale, void* stream);

/*
 * Rotary position embedding of x [B, H, N, D] (f16 / bf16; strides in elements: batch, head, row; D contiguous) into
 * out (may be x).  cos_table / sin_table: float32 [max_pos, rotary_dim / 2]; row n of batch b uses position
 * offsets[b] + n (offsets: device int32 [B]) or offset + n when offsets is null.  interleaved != 0 rotates pairs
 * (2i, 2i+1), else (i, i + rotary_dim/2); elements beyond rotary_dim pass through; inverse != 0 applies the
 * transposed rotation (for gradients).  With a device `offsets` array the caller guarantees offsets[b] + N <= max_pos.
 * Replaces the in-kernel rotation of mfa_attention_rope_forward (csrc/bindings.cpp, csrc/mfa_steel_fwd.cpp:704-734,
 * 831-858) and _apply_rope_mlx (mlx_mfa/attention.py:2128-2210).
 */
int32_t b200fa_rope(int32_t dtype, int32_t B, int32_t H, int32_t N, int32_t D, int32_t rotary_dim, int32_t interleaved,
                    int32_t inverse, const void* x, const int64_t* x_strides, void* out, const int64_t* out_strides,
                    const float* cos_table, const float* sin_table, int32_t max_pos, const int32_t* offsets, int32_t offset,
                    void* stream);

/*
 * Reads and clears the library-wide device status word of the tcgen05 kernels
 * (forward, backward): 0 = ok, bit 0 = a bounded mbarrier wait inside a kernel
 * gave up after about a second (its outputs are then undefined).  Waits for
 * `stream`.  No counterpart in the reference, whose kernels report nothing back.
 */
int32_t b200fa_kernel_status(void* stream, int32_t* status_out);

/*
 * Reads the error word the decode kernel keeps at the start of its workspace
 * (0 = ok, bit 0 = a bounded wait inside the kernel gave up, bit 1 = a
 * block_table entry pointed beyond num_pages and was treated as a hole).
 * This is the one entry point that synchronises: it waits for `stream`.
 * No counterpart in the reference, whose kernels report nothing back.
 */
int32_t b200fa_workspace_status(const void* workspace, void* stream, int32_t* status_out);

/*
 * Page gather: out[b,h,t,:] = pool[block_table[b, t / block_size], t % block_size, h, :]
 * for t < seq_lens[b] and a non-negative table entry, else zero.  Bit-exact copy.
 * Replaces mfa_paged_kv_gather (csrc/bindings.cpp:346-364) /
 * MFAPagedKVGather (csrc/mfa_paged_gather.cpp:44-80, 89-129).
 * elem_bytes in {1,2,4}; D*elem_bytes must be a multiple of 16.
 */
int32_t b200fa_paged_kv_gather(const void* pool, const int32_t* block_table,
                               const int32_t* seq_lens,
                               int32_t B, int32_t H, int32_t D, int32_t elem_bytes,
                               int32_t block_size, int32_t max_blocks, int32_t max_kv_len,
                               void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200FA_H_ */
