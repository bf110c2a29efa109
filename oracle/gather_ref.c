/*
 * Plain-C restatement of the reference's CPU page gather.  TEST INFRASTRUCTURE ONLY.
 *
 * Follows MFAPagedKVGather::eval_cpu (csrc/mfa_paged_gather.cpp:89-129): the output
 * is zero-filled, then for every batch b, every token t < seq_lens[b] whose page
 * block_table[b, t / block_size] is non-negative, every head h and every element,
 *   out[b, h, t, :] = pool[page, t % block_size, h, :].
 * The reference indexes with 32-bit int; 64-bit offsets are used here so that pools
 * beyond 2^31 elements work.  `elem_bytes` generalises the reference's uint16 copy.
 */
#include <stdint.h>
#include <string.h>

void oracle_paged_gather(const unsigned char* pool, const int32_t* block_table, const int32_t* seq_lens,
                         int B, int H, int D, int elem_bytes, int block_size, int max_blocks,
                         int max_kv_len, unsigned char* out) {
  const int64_t row = (int64_t)D * elem_bytes;
  memset(out, 0, (size_t)B * H * max_kv_len * row);
  for (int b = 0; b < B; b++) {
    int kv_len = seq_lens[b];
    for (int t = 0; t < kv_len && t < max_kv_len; t++) {
      int log_blk = t / block_size;
      int tok_off = t % block_size;
      int phys = block_table[(int64_t)b * max_blocks + log_blk];
      if (phys < 0) continue;
      for (int h = 0; h < H; h++) {
        int64_t src = (((int64_t)phys * block_size + tok_off) * H + h) * row;
        int64_t dst = (((int64_t)b * H + h) * max_kv_len + t) * row;
        memcpy(out + dst, pool + src, (size_t)row);
      }
    }
  }
}
