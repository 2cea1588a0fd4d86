// Launch interface of the paged GQA attention kernels (RMSNorm+RoPE+KV append, attention, combine).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

constexpr int kHeadDim = 256;
constexpr int kPageTokens = 16;

struct RopeKvParams {
  __nv_bfloat16* qkv;          // [M][ld]: q heads at q_off, k heads at k_off, v heads at v_off
  __nv_bfloat16* q_out;        // [M][nq][256] normalised + rotated queries
  const float* q_norm_w;       // [256]
  const float* k_norm_w;       // [256]
  const int32_t* pos;          // [3][M] (t, h, w) positions; text rows carry t = h = w
  const int32_t* slot_map;     // [M] physical token slot (block * 16 + offset), < 0 = skip the write
  uint8_t* kv_cache;           // fp8 e4m3 [nblocks][nkv][2][16][256]
  int M, ld, nq, nkv, q_off, k_off, v_off;
  int rot_dim;                 // rotary dims (64), rotate-half pairing inside them
  int sec_h, sec_w;            // interleaved M-RoPE section sizes of the h and w axes
  float theta, eps, w_offset;  // w_offset = 1 for (1 + w)
  float k_inv_scale, v_inv_scale;  // stored = value * inv_scale
  // Byte order inside a 4 KiB page.  0: [16 tokens][256 dims].  1: the order the tcgen05 attention
  // multiplies in place (core matrices of 8 rows x 16 bytes): K [2 key groups][16 dim chunks][8 keys][16 dims],
  // V [32 dim groups][8 dims][16 keys].
  int page_layout;
};

struct AttnParams {
  const __nv_bfloat16* q;      // [M][nq][256]
  const uint8_t* kv_cache;     // [nblocks][nkv][2][16][256] fp8
  const int32_t* block_table;  // [nseq][max_blocks]
  const int32_t* cu_q;         // [nseq + 1]
  const int32_t* kv_len;       // [nseq] keys visible to the LAST row of the sequence (rows included)
  __nv_bfloat16* out;          // [M][nq][256]
  float* part_o;               // [nseq][nq][splits][16][256]
  float* part_ml;              // [nseq][nq][splits][16][2]
  int nseq, nq, nkv, max_blocks, splits, q_tiles;
  float sm_scale, k_scale, v_scale;
  uint32_t* err;               // status word of the bounded waits (may be null)
  int pack_rows;               // decode: upper bound of the rows of one sequence (1..8 packs heads into a tile; 0 = off)
  int n_blocks;                // blocks in kv_cache (0 = unknown): a table entry outside [0, n_blocks) is
                               // recorded in the status word and its page is treated as empty
  int impl;                    // 0: warp-level MMA kernel on [16][256] pages; 1: tcgen05 kernel on core-matrix pages
  int window;                  // > 0: sliding window -- a row sees its last `window` keys only (tcgen05 kernel); 0: all
};

}  // namespace saber

extern "C" int saber_rope_kv_launch(const saber::RopeKvParams* p, cudaStream_t stream);
extern "C" int saber_attn_launch(const saber::AttnParams* p, cudaStream_t stream);
extern "C" int saber_attn_tc_launch(const saber::AttnParams* p, cudaStream_t stream);
