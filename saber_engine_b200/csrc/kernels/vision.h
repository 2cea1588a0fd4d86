// Launch interface of the vision tower's own kernels (the tower's linears run on the tcgen05 GEMM in
// its bf16 mode, see gemm_i8.h).  Plain C types only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

// Rows -> the GEMM's bf16 token operand: [K_total_pad/64][M_pad][128 bytes], 16-byte chunks XOR-swizzled
// by (row & 7).  Optional LayerNorm (weight and bias) on the way; optional row grouping (the merger's
// view [L/4, 4*K]): source row m lands in operand row m / group at column (m % group) * K.
struct VisRowsParams {
  const void* x;           // [M][ldx] fp32 (x_f32 = 1) or bf16
  int x_f32, ldx;
  const float* ln_w;       // [K] or null: no normalisation, a cast
  const float* ln_b;       // [K]
  float eps;
  uint8_t* tiled;
  int M, K;                // K a multiple of 8
  int K_pad;               // operand columns per SOURCE row, a multiple of 64 when group == 1 (zero filled past K)
  int M_pad;               // operand rows (>= ceil(M / group), a multiple of the GEMM's token tile)
  int group;               // 1 or 4 (K a multiple of 64 when > 1)
};

// x[m][:] += sum_i table[idx[m][i]][:] * wt[m][i]   (bilinear gather of the learned position table);
// weights and products rounded to bf16, the four products added left to right in bf16.
struct VisPosAddParams {
  __nv_bfloat16* x; int ldx;
  const __nv_bfloat16* table; int ldt;
  const int* idx;          // [M][4]
  const float* wt;         // [M][4]
  int M, K;
};

// Non-causal attention inside each image; head dim 72.  The rotary kernel (in place on the q and k
// parts of qkv, before the attention kernel) takes the same block; `blocks` rows cover 64 queries.
struct VisAttnParams {
  const __nv_bfloat16* qkv; int ldq;     // [L][3 * width]: q | k | v, head-major inside each
  const float* cos_t; const float* sin_t; // [L][36]
  uint8_t* out_tiled; int M_pad;          // the projection GEMM's token operand (width columns)
  const int4* blocks;                     // per CTA row block {first row of the image, rows of the image, first query (relative), 0}
  int heads, width;
  float scale;                            // 1 / sqrt(72)
};

}  // namespace saber

extern "C" int saber_vis_rows_launch(const saber::VisRowsParams* p, cudaStream_t stream);
extern "C" int saber_vis_pos_add_launch(const saber::VisPosAddParams* p, cudaStream_t stream);
extern "C" int saber_vis_attn_launch(const saber::VisAttnParams* p, int n_blocks, cudaStream_t stream);
extern "C" int saber_vis_rope_launch(const saber::VisAttnParams* p, int rows, cudaStream_t stream);
