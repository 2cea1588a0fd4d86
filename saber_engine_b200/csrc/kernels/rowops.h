// Launch interface of the row producers (norm / activation / gate ops with fused int8 quant).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

enum RowMode : int {
  kRowAddRms = 0,
  kRowSiluMul = 1,
  kRowGateSig = 2,
  kRowGdnNorm = 3,
  kRowPlain = 4,
};

struct RowOpParams {
  const __nv_bfloat16* a;   // primary input (x / gate|up / attn out / raw row)
  const float* a_f32;       // GDN_NORM only: fp32 primary input instead of `a`
  const __nv_bfloat16* b;   // secondary input (gate for GATE_SIG, z for GDN_NORM)
  __nv_bfloat16* res;       // ADD_RMS: residual stream, updated in place (may be null)
  const float* w;           // norm weight (K for ADD_RMS, 128 for GDN_NORM)
  float w_offset;           // 1 for the (1 + w) form, 0 for plain w
  float eps;
  __nv_bfloat16* out;       // optional bf16 copy of the produced row (may be null)
  int8_t* q;                // optional tiled int8 output [K/128][M_pad][128] (may be null)
  float* scale;             // [M_pad]
  int M, M_pad, K;
  int lda, ldb, ldres, ldout;  // row strides in elements
  // ADD_RMS as the consumer of a tensor-parallel GEMM (tp_nranks > 1): instead of reading `a`,
  // wait (bounded) for every rank's tiles of this row and add the bf16 partials in rank order.
  const __nv_bfloat16* tp_recv;   // THIS rank's receive region [2][nranks][tp_rows][tp_ld]
  const uint32_t* tp_flags;       // THIS rank's flag region    [2][nranks][kTpMaxTiles]
  const uint32_t* tp_seq_base;
  uint32_t* err;
  int tp_nranks, tp_site, tp_rows, tp_ld, tp_nt, tp_tiles_n;
  // optional device row count: blocks of rows >= *m_live leave without writing (expert-major row
  // spaces whose live length is only known on the device)
  const int32_t* m_live;
  // quantised output format: 0 = int8 (scale amax / 127), 1 = fp8 e4m3 (scale amax / 448)
  int qfmt;
  // optional rotation before the quantisation (register-resident modes only): every 32-block of the
  // row is multiplied by the signs had_sign[k] (+-1) and by the orthonormal 32-point Hadamard matrix;
  // the consuming linear's weights were rotated the same way, so the product is unchanged while
  // outliers are spread over the block.  Null = off.
  const float* had_sign;
  // Sequence-parallel ADD_RMS (sp_rpr > 0, with tp_nranks > 1): only the rows this rank owns are
  // processed (owner = row / sp_rpr); their partial sums arrive by reduce-scatter; the residual
  // stream is sharded by rows; the quantised row and its scale are stored into EVERY rank's
  // activation buffer (all-gather by peer stores), and the CTA that completes a 128-row tile
  // raises that tile's arrival flag on every rank.
  int8_t* sp_q[8];
  float* sp_scale[8];
  uint32_t* sp_flags[8];        // each rank's arrival flags [2 parity][64 row tiles]
  uint32_t* sp_counter;         // this rank's rows-done counters [64 row tiles] (zero between uses)
  int sp_rpr, sp_rank;
  // ADD_RMS: optional second copy of the updated residual row (same row stride as `res`): the
  // drafter's tap of this layer, written here instead of by a copy launch.  Null = off.
  __nv_bfloat16* res_copy;
  // SILU_MUL on the output of a PAIRED gate | up linear: gate and up of feature 128 t + c sit at
  // columns 256 t + c and 256 t + 128 + c (instead of c and K + c).
  int silu_pair;
  // ADD_RMS as the row tail of a split-K GEMM on one GPU (filled in by the GEMM launcher): the
  // primary input is not `a` but the GEMM's int32 accumulator blocks ([tile][c4][acc_nt rows][4]);
  // the row op scales and rounds them exactly as the GEMM's own read-out would
  // (bf16(acc * (a_scale[m] * w_scale[n]))).  The blocks are left as they are: a GEMM launch in
  // this mode cleans them itself before its splits add.
  int32_t* acc;
  const float* acc_a_scale;
  const float* acc_w_scale;
  int acc_nt, acc_tiles_n;
  // qfmt == 2: NVFP4 rows -- packed e2m1 [K/256][M_pad][128 bytes] in `q`, one ue4m3 scale per 16 values as
  // 512-byte atoms [K/256][sf_m_tiles][4][512] in `q_sf`, the per-token fp32 scale amax / (6 * 448) in `scale`
  uint8_t* q_sf;
  int sf_m_tiles;
};

}  // namespace saber

extern "C" int saber_row_producer_launch(int mode, const saber::RowOpParams* p, cudaStream_t stream);
extern "C" int saber_embed_gather_launch(const void* table, const int32_t* ids, void* out, int M,
                                         int H, int vocab_lo, int vocab_n, int ldout,
                                         cudaStream_t stream);
extern "C" int saber_block_expand_launch(const void* ctx, const void* tok, const void* pos, void* out,
                                         int nseq, int block, int H, cudaStream_t stream);
