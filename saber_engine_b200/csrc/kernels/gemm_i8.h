// Launch interface of the integer (W4A8 / W8A8) tcgen05 GEMM. Plain C types only so that both the
// torch binding and C callers can use it.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

constexpr int kTpMaxTiles = 512;   // flag words per (parity, source rank): one per (m tile, n tile)

struct GemmI8Params {
  const uint8_t* w;        // pre-tiled weights [N_pad/128][K/128][8 KiB (W4) | 16 KiB (W8)]
  const float* w_scale;    // [N] per output feature; for W4 it already carries the 1/16
  const int8_t* a;         // pre-tiled activations [K/128][M_pad][128]
  const float* a_scale;    // [M_pad] per token
  __nv_bfloat16* out;      // [M][ldo]
  int32_t* ws;             // split-K scratch [splits][M_pad][N_pad] int32 (contents do not persist)
  uint32_t* counters;      // split-K arrival counters, one per (m tile, n tile), zero between launches
  uint32_t* err;           // status word: 0, or the code of the first bounded wait that ran out
  int M, M_pad, N, N_pad, K;
  int nt;                  // tokens per CTA tile: multiple of 16, <= 256, divides M_pad
  int splits;              // split-K factor (gridDim.z)
  int w4;                  // 0: int8 tiles, 1: packed int4, 2: MXFP4, 3: bf16 x bf16 (both operands bf16, K counted in bytes)
  int ldo;                 // row stride of out, in elements
  int dbg_mma;             // debugging only: MMAs issued per k-block (0 = all four)
  // Tensor-parallel fused epilogue (tp_nranks > 1): the finished tile is not written to `out`
  // but pushed, as bf16 partial sums, into EVERY rank's receive region over NVLink, followed by
  // one release flag per (destination, tile); the consumer kernel of the next op waits on the
  // flags and adds the partials in rank order.
  void* tp_recv[8];        // each rank's receive region: [2 parity][nranks src][tp_rows][tp_ld] bf16
  uint32_t* tp_flags[8];   // each rank's flag region:    [2 parity][nranks src][kTpMaxTiles]
  const uint32_t* tp_seq_base;
  int tp_nranks, tp_rank, tp_site, tp_rows, tp_ld;
  // Sequence-parallel forms.  tp_rpr > 0: reduce-scatter -- a row's partial sums go ONLY to the rank
  // that owns the row (owner = row / tp_rpr; tp_rpr is a multiple of the token tile) and only that
  // rank's flags are raised.  ag_flags != null: all-gather fused into the operand load -- the token
  // rows of this GEMM were written into local memory by their owners (the add-norm-quant kernel of
  // every rank pushes its rows to all ranks); the producer warp waits (bounded) for the arrival flag
  // of its 128-row tile before it issues the first token-tile copy.
  int tp_rpr;
  const uint32_t* ag_flags;      // THIS rank's arrival flags [2 parity][64 row tiles]
  const uint32_t* ag_seq_base;
  int ag_site;
  // Grouped (mixture-of-experts) mode, group_tiles != null: blockIdx.y walks a device-built tile
  // table {expert, first row, live rows, 0}; rows are the expert-major sorted token rows.  CTAs
  // beyond *group_ntiles leave at once, so the grid is static (graph-capturable) and sized for the
  // worst case.  Weights / scales of expert e start at w + e * group_w_stride / w_scale + e * N_pad.
  const int4* group_tiles;
  const int* group_ntiles;
  unsigned long long group_w_stride;
  // split-K reduction mode. Callers leave 0 (the launcher turns the cooperative form on when the
  // whole grid is resident) or set -1 to force the last-arriver form.
  int coop;
  // token tiles per CTA, chosen by the launcher (callers leave 0; 2 asks for pairs whenever the shape
  // allows, -1 forbids them): 2 for long row runs (prefill) of
  // 4-bit weights -- one widened weight block then feeds two 128-row MMAs with their own TMEM
  // accumulators, which halves the widening work per output.
  int mtiles;
  unsigned long long* dbg; // optional: 16 global-timer stamps of CTA (0,0,0) (null = off)
  // bf16 mode (w4 == 3; splits == 1): operands are bf16 in the same byte tiling (a 128-byte row of a
  // k-block holds 64 values; K is the reduction length in BYTES), fp32 accumulation, scales optional
  // (null = 1).  y = bf16(acc + bias[n]); then epi 1: gelu_tanh(y), 2: gelu_erf(y), 3: y + res[m][n]
  // (res has out's row stride and may alias out), each rounded to bf16 once more.
  const float* bias;           // [N] or null
  const __nv_bfloat16* res;    // epi 3
  int epi;
};

}  // namespace saber

extern "C" int saber_gemm_i8_smem_bytes(int nt, int stages);
extern "C" int saber_gemm_i8_smem_bytes_w(int nt, int stages, int w4);
extern "C" int saber_gemm_i8_parts(const saber::GemmI8Params* p);
extern "C" int saber_gemm_i8_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream);
