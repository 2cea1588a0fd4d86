// Launch interface of the integer (W4A8 / W8A8) tcgen05 GEMM. Plain C types only so that both the
// torch binding and C callers can use it.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

struct RowOpParams;

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
  // ---- Fused tails (integer / MXFP4 instantiation only).  Both forms need every CTA of the grid
  // resident at the same time (one CTA per SM: grid <= SM count); the launcher refuses other shapes.
  //   1  silu(gate) * up + per-token int8 quantisation INSIDE the tile: the weight tiles are paired
  //      (rows 0-127 of tile t = gate features [128 t, 128 t + 128), rows 128-255 = the up features
  //      of the same indices), so a CTA owns whole (gate, up) pairs; the row maxima meet in
  //      tail_sync, one grid-wide barrier, then every CTA writes its 128 bytes of each row straight
  //      into the next GEMM's operand (tail_q / tail_scale).  splits must be 1; `out` is not written.
  //   2  row tail: after the output is complete (all tiles, all split-K parts) and a grid-wide
  //      barrier, the CTAs walk the rows with the row producer `tail_row_mode` on *tail_row
  //      (add + RMSNorm + quantise of the NEXT op's input, the consumer side of the tensor-parallel
  //      push included), so the row op costs no launch.
  int tail_mode;
  int tail_row_mode;
  const RowOpParams* tail_row;   // HOST pointer, copied into the launch
  int8_t* tail_q;                // mode 1: tiled int8 [N / 256][tail_M_pad][128]
  float* tail_scale;             // mode 1: [tail_M_pad]
  int tail_M_pad;
  uint32_t* tail_sync;           // device words, zero between launches: [0] barrier counter, [64 + 32 r] maximum of row r (256 rows)
  // ---- L2 prefetch of the NEXT GEMM's leading weight tiles (filled in by the step program): when
  // this CTA has issued its last copy, it asks for the first next_pref k-blocks of the CTAs
  // (tile, split) of the next launch, so that launch starts from L2 instead of cold HBM.
  const uint8_t* next_w;
  int next_tiles, next_splits, next_KB, next_kb_per, next_wbytes, next_pref;
  // ---- split-K accumulator blocks (integer formats): one block of nt x 256 int32 per (m tile, n tile),
  // ZERO between launches.  Non-null: the splits add their partial tiles into it with asynchronous
  // bulk reductions in L2 (order-free, exact) instead of keeping private copies in `ws`; the CTAs
  // that read a tile out put its block back to zero.  Null: private copies.
  int32_t* acc;
  // Blocks for launches whose row tail reads the accumulators itself (split-K + row tail on one
  // GPU): same shape, NOT zero between launches -- such a launch cleans its blocks itself.  Null:
  // the row tail reads the bf16 tile the GEMM's own read-out wrote.
  int32_t* acc_tail;
  // Half tiles (packed int4 weights, splits == 1, no tail, one GPU): halves == 2 launches two CTAs
  // per 256-row weight tile; each copies the whole packed tile but widens and multiplies only its
  // 128 rows (the low or the high nibbles).  For shapes whose tile count fills less than half of
  // the SMs this doubles the CTAs without any split-K round trip.  0 / 1 = whole tiles.
  int halves;
  // Native FP4 (w4 = 4: NVFP4, one ue4m3 scale per 16 values; w4 = 5: MXFP4, one ue8m0 per 32): `w` tiles are
  // [N_pad/256][K/256][32768 packed e2m1 bytes + scale atoms], `a` is [K/256][M_pad][128 packed bytes] and
  // `a_sf` the token scales [K/256][ceil(M_pad/128)][atoms x 512].  K counts VALUES; w_scale / a_scale carry
  // the per-tensor and per-token fp32 scales.  No tails, no tensor-parallel push, no grouped mode.
  const uint8_t* a_sf;
};

}  // namespace saber

extern "C" int saber_gemm_i8_smem_bytes(int nt, int stages);
extern "C" int saber_gemm_i8_smem_bytes_w(int nt, int stages, int w4);
extern "C" int saber_gemm_i8_parts(const saber::GemmI8Params* p);
extern "C" int saber_gemm_i8_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream);
// 1 when the launch of `p` keeps its whole grid resident (what the fused tails need), else 0.
extern "C" int saber_gemm_i8_tail_ok(const saber::GemmI8Params* p);

// int8 weights on CTA pairs (tcgen05 cta_group::2) for long row runs: gemm_w8_2sm.cu
extern "C" int saber_gemm_w8_2sm_ok(const saber::GemmI8Params* p);
extern "C" int saber_gemm_w8_2sm_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream);
extern "C" void saber_set_gemm_2sm(int on);
extern "C" int saber_get_gemm_2sm();
