// Launch interface of the mixture-of-experts routing kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

constexpr int kMoeMaxTopK = 16;

struct MoeRouteParams {
  const __nv_bfloat16* logits;   // [M][ld] router logits
  int32_t* topk_id;              // [M][top_k]
  float* topk_w;                 // [M][top_k] renormalised probabilities
  int32_t* counts;               // [E_local] routes per local expert (zeroed by plan at the end of its run)
  int32_t* offsets;              // [E_local + 1] first padded row of each expert
  int32_t* cursors;              // [E_local] placement cursors
  int4* tiles;                   // tile table for the grouped GEMM
  int32_t* ntiles;               // [2]: live tiles, total padded rows
  int32_t* src_row;              // [rows_cap] token row of every sorted row (-1 = padding)
  int32_t* slot_of;              // [M][top_k] sorted row of every route (-1 = expert lives elsewhere)
  int M, ld, E, top_k, nt, rows_cap;
  int e_lo, e_n;                 // this rank's experts are [e_lo, e_lo + e_n)
  int norm_topk;
};

struct MoeCombineParams {
  const __nv_bfloat16* y;        // [rows_cap][H] expert outputs in sorted order
  const __nv_bfloat16* shared;   // [M][H] shared-expert output (may be null)
  const __nv_bfloat16* shared_gate;  // gate logit of row m at shared_gate[m * ldg] (null: factor 1)
  const float* topk_w;
  const int32_t* slot_of;
  __nv_bfloat16* out;            // [M][H] (not written in push mode)
  int M, H, top_k, nt, ldg;
  // push mode (tp_nranks > 1): this rank's sums go to every rank's receive region with the same
  // slot / flag protocol as the row-parallel GEMM epilogue; the next add-norm sums the ranks
  void* tp_recv[8];
  uint32_t* tp_flags[8];
  const uint32_t* tp_seq_base;
  int tp_nranks, tp_rank, tp_site, tp_rows, tp_ld;
};

}  // namespace saber

// Copies quantised activation rows (tiled int8 [K/128][M_pad][128] + per-row scale) into
// expert-major order: sorted row r takes token row src_row[r]; padding rows become zeros.
extern "C" int saber_moe_gather_launch(const int8_t* q, const float* scale, int M_pad, const int32_t* src_row,
                                       const int32_t* ntiles, int8_t* q_out, float* scale_out, int rows_cap,
                                       int M_pad_out, int K, int to_fp8, cudaStream_t stream);
extern "C" int saber_moe_route_launch(const saber::MoeRouteParams* p, cudaStream_t stream);
extern "C" int saber_moe_combine_launch(const saber::MoeCombineParams* p, cudaStream_t stream);
