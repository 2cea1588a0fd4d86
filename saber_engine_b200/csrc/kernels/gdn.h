// Launch interface of the Gated DeltaNet step kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

struct GdnConvParams {
  const __nv_bfloat16* x;   // [M][ldx] projected q|k|v channels of this step's rows
  const float* conv_w;      // [C][4], tap 3 multiplies the current input
  __nv_bfloat16* hist;      // [nslots][hist_rows][C]: rows 0..2 committed window, 3.. this step's inputs
  const int32_t* cu_rows;   // [nseq + 1] first row of each sequence
  const int32_t* slots;     // [nseq] state slot, < 0 = padding sequence
  const int32_t* shift;     // [nseq] rows of the previous step that were accepted (0 after a commit)
  float* out;               // [M][C] conv+SiLU (+L2 norm for q,k; q also scaled)
  int C, n_q, n_k, ldx, hist_rows, commit;
  float q_scale;
  int max_rows;             // upper bound of the rows of one sequence in this step (sizes the grid)
  int dual;                 // 1: a slot holds TWO windows of hist_rows rows and a word that names the current one
                            //    ([2 * hist_rows + 1][C] per slot; see GdnStepParams); committing steps only
};

struct GdnRecParams {
  const float* qkv;         // [M][C] output of the conv kernel
  const __nv_bfloat16* ba;  // [M][ldba]: b (beta logits) at [0, HV), a (decay input) at [HV, 2 HV)
  const float* A_log;       // [HV]
  const float* dt_bias;     // [HV]
  float* state;             // [nslots][HV][128][128] committed recurrent state
  float* stash;             // [nslots][stash_rows][HV][VS][128 + 128/VS + 4]
  const int32_t* cu_rows;
  const int32_t* slots;
  const int32_t* shift;
  float* out;               // [M][HV * 128]
  int C, n_q, n_k, HV, HK, ldba, stash_rows, commit;
  int prefill_rows;         // commit mode only: 1 = use the eight-threads-per-row kernel (every shift must be 0)
  int chunk_impl;           // chunked prefill: 0 = fp32 on the CUDA cores, 1 = tensor cores (tf32 prep, tcgen05 scan)
  uint32_t* err;            // status word for waits that ran out (tensor-core scan); may be null
};

// One launch per layer and decode step: conv + recurrence + gated RMSNorm + per-token quantisation.
// Conv windows alternate between two buffers: a slot of `hist` is [2 * hist_rows + 1][C] bf16, rows
// [0, hist_rows) buffer 0, [hist_rows, 2 hist_rows) buffer 1, and the first four bytes of the last row
// hold the index of the CURRENT buffer (a step reads the current one, writes the other and flips the
// word when the sequence's last CTA is done, so no CTA reads what another one writes).
struct GdnStepParams {
  const __nv_bfloat16* x;   // [M][ldx] projected q|k|v channels
  const __nv_bfloat16* z;   // [M][ldz] gate of the output norm, HV * 128 wide
  const __nv_bfloat16* ba;  // [M][ldba] beta logits | decay inputs
  const float* conv_w;      // [C][4]
  const float* A_log;       // [HV]
  const float* dt_bias;     // [HV]
  const float* norm_w;      // [128]
  __nv_bfloat16* hist;      // [nslots][2 * hist_rows + 1][C]
  float* state;             // [nslots][HV][128][128]
  float* stash;             // [nslots][stash_rows][HV][260]
  const int32_t* cu_rows;
  const int32_t* slots;
  const int32_t* shift;
  __nv_bfloat16* hout;      // [M][HV * 128] normed, gated head outputs (scratch between the two phases)
  float* amax_part;         // [M][HV] row maxima per head
  uint32_t* tickets;        // [nseq] zero between launches
  int8_t* q;                // tiled quantised rows [HV][M_pad][128]
  float* scale;             // [M_pad]
  int C, n_q, n_k, HV, HK, ldx, ldz, ldba, hist_rows, stash_rows, M_pad, qfmt, max_rows;
  float q_scale, eps, w_offset;
};

}  // namespace saber

extern "C" int saber_gdn_conv_launch(const saber::GdnConvParams* p, int nseq, cudaStream_t stream);
extern "C" size_t saber_gdn_chunk_scratch_bytes(int max_rows, int nseq, int HV);
extern "C" int saber_gdn_chunk_launch(const saber::GdnRecParams* p, int nseq, int max_rows, float* scratch,
                                      cudaStream_t stream);
extern "C" size_t saber_gdn_chunk_tc_scratch_bytes(int max_rows, int nseq, int HV);
extern "C" int saber_gdn_chunk_tc_launch(const saber::GdnRecParams* p, int nseq, int max_rows, float* scratch,
                                         cudaStream_t stream);
extern "C" int saber_gdn_step_launch(const saber::GdnStepParams* p, int nseq, cudaStream_t stream);
extern "C" int saber_gdn_recurrent_launch(const saber::GdnRecParams* p, int nseq, int vs,
                                          cudaStream_t stream);
