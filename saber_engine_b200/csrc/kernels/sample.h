// Launch interface of the head-side kernels (argmax, top-k seam, verify/accept).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

constexpr int kSeamK = 64;

struct VerifyParams {
  const int32_t* draft;     // [M] token fed at each row (row 0 of a sequence = last committed token)
  const int32_t* target;    // [M] model pick after each row
  const int32_t* cu_rows;   // [nseq + 1]
  const int32_t* seq_uid;   // [nseq] stable id of the sequence (seeds the oracle)
  const int32_t* step_no;   // [nseq] decode step index of the sequence (seeds the oracle)
  int32_t* n_commit;        // [nseq] tokens committed this step (accepted drafts + 1 bonus)
  int32_t* out_tokens;      // [nseq][max_w]
  int32_t* accept_row;      // [nseq] global row index of the last committed row (may be null)
  int32_t* bonus;           // [nseq] the bonus token, i.e. the next step's first row (may be null)
  int nseq, max_w;
  float oracle_p;           // 0: greedy prefix match; > 0: seeded geometric(p) acceptance
  uint64_t seed;
};

// Index tables of the drafter's block rows (the drafter's attention layers): block row j of sequence b sits at the
// position that follows the last committed row of the step by j + 1 tokens.
struct DraftIndexParams {
  const int32_t* pos;          // [3][M] rope positions of the step's rows
  const int32_t* cu_rows;      // [nseq + 1]
  const int32_t* kv_len;       // [nseq] tokens of the sequence after this step's rows
  const int32_t* acc_row;      // [nseq] global row index of the last committed row
  const int32_t* block_table;  // [nseq][max_blocks]
  int32_t* pos_out;            // [3][nseq * block]
  int32_t* slot_out;           // [nseq * block] KV slot of the block row (-1: none)
  int32_t* kv_len_out;         // [nseq] context + block rows, what the block's attention sees
  int M, nseq, block, max_blocks, page_tokens;
};

}  // namespace saber

extern "C" int saber_draft_index_launch(const saber::DraftIndexParams* p, cudaStream_t stream);

extern "C" int saber_argmax_launch(const void* logits, int rows, int ld, int V, int id_offset,
                                   int32_t* out_idx, float* out_val, cudaStream_t stream);
extern "C" int saber_topk_seam_launch(const void* logits, int rows, int ld, int V, int id_offset,
                                      const float* temps, int32_t* ids, float* vals, float* lse,
                                      cudaStream_t stream);
extern "C" int saber_verify_launch(const saber::VerifyParams* p, cudaStream_t stream);
extern "C" int saber_sample_seam_launch(const int32_t* ids, const float* vals, const float* samp, const float* u,
                                        int32_t* picks, int rows, cudaStream_t stream);
extern "C" int saber_logit_gather_launch(const void* logits, int rows, int ld, int V, int id_offset,
                                         const int32_t* ids, float* out, cudaStream_t stream);
