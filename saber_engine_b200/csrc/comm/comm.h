// Peer-memory communication: symmetric-heap helpers (CUDA IPC) and the one-shot all-reduce family.
//
// Every rank allocates the same regions at the same offsets of its own heap and maps every peer's
// heap; kernels then store straight into peers over NVLink and signal with system-scope flags.
// Sequence numbers instead of toggling bits: each collective call site of a program has a static
// index, the rank keeps one device word `seq_base` that advances by the program's site count at
// the end of every program run, and a call's sequence is seq_base + site + 1.  Ranks run the same
// programs in the same order, so sequences agree without any host exchange, receive slots are
// double-buffered by sequence parity, and every flag wait is bounded (error word, no hang).
//
// Parity: the reference's 2-rank one-shot push all-reduce with parity slots and bounded spins
// (crates/saber-kernels/hip/sar_exact.h:1-10, sar_prims.h:78-120) and its global-parity form
// (flashnext_ar_gp.hip:1-8), generalised to 8 ranks over NVSwitch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

constexpr int kMaxRanks = 8;
constexpr int kArBlocks = 32;   // fixed grid of the stand-alone all-reduce: flags are per block

struct AllReduceParams {
  const __nv_bfloat16* in;      // [n_elems] this rank's partial
  __nv_bfloat16* out;           // [n_elems] reduced result (may alias in)
  void* peer_recv[kMaxRanks];   // each rank's receive region: [2][nranks][max_elems] bf16
  uint32_t* peer_flags[kMaxRanks];  // each rank's flag region: [2][nranks][kArBlocks]
  const uint32_t* seq_base;     // this rank's sequence base (device word)
  uint32_t* err;
  int n_elems, max_elems, site, nranks, rank;
  uint32_t spin_limit_us;       // 0 = default bound
  // checked twin only (the served kernel reads none of these):
  uint32_t* diag;               // [kArDiagWords] LOCAL words the peers never write (see kArD* below)
  int chk_fault;                // test control: 1 = this rank pushes its payload but no check word
};

// Race check of the all-reduce (the checked twin computes the served bytes and, beside them, these
// counters).  The sender XORs a position- and sequence-keyed hash of every 16-byte word it pushes into
// one check word per block at the TAIL of the peer's slot (the last kArBlocks words of a slot: a
// checked message must leave them free); the receiver hashes what it READ after the flag and
// compares.  A mismatch is a read of data the peer had not landed: it is counted, its first (sequence,
// block, source) is kept, and the piece is re-read at system scope for at most kArProbeMax polls to
// tell "landed late" (converges) from "another call's data" (never).  The re-read is a diagnostic only.
constexpr int kArDiagWords = 16;
constexpr int kArProbeMax = 256;
constexpr int kArDBlocks = 0, kArDMismatch = 1, kArDConverged = 2, kArDNever = 3, kArDAhead = 4, kArDDrift = 5,
              kArDTimeout = 6, kArDFirstSeq = 8, kArDFirstBlock = 9, kArDFirstSrc = 10, kArDPolls = 11, kArDLastSeq = 12;

// Sampling on vocabulary-sharded ranks: every rank holds the 64 best (value, id) of its shard per head
// row and the row's two log-sum-exps; the ranks swap them through peer windows and each merges the
// union to the global best 64 (value desc, id asc) and the global log-sum-exps, in place.  The device
// draw then runs on identical candidates on every rank.
constexpr int kSeamWords = 64 * 2 + 2;            // ids | value bits | two lse words, per row
struct SeamMergeParams {
  int32_t* ids;                 // [rows][64] in: this shard's candidates (global ids), out: the merged ones
  float* vals;                  // [rows][64]
  float* lse;                   // [rows][2]
  void* peer_win[kMaxRanks];    // each rank's window: [2][nranks][rows_max][kSeamWords] words
  uint32_t* peer_flags[kMaxRanks];  // each rank's flags: [2][nranks]
  const uint32_t* seq_base;
  uint32_t* err;
  int rows, rows_max, site, nranks, rank;
};
struct SeamEmulParams {         // test form: all ranks of a one-device group in ONE cooperative launch
  SeamMergeParams r[kMaxRanks];
  int nranks;
};

struct ArEmulParams {           // test form: every rank of a one-device group in ONE cooperative launch
  AllReduceParams r[kMaxRanks];
  int nranks, checked;
};

// Vocab-parallel head: every rank holds (value, id) of its shard's best token per row; the ranks
// swap them through peer windows and each keeps the global winner (value desc, id asc).
struct PickMergeParams {
  int32_t* idx;                 // [rows] in: local pick (global id), out: winner
  float* val;                   // [rows] in: local value, out: winner's value
  void* peer_win[kMaxRanks];    // each rank's window: [2][nranks][rows_max] x 8 bytes
  uint32_t* peer_flags[kMaxRanks];  // each rank's flags: [2][nranks]
  const uint32_t* seq_base;
  uint32_t* err;
  int rows, rows_max, site, nranks, rank;
};

}  // namespace saber

extern "C" int saber_pick_merge_launch(const saber::PickMergeParams* p, cudaStream_t stream);
extern "C" int saber_allreduce_launch(const saber::AllReduceParams* p, cudaStream_t stream);
extern "C" int saber_seam_merge_launch(const saber::SeamMergeParams* p, cudaStream_t stream);
extern "C" int saber_seam_merge_emul_launch(const saber::SeamEmulParams* p, cudaStream_t stream);
extern "C" int saber_allreduce_chk_launch(const saber::AllReduceParams* p, cudaStream_t stream);
extern "C" int saber_allreduce_emul_launch(const saber::ArEmulParams* p, cudaStream_t stream);
extern "C" int saber_comm_advance_launch(uint32_t* seq_base, uint32_t by, cudaStream_t stream);
extern "C" int saber_ipc_get_handle(void* dev_ptr, void* out_handle_64);
extern "C" int saber_ipc_open_handle(const void* handle_64, void** out_ptr);
extern "C" int saber_ipc_close(void* ptr);
extern "C" int saber_dev_malloc(void** out, size_t bytes);
extern "C" int saber_dev_free(void* p);
