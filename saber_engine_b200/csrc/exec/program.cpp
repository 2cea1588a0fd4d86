// Step program: the native executor of a decode/prefill bucket.
//
// A program is an ordered list of kernel launches whose parameter blocks (pointers, shapes,
// strides) are all fixed when the bucket is built; everything that changes from step to step
// (positions, block tables, slot ids, accepted-row counts) lives in device index buffers the
// kernels read.  The same list is therefore (a) walked eagerly, one launch per op, and (b) captured
// once into a CUDA graph and replayed with a single launch per step.  After capture the graph's
// kernel-node count must equal the launches the ops declared, so a silent extra or missing launch
// is a build error, not a performance mystery.
//
// Parity: this is the role of the reference's CapturedBucket / Launcher / BlockPlan trio
// (crates/saber-exec/src/capture.rs:13-30 asserted node counts, src/launch.rs:1-25,
// src/layer.rs:1-45), re-shaped for CUDA graphs and typed parameter blocks instead of packed
// kernarg buffers.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <string>
#include <variant>
#include <vector>

#include "../comm/comm.h"
#include "../kernels/attn.h"
#include "../kernels/gdn.h"
#include "../kernels/gemm_i8.h"
#include "../kernels/moe.h"
#include "../kernels/rowops.h"
#include "../kernels/sample.h"

extern "C" int saber_digest_launch(const void* buf, size_t bytes, unsigned long long* out, cudaStream_t stream);
extern "C" int saber_digest_clear_launch(unsigned long long* out, int n, cudaStream_t stream);

namespace {

struct OpGemm { saber::GemmI8Params p; int stages; saber::RowOpParams tail; bool has_tail; };
struct OpRow { int mode; saber::RowOpParams p; };
struct OpEmbed { const void* table; const int32_t* ids; void* out; int M, H, vocab_lo, vocab_n, ldout; };
struct OpExpand { const void* ctx; const void* tok; const void* pos; void* out; int nseq, block, H; };
struct OpAdvance { uint32_t* seq_base; uint32_t by; };
struct OpGdnConv { saber::GdnConvParams p; int nseq; };
struct OpGdnRec { saber::GdnRecParams p; int nseq, vs; };
struct OpSeamMerge { saber::SeamMergeParams p; };
struct OpGdnStep { saber::GdnStepParams p; int nseq; };
struct OpGdnChunk { saber::GdnRecParams p; int nseq, max_rows; float* scratch; };
struct OpRope { saber::RopeKvParams p; };
struct OpAttn { saber::AttnParams p; };
struct OpArgmax { const void* logits; int rows, ld, V, id_offset; int32_t* idx; float* val; };
struct OpSeam { const void* logits; int rows, ld, V, id_offset; const float* temps; int32_t* ids; float* vals; float* lse; };
struct OpVerify { saber::VerifyParams p; };
struct OpDraftIndex { saber::DraftIndexParams p; };
struct OpMemset { void* dst; int value; size_t bytes; };
struct OpCopy { void* dst; const void* src; size_t bytes; };
struct OpAllReduce { saber::AllReduceParams p; };
struct OpPickMerge { saber::PickMergeParams p; };
struct OpMoeRoute { saber::MoeRouteParams p; };
struct OpMoeCombine { saber::MoeCombineParams p; };
struct OpDigest { const void* buf; size_t bytes; unsigned long long* out; };
struct OpDigestClear { unsigned long long* out; int n; };
struct OpSampleSeam { const int32_t* ids; const float* vals; const float* samp; const float* u; int32_t* picks; int rows; };
struct OpLogitGather { const void* logits; int rows, ld, V, id_offset; const int32_t* ids; float* out; };
struct OpMoeGather { const int8_t* q; const float* scale; int M_pad; const int32_t* src_row; const int32_t* ntiles;
                     int8_t* q_out; float* scale_out; int rows_cap, M_pad_out, K, to_fp8; };

using Op = std::variant<OpGemm, OpRow, OpEmbed, OpGdnConv, OpGdnRec, OpRope, OpAttn, OpArgmax,
                        OpSeam, OpVerify, OpMemset, OpCopy, OpAllReduce, OpExpand, OpAdvance, OpPickMerge, OpMoeRoute, OpMoeCombine, OpMoeGather, OpDigest, OpDigestClear, OpGdnChunk, OpLogitGather, OpSampleSeam, OpGdnStep, OpSeamMerge, OpDraftIndex>;

struct Entry {
  Op op;
  int launches;      // kernel/memset/memcpy nodes this op contributes to a captured graph
  std::string tag;   // label for explain / tracing
};

struct Program {
  std::vector<Entry> ops;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int captured_nodes = -1;
  int last_failed_op = -1;
};

int launch(const Op& op, cudaStream_t s) {
  return std::visit(
      [&](auto&& o) -> int {
        using T = std::decay_t<decltype(o)>;
        if constexpr (std::is_same_v<T, OpGemm>) {
          if (!o.has_tail) return saber_gemm_i8_launch(&o.p, o.stages, s);
          saber::GemmI8Params q = o.p;      // the row tail's block lives in this op: point at it now
          q.tail_row = &o.tail;             // (the op list may have moved since the op was added)
          return saber_gemm_i8_launch(&q, o.stages, s);
        }
        else if constexpr (std::is_same_v<T, OpRow>) return saber_row_producer_launch(o.mode, &o.p, s);
        else if constexpr (std::is_same_v<T, OpEmbed>)
          return saber_embed_gather_launch(o.table, o.ids, o.out, o.M, o.H, o.vocab_lo, o.vocab_n, o.ldout, s);
        else if constexpr (std::is_same_v<T, OpExpand>)
          return saber_block_expand_launch(o.ctx, o.tok, o.pos, o.out, o.nseq, o.block, o.H, s);
        else if constexpr (std::is_same_v<T, OpAdvance>) return saber_comm_advance_launch(o.seq_base, o.by, s);
        else if constexpr (std::is_same_v<T, OpGdnConv>) return saber_gdn_conv_launch(&o.p, o.nseq, s);
        else if constexpr (std::is_same_v<T, OpGdnStep>) return saber_gdn_step_launch(&o.p, o.nseq, s);
        else if constexpr (std::is_same_v<T, OpGdnRec>) return saber_gdn_recurrent_launch(&o.p, o.nseq, o.vs, s);
        else if constexpr (std::is_same_v<T, OpGdnChunk>) return saber_gdn_chunk_launch(&o.p, o.nseq, o.max_rows, o.scratch, s);
        else if constexpr (std::is_same_v<T, OpRope>) return saber_rope_kv_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpAttn>) return saber_attn_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpArgmax>)
          return saber_argmax_launch(o.logits, o.rows, o.ld, o.V, o.id_offset, o.idx, o.val, s);
        else if constexpr (std::is_same_v<T, OpSeam>)
          return saber_topk_seam_launch(o.logits, o.rows, o.ld, o.V, o.id_offset, o.temps, o.ids, o.vals, o.lse, s);
        else if constexpr (std::is_same_v<T, OpVerify>) return saber_verify_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpDraftIndex>) return saber_draft_index_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpMemset>)
          return static_cast<int>(cudaMemsetAsync(o.dst, o.value, o.bytes, s));
        else if constexpr (std::is_same_v<T, OpCopy>)
          return static_cast<int>(cudaMemcpyAsync(o.dst, o.src, o.bytes, cudaMemcpyDeviceToDevice, s));
        else if constexpr (std::is_same_v<T, OpAllReduce>) return saber_allreduce_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpSeamMerge>) return saber_seam_merge_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpPickMerge>) return saber_pick_merge_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpMoeRoute>) return saber_moe_route_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpMoeCombine>) return saber_moe_combine_launch(&o.p, s);
        else if constexpr (std::is_same_v<T, OpDigest>) return saber_digest_launch(o.buf, o.bytes, o.out, s);
        else if constexpr (std::is_same_v<T, OpDigestClear>) return saber_digest_clear_launch(o.out, o.n, s);
        else if constexpr (std::is_same_v<T, OpSampleSeam>) return saber_sample_seam_launch(o.ids, o.vals, o.samp, o.u, o.picks, o.rows, s);
        else if constexpr (std::is_same_v<T, OpLogitGather>) return saber_logit_gather_launch(o.logits, o.rows, o.ld, o.V, o.id_offset, o.ids, o.out, s);
        else if constexpr (std::is_same_v<T, OpMoeGather>)
          return saber_moe_gather_launch(o.q, o.scale, o.M_pad, o.src_row, o.ntiles, o.q_out, o.scale_out, o.rows_cap,
                                         o.M_pad_out, o.K, o.to_fp8, s);
        else return static_cast<int>(cudaErrorInvalidValue);
      },
      op);
}

int add(void* h, Op op, int launches, const char* tag) {
  auto* pr = static_cast<Program*>(h);
  pr->ops.push_back(Entry{std::move(op), launches, tag ? tag : ""});
  return static_cast<int>(pr->ops.size()) - 1;
}

}  // namespace

extern "C" {

void* saber_program_create() { return new Program(); }

void saber_program_destroy(void* h) {
  auto* pr = static_cast<Program*>(h);
  if (!pr) return;
  if (pr->exec) cudaGraphExecDestroy(pr->exec);
  if (pr->graph) cudaGraphDestroy(pr->graph);
  delete pr;
}

int saber_program_add_gemm(void* h, const saber::GemmI8Params* p, int stages, const char* tag) {
  OpGemm op{*p, stages, saber::RowOpParams{}, false};
  if (p->tail_mode == 2 && p->tail_row != nullptr) {
    op.tail = *p->tail_row;
    op.has_tail = true;
    op.p.tail_row = nullptr;
  }
  return add(h, std::move(op), 1, tag);
}

// Chains the GEMMs of the program for L2 prefetch: every (non-grouped) GEMM learns where the next
// one's weight tiles start and how its grid walks them, so that its CTAs can ask L2 for the leading
// k-blocks of every CTA of that next launch once their own copies are all issued.  Call once, after
// the last op was added and before the program is run or captured.  Returns the number of links.
int saber_program_link_prefetch(void* h, int pref_bytes) {
  auto* pr = static_cast<Program*>(h);
  OpGemm* prev = nullptr;
  int links = 0;
  for (auto& e : pr->ops) {
    auto* g = std::get_if<OpGemm>(&e.op);
    if (!g) continue;
    if (g->p.group_tiles != nullptr) { prev = nullptr; continue; }   // expert tiles are only known on the device
    if (prev != nullptr) {
      const saber::GemmI8Params& n = g->p;
      const int wbytes = n.w4 == 1 ? 16384 : (n.w4 == 2 ? 17408 : 32768);
      const int KB = n.K >> 7;
      prev->p.next_w = n.w;
      prev->p.next_tiles = n.N_pad / 256;
      prev->p.next_splits = n.splits;
      prev->p.next_KB = KB;
      prev->p.next_kb_per = (KB + n.splits - 1) / n.splits;
      prev->p.next_wbytes = wbytes;
      prev->p.next_pref = pref_bytes / wbytes > 0 ? pref_bytes / wbytes : 1;
      ++links;
    }
    prev = g;
  }
  return links;
}
int saber_program_add_row(void* h, int mode, const saber::RowOpParams* p, const char* tag) {
  return add(h, OpRow{mode, *p}, 1, tag);
}
int saber_program_add_embed(void* h, const void* table, const int32_t* ids, void* out, int M, int H,
                            int vocab_lo, int vocab_n, int ldout, const char* tag) {
  return add(h, OpEmbed{table, ids, out, M, H, vocab_lo, vocab_n, ldout}, 1, tag);
}
int saber_program_add_expand(void* h, const void* ctx, const void* tok, const void* pos, void* out,
                             int nseq, int block, int H, const char* tag) {
  return add(h, OpExpand{ctx, tok, pos, out, nseq, block, H}, 1, tag);
}
int saber_program_add_advance(void* h, uint32_t* seq_base, uint32_t by, const char* tag) {
  return add(h, OpAdvance{seq_base, by}, 1, tag);
}
int saber_program_add_gdn_conv(void* h, const saber::GdnConvParams* p, int nseq, const char* tag) {
  return add(h, OpGdnConv{*p, nseq}, p->commit ? 2 : 1, tag);
}
int saber_program_add_gdn_step(void* h, const saber::GdnStepParams* p, int nseq, const char* tag) {
  return add(h, OpGdnStep{*p, nseq}, 1, tag);
}
int saber_program_add_gdn_rec(void* h, const saber::GdnRecParams* p, int nseq, int vs, const char* tag) {
  return add(h, OpGdnRec{*p, nseq, vs}, 1, tag);
}
int saber_program_add_gdn_chunk(void* h, const saber::GdnRecParams* p, int nseq, int max_rows, float* scratch,
                                const char* tag) {
  return add(h, OpGdnChunk{*p, nseq, max_rows, scratch}, 2, tag);
}
int saber_program_add_rope(void* h, const saber::RopeKvParams* p, const char* tag) {
  return add(h, OpRope{*p}, 1, tag);
}
int saber_program_add_attn(void* h, const saber::AttnParams* p, const char* tag) {
  return add(h, OpAttn{*p}, p->splits > 1 ? 2 : 1, tag);
}
int saber_program_add_argmax(void* h, const void* logits, int rows, int ld, int V, int id_offset,
                             int32_t* idx, float* val, const char* tag) {
  return add(h, OpArgmax{logits, rows, ld, V, id_offset, idx, val}, 1, tag);
}
int saber_program_add_seam(void* h, const void* logits, int rows, int ld, int V, int id_offset,
                           const float* temps, int32_t* ids, float* vals, float* lse, const char* tag) {
  return add(h, OpSeam{logits, rows, ld, V, id_offset, temps, ids, vals, lse}, 1, tag);
}
int saber_program_add_verify(void* h, const saber::VerifyParams* p, const char* tag) {
  return add(h, OpVerify{*p}, 1, tag);
}
int saber_program_add_draft_index(void* h, const saber::DraftIndexParams* p, const char* tag) {
  return add(h, OpDraftIndex{*p}, 1, tag);
}
int saber_program_add_memset(void* h, void* dst, int value, size_t bytes, const char* tag) {
  return add(h, OpMemset{dst, value, bytes}, 1, tag);
}
int saber_program_add_copy(void* h, void* dst, const void* src, size_t bytes, const char* tag) {
  return add(h, OpCopy{dst, src, bytes}, 1, tag);
}
int saber_program_add_seam_merge(void* h, const saber::SeamMergeParams* p, const char* tag) {
  return add(h, OpSeamMerge{*p}, 1, tag);
}
int saber_program_add_pick_merge(void* h, const saber::PickMergeParams* p, const char* tag) {
  return add(h, OpPickMerge{*p}, p->nranks > 1 ? 1 : 0, tag);
}
int saber_program_add_moe_route(void* h, const saber::MoeRouteParams* p, const char* tag) {
  return add(h, OpMoeRoute{*p}, 3, tag);
}
int saber_program_add_moe_gather(void* h, const int8_t* q, const float* scale, int M_pad, const int32_t* src_row,
                                 const int32_t* ntiles, int8_t* q_out, float* scale_out, int rows_cap,
                                 int M_pad_out, int K, int to_fp8, const char* tag) {
  return add(h, OpMoeGather{q, scale, M_pad, src_row, ntiles, q_out, scale_out, rows_cap, M_pad_out, K, to_fp8}, 1, tag);
}
int saber_program_add_digest(void* h, const void* buf, size_t bytes, unsigned long long* out, const char* tag) {
  return add(h, OpDigest{buf, bytes, out}, 1, tag);
}
int saber_program_add_sample_seam(void* h, const int32_t* ids, const float* vals, const float* samp, const float* u,
                                  int32_t* picks, int rows, const char* tag) {
  return add(h, OpSampleSeam{ids, vals, samp, u, picks, rows}, 1, tag);
}
int saber_program_add_logit_gather(void* h, const void* logits, int rows, int ld, int V, int id_offset,
                                   const int32_t* ids, float* out, const char* tag) {
  return add(h, OpLogitGather{logits, rows, ld, V, id_offset, ids, out}, 1, tag);
}
int saber_program_add_digest_clear(void* h, unsigned long long* out, int n, const char* tag) {
  return add(h, OpDigestClear{out, n}, 1, tag);
}
int saber_program_add_moe_combine(void* h, const saber::MoeCombineParams* p, const char* tag) {
  return add(h, OpMoeCombine{*p}, 1, tag);
}
int saber_program_add_allreduce(void* h, const saber::AllReduceParams* p, const char* tag) {
  return add(h, OpAllReduce{*p}, 1, tag);
}

int saber_program_num_ops(void* h) { return static_cast<int>(static_cast<Program*>(h)->ops.size()); }

int saber_program_declared_launches(void* h) {
  int n = 0;
  for (auto& e : static_cast<Program*>(h)->ops) n += e.launches;
  return n;
}

const char* saber_program_op_tag(void* h, int i) {
  auto* pr = static_cast<Program*>(h);
  return (i >= 0 && i < static_cast<int>(pr->ops.size())) ? pr->ops[i].tag.c_str() : "";
}

int saber_program_last_failed_op(void* h) { return static_cast<Program*>(h)->last_failed_op; }

// Eager walk of ops [first, last). Returns 0 or the CUDA error of the first failing launch.
int saber_program_run_range(void* h, int first, int last, cudaStream_t stream) {
  auto* pr = static_cast<Program*>(h);
  const int n = static_cast<int>(pr->ops.size());
  if (last < 0 || last > n) last = n;
  for (int i = first; i < last; ++i) {
    const int e = launch(pr->ops[i].op, stream);
    if (e != 0) { pr->last_failed_op = i; return e; }
  }
  return 0;
}

int saber_program_run(void* h, cudaStream_t stream) { return saber_program_run_range(h, 0, -1, stream); }

// Capture the whole program on `stream` (which must not be the legacy default stream) and
// instantiate it. Returns the number of nodes in the captured graph, or -(cuda error).
int saber_program_capture(void* h, cudaStream_t stream) {
  auto* pr = static_cast<Program*>(h);
  if (pr->exec) { cudaGraphExecDestroy(pr->exec); pr->exec = nullptr; }
  if (pr->graph) { cudaGraphDestroy(pr->graph); pr->graph = nullptr; }
  cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) return -static_cast<int>(e);
  const int le = saber_program_run(h, stream);
  cudaGraph_t g = nullptr;
  e = cudaStreamEndCapture(stream, &g);
  if (le != 0) { if (g) cudaGraphDestroy(g); return -le; }
  if (e != cudaSuccess) return -static_cast<int>(e);
  size_t nodes = 0;
  e = cudaGraphGetNodes(g, nullptr, &nodes);
  if (e != cudaSuccess) { cudaGraphDestroy(g); return -static_cast<int>(e); }
  cudaGraphExec_t ex = nullptr;
  e = cudaGraphInstantiate(&ex, g, 0);
  if (e != cudaSuccess) { cudaGraphDestroy(g); return -static_cast<int>(e); }
  pr->graph = g;
  pr->exec = ex;
  pr->captured_nodes = static_cast<int>(nodes);
  return pr->captured_nodes;
}

int saber_program_replay(void* h, cudaStream_t stream) {
  auto* pr = static_cast<Program*>(h);
  if (!pr->exec) return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGraphLaunch(pr->exec, stream));
}

int saber_program_captured_nodes(void* h) { return static_cast<Program*>(h)->captured_nodes; }

}  // extern "C"
