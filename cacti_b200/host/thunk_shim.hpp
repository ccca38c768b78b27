// Host-side shim: the part of cacti's run-time that a GPU thunk implementation lives under, restated in
// C++ so that the new kernels can be exercised under the reference's memory policy without its Rust host.
//
//   Arena      one device region with a front and a back bump cursor and a first-fit free list, 256-byte alignment
//              (NvGpuMemPool, src/pctx/nvgpu.rs:1377-1522; ALLOC_ALIGN :30).  Long-lived cells (parameters, optimizer
//              state: `stable`) come from the back, as the reference places its constants there
//              (src/thunk/mod.rs:2057,2077), so that the front stays one run of short-lived activations.
//   Cell       a logical tensor with at most one device replica and one host replica, reference-style
//              pin counts (src/pctx/nvgpu.rs:1179-1337) and the "unlive" mark the liveness pass sets
//              (src/spine.rs:1974-1979).
//   PCtx       allocation with the soft-OOM policy of _try_soft_oom (src/pctx/nvgpu.rs:2004-2283): first
//              drop device replicas of unlive cells (spilling stable ones to the host), then walk cells in
//              creation order from a resumable cursor, preferring cells at least as large as the request,
//              spill each to the host and free its device replica, and retry (PCtx::alloc,
//              src/pctx/mod.rs:342-402).  Pinned cells are never touched.
//   thunks     Apply / Accumulate / Initialize wrappers in the shape of ThunkImpl (src/thunk/mod.rs:347-351): look
//              up or allocate replicas (pread / pwrite / prewrite, src/ctx.rs:1777-1973), pin every argument and
//              output from pointer lookup until the launch has been issued, call the C ABI, unpin.  Workspaces are
//              cells of the same arena, freed when the launch has been issued (re-use is stream-ordered).
//
// Everything runs on ONE stream (Backend::stream()): frees, re-use and spill copies are thereby ordered behind the
// kernels that touched the memory without per-cell events, which is why a pin can be dropped as soon as the launch
// has been issued.  A host that launched on several streams would have to hold each pin until an event behind the
// launch has completed.  The reference instead synchronises around every thunk and
// pins nothing (src/thunk/mod.rs:3478-3536); `sync_each_thunk` restores that behaviour.
//
// The device is reached through a Backend so that the policy can be tested without a GPU.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <set>
#include <vector>

namespace cbh {

constexpr size_t kAlign = 256;

struct Backend {
  virtual ~Backend() {}
  virtual void* arena_alloc(size_t bytes) = 0;
  virtual void arena_free(void* p) = 0;
  virtual void* host_alloc(size_t bytes) = 0;
  virtual void host_free(void* p) = 0;
  virtual int d2h(void* dst, const void* src, size_t bytes) = 0;   // stream-ordered
  virtual int h2d(void* dst, const void* src, size_t bytes) = 0;   // stream-ordered
  virtual int sync() = 0;
  virtual void* stream() = 0;
};
Backend* make_fake_backend();   // host memory stands in for the device
Backend* make_cuda_backend();   // CUDA runtime, one non-default stream

class Arena {
 public:
  void init(size_t bytes);
  // returns offset or SIZE_MAX; back: take the block from the back cursor (or a hole behind it)
  size_t alloc(size_t bytes, bool back = false);
  void free(size_t off);
  size_t in_use() const { return in_use_; }
  size_t capacity() const { return cap_; }
  size_t front() const { return front_; }
  size_t back() const { return back_; }
 private:
  size_t cap_ = 0, front_ = 0, back_ = 0, in_use_ = 0;   // [0, front_) and [back_, cap_) have been handed out
  std::map<size_t, size_t> live_;      // offset -> size
  std::map<size_t, size_t> holes_;     // offset -> size, below front_ or at / above back_
};

struct Cell {
  size_t bytes = 0;
  size_t dev_off = SIZE_MAX;   // SIZE_MAX: no device replica
  void* host = nullptr;        // host replica (spill target)
  bool host_valid = false, dev_valid = false;
  bool stable = false, unlive = false, dead = false;
  int pins = 0;
};

// spills: evictions that kept the value on the host (spill_copies of them needed a device-to-host copy)
struct Stats {
  long spills = 0, drops = 0, reloads = 0, oom_retries = 0, hard_oom = 0, spill_copies = 0;
  long long spill_bytes = 0, reload_bytes = 0;      // bytes copied device-to-host by spills, host-to-device by reloads
  size_t peak_in_use = 0;
};

// Apply: fresh output.  Accumulate: out += f(args).  Initialize: the output is read and overwritten in place, what the
// optimizer's update thunks do (src/thunk/mod.rs:347-351; src/op.rs:950-1023).
enum Mode { kApply = 0, kAccumulate = 1, kInitialize = 2 };

// CACTI_VMEM_SOFT_LIMIT as the reference reads it (src/pctx/nvgpu.rs:1438-1463): a string that parses as a decimal
// number is a fraction of `total` (clamped to [0, 1] and to avail - 32 MiB); otherwise a byte size with an optional
// K / M / G / T prefix (powers of 1000, or of 1024 with an `i`) and an optional B; the result is rounded down to
// 64 KiB.  Returns 0 when the string is neither.
size_t parse_vmem_soft_limit(const char* text, size_t total, size_t avail);

class PCtx {
 public:
  PCtx(Backend* b, size_t arena_bytes, size_t soft_limit);
  ~PCtx();
  int64_t cell_new(size_t bytes, bool stable);
  int cell_put(int64_t c, const void* host, size_t bytes);     // resume_put: host data becomes the cell's value
  int cell_get(int64_t c, void* host, size_t bytes);           // with_mem read-back (synchronises)
  int cell_unlive(int64_t c);
  int cell_free(int64_t c);                                    // the cell is gone; its id is handed out again
  bool resident(int64_t c) const { return cells_[c].dev_off != SIZE_MAX; }
  size_t cell_bytes(int64_t c) const { return cells_[c].bytes; }
  // device pointers; each may trigger allocation, reload from host, or the soft-OOM policy.  0 = hard OOM.
  uint64_t pread(int64_t c);        // current value must exist
  uint64_t pwrite(int64_t c);       // fresh output: old contents irrelevant
  uint64_t prewrite(int64_t c);     // read-modify-write output (Accumulate)
  void pin(int64_t c) { ++cells_[c].pins; }
  void unpin(int64_t c) { --cells_[c].pins; }
  void* stream() { return be_->stream(); }
  int sync() { return be_->sync(); }
  const Stats& stats() const { return stats_; }
  size_t in_use() const { return arena_.in_use(); }
  size_t soft_limit() const { return soft_limit_; }
  bool sync_each_thunk = false;

 private:
  size_t alloc_with_policy(size_t bytes, bool back = false);
  bool try_soft_oom(size_t req);
  bool evict(int64_t c, bool must_keep_value);
  void* host_buffer(size_t bytes);
  Backend* be_;
  Arena arena_;
  char* base_ = nullptr;
  size_t soft_limit_;
  std::vector<Cell> cells_;
  std::vector<int64_t> free_ids_;
  std::multimap<size_t, void*> host_pool_;      // page-locked buffers of freed cells, by size
  std::set<int64_t> unlive_;
  size_t cursor_ = 0;
  Stats stats_;
};

// ThunkImpl-shaped wrappers.  An output is bound as pwrite (Apply) or prewrite (Accumulate, Initialize); cells are ids
// of `p`.  Shapes are run-time values as in the reference (its impl cache keys on rank and dtype only,
// src/ctx.rs:1054-1082); a cell may be used under several shapes (reshapes are free aliases there, src/ctx.rs:515-539).
// Return the C-ABI code, or -1 for a hard OOM (the reference panics, src/pctx/nvgpu.rs:2433-2441).
int thunk_rmsnorm_fwd(PCtx& p, Mode m, int64_t y, int64_t x, int64_t gamma, float eps, int64_t rows, int64_t cols, int dtype);
int thunk_add_rmsnorm_fwd(PCtx& p, Mode m, int64_t y, int64_t sum, int64_t a, int64_t b, int64_t gamma, float eps, int64_t rows,
                          int64_t cols, int dtype);
// two outputs, each with its own mode; the column-partial workspace is a temporary cell
int thunk_rmsnorm_bwd(PCtx& p, Mode m_dx, Mode m_dgamma, int64_t dx, int64_t dgamma, int64_t dy, int64_t x, int64_t gamma, float eps,
                      int64_t rows, int64_t cols, int dtype, int dgamma_dtype);
int thunk_softmax_fwd(PCtx& p, Mode m, int64_t prob, int64_t s, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype);
int thunk_softmax_bwd(PCtx& p, Mode m, int64_t ds, int64_t s, int64_t dp, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype);
int thunk_add(PCtx& p, Mode m, int64_t out, int64_t a, int64_t b, int64_t n, int dtype);
int thunk_matmul(PCtx& p, Mode m, int64_t c, int64_t a, int64_t b, int64_t mm, int64_t nn, int64_t kk, int ta, int tb, float alpha, int dtype);
int thunk_rope_fwd(PCtx& p, Mode m, int64_t y, int64_t x, int64_t cos, int64_t sin, int64_t tokens, int64_t heads, int64_t hd,
                   int64_t pos_mod, int64_t head_pitch /* 0: packed output */, int dtype);
int thunk_rope_bwd(PCtx& p, Mode m, int64_t dx, int64_t dy, int64_t cos, int64_t sin, int64_t tokens, int64_t heads, int64_t hd,
                   int64_t pos_mod, int dtype);
int thunk_swiglu_fwd(PCtx& p, Mode m, int64_t h, int64_t gate, int64_t up, int64_t n, int dtype);
int thunk_swiglu_bwd(PCtx& p, Mode m_dgate, Mode m_dup, int64_t dgate, int64_t dup, int64_t gate, int64_t up, int64_t dh, int64_t n, int dtype);
// loss_sum (f32[1]) and dlogits; status: u32 cell the caller zeroed; the per-row workspace is a temporary cell
int thunk_softmax_nll(PCtx& p, Mode m_dlogits, int64_t loss_sum, int64_t dlogits, int64_t logits, int64_t targets, int target_dtype,
                      float w, int64_t rows, int64_t vocab, int dtype, int64_t status);
int thunk_gather_rows(PCtx& p, Mode m, int64_t out, int64_t table, int64_t tokens, int token_dtype, int64_t n, int64_t vocab,
                      int64_t cols, int dtype, int64_t status);
int thunk_scatter_add_rows(PCtx& p, Mode m, int64_t dtable, int64_t dy, int64_t tokens, int token_dtype, int64_t n, int64_t vocab,
                           int64_t cols, int dtype, int64_t status);
int thunk_block_pad(PCtx& p, Mode m, int64_t dst, int64_t src, int64_t nrow, int64_t rows, int64_t ncol, int64_t cols, int64_t cols_pad, int dtype);
// block matmul on the reference's 4-d layout: a is [nrow, a_rows, ncol, a_ld], b likewise (a_ld / b_ld: stored block
// width, larger than the logical width for zero-padded operands); tri / diag / flags as cacti_b200_gemm_strided_batched_tri
int thunk_block_matmul(PCtx& p, Mode m, int64_t c, int64_t a, int64_t b, int64_t nrow, int64_t ncol, int64_t mm, int64_t nn, int64_t kk,
                       int64_t a_ld, int64_t b_ld, int ta, int tb, float alpha, int tri, int64_t diag, int flags, int dtype);
int thunk_attention_fwd(PCtx& p, Mode m, int64_t ctx, int64_t stats, int64_t q, int64_t k, int64_t v, int64_t batch, int64_t seq,
                        int64_t heads, int64_t hd, float alpha, int dtype);
int thunk_attention_bwd_prep(PCtx& p, Mode m, int64_t prob, int64_t ds, int64_t q, int64_t k, int64_t v, int64_t dctx, int64_t ctx,
                             int64_t stats, int64_t batch, int64_t seq, int64_t heads, int64_t hd, float alpha, int dtype);
// three outputs (dq, dk, dv); P and dS never exist as cells
int thunk_attention_bwd(PCtx& p, Mode m, int64_t dq, int64_t dk, int64_t dv, int64_t q, int64_t k, int64_t v, int64_t dctx, int64_t ctx,
                        int64_t stats, int64_t batch, int64_t seq, int64_t heads, int64_t hd, float alpha, int dtype);
// Initialize mode only: master, grad1_avg, grad2_avg are read and overwritten, param_out rewritten (AdamW32::step,
// src/librarium/adamw.rs:46-61)
int thunk_adamw32_step(PCtx& p, Mode m, int64_t master, int64_t grad1_avg, int64_t grad2_avg, int64_t param_out, int64_t grad, int64_t n,
                       int grad_dtype, int param_dtype, float grad_unscale, float lr, float wd, float a1, float a2, float eps, int iter_nr);

}  // namespace cbh
