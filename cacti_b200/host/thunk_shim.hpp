// Host-side shim: the part of cacti's run-time that a GPU thunk implementation lives under, restated in
// C++ so that the new kernels can be exercised under the reference's memory policy without its Rust host.
//
//   Arena      one device region with a front bump cursor and a first-fit free list, 256-byte alignment
//              (NvGpuMemPool, src/pctx/nvgpu.rs:1377-1522; ALLOC_ALIGN :30).
//   Cell       a logical tensor with at most one device replica and one host replica, reference-style
//              pin counts (src/pctx/nvgpu.rs:1179-1337) and the "unlive" mark the liveness pass sets
//              (src/spine.rs:1974-1979).
//   PCtx       allocation with the soft-OOM policy of _try_soft_oom (src/pctx/nvgpu.rs:2004-2283): first
//              drop device replicas of unlive cells (spilling stable ones to the host), then walk cells in
//              creation order from a resumable cursor, preferring cells at least as large as the request,
//              spill each to the host and free its device replica, and retry (PCtx::alloc,
//              src/pctx/mod.rs:342-402).  Pinned cells are never touched.
//   thunks     Apply / Accumulate wrappers in the shape of ThunkImpl (src/thunk/mod.rs:347-351): look up or
//              allocate replicas (pread / pwrite / prewrite, src/ctx.rs:1777-1973), pin every argument and the
//              output from pointer lookup until the launch has been issued, call the C ABI, unpin.
//
// Everything runs on one stream, so frees, re-use and spill copies are ordered behind the kernels that
// touched the memory without per-cell events.  The reference instead synchronises around every thunk and
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
  // returns offset or SIZE_MAX
  size_t alloc(size_t bytes);
  void free(size_t off);
  size_t in_use() const { return in_use_; }
  size_t capacity() const { return cap_; }
 private:
  size_t cap_ = 0, front_ = 0, in_use_ = 0;
  std::map<size_t, size_t> live_;      // offset -> size
  std::map<size_t, size_t> holes_;     // offset -> size, below front_
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
struct Stats { long spills = 0, drops = 0, reloads = 0, oom_retries = 0, hard_oom = 0, spill_copies = 0; };

enum Mode { kApply = 0, kAccumulate = 1 };

class PCtx {
 public:
  PCtx(Backend* b, size_t arena_bytes, size_t soft_limit);
  ~PCtx();
  int64_t cell_new(size_t bytes, bool stable);
  int cell_put(int64_t c, const void* host, size_t bytes);     // resume_put: host data becomes the cell's value
  int cell_get(int64_t c, void* host, size_t bytes);           // with_mem read-back (synchronises)
  int cell_unlive(int64_t c);
  bool resident(int64_t c) const { return cells_[c].dev_off != SIZE_MAX; }
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
  bool sync_each_thunk = false;

 private:
  size_t alloc_with_policy(size_t bytes);
  bool try_soft_oom(size_t req);
  bool evict(int64_t c, bool must_keep_value);
  Backend* be_;
  Arena arena_;
  char* base_ = nullptr;
  size_t soft_limit_;
  std::vector<Cell> cells_;
  std::set<int64_t> unlive_;
  size_t cursor_ = 0;
  Stats stats_;
};

// ThunkImpl-shaped wrappers: `out` is bound as pwrite (Apply) or prewrite (Accumulate).  Return the C-ABI code,
// or -1 for a hard OOM.
int thunk_rmsnorm_fwd(PCtx& p, Mode m, int64_t y, int64_t x, int64_t gamma, float eps, int64_t rows, int64_t cols, int dtype);
int thunk_add_rmsnorm_fwd(PCtx& p, Mode m, int64_t y, int64_t sum, int64_t a, int64_t b, int64_t gamma, float eps, int64_t rows,
                          int64_t cols, int dtype);
int thunk_softmax_fwd(PCtx& p, Mode m, int64_t prob, int64_t s, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype);
int thunk_softmax_bwd(PCtx& p, Mode m, int64_t ds, int64_t s, int64_t dp, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype);
int thunk_add(PCtx& p, Mode m, int64_t out, int64_t a, int64_t b, int64_t n, int dtype);
int thunk_matmul(PCtx& p, Mode m, int64_t c, int64_t a, int64_t b, int64_t mm, int64_t nn, int64_t kk, int ta, int tb, float alpha, int dtype);

}  // namespace cbh
