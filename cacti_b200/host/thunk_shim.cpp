#include "thunk_shim.hpp"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "../../include/cacti_b200.h"

namespace cbh {

static size_t up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// ---- backends -----------------------------------------------------------------------------------
namespace {
struct FakeBackend : Backend {
  void* arena_alloc(size_t b) override {
    void* p = std::aligned_alloc(kAlign, up(b ? b : 1));
    if (p) std::memset(p, 0, up(b ? b : 1));
    return p;
  }
  void arena_free(void* p) override { std::free(p); }
  void* host_alloc(size_t b) override { return std::malloc(b ? b : 1); }
  void host_free(void* p) override { std::free(p); }
  int d2h(void* d, const void* s, size_t b) override { std::memcpy(d, s, b); return 0; }
  int h2d(void* d, const void* s, size_t b) override { std::memcpy(d, s, b); return 0; }
  int sync() override { return 0; }
  void* stream() override { return nullptr; }
};
struct CudaBackend : Backend {
  cudaStream_t st = nullptr;
  CudaBackend() { cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking); }
  ~CudaBackend() override { if (st) cudaStreamDestroy(st); }
  void* arena_alloc(size_t b) override { void* p = nullptr; return cudaMalloc(&p, b) == cudaSuccess ? p : nullptr; }
  void arena_free(void* p) override { cudaFree(p); }
  // page-locked, like CACTI_NVGPU_MEM_ALLOC=pagelocked (src/pctx/nvgpu.rs:996-1002)
  void* host_alloc(size_t b) override { void* p = nullptr; return cudaMallocHost(&p, b ? b : 1) == cudaSuccess ? p : nullptr; }
  void host_free(void* p) override { cudaFreeHost(p); }
  int d2h(void* d, const void* s, size_t b) override { return cudaMemcpyAsync(d, s, b, cudaMemcpyDeviceToHost, st) != cudaSuccess; }
  int h2d(void* d, const void* s, size_t b) override { return cudaMemcpyAsync(d, s, b, cudaMemcpyHostToDevice, st) != cudaSuccess; }
  int sync() override { return cudaStreamSynchronize(st) != cudaSuccess; }
  void* stream() override { return st; }
};
}  // namespace
Backend* make_fake_backend() { return new FakeBackend; }
Backend* make_cuda_backend() { return new CudaBackend; }

// ---- arena ----------------------------------------------------------------------------------------
void Arena::init(size_t bytes) { cap_ = bytes / kAlign * kAlign; front_ = in_use_ = 0; live_.clear(); holes_.clear(); }

size_t Arena::alloc(size_t bytes) {
  const size_t need = up(bytes ? bytes : 1);
  for (auto it = holes_.begin(); it != holes_.end(); ++it) {       // first fit in the free list
    if (it->second >= need) {
      const size_t off = it->first, rest = it->second - need;
      holes_.erase(it);
      if (rest) holes_[off + need] = rest;
      live_[off] = need; in_use_ += need;
      return off;
    }
  }
  if (front_ + need > cap_) return SIZE_MAX;
  const size_t off = front_;
  front_ += need; live_[off] = need; in_use_ += need;
  return off;
}

void Arena::free(size_t off) {
  auto it = live_.find(off);
  if (it == live_.end()) return;
  size_t sz = it->second;
  live_.erase(it); in_use_ -= sz;
  // coalesce with neighbours; a hole that touches the bump cursor lowers the cursor instead
  auto nx = holes_.find(off + sz);
  if (nx != holes_.end()) { sz += nx->second; holes_.erase(nx); }
  auto pv = holes_.lower_bound(off);
  if (pv != holes_.begin()) {
    --pv;
    if (pv->first + pv->second == off) { off = pv->first; sz += pv->second; holes_.erase(pv); }
  }
  if (off + sz == front_) front_ = off; else holes_[off] = sz;
}

// ---- pctx -------------------------------------------------------------------------------------------
PCtx::PCtx(Backend* b, size_t arena_bytes, size_t soft_limit) : be_(b), soft_limit_(soft_limit ? soft_limit : arena_bytes) {
  base_ = static_cast<char*>(be_->arena_alloc(arena_bytes));
  arena_.init(base_ ? arena_bytes : 0);
}
PCtx::~PCtx() {
  be_->sync();
  for (auto& c : cells_) if (c.host) be_->host_free(c.host);
  if (base_) be_->arena_free(base_);
  delete be_;
}

int64_t PCtx::cell_new(size_t bytes, bool stable) {
  Cell c; c.bytes = bytes; c.stable = stable;
  cells_.push_back(c);
  return (int64_t)cells_.size() - 1;
}

// Frees the device replica of c.  must_keep_value: copy it to the host first (a spill).
bool PCtx::evict(int64_t id, bool must_keep_value) {
  Cell& c = cells_[id];
  if (c.dev_off == SIZE_MAX || c.pins > 0) return false;
  if (must_keep_value) {
    if (c.dev_valid && !c.host_valid) {          // the device holds the only current replica: copy it out
      if (!c.host) c.host = be_->host_alloc(c.bytes);
      if (!c.host || be_->d2h(c.host, base_ + c.dev_off, c.bytes)) return false;
      c.host_valid = true;
      ++stats_.spill_copies;
    }
    ++stats_.spills;
  } else {
    ++stats_.drops;
  }
  arena_.free(c.dev_off);          // re-use is ordered behind the copy: same stream
  c.dev_off = SIZE_MAX; c.dev_valid = false;
  return true;
}

bool PCtx::try_soft_oom(size_t req) {
  bool freed = false;
  // (1) cells the liveness pass marked unlive: non-stable ones lose their value, stable ones are spilled
  for (auto it = unlive_.begin(); it != unlive_.end();) {
    Cell& c = cells_[*it];
    if (c.dev_off != SIZE_MAX && c.pins == 0) {
      const bool keep = c.stable;
      if (evict(*it, keep)) { freed = true; if (!keep) c.dead = true; }
      it = unlive_.erase(it);
    } else {
      ++it;
    }
    if (freed && arena_.in_use() + up(req) <= soft_limit_) return true;
  }
  if (freed) return true;
  // (2) creation order from a resumable cursor; first pass prefers cells at least as large as the request
  for (int pass = 0; pass < 2; ++pass) {
    const size_t n = cells_.size();
    for (size_t step = 0; step < n; ++step) {
      const size_t i = (cursor_ + step) % n;
      Cell& c = cells_[i];
      if (c.dev_off == SIZE_MAX || c.pins > 0 || c.dead) continue;
      if (pass == 0 && c.bytes < req) continue;
      if (evict((int64_t)i, true)) { cursor_ = (i + 1) % n; return true; }
    }
  }
  return false;
}

size_t PCtx::alloc_with_policy(size_t bytes) {
  for (;;) {
    if (arena_.in_use() + up(bytes) <= soft_limit_) {
      const size_t off = arena_.alloc(bytes);
      if (off != SIZE_MAX) return off;
    }
    ++stats_.oom_retries;
    if (!try_soft_oom(bytes)) { ++stats_.hard_oom; return SIZE_MAX; }
  }
}

int PCtx::cell_put(int64_t id, const void* host, size_t bytes) {
  Cell& c = cells_[id];
  if (bytes != c.bytes) return 1;
  if (!c.host) c.host = be_->host_alloc(c.bytes);
  if (!c.host) return 1;
  be_->sync();                                  // the host replica may still be the target of a spill copy
  std::memcpy(c.host, host, bytes);
  c.host_valid = true; c.dev_valid = false; c.dead = false;
  return 0;
}

int PCtx::cell_get(int64_t id, void* host, size_t bytes) {
  Cell& c = cells_[id];
  if (bytes != c.bytes || c.dead) return 1;
  if (c.dev_valid) {
    if (be_->d2h(host, base_ + c.dev_off, bytes)) return 1;
    return be_->sync();
  }
  if (!c.host_valid) return 1;
  if (be_->sync()) return 1;
  std::memcpy(host, c.host, bytes);
  return 0;
}

int PCtx::cell_unlive(int64_t id) { cells_[id].unlive = true; unlive_.insert(id); return 0; }

uint64_t PCtx::pread(int64_t id) {
  if (cells_[id].dead) return 0;
  if (cells_[id].dev_off == SIZE_MAX) {
    pin(id);                                                 // not evictable while being brought in
    const size_t off = alloc_with_policy(cells_[id].bytes);
    unpin(id);
    if (off == SIZE_MAX) return 0;
    cells_[id].dev_off = off;
  }
  Cell& c = cells_[id];
  if (!c.dev_valid) {
    if (!c.host_valid) return 0;                             // no value anywhere
    if (be_->h2d(base_ + c.dev_off, c.host, c.bytes)) return 0;
    c.dev_valid = true;
    ++stats_.reloads;
  }
  return reinterpret_cast<uint64_t>(base_ + c.dev_off);
}

uint64_t PCtx::pwrite(int64_t id) {
  if (cells_[id].dev_off == SIZE_MAX) {
    const size_t off = alloc_with_policy(cells_[id].bytes);
    if (off == SIZE_MAX) return 0;
    cells_[id].dev_off = off;
  }
  Cell& c = cells_[id];
  c.dev_valid = true; c.host_valid = false; c.dead = false;
  return reinterpret_cast<uint64_t>(base_ + c.dev_off);
}

uint64_t PCtx::prewrite(int64_t id) {
  const uint64_t p = pread(id);
  if (p) cells_[id].host_valid = false;
  return p;
}

// ---- thunks -----------------------------------------------------------------------------------------
namespace {
// Pins cells as their pointers are looked up; unpins on scope exit (after the launch has been issued).
struct Binding {
  PCtx& p; std::vector<int64_t> pinned; bool ok = true;
  explicit Binding(PCtx& p_) : p(p_) {}
  uint64_t in(int64_t c) { uint64_t d = p.pread(c); if (!d) ok = false; else { p.pin(c); pinned.push_back(c); } return d; }
  uint64_t out(int64_t c, Mode m) {
    uint64_t d = m == kApply ? p.pwrite(c) : p.prewrite(c);
    if (!d) ok = false; else { p.pin(c); pinned.push_back(c); }
    return d;
  }
  ~Binding() { if (p.sync_each_thunk) p.sync(); for (int64_t c : pinned) p.unpin(c); }
};
size_t esize(int dtype) { return dtype == CACTI_B200_R_32F ? 4 : 2; }
}  // namespace

int thunk_rmsnorm_fwd(PCtx& p, Mode m, int64_t y, int64_t x, int64_t gamma, float eps, int64_t rows, int64_t cols, int dtype) {
  Binding b(p);
  const uint64_t dx = b.in(x), dg = b.in(gamma);
  if (m == kApply) {
    const uint64_t dy = b.out(y, kApply);
    if (!b.ok) return -1;
    return cacti_b200_rmsnorm_fwd(dy, dx, dg, eps, rows, cols, dtype, p.stream());
  }
  // Accumulate on a forward output: compute into a temporary cell, then out += tmp (what the reference does for
  // an out-of-place accumulate, src/thunk/mod.rs:3815-3856)
  const int64_t tmp = p.cell_new((size_t)rows * cols * esize(dtype), false);
  const uint64_t dt = b.out(tmp, kApply), dy = b.out(y, kAccumulate);
  if (!b.ok) return -1;
  int rc = cacti_b200_rmsnorm_fwd(dt, dx, dg, eps, rows, cols, dtype, p.stream());
  if (!rc) rc = cacti_b200_accumulate(dy, dt, rows * cols, dtype, p.stream());
  p.cell_unlive(tmp);
  return rc;
}

// Two-output thunk: sum = a + b and y = rmsnorm(sum) in one kernel (the residual add fused into the norm that follows
// it, src/librarium/llama.rs:514-516).  Apply only: both outputs are fresh cells of the forward pass.
int thunk_add_rmsnorm_fwd(PCtx& p, Mode m, int64_t y, int64_t sum, int64_t a, int64_t b_, int64_t gamma, float eps, int64_t rows,
                          int64_t cols, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t da = b.in(a), db = b.in(b_), dg = b.in(gamma);
  const uint64_t dy = b.out(y, kApply), ds = b.out(sum, kApply);
  if (!b.ok) return -1;
  return cacti_b200_add_rmsnorm_fwd(dy, ds, da, db, dg, eps, rows, cols, dtype, p.stream());
}

int thunk_softmax_fwd(PCtx& p, Mode m, int64_t prob, int64_t s, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t ds = b.in(s), dp = b.out(prob, kApply);
  if (!b.ok) return -1;
  return cacti_b200_softmax_fwd(dp, ds, rows, cols, q_div > 0 ? CACTI_B200_MASK_CAUSAL : CACTI_B200_MASK_NONE,
                                q_div > 0 ? q_div : 1, q_mod > 0 ? q_mod : 1, 0, dtype, p.stream());
}

int thunk_softmax_bwd(PCtx& p, Mode m, int64_t dsc, int64_t s, int64_t dpr, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype) {
  Binding b(p);
  const uint64_t ds_ = b.in(s), dp_ = b.in(dpr), out = b.out(dsc, m);
  if (!b.ok) return -1;
  return cacti_b200_softmax_bwd(out, ds_, dp_, rows, cols, q_div > 0 ? CACTI_B200_MASK_CAUSAL : CACTI_B200_MASK_NONE,
                                q_div > 0 ? q_div : 1, q_mod > 0 ? q_mod : 1, 0, dtype, m == kAccumulate, p.stream());
}

int thunk_add(PCtx& p, Mode m, int64_t out, int64_t a, int64_t bb, int64_t n, int dtype) {
  Binding b(p);
  const uint64_t da = b.in(a), db = b.in(bb);
  if (m == kApply) {
    const uint64_t d = b.out(out, kApply);
    if (!b.ok) return -1;
    return cacti_b200_add(d, da, db, n, dtype, p.stream());
  }
  const uint64_t d = b.out(out, kAccumulate);
  if (!b.ok) return -1;
  int rc = cacti_b200_accumulate(d, da, n, dtype, p.stream());
  if (!rc) rc = cacti_b200_accumulate(d, db, n, dtype, p.stream());
  return rc;
}

int thunk_matmul(PCtx& p, Mode m, int64_t c, int64_t a, int64_t bb, int64_t mm, int64_t nn, int64_t kk, int ta, int tb,
                 float alpha, int dtype) {
  Binding b(p);
  const uint64_t da = b.in(a), db = b.in(bb), dc = b.out(c, m);
  if (!b.ok) return -1;
  const float beta = m == kAccumulate ? 1.f : 0.f;      // src/thunk/op.rs:5053-5067
  const int64_t lda = ta ? mm : kk, ldb = tb ? kk : nn;
  return cacti_b200_gemm(dc, da, db, mm, nn, kk, lda, ldb, nn, ta, tb, &alpha, &beta, dtype, 0, 0, p.stream());
}

}  // namespace cbh

// ---- flat test ABI (ctypes) ----------------------------------------------------------------------
extern "C" {
void* cbh_ctx_create(int cuda, size_t arena_bytes, size_t soft_limit, int sync_each_thunk) {
  cbh::PCtx* p = new cbh::PCtx(cuda ? cbh::make_cuda_backend() : cbh::make_fake_backend(), arena_bytes, soft_limit);
  p->sync_each_thunk = sync_each_thunk != 0;
  return p;
}
void cbh_ctx_destroy(void* c) { delete static_cast<cbh::PCtx*>(c); }
int64_t cbh_cell_new(void* c, size_t bytes, int stable) { return static_cast<cbh::PCtx*>(c)->cell_new(bytes, stable != 0); }
int cbh_cell_put(void* c, int64_t cell, const void* host, size_t bytes) { return static_cast<cbh::PCtx*>(c)->cell_put(cell, host, bytes); }
int cbh_cell_get(void* c, int64_t cell, void* host, size_t bytes) { return static_cast<cbh::PCtx*>(c)->cell_get(cell, host, bytes); }
int cbh_cell_unlive(void* c, int64_t cell) { return static_cast<cbh::PCtx*>(c)->cell_unlive(cell); }
int cbh_cell_resident(void* c, int64_t cell) { return static_cast<cbh::PCtx*>(c)->resident(cell); }
uint64_t cbh_pread(void* c, int64_t cell) { return static_cast<cbh::PCtx*>(c)->pread(cell); }
uint64_t cbh_pwrite(void* c, int64_t cell) { return static_cast<cbh::PCtx*>(c)->pwrite(cell); }
void cbh_pin(void* c, int64_t cell) { static_cast<cbh::PCtx*>(c)->pin(cell); }
void cbh_unpin(void* c, int64_t cell) { static_cast<cbh::PCtx*>(c)->unpin(cell); }
size_t cbh_in_use(void* c) { return static_cast<cbh::PCtx*>(c)->in_use(); }
int cbh_sync(void* c) { return static_cast<cbh::PCtx*>(c)->sync(); }
void cbh_stats(void* c, long* out5) {   // six values
  const cbh::Stats& s = static_cast<cbh::PCtx*>(c)->stats();
  out5[0] = s.spills; out5[1] = s.drops; out5[2] = s.reloads; out5[3] = s.oom_retries; out5[4] = s.hard_oom; out5[5] = s.spill_copies;
}
int cbh_thunk_rmsnorm_fwd(void* c, int mode, int64_t y, int64_t x, int64_t gamma, float eps, int64_t rows, int64_t cols, int dtype) {
  return cbh::thunk_rmsnorm_fwd(*static_cast<cbh::PCtx*>(c), (cbh::Mode)mode, y, x, gamma, eps, rows, cols, dtype);
}
int cbh_thunk_add_rmsnorm_fwd(void* c, int mode, int64_t y, int64_t sum, int64_t a, int64_t b, int64_t gamma, float eps, int64_t rows,
                              int64_t cols, int dtype) {
  return cbh::thunk_add_rmsnorm_fwd(*static_cast<cbh::PCtx*>(c), (cbh::Mode)mode, y, sum, a, b, gamma, eps, rows, cols, dtype);
}
int cbh_thunk_softmax_fwd(void* c, int mode, int64_t p, int64_t s, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype) {
  return cbh::thunk_softmax_fwd(*static_cast<cbh::PCtx*>(c), (cbh::Mode)mode, p, s, rows, cols, q_div, q_mod, dtype);
}
int cbh_thunk_softmax_bwd(void* c, int mode, int64_t ds, int64_t s, int64_t dp, int64_t rows, int64_t cols, int64_t q_div, int64_t q_mod, int dtype) {
  return cbh::thunk_softmax_bwd(*static_cast<cbh::PCtx*>(c), (cbh::Mode)mode, ds, s, dp, rows, cols, q_div, q_mod, dtype);
}
int cbh_thunk_add(void* c, int mode, int64_t out, int64_t a, int64_t b, int64_t n, int dtype) {
  return cbh::thunk_add(*static_cast<cbh::PCtx*>(c), (cbh::Mode)mode, out, a, b, n, dtype);
}
int cbh_thunk_matmul(void* c, int mode, int64_t cc, int64_t a, int64_t b, int64_t m, int64_t n, int64_t k, int ta, int tb, float alpha, int dtype) {
  return cbh::thunk_matmul(*static_cast<cbh::PCtx*>(c), (cbh::Mode)mode, cc, a, b, m, n, k, ta, tb, alpha, dtype);
}
}
