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
void Arena::init(size_t bytes) {
  cap_ = bytes / kAlign * kAlign; front_ = in_use_ = 0; back_ = cap_; live_.clear(); holes_.clear();
}

size_t Arena::alloc(size_t bytes, bool back) {
  const size_t need = up(bytes ? bytes : 1);
  // first fit in the free list, on the side of the arena the request belongs to
  for (auto it = holes_.begin(); it != holes_.end(); ++it) {
    if (it->second >= need && (it->first >= back_) == back) {
      const size_t off = it->first, rest = it->second - need;
      holes_.erase(it);
      if (rest) holes_[off + need] = rest;
      live_[off] = need; in_use_ += need;
      return off;
    }
  }
  if (front_ + need > back_) return SIZE_MAX;          // the two cursors would cross
  size_t off;
  if (back) { back_ -= need; off = back_; }
  else { off = front_; front_ += need; }
  live_[off] = need; in_use_ += need;
  return off;
}

void Arena::free(size_t off) {
  auto it = live_.find(off);
  if (it == live_.end()) return;
  size_t sz = it->second;
  live_.erase(it); in_use_ -= sz;
  const bool back = off >= back_;
  // coalesce with neighbouring holes of the same side; a hole that touches a bump cursor moves the cursor instead
  auto nx = holes_.find(off + sz);
  if (nx != holes_.end() && (nx->first >= back_) == back) { sz += nx->second; holes_.erase(nx); }
  auto pv = holes_.lower_bound(off);
  if (pv != holes_.begin()) {
    --pv;
    if (pv->first + pv->second == off && (pv->first >= back_) == back) { off = pv->first; sz += pv->second; holes_.erase(pv); }
  }
  if (!back && off + sz == front_) front_ = off;
  else if (back && off == back_) {
    back_ = off + sz;
    // holes that now touch the cursor go with it
    for (auto h = holes_.find(back_); h != holes_.end() && h->first == back_; h = holes_.find(back_)) { back_ += h->second; holes_.erase(h); }
  } else holes_[off] = sz;
}

// ---- CACTI_VMEM_SOFT_LIMIT ---------------------------------------------------------------------------
size_t parse_vmem_soft_limit(const char* text, size_t total, size_t avail) {
  if (!text) return 0;
  while (*text == ' ') ++text;
  char* end = nullptr;
  const double v = std::strtod(text, &end);
  if (end == text || !(v >= 0.0)) return 0;
  const char* q = end;
  while (*q == ' ') ++q;
  size_t bytes;
  if (*q == '\0') {
    // a bare number is a fraction of the device's memory, never all of it (32 MiB stay outside)
    double f = v > 1.0 ? 1.0 : v;
    double b = (double)total * f;
    const double cap = avail > (32u << 20) ? (double)avail - (double)(32u << 20) : 0.0;
    if (b > cap) b = cap;
    bytes = (size_t)b;
  } else {
    double mul = 1.0;
    int power = 0;
    switch (*q) {
      case 'k': case 'K': power = 1; break;
      case 'm': case 'M': power = 2; break;
      case 'g': case 'G': power = 3; break;
      case 't': case 'T': power = 4; break;
      default: break;
    }
    if (power) {
      ++q;
      const double base = (*q == 'i' || *q == 'I') ? (++q, 1024.0) : 1000.0;
      for (int i = 0; i < power; ++i) mul *= base;
    }
    if (*q == 'b' || *q == 'B') ++q;
    while (*q == ' ') ++q;
    if (*q != '\0') return 0;
    bytes = (size_t)(v * mul);
  }
  return bytes >> 16 << 16;
}

// ---- pctx -------------------------------------------------------------------------------------------
PCtx::PCtx(Backend* b, size_t arena_bytes, size_t soft_limit) : be_(b), soft_limit_(soft_limit ? soft_limit : arena_bytes) {
  base_ = static_cast<char*>(be_->arena_alloc(arena_bytes));
  arena_.init(base_ ? arena_bytes : 0);
}
void* PCtx::host_buffer(size_t bytes) {
  auto it = host_pool_.find(bytes);
  if (it != host_pool_.end()) { void* p = it->second; host_pool_.erase(it); return p; }
  return be_->host_alloc(bytes);
}
PCtx::~PCtx() {
  be_->sync();
  for (auto& c : cells_) if (c.host) be_->host_free(c.host);
  for (auto& kv : host_pool_) be_->host_free(kv.second);
  if (base_) be_->arena_free(base_);
  delete be_;
}

int64_t PCtx::cell_new(size_t bytes, bool stable) {
  Cell c; c.bytes = bytes; c.stable = stable;
  if (!free_ids_.empty()) {
    const int64_t id = free_ids_.back();
    free_ids_.pop_back();
    cells_[id] = c;
    return id;
  }
  cells_.push_back(c);
  return (int64_t)cells_.size() - 1;
}

// Frees both replicas.  The device block may be handed out again at once: whatever still reads or writes it was
// launched earlier on the one stream every later use is launched on.
int PCtx::cell_free(int64_t id) {
  if (id < 0 || (size_t)id >= cells_.size()) return 1;
  Cell& c = cells_[id];
  if (c.pins > 0) return 1;
  if (c.dev_off != SIZE_MAX) arena_.free(c.dev_off);
  // the host replica goes to a pool of page-locked buffers: its next use is as the target of a spill copy (ordered
  // on the stream behind any copy still running into it) or in cell_put, which drains the stream first
  if (c.host) host_pool_.emplace(c.bytes, c.host);
  unlive_.erase(id);
  c = Cell();
  c.dead = true;
  free_ids_.push_back(id);
  return 0;
}

// Frees the device replica of c.  must_keep_value: copy it to the host first (a spill).
bool PCtx::evict(int64_t id, bool must_keep_value) {
  Cell& c = cells_[id];
  if (c.dev_off == SIZE_MAX || c.pins > 0) return false;
  if (must_keep_value) {
    if (c.dev_valid && !c.host_valid) {          // the device holds the only current replica: copy it out
      if (!c.host) c.host = host_buffer(c.bytes);
      if (!c.host || be_->d2h(c.host, base_ + c.dev_off, c.bytes)) return false;
      c.host_valid = true;
      ++stats_.spill_copies;
      stats_.spill_bytes += (long long)c.bytes;
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
      if (evict(*it, keep)) {                    // the mark is consumed only by an eviction that happened
        freed = true;
        if (!keep) c.dead = true;
        it = unlive_.erase(it);
      } else {
        ++it;
      }
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

size_t PCtx::alloc_with_policy(size_t bytes, bool back) {
  for (;;) {
    if (arena_.in_use() + up(bytes) <= soft_limit_) {
      const size_t off = arena_.alloc(bytes, back);
      if (off != SIZE_MAX) {
        if (arena_.in_use() > stats_.peak_in_use) stats_.peak_in_use = arena_.in_use();
        return off;
      }
    }
    ++stats_.oom_retries;
    if (!try_soft_oom(bytes)) { ++stats_.hard_oom; return SIZE_MAX; }
  }
}

int PCtx::cell_put(int64_t id, const void* host, size_t bytes) {
  Cell& c = cells_[id];
  if (bytes != c.bytes) return 1;
  if (!c.host) c.host = host_buffer(c.bytes);
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
    const size_t off = alloc_with_policy(cells_[id].bytes, cells_[id].stable);
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
    stats_.reload_bytes += (long long)c.bytes;
  }
  return reinterpret_cast<uint64_t>(base_ + c.dev_off);
}

uint64_t PCtx::pwrite(int64_t id) {
  if (cells_[id].dev_off == SIZE_MAX) {
    const size_t off = alloc_with_policy(cells_[id].bytes, cells_[id].stable);
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
// Pins cells as their pointers are looked up; unpins on scope exit, after the launch has been issued (the one stream
// orders every later spill, free or re-use behind it).  Temporaries (workspaces) are cells that die with the scope.
struct Binding {
  PCtx& p; std::vector<int64_t> pinned, temps; bool ok = true;
  explicit Binding(PCtx& p_) : p(p_) {}
  uint64_t in(int64_t c) { uint64_t d = p.pread(c); if (!d) ok = false; else { p.pin(c); pinned.push_back(c); } return d; }
  uint64_t out(int64_t c, Mode m) {
    uint64_t d = m == kApply ? p.pwrite(c) : p.prewrite(c);
    if (!d) ok = false; else { p.pin(c); pinned.push_back(c); }
    return d;
  }
  uint64_t opt_in(int64_t c) { return c < 0 ? 0 : in(c); }
  uint64_t opt_out(int64_t c, Mode m) { return c < 0 ? 0 : out(c, m); }
  uint64_t temp(size_t bytes) {
    if (!bytes) return 0;
    const int64_t c = p.cell_new(bytes, false);
    temps.push_back(c);
    return out(c, kApply);
  }
  ~Binding() {
    if (p.sync_each_thunk) p.sync();
    for (int64_t c : pinned) p.unpin(c);
    for (int64_t c : temps) p.cell_free(c);
  }
};
size_t esize(int dtype) { return dtype == CACTI_B200_R_32F ? 4 : 2; }
int beta_of(Mode m) { return m == kAccumulate ? 1 : 0; }
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
  const uint64_t dt = b.temp((size_t)rows * cols * esize(dtype)), dy = b.out(y, kAccumulate);
  if (!b.ok) return -1;
  int rc = cacti_b200_rmsnorm_fwd(dt, dx, dg, eps, rows, cols, dtype, p.stream());
  if (!rc) rc = cacti_b200_accumulate(dy, dt, rows * cols, dtype, p.stream());
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

int thunk_rmsnorm_bwd(PCtx& p, Mode m_dx, Mode m_dgamma, int64_t dx, int64_t dgamma, int64_t dy, int64_t x, int64_t gamma, float eps,
                      int64_t rows, int64_t cols, int dtype, int dgamma_dtype) {
  if (m_dx == kInitialize || m_dgamma == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t ddy = b.in(dy), dxx = b.in(x), dg = b.in(gamma);
  const uint64_t ddx = b.out(dx, m_dx), ddg = b.out(dgamma, m_dgamma);
  const size_t wsb = cacti_b200_rmsnorm_workspace_bytes(rows, cols);
  const uint64_t ws = b.temp(wsb);                    // the column partials live in a cell of the same arena
  if (!b.ok) return -1;
  return cacti_b200_rmsnorm_bwd(ddx, ddg, ddy, dxx, dg, eps, rows, cols, dtype, dgamma_dtype, beta_of(m_dx), beta_of(m_dgamma), ws, wsb,
                                p.stream());
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
  if (m == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t ds_ = b.in(s), dp_ = b.in(dpr), out = b.out(dsc, m);
  if (!b.ok) return -1;
  return cacti_b200_softmax_bwd(out, ds_, dp_, rows, cols, q_div > 0 ? CACTI_B200_MASK_CAUSAL : CACTI_B200_MASK_NONE,
                                q_div > 0 ? q_div : 1, q_mod > 0 ? q_mod : 1, 0, dtype, m == kAccumulate, p.stream());
}

int thunk_add(PCtx& p, Mode m, int64_t out, int64_t a, int64_t bb, int64_t n, int dtype) {
  if (m == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t da = b.in(a), db = b.in(bb);
  if (m == kApply) {
    const uint64_t d = b.out(out, kApply);
    if (!b.ok) return -1;
    return cacti_b200_add(d, da, db, n, dtype, p.stream());
  }
  // out += T(a + b): the sum is rounded to the cell type once before the accumulate, as the reference's out-of-place
  // accumulate does (src/thunk/mod.rs:1691-1733), not added in two separately rounded steps
  const uint64_t dt = b.temp((size_t)n * esize(dtype)), d = b.out(out, kAccumulate);
  if (!b.ok) return -1;
  int rc = cacti_b200_add(dt, da, db, n, dtype, p.stream());
  if (!rc) rc = cacti_b200_accumulate(d, dt, n, dtype, p.stream());
  return rc;
}

int thunk_matmul(PCtx& p, Mode m, int64_t c, int64_t a, int64_t bb, int64_t mm, int64_t nn, int64_t kk, int ta, int tb,
                 float alpha, int dtype) {
  if (m == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t da = b.in(a), db = b.in(bb), dc = b.out(c, m);
  const float beta = m == kAccumulate ? 1.f : 0.f;      // src/thunk/op.rs:5053-5067
  const int64_t lda = ta ? mm : kk, ldb = tb ? kk : nn;
  // cells start 256-byte aligned, so only a row pitch that is not a multiple of 16 bytes needs the repack workspace
  size_t wsb = 0;
  if ((lda * 2) % 16 || (ldb * 2) % 16) wsb = cacti_b200_gemm_workspace_bytes(mm, nn, kk, 1, 1);
  const uint64_t ws = b.temp(wsb);
  if (!b.ok) return -1;
  return cacti_b200_gemm(dc, da, db, mm, nn, kk, lda, ldb, nn, ta, tb, &alpha, &beta, dtype, ws, wsb, p.stream());
}

int thunk_rope_fwd(PCtx& p, Mode m, int64_t y, int64_t x, int64_t cos, int64_t sin, int64_t tokens, int64_t heads, int64_t hd,
                   int64_t pos_mod, int64_t head_pitch, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dx = b.in(x), dc = b.in(cos), ds = b.in(sin), dy = b.out(y, kApply);
  if (!b.ok) return -1;
  if (head_pitch > 0)
    return cacti_b200_rope_fwd_pitched(dy, dx, dc, ds, tokens, heads, hd, head_pitch, pos_mod, 0, dtype, p.stream());
  return cacti_b200_rope_fwd(dy, dx, dc, ds, tokens, heads, hd, pos_mod, 0, dtype, p.stream());
}

int thunk_rope_bwd(PCtx& p, Mode m, int64_t dx, int64_t dy, int64_t cos, int64_t sin, int64_t tokens, int64_t heads, int64_t hd,
                   int64_t pos_mod, int dtype) {
  if (m == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t ddy = b.in(dy), dc = b.in(cos), ds = b.in(sin), ddx = b.out(dx, m);
  if (!b.ok) return -1;
  return cacti_b200_rope_bwd(ddx, ddy, dc, ds, tokens, heads, hd, pos_mod, 0, dtype, beta_of(m), p.stream());
}

int thunk_swiglu_fwd(PCtx& p, Mode m, int64_t h, int64_t gate, int64_t up_, int64_t n, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dg = b.in(gate), du = b.in(up_), dh = b.out(h, kApply);
  if (!b.ok) return -1;
  return cacti_b200_swiglu_fwd(dh, dg, du, n, dtype, p.stream());
}

int thunk_swiglu_bwd(PCtx& p, Mode m_dgate, Mode m_dup, int64_t dgate, int64_t dup, int64_t gate, int64_t up_, int64_t dh, int64_t n,
                     int dtype) {
  if (m_dgate == kInitialize || m_dup == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dg = b.in(gate), du = b.in(up_), ddh = b.in(dh);
  const uint64_t o1 = b.out(dgate, m_dgate), o2 = b.out(dup, m_dup);
  if (!b.ok) return -1;
  return cacti_b200_swiglu_bwd(o1, o2, dg, du, ddh, n, dtype, beta_of(m_dgate), beta_of(m_dup), p.stream());
}

int thunk_softmax_nll(PCtx& p, Mode m_dlogits, int64_t loss_sum, int64_t dlogits, int64_t logits, int64_t targets, int target_dtype,
                      float w, int64_t rows, int64_t vocab, int dtype, int64_t status) {
  if (m_dlogits == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dl = b.in(logits), dt = b.in(targets);
  const uint64_t dsum = b.opt_out(loss_sum, kApply), dd = b.opt_out(dlogits, m_dlogits), dst = b.opt_out(status, kAccumulate);
  const size_t wsb = cacti_b200_softmax_nll_workspace_bytes(rows);
  const uint64_t ws = b.temp(wsb);
  if (!b.ok) return -1;
  return cacti_b200_softmax_nll_fwd_bwd(dsum, 0, dd, dl, dt, target_dtype, 0, w, rows, vocab, dtype, beta_of(m_dlogits), dst, ws, wsb,
                                        p.stream());
}

int thunk_gather_rows(PCtx& p, Mode m, int64_t out, int64_t table, int64_t tokens, int token_dtype, int64_t n, int64_t vocab,
                      int64_t cols, int dtype, int64_t status) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dt = b.in(table), dk = b.in(tokens), d = b.out(out, kApply), dst = b.opt_out(status, kAccumulate);
  if (!b.ok) return -1;
  return cacti_b200_gather_rows(d, dt, dk, token_dtype, n, vocab, cols, dtype, dst, p.stream());
}

int thunk_scatter_add_rows(PCtx& p, Mode m, int64_t dtable, int64_t dy, int64_t tokens, int token_dtype, int64_t n, int64_t vocab,
                           int64_t cols, int dtype, int64_t status) {
  if (m == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t ddy = b.in(dy), dk = b.in(tokens), d = b.out(dtable, m), dst = b.opt_out(status, kAccumulate);
  const size_t wsb = cacti_b200_scatter_add_rows_workspace_bytes(n, vocab);
  const uint64_t ws = b.temp(wsb);
  if (!b.ok) return -1;
  return cacti_b200_scatter_add_rows(d, ddy, dk, token_dtype, n, vocab, cols, dtype, beta_of(m), ws, wsb, dst, p.stream());
}

int thunk_block_pad(PCtx& p, Mode m, int64_t dst, int64_t src, int64_t nrow, int64_t rows, int64_t ncol, int64_t cols, int64_t cols_pad,
                    int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t ds = b.in(src), dd = b.out(dst, kApply);
  if (!b.ok) return -1;
  return cacti_b200_block_pad(dd, ds, nrow, rows, ncol, cols, cols_pad, dtype, p.stream());
}

// Strides of the reference's packed 4-d block layout [nrow, rows, ncol, ld] (src/thunk/op.rs:5121-5123, :5174-5189)
int thunk_block_matmul(PCtx& p, Mode m, int64_t c, int64_t a, int64_t bb, int64_t nrow, int64_t ncol, int64_t mm, int64_t nn, int64_t kk,
                       int64_t a_ld, int64_t b_ld, int ta, int tb, float alpha, int tri, int64_t diag, int flags, int dtype) {
  if (m == kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t da = b.in(a), db = b.in(bb), dc = b.out(c, m);
  const float beta = m == kAccumulate ? 1.f : 0.f;
  const int64_t a_rows = ta ? kk : mm, b_rows = tb ? nn : kk;
  const int64_t lda = ncol * a_ld, ldb = ncol * b_ld, ldc = ncol * nn;
  // cells start 256-byte aligned: the repack workspace is needed only when a row pitch or a block stride is not a
  // multiple of 16 bytes (head_dim 100 unpadded), and then it is a cell like any other
  const bool aligned = (lda * 2) % 16 == 0 && (ldb * 2) % 16 == 0 && (a_ld * 2) % 16 == 0 && (b_ld * 2) % 16 == 0;
  const size_t wsb = aligned ? 0 : cacti_b200_gemm_workspace_bytes(mm, nn, kk, nrow, ncol);
  const uint64_t ws = b.temp(wsb);
  if (!b.ok) return -1;
  return cacti_b200_gemm_strided_batched_tri(dc, da, db, mm, nn, kk, lda, ldb, ldc, ta, tb, &alpha, &beta, nrow, ncol, a_rows * lda, a_ld,
                                             b_rows * ldb, b_ld, mm * ldc, nn, tri, diag, flags, dtype, ws, wsb, p.stream());
}

int thunk_attention_fwd(PCtx& p, Mode m, int64_t ctx, int64_t stats, int64_t q, int64_t k, int64_t v, int64_t batch, int64_t seq,
                        int64_t heads, int64_t hd, float alpha, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dq = b.in(q), dk = b.in(k), dv = b.in(v), dc = b.out(ctx, kApply), dst = b.out(stats, kApply);
  if (!b.ok) return -1;
  return cacti_b200_attention_fwd(dc, dst, dq, dk, dv, batch, seq, heads, hd, alpha, dtype, p.stream());
}

int thunk_attention_bwd_prep(PCtx& p, Mode m, int64_t prob, int64_t ds, int64_t q, int64_t k, int64_t v, int64_t dctx, int64_t ctx,
                             int64_t stats, int64_t batch, int64_t seq, int64_t heads, int64_t hd, float alpha, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dq = b.in(q), dk = b.in(k), dv = b.in(v), ddc = b.in(dctx), dc = b.in(ctx);
  const uint64_t dst = b.out(stats, kInitialize);        // two of its words are scratch of this thunk
  const uint64_t dp = b.out(prob, kApply), dds = b.out(ds, kApply);
  if (!b.ok) return -1;
  return cacti_b200_attention_bwd_prep(dp, dds, dq, dk, dv, ddc, dc, dst, batch, seq, heads, hd, alpha, dtype, p.stream());
}

int thunk_attention_bwd(PCtx& p, Mode m, int64_t dq, int64_t dk, int64_t dv, int64_t q, int64_t k, int64_t v, int64_t dctx, int64_t ctx,
                        int64_t stats, int64_t batch, int64_t seq, int64_t heads, int64_t hd, float alpha, int dtype) {
  if (m != kApply) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t pq = b.in(q), pk = b.in(k), pv = b.in(v), pdc = b.in(dctx), pc = b.in(ctx);
  const uint64_t pst = b.out(stats, kInitialize);        // two of its words are scratch of this thunk
  const uint64_t o1 = b.out(dq, kApply), o2 = b.out(dk, kApply), o3 = b.out(dv, kApply);
  if (!b.ok) return -1;
  return cacti_b200_attention_bwd(o1, o2, o3, pq, pk, pv, pdc, pc, pst, batch, seq, heads, hd, alpha, dtype, p.stream());
}

int thunk_adamw32_step(PCtx& p, Mode m, int64_t master, int64_t grad1_avg, int64_t grad2_avg, int64_t param_out, int64_t grad, int64_t n,
                       int grad_dtype, int param_dtype, float grad_unscale, float lr, float wd, float a1, float a2, float eps, int iter_nr) {
  if (m != kInitialize) return CACTI_B200_ERR_INVALID_VALUE;
  Binding b(p);
  const uint64_t dg = b.in(grad);
  const uint64_t dw = b.out(master, kInitialize), d1 = b.out(grad1_avg, kInitialize), d2 = b.out(grad2_avg, kInitialize);
  const uint64_t dp = b.opt_out(param_out, kApply);
  if (!b.ok) return -1;
  return cacti_b200_adamw32_step(dw, d1, d2, dp, dg, n, grad_dtype, param_dtype, grad_unscale, lr, wd, a1, a2, eps, iter_nr, p.stream());
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
#define CBH_P (*static_cast<cbh::PCtx*>(c))
#define CBH_M(x) ((cbh::Mode)(x))
int cbh_cell_free(void* c, int64_t cell) { return CBH_P.cell_free(cell); }
size_t cbh_soft_limit(void* c) { return CBH_P.soft_limit(); }
void* cbh_stream(void* c) { return CBH_P.stream(); }
size_t cbh_parse_vmem_soft_limit(const char* text, size_t total, size_t avail) { return cbh::parse_vmem_soft_limit(text, total, avail); }
void cbh_stats_bytes(void* c, long long* out3) {
  const cbh::Stats& s = CBH_P.stats();
  out3[0] = s.spill_bytes; out3[1] = s.reload_bytes; out3[2] = (long long)s.peak_in_use;
}
// arena alone, for the allocator tests: returns the offset or SIZE_MAX
void* cbh_arena_create(size_t bytes) { cbh::Arena* a = new cbh::Arena; a->init(bytes); return a; }
void cbh_arena_destroy(void* a) { delete static_cast<cbh::Arena*>(a); }
size_t cbh_arena_alloc(void* a, size_t bytes, int back) { return static_cast<cbh::Arena*>(a)->alloc(bytes, back != 0); }
void cbh_arena_free(void* a, size_t off) { static_cast<cbh::Arena*>(a)->free(off); }
size_t cbh_arena_front(void* a) { return static_cast<cbh::Arena*>(a)->front(); }
size_t cbh_arena_back(void* a) { return static_cast<cbh::Arena*>(a)->back(); }
size_t cbh_arena_in_use(void* a) { return static_cast<cbh::Arena*>(a)->in_use(); }
int cbh_thunk_rmsnorm_bwd(void* c, int m_dx, int m_dg, int64_t dx, int64_t dgamma, int64_t dy, int64_t x, int64_t gamma, float eps,
                          int64_t rows, int64_t cols, int dtype, int dgamma_dtype) {
  return cbh::thunk_rmsnorm_bwd(CBH_P, CBH_M(m_dx), CBH_M(m_dg), dx, dgamma, dy, x, gamma, eps, rows, cols, dtype, dgamma_dtype);
}
int cbh_thunk_rope_fwd(void* c, int mode, int64_t y, int64_t x, int64_t cos, int64_t sin, int64_t tokens, int64_t heads, int64_t hd,
                       int64_t pos_mod, int64_t head_pitch, int dtype) {
  return cbh::thunk_rope_fwd(CBH_P, CBH_M(mode), y, x, cos, sin, tokens, heads, hd, pos_mod, head_pitch, dtype);
}
int cbh_thunk_rope_bwd(void* c, int mode, int64_t dx, int64_t dy, int64_t cos, int64_t sin, int64_t tokens, int64_t heads, int64_t hd,
                       int64_t pos_mod, int dtype) {
  return cbh::thunk_rope_bwd(CBH_P, CBH_M(mode), dx, dy, cos, sin, tokens, heads, hd, pos_mod, dtype);
}
int cbh_thunk_swiglu_fwd(void* c, int mode, int64_t h, int64_t gate, int64_t up, int64_t n, int dtype) {
  return cbh::thunk_swiglu_fwd(CBH_P, CBH_M(mode), h, gate, up, n, dtype);
}
int cbh_thunk_swiglu_bwd(void* c, int m_dgate, int m_dup, int64_t dgate, int64_t dup, int64_t gate, int64_t up, int64_t dh, int64_t n, int dtype) {
  return cbh::thunk_swiglu_bwd(CBH_P, CBH_M(m_dgate), CBH_M(m_dup), dgate, dup, gate, up, dh, n, dtype);
}
int cbh_thunk_softmax_nll(void* c, int m_dlogits, int64_t loss_sum, int64_t dlogits, int64_t logits, int64_t targets, int target_dtype,
                          float w, int64_t rows, int64_t vocab, int dtype, int64_t status) {
  return cbh::thunk_softmax_nll(CBH_P, CBH_M(m_dlogits), loss_sum, dlogits, logits, targets, target_dtype, w, rows, vocab, dtype, status);
}
int cbh_thunk_gather_rows(void* c, int mode, int64_t out, int64_t table, int64_t tokens, int token_dtype, int64_t n, int64_t vocab,
                          int64_t cols, int dtype, int64_t status) {
  return cbh::thunk_gather_rows(CBH_P, CBH_M(mode), out, table, tokens, token_dtype, n, vocab, cols, dtype, status);
}
int cbh_thunk_scatter_add_rows(void* c, int mode, int64_t dtable, int64_t dy, int64_t tokens, int token_dtype, int64_t n, int64_t vocab,
                               int64_t cols, int dtype, int64_t status) {
  return cbh::thunk_scatter_add_rows(CBH_P, CBH_M(mode), dtable, dy, tokens, token_dtype, n, vocab, cols, dtype, status);
}
int cbh_thunk_block_pad(void* c, int mode, int64_t dst, int64_t src, int64_t nrow, int64_t rows, int64_t ncol, int64_t cols, int64_t cols_pad,
                        int dtype) {
  return cbh::thunk_block_pad(CBH_P, CBH_M(mode), dst, src, nrow, rows, ncol, cols, cols_pad, dtype);
}
int cbh_thunk_block_matmul(void* c, int mode, int64_t cc, int64_t a, int64_t b, int64_t nrow, int64_t ncol, int64_t m, int64_t n, int64_t k,
                           int64_t a_ld, int64_t b_ld, int ta, int tb, float alpha, int tri, int64_t diag, int flags, int dtype) {
  return cbh::thunk_block_matmul(CBH_P, CBH_M(mode), cc, a, b, nrow, ncol, m, n, k, a_ld, b_ld, ta, tb, alpha, tri, diag, flags, dtype);
}
int cbh_thunk_attention_fwd(void* c, int mode, int64_t ctx, int64_t stats, int64_t q, int64_t k, int64_t v, int64_t batch, int64_t seq,
                            int64_t heads, int64_t hd, float alpha, int dtype) {
  return cbh::thunk_attention_fwd(CBH_P, CBH_M(mode), ctx, stats, q, k, v, batch, seq, heads, hd, alpha, dtype);
}
int cbh_thunk_attention_bwd_prep(void* c, int mode, int64_t prob, int64_t ds, int64_t q, int64_t k, int64_t v, int64_t dctx, int64_t ctx,
                                 int64_t stats, int64_t batch, int64_t seq, int64_t heads, int64_t hd, float alpha, int dtype) {
  return cbh::thunk_attention_bwd_prep(CBH_P, CBH_M(mode), prob, ds, q, k, v, dctx, ctx, stats, batch, seq, heads, hd, alpha, dtype);
}
int cbh_thunk_attention_bwd(void* c, int mode, int64_t dq, int64_t dk, int64_t dv, int64_t q, int64_t k, int64_t v, int64_t dctx,
                            int64_t ctx, int64_t stats, int64_t batch, int64_t seq, int64_t heads, int64_t hd, float alpha, int dtype) {
  return cbh::thunk_attention_bwd(CBH_P, CBH_M(mode), dq, dk, dv, q, k, v, dctx, ctx, stats, batch, seq, heads, hd, alpha, dtype);
}
int cbh_thunk_adamw32_step(void* c, int mode, int64_t master, int64_t g1, int64_t g2, int64_t param_out, int64_t grad, int64_t n,
                           int grad_dtype, int param_dtype, float grad_unscale, float lr, float wd, float a1, float a2, float eps, int iter_nr) {
  return cbh::thunk_adamw32_step(CBH_P, CBH_M(mode), master, g1, g2, param_out, grad, n, grad_dtype, param_dtype, grad_unscale, lr, wd, a1,
                                 a2, eps, iter_nr);
}
#undef CBH_P
#undef CBH_M
}
