// K1: RMSNorm forward / backward / fused forward+backward.
//
// Replaces the reference's rms_norm closure (src/librarium/llama.rs:442-451): cast -> square ->
// inner_mean -> add eps -> sqrt -> broadcast div -> broadcast mul -> lossy cast, eight primitive
// thunks forward and about fourteen backward, each a separate Futhark program.  Here one kernel
// reads x (and dy) once, keeps the row in registers, and writes y (and dx) once; the two row sums
// the fused form needs (sum x^2 and sum gamma*dy*x) are reduced together.
//
// dgamma is a sum over rows.  Each CTA walks its rows with every thread owning fixed columns, so
// the per-thread dgamma terms accumulate in registers; at the end the CTA folds its row groups
// through shared memory and writes one f32 partial row.  A second small kernel adds the partials
// in a fixed order.  No floating-point atomics: results are run-to-run identical, as the
// reference's cuBLAS setup also demands (cacti_gpu_cu_ffi/src/lib.rs:749).
#include "common.cuh"
#include <atomic>

namespace cb {

int g_rmsnorm_threads = 512;      // target threads per CTA on the vector path
int g_rmsnorm_gpref = 256;        // preferred threads per row group
int g_rmsnorm_smem_kb = 96;       // shared memory per CTA spent on the row ring
int g_rmsnorm_bulk_out = 1;       // 1: outputs leave by bulk stores from shared memory; 0: by per-thread streaming stores

constexpr int kRmsMaxPartials = kNumSMs * 8;

// ADD (forward only): the normalised row is T(X + R), the residual add that precedes every norm of the decoder
// layer (src/librarium/llama.rs:514,533); the rounded sum is also written to SUM.  The second stage row then holds R.
template <typename T, int NV, bool FWD, bool BWD, bool ADD = false, bool ACC = false>
__global__ void __launch_bounds__(512)
rmsnorm_rows_kernel(T* __restrict__ Y, T* __restrict__ dX, float* __restrict__ partial,
                    const T* __restrict__ X, const T* __restrict__ gamma, const T* __restrict__ dY,
                    float eps, int64_t rows, int cols, int G, int nstages, int beta_dx,
                    const T* __restrict__ R = nullptr, T* __restrict__ SUM = nullptr, int bulk_out_arg = 0) {
  static_assert(!ADD || (FWD && !BWD), "the residual add is fused into the forward norm only");
  static_assert(!ACC || BWD, "ACC is the Accumulate mode of the adjoint");
  const int bulk_out = BWD ? 0 : bulk_out_arg;      // the backward kernels carry no bulk-store code (see launch_rmsnorm)
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int VEC = Elem<T>::VEC;
  const int groups = blockDim.x / G;
  const unsigned row_bytes = (unsigned)cols * sizeof(T);
  // Accumulate mode of the adjoint (dX += ...): the old dX row rides in the stage behind x and dy
  constexpr bool acc_dx = ACC;          // (a kernel of its own: the overwrite forms keep their code and registers)
  const unsigned stage_bytes = row_bytes * ((BWD || ADD) ? 2 : 1) + (acc_dx ? row_bytes : 0u);
  // shared: [groups][nstages] stage buffers (x row, dy row[, old dx row]) | mbarriers | reduction slots | dgamma fold [cols]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)groups * nstages * stage_bytes);
  float* red = reinterpret_cast<float*>(bars + groups * nstages);
  float* colacc = red + (size_t)2 * groups * kMaxWarpsPerGroup * 2;
  GroupCtx g = make_group(G, red);
  unsigned char* stage0 = smem_raw + (size_t)g.gid * nstages * stage_bytes;
  uint64_t* bar0 = bars + g.gid * nstages;
  if (g.lane < nstages) mbar_init(bar0 + g.lane, 1);
  mbar_fence_init();
  __syncthreads();
  const float inv_cols = 1.f / (float)cols;

  uint4 graw[NV];       // gamma for this thread's columns, raw
  float dg[NV][VEC];    // dgamma accumulators
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int col0 = (g.lane + k * G) * VEC;
    if (col0 < cols) graw[k] = ld_keep(gamma + col0);
#pragma unroll
    for (int e = 0; e < VEC; ++e) dg[k][e] = 0.f;
  }

  const int64_t stride = (int64_t)gridDim.x * groups;
  const int64_t row0 = (int64_t)blockIdx.x * groups + g.gid;
  // a ring of nstages rows per group keeps (nstages - 1) rows in flight while one is reduced
  auto issue = [&](int64_t r, int sl) {
    if (g.lane == 0) {
      unsigned char* dst = stage0 + (size_t)sl * stage_bytes;
      mbar_expect_tx(bar0 + sl, stage_bytes);
      bulk_g2s(dst, X + r * cols, row_bytes, bar0 + sl);
      if (BWD) bulk_g2s(dst + row_bytes, dY + r * cols, row_bytes, bar0 + sl);
      if (acc_dx) bulk_g2s(dst + 2 * row_bytes, dX + r * cols, row_bytes, bar0 + sl);
      if (ADD) bulk_g2s(dst + row_bytes, R + r * cols, row_bytes, bar0 + sl);
    }
  };
  for (int sl = 0; sl < nstages; ++sl)
    if (row0 + sl * stride < rows) issue(row0 + sl * stride, sl);
  int slot = 0;
  unsigned phase = 0;
  bool alive = true;
  // bulk_out: the output rows are assembled in one of two shared-memory buffers of the group and leave by bulk
  // stores, so that the copy engine carries all the traffic of the row and the threads never wait on a store; a
  // buffer is reused two rows later, after lane 0 has seen the store that read it finish reading.
  constexpr int kOutRows = (ADD || (FWD && BWD)) ? 2 : 1;
  const unsigned out_bytes = row_bytes * kOutRows;
  unsigned char* outbuf0 = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(colacc + (BWD ? cols : 0)) + 15) & ~(uintptr_t)15) + (size_t)g.gid * 2 * out_bytes;
  unsigned it = 0;
  for (int64_t row = row0; row < rows; row += stride) {
    // a wait that ran out is agreed on by the whole group at the reduction's barrier below: no lane leaves alone
    bool gave_up = !mbar_wait_bounded(bar0 + slot, phase, kDevErrStageTimeout);
    const unsigned char* stage = stage0 + (size_t)slot * stage_bytes;
    unsigned char* ob = outbuf0 + (size_t)(it & 1) * out_bytes;
    ++it;
    if (bulk_out && g.lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    uint4 xraw[NV], yraw[NV], oraw[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) {
        xraw[k] = *reinterpret_cast<const uint4*>(stage + (size_t)col0 * sizeof(T));
        if (BWD) yraw[k] = *reinterpret_cast<const uint4*>(stage + row_bytes + (size_t)col0 * sizeof(T));
        if (acc_dx) oraw[k] = *reinterpret_cast<const uint4*>(stage + 2 * row_bytes + (size_t)col0 * sizeof(T));
        if (ADD) {
          float a[VEC], b[VEC];
          unpack<T>(xraw[k], a);
          unpack<T>(*reinterpret_cast<const uint4*>(stage + row_bytes + (size_t)col0 * sizeof(T)), b);
#pragma unroll
          for (int e = 0; e < VEC; ++e) a[e] = __fadd_rn(a[e], b[e]);
          xraw[k] = pack<T>(a);                  // rounded to T: what a separate add would have stored
          if (!bulk_out) st_stream(SUM + row * cols + col0, xraw[k]);
        }
      }
    }
    const int cur_slot = slot;
    if (++slot == nstages) { slot = 0; phase ^= 1; }

    // pass 1: ss = sum x^2, c1 = sum gamma*dy*x
    float sq[4] = {0.f, 0.f, 0.f, 0.f}, cq[4] = {0.f, 0.f, 0.f, 0.f};   // independent chains
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) {
        float x[VEC];
        unpack<T>(xraw[k], x);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sq[e & 3] = __fmaf_rn(x[e], x[e], sq[e & 3]);
        if (BWD) {
          float gy[VEC], gm[VEC];
          unpack<T>(yraw[k], gy);
          unpack<T>(graw[k], gm);
#pragma unroll
          for (int e = 0; e < VEC; ++e) cq[e & 3] = __fmaf_rn(__fmul_rn(gm[e], gy[e]), x[e], cq[e & 3]);
        }
      }
    }
    float ss = __fadd_rn(__fadd_rn(sq[0], sq[1]), __fadd_rn(sq[2], sq[3]));
    float c1 = __fadd_rn(__fadd_rn(cq[0], cq[1]), __fadd_rn(cq[2], cq[3]));
    group_reduce2<SumOp>(g, ss, c1, &gave_up);   // its barrier also orders every lane's reads of the stage slot
    if (gave_up) { alive = false; break; }
    if (G == 32) __syncwarp();
    if (row + (int64_t)nstages * stride < rows) issue(row + (int64_t)nstages * stride, cur_slot);
    const float s = __fsqrt_rn(__fmaf_rn(ss, inv_cols, eps));
    const float rs = __frcp_rn(s);
    // c1 / (cols * s^3); explicitly rounded ops so that fwd, bwd and fwd_bwd give the same bits
    const float coef = BWD ? __fmul_rn(__fmul_rn(__fmul_rn(c1, inv_cols), rs), __fmul_rn(rs, rs)) : 0.f;
    // pass 2: outputs
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) {
        float x[VEC], gm[VEC], t[VEC];
        unpack<T>(xraw[k], x);
        unpack<T>(graw[k], gm);
#pragma unroll
        for (int e = 0; e < VEC; ++e) t[e] = __fmul_rn(x[e], rs);
        if (FWD) {
          float y[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) y[e] = __fmul_rn(gm[e], t[e]);
          if (bulk_out) {
            if (ADD) *reinterpret_cast<uint4*>(ob + (size_t)col0 * sizeof(T)) = xraw[k];
            *reinterpret_cast<uint4*>(ob + (ADD ? row_bytes : 0u) + (size_t)col0 * sizeof(T)) = pack<T>(y);
          } else {
            st_stream(Y + row * cols + col0, pack<T>(y));
          }
        }
        if (BWD) {
          float gy[VEC], d[VEC];
          unpack<T>(yraw[k], gy);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            dg[k][e] = __fmaf_rn(gy[e], t[e], dg[k][e]);
            d[e] = __fmaf_rn(__fmul_rn(gm[e], gy[e]), rs, -__fmul_rn(x[e], coef));
          }
          T* o = dX + row * cols + col0;
          if (acc_dx) st_stream(o, pack_accumulate<T>(d, oraw[k]));
          else if (bulk_out) *reinterpret_cast<uint4*>(ob + (FWD ? row_bytes : 0u) + (size_t)col0 * sizeof(T)) = pack<T>(d);
          else st_stream(o, pack<T>(d));
        }
      }
    }
    if (bulk_out) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      group_barrier(g);
      if (g.lane == 0) {
        if (ADD) {
          bulk_s2g(SUM + row * cols, ob, row_bytes);
          bulk_s2g(Y + row * cols, ob + row_bytes, row_bytes);
        } else {
          if (FWD) bulk_s2g(Y + row * cols, ob, row_bytes);
          if (BWD) bulk_s2g(dX + row * cols, ob + (FWD ? row_bytes : 0u), row_bytes);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
  }
  (void)alive;
  if (bulk_out && g.lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");

  if (BWD) {
    dependents_may_launch();      // the finalize kernel may be scheduled while the last CTAs fold their partials
    // fold the CTA's row groups in group order, then one partial row per CTA
    for (int q = 0; q < groups; ++q) {
      if (g.gid == q) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int col0 = (g.lane + k * G) * VEC;
          if (col0 < cols) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              if (q == 0) colacc[col0 + e] = dg[k][e];
              else colacc[col0 + e] += dg[k][e];
            }
          }
        }
      }
      __syncthreads();
    }
    float* prow = partial + (size_t)blockIdx.x * cols;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) prow[j] = colacc[j];
  }
}

// dgamma[j] (+)= sum_p partial[p][j], p in increasing order within fixed slices.
template <typename TO>
__global__ void __launch_bounds__(512)
rmsnorm_dgamma_finalize_kernel(TO* __restrict__ dgamma, const float* __restrict__ partial, int nparts, int cols,
                               int beta) {
  __shared__ float sm[16][33];
  const int cx = threadIdx.x & 31, sy = threadIdx.x >> 5;     // 32 columns x 16 slices
  const int j = blockIdx.x * 32 + cx;
  float acc = 0.f;
  dependent_wait();                                           // the partial rows come from the kernel before this one
  if (j < cols) for (int p = sy; p < nparts; p += 16) acc += partial[(size_t)p * cols + j];
  sm[sy][cx] = acc;
  __syncthreads();
  if (sy == 0 && j < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) t += sm[i][cx];
    if (beta) dgamma[j] = Elem<TO>::from_f32(Elem<TO>::to_f32(dgamma[j]) + round_to<TO>(t));
    else dgamma[j] = Elem<TO>::from_f32(t);
  }
}

// Element-wise fallback (any cols / alignment): one CTA per row; 1/s per row goes to the workspace
// so that a column kernel can form dgamma without atomics.
template <typename T, bool FWD, bool BWD>
__global__ void __launch_bounds__(256)
rmsnorm_rows_generic_kernel(T* __restrict__ Y, T* __restrict__ dX, float* __restrict__ row_s,
                            const T* __restrict__ X, const T* __restrict__ gamma, const T* __restrict__ dY,
                            float eps, int64_t rows, int64_t cols, int beta_dx) {
  __shared__ float sm[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* x = X + row * cols;
    float ss = 0.f, c1 = 0.f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
      const float xv = Elem<T>::to_f32(x[j]);
      ss = fmaf(xv, xv, ss);
      if (BWD) c1 = fmaf(Elem<T>::to_f32(gamma[j]) * Elem<T>::to_f32(dY[row * cols + j]), xv, c1);
    }
    ss = block_reduce<SumOp>(ss, sm);
    if (BWD) c1 = block_reduce<SumOp>(c1, sm);
    const float s = sqrtf(ss / (float)cols + eps);
    const float coef = BWD ? c1 / (s * s) / (s + s) / (float)cols * 2.f : 0.f;
    if (BWD && threadIdx.x == 0) row_s[row] = s;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
      const float xv = Elem<T>::to_f32(x[j]), gm = Elem<T>::to_f32(gamma[j]);
      if (FWD) Y[row * cols + j] = Elem<T>::from_f32(gm * (xv / s));
      if (BWD) {
        const float d = (gm * Elem<T>::to_f32(dY[row * cols + j])) / s - xv * coef;
        T* o = dX + row * cols + j;
        *o = beta_dx ? Elem<T>::from_f32(Elem<T>::to_f32(*o) + round_to<T>(d)) : Elem<T>::from_f32(d);
      }
    }
  }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_dgamma_generic_kernel(TO* __restrict__ dgamma, const float* __restrict__ row_s, const T* __restrict__ X,
                              const T* __restrict__ dY, int64_t rows, int64_t cols, int beta) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= cols) return;
  float acc = 0.f;
  for (int64_t i = 0; i < rows; ++i)
    acc = fmaf(Elem<T>::to_f32(dY[i * cols + j]), Elem<T>::to_f32(X[i * cols + j]) / row_s[i], acc);
  if (beta) dgamma[j] = Elem<TO>::from_f32(Elem<TO>::to_f32(dgamma[j]) + round_to<TO>(acc));
  else dgamma[j] = Elem<TO>::from_f32(acc);
}

static size_t rmsnorm_ws_bytes(int64_t rows, int64_t cols, int max_partials = kRmsMaxPartials) {
  size_t a = (size_t)max_partials * (size_t)cols * sizeof(float);
  size_t b = (size_t)rows * sizeof(float);
  return (a > b ? a : b) + 256;
}

// Returns -1 (nothing launched) when ADD is set and the shape does not fit the row kernel.
template <typename T, typename TO, bool FWD, bool BWD, bool ADD = false>
static int launch_rmsnorm(uint64_t y, uint64_t dx, uint64_t dgamma, uint64_t x, uint64_t gamma, uint64_t dy,
                          float eps, int64_t rows, int64_t cols, int beta_dx, int beta_dg, uint64_t ws,
                          cudaStream_t st, int max_partials = kRmsMaxPartials, uint64_t r = 0, uint64_t sum = 0) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int NVMAX = 4;
  T* Y = reinterpret_cast<T*>(y); T* dX = reinterpret_cast<T*>(dx);
  const T* X = reinterpret_cast<const T*>(x); const T* Gm = reinterpret_cast<const T*>(gamma);
  const T* dY = reinterpret_cast<const T*>(dy);
  TO* dG = reinterpret_cast<TO*>(dgamma);
  float* wsf = reinterpret_cast<float*>(ws);
  const T* Rp = reinterpret_cast<const T*>(r); T* Sp = reinterpret_cast<T*>(sum);
  const bool vec_ok = (cols % VEC == 0) && aligned16(x) && aligned16(gamma) && (!FWD || aligned16(y)) &&
                      (!BWD || (aligned16(dx) && aligned16(dy))) && (!ADD || (aligned16(r) && aligned16(sum))) && cols / VEC <= 512LL * NVMAX &&
                      (size_t)cols * sizeof(float) <= 64 * 1024;
  if (vec_ok) {
    GroupPlan pl = plan_group(cols / VEC, NVMAX, g_rmsnorm_gpref, g_rmsnorm_threads);
    if (pl.ok) {
      const int threads = pl.G * pl.groups;
      const int64_t want = (rows + pl.groups - 1) / pl.groups;
      const size_t stage = (size_t)cols * sizeof(T) * (((BWD || ADD) ? 2 : 1) + ((BWD && beta_dx) ? 1 : 0));
      // measured at [16384, 3200] f16: the forward kernels (four row groups per SM) gain from bulk stores (add + norm
      // 81 -> 75 us); the backward kernels hold two row groups per SM (registers), where the extra barrier per row
      // costs more than the stores (fused forward + backward 90 -> 99-108 us), so they keep per-thread stores
      const int want_bulk = g_rmsnorm_bulk_out && !BWD ? 1 : 0;
      const size_t out_rows = (ADD || (FWD && BWD)) ? 2 : 1;
      auto smem_for = [&](int ns) {
        return pl.groups * ns * (stage + sizeof(uint64_t)) +
               ((size_t)2 * pl.groups * kMaxWarpsPerGroup * 2 + (BWD ? (size_t)cols : 0)) * sizeof(float) +
               (want_bulk ? 16 + (size_t)pl.groups * 2 * out_rows * cols * sizeof(T) : 0);
      };
      // ring depth: fill about g_rmsnorm_smem_kb of shared memory per CTA, at most 8 rows per group
      // (the accumulating adjoint stages three rows per slot and runs one CTA per SM anyway: it may take more)
      const size_t ring_budget = (size_t)g_rmsnorm_smem_kb * 1024 * ((BWD && beta_dx) ? 3 : 2) / 2;
      int nstages = 8;
      while (nstages > 1 && smem_for(nstages) > ring_budget) --nstages;
      const size_t smem = smem_for(nstages);
      const int bulk_out = want_bulk;
      int64_t grid = 0;
#define CB_LAUNCH(NV_)                                                                                      \
  do {                                                                                                      \
    auto kern = (BWD && beta_dx) ? rmsnorm_rows_kernel<T, NV_, FWD, BWD, ADD, BWD>                          \
                                 : rmsnorm_rows_kernel<T, NV_, FWD, BWD, ADD, false>;                       \
    grid = (int64_t)kNumSMs * resident_ctas(kern, threads, smem);                                           \
    if (grid > max_partials) grid = max_partials;                                                           \
    if (grid > want) grid = want;                                                                           \
    kern<<<(unsigned)grid, threads, smem, st>>>(Y, dX, wsf, X, Gm, dY, eps, rows, (int)cols, pl.G, nstages, beta_dx, \
                                                Rp, Sp, bulk_out);                                          \
  } while (0)
      if (smem <= kMaxDynSmem) {
        switch (pl.NV) {
          case 1: CB_LAUNCH(1); break;
          case 2: CB_LAUNCH(2); break;
          default: CB_LAUNCH(4); break;
        }
#undef CB_LAUNCH
        int rc = check_launch();
        if (rc || !BWD) return rc;
        launch_dependent(rmsnorm_dgamma_finalize_kernel<TO>, (unsigned)((cols + 31) / 32), 512u, st, dG,
                         (const float*)wsf, (int)grid, (int)cols, beta_dg);
        return check_launch();
      }
    }
  }
  if (ADD) return -1;
  int64_t grid = rows < (int64_t)kNumSMs * 8 ? rows : (int64_t)kNumSMs * 8;
  rmsnorm_rows_generic_kernel<T, FWD, BWD><<<(unsigned)grid, 256, 0, st>>>(Y, dX, wsf, X, Gm, dY, eps, rows, cols,
                                                                           beta_dx);
  int rc = check_launch();
  if (rc || !BWD) return rc;
  rmsnorm_dgamma_generic_kernel<T, TO><<<(unsigned)((cols + 255) / 256), 256, 0, st>>>(dG, wsf, X, dY, rows, cols,
                                                                                       beta_dg);
  return check_launch();
}

static int rmsnorm_entry(bool fwd, bool bwd, uint64_t y, uint64_t dx, uint64_t dgamma, uint64_t x, uint64_t gamma,
                         uint64_t dy, float eps, int64_t rows, int64_t cols, int dtype, int dg_dtype, int beta_dx,
                         int beta_dg, uint64_t ws, size_t ws_bytes, void* stream, int max_partials = kRmsMaxPartials) {
  if (rows < 0 || cols < 0 || cols > 0x7fffffffLL) return CACTI_B200_ERR_INVALID_VALUE;
  if ((beta_dx | beta_dg) & ~1) return CACTI_B200_ERR_INVALID_VALUE;
  if (rows == 0 || cols == 0) return CACTI_B200_OK;   // reference: an empty cell is a no-op
  if (!x || !gamma || (fwd && !y) || (bwd && (!dx || !dy || !dgamma))) return CACTI_B200_ERR_INVALID_VALUE;
  if (bwd) {
    if (dg_dtype != dtype && dg_dtype != CACTI_B200_R_32F) return CACTI_B200_ERR_DTYPE;
    if (!ws || ws_bytes < rmsnorm_ws_bytes(rows, cols, max_partials) || (ws & 3)) return CACTI_B200_ERR_WORKSPACE;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
#define CB_GO(TO_)                                                                                                 \
  (fwd && bwd) ? launch_rmsnorm<T, TO_, true, true>(y, dx, dgamma, x, gamma, dy, eps, rows, cols, beta_dx, beta_dg, ws, st, max_partials) \
  : fwd        ? launch_rmsnorm<T, TO_, true, false>(y, dx, dgamma, x, gamma, dy, eps, rows, cols, beta_dx, beta_dg, ws, st, max_partials) \
               : launch_rmsnorm<T, TO_, false, true>(y, dx, dgamma, x, gamma, dy, eps, rows, cols, beta_dx, beta_dg, ws, st, max_partials)
    if (bwd && dg_dtype == CACTI_B200_R_32F) return CB_GO(float);
    return CB_GO(T);
#undef CB_GO
  });
}

// ---- entry point that needs no caller workspace --------------------------------------------------
// The column partials of the dgamma reduction live in this file-scope device array instead of a
// caller-provided buffer.  Every device that loads the library holds the array (about 4.6 MiB) until
// the process exits.
constexpr int kNoAllocMaxCols = 4096;                        // widest row this entry point accepts
constexpr int kNoAllocMaxPartials = 2 * kNumSMs;             // per-CTA partial rows kept in the array
constexpr size_t kNoAllocRowLimit = (size_t)kNoAllocMaxPartials * kNoAllocMaxCols;
constexpr size_t kNoAllocFloats = kNoAllocRowLimit + 64;    // + the slack the workspace check asks for
static __device__ __align__(256) float g_rmsnorm_scratch[kNoAllocFloats];

// `g_rmsnorm_scratch` in host code is only the host-side handle of the symbol, not an address a kernel
// can use.  The device address is looked up once per device (with that device current) and cached.
// The address belongs to the device's context: a caller that resets the device (cudaDeviceReset) or releases and
// retains its primary context must not use this entry point afterwards in the same process.
static int noalloc_scratch(float** out) {
  static std::atomic<float*> cache[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    g_last_cuda_error = (int)cudaGetLastError();
    return CACTI_B200_ERR_LAUNCH;
  }
  float* addr = cache[dev].load(std::memory_order_acquire);
  if (!addr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_rmsnorm_scratch);
    if (e != cudaSuccess || !p) {
      g_last_cuda_error = (int)e;
      (void)cudaGetLastError();
      return CACTI_B200_ERR_LAUNCH;
    }
    addr = static_cast<float*>(p);
    cache[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return CACTI_B200_OK;
}

}  // namespace cb

extern "C" {
size_t cacti_b200_rmsnorm_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows < 0 || cols < 0) return 0;
  return cb::rmsnorm_ws_bytes(rows, cols);
}
int cacti_b200_rmsnorm_fwd(cacti_b200_dptr y, cacti_b200_dptr x, cacti_b200_dptr gamma, float eps, int64_t rows,
                           int64_t cols, int dtype, cacti_b200_stream stream) {
  return cb::rmsnorm_entry(true, false, y, 0, 0, x, gamma, 0, eps, rows, cols, dtype, dtype, 0, 0, 0, 0, stream);
}
int cacti_b200_add_rmsnorm_fwd(cacti_b200_dptr y, cacti_b200_dptr sum, cacti_b200_dptr a, cacti_b200_dptr b,
                               cacti_b200_dptr gamma, float eps, int64_t rows, int64_t cols, int dtype,
                               cacti_b200_stream stream) {
  using namespace cb;
  if (rows < 0 || cols < 0 || cols > 0x7fffffffLL) return CACTI_B200_ERR_INVALID_VALUE;
  if (rows == 0 || cols == 0) return CACTI_B200_OK;
  if (!y || !sum || !a || !b || !gamma) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int rc = dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    return launch_rmsnorm<T, T, true, false, true>(y, 0, 0, a, gamma, 0, eps, rows, cols, 0, 0, 0, st, kRmsMaxPartials, b, sum);
  });
  if (rc != -1) return rc;
  // shapes the row kernel does not take: the two steps as separate launches, same results
  const int rc2 = cacti_b200_add(sum, a, b, rows * cols, dtype, stream);
  if (rc2) return rc2;
  return rmsnorm_entry(true, false, y, 0, 0, sum, gamma, 0, eps, rows, cols, dtype, dtype, 0, 0, 0, 0, stream);
}
int cacti_b200_rmsnorm_bwd(cacti_b200_dptr dx, cacti_b200_dptr dgamma, cacti_b200_dptr dy, cacti_b200_dptr x,
                           cacti_b200_dptr gamma, float eps, int64_t rows, int64_t cols, int dtype, int dgamma_dtype,
                           int beta_dx, int beta_dgamma, cacti_b200_dptr workspace, size_t workspace_bytes,
                           cacti_b200_stream stream) {
  return cb::rmsnorm_entry(false, true, 0, dx, dgamma, x, gamma, dy, eps, rows, cols, dtype, dgamma_dtype, beta_dx,
                           beta_dgamma, workspace, workspace_bytes, stream);
}
int cacti_b200_rmsnorm_fwd_bwd(cacti_b200_dptr y, cacti_b200_dptr dx, cacti_b200_dptr dgamma, cacti_b200_dptr x,
                               cacti_b200_dptr gamma, cacti_b200_dptr dy, float eps, int64_t rows, int64_t cols,
                               int dtype, int dgamma_dtype, int beta_dx, int beta_dgamma, cacti_b200_dptr workspace,
                               size_t workspace_bytes, cacti_b200_stream stream) {
  return cb::rmsnorm_entry(true, true, y, dx, dgamma, x, gamma, dy, eps, rows, cols, dtype, dgamma_dtype, beta_dx,
                           beta_dgamma, workspace, workspace_bytes, stream);
}

int cacti_b200_rmsnorm_fwd_bwd_noalloc(cacti_b200_dptr y, cacti_b200_dptr dx, cacti_b200_dptr dgamma, cacti_b200_dptr x,
                                       cacti_b200_dptr gamma, cacti_b200_dptr dy, float eps, int64_t rows, int64_t cols,
                                       int dtype, int dgamma_dtype, int beta_dx, int beta_dgamma,
                                       cacti_b200_stream stream) {
  using namespace cb;
  if (rows < 0 || cols < 0) return CACTI_B200_ERR_INVALID_VALUE;
  // limits of the built-in array: the vector path stores 2*148 partial rows of `cols` floats, the
  // element-wise path one float per row
  if (cols > kNoAllocMaxCols || (size_t)rows > kNoAllocRowLimit) return CACTI_B200_ERR_SCRATCH_LIMIT;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  return rmsnorm_entry(true, true, y, dx, dgamma, x, gamma, dy, eps, rows, cols, dtype, dgamma_dtype, beta_dx,
                       beta_dgamma, reinterpret_cast<uint64_t>(scratch), kNoAllocFloats * sizeof(float), stream,
                       kNoAllocMaxPartials);
}
}
