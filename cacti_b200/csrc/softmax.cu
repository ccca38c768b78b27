// K2: masked row softmax, forward / backward / fused forward+backward.
//
// Replaces, per row of a [.., cols] tensor, the reference chain
//   cast(f32) -> block_tri_elem_affine (causal mask) -> inner_softmax -> lossy_cast
// (src/librarium/llama.rs:502-505, src/thunk/op.rs:4189-4278, :3257-3383) and the adjoint
//   inner_softmax_post_adj over a recomputed softmax + mask adjoint + lossy cast
// (src/thunk/op.rs:3376-3382, :3386-3457, :4265-4276).
//
// Fast path: one row per group of G threads, the row's 16-byte vectors held raw in registers
// (S and dP), three register passes (max, sum of exp, outputs).  Every input byte is read from
// HBM once, every output byte written once; masked inputs are never read.  All loads of a row
// are issued before the first use so a warp keeps NV*2 128-bit loads per lane in flight.
#include "common.cuh"
#include <type_traits>

namespace cb {

int g_softmax_threads = 256;   // threads per CTA on the warp-per-row path (tunable)
int g_softmax_waves = 1;       // grid = SMs * resident CTAs * this (capped by the row count)

__device__ __forceinline__ int active_cols(int64_t row, int cols, int mask_mode,
                                           int64_t q_div, int64_t q_mod, int64_t q_off) {
  if (mask_mode == CACTI_B200_MASK_NONE) return cols;
  int64_t q = (row / q_div) % q_mod + q_off;
  if (q < 0) return 0;
  return (q + 1 < (int64_t)cols) ? (int)(q + 1) : cols;
}

// Columns of a row that get written.  CACTI_B200_MASK_CAUSAL_TRIM zero-fills the masked tail only as far as a
// consumer with a CACTI_B200_TRI_A_* hint can read (tiles of at most 256 rows, k-blocks of 64): up to the next
// multiple of 256 past q_pos when q_off is a multiple of 256, else 320 columns past it.
__device__ __forceinline__ int written_cols(int active, int cols, int mask_mode, int64_t q_off) {
  if (mask_mode != CACTI_B200_MASK_CAUSAL_TRIM || active <= 0) return cols;
  const int64_t q = (int64_t)active - 1;
  const int64_t b = (q_off & 255) == 0 ? (q & ~(int64_t)255) + 256 : ((q + 320 + 7) & ~(int64_t)7);
  return b < (int64_t)cols ? (int)b : cols;
}

// -inf / 0 fill of the masked tail of the one vector that straddles the causal boundary, so that the
// three passes below need no per-element predicate.
template <typename T>
__device__ __forceinline__ void mask_tail(uint4& s, uint4& g, int nact, bool bwd) {
  constexpr int VEC = Elem<T>::VEC;
  float a[VEC];
  unpack<T>(s, a);
#pragma unroll
  for (int e = 0; e < VEC; ++e) if (e >= nact) a[e] = -INFINITY;
  s = pack<T>(a);
  if (bwd) {
    unpack<T>(g, a);
#pragma unroll
    for (int e = 0; e < VEC; ++e) if (e >= nact) a[e] = 0.f;
    g = pack<T>(a);
  }
}

template <typename T, int NV, bool FWD, bool BWD>
__global__ void __launch_bounds__(512)
softmax_rows_kernel(T* __restrict__ P, T* __restrict__ dS, const T* __restrict__ S, const T* __restrict__ dP,
                    int64_t rows, int cols, int G, int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off,
                    int beta) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int VEC = Elem<T>::VEC;
  const int groups = blockDim.x / G;
  const unsigned row_bytes = (unsigned)cols * sizeof(T);
  const unsigned stage_bytes = row_bytes * (BWD ? 2 : 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)groups * stage_bytes);
  float* red = reinterpret_cast<float*>(bars + groups);
  GroupCtx g = make_group(G, red);
  unsigned char* stage = smem_raw + (size_t)g.gid * stage_bytes;
  uint64_t* bar = bars + g.gid;
  if (g.lane == 0) mbar_init(bar, 1);
  mbar_fence_init();
  __syncthreads();

  const int64_t stride = (int64_t)gridDim.x * groups;
  int64_t row = (int64_t)blockIdx.x * groups + g.gid;
  unsigned phase = 0;
  // lane 0 of the group starts the bulk copies of a row's unmasked prefix; returns its length in columns
  auto issue = [&](int64_t r) -> int {
    const int act = active_cols(r, cols, mask_mode, q_div, q_mod, q_off);
    if (act > 0 && g.lane == 0) {
      const unsigned bytes = ((unsigned)act * sizeof(T) + 15u) & ~15u;
      mbar_expect_tx(bar, bytes * (BWD ? 2u : 1u));
      bulk_g2s(stage, S + r * cols, bytes, bar);
      if (BWD) bulk_g2s(stage + row_bytes, dP + r * cols, bytes, bar);
    }
    return act;
  };
  int active = row < rows ? issue(row) : 0;
  for (; row < rows; row += stride) {
    uint4 sraw[NV], graw[NV];
    bool gave_up = false;
    if (active > 0) {
      gave_up = !mbar_wait_bounded(bar, phase, kDevErrStageTimeout);
      phase ^= 1;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int col0 = (g.lane + k * G) * VEC;
        if (col0 < active) {
          sraw[k] = *reinterpret_cast<const uint4*>(stage + (size_t)col0 * sizeof(T));
          if (BWD) graw[k] = *reinterpret_cast<const uint4*>(stage + row_bytes + (size_t)col0 * sizeof(T));
          if (active - col0 < VEC) mask_tail<T>(sraw[k], graw[k], active - col0, BWD);
        }
      }
    }
    // the stage buffer has been consumed by every lane; a wait that ran out on any lane ends the group's work
    // here, all lanes together
    if (group_any(g, gave_up)) return;
    const int cur_active = active;
    active = (row + stride < rows) ? issue(row + stride) : 0;

    // pass 1: row maximum
    float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains
    // (measured at [65536, 2048] f16, causal: the packed maximum below takes the forward kernel from 101 to 96 us and
    // the backward kernel from 121 to 115 us, but the fused kernel from 136 to 145 us, so that one keeps the f32 form)
    if constexpr (std::is_same<T, float>::value || (FWD && BWD)) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int col0 = (g.lane + k * G) * VEC;
        if (col0 < cur_active) {
          float a[VEC];
          unpack<T>(sraw[k], a);
#pragma unroll
          for (int e = 0; e < VEC; ++e) mq[e & 3] = fmaxf(mq[e & 3], a[e]);
        }
      }
    } else {
      // 16-bit storage: the maximum is exact in the storage type, so it is taken on the packed pairs (one
      // instruction per two elements, no conversion) and widened once
      using H2 = typename Pair16<T>::type;
      H2 hq[2] = {Pair16<T>::neg_inf(), Pair16<T>::neg_inf()};
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int col0 = (g.lane + k * G) * VEC;
        if (col0 < cur_active) {
          const H2* h = reinterpret_cast<const H2*>(&sraw[k]);
          hq[0] = __hmax2(hq[0], h[0]); hq[1] = __hmax2(hq[1], h[1]);
          hq[0] = __hmax2(hq[0], h[2]); hq[1] = __hmax2(hq[1], h[3]);
        }
      }
      const H2 hm = __hmax2(hq[0], hq[1]);
      mq[0] = Elem<T>::to_f32(hm.x); mq[1] = Elem<T>::to_f32(hm.y);
    }
    float m = group_reduce<MaxOp>(g, fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])));
    const float nml2e = __fmul_rn(-m, 1.4426950408889634f);
    // pass 2: Z = sum exp(a - m); cg = sum exp(a - m) * g  (sum_j y_j g_j = cg / Z)
    float zq[4] = {0.f, 0.f, 0.f, 0.f}, cq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cur_active) {
        float a[VEC], gv[VEC];
        unpack<T>(sraw[k], a);
        if (BWD) unpack<T>(graw[k], gv);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float ex = exp_shifted<T>(a[e], m, nml2e);
          zq[e & 3] = __fadd_rn(zq[e & 3], ex);
          if (BWD) cq[e & 3] = __fmaf_rn(ex, gv[e], cq[e & 3]);
        }
      }
    }
    float z = __fadd_rn(__fadd_rn(zq[0], zq[1]), __fadd_rn(zq[2], zq[3]));
    float cg = __fadd_rn(__fadd_rn(cq[0], cq[1]), __fadd_rn(cq[2], cq[3]));
    group_reduce2<SumOp>(g, z, cg);
    // An all-masked row has max = -inf and exp(-inf - -inf) = NaN in the reference chain.
    const bool dead = (cur_active <= 0);
    const float rz = __frcp_rn(z);
    const float c = __fmul_rn(cg, rz);
    T* prow = FWD ? P + row * cols : nullptr;
    T* drow = BWD ? dS + row * cols : nullptr;
    // pass 3: outputs (explicitly rounded ops: every entry point produces the same bits)
    const int wcols = written_cols(cur_active, cols, mask_mode, q_off);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < wcols) {
        float y[VEC], d[VEC];
        if (col0 < cur_active) {
          float a[VEC], gv[VEC];
          unpack<T>(sraw[k], a);
          if (BWD) unpack<T>(graw[k], gv);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float ex = exp_shifted<T>(a[e], m, nml2e);
            y[e] = std::is_same<T, float>::value ? __fdiv_rn(ex, z) : __fmul_rn(ex, rz);
            if (BWD) d[e] = __fmaf_rn(y[e], gv[e], -__fmul_rn(c, y[e]));
          }
        } else {
          const float fill = dead ? __int_as_float(0x7fc00000) : 0.f;
#pragma unroll
          for (int e = 0; e < VEC; ++e) { y[e] = fill; d[e] = fill; }
        }
        if (FWD) st_stream(prow + col0, pack<T>(y));
        if (BWD) {
          if (beta) st_stream(drow + col0, pack_accumulate<T>(d, ld_stream(drow + col0)));
          else st_stream(drow + col0, pack<T>(d));
        }
      }
    }
  }
}

// Element-wise fallback: any cols, any element-aligned pointers.  One CTA per row, rows re-read
// from global memory (L1/L2) in each pass.
template <typename T, bool FWD, bool BWD>
__global__ void __launch_bounds__(256)
softmax_rows_generic_kernel(T* __restrict__ P, T* __restrict__ dS, const T* __restrict__ S, const T* __restrict__ dP,
                            int64_t rows, int64_t cols, int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off,
                            int beta) {
  __shared__ float sm[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    int64_t active = cols;
    if (mask_mode != CACTI_B200_MASK_NONE) {
      int64_t q = (row / q_div) % q_mod + q_off;
      active = q < 0 ? 0 : (q + 1 < cols ? q + 1 : cols);
    }
    const int64_t wcols = written_cols((int)active, (int)cols, mask_mode, q_off);
    const T* srow = S + row * cols;
    float m = -INFINITY;
    for (int64_t j = threadIdx.x; j < active; j += blockDim.x) m = fmaxf(m, Elem<T>::to_f32(srow[j]));
    m = block_reduce<MaxOp>(m, sm);
    const float nml2e = __fmul_rn(-m, 1.4426950408889634f);
    float z = 0.f, cg = 0.f;
    for (int64_t j = threadIdx.x; j < active; j += blockDim.x) {
      const float ex = exp_shifted<T>(Elem<T>::to_f32(srow[j]), m, nml2e);
      z += ex;
      if (BWD) cg = fmaf(ex, Elem<T>::to_f32(dP[row * cols + j]), cg);
    }
    z = block_reduce<SumOp>(z, sm);
    if (BWD) cg = block_reduce<SumOp>(cg, sm);
    const float rz = 1.f / z, c = cg * rz;
    const float fill = active <= 0 ? __int_as_float(0x7fc00000) : 0.f;
    for (int64_t j = threadIdx.x; j < wcols; j += blockDim.x) {
      float y = fill, d = fill;
      if (j < active) {
        const float ex = exp_shifted<T>(Elem<T>::to_f32(srow[j]), m, nml2e);
        y = std::is_same<T, float>::value ? ex / z : ex * rz;
        if (BWD) d = y * Elem<T>::to_f32(dP[row * cols + j]) - c * y;
      }
      if (FWD) P[row * cols + j] = Elem<T>::from_f32(y);
      if (BWD) {
        T* o = dS + row * cols + j;
        *o = beta ? Elem<T>::from_f32(Elem<T>::to_f32(*o) + round_to<T>(d)) : Elem<T>::from_f32(d);
      }
    }
  }
}

template <typename T, bool FWD, bool BWD>
static int launch_softmax(uint64_t p, uint64_t ds, uint64_t s, uint64_t dp, int64_t rows, int64_t cols,
                          int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off, int beta, cudaStream_t st) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int NVMAX = 8;
  T* P = reinterpret_cast<T*>(p); T* dS = reinterpret_cast<T*>(ds);
  const T* S = reinterpret_cast<const T*>(s); const T* dP = reinterpret_cast<const T*>(dp);
  const bool vec_ok = (cols % VEC == 0) && aligned16(s) && (!FWD || aligned16(p)) &&
                      (!BWD || (aligned16(ds) && aligned16(dp))) && cols / VEC <= 512LL * NVMAX;
  if (vec_ok) {
    GroupPlan pl = plan_group(cols / VEC, NVMAX, 128, g_softmax_threads);
    if (pl.ok) {
      const int threads = pl.G * pl.groups;
      const size_t stage = (size_t)cols * sizeof(T) * (BWD ? 2 : 1);
      const size_t smem = pl.groups * stage + pl.groups * sizeof(uint64_t) +
                          (size_t)2 * pl.groups * kMaxWarpsPerGroup * 2 * sizeof(float);
      const int64_t want = (rows + pl.groups - 1) / pl.groups;
#define CB_LAUNCH(NV_)                                                                               \
  do {                                                                                               \
    auto kern = softmax_rows_kernel<T, NV_, FWD, BWD>;                                               \
    int64_t grid = (int64_t)kNumSMs * resident_ctas(kern, threads, smem) * g_softmax_waves;          \
    if (grid > want) grid = want;                                                                    \
    kern<<<(unsigned)grid, threads, smem, st>>>(P, dS, S, dP, rows, (int)cols, pl.G, mask_mode,      \
                                                q_div, q_mod, q_off, beta);                          \
  } while (0)
      if (smem <= kMaxDynSmem) {
        switch (pl.NV) {
          case 1: CB_LAUNCH(1); break;
          case 2: CB_LAUNCH(2); break;
          case 4: CB_LAUNCH(4); break;
          default: CB_LAUNCH(8); break;
        }
#undef CB_LAUNCH
        return check_launch();
      }
    }
  }
  int64_t grid = rows < (int64_t)kNumSMs * 8 ? rows : (int64_t)kNumSMs * 8;
  softmax_rows_generic_kernel<T, FWD, BWD><<<(unsigned)grid, 256, 0, st>>>(P, dS, S, dP, rows, cols, mask_mode,
                                                                           q_div, q_mod, q_off, beta);
  return check_launch();
}

static int softmax_entry(bool fwd, bool bwd, uint64_t p, uint64_t ds, uint64_t s, uint64_t dp, int64_t rows,
                         int64_t cols, int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off, int dtype,
                         int beta, void* stream) {
  if (rows < 0 || cols < 0 || cols > 0x7fffffffLL) return CACTI_B200_ERR_INVALID_VALUE;
  if (mask_mode < CACTI_B200_MASK_NONE || mask_mode > CACTI_B200_MASK_CAUSAL_TRIM) return CACTI_B200_ERR_INVALID_VALUE;
  if (mask_mode != CACTI_B200_MASK_NONE && (q_div <= 0 || q_mod <= 0)) return CACTI_B200_ERR_INVALID_VALUE;
  if (beta != 0 && beta != 1) return CACTI_B200_ERR_INVALID_VALUE;
  if (rows == 0 || cols == 0) return CACTI_B200_OK;
  if (!s || (fwd && !p) || (bwd && (!ds || !dp))) return CACTI_B200_ERR_INVALID_VALUE;
  if (mask_mode == CACTI_B200_MASK_NONE) { q_div = 1; q_mod = 1; q_off = 0; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    if (fwd && bwd) return launch_softmax<T, true, true>(p, ds, s, dp, rows, cols, mask_mode, q_div, q_mod, q_off, beta, st);
    if (fwd) return launch_softmax<T, true, false>(p, ds, s, dp, rows, cols, mask_mode, q_div, q_mod, q_off, beta, st);
    return launch_softmax<T, false, true>(p, ds, s, dp, rows, cols, mask_mode, q_div, q_mod, q_off, beta, st);
  });
}

}  // namespace cb

extern "C" {
int cacti_b200_softmax_fwd(cacti_b200_dptr p, cacti_b200_dptr s, int64_t rows, int64_t cols, int mask_mode,
                           int64_t q_div, int64_t q_mod, int64_t q_off, int dtype, cacti_b200_stream stream) {
  return cb::softmax_entry(true, false, p, 0, s, 0, rows, cols, mask_mode, q_div, q_mod, q_off, dtype, 0, stream);
}
int cacti_b200_softmax_bwd(cacti_b200_dptr ds, cacti_b200_dptr s, cacti_b200_dptr dp, int64_t rows, int64_t cols,
                           int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off, int dtype, int beta_ds,
                           cacti_b200_stream stream) {
  return cb::softmax_entry(false, true, 0, ds, s, dp, rows, cols, mask_mode, q_div, q_mod, q_off, dtype, beta_ds, stream);
}
int cacti_b200_softmax_fwd_bwd(cacti_b200_dptr p, cacti_b200_dptr ds, cacti_b200_dptr s, cacti_b200_dptr dp,
                               int64_t rows, int64_t cols, int mask_mode, int64_t q_div, int64_t q_mod,
                               int64_t q_off, int dtype, int beta_ds, cacti_b200_stream stream) {
  return cb::softmax_entry(true, true, p, ds, s, dp, rows, cols, mask_mode, q_div, q_mod, q_off, dtype, beta_ds, stream);
}
}
