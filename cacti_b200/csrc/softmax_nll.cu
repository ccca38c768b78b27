// K5: softmax cross-entropy, loss and dlogits in one pass over the logits.
//
// Replaces cast(f32) -> inner_softmax_categorical_nll (src/thunk/op.rs:3460-3569, call site
// src/librarium/llama.rs:542-545) and its adjoint, which in the reference recomputes the softmax,
// materialises a dense f32 one-hot [rows, vocab] (src/thunk/op.rs:883-997), subtracts and scales.
// Here a row of logits is fetched from HBM once (one bulk copy into shared memory), reduced twice
// (max, sum of exp) and the gradient is written once; the one-hot is a comparison on the column index.
// Two kernels: rows of up to 4096 elements are held in the registers of one warp
// (softmax_nll_rows_kernel); longer rows stay in shared memory and are swept three times by a
// 256-thread CTA, three CTAs per SM (softmax_nll_smem_kernel).  Measured at [8192, 32000] f16: 200 us
// against 222-260 us for the register-resident form with one 512-thread CTA per SM, whose phases
// (load, max, exp, store) could not overlap.
#include "common.cuh"
#include <type_traits>

namespace cb {

int g_nll_gpref = 512;
int g_nll_stages = 3;
int g_nll_smem_threads = 256;
int g_nll_mode = 1;      // 1: rows longer than a warp-group use the shared-memory-resident kernel, 0: registers

template <typename TI> __device__ __forceinline__ int64_t load_index(const void* p, int64_t i);
template <> __device__ __forceinline__ int64_t load_index<int32_t>(const void* p, int64_t i) {
  return (int64_t) reinterpret_cast<const int32_t*>(p)[i];
}
template <> __device__ __forceinline__ int64_t load_index<uint16_t>(const void* p, int64_t i) {
  return (int64_t) reinterpret_cast<const uint16_t*>(p)[i];
}

// exp(d) for the (max, sum) combine: d <= 0 or -inf.
template <typename T> __device__ __forceinline__ float exp_rescale(float d) {
  if constexpr (std::is_same<T, float>::value) return expf(d);
  else return exp2f_approx(d * 1.4426950408889634f);
}

template <typename T, typename TI, int NV, bool BWD>
__global__ void __launch_bounds__(512)
softmax_nll_rows_kernel(float* __restrict__ loss_rows, T* __restrict__ dL, const T* __restrict__ L,
                        const void* __restrict__ targets, const float* __restrict__ w_rows, float w_scalar,
                        int64_t rows, int cols, int G, int nstages, int beta, unsigned* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int VEC = Elem<T>::VEC;
  const int groups = blockDim.x / G;
  const unsigned row_bytes = (unsigned)cols * sizeof(T);
  // shared: [groups][nstages] row buffers | [groups][nstages] mbarriers | reduction slots
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)groups * nstages * row_bytes);
  float* red = reinterpret_cast<float*>(bars + groups * nstages);
  GroupCtx g = make_group(G, red);
  unsigned char* stage0 = smem_raw + (size_t)g.gid * nstages * row_bytes;
  uint64_t* bar0 = bars + g.gid * nstages;
  if (g.lane < nstages) mbar_init(bar0 + g.lane, 1);
  mbar_fence_init();
  __syncthreads();
  const int64_t stride = (int64_t)gridDim.x * groups;
  const int64_t row0 = (int64_t)blockIdx.x * groups + g.gid;
  auto issue = [&](int64_t r, int slot) {
    if (g.lane == 0) {
      mbar_expect_tx(bar0 + slot, row_bytes);
      bulk_g2s(stage0 + (size_t)slot * row_bytes, L + r * cols, row_bytes, bar0 + slot);
    }
  };
  for (int s = 0; s < nstages; ++s)
    if (row0 + s * stride < rows) issue(row0 + s * stride, s);
  int slot = 0;
  unsigned phase = 0;
  // The target index and row weight are fetched one row ahead: under a saturated memory system a
  // dependent global load costs about a microsecond, which would otherwise stall every row.
  int64_t tgt_next = row0 < rows ? load_index<TI>(targets, row0) : 0;
  float w_next = (row0 < rows && w_rows) ? w_rows[row0] : w_scalar;
  for (int64_t row = row0; row < rows; row += stride) {
    const int64_t tgt = tgt_next;
    const float w = w_next;
    if (row + stride < rows) {
      tgt_next = load_index<TI>(targets, row + stride);
      if (w_rows) w_next = w_rows[row + stride];
    }
    const bool tgt_ok = tgt >= 0 && tgt < cols;
    // a wait that ran out: a one-warp group agrees at once, a larger one at the group barrier below
    bool gave_up = !mbar_wait_bounded(bar0 + slot, phase, kDevErrStageTimeout);
    if (G == 32 && __any_sync(0xffffffffu, gave_up)) return;
    const unsigned char* stage = stage0 + (size_t)slot * row_bytes;
    // the row as f32 in registers; it is overwritten by exp(a - m) in pass 2 and scaled in pass 3
    float a[NV][VEC];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) unpack<T>(*reinterpret_cast<const uint4*>(stage + (size_t)col0 * sizeof(T)), a[k]);
    }
    // the target logit, read from the staged row (the stored bit pattern, converted exactly)
    const float a_t = tgt_ok ? Elem<T>::to_f32(reinterpret_cast<const T*>(stage)[tgt]) : 0.f;
    const int cur_slot = slot;
    if (++slot == nstages) { slot = 0; phase ^= 1; }

    // Warp-local online softmax: each warp reduces its own part of the row against its own maximum
    // and the warps then combine (max, sum) pairs once.  One group barrier per row, and between two
    // barriers the warps run independently, so one warp's exp phase overlaps another's loads.
    // (four independent accumulators per reduction: the dependent chain is a quarter as long)
    float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if ((g.lane + k * G) * VEC < cols) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) mq[e & 3] = fmaxf(mq[e & 3], a[k][e]);
      }
    }
    float mw = warp_reduce<MaxOp>(fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])));
    // a warp whose part of the row is empty has mw = -inf; use 0 so that no inf - inf appears
    const float mw_f = mw == -INFINITY ? 0.f : mw;
    const float nml = -mw_f * 1.4426950408889634f;
    float zq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if ((g.lane + k * G) * VEC < cols) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) { a[k][e] = exp_shifted<T>(a[k][e], mw_f, nml); zq[e & 3] += a[k][e]; }
      }
    }
    float zw = warp_reduce<SumOp>((zq[0] + zq[1]) + (zq[2] + zq[3]));
    float m = mw, z = zw, rescale = 1.f;
    if (G > 32) {
      const int groups_ = blockDim.x / G;
      float2* sl = reinterpret_cast<float2*>(g.red) + (size_t)(g.phase * groups_ + g.gid) * kMaxWarpsPerGroup;
      const int wi = g.lane >> 5, l = g.lane & 31;
      if (l == 0) sl[wi] = make_float2(mw, zw);
      if (group_any(g, gave_up)) return;                 // also: every lane has consumed the stage slot
      const float2 v = l < g.nwarps ? sl[l] : make_float2(-INFINITY, 0.f);
      m = warp_reduce<MaxOp>(v.x);
      const float term = v.y * exp_rescale<T>(v.x == -INFINITY ? -INFINITY : v.x - m);
      z = warp_reduce<SumOp>(term);
      rescale = exp_rescale<T>(mw == -INFINITY ? -INFINITY : mw - m);
      g.phase ^= 1;
    } else {
      __syncwarp();
    }
    if (row + (int64_t)nstages * stride < rows) issue(row + (int64_t)nstages * stride, cur_slot);
    if (g.lane == 0) {
      if (!tgt_ok && status) atomicMax(status, (unsigned)CACTI_B200_ERR_INDEX_RANGE);
      // -log(y_k) with y_k = exp(a_k - m) / z, formed as in the reference (src/thunk/op.rs:3543)
      if (loss_rows) loss_rows[row] = tgt_ok ? -logf(expf(a_t - m) / z) : __int_as_float(0x7fc00000);
    }
    if (BWD) {
      // w*(y - onehot) = e*(w/z) - w*onehot: one multiply per element, the target column fixed up
      const float rz = rescale / z;                      // e was formed against the warp's own maximum
      const float sc = w * rz;
      T* drow = dL + row * cols;
      const int tcol = tgt_ok ? (int)tgt : -1;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int col0 = (g.lane + k * G) * VEC;
        if (col0 < cols) {
          float d[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            d[e] = a[k][e] * sc;
          }
          if (tcol >= col0 && tcol < col0 + VEC) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) if (col0 + e == tcol) d[e] = w * (a[k][e] * rz - 1.f);
          }
          if (beta) st_stream(drow + col0, pack_accumulate<T>(d, ld_stream(drow + col0)));
          else st_stream(drow + col0, pack<T>(d));
        }
      }
    }
  }
}

// Shared-memory-resident variant: a 256-thread CTA keeps one row in shared memory (staged by one bulk copy)
// and sweeps it three times (max; sum of exp; gradient), so a thread needs few registers and three CTAs fit
// on an SM.  While one CTA waits for its next row the others compute: the phases of different rows overlap,
// which the register-resident kernel (one 512-thread CTA per SM, all warps in the same phase) cannot do.
// The price is a second exp per element in the gradient sweep.
template <typename T, typename TI, bool BWD, int THREADS>
__global__ void __launch_bounds__(THREADS, 3)
softmax_nll_smem_kernel(float* __restrict__ loss_rows, T* __restrict__ dL, const T* __restrict__ L,
                        const void* __restrict__ targets, const float* __restrict__ w_rows, float w_scalar,
                        int64_t rows, int cols, int beta, unsigned* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int VEC = Elem<T>::VEC;
  const unsigned row_bytes = (unsigned)cols * sizeof(T);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw + row_bytes);
  float* red = reinterpret_cast<float*>(bar + 1);                  // >= 33 floats
  const int nvec = cols / VEC;
  if (threadIdx.x == 0) mbar_init(bar, 1);
  mbar_fence_init();
  __syncthreads();
  unsigned phase = 0;
  int64_t row = blockIdx.x;
  if (row < rows && threadIdx.x == 0) { mbar_expect_tx(bar, row_bytes); bulk_g2s(smem_raw, L + row * cols, row_bytes, bar); }
  int64_t tgt_next = row < rows ? load_index<TI>(targets, row) : 0;
  float w_next = (row < rows && w_rows) ? w_rows[row] : w_scalar;
  for (; row < rows; row += gridDim.x) {
    const int64_t tgt = tgt_next;
    const float w = w_next;
    const int64_t nrow = row + gridDim.x;
    if (nrow < rows) { tgt_next = load_index<TI>(targets, nrow); if (w_rows) w_next = w_rows[nrow]; }
    const bool tgt_ok = tgt >= 0 && tgt < cols;
    bool gave_up = !mbar_wait_bounded(bar, phase, kDevErrStageTimeout);   // agreed on by the CTA at the first reduction
    phase ^= 1;
    const uint4* srow = reinterpret_cast<const uint4*>(smem_raw);
    // sweep 1: maximum
    float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      float a[VEC];
      unpack<T>(srow[v], a);
#pragma unroll
      for (int e = 0; e < VEC; ++e) mq[e & 3] = fmaxf(mq[e & 3], a[e]);
    }
    const float m = block_reduce<MaxOp>(fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])), red, &gave_up);
    if (gave_up) return;
    const float nml = -m * 1.4426950408889634f;
    // sweep 2: Z
    float zq[4] = {0.f, 0.f, 0.f, 0.f};
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      float a[VEC];
      unpack<T>(srow[v], a);
#pragma unroll
      for (int e = 0; e < VEC; ++e) zq[e & 3] += exp_shifted<T>(a[e], m, nml);
    }
    const float z = block_reduce<SumOp>((zq[0] + zq[1]) + (zq[2] + zq[3]), red);
    if (threadIdx.x == 0) {
      if (!tgt_ok && status) atomicMax(status, (unsigned)CACTI_B200_ERR_INDEX_RANGE);
      if (loss_rows) {
        const float a_t = tgt_ok ? Elem<T>::to_f32(reinterpret_cast<const T*>(smem_raw)[tgt]) : 0.f;
        loss_rows[row] = tgt_ok ? -logf(expf(a_t - m) / z) : __int_as_float(0x7fc00000);
      }
    }
    if (BWD) {
      const float rz = 1.f / z, sc = w * rz;
      T* drow = dL + row * cols;
      const int tcol = tgt_ok ? (int)tgt : -1;
      for (int v = threadIdx.x; v < nvec; v += THREADS) {
        float a[VEC], d[VEC];
        unpack<T>(srow[v], a);
        const int col0 = v * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) d[e] = exp_shifted<T>(a[e], m, nml) * sc;
        if (tcol >= col0 && tcol < col0 + VEC) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) if (col0 + e == tcol) d[e] = w * (exp_shifted<T>(a[e], m, nml) * rz - 1.f);
        }
        if (beta) st_stream(drow + col0, pack_accumulate<T>(d, ld_stream(drow + col0)));
        else st_stream(drow + col0, pack<T>(d));
      }
    }
    __syncthreads();                        // every thread is done with the row buffer
    if (nrow < rows && threadIdx.x == 0) { mbar_expect_tx(bar, row_bytes); bulk_g2s(smem_raw, L + nrow * cols, row_bytes, bar); }
  }
}

template <typename T, typename TI, bool BWD>
__global__ void __launch_bounds__(256)
softmax_nll_rows_generic_kernel(float* __restrict__ loss_rows, T* __restrict__ dL, const T* __restrict__ L,
                                const void* __restrict__ targets, const float* __restrict__ w_rows, float w_scalar,
                                int64_t rows, int64_t cols, int beta, unsigned* __restrict__ status) {
  __shared__ float sm[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lrow = L + row * cols;
    const int64_t tgt = load_index<TI>(targets, row);
    const bool tgt_ok = tgt >= 0 && tgt < cols;
    const float w = w_rows ? w_rows[row] : w_scalar;
    float m = -INFINITY;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, Elem<T>::to_f32(lrow[j]));
    m = block_reduce<MaxOp>(m, sm);
    float z = 0.f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) z += exp_for<T>(Elem<T>::to_f32(lrow[j]) - m);
    z = block_reduce<SumOp>(z, sm);
    if (threadIdx.x == 0) {
      if (!tgt_ok && status) atomicMax(status, (unsigned)CACTI_B200_ERR_INDEX_RANGE);
      if (loss_rows)
        loss_rows[row] = tgt_ok ? -logf(expf(Elem<T>::to_f32(lrow[tgt]) - m) / z) : __int_as_float(0x7fc00000);
    }
    if (BWD) {
      const float rz = 1.f / z;
      for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
        const float ex = exp_for<T>(Elem<T>::to_f32(lrow[j]) - m);
        const float y = std::is_same<T, float>::value ? ex / z : ex * rz;
        const float d = w * (y - ((tgt_ok && j == tgt) ? 1.f : 0.f));
        T* o = dL + row * cols + j;
        *o = beta ? Elem<T>::from_f32(Elem<T>::to_f32(*o) + round_to<T>(d)) : Elem<T>::from_f32(d);
      }
    }
  }
}

// loss_sum = sum_i w_i * loss_i in a fixed order: 1024 strided partial sums, then a tree.
__global__ void __launch_bounds__(1024)
nll_loss_sum_kernel(float* __restrict__ loss_sum, const float* __restrict__ loss_rows,
                    const float* __restrict__ w_rows, float w_scalar, int64_t rows) {
  __shared__ float sm[1024];
  float acc = 0.f;
  dependent_wait();                                           // the per-row losses come from the kernel before this one
  for (int64_t i = threadIdx.x; i < rows; i += 1024) acc += (w_rows ? w_rows[i] : w_scalar) * loss_rows[i];
  sm[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 512; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) sm[threadIdx.x] += sm[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) *loss_sum = sm[0];
}

template <typename T, typename TI, bool BWD>
static int launch_nll(float* loss_rows, uint64_t dl, uint64_t l, const void* targets, const float* w_rows,
                      float w_scalar, int64_t rows, int64_t cols, int beta, unsigned* status, cudaStream_t st) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int NVMAX = 16;
  T* dL = reinterpret_cast<T*>(dl);
  const T* L = reinterpret_cast<const T*>(l);
  const bool vec_ok = (cols % VEC == 0) && aligned16(l) && (!BWD || aligned16(dl)) && cols / VEC <= 512LL * NVMAX;
  if (vec_ok && g_nll_mode == 1 && cols / VEC > 512 && (size_t)cols * sizeof(T) + 512 <= kMaxDynSmem) {
    const size_t smem = (size_t)cols * sizeof(T) + sizeof(uint64_t) + 40 * sizeof(float);
    const int thr = g_nll_smem_threads >= 384 ? 384 : 256;
    auto kern = thr == 384 ? softmax_nll_smem_kernel<T, TI, BWD, 384> : softmax_nll_smem_kernel<T, TI, BWD, 256>;
    int64_t grid = (int64_t)kNumSMs * resident_ctas(kern, thr, smem);
    if (grid > rows) grid = rows;
    kern<<<(unsigned)grid, thr, smem, st>>>(loss_rows, dL, L, targets, w_rows, w_scalar, rows, (int)cols, beta, status);
    return check_launch();
  }
  if (vec_ok) {
    GroupPlan pl = plan_group(cols / VEC, NVMAX, g_nll_gpref, 256);
    if (pl.ok) {
      const int threads = pl.G * pl.groups;
      const int64_t want = (rows + pl.groups - 1) / pl.groups;
      // as many row buffers per group as fit (up to g_nll_stages), so a full row is always in flight
      int nstages = g_nll_stages;
      auto smem_for = [&](int ns) {
        return pl.groups * ns * ((size_t)cols * sizeof(T) + sizeof(uint64_t)) +
               (size_t)2 * pl.groups * kMaxWarpsPerGroup * 2 * sizeof(float);
      };
      while (nstages > 1 && smem_for(nstages) > kMaxDynSmem) --nstages;
      const size_t smem = smem_for(nstages);
#define CB_LAUNCH(NV_)                                                                          \
  do {                                                                                          \
    auto kern = softmax_nll_rows_kernel<T, TI, NV_, BWD>;                                       \
    int64_t grid = (int64_t)kNumSMs * resident_ctas(kern, threads, smem);                       \
    if (grid > want) grid = want;                                                               \
    kern<<<(unsigned)grid, threads, smem, st>>>(loss_rows, dL, L, targets, w_rows, w_scalar,    \
                                                rows, (int)cols, pl.G, nstages, beta, status);             \
  } while (0)
      if (smem <= kMaxDynSmem) {
        switch (pl.NV) {
          case 1: CB_LAUNCH(1); break;
          case 2: CB_LAUNCH(2); break;
          case 4: CB_LAUNCH(4); break;
          case 8: CB_LAUNCH(8); break;
          default: CB_LAUNCH(16); break;
        }
#undef CB_LAUNCH
        return check_launch();
      }
    }
  }
  int64_t grid = rows < (int64_t)kNumSMs * 8 ? rows : (int64_t)kNumSMs * 8;
  softmax_nll_rows_generic_kernel<T, TI, BWD><<<(unsigned)grid, 256, 0, st>>>(loss_rows, dL, L, targets, w_rows,
                                                                              w_scalar, rows, cols, beta, status);
  return check_launch();
}

}  // namespace cb

extern "C" {
size_t cacti_b200_softmax_nll_workspace_bytes(int64_t rows) {
  return rows > 0 ? (size_t)rows * sizeof(float) + 256 : 256;
}

int cacti_b200_softmax_nll_fwd_bwd(cacti_b200_dptr loss_sum, cacti_b200_dptr loss_rows, cacti_b200_dptr dlogits,
                                   cacti_b200_dptr logits, cacti_b200_dptr targets, int target_dtype,
                                   cacti_b200_dptr w_rows, float w_scalar, int64_t rows, int64_t vocab, int dtype,
                                   int beta_dlogits, cacti_b200_dptr status, cacti_b200_dptr workspace,
                                   size_t workspace_bytes, cacti_b200_stream stream) {
  using namespace cb;
  if (rows < 0 || vocab < 0 || vocab > 0x7fffffffLL) return CACTI_B200_ERR_INVALID_VALUE;
  if (beta_dlogits & ~1) return CACTI_B200_ERR_INVALID_VALUE;
  if (target_dtype != CACTI_B200_R_32I && target_dtype != CACTI_B200_R_16U) return CACTI_B200_ERR_DTYPE;
  if (dtype != CACTI_B200_R_32F && dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (rows == 0 || vocab == 0) return CACTI_B200_OK;
  if (!logits || !targets) return CACTI_B200_ERR_INVALID_VALUE;
  if ((loss_rows & 3) || (loss_sum & 3) || (w_rows & 3) || (status & 3)) return CACTI_B200_ERR_INVALID_VALUE;
  float* lrows = reinterpret_cast<float*>(loss_rows);
  if (loss_sum && !lrows) {
    if (!workspace || (workspace & 3) || workspace_bytes < cacti_b200_softmax_nll_workspace_bytes(rows))
      return CACTI_B200_ERR_WORKSPACE;
    lrows = reinterpret_cast<float*>(workspace);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const void* tg = reinterpret_cast<const void*>(targets);
  const float* wr = reinterpret_cast<const float*>(w_rows);
  unsigned* stw = reinterpret_cast<unsigned*>(status);
  const bool bwd = dlogits != 0;
  int rc = dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    if (target_dtype == CACTI_B200_R_32I) {
      return bwd ? launch_nll<T, int32_t, true>(lrows, dlogits, logits, tg, wr, w_scalar, rows, vocab, beta_dlogits, stw, st)
                 : launch_nll<T, int32_t, false>(lrows, dlogits, logits, tg, wr, w_scalar, rows, vocab, beta_dlogits, stw, st);
    }
    return bwd ? launch_nll<T, uint16_t, true>(lrows, dlogits, logits, tg, wr, w_scalar, rows, vocab, beta_dlogits, stw, st)
               : launch_nll<T, uint16_t, false>(lrows, dlogits, logits, tg, wr, w_scalar, rows, vocab, beta_dlogits, stw, st);
  });
  if (rc) return rc;
  if (loss_sum) {
    launch_dependent(nll_loss_sum_kernel, 1u, 1024u, st, reinterpret_cast<float*>(loss_sum), (const float*)lrows,
                     (const float*)wr, w_scalar, rows);
    return check_launch();
  }
  return CACTI_B200_OK;
}
}
