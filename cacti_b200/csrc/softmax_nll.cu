// K5: softmax cross-entropy, loss and dlogits in one pass over the logits.
//
// Replaces cast(f32) -> inner_softmax_categorical_nll (src/thunk/op.rs:3460-3569, call site
// src/librarium/llama.rs:542-545) and its adjoint, which in the reference recomputes the softmax,
// materialises a dense f32 one-hot [rows, vocab] (src/thunk/op.rs:883-997), subtracts and scales.
// Here a row of logits is read once into registers (raw 16-byte vectors), reduced twice (max,
// sum of exp) and the gradient is written once; the one-hot is a comparison on the column index.
#include "common.cuh"
#include <type_traits>

namespace cb {

int g_nll_gpref = 512;

template <typename TI> __device__ __forceinline__ int64_t load_index(const void* p, int64_t i);
template <> __device__ __forceinline__ int64_t load_index<int32_t>(const void* p, int64_t i) {
  return (int64_t) reinterpret_cast<const int32_t*>(p)[i];
}
template <> __device__ __forceinline__ int64_t load_index<uint16_t>(const void* p, int64_t i) {
  return (int64_t) reinterpret_cast<const uint16_t*>(p)[i];
}

template <typename T, typename TI, int NV, bool BWD>
__global__ void __launch_bounds__(512)
softmax_nll_rows_kernel(float* __restrict__ loss_rows, T* __restrict__ dL, const T* __restrict__ L,
                        const void* __restrict__ targets, const float* __restrict__ w_rows, float w_scalar,
                        int64_t rows, int cols, int G, int beta, unsigned* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int VEC = Elem<T>::VEC;
  const int groups = blockDim.x / G;
  const unsigned row_bytes = (unsigned)cols * sizeof(T);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)groups * row_bytes);
  float* red = reinterpret_cast<float*>(bars + groups);
  GroupCtx g = make_group(G, red);
  unsigned char* stage = smem_raw + (size_t)g.gid * row_bytes;
  uint64_t* bar = bars + g.gid;
  if (g.lane == 0) mbar_init(bar, 1);
  mbar_fence_init();
  __syncthreads();
  const int64_t stride = (int64_t)gridDim.x * groups;
  int64_t row = (int64_t)blockIdx.x * groups + g.gid;
  unsigned phase = 0;
  auto issue = [&](int64_t r) {
    if (g.lane == 0) { mbar_expect_tx(bar, row_bytes); bulk_g2s(stage, L + r * cols, row_bytes, bar); }
  };
  if (row < rows) issue(row);
  for (; row < rows; row += stride) {
    const int64_t tgt = load_index<TI>(targets, row);
    const bool tgt_ok = tgt >= 0 && tgt < cols;
    const float w = w_rows ? w_rows[row] : w_scalar;
    if (!mbar_wait_bounded(bar, phase, kDevErrStageTimeout)) return;
    phase ^= 1;
    uint4 raw[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) raw[k] = *reinterpret_cast<const uint4*>(stage + (size_t)col0 * sizeof(T));
    }
    // the target logit, read from the staged row (the stored bit pattern, converted exactly)
    const float a_t = tgt_ok ? Elem<T>::to_f32(reinterpret_cast<const T*>(stage)[tgt]) : 0.f;
    group_barrier(g);
    if (row + stride < rows) issue(row + stride);

    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) {
        float a[VEC];
        unpack<T>(raw[k], a);
#pragma unroll
        for (int e = 0; e < VEC; ++e) m = fmaxf(m, a[e]);
      }
    }
    m = group_reduce<MaxOp>(g, m);
    float z = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int col0 = (g.lane + k * G) * VEC;
      if (col0 < cols) {
        float a[VEC];
        unpack<T>(raw[k], a);
#pragma unroll
        for (int e = 0; e < VEC; ++e) z += exp_for<T>(a[e] - m);
      }
    }
    z = group_reduce<SumOp>(g, z);
    if (g.lane == 0) {
      if (!tgt_ok && status) atomicMax(status, (unsigned)CACTI_B200_ERR_INDEX_RANGE);
      // -log(y_k) with y_k = exp(a_k - m) / z, formed as in the reference (src/thunk/op.rs:3543)
      if (loss_rows) loss_rows[row] = tgt_ok ? -logf(expf(a_t - m) / z) : __int_as_float(0x7fc00000);
    }
    if (BWD) {
      const float rz = 1.f / z;
      T* drow = dL + row * cols;
      const int tcol = tgt_ok ? (int)tgt : -1;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int col0 = (g.lane + k * G) * VEC;
        if (col0 < cols) {
          float a[VEC], d[VEC];
          unpack<T>(raw[k], a);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float ex = exp_for<T>(a[e] - m);
            const float y = std::is_same<T, float>::value ? ex / z : ex * rz;
            d[e] = w * (y - ((col0 + e) == tcol ? 1.f : 0.f));
          }
          if (beta) st_stream(drow + col0, pack_accumulate<T>(d, ld_stream(drow + col0)));
          else st_stream(drow + col0, pack<T>(d));
        }
      }
    }
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
  if (vec_ok) {
    GroupPlan pl = plan_group(cols / VEC, NVMAX, g_nll_gpref, 256);
    if (pl.ok) {
      const int threads = pl.G * pl.groups;
      const int64_t want = (rows + pl.groups - 1) / pl.groups;
      const size_t smem = pl.groups * ((size_t)cols * sizeof(T) + sizeof(uint64_t)) +
                          (size_t)2 * pl.groups * kMaxWarpsPerGroup * 2 * sizeof(float);
#define CB_LAUNCH(NV_)                                                                          \
  do {                                                                                          \
    auto kern = softmax_nll_rows_kernel<T, TI, NV_, BWD>;                                       \
    int64_t grid = (int64_t)kNumSMs * resident_ctas(kern, threads, smem);                       \
    if (grid > want) grid = want;                                                               \
    kern<<<(unsigned)grid, threads, smem, st>>>(loss_rows, dL, L, targets, w_rows, w_scalar,    \
                                                rows, (int)cols, pl.G, beta, status);           \
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
    nll_loss_sum_kernel<<<1, 1024, 0, st>>>(reinterpret_cast<float*>(loss_sum), lrows, wr, w_scalar, rows);
    return check_launch();
  }
  return CACTI_B200_OK;
}
}
