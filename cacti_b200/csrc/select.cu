// K6 / K6b: embedding row gather and its adjoint (scatter-add), and K7: add / accumulate.
//
// gather_rows replaces OuterSelect (src/thunk/op.rs:1229-1314): a bit-exact row copy by token id.
// scatter_add_rows is its adjoint.  The reference gets it from Futhark's vjp of the gather; here it is
// made deterministic: tokens are bucketed by id with a stable counting sort (integer atomics only for
// the histogram), then one CTA per table row adds that row's contributions in token order in f32 and
// rounds once.  accumulate / add replace the NVRTC accumulate_1d kernels (src/pctx/nvgpu.rs:2598-2668)
// and AddFutThunkSpec (src/thunk/op.rs:1480-1535).
#include "common.cuh"
#include <type_traits>

namespace cb {

template <typename TI> __device__ __forceinline__ int64_t tok_at(const void* p, int64_t i);
template <> __device__ __forceinline__ int64_t tok_at<int32_t>(const void* p, int64_t i) {
  return (int64_t) reinterpret_cast<const int32_t*>(p)[i];
}
template <> __device__ __forceinline__ int64_t tok_at<uint16_t>(const void* p, int64_t i) {
  return (int64_t) reinterpret_cast<const uint16_t*>(p)[i];
}

// ---- gather ------------------------------------------------------------------------------
// COPY = uint4 (16-byte rows) or uint16_t / uint32_t (element copies for unaligned views).
template <typename TI, typename COPY>
__global__ void __launch_bounds__(128)
gather_rows_kernel(COPY* __restrict__ out, const COPY* __restrict__ table, const void* __restrict__ tokens,
                   int64_t n_tokens, int64_t vocab, int64_t units_per_row, unsigned* __restrict__ status) {
  for (int64_t i = blockIdx.x; i < n_tokens; i += gridDim.x) {
    const int64_t k = tok_at<TI>(tokens, i);
    if (k < 0 || k >= vocab) {           // reference: Futhark bounds failure; here: report and skip the row
      if (threadIdx.x == 0 && status) atomicMax(status, (unsigned)CACTI_B200_ERR_INDEX_RANGE);
      continue;
    }
    const COPY* src = table + k * units_per_row;
    COPY* dst = out + i * units_per_row;
    for (int64_t j = threadIdx.x; j < units_per_row; j += blockDim.x) dst[j] = src[j];
  }
}

// ---- scatter-add ---------------------------------------------------------------------------
template <typename TI>
__global__ void token_histogram_kernel(int* __restrict__ counts, const void* __restrict__ tokens, int64_t n_tokens,
                                       int64_t vocab, unsigned* __restrict__ status) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_tokens; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t k = tok_at<TI>(tokens, i);
    if (k < 0 || k >= vocab) { if (status) atomicMax(status, (unsigned)CACTI_B200_ERR_INDEX_RANGE); }
    else atomicAdd(&counts[k], 1);
  }
}

// In place: counts[v] -> start offset of bucket v; counts[vocab] = total.  One CTA.
__global__ void __launch_bounds__(1024) bucket_scan_kernel(int* __restrict__ counts, int64_t vocab) {
  __shared__ int sm[1024];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < vocab; base += 1024) {
    const int64_t j = base + threadIdx.x;
    const int c = j < vocab ? counts[j] : 0;
    sm[threadIdx.x] = c;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const int t = (int)threadIdx.x >= o ? sm[threadIdx.x - o] : 0;
      __syncthreads();
      sm[threadIdx.x] += t;
      __syncthreads();
    }
    const int incl = sm[threadIdx.x];
    if (j < vocab) counts[j] = carry + incl - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry += incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[vocab] = carry;
}

// Stable placement: order[start[k] + (number of earlier tokens with the same id)] = token index.
// One CTA walks the tokens in chunks of 1024, so "earlier" is well defined without sorting.
template <typename TI>
__global__ void __launch_bounds__(1024)
bucket_place_kernel(int* __restrict__ order, int* __restrict__ fill, const int* __restrict__ start,
                    const void* __restrict__ tokens, int64_t n_tokens, int64_t vocab) {
  __shared__ int keys[1024];
  for (int64_t base = 0; base < n_tokens; base += 1024) {
    const int64_t i = base + threadIdx.x;
    int64_t k = i < n_tokens ? tok_at<TI>(tokens, i) : -1;
    if (k < 0 || k >= vocab) k = -1;
    keys[threadIdx.x] = (int)k;
    __syncthreads();
    int before = 0, total = 0, f = 0;
    if (k >= 0) {
      const int lim = (int)((n_tokens - base) < 1024 ? (n_tokens - base) : 1024);
      for (int t = 0; t < lim; ++t) {
        const bool same = keys[t] == (int)k;
        total += same;
        before += same && t < (int)threadIdx.x;
      }
      f = fill[k];
      order[start[k] + f + before] = (int)i;
    }
    __syncthreads();                        // every fill[k] is read before any is updated
    if (k >= 0 && before == total - 1) fill[k] = f + total;
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
scatter_sum_kernel(T* __restrict__ dtable, const T* __restrict__ dy, const int* __restrict__ order,
                   const int* __restrict__ start, int64_t vocab, int64_t cols, int beta, int vec) {
  constexpr int VEC = Elem<T>::VEC;
  for (int64_t v = blockIdx.x; v < vocab; v += gridDim.x) {
    const int b = start[v], e = start[v + 1];
    if (b == e && beta) continue;
    T* orow = dtable + v * cols;
    if (vec) {
      for (int64_t c0 = (int64_t)threadIdx.x * VEC; c0 < cols; c0 += (int64_t)blockDim.x * VEC) {
        float acc[VEC];
#pragma unroll
        for (int q = 0; q < VEC; ++q) acc[q] = 0.f;
        for (int t = b; t < e; ++t) {
          float f[VEC];
          unpack<T>(ld_stream(dy + (int64_t)order[t] * cols + c0), f);
#pragma unroll
          for (int q = 0; q < VEC; ++q) acc[q] += f[q];
        }
        if (beta) st_stream(orow + c0, pack_accumulate<T>(acc, ld_stream(orow + c0)));
        else st_stream(orow + c0, pack<T>(acc));
      }
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        float acc = 0.f;
        for (int t = b; t < e; ++t) acc += Elem<T>::to_f32(dy[(int64_t)order[t] * cols + c]);
        orow[c] = beta ? Elem<T>::from_f32(Elem<T>::to_f32(orow[c]) + round_to<T>(acc)) : Elem<T>::from_f32(acc);
      }
    }
  }
}

// ---- add / accumulate ------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ uint4 add_vec(const uint4& a, const uint4& b) {
  if constexpr (std::is_same<T, __half>::value) {
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 y = __hadd2_rn(*reinterpret_cast<const __half2*>(&aw[i]), *reinterpret_cast<const __half2*>(&bw[i]));
      r[i] = *reinterpret_cast<const uint32_t*>(&y);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
  } else {
    float fa[Elem<T>::VEC], fb[Elem<T>::VEC];
    unpack<T>(a, fa); unpack<T>(b, fb);
#pragma unroll
    for (int i = 0; i < Elem<T>::VEC; ++i) fa[i] = __fadd_rn(fa[i], fb[i]);
    return pack<T>(fa);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
add_vec_kernel(T* out, const T* a, const T* b, int64_t nvec) {   // out may alias a (accumulate)
  constexpr int VEC = Elem<T>::VEC;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; v + stride < nvec; v += 2 * stride) {
    const uint4 a0 = ld_stream(a + v * VEC), b0 = ld_stream(b + v * VEC);
    const uint4 a1 = ld_stream(a + (v + stride) * VEC), b1 = ld_stream(b + (v + stride) * VEC);
    st_stream(out + v * VEC, add_vec<T>(a0, b0));
    st_stream(out + (v + stride) * VEC, add_vec<T>(a1, b1));
  }
  for (; v < nvec; v += stride) st_stream(out + v * VEC, add_vec<T>(ld_stream(a + v * VEC), ld_stream(b + v * VEC)));
}

template <typename T>
__global__ void __launch_bounds__(256)
add_scalar_kernel(T* out, const T* a, const T* b, int64_t begin, int64_t n) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = Elem<T>::from_f32(__fadd_rn(Elem<T>::to_f32(a[i]), Elem<T>::to_f32(b[i])));
}

static int add_entry(uint64_t out, uint64_t a, uint64_t b, int64_t n, int dtype, void* stream) {
  if (n < 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (n == 0) return CACTI_B200_OK;
  if (!out || !a || !b) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Elem<T>::VEC;
    T* O = reinterpret_cast<T*>(out);
    const T* A = reinterpret_cast<const T*>(a); const T* B = reinterpret_cast<const T*>(b);
    int64_t done = 0;
    if (aligned16(out) && aligned16(a) && aligned16(b) && n >= VEC) {
      const int64_t nvec = n / VEC;
      int64_t grid = (nvec + 511) / 512;
      if (grid > (int64_t)kNumSMs * 8) grid = (int64_t)kNumSMs * 8;
      add_vec_kernel<T><<<(unsigned)grid, 256, 0, st>>>(O, A, B, nvec);
      int rc = check_launch();
      if (rc) return rc;
      done = nvec * VEC;
    }
    if (done < n) {
      int64_t grid = (n - done + 255) / 256;
      if (grid > (int64_t)kNumSMs * 16) grid = (int64_t)kNumSMs * 16;
      add_scalar_kernel<T><<<(unsigned)grid, 256, 0, st>>>(O, A, B, done, n);
      return check_launch();
    }
    return CACTI_B200_OK;
  });
}

static size_t scatter_ws_bytes(int64_t n_tokens, int64_t vocab) {
  // start[vocab+1] | fill[vocab] | order[n_tokens], 4-byte ints, each block 256-byte aligned
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  return up((size_t)(vocab + 1) * 4) + up((size_t)vocab * 4) + up((size_t)n_tokens * 4) + 256;
}

}  // namespace cb

extern "C" {

int cacti_b200_gather_rows(cacti_b200_dptr out, cacti_b200_dptr table, cacti_b200_dptr tokens, int token_dtype,
                           int64_t n_tokens, int64_t vocab, int64_t cols, int dtype, cacti_b200_dptr status,
                           cacti_b200_stream stream) {
  using namespace cb;
  if (n_tokens < 0 || vocab < 0 || cols < 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (token_dtype != CACTI_B200_R_32I && token_dtype != CACTI_B200_R_16U) return CACTI_B200_ERR_DTYPE;
  int esize;
  switch (dtype) {
    case CACTI_B200_R_32F: esize = 4; break;
    case CACTI_B200_R_16F: case CACTI_B200_R_16BF: esize = 2; break;
    default: return CACTI_B200_ERR_DTYPE;
  }
  if (n_tokens == 0 || cols == 0) return CACTI_B200_OK;
  if (!out || !table || !tokens || (status & 3)) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned* stw = reinterpret_cast<unsigned*>(status);
  const void* tk = reinterpret_cast<const void*>(tokens);
  const int64_t row_bytes = cols * esize;
  int64_t grid = n_tokens < (int64_t)kNumSMs * 16 ? n_tokens : (int64_t)kNumSMs * 16;
#define CB_GATHER(TI_, COPY_, UNITS_)                                                                          \
  gather_rows_kernel<TI_, COPY_><<<(unsigned)grid, 128, 0, st>>>(reinterpret_cast<COPY_*>(out),                \
      reinterpret_cast<const COPY_*>(table), tk, n_tokens, vocab, (UNITS_), stw)
  const bool i32 = token_dtype == CACTI_B200_R_32I;
  if (row_bytes % 16 == 0 && aligned16(out) && aligned16(table)) {
    if (i32) CB_GATHER(int32_t, uint4, row_bytes / 16); else CB_GATHER(uint16_t, uint4, row_bytes / 16);
  } else if (esize == 4) {
    if (i32) CB_GATHER(int32_t, uint32_t, cols); else CB_GATHER(uint16_t, uint32_t, cols);
  } else {
    if (i32) CB_GATHER(int32_t, uint16_t, cols); else CB_GATHER(uint16_t, uint16_t, cols);
  }
#undef CB_GATHER
  return check_launch();
}

size_t cacti_b200_scatter_add_rows_workspace_bytes(int64_t n_tokens, int64_t vocab) {
  if (n_tokens < 0 || vocab < 0) return 0;
  return cb::scatter_ws_bytes(n_tokens, vocab);
}

int cacti_b200_scatter_add_rows(cacti_b200_dptr dtable, cacti_b200_dptr dy, cacti_b200_dptr tokens, int token_dtype,
                                int64_t n_tokens, int64_t vocab, int64_t cols, int dtype, int beta,
                                cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_dptr status,
                                cacti_b200_stream stream) {
  using namespace cb;
  if (n_tokens < 0 || vocab < 0 || cols < 0 || (beta & ~1)) return CACTI_B200_ERR_INVALID_VALUE;
  if (n_tokens > 0x7fffffffLL || vocab >= 0x7fffffffLL) return CACTI_B200_ERR_SHAPE;
  if (token_dtype != CACTI_B200_R_32I && token_dtype != CACTI_B200_R_16U) return CACTI_B200_ERR_DTYPE;
  if (dtype != CACTI_B200_R_32F && dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (vocab == 0 || cols == 0) return CACTI_B200_OK;
  if (!dtable || (n_tokens > 0 && (!dy || !tokens)) || (status & 3)) return CACTI_B200_ERR_INVALID_VALUE;
  if (!workspace || (workspace & 255) || workspace_bytes < scatter_ws_bytes(n_tokens, vocab)) return CACTI_B200_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  int* start = reinterpret_cast<int*>(workspace);
  int* fill = reinterpret_cast<int*>(workspace + up((size_t)(vocab + 1) * 4));
  int* order = reinterpret_cast<int*>(workspace + up((size_t)(vocab + 1) * 4) + up((size_t)vocab * 4));
  unsigned* stw = reinterpret_cast<unsigned*>(status);
  const void* tk = reinterpret_cast<const void*>(tokens);
  // start and fill are adjacent: one clear covers both
  if (cudaMemsetAsync(start, 0, up((size_t)(vocab + 1) * 4) + up((size_t)vocab * 4), st) != cudaSuccess) return check_launch();
  const bool i32 = token_dtype == CACTI_B200_R_32I;
  if (n_tokens > 0) {
    int64_t grid = (n_tokens + 255) / 256;
    if (grid > kNumSMs * 4) grid = kNumSMs * 4;
    if (i32) token_histogram_kernel<int32_t><<<(unsigned)grid, 256, 0, st>>>(start, tk, n_tokens, vocab, stw);
    else token_histogram_kernel<uint16_t><<<(unsigned)grid, 256, 0, st>>>(start, tk, n_tokens, vocab, stw);
    int rc = check_launch();
    if (rc) return rc;
  }
  bucket_scan_kernel<<<1, 1024, 0, st>>>(start, vocab);
  int rc = check_launch();
  if (rc) return rc;
  if (n_tokens > 0) {
    if (i32) bucket_place_kernel<int32_t><<<1, 1024, 0, st>>>(order, fill, start, tk, n_tokens, vocab);
    else bucket_place_kernel<uint16_t><<<1, 1024, 0, st>>>(order, fill, start, tk, n_tokens, vocab);
    rc = check_launch();
    if (rc) return rc;
  }
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VEC = Elem<T>::VEC;
    const int vec = (cols % VEC == 0) && aligned16(dtable) && aligned16(dy);
    int64_t grid = vocab < (int64_t)kNumSMs * 32 ? vocab : (int64_t)kNumSMs * 32;
    scatter_sum_kernel<T><<<(unsigned)grid, 128, 0, st>>>(reinterpret_cast<T*>(dtable), reinterpret_cast<const T*>(dy),
                                                         order, start, vocab, cols, beta, vec);
    return check_launch();
  });
}

int cacti_b200_accumulate(cacti_b200_dptr dst, cacti_b200_dptr src, int64_t n, int dtype, cacti_b200_stream stream) {
  return cb::add_entry(dst, dst, src, n, dtype, stream);
}
int cacti_b200_add(cacti_b200_dptr out, cacti_b200_dptr a, cacti_b200_dptr b, int64_t n, int dtype,
                   cacti_b200_stream stream) {
  return cb::add_entry(out, a, b, n, dtype, stream);
}
}
