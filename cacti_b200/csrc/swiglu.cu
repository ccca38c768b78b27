// K4: SwiGLU forward / backward / fused forward+backward.
//
// Replaces `gate.standard_silu() * up` (src/librarium/llama.rs:526-527): StandardSilu
// (src/thunk/op.rs:2867-2910) + Mul (:2001-2056) forward, and about nine programs backward
// (silu and logistic recomputed, :2901-2908, :2821-2865).  One streaming pass here:
//   y = g / (1 + exp(-g));  h = y*u;  du = y*dh;  dy = dh*u;  t = 1/(1 + exp(-g));
//   dg = dy * (y*(1 - t) + t)
// f16: every primitive rounds to f16 as in the reference (the cells between thunks are f16);
// products/sums/differences use the non-contracting half2 *_rn intrinsics, exp and the two
// divisions are evaluated in f32 and rounded.  f32: separately rounded f32 ops.  bf16 (no
// reference chain) computes in f32 and rounds each output once.
#include "common.cuh"
#include <type_traits>

namespace cb {

int g_swiglu_threads = 256;
int g_swiglu_ctas_per_sm = 8;

// Scalar chain on f32 carriers; R rounds to the cell dtype at a thunk boundary.
template <typename T> struct Chain {
  static __device__ __forceinline__ float R(float v) { return round_to<T>(v); }
};
template <> struct Chain<__nv_bfloat16> {
  static __device__ __forceinline__ float R(float v) { return v; }
};

template <typename T, bool FWD, bool BWD>
__device__ __forceinline__ void swiglu_elem(float g, float u, float dh, float& h, float& dg, float& du) {
  using C = Chain<T>;
  const float e = C::R(exp_for<T>(-g));
  const float d = C::R(__fadd_rn(1.f, e));
  const float y = C::R(__fdiv_rn(g, d));
  if (FWD) h = C::R(__fmul_rn(y, u));
  if (BWD) {
    du = C::R(__fmul_rn(y, dh));
    const float dy = C::R(__fmul_rn(dh, u));
    const float t = C::R(__fdiv_rn(1.f, d));
    const float a = C::R(__fsub_rn(1.f, t));
    const float b = C::R(__fmul_rn(y, a));
    const float c = C::R(__fadd_rn(b, t));
    dg = C::R(__fmul_rn(dy, c));
  }
}

// One 4-byte unit of f16 data (two elements) through the chain.
template <bool FWD, bool BWD>
__device__ __forceinline__ void swiglu_h2(uint32_t gw, uint32_t uw, uint32_t dhw, uint32_t& hw, uint32_t& dgw,
                                          uint32_t& duw) {
  const __half2 g = *reinterpret_cast<__half2*>(&gw), u = *reinterpret_cast<__half2*>(&uw);
  const __half2 one = __float2half2_rn(1.f);
  const float2 gf = __half22float2(g);
  const __half2 e = __floats2half2_rn(__expf(-gf.x), __expf(-gf.y));
  const __half2 d = __hadd2_rn(one, e);
  const float2 df = __half22float2(d);
  float rx, ry;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rx) : "f"(df.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(ry) : "f"(df.y));
  const __half2 y = __floats2half2_rn(gf.x * rx, gf.y * ry);
  if (FWD) { const __half2 h = __hmul2_rn(y, u); hw = *reinterpret_cast<const uint32_t*>(&h); }
  if (BWD) {
    const __half2 dh = *reinterpret_cast<__half2*>(&dhw);
    const __half2 du = __hmul2_rn(y, dh);
    const __half2 dy = __hmul2_rn(dh, u);
    const __half2 t = __floats2half2_rn(rx, ry);
    const __half2 a = __hsub2_rn(one, t);
    const __half2 b = __hmul2_rn(y, a);
    const __half2 c = __hadd2_rn(b, t);
    const __half2 dg = __hmul2_rn(dy, c);
    duw = *reinterpret_cast<const uint32_t*>(&du);
    dgw = *reinterpret_cast<const uint32_t*>(&dg);
  }
}

__device__ __forceinline__ uint32_t hadd_unit(uint32_t a, uint32_t b) {
  const __half2 y = __hadd2_rn(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&y);
}

template <typename T, bool FWD, bool BWD>
__device__ __forceinline__ void swiglu_vec(const uint4& g, const uint4& u, const uint4& dh, uint4& h, uint4& dg,
                                           uint4& du) {
  if constexpr (std::is_same<T, __half>::value) {
    swiglu_h2<FWD, BWD>(g.x, u.x, dh.x, h.x, dg.x, du.x);
    swiglu_h2<FWD, BWD>(g.y, u.y, dh.y, h.y, dg.y, du.y);
    swiglu_h2<FWD, BWD>(g.z, u.z, dh.z, h.z, dg.z, du.z);
    swiglu_h2<FWD, BWD>(g.w, u.w, dh.w, h.w, dg.w, du.w);
  } else {
    constexpr int VEC = Elem<T>::VEC;
    float gf[VEC], uf[VEC], df[VEC], hf[VEC], dgf[VEC], duf[VEC];
    unpack<T>(g, gf); unpack<T>(u, uf);
    if (BWD) unpack<T>(dh, df);
#pragma unroll
    for (int e = 0; e < VEC; ++e) swiglu_elem<T, FWD, BWD>(gf[e], uf[e], BWD ? df[e] : 0.f, hf[e], dgf[e], duf[e]);
    if (FWD) h = pack<T>(hf);
    if (BWD) { dg = pack<T>(dgf); du = pack<T>(duf); }
  }
}

template <typename T> __device__ __forceinline__ uint4 vec_accumulate(const uint4& old, const uint4& v) {
  if constexpr (std::is_same<T, __half>::value) {
    return make_uint4(hadd_unit(old.x, v.x), hadd_unit(old.y, v.y), hadd_unit(old.z, v.z), hadd_unit(old.w, v.w));
  } else {
    float f[Elem<T>::VEC];
    unpack<T>(v, f);
    return pack_accumulate<T>(f, old);
  }
}

template <typename T, bool FWD, bool BWD>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(T* __restrict__ H, T* __restrict__ dG, T* __restrict__ dU, const T* __restrict__ G,
                  const T* __restrict__ U, const T* __restrict__ dH, int64_t n, int beta_g, int beta_u) {
  constexpr int VEC = Elem<T>::VEC;
  const int64_t nvec = n / VEC;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // two vectors per thread per trip: 4 (fwd) or 6 (fwd+bwd) 16-byte loads in flight
  for (; v + stride < nvec; v += 2 * stride) {
    uint4 g[2], u[2], dh[2], h[2], dg[2], du[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int64_t e0 = (v + i * stride) * VEC;
      g[i] = ld_stream(G + e0); u[i] = ld_stream(U + e0);
      if (BWD) dh[i] = ld_stream(dH + e0);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int64_t e0 = (v + i * stride) * VEC;
      swiglu_vec<T, FWD, BWD>(g[i], u[i], dh[i], h[i], dg[i], du[i]);
      if (FWD) st_stream(H + e0, h[i]);
      if (BWD) {
        if (beta_g) dg[i] = vec_accumulate<T>(ld_stream(dG + e0), dg[i]);
        if (beta_u) du[i] = vec_accumulate<T>(ld_stream(dU + e0), du[i]);
        st_stream(dG + e0, dg[i]); st_stream(dU + e0, du[i]);
      }
    }
  }
  for (; v < nvec; v += stride) {
    const int64_t e0 = v * VEC;
    uint4 g = ld_stream(G + e0), u = ld_stream(U + e0), dh, h, dg, du;
    if (BWD) dh = ld_stream(dH + e0);
    swiglu_vec<T, FWD, BWD>(g, u, dh, h, dg, du);
    if (FWD) st_stream(H + e0, h);
    if (BWD) {
      if (beta_g) dg = vec_accumulate<T>(ld_stream(dG + e0), dg);
      if (beta_u) du = vec_accumulate<T>(ld_stream(dU + e0), du);
      st_stream(dG + e0, dg); st_stream(dU + e0, du);
    }
  }
}

// Element-wise kernel: the tail after the last full vector, or the whole array when a pointer is
// not 16-byte aligned.
template <typename T, bool FWD, bool BWD>
__global__ void __launch_bounds__(256)
swiglu_scalar_kernel(T* __restrict__ H, T* __restrict__ dG, T* __restrict__ dU, const T* __restrict__ G,
                     const T* __restrict__ U, const T* __restrict__ dH, int64_t begin, int64_t n, int beta_g,
                     int beta_u) {
  for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float h, dg, du;
    swiglu_elem<T, FWD, BWD>(Elem<T>::to_f32(G[i]), Elem<T>::to_f32(U[i]), BWD ? Elem<T>::to_f32(dH[i]) : 0.f, h, dg, du);
    if (FWD) H[i] = Elem<T>::from_f32(h);
    if (BWD) {
      dG[i] = beta_g ? Elem<T>::from_f32(Elem<T>::to_f32(dG[i]) + round_to<T>(dg)) : Elem<T>::from_f32(dg);
      dU[i] = beta_u ? Elem<T>::from_f32(Elem<T>::to_f32(dU[i]) + round_to<T>(du)) : Elem<T>::from_f32(du);
    }
  }
}

template <typename T, bool FWD, bool BWD>
static int launch_swiglu(uint64_t h, uint64_t dg, uint64_t du, uint64_t g, uint64_t u, uint64_t dh, int64_t n,
                         int beta_g, int beta_u, cudaStream_t st) {
  constexpr int VEC = Elem<T>::VEC;
  T* H = reinterpret_cast<T*>(h); T* dG = reinterpret_cast<T*>(dg); T* dU = reinterpret_cast<T*>(du);
  const T* G = reinterpret_cast<const T*>(g); const T* U = reinterpret_cast<const T*>(u);
  const T* dH = reinterpret_cast<const T*>(dh);
  const bool vec_ok = aligned16(g) && aligned16(u) && (!FWD || aligned16(h)) &&
                      (!BWD || (aligned16(dh) && aligned16(dg) && aligned16(du)));
  const int threads = g_swiglu_threads;
  int64_t done = 0;
  if (vec_ok && n >= VEC) {
    const int64_t nvec = n / VEC;
    int64_t grid = (nvec + 2 * threads - 1) / (2 * threads);
    const int64_t cap = (int64_t)kNumSMs * g_swiglu_ctas_per_sm;
    if (grid > cap) grid = cap;
    swiglu_vec_kernel<T, FWD, BWD><<<(unsigned)grid, threads, 0, st>>>(H, dG, dU, G, U, dH, n, beta_g, beta_u);
    int rc = check_launch();
    if (rc) return rc;
    done = nvec * VEC;
  }
  if (done < n) {
    int64_t grid = (n - done + threads - 1) / threads;
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (grid > cap) grid = cap;
    swiglu_scalar_kernel<T, FWD, BWD><<<(unsigned)grid, threads, 0, st>>>(H, dG, dU, G, U, dH, done, n, beta_g, beta_u);
    return check_launch();
  }
  return CACTI_B200_OK;
}

static int swiglu_entry(bool fwd, bool bwd, uint64_t h, uint64_t dg, uint64_t du, uint64_t g, uint64_t u, uint64_t dh,
                        int64_t n, int dtype, int beta_g, int beta_u, void* stream) {
  if (n < 0 || ((beta_g | beta_u) & ~1)) return CACTI_B200_ERR_INVALID_VALUE;
  if (n == 0) return CACTI_B200_OK;
  if (!g || !u || (fwd && !h) || (bwd && (!dh || !dg || !du))) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    if (fwd && bwd) return launch_swiglu<T, true, true>(h, dg, du, g, u, dh, n, beta_g, beta_u, st);
    if (fwd) return launch_swiglu<T, true, false>(h, dg, du, g, u, dh, n, beta_g, beta_u, st);
    return launch_swiglu<T, false, true>(h, dg, du, g, u, dh, n, beta_g, beta_u, st);
  });
}

}  // namespace cb

extern "C" {
int cacti_b200_swiglu_fwd(cacti_b200_dptr h, cacti_b200_dptr gate, cacti_b200_dptr up, int64_t n, int dtype,
                          cacti_b200_stream stream) {
  return cb::swiglu_entry(true, false, h, 0, 0, gate, up, 0, n, dtype, 0, 0, stream);
}
int cacti_b200_swiglu_bwd(cacti_b200_dptr dgate, cacti_b200_dptr dup, cacti_b200_dptr gate, cacti_b200_dptr up,
                          cacti_b200_dptr dh, int64_t n, int dtype, int beta_dgate, int beta_dup,
                          cacti_b200_stream stream) {
  return cb::swiglu_entry(false, true, 0, dgate, dup, gate, up, dh, n, dtype, beta_dgate, beta_dup, stream);
}
int cacti_b200_swiglu_fwd_bwd(cacti_b200_dptr h, cacti_b200_dptr dgate, cacti_b200_dptr dup, cacti_b200_dptr gate,
                              cacti_b200_dptr up, cacti_b200_dptr dh, int64_t n, int dtype, int beta_dgate,
                              int beta_dup, cacti_b200_stream stream) {
  return cb::swiglu_entry(true, true, h, dgate, dup, gate, up, dh, n, dtype, beta_dgate, beta_dup, stream);
}
}
