// K8: AdamW32 parameter update, the three in-place ("Initialize") optimizer thunks of the reference fused into
// one streaming pass.
//
// Reference (src/librarium/adamw.rs:46-61 and src/op.rs:950-1023):
//   grad1_avg.init_online_average_scale(grad, s, a1)         m <- m + a1 * (s * f32(g) - m)            src/thunk/op.rs:3929-3934
//   grad2_avg.init_online_average_square_scale(grad, s, a2)  v <- v + a2 * ((s*f32(g)) * (s*f32(g)) - v)  :3991-3998
//   master.init_online_adamw_update32(m, v, t, lr, wd, ...)  w <- w + (-lr) * (u * (m / (sqrt(v) + e)) + wd * w)  :4051-4055
// with u = unbias2 / unbias1, e = eps * unbias2, unbias1 = 1 - (1 - a1)^t (a1 when t = 1),
// unbias2 = sqrt(1 - (1 - a2)^t) (sqrt(a2) when t = 1), all computed on the host in f32 as src/op.rs:985-1012 does.
// m, v, w are f32 cells updated in place; g is the (f16, bf16 or f32) gradient.  The example then refreshes the
// 16-bit parameter from the f32 master with a lossy cast; `param_out` (optional) receives that cast in the same pass.
// Every f32 operation is issued with an explicit round-to-nearest intrinsic in the reference's order, so the
// result is bit-identical to evaluating the three programs one after the other.
// HBM-bound: 14 bytes read and 14 written per parameter with f16 gradients and a 16-bit parameter copy.
#include "common.cuh"
#include <math.h>
#include <type_traits>

namespace cb {

// f32 integer power by repeated squaring, the algorithm behind Rust's f32::powi used at src/op.rs:990,1000
static float powi_f32(float a, int b) {
  float r = 1.0f;
  for (;;) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return r;
}

struct AdamwScalars { float s, a1, a2, neg_lr, u, wd, e; };

__device__ __forceinline__ void adamw_one(float g, float& m, float& v, float& w, const AdamwScalars& c) {
  const float sg = __fmul_rn(c.s, g);
  m = __fadd_rn(m, __fmul_rn(c.a1, __fsub_rn(sg, m)));
  v = __fadd_rn(v, __fmul_rn(c.a2, __fsub_rn(__fmul_rn(sg, sg), v)));
  const float r = __fdiv_rn(m, __fadd_rn(__fsqrt_rn(v), c.e));
  w = __fadd_rn(w, __fmul_rn(c.neg_lr, __fadd_rn(__fmul_rn(c.u, r), __fmul_rn(c.wd, w))));
}

// TG: gradient type, TP: type of the optional parameter copy.  VEC_G elements of g per thread per trip.
template <typename TG, typename TP>
__global__ void __launch_bounds__(256)
adamw32_kernel(float* __restrict__ W, float* __restrict__ M, float* __restrict__ V, TP* __restrict__ P,
               const TG* __restrict__ G, int64_t n, AdamwScalars c, int vec_ok) {
  constexpr int VG = Elem<TG>::VEC;                 // 8 (16-bit gradients) or 4 (f32)
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (vec_ok) {
    const int64_t nvec = n / VG;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
      const int64_t e0 = i * VG;
      float g[VG], m[VG], v[VG], w[VG];
      unpack<TG>(ld_stream(G + e0), g);
#pragma unroll
      for (int q = 0; q < VG / 4; ++q) {
        float t[4];
        unpack<float>(ld_stream(M + e0 + 4 * q), t);
#pragma unroll
        for (int j = 0; j < 4; ++j) m[4 * q + j] = t[j];
        unpack<float>(ld_stream(V + e0 + 4 * q), t);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[4 * q + j] = t[j];
        unpack<float>(ld_stream(W + e0 + 4 * q), t);
#pragma unroll
        for (int j = 0; j < 4; ++j) w[4 * q + j] = t[j];
      }
#pragma unroll
      for (int j = 0; j < VG; ++j) adamw_one(g[j], m[j], v[j], w[j], c);
#pragma unroll
      for (int q = 0; q < VG / 4; ++q) {
        float t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = m[4 * q + j];
        st_stream(M + e0 + 4 * q, pack<float>(t));
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = v[4 * q + j];
        st_stream(V + e0 + 4 * q, pack<float>(t));
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = w[4 * q + j];
        st_stream(W + e0 + 4 * q, pack<float>(t));
      }
      if (P) {
        if constexpr (Elem<TP>::VEC == VG) {
          st_stream(P + e0, pack<TP>(w));
        } else {
#pragma unroll
          for (int j = 0; j < VG; ++j) P[e0 + j] = Elem<TP>::from_f32(w[j]);
        }
      }
    }
    done = nvec * VG;
  }
  for (int64_t i = done + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float m = M[i], v = V[i], w = W[i];
    adamw_one(Elem<TG>::to_f32(G[i]), m, v, w, c);
    M[i] = m; V[i] = v; W[i] = w;
    if (P) P[i] = Elem<TP>::from_f32(w);
  }
}

}  // namespace cb

extern "C" int cacti_b200_adamw32_step(cacti_b200_dptr master, cacti_b200_dptr grad1_avg, cacti_b200_dptr grad2_avg,
                                       cacti_b200_dptr param_out, cacti_b200_dptr grad, int64_t n, int grad_dtype,
                                       int param_dtype, float grad_unscale, float lr, float wd, float a1, float a2,
                                       float eps, int iter_nr, cacti_b200_stream stream) {
  using namespace cb;
  if (n < 0 || iter_nr <= 0) return CACTI_B200_ERR_INVALID_VALUE;        // the reference panics on iter_nr <= 0
  if (n == 0) return CACTI_B200_OK;
  if (!master || !grad1_avg || !grad2_avg || !grad) return CACTI_B200_ERR_INVALID_VALUE;
  if ((master | grad1_avg | grad2_avg) & 3) return CACTI_B200_ERR_INVALID_VALUE;
  // src/op.rs:985-1012, in f32
  const float unbias1 = iter_nr == 1 ? a1 : 1.0f - powi_f32(1.0f - a1, iter_nr);
  const float unbias2 = iter_nr == 1 ? sqrtf(a2) : sqrtf(1.0f - powi_f32(1.0f - a2, iter_nr));
  AdamwScalars c{grad_unscale, a1, a2, -lr, unbias2 / unbias1, wd, eps * unbias2};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t grid = (n / 8 + 255) / 256 + 1;
  if (grid > (int64_t)kNumSMs * 8) grid = (int64_t)kNumSMs * 8;
  const int vec_ok = aligned16(master) && aligned16(grad1_avg) && aligned16(grad2_avg) && aligned16(grad) &&
                     (!param_out || aligned16(param_out));
  float* W = reinterpret_cast<float*>(master); float* M = reinterpret_cast<float*>(grad1_avg);
  float* V = reinterpret_cast<float*>(grad2_avg);
  return dispatch_dtype(grad_dtype, [&](auto gtag) -> int {
    using TG = decltype(gtag);
    const TG* G = reinterpret_cast<const TG*>(grad);
    if (!param_out) {
      adamw32_kernel<TG, __half><<<(unsigned)grid, 256, 0, st>>>(W, M, V, nullptr, G, n, c, vec_ok);
      return check_launch();
    }
    return dispatch_dtype(param_dtype, [&](auto ptag) -> int {
      using TP = decltype(ptag);
      adamw32_kernel<TG, TP><<<(unsigned)grid, 256, 0, st>>>(W, M, V, reinterpret_cast<TP*>(param_out), G, n, c, vec_ok);
      return check_launch();
    });
  });
}
