// Shared device/host helpers for the sm_100a thunk kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/cacti_b200.h"

namespace cb {

constexpr int kNumSMs = 148;          // B200: 2 dies x 74 SMs; grids are sized in multiples of this

extern thread_local int g_last_cuda_error;

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return CACTI_B200_ERR_LAUNCH; }
  return CACTI_B200_OK;
}

inline bool aligned16(uint64_t p) { return (p & 15u) == 0; }

// Ordinal of the current device, for caches of per-device state (function attributes, occupancy, symbol addresses).
constexpr int kMaxDevices = 64;
inline int device_ordinal() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) d = 0;
  return d;
}
// Raise a kernel's dynamic shared memory limit once per device (the attribute belongs to the device's copy of the
// function: a process that drives a second device must set it there too).
template <typename K> inline void ensure_dynamic_smem(K kern, size_t smem, bool (&done)[kMaxDevices]) {
  const int d = device_ordinal();
  if (!done[d]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    done[d] = true;
  }
}

// Programmatic dependent launch, for a short second kernel that consumes what the kernel before it in the stream
// wrote (a partial-sum fold): launched this way, its launch and block scheduling overlap the tail of the previous
// kernel instead of following its completion.  The kernel launched with launch_dependent() must execute
// dependent_wait() before it reads anything the previous kernel wrote (the wait returns once that kernel has
// completed and its writes are visible); the previous kernel may call dependents_may_launch() once a CTA has
// nothing long left to do, otherwise the hand-over happens as its CTAs exit.
__device__ __forceinline__ void dependent_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kern)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(block); cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- element traits ------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int VEC = 4;                   // elements per 16-byte vector
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__half> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// Packed pair of a 16-bit type (float has none: code that uses it sits behind `if constexpr`).
template <typename T> struct Pair16 { using type = float2; static __device__ __forceinline__ float2 neg_inf() { return make_float2(0.f, 0.f); } };
template <> struct Pair16<__half> {
  using type = __half2;
  static __device__ __forceinline__ __half2 neg_inf() { return __half2half2(__ushort_as_half((unsigned short)0xfc00)); }
};
template <> struct Pair16<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ __nv_bfloat162 neg_inf() { return __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)0xff80)); }
};

// Round an f32 value to T and back: the rounding point of a primitive thunk whose output cell is T.
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return Elem<T>::to_f32(Elem<T>::from_f32(v));
}

// ---- 16-byte vectors -------------------------------------------------------------------
// Streaming loads/stores: every activation is touched once, so bypass L1 allocation and mark
// the lines evict-first in L2.
__device__ __forceinline__ uint4 ld_stream(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream(void* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }
__device__ __forceinline__ uint4 ld_keep(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

template <typename T> __device__ __forceinline__ void unpack(const uint4& v, float (&f)[Elem<T>::VEC]);
template <> __device__ __forceinline__ void unpack<float>(const uint4& v, float (&f)[4]) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__half>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {      // bf16 -> f32 is a 16-bit shift
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T> __device__ __forceinline__ uint4 pack(const float (&f)[Elem<T>::VEC]);
template <> __device__ __forceinline__ uint4 pack<float>(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack<__half>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// out = T(f32(old) + f32(T(v))): Accumulate mode adds in the output dtype after the new value
// has itself been rounded to that dtype.
template <typename T>
__device__ __forceinline__ uint4 pack_accumulate(const float (&f)[Elem<T>::VEC], const uint4& old) {
  float o[Elem<T>::VEC], r[Elem<T>::VEC];
  unpack<T>(old, o);
#pragma unroll
  for (int i = 0; i < Elem<T>::VEC; ++i) r[i] = o[i] + round_to<T>(f[i]);
  return pack<T>(r);
}

// ---- row groups --------------------------------------------------------------------------
// A row is processed by a group of G threads (G a multiple of 32).  G == 32: the group is a warp
// and reductions are shuffles only.  G > 32: warps exchange through shared memory and meet on a
// named barrier that belongs to the group, so several groups share one CTA without blocking
// each other.  All threads of the group get the same, order-fixed result.
constexpr int kMaxGroupsPerCta = 15;             // named barriers 1..15 (0 is __syncthreads)
constexpr int kMaxWarpsPerGroup = 32;

struct GroupCtx {
  int G;            // threads per group
  int gid;          // group index inside the CTA
  int lane;         // thread index inside the group
  int nwarps;       // warps per group
  int phase;        // alternates the shared slot so one barrier per reduction is enough
  float* red;       // shared: [2][groups][kMaxWarpsPerGroup][2]
};

__device__ __forceinline__ void group_barrier(const GroupCtx& g) {
  if (g.G == 32) __syncwarp();
  else asm volatile("bar.sync %0, %1;" ::"r"(g.gid + 1), "r"(g.G) : "memory");
}

__device__ __forceinline__ size_t group_red_floats(int groups) { return (size_t)2 * groups * kMaxWarpsPerGroup * 2; }

__device__ __forceinline__ GroupCtx make_group(int G, float* red_smem) {
  GroupCtx g;
  g.G = G; g.gid = threadIdx.x / G; g.lane = threadIdx.x % G; g.nwarps = G >> 5; g.phase = 0; g.red = red_smem;
  return g;
}

// Group barrier that also ORs a per-thread flag over the group: every thread gets the same answer.  Used to turn a
// per-thread event (a bounded wait that ran out) into a decision the whole group takes together, at a barrier the
// group meets anyway: threads that left on their own would leave the others waiting at the next barrier for ever.
__device__ __forceinline__ bool group_any(const GroupCtx& g, bool flag) {
  if (g.G == 32) return __any_sync(0xffffffffu, flag);
  unsigned r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"(g.gid + 1), "r"(g.G), "r"((unsigned)flag) : "memory");
  return r != 0;
}

struct SumOp { static __device__ __forceinline__ float f(float a, float b) { return a + b; } static __device__ __forceinline__ float id() { return 0.f; } };
struct MaxOp { static __device__ __forceinline__ float f(float a, float b) { return fmaxf(a, b); } static __device__ __forceinline__ float id() { return -INFINITY; } };

template <typename Op> __device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::f(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduce two values at once (a and b use the same Op).  Stage 1: shuffles inside each warp; lane 0
// of every warp publishes its pair; stage 2 after the group barrier: lane l of every warp picks up
// warp l's pair and the warp reduces again with shuffles (a group has at most 32 warps).
// `any` (optional): in: this thread's flag; out: the OR over the group, taken at the reduction's own barrier.
template <typename Op> __device__ __forceinline__ void group_reduce2(GroupCtx& g, float& a, float& b, bool* any = nullptr) {
  a = warp_reduce<Op>(a);
  b = warp_reduce<Op>(b);
  if (g.G == 32) {
    if (any) *any = __any_sync(0xffffffffu, *any);
    return;
  }
  const int groups = blockDim.x / g.G;
  float2* slot = reinterpret_cast<float2*>(g.red) + (size_t)(g.phase * groups + g.gid) * kMaxWarpsPerGroup;
  const int w = g.lane >> 5, l = g.lane & 31;
  if (l == 0) slot[w] = make_float2(a, b);
  if (any) *any = group_any(g, *any);
  else group_barrier(g);
  float2 v = l < g.nwarps ? slot[l] : make_float2(Op::id(), Op::id());
  a = warp_reduce<Op>(v.x);
  b = warp_reduce<Op>(v.y);
  g.phase ^= 1;
}
template <typename Op> __device__ __forceinline__ float group_reduce(GroupCtx& g, float a) {
  float b = Op::id();
  group_reduce2<Op>(g, a, b);
  return a;
}

// ---- row staging: bulk async copies (TMA, untiled) into shared memory, completed on an mbarrier ----
// Each row group owns one stage buffer and one mbarrier.  The group's first lane arms the barrier
// with the byte count and issues cp.async.bulk for the row(s); every lane then waits on the phase
// bit.  After the group has moved the row from shared memory into registers it meets on its barrier
// and the next row's copy is issued into the same buffer, so a row is always in flight while the
// previous one is being reduced.  Sources and sizes must be multiples of 16 bytes.
// Every wait is bounded: if a copy never completes the kernel records kDevErrStageTimeout in
// g_dev_error and the group stops; it never spins forever.
constexpr unsigned kDevErrStageTimeout = 1u;
constexpr unsigned kDevErrGemmTimeout = 2u;
extern __device__ unsigned g_dev_error;
constexpr unsigned g_mbar_suspend_ns = 4000u;      // per-poll suspend hint of mbar_try_wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the thread for up to that long while the phase is
// incomplete (it resumes at once when the phase completes), so that waiting warps do not take issue slots from the
// warps that compute on the same scheduler.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(g_mbar_suspend_ns) : "memory");
  return ok != 0;
}
// One look, no parking: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Returns false after `polls` failed polls (default 2^20: at most about 4 s, every poll parked for the full hint; at
// least a few tens of milliseconds, polls that return at once; far beyond any wait of a healthy kernel).  The answer
// is per thread: a caller that shares barriers or warp-wide instructions with other threads must agree on it with
// them (group_any, __all_sync) before acting on it.
constexpr unsigned kMbarPolls = 1u << 20;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, unsigned err_code, unsigned polls = kMbarPolls) {
  for (unsigned it = 0; it < polls; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  atomicMax(&g_dev_error, err_code);
  return false;
}
// The same for a converged warp: true only if every lane saw the phase complete.
__device__ __forceinline__ bool mbar_wait_bounded_warp(uint64_t* bar, unsigned parity, unsigned err_code) {
  return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, err_code));
}
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Bulk store shared -> global (16-byte aligned addresses and size), joined to the thread's current bulk group.
// Shared memory written by ordinary stores needs fence.proxy.async before the copy engine reads it.
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(dst_gmem), "r"(smem_u32(src_smem)), "r"(bytes) : "memory");
}

// ---- block reduction for the element-wise fallback kernels (whole CTA = one row) -----------
// `any` (optional): in: this thread's flag; out: the OR over the CTA, taken at the reduction's first barrier.
template <typename Op> __device__ __forceinline__ float block_reduce(float v, float* smem /* >= 33 floats */, bool* any = nullptr) {
  v = warp_reduce<Op>(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (any) *any = __syncthreads_or(*any) != 0;
  else __syncthreads();                  // protect smem from the previous use
  if ((threadIdx.x & 31) == 0) smem[w] = v;
  __syncthreads();
  float r = Op::id();
  for (int i = 0; i < nw; ++i) r = Op::f(r, smem[i]);
  return r;
}

// exp in f32.  16-bit storage: ex2.approx (relative error ~1e-6, far below the storage
// rounding).  f32 storage: the accurate library exp, so fp32 results stay within 1e-5 relative.
__device__ __forceinline__ float exp2f_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T> __device__ __forceinline__ float exp_for(float x) { return __expf(x); }
template <> __device__ __forceinline__ float exp_for<float>(float x) { return expf(x); }

// exp(a - m) as one FFMA and one MUFU: ex2(a*log2e - m*log2e), neg_m_log2e = -m * log2e formed once per row.  Used for
// 16-bit storage, where its ~1e-6 relative error is far below the storage rounding; f32 storage uses the accurate
// expf.  (__expf without flush-to-zero costs a compare and two predicated multiplies around the MUFU for the
// subnormal range, which a result that is rounded to 16 bits never shows.)
template <typename T> __device__ __forceinline__ float exp_shifted(float a, float m, float neg_m_log2e) {
  if constexpr (std::is_same<T, float>::value) return expf(a - m);
  else return exp2f_approx(__fmaf_rn(a, 1.4426950408889634f, neg_m_log2e));
}

template <typename F> inline int dispatch_dtype(int dtype, F&& f) {
  switch (dtype) {
    case CACTI_B200_R_32F:  return f(float{});
    case CACTI_B200_R_16F:  return f(__half{});
    case CACTI_B200_R_16BF: return f(__nv_bfloat16{});
    default: return CACTI_B200_ERR_DTYPE;
  }
}

// Pick (threads per row group, 16-byte vectors per thread) for a row of `nvec` vectors.
// Rows of up to 32*nv_max vectors go to one warp (shuffle-only reductions, several rows per CTA).
// Longer rows go to a multi-warp group: the fewest vectors per thread that keeps the group at
// or below g_pref threads, else nv_max vectors per thread and up to 512 threads.
constexpr size_t kMaxDynSmem = 200 * 1024;      // of the 227 KB a CTA may use

// CTAs of `kern` that fit on one SM with this block size and dynamic shared memory; also raises the
// kernel's dynamic shared memory limit when needed (never lowers it).  Cached per (kernel, config).
template <typename K> inline int resident_ctas(K kern, int threads, size_t smem) {
  struct Key { const void* k; int dev; int t; size_t s; int n; };
  struct Lim { const void* k; int dev; size_t s; };
  static thread_local Key cache[128];
  static thread_local Lim lim[128];
  static thread_local int used = 0, nlim = 0;
  const void* kp = reinterpret_cast<const void*>(kern);
  const int dev = device_ordinal();
  if (smem > 48 * 1024) {
    int i = 0;
    for (; i < nlim; ++i) if (lim[i].k == kp && lim[i].dev == dev) break;
    if (i == nlim && nlim < 128) lim[nlim++] = Lim{kp, dev, 0};
    if (i >= 128 || lim[i].s < smem) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (i < 128) lim[i].s = smem;
    }
  }
  for (int i = 0; i < used; ++i)
    if (cache[i].k == kp && cache[i].dev == dev && cache[i].t == threads && cache[i].s == smem) return cache[i].n;
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem) != cudaSuccess || n < 1) n = 1;
  if (used < 128) cache[used++] = Key{kp, dev, threads, smem, n};
  return n;
}

struct GroupPlan { int G; int NV; int groups; bool ok; };
inline GroupPlan plan_group(int64_t nvec, int nv_max, int g_pref, int target_threads) {
  GroupPlan p{32, 1, 1, false};
  if (nvec <= 0) return p;
  for (int nv = 1; nv <= nv_max; nv *= 2) {
    if (nvec <= 32LL * nv) {
      p.G = 32; p.NV = nv; p.groups = target_threads / 32; if (p.groups < 1) p.groups = 1; p.ok = true;
      return p;
    }
  }
  for (int nv = 1; nv <= nv_max; nv *= 2) {
    int64_t g = ((nvec + nv - 1) / nv + 31) / 32 * 32;
    const int64_t cap = (nv == nv_max) ? 512 : g_pref;
    if (g <= cap) {
      p.G = (int)g; p.NV = nv;
      p.groups = target_threads / p.G; if (p.groups < 1) p.groups = 1;
      if (p.groups > kMaxGroupsPerCta) p.groups = kMaxGroupsPerCta;
      p.ok = true;
      return p;
    }
  }
  return p;
}

}  // namespace cb
