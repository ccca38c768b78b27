// Library-level entry points: version, error strings, tuning knobs.
#include "common.cuh"
#include <string.h>

namespace cb {
thread_local int g_last_cuda_error = 0;
__device__ unsigned g_dev_error = 0;
extern int g_softmax_threads, g_softmax_waves;
extern int g_rmsnorm_threads, g_rmsnorm_gpref, g_rmsnorm_smem_kb, g_rmsnorm_bulk_out;
extern int g_nll_gpref, g_nll_stages, g_nll_mode, g_nll_smem_threads;
extern int g_rope_threads, g_rope_ctas_per_sm, g_rope_staged, g_rope_staged_g, g_rope_staged_groups, g_rope_staged_stages;
extern int g_swiglu_threads, g_swiglu_ctas_per_sm;
extern int g_gemm_bn, g_gemm_group_m, g_gemm_sms, g_gemm_pair, g_gemm_split, g_gemm_dynamic;
extern int g_attn_fwd_single, g_attn_fwd_persistent, g_attn_fwd_pair;
}  // namespace cb

extern "C" {

int cacti_b200_version(void) { return 100; }   // 0.1.0

const char* cacti_b200_error_string(int code) {
  switch (code) {
    case CACTI_B200_OK: return "ok";
    case CACTI_B200_ERR_INVALID_VALUE: return "invalid value";
    case CACTI_B200_ERR_DTYPE: return "unsupported dtype";
    case CACTI_B200_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case CACTI_B200_ERR_LAUNCH: return "CUDA launch failed";
    case CACTI_B200_ERR_SHAPE: return "unsupported shape";
    case CACTI_B200_ERR_INDEX_RANGE: return "index out of range in device data";
    case CACTI_B200_ERR_NO_DEVICE: return "no sm_100 device";
    case CACTI_B200_ERR_SCRATCH_LIMIT: return "shape exceeds the scratch array built into this no-allocation entry point";
    default: return "unknown error";
  }
}

int cacti_b200_last_cuda_error(void) { return cb::g_last_cuda_error; }

namespace cb {
// Self-test of the time-out path every staged or pipelined kernel relies on: a CTA (two row groups of 64 threads, one
// of them also holding tensor memory) waits, with a short poll limit, on an mbarrier that nothing ever arms.  Every
// thread's wait runs out; the groups agree on it at their barrier (group_any) and leave together, the tensor memory
// is released, and the device error word holds kDevErrSelfTest.  No access faults and nothing spins without a limit.
constexpr unsigned kDevErrSelfTest = 5u;
__global__ void __launch_bounds__(128) bounded_wait_selftest_kernel(unsigned polls, unsigned* __restrict__ out) {
  __shared__ uint64_t bars[2];
  __shared__ uint32_t tmem_slot;
  GroupCtx g = make_group(64, nullptr);
  if (g.lane == 0) mbar_init(bars + g.gid, 1);
  mbar_fence_init();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;
  // lanes give up after different numbers of polls, as they would when a slow copy lands between two lanes' last polls
  const bool gave_up = !mbar_wait_bounded(bars + g.gid, 0, kDevErrSelfTest, polls + (threadIdx.x & 7));
  const bool all_leave = group_any(g, gave_up);
  if (g.lane == 0) out[1 + g.gid] = all_leave ? 1u : 0u;
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32) : "memory");
  }
  if (threadIdx.x == 0) out[0] = 1u;          // the kernel reached its end
}
}  // namespace cb

int cacti_b200_selftest_bounded_wait(cacti_b200_dptr result, int polls, cacti_b200_stream stream) {
  if (!result || (result & 3) || polls < 1 || polls > 4096) return CACTI_B200_ERR_INVALID_VALUE;
  cb::bounded_wait_selftest_kernel<<<1, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>((unsigned)polls,
                                                                                         reinterpret_cast<unsigned*>(result));
  return cb::check_launch();
}

// Reads (and clears) the sticky device-side error word: 0 = none, 1 = a staged row copy never completed,
// 2 = a GEMM pipeline wait ran out, 3 = an attention pipeline wait ran out,
// 4 = a k-split GEMM never received another CTA's partial sum.  Synchronises the device.
int cacti_b200_device_error(unsigned* out) {
  if (!out) return CACTI_B200_ERR_INVALID_VALUE;
  unsigned v = 0, zero = 0;
  // every stream of the device, blocking or not: a copy from a symbol alone would not wait for non-blocking streams
  if (cudaDeviceSynchronize() != cudaSuccess) { cb::check_launch(); return CACTI_B200_ERR_LAUNCH; }
  if (cudaMemcpyFromSymbol(&v, cb::g_dev_error, sizeof(v)) != cudaSuccess) { cb::check_launch(); return CACTI_B200_ERR_LAUNCH; }
  if (v) cudaMemcpyToSymbol(cb::g_dev_error, &zero, sizeof(zero));
  *out = v;
  return CACTI_B200_OK;
}

// Launch-shape knobs for measurement sweeps; not part of the thunk contract.  Returns 0, or
// CACTI_B200_ERR_INVALID_VALUE for an unknown name or a value outside the knob's range.
int cacti_b200_tune(const char* name, int value) {
  using namespace cb;
  struct Knob { const char* name; int* p; int lo, hi; };
  const Knob knobs[] = {
      {"softmax_threads", &g_softmax_threads, 32, 512},   {"softmax_waves", &g_softmax_waves, 1, 64},
      {"rmsnorm_threads", &g_rmsnorm_threads, 32, 512},   {"rmsnorm_gpref", &g_rmsnorm_gpref, 32, 512},
      {"rmsnorm_smem_kb", &g_rmsnorm_smem_kb, 16, 200},    {"rmsnorm_bulk_out", &g_rmsnorm_bulk_out, 0, 1},
      {"nll_gpref", &g_nll_gpref, 32, 512},               {"nll_stages", &g_nll_stages, 1, 4}, {"nll_mode", &g_nll_mode, 0, 1}, {"nll_smem_threads", &g_nll_smem_threads, 256, 384},
      {"rope_threads", &g_rope_threads, 32, 256},         {"rope_ctas_per_sm", &g_rope_ctas_per_sm, 1, 64},
      {"rope_staged", &g_rope_staged, 0, 1},              {"rope_staged_g", &g_rope_staged_g, 32, 512},
      {"rope_staged_groups", &g_rope_staged_groups, 1, 15}, {"rope_staged_stages", &g_rope_staged_stages, 2, 8},
      {"gemm_bn", &g_gemm_bn, 0, 256}, {"gemm_group_m", &g_gemm_group_m, 0, 4096}, {"gemm_sms", &g_gemm_sms, 0, 148}, {"gemm_pair", &g_gemm_pair, 0, 1}, {"gemm_split", &g_gemm_split, 0, 1}, {"gemm_dynamic", &g_gemm_dynamic, 0, 1},
      {"swiglu_threads", &g_swiglu_threads, 32, 256},     {"swiglu_ctas_per_sm", &g_swiglu_ctas_per_sm, 1, 64},
      {"attn_fwd_single", &g_attn_fwd_single, 0, 1},     {"attn_fwd_persistent", &g_attn_fwd_persistent, 0, 2}, {"attn_fwd_pair", &g_attn_fwd_pair, 0, 1},
  };
  if (!name) return CACTI_B200_ERR_INVALID_VALUE;
  for (const Knob& k : knobs) {
    if (strcmp(k.name, name) == 0) {
      if (value < k.lo || value > k.hi || (k.lo == 32 && value % 32)) return CACTI_B200_ERR_INVALID_VALUE;
      if (k.p == &g_gemm_bn && value != 0 && value != 128 && value != 192 && value != 256) return CACTI_B200_ERR_INVALID_VALUE;
      *k.p = value;
      return CACTI_B200_OK;
    }
  }
  return CACTI_B200_ERR_INVALID_VALUE;
}
}
