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
extern int g_gemm_bn, g_gemm_group_m, g_gemm_sms, g_gemm_pair;
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

// Reads (and clears) the sticky device-side error word: 0 = none, 1 = a staged row copy never completed,
// 2 = a GEMM pipeline wait ran out.  Synchronises the device.
int cacti_b200_device_error(unsigned* out) {
  if (!out) return CACTI_B200_ERR_INVALID_VALUE;
  unsigned v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, cb::g_dev_error, sizeof(v)) != cudaSuccess) return cb::check_launch() ? CACTI_B200_ERR_LAUNCH : CACTI_B200_ERR_LAUNCH;
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
      {"gemm_bn", &g_gemm_bn, 0, 256}, {"gemm_group_m", &g_gemm_group_m, 0, 4096}, {"gemm_sms", &g_gemm_sms, 0, 148}, {"gemm_pair", &g_gemm_pair, 0, 1},
      {"swiglu_threads", &g_swiglu_threads, 32, 256},     {"swiglu_ctas_per_sm", &g_swiglu_ctas_per_sm, 1, 64},
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
