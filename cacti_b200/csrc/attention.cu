// Fused causal attention on the 5th-generation tensor cores, and the head-dimension padding that feeds it.
//
// The reference runs attention as separate thunks: block_matmul_scale (Q K^T), cast, block_causal_attention_mask,
// inner_softmax, lossy_cast, block_matmul (P V) (src/librarium/llama.rs:501-507), each a full pass over the
// [B, S, H, S] score tensor in HBM (268 MB per sequence at S = 2048, H = 32).  Here one kernel per 128 query rows
// keeps the scores in tensor memory and the probabilities in shared memory; HBM sees Q, K, V, the context rows and
// two floats of row statistics.
//
// Arithmetic follows the reference chain where it rounds: scores are alpha * (q . k) accumulated in f32 and rounded
// to the 16-bit type (block_matmul_scale's output), the softmax runs in f32 on those rounded scores with the row
// maximum subtracted (inner_softmax, src/thunk/op.rs:3257-3383).  It departs from it in one place: the unnormalised
// exp(s - m) is what gets rounded to 16 bits and multiplied with V, and the division by the row sum is applied to the
// f32 context row (the reference rounds exp(s - m) / sum and multiplies that).  Both roundings are relative 2^-11 per
// probability, so the context differs from the unfused chain by rounding noise only (tests bound it at the fp16
// tolerance of the block matmul).
//
// Kernel layout (one CTA = 128 query rows of one (batch, head); 192 threads):
//   warp 0      TMA producer: Q once, then K tiles (pass 1), then K and V tiles (pass 2) through two-slot rings
//   warp 1      allocates tensor memory, issues tcgen05.mma: S = Q K^T (128 x 128 x hd_pad) into one of two S
//               buffers; in pass 2 also O += P V
//   warps 2..5  one thread per query row (TMEM lane = row): pass 1 reads S and keeps the row maximum; pass 2 reads S
//               again, forms exp(s - m), sums it, writes the 16-bit probabilities into shared memory in the
//               128-byte-swizzled K-major layout the MMA reads; at the end scales O by 1 / sum and stores the row
// Two passes (max first, then exp / sum / P V) instead of an online softmax: no rescaling of O in tensor memory, and
// the row maximum is the true one as in the reference; the price is computing S twice (K = hd_pad, cheap).
// Every wait is bounded (kDevErrAttnTimeout); no load uses cluster multicast.
#include "tc_common.cuh"
#include <type_traits>

namespace cb {

constexpr unsigned kDevErrAttnTimeout = 3u;
constexpr int kAttnRows = 128;      // query rows per CTA = keys per tile
constexpr int kAttnHd = 128;        // padded head dimension
constexpr int kAttnThreads = 192;

struct AttnParams {
  int batch, seq, heads, head_dim;
  float alpha;
  uint32_t idesc_s, idesc_pv;
};

// Q / K tiles: [128 rows][128 hd] as two 128-byte-swizzled boxes of 64 columns (16 KB each).
// V tile as the MN-major B operand of P V: [128 keys][128 hd] as four boxes {64 hd, 64 keys} (8 KB each), ordered
// [key half][hd half].
constexpr uint32_t kTileBytes = kAttnRows * kAttnHd * 2;      // 32 KB

__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int k16) {       // k16: 16-element step along hd / keys
  return make_desc(base + (uint32_t)(k16 >> 2) * 16384u + (uint32_t)(k16 & 3) * 32u, 1, 64);
}
__device__ __forceinline__ uint64_t v_desc(uint32_t base, int k16) {            // k16: 16-key step
  return make_desc(base + (uint32_t)(k16 >> 2) * 16384u + (uint32_t)(k16 & 3) * 2048u, 512, 64);
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, T* __restrict__ ctx, float* __restrict__ stats,
                     const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = base;                        // 32 KB
  unsigned char* sK = sQ + kTileBytes;             // 2 x 32 KB
  unsigned char* sV = sK + 2 * kTileBytes;         // 2 x 32 KB
  unsigned char* sP = sV + 2 * kTileBytes;         // 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kTileBytes);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // 2
  uint64_t* k_empty = bars + 3;                    // 2
  uint64_t* v_full = bars + 5;                     // 2
  uint64_t* v_empty = bars + 7;                    // 2
  uint64_t* s_full = bars + 9;                     // 2
  uint64_t* s_empty = bars + 11;                   // 2
  uint64_t* p_full = bars + 13;                    // 1
  uint64_t* p_empty = bars + 14;                   // 1
  uint64_t* o_full = bars + 15;                    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // heaviest query tiles (most key tiles under the diagonal) are launched first
  const int nq = p.seq / kAttnRows, bh_count = p.batch * p.heads;
  const int qi = nq - 1 - (int)(blockIdx.x / bh_count);
  const int bh = (int)(blockIdx.x % bh_count);
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int ntiles = qi + 1;                       // key tiles 0 .. qi
  const int q0 = qi * kAttnRows;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1); mbar_init(s_empty + s, 4);
    }
    mbar_init(p_full, 4); mbar_init(p_empty, 1); mbar_init(o_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128u};
  const uint32_t tO = tmem_base + 256u;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    mbar_expect_tx(q_full, kTileBytes);
    tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
    tma_load_4d(sQ + 16384, &tmQ, q_full, 64, q0, h, b);
    int n = 0;                                     // K tiles issued so far (both passes)
    for (int pass = 0; pass < 2; ++pass) {
      for (int j = 0; j < ntiles; ++j, ++n) {
        const int ks = n & 1;
        if (!mbar_wait_bounded(k_empty + ks, (unsigned)((n >> 1) & 1) ^ 1, kDevErrAttnTimeout)) goto done;
        unsigned char* dk = sK + (size_t)ks * kTileBytes;
        mbar_expect_tx(k_full + ks, kTileBytes);
        tma_load_4d(dk, &tmK, k_full + ks, 0, j * kAttnRows, h, b);
        tma_load_4d(dk + 16384, &tmK, k_full + ks, 64, j * kAttnRows, h, b);
        if (pass == 1) {
          const int vs = j & 1;
          if (!mbar_wait_bounded(v_empty + vs, (unsigned)((j >> 1) & 1) ^ 1, kDevErrAttnTimeout)) goto done;
          unsigned char* dv = sV + (size_t)vs * kTileBytes;
          mbar_expect_tx(v_full + vs, kTileBytes);
#pragma unroll
          for (int kh = 0; kh < 2; ++kh)
#pragma unroll
            for (int nh = 0; nh < 2; ++nh)
              tma_load_4d(dv + kh * 16384 + nh * 8192, &tmV, v_full + vs, nh * 64, j * kAttnRows + kh * 64, h, b);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    if (!mbar_wait_bounded(q_full, 0, kDevErrAttnTimeout)) goto done;
    const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
    auto issue_s = [&](int n) -> bool {             // S[n & 1] = Q K_n^T
      const int ks = n & 1;
      const unsigned ph = (unsigned)((n >> 1) & 1);
      if (!mbar_wait_bounded(k_full + ks, ph, kDevErrAttnTimeout)) return false;
      if (!mbar_wait_bounded(s_empty + ks, ph ^ 1, kDevErrAttnTimeout)) return false;
      tc_fence_after();
      const uint32_t aK = smem_u32(sK + (size_t)ks * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
        tc_mma_f16(tS[ks], kmajor_desc(aQ, k16), kmajor_desc(aK, k16), p.idesc_s, k16 ? 1u : 0u);
      tc_commit(k_empty + ks);
      tc_commit(s_full + ks);
      return true;
    };
    int n = 0;
    for (int j = 0; j < ntiles; ++j, ++n)           // pass 1: scores only
      if (!issue_s(n)) goto done;
    if (!issue_s(n)) goto done;                     // first S of pass 2
    ++n;
    for (int j = 0; j < ntiles; ++j) {
      if (j + 1 < ntiles) { if (!issue_s(n)) goto done; ++n; }      // S of the next tile overlaps this tile's softmax
      const int vs = j & 1;
      if (!mbar_wait_bounded(v_full + vs, (unsigned)((j >> 1) & 1), kDevErrAttnTimeout)) goto done;
      if (!mbar_wait_bounded(p_full, (unsigned)(j & 1), kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      const uint32_t aV = smem_u32(sV + (size_t)vs * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnRows / 16; ++k16)
        tc_mma_f16(tO, kmajor_desc(aP, k16), v_desc(aV, k16), p.idesc_pv, (j | k16) ? 1u : 0u);
      tc_commit(v_empty + vs);
      tc_commit(p_empty);
    }
    tc_commit(o_full);
  } else if (warp >= 2) {
    // ---------------- softmax warps: thread = query row ----------------
    const int qq = warp & 3;                        // TMEM lane quarter
    const int r = qq * 32 + lane;                   // row inside the tile
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    float m = -INFINITY;
    int n = 0;
    for (int j = 0; j < ntiles; ++j, ++n) {         // pass 1: row maximum of the rounded, scaled, masked scores
      const int sb = n & 1;
      if (!mbar_wait_bounded(s_full + sb, (unsigned)((n >> 1) & 1), kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      const int lim = (j == qi) ? r : kAttnRows;    // columns <= lim are unmasked (diagonal tile: c <= r)
#pragma unroll 1
      for (int c0 = 0; c0 < kAttnRows; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tS[sb] + lane_off + (uint32_t)c0, v);
        tc_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = Elem<T>::to_f32(Elem<T>::from_f32(p.alpha * __uint_as_float(v[i])));
          if (c0 + i <= lim) m = fmaxf(m, s);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + sb);
    }
    float l = 0.f;
    const float mb = m * kLog2e;
    for (int j = 0; j < ntiles; ++j, ++n) {         // pass 2: exp, row sum, probabilities to shared memory
      const int sb = n & 1;
      if (!mbar_wait_bounded(s_full + sb, (unsigned)((n >> 1) & 1), kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      // the previous tile's P V has read the probability buffer
      if (!mbar_wait_bounded(p_empty, (unsigned)(j & 1) ^ 1, kDevErrAttnTimeout)) goto done;
      const int lim = (j == qi) ? r : kAttnRows;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttnRows; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tS[sb] + lane_off + (uint32_t)c0, v);
        tc_ld_wait();
        unsigned char* prow = sP + (size_t)(c0 >> 6) * 16384 + (size_t)r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float e8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float s = Elem<T>::to_f32(Elem<T>::from_f32(p.alpha * __uint_as_float(v[g * 8 + i])));
            const float e = (c0 + g * 8 + i <= lim) ? exp2f_approx(__fmaf_rn(s, kLog2e, -mb)) : 0.f;
            l += e;
            e8[i] = e;
          }
          const int chunk = ((c0 & 63) >> 3) + g;   // 16-byte chunk inside the 128-byte row of this key half
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = pack<T>(e8);
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) { mbar_arrive(s_empty + sb); mbar_arrive(p_full); }
    }
    // context row = O / l
    if (!mbar_wait_bounded(o_full, 0, kDevErrAttnTimeout)) goto done;
    tc_fence_after();
    const float rl = 1.f / l;
    const long long row = (long long)b * p.seq + q0 + r;
    T* out = ctx + (row * p.heads + h) * p.head_dim;
    float* st = stats + (((long long)b * p.heads + h) * p.seq + q0 + r) * 2;
    st[0] = m; st[1] = l;
#pragma unroll 1
    for (int c0 = 0; c0 < p.head_dim; c0 += 32) {
      uint32_t v[32];
      tc_ld32(tO + lane_off + (uint32_t)c0, v);
      tc_ld_wait();
#pragma unroll
      for (int g = 0; g < 8; ++g) {                 // 4 elements = 8 bytes per store (rows start 8-byte aligned when hd % 4 == 0)
        const int c = c0 + g * 4;
        if (c + 4 <= p.head_dim) {
          float f4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) f4[i] = __uint_as_float(v[g * 4 + i]) * rl;
          uint2 w;
          if constexpr (std::is_same<T, __half>::value) {
            __half2 a = __floats2half2_rn(f4[0], f4[1]), bb = __floats2half2_rn(f4[2], f4[3]);
            w.x = *reinterpret_cast<uint32_t*>(&a); w.y = *reinterpret_cast<uint32_t*>(&bb);
          } else {
            __nv_bfloat162 a = __floats2bfloat162_rn(f4[0], f4[1]), bb = __floats2bfloat162_rn(f4[2], f4[3]);
            w.x = *reinterpret_cast<uint32_t*>(&a); w.y = *reinterpret_cast<uint32_t*>(&bb);
          }
          *reinterpret_cast<uint2*>(out + c) = w;
        }
      }
    }
    tc_fence_before();
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// Zero-pad the inner dimension of a block tensor [nrow, rows, ncol, cols] to cols_pad (BlockPadFutThunkSpec,
// src/thunk/op.rs:4065-4186, which the reference stages before every block matmul whose blocks are not 16-byte
// multiples, src/op.rs:1454-1482).  One thread per 8-byte unit of the destination when cols % 4 == 0, else per element.
template <typename U, int EPU /* elements per unit */>
__global__ void __launch_bounds__(256)
block_pad_kernel(U* __restrict__ dst, const U* __restrict__ src, long long groups /* nrow*rows*ncol */, int cols_u,
                 int cols_pad_u) {
  const long long total = groups * cols_pad_u;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long gidx = i / cols_pad_u;
    const int c = (int)(i - gidx * cols_pad_u);
    U v{};
    if (c < cols_u) v = src[gidx * cols_u + c];
    dst[i] = v;
  }
}

static int encode_bshd(CUtensorMap* map, uint64_t ptr, int batch, int seq, int heads, int hdp, int box_inner, int box_rows,
                       bool bf16) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CACTI_B200_ERR_LAUNCH;
  cuuint64_t dims[4] = {(cuuint64_t)hdp, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)heads * hdp * 2, (cuuint64_t)hdp * 2, (cuuint64_t)seq * heads * hdp * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  reinterpret_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return CACTI_B200_ERR_LAUNCH; }
  return CACTI_B200_OK;
}

constexpr size_t kAttnFwdSmem = 1024 + 6 * (size_t)kTileBytes + 256;

template <typename T>
static int attention_fwd_run(uint64_t ctx, uint64_t stats, uint64_t q, uint64_t k, uint64_t v, int batch, int seq, int heads,
                             int head_dim, float alpha, cudaStream_t st) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  CUtensorMap tmQ, tmK, tmV;
  int rc = encode_bshd(&tmQ, q, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmK, k, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmV, v, batch, seq, heads, kAttnHd, 64, 64, bf16);
  if (rc) return rc;
  AttnParams p;
  p.batch = batch; p.seq = seq; p.heads = heads; p.head_dim = head_dim; p.alpha = alpha;
  const uint32_t common = (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(128 >> 3) << 17) |
                          ((uint32_t)(128 >> 4) << 24);
  p.idesc_s = common;                       // A, B K-major
  p.idesc_pv = common | (1u << 16);         // B (V) MN-major
  auto kern = attention_fwd_kernel<T>;
  static bool attr_set = false;
  if (!attr_set) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnFwdSmem); attr_set = true; }
  const long long grid = (long long)batch * heads * (seq / kAttnRows);
  kern<<<(unsigned)grid, kAttnThreads, kAttnFwdSmem, st>>>(tmQ, tmK, tmV, reinterpret_cast<T*>(ctx),
                                                           reinterpret_cast<float*>(stats), p);
  return check_launch();
}

}  // namespace cb

extern "C" {

int cacti_b200_block_pad(cacti_b200_dptr dst, cacti_b200_dptr src, int64_t nrow, int64_t rows, int64_t ncol, int64_t cols,
                         int64_t cols_pad, int dtype, cacti_b200_stream stream) {
  using namespace cb;
  if (nrow < 0 || rows < 0 || ncol < 0 || cols < 0 || cols_pad < cols) return CACTI_B200_ERR_INVALID_VALUE;
  if (dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  const long long groups = nrow * rows * ncol;
  if (groups == 0 || cols_pad == 0) return CACTI_B200_OK;
  if (!dst || (!src && cols > 0)) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool wide = (cols % 4 == 0) && (cols_pad % 4 == 0) && (dst % 8 == 0) && (src % 8 == 0);
  const long long total = groups * (wide ? cols_pad / 4 : cols_pad);
  long long grid = (total + 255) / 256;
  if (grid > (long long)kNumSMs * 32) grid = (long long)kNumSMs * 32;
  if (wide)
    block_pad_kernel<uint2, 4><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<uint2*>(dst), reinterpret_cast<const uint2*>(src),
                                                                groups, (int)(cols / 4), (int)(cols_pad / 4));
  else
    block_pad_kernel<uint16_t, 1><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<uint16_t*>(dst),
                                                                   reinterpret_cast<const uint16_t*>(src), groups, (int)cols,
                                                                   (int)cols_pad);
  return check_launch();
}

int cacti_b200_attention_fwd(cacti_b200_dptr ctx, cacti_b200_dptr stats, cacti_b200_dptr q, cacti_b200_dptr k,
                             cacti_b200_dptr v, int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, float alpha,
                             int dtype, cacti_b200_stream stream) {
  using namespace cb;
  if (batch < 0 || seq < 0 || heads < 0 || head_dim <= 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (head_dim > kAttnHd || head_dim % 4 || seq % kAttnRows || batch * heads * (seq / kAttnRows) > 0x7fffffffLL)
    return CACTI_B200_ERR_SHAPE;
  if (batch == 0 || seq == 0 || heads == 0) return CACTI_B200_OK;
  if (!ctx || !stats || !q || !k || !v || (q & 15) || (k & 15) || (v & 15) || (ctx & 7) || (stats & 7))
    return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == CACTI_B200_R_16F)
    return attention_fwd_run<__half>(ctx, stats, q, k, v, (int)batch, (int)seq, (int)heads, (int)head_dim, alpha, st);
  return attention_fwd_run<__nv_bfloat16>(ctx, stats, q, k, v, (int)batch, (int)seq, (int)heads, (int)head_dim, alpha, st);
}
}
