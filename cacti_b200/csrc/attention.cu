// Fused causal attention on the 5th-generation tensor cores, and the head-dimension padding that feeds it.
//
// The reference runs attention as separate thunks: block_matmul_scale (Q K^T), cast, block_causal_attention_mask,
// inner_softmax, lossy_cast, block_matmul (P V) (src/librarium/llama.rs:501-507), each a full pass over the
// [B, S, H, S] score tensor in HBM (268 MB per sequence at S = 2048, H = 32).  Here one kernel per 128 query rows
// keeps the scores in tensor memory and the probabilities in shared memory; HBM sees Q, K, V, the context rows and
// the row statistics (maximum and sum; 16 bytes per row with two words of scratch for the backward pass).
//
// Arithmetic follows the reference chain where it rounds: scores are alpha * (q . k) accumulated in f32 and rounded
// to the 16-bit type (block_matmul_scale's output), the softmax runs in f32 on those rounded scores with the row
// maximum subtracted (inner_softmax, src/thunk/op.rs:3257-3383).  It departs from it in one place: the unnormalised
// exp(s - m) is what gets rounded to 16 bits and multiplied with V, and the division by the row sum is applied to the
// f32 context row (the reference rounds exp(s - m) / sum and multiplies that).  Both roundings are relative 2^-11 per
// probability, so the context differs from the unfused chain by rounding noise only (tests bound it at the fp16
// tolerance of the block matmul).
//
// Kernel layout (one CTA = 128 query rows of one (batch, head); 320 threads):
//   warp 0      TMA producer: Q once, then K tiles (pass 1), then K and V tiles (pass 2) through two-slot rings
//   warp 1      allocates tensor memory, issues tcgen05.mma: S = Q K^T (128 x 128 x hd_pad) into one of two S
//               buffers; in pass 2 also O += P V
//   warps 2..9  two softmax groups of 128 threads, one thread per query row (TMEM lane = row), group g on key tiles
//               j = g (mod 2) with its own S buffer and probability buffer: pass 1 reads S and keeps the row maximum;
//               pass 2 reads S again, forms exp(s - m), sums it, writes the 16-bit probabilities into shared memory
//               in the 128-byte-swizzled K-major layout the MMA reads; the groups' maxima and sums are combined
//               through shared memory; at the end each group scales half of O's columns by 1 / sum and stores them
// That is attention_fwd_kernel: two passes (max first, then exp / sum / P V), no rescaling of O in tensor memory, the
// price being S computed twice.  attention_fwd1_kernel forms S once: a running maximum and an O accumulator per
// softmax group, rescaled in tensor memory when the maximum has moved far (see the comment at that kernel); measured
// 560 against 620 us at [8, 2048, 32, 100].  attention_fwd1p_kernel is that kernel with one CTA per SM walking many
// (batch, query tile, head) items (short sequences with an odd number of query tiles).  attention_fwd2_kernel, the
// default wherever the number of query tiles is even, gives each softmax group a query tile of its own (455 us).  All write the true row maximum and the sum relative
// to it.
// Every wait is bounded (kDevErrAttnTimeout); no load uses cluster multicast.
#include "tc_common.cuh"
#include <type_traits>

namespace cb {

int pitched_rows_staged(bool rotate, uint64_t y, uint64_t x, uint64_t cos, uint64_t sin, int64_t n_tokens, int64_t heads,
                        int64_t head_dim, int64_t head_pitch, int64_t pos_mod, int64_t pos_offset, int dtype, cudaStream_t st);   // rope.cu

constexpr unsigned kDevErrAttnTimeout = 3u;
constexpr int kAttnRows = 128;      // query rows per CTA = keys per tile
constexpr int kAttnHd = 128;        // padded head dimension
constexpr int kAttnThreads = 320;  // producer warp, MMA warp, two softmax groups of 4 warps

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

// alpha * acc for two accumulator words, rounded to the 16-bit type (the stored score of the reference), as floats
template <typename T>
__device__ __forceinline__ float2 rounded_scores(float alpha, uint32_t a, uint32_t b) {
  if constexpr (std::is_same<T, __half>::value) {
    return __half22float2(__floats2half2_rn(alpha * __uint_as_float(a), alpha * __uint_as_float(b)));
  } else {
    return __bfloat1622float2(__floats2bfloat162_rn(alpha * __uint_as_float(a), alpha * __uint_as_float(b)));
  }
}
template <typename T>
__device__ __forceinline__ float2 rounded_pair(uint32_t a, uint32_t b) {         // the same without the scaling
  if constexpr (std::is_same<T, __half>::value) {
    return __half22float2(__floats2half2_rn(__uint_as_float(a), __uint_as_float(b)));
  } else {
    return __bfloat1622float2(__floats2bfloat162_rn(__uint_as_float(a), __uint_as_float(b)));
  }
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (std::is_same<T, __half>::value) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
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
  unsigned char* sP = sV + 2 * kTileBytes;         // 2 x 32 KB (one per softmax group)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kTileBytes);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // 2
  uint64_t* k_empty = bars + 3;                    // 2
  uint64_t* v_full = bars + 5;                     // 2
  uint64_t* v_empty = bars + 7;                    // 2
  uint64_t* s_full = bars + 9;                     // 2
  uint64_t* s_empty = bars + 11;                   // 2
  uint64_t* p_full = bars + 13;                    // 2
  uint64_t* p_empty = bars + 15;                   // 2
  uint64_t* o_full = bars + 17;                    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  float* part = reinterpret_cast<float*>(bars + 20);       // [2 groups][128 rows] partial max, then partial sum
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Launch order: batch element slowest, then query tile (heaviest first), then head.  The CTAs that run at the same
  // time then belong to one or two batch elements, whose K and V (2 x 8 MB at 2048 x 32 x 128) stay in L2 while all 16
  // query tiles stream them, and the tiles that finish the kernel are light ones.  (Query tile slowest over the whole
  // batch: K and V no longer fit L2 between uses.  (batch, head) slowest: the last CTAs are heavy and leave a tail.)
  const int nq = p.seq / kAttnRows;
  const int b = (int)(blockIdx.x / (nq * p.heads));
  const int rem = (int)(blockIdx.x % (nq * p.heads));
  const int qi = nq - 1 - rem / p.heads;
  const int h = rem % p.heads;
  const int ntiles = qi + 1;                       // key tiles 0 .. qi
  const int q0 = qi * kAttnRows;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1); mbar_init(s_empty + s, 4); mbar_init(p_full + s, 4); mbar_init(p_empty + s, 1);
    }
    mbar_init(o_full, 1);
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
  const uint32_t tO = tmem_base + 256u;            // S buffers at columns 0 and 128

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
    const uint32_t aQ = smem_u32(sQ);
    auto issue_s = [&](int n) -> bool {             // S[n & 1] = Q K_n^T
      const int ks = n & 1;
      const unsigned ph = (unsigned)((n >> 1) & 1);
      if (!mbar_wait_bounded(k_full + ks, ph, kDevErrAttnTimeout)) return false;
      if (!mbar_wait_bounded(s_empty + ks, ph ^ 1, kDevErrAttnTimeout)) return false;
      tc_fence_after();
      const uint32_t aK = smem_u32(sK + (size_t)ks * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
        tc_mma_f16(tmem_base + (uint32_t)ks * 128u, kmajor_desc(aQ, k16), kmajor_desc(aK, k16), p.idesc_s, k16 ? 1u : 0u);
      tc_commit(k_empty + ks);
      tc_commit(s_full + ks);
      return true;
    };
    int n = 0;
    for (int j = 0; j < ntiles; ++j, ++n)           // pass 1: scores only
      if (!issue_s(n)) goto done;
    // pass 2: both S buffers are filled ahead; each P V follows its group's probabilities
    for (int j = 0; j < 2 && j < ntiles; ++j, ++n)
      if (!issue_s(n)) goto done;
    for (int j = 0; j < ntiles; ++j) {
      const int vs = j & 1;
      const unsigned ph = (unsigned)((j >> 1) & 1);
      if (!mbar_wait_bounded(v_full + vs, ph, kDevErrAttnTimeout)) goto done;
      if (!mbar_wait_bounded(p_full + vs, ph, kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      const uint32_t aV = smem_u32(sV + (size_t)vs * kTileBytes), aP = smem_u32(sP + (size_t)vs * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnRows / 16; ++k16)
        tc_mma_f16(tO, kmajor_desc(aP, k16), v_desc(aV, k16), p.idesc_pv, (j | k16) ? 1u : 0u);
      tc_commit(v_empty + vs);
      tc_commit(p_empty + vs);
      if (j + 2 < ntiles) { if (!issue_s(n)) goto done; ++n; }
    }
    tc_commit(o_full);
  } else if (warp >= 2) {
    // ---------------- softmax groups: 2 x 128 threads, thread = query row, group g takes key tiles j = g (mod 2) ------
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;                        // TMEM lane quarter this warp may read
    const int r = qq * 32 + lane;                   // row inside the tile
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    float m = -INFINITY;
    const bool neg = p.alpha < 0.f;
    bool ok = true;   // a wait that ran out ends this warp's work (all 32 lanes together: the tcgen05.ld below are
                      // warp-wide), but the warp still meets the group barriers below
    for (int j = grp; j < ntiles; j += 2) {         // pass 1: row maximum of the rounded, scaled, masked scores
      const int sb = j & 1;
      if (!mbar_wait_bounded_warp(s_full + sb, (unsigned)((j >> 1) & 1), kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)sb * 128u + lane_off;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t v[2][32];
        tc_ld32(ts + (uint32_t)(half * 64), v[0]);
        tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
        tc_ld_wait();
        if (half == 1) {                            // the accumulator is in registers: the next S may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + sb);
        }
        // Scaling by alpha and rounding to the storage type are monotone, so the maximum of the rounded scores is the
        // rounded, scaled maximum (minimum, for a negative alpha) of the raw accumulators: one instruction per score
        // here, four independent chains, and one scaling and rounding after the loop.
        float mq[4] = {m, -INFINITY, -INFINITY, -INFINITY};
        if (j != qi) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float a = __uint_as_float(v[i >> 5][i & 31]);
            mq[i & 3] = fmaxf(mq[i & 3], neg ? -a : a);
          }
        } else {                                    // diagonal tile: columns c <= r are unmasked
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float a = __uint_as_float(v[i >> 5][i & 31]);
            if (half * 64 + i <= r) mq[i & 3] = fmaxf(mq[i & 3], neg ? -a : a);
          }
        }
        m = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
      }
    }
    // m holds the extreme raw accumulator (sign-folded); back to a rounded, scaled score.  Rows with no unmasked
    // key in this group's tiles keep -inf.
    if (m != -INFINITY) m = Elem<T>::to_f32(Elem<T>::from_f32(p.alpha * (neg ? -m : m)));
    part[grp * kAttnRows + r] = m;
    named_barrier(1, 256);
    m = fmaxf(part[r], part[kAttnRows + r]);
    named_barrier(1, 256);                          // everyone has read the maxima before the sums overwrite them
    float l = 0.f;
    const float mb = m * kLog2e;
    unsigned char* myP = sP + (size_t)grp * kTileBytes;
    for (int j = grp; ok && j < ntiles; j += 2) {   // pass 2: exp, row sum, probabilities to shared memory
      const int n = ntiles + j, sb = n & 1;
      if (!mbar_wait_bounded_warp(s_full + sb, (unsigned)((n >> 1) & 1), kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)sb * 128u + lane_off;
      uint4 pk[16];                                 // this row's 128 probabilities, 8 per 16-byte chunk
      float lq[4] = {0.f, 0.f, 0.f, 0.f};           // independent partial row sums
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[2][32];
        tc_ld32(ts + (uint32_t)(half * 64), v[0]);
        tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
        tc_ld_wait();
        if (half == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + sb);
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int idx = g * 8 + i * 2;
            const float2 s2 = rounded_scores<T>(p.alpha, v[idx >> 5][idx & 31], v[idx >> 5][(idx & 31) + 1]);
            float e0 = exp2f_approx(__fmaf_rn(s2.x, kLog2e, -mb));
            float e1 = exp2f_approx(__fmaf_rn(s2.y, kLog2e, -mb));
            if (j == qi) {
              const int c = half * 64 + idx;
              if (c > r) e0 = 0.f;
              if (c + 1 > r) e1 = 0.f;
            }
            lq[i] += e0 + e1;
            w[i] = pack2<T>(e0, e1);
          }
          pk[half * 8 + g] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l += (lq[0] + lq[1]) + (lq[2] + lq[3]);
      // the P V two tiles back has read this group's probability buffer
      if (!mbar_wait_bounded_warp(p_empty + grp, (unsigned)((j >> 1) & 1) ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
#pragma unroll
      for (int c = 0; c < 16; ++c)                  // chunk c: keys 8c .. 8c+7; key half c >> 3, chunk c & 7 of the 128-byte row
        *reinterpret_cast<uint4*>(myP + (size_t)(c >> 3) * 16384 + (size_t)r * 128 + (((c & 7) ^ (r & 7)) << 4)) = pk[c];
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + grp);
    }
    part[grp * kAttnRows + r] = l;
    named_barrier(1, 256);
    l = part[r] + part[kAttnRows + r];
    // context rows = O / l.  Each thread scales its row (group 0 columns 0..63, group 1 the rest) into a packed
    // [128][head_dim] staging area (the probability buffers are free once the last P V has completed); the warps then
    // write whole rows with consecutive lanes on consecutive 8-byte pieces (a thread = row store would touch 32
    // sectors per instruction).
    const bool fin = ok && mbar_wait_bounded_warp(o_full, 0, kDevErrAttnTimeout);
    unsigned char* rowbuf = sP;
    if (fin) {
      tc_fence_after();
      const float rl = 1.f / l;
      if (grp == 0) {
        float* st = stats + (((long long)b * p.heads + h) * p.seq + q0 + r) * 4;
        st[0] = m; st[1] = l;
      }
#pragma unroll 1
      for (int c0 = grp * 64; c0 < grp * 64 + 64 && c0 < p.head_dim; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tO + lane_off + (uint32_t)c0, v);
        tc_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {               // 4 elements = 8 bytes (head_dim % 4 == 0)
          const int c = c0 + g * 4;
          if (c + 4 <= p.head_dim) {
            uint2 w;
            w.x = pack2<T>(__uint_as_float(v[g * 4]) * rl, __uint_as_float(v[g * 4 + 1]) * rl);
            w.y = pack2<T>(__uint_as_float(v[g * 4 + 2]) * rl, __uint_as_float(v[g * 4 + 3]) * rl);
            *reinterpret_cast<uint2*>(rowbuf + ((size_t)r * p.head_dim + c) * sizeof(T)) = w;
          }
        }
      }
      tc_fence_before();
    }
    named_barrier(1, 256);
    if (fin) {
      const int cw = warp - 2;                      // 8 softmax warps, 16 rows each
      for (int rr = cw * 16; rr < cw * 16 + 16; ++rr) {
        T* out = ctx + (((long long)b * p.seq + q0 + rr) * p.heads + h) * p.head_dim;
        if (lane < p.head_dim / 4)
          reinterpret_cast<uint2*>(out)[lane] = *reinterpret_cast<const uint2*>(rowbuf + ((size_t)rr * p.head_dim + lane * 4) * sizeof(T));
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

// Single-pass form of the forward kernel: S = Q K^T is formed once per key tile.  Each softmax group keeps a running
// maximum of its own tiles and its own O accumulator in tensor memory (S0, S1, O0, O1: 4 x 128 columns), and the two
// are merged at the end.  Per tile the group reads S from tensor memory twice (maximum first, then exponentials)
// instead of having the tensor cores recompute it.  The exponent reference m_used of a group only follows its true
// running maximum when that has moved by more than 2^8 (probabilities then stay below 256 in 16 bits, relative
// rounding unchanged); when it moves, the group scales its O rows and its row sum by 2^(old - new) in place, after
// the P V that last wrote them has completed.  Row statistics written: the true maximum and the sum relative to it,
// as the two-pass kernel writes them.
int g_attn_fwd_single = 1;

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fwd1_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, T* __restrict__ ctx, float* __restrict__ stats,
                      const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = base;                        // 32 KB
  unsigned char* sK = sQ + kTileBytes;             // 2 x 32 KB
  unsigned char* sV = sK + 2 * kTileBytes;         // 2 x 32 KB
  unsigned char* sP = sV + 2 * kTileBytes;         // 2 x 32 KB (one per softmax group)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kTileBytes);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // 2
  uint64_t* k_empty = bars + 3;                    // 2
  uint64_t* v_full = bars + 5;                     // 2
  uint64_t* v_empty = bars + 7;                    // 2
  uint64_t* s_full = bars + 9;                     // 2
  uint64_t* s_empty = bars + 11;                   // 2
  uint64_t* p_full = bars + 13;                    // 2
  uint64_t* p_empty = bars + 15;                   // 2
  uint64_t* o_full = bars + 17;                    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  float* part = reinterpret_cast<float*>(bars + 20);       // [2 groups][128 rows] exchange area
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // launch order as in attention_fwd_kernel: batch slowest, heaviest query tile first, then head
  const int nq = p.seq / kAttnRows;
  const int b = (int)(blockIdx.x / (nq * p.heads));
  const int rem = (int)(blockIdx.x % (nq * p.heads));
  const int qi = nq - 1 - rem / p.heads;
  const int h = rem % p.heads;
  const int ntiles = qi + 1;                       // key tiles 0 .. qi
  const int q0 = qi * kAttnRows;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1); mbar_init(s_empty + s, 4); mbar_init(p_full + s, 4); mbar_init(p_empty + s, 1);
    }
    mbar_init(o_full, 1);
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
  const uint32_t tO = tmem_base + 256u;            // S buffers at columns 0 and 128, O of group g at 256 + 128 g

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    mbar_expect_tx(q_full, kTileBytes);
    tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
    tma_load_4d(sQ + 16384, &tmQ, q_full, 64, q0, h, b);
    for (int j = 0; j < ntiles; ++j) {
      const int sl = j & 1;
      const unsigned ph = (unsigned)((j >> 1) & 1);
      if (!mbar_wait_bounded(k_empty + sl, ph ^ 1, kDevErrAttnTimeout)) goto done;
      unsigned char* dk = sK + (size_t)sl * kTileBytes;
      mbar_expect_tx(k_full + sl, kTileBytes);
      tma_load_4d(dk, &tmK, k_full + sl, 0, j * kAttnRows, h, b);
      tma_load_4d(dk + 16384, &tmK, k_full + sl, 64, j * kAttnRows, h, b);
      if (!mbar_wait_bounded(v_empty + sl, ph ^ 1, kDevErrAttnTimeout)) goto done;
      unsigned char* dv = sV + (size_t)sl * kTileBytes;
      mbar_expect_tx(v_full + sl, kTileBytes);
#pragma unroll
      for (int kh = 0; kh < 2; ++kh)
#pragma unroll
        for (int nh = 0; nh < 2; ++nh)
          tma_load_4d(dv + kh * 16384 + nh * 8192, &tmV, v_full + sl, nh * 64, j * kAttnRows + kh * 64, h, b);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    if (!mbar_wait_bounded(q_full, 0, kDevErrAttnTimeout)) goto done;
    const uint32_t aQ = smem_u32(sQ);
    auto issue_s = [&](int n) -> bool {             // S[n & 1] = Q K_n^T
      const int ks = n & 1;
      const unsigned ph = (unsigned)((n >> 1) & 1);
      if (!mbar_wait_bounded(k_full + ks, ph, kDevErrAttnTimeout)) return false;
      if (!mbar_wait_bounded(s_empty + ks, ph ^ 1, kDevErrAttnTimeout)) return false;
      tc_fence_after();
      const uint32_t aK = smem_u32(sK + (size_t)ks * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
        tc_mma_f16(tmem_base + (uint32_t)ks * 128u, kmajor_desc(aQ, k16), kmajor_desc(aK, k16), p.idesc_s, k16 ? 1u : 0u);
      tc_commit(k_empty + ks);
      tc_commit(s_full + ks);
      return true;
    };
    int n = 0;
    for (int j = 0; j < 2 && j < ntiles; ++j, ++n)
      if (!issue_s(n)) goto done;
    for (int j = 0; j < ntiles; ++j) {
      const int vs = j & 1;
      const unsigned ph = (unsigned)((j >> 1) & 1);
      if (!mbar_wait_bounded(v_full + vs, ph, kDevErrAttnTimeout)) goto done;
      if (!mbar_wait_bounded(p_full + vs, ph, kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      const uint32_t aV = smem_u32(sV + (size_t)vs * kTileBytes), aP = smem_u32(sP + (size_t)vs * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnRows / 16; ++k16)     // O of the tile's group; its first tile overwrites
        tc_mma_f16(tO + (uint32_t)vs * 128u, kmajor_desc(aP, k16), v_desc(aV, k16), p.idesc_pv, (j >= 2 || k16) ? 1u : 0u);
      tc_commit(v_empty + vs);
      tc_commit(p_empty + vs);
      if (j + 2 < ntiles) { if (!issue_s(n)) goto done; ++n; }
    }
    tc_commit(o_full);
  } else if (warp >= 2) {
    // ---------------- softmax groups: 2 x 128 threads, thread = query row, group g takes key tiles j = g (mod 2) ------
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;                        // TMEM lane quarter this warp may read
    const int r = qq * 32 + lane;                   // row inside the tile
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kLazy = 8.f;                    // the exponent reference follows the maximum in steps of more than 2^8
    const bool neg = p.alpha < 0.f;
    float m_true = -INFINITY;                       // running maximum of the rounded, scaled, unmasked scores of this group's tiles
    float mb = 0.f;                                 // exponent reference of this group, times log2(e)
    float l = 0.f;                                  // running row sum relative to that reference
    bool ok = true;   // a wait that ran out ends this warp's work (all 32 lanes together), but it still meets the barriers
    unsigned char* myP = sP + (size_t)grp * kTileBytes;
    const uint32_t tOg = tO + (uint32_t)grp * 128u + lane_off;
    for (int j = grp; j < ntiles; j += 2) {
      const int sb = j & 1;                         // == grp
      const unsigned ph = (unsigned)((j >> 1) & 1);
      if (!mbar_wait_bounded_warp(s_full + sb, ph, kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)sb * 128u + lane_off;
      // first reading of the tile: its row maximum (sign-folded raw accumulators; scaling by alpha and rounding to the
      // storage type are monotone, so they are applied to the extreme value only)
      float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t v[2][32];
        tc_ld32(ts + (uint32_t)(half * 64), v[0]);
        tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
        tc_ld_wait();
        if (j != qi) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float a = __uint_as_float(v[i >> 5][i & 31]);
            mq[i & 3] = fmaxf(mq[i & 3], neg ? -a : a);
          }
        } else {                                    // diagonal tile: columns c <= r are unmasked
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float a = __uint_as_float(v[i >> 5][i & 31]);
            if (half * 64 + i <= r) mq[i & 3] = fmaxf(mq[i & 3], neg ? -a : a);
          }
        }
      }
      float tm = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
      tm = Elem<T>::to_f32(Elem<T>::from_f32(p.alpha * (neg ? -tm : tm)));       // every row has an unmasked key in every tile
      m_true = fmaxf(m_true, tm);
      // move the exponent reference?  (first tile of the group: set it; O and l hold nothing yet)
      const bool first = j == grp;
      const float mb_new = m_true * kLog2e;
      const bool move = first || (mb_new - mb > kLazy);
      if (__any_sync(0xffffffffu, move && !first)) {
        // the P V that last wrote this group's O rows must have completed before they are read
        if (!mbar_wait_bounded_warp(p_empty + grp, ph ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
        tc_fence_after();
        const float f = move ? exp2f_approx(mb - mb_new) : 1.f;
        l *= f;
#pragma unroll 1
        for (int c0 = 0; c0 < kAttnHd; c0 += 32) {
          uint32_t o[32];
          tc_ld32(tOg + (uint32_t)c0, o);
          tc_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tc_st32(tOg + (uint32_t)c0, o);
        }
        tc_st_wait();
      }
      if (move) mb = mb_new;
      // second reading: exponentials relative to the reference, row sum, probabilities
      uint4 pk[16];                                 // this row's 128 probabilities, 8 per 16-byte chunk
      float lq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[2][32];
        tc_ld32(ts + (uint32_t)(half * 64), v[0]);
        tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
        tc_ld_wait();
        if (half == 1) {                            // the accumulator is in registers: the next S may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + sb);
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int idx = g * 8 + i * 2;
            const float2 s2 = rounded_scores<T>(p.alpha, v[idx >> 5][idx & 31], v[idx >> 5][(idx & 31) + 1]);
            float e0 = exp2f_approx(__fmaf_rn(s2.x, kLog2e, -mb));
            float e1 = exp2f_approx(__fmaf_rn(s2.y, kLog2e, -mb));
            if (j == qi) {
              const int c = half * 64 + idx;
              if (c > r) e0 = 0.f;
              if (c + 1 > r) e1 = 0.f;
            }
            lq[i] += e0 + e1;
            w[i] = pack2<T>(e0, e1);
          }
          pk[half * 8 + g] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l += (lq[0] + lq[1]) + (lq[2] + lq[3]);
      // the P V two tiles back has read this group's probability buffer
      if (!mbar_wait_bounded_warp(p_empty + grp, ph ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
#pragma unroll
      for (int c = 0; c < 16; ++c)                  // chunk c: keys 8c .. 8c+7; key half c >> 3, chunk c & 7 of the 128-byte row
        *reinterpret_cast<uint4*>(myP + (size_t)(c >> 3) * 16384 + (size_t)r * 128 + (((c & 7) ^ (r & 7)) << 4)) = pk[c];
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();                            // (orders the in-place scaling of O before the P V that follows)
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + grp);
    }
    // merge the two groups: common maximum, then each group's factor 2^(mb_g - m log2e) for its sum and its O rows
    part[grp * kAttnRows + r] = m_true;
    named_barrier(1, 256);
    const float m = fmaxf(part[r], part[kAttnRows + r]);
    named_barrier(1, 256);
    const bool has = ntiles > grp;                  // (a group without tiles holds nothing: factor 0, its O rows are not read)
    const float f_own = has ? exp2f_approx(mb - m * kLog2e) : 0.f;
    part[grp * kAttnRows + r] = l * f_own;
    named_barrier(1, 256);
    l = part[r] + part[kAttnRows + r];
    named_barrier(1, 256);
    part[grp * kAttnRows + r] = f_own;
    named_barrier(1, 256);
    const float f0 = part[r], f1 = part[kAttnRows + r];
    // context rows = (f0 O0 + f1 O1) / l: group 0 columns 0..63, group 1 the rest, through a packed staging area as in
    // attention_fwd_kernel
    const bool fin = ok && mbar_wait_bounded_warp(o_full, 0, kDevErrAttnTimeout);
    unsigned char* rowbuf = sP;
    if (fin) {
      tc_fence_after();
      const float rl = 1.f / l;
      const float g0 = f0 * rl, g1 = f1 * rl;
      if (grp == 0) {
        float* st = stats + (((long long)b * p.heads + h) * p.seq + q0 + r) * 4;
        st[0] = m; st[1] = l;
      }
#pragma unroll 1
      for (int c0 = grp * 64; c0 < grp * 64 + 64 && c0 < p.head_dim; c0 += 32) {
        uint32_t v0[32], v1[32];
        tc_ld32(tO + lane_off + (uint32_t)c0, v0);
        if (ntiles > 1) tc_ld32(tO + 128u + lane_off + (uint32_t)c0, v1);
        tc_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {               // 4 elements = 8 bytes (head_dim % 4 == 0)
          const int c = c0 + g * 4;
          if (c + 4 <= p.head_dim) {
            float o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              o[i] = __uint_as_float(v0[g * 4 + i]) * g0;
              if (ntiles > 1) o[i] = __fmaf_rn(__uint_as_float(v1[g * 4 + i]), g1, o[i]);
            }
            uint2 w;
            w.x = pack2<T>(o[0], o[1]);
            w.y = pack2<T>(o[2], o[3]);
            *reinterpret_cast<uint2*>(rowbuf + ((size_t)r * p.head_dim + c) * sizeof(T)) = w;
          }
        }
      }
      tc_fence_before();
    }
    named_barrier(1, 256);
    if (fin) {
      const int cw = warp - 2;                      // 8 softmax warps, 16 rows each
      for (int rr = cw * 16; rr < cw * 16 + 16; ++rr) {
        T* out = ctx + (((long long)b * p.seq + q0 + rr) * p.heads + h) * p.head_dim;
        if (lane < p.head_dim / 4)
          reinterpret_cast<uint2*>(out)[lane] = *reinterpret_cast<const uint2*>(rowbuf + ((size_t)rr * p.head_dim + lane * 4) * sizeof(T));
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

// Persistent form of attention_fwd1_kernel: one CTA per SM walks a list of (batch, query tile, head) items instead of
// ending after one.  Measured on the one-item form with 28 CTAs per SM: 8.1 us per CTA with one key tile, 20.5 us with
// 8.5 on average, i.e. 1.65 us per tile and 6.5 us per CTA that no tile accounts for (launch, barrier and tensor-memory
// set-up, the first loads' latency, the context rows' way out, exit), a third of the kernel at config 5.  Here the
// rings, the barriers and the tensor memory live across items, and the roles run ahead of one another across the item
// boundary: while the softmax warps merge, scale and store the context rows of an item, the producer has loaded the next
// Q and K / V tiles and the tensor cores have formed its first scores.
// Items are dealt in rounds of gridDim.x, every other round in reverse CTA order (the list is sorted heaviest first, so
// a CTA's long items are paired with short ones); every role derives the same sequence on its own.  (Drawing the items
// from a global counter instead, handed to the roles through a ring in shared memory, balanced better on paper and
// measured slower everywhere: 578 against 559 us at seq = 2048, 196 against 187 us at seq = 128.)  Tiles are counted
// across items (n): key tile n goes through ring slot, S buffer, softmax group and O accumulator n & 1.
int g_attn_fwd_persistent = 1;

struct AttnItem { int b, qi, h, ntiles; };
__device__ __forceinline__ bool attn_item(const AttnParams& p, int round, AttnItem& it) {
  const int nq = p.seq / kAttnRows;
  const long long total = (long long)p.batch * nq * p.heads;
  const long long w = (long long)round * gridDim.x + ((round & 1) ? (long long)(gridDim.x - 1 - blockIdx.x) : (long long)blockIdx.x);
  if (w >= total) return false;
  it.b = (int)(w / (nq * p.heads));
  const int rem = (int)(w % (nq * p.heads));
  it.qi = nq - 1 - rem / p.heads;                  // launch order as in attention_fwd_kernel: heaviest query tile first
  it.h = rem % p.heads;
  it.ntiles = it.qi + 1;
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fwd1p_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, T* __restrict__ ctx, float* __restrict__ stats,
                       const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = base;                        // 32 KB
  unsigned char* sK = sQ + kTileBytes;             // 2 x 32 KB
  unsigned char* sV = sK + 2 * kTileBytes;         // 2 x 32 KB
  unsigned char* sP = sV + 2 * kTileBytes;         // 2 x 32 KB (one per softmax group)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kTileBytes);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // 2
  uint64_t* k_empty = bars + 3;                    // 2
  uint64_t* v_full = bars + 5;                     // 2
  uint64_t* v_empty = bars + 7;                    // 2
  uint64_t* s_full = bars + 9;                     // 2
  uint64_t* s_empty = bars + 11;                   // 2
  uint64_t* p_full = bars + 13;                    // 2
  uint64_t* p_empty = bars + 15;                   // 2
  uint64_t* o_full = bars + 17;                    // 1
  uint64_t* q_empty = bars + 18;                   // 1: the item's last S matmul has read Q
  uint64_t* o_empty = bars + 19;                   // 1: the item's context rows have left the O accumulators
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1); // set by any role whose bounded wait ran out
  int* group_stop = abort_flag + 1;                        // what the softmax warps agreed on at an item's last barrier
  float* part = reinterpret_cast<float*>(bars + 22);       // [2 groups][128 rows] exchange area
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = p.seq / kAttnRows;
  const long long total = (long long)p.batch * nq * p.heads;
  const int rounds = (int)((total + gridDim.x - 1) / gridDim.x);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1); mbar_init(s_empty + s, 4); mbar_init(p_full + s, 4); mbar_init(p_empty + s, 1);
    }
    mbar_init(o_full, 1); mbar_init(q_empty, 1); mbar_init(o_empty, 8);
    *abort_flag = 0; *group_stop = 0;
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
  const uint32_t tO = tmem_base + 256u;            // S buffers at columns 0 and 128, O of group g at 256 + 128 g

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    unsigned n = 0, it = 0;                         // key tiles and items so far
    for (int round = 0; round < rounds; ++round) {
      AttnItem a;
      if (!attn_item(p, round, a)) continue;
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      if (it > 0 && !mbar_wait_bounded(q_empty, (it - 1) & 1u, kDevErrAttnTimeout)) break;
      const int q0 = a.qi * kAttnRows;
      mbar_expect_tx(q_full, kTileBytes);
      tma_load_4d(sQ, &tmQ, q_full, 0, q0, a.h, a.b);
      tma_load_4d(sQ + 16384, &tmQ, q_full, 64, q0, a.h, a.b);
      bool fail = false;
      for (int j = 0; j < a.ntiles; ++j, ++n) {
        const unsigned sl = n & 1u, ph = (n >> 1) & 1u;
        if (!mbar_wait_bounded(k_empty + sl, ph ^ 1u, kDevErrAttnTimeout)) { fail = true; break; }
        unsigned char* dk = sK + (size_t)sl * kTileBytes;
        mbar_expect_tx(k_full + sl, kTileBytes);
        tma_load_4d(dk, &tmK, k_full + sl, 0, j * kAttnRows, a.h, a.b);
        tma_load_4d(dk + 16384, &tmK, k_full + sl, 64, j * kAttnRows, a.h, a.b);
        if (!mbar_wait_bounded(v_empty + sl, ph ^ 1u, kDevErrAttnTimeout)) { fail = true; break; }
        unsigned char* dv = sV + (size_t)sl * kTileBytes;
        mbar_expect_tx(v_full + sl, kTileBytes);
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
          for (int nh = 0; nh < 2; ++nh)
            tma_load_4d(dv + kh * 16384 + nh * 8192, &tmV, v_full + sl, nh * 64, j * kAttnRows + kh * 64, a.h, a.b);
      }
      if (fail) { *reinterpret_cast<volatile int*>(abort_flag) = 1; break; }
      ++it;
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    const uint32_t aQ = smem_u32(sQ);
    auto issue_s = [&](unsigned nn) -> bool {        // S[nn & 1] = Q K_nn^T
      const unsigned ks = nn & 1u, ph = (nn >> 1) & 1u;
      if (!mbar_wait_bounded(k_full + ks, ph, kDevErrAttnTimeout)) return false;
      if (!mbar_wait_bounded(s_empty + ks, ph ^ 1u, kDevErrAttnTimeout)) return false;
      tc_fence_after();
      const uint32_t aK = smem_u32(sK + (size_t)ks * kTileBytes);
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
        tc_mma_f16(tmem_base + ks * 128u, kmajor_desc(aQ, k16), kmajor_desc(aK, k16), p.idesc_s, k16 ? 1u : 0u);
      tc_commit(k_empty + ks);
      tc_commit(s_full + ks);
      return true;
    };
    unsigned n = 0, it = 0;
    for (int round = 0; round < rounds; ++round) {
      AttnItem a;
      if (!attn_item(p, round, a)) continue;
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      bool fail = !mbar_wait_bounded(q_full, it & 1u, kDevErrAttnTimeout);
      const unsigned n0 = n;
      int issued = 0;
      for (; !fail && issued < 2 && issued < a.ntiles; ++issued) {
        fail = !issue_s(n0 + issued);
        if (!fail && issued + 1 == a.ntiles) tc_commit(q_empty);
      }
      // the previous item's context rows have been read out of both O accumulators
      if (!fail && it > 0) fail = !mbar_wait_bounded(o_empty, (it - 1) & 1u, kDevErrAttnTimeout);
      for (int j = 0; !fail && j < a.ntiles; ++j) {
        const unsigned nn = n0 + j, vs = nn & 1u, ph = (nn >> 1) & 1u;
        if (!mbar_wait_bounded(v_full + vs, ph, kDevErrAttnTimeout) || !mbar_wait_bounded(p_full + vs, ph, kDevErrAttnTimeout)) { fail = true; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + (size_t)vs * kTileBytes), aP = smem_u32(sP + (size_t)vs * kTileBytes);
#pragma unroll
        for (int k16 = 0; k16 < kAttnRows / 16; ++k16)   // the group's first tile of the item overwrites its accumulator
          tc_mma_f16(tO + vs * 128u, kmajor_desc(aP, k16), v_desc(aV, k16), p.idesc_pv, (j >= 2 || k16) ? 1u : 0u);
        tc_commit(v_empty + vs);
        tc_commit(p_empty + vs);
        if (issued < a.ntiles) {
          fail = !issue_s(n0 + issued);
          ++issued;
          if (!fail && issued == a.ntiles) tc_commit(q_empty);
        }
      }
      if (fail) { *reinterpret_cast<volatile int*>(abort_flag) = 1; break; }
      tc_commit(o_full);
      n = n0 + a.ntiles;
      ++it;
    }
  } else if (warp >= 2) {
    // ---------------- softmax groups: 2 x 128 threads, thread = query row, group g takes key tiles n = g (mod 2) ------
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;                        // TMEM lane quarter this warp may read
    const int r = qq * 32 + lane;                   // row inside the tile
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kLazy = 8.f;
    const bool neg = p.alpha < 0.f;
    unsigned char* myP = sP + (size_t)grp * kTileBytes;
    const uint32_t tOg = tO + (uint32_t)grp * 128u + lane_off;
    unsigned n = 0, it = 0;
    bool ok = true;   // a wait that ran out: this warp stops working on tiles but meets every barrier of the item; the
                      // whole group then leaves the item loop together after the item's last barrier
    for (int round = 0; round < rounds; ++round) {
      AttnItem a;
      if (!attn_item(p, round, a)) continue;
      const int q0 = a.qi * kAttnRows;
      const unsigned n0 = n;
      float m_true = -INFINITY, mb = 0.f, l = 0.f;
      bool first = true;
      for (int j = 0; ok && j < a.ntiles; ++j) {
        const unsigned nn = n0 + j;
        if ((int)(nn & 1u) != grp) continue;
        const unsigned ph = (nn >> 1) & 1u;
        if (!mbar_wait_bounded_warp(s_full + grp, ph, kDevErrAttnTimeout)) { ok = false; break; }
        // The tensor pipe runs its matmuls in issue order and this S was issued after the group's previous P V, so
        // that one has completed too: the wait below returns at once.  It makes the group's O rows and its
        // probability buffer safe to touch from here on.
        if (!mbar_wait_bounded_warp(p_empty + grp, ph ^ 1u, kDevErrAttnTimeout)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ts = tmem_base + (uint32_t)grp * 128u + lane_off;
        float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t v[2][32];
          tc_ld32(ts + (uint32_t)(half * 64), v[0]);
          tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
          tc_ld_wait();
          if (j != a.qi) {
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const float x = __uint_as_float(v[i >> 5][i & 31]);
              mq[i & 3] = fmaxf(mq[i & 3], neg ? -x : x);
            }
          } else {                                  // diagonal tile: columns c <= r are unmasked
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const float x = __uint_as_float(v[i >> 5][i & 31]);
              if (half * 64 + i <= r) mq[i & 3] = fmaxf(mq[i & 3], neg ? -x : x);
            }
          }
        }
        float tm = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
        tm = Elem<T>::to_f32(Elem<T>::from_f32(p.alpha * (neg ? -tm : tm)));
        m_true = fmaxf(m_true, tm);
        const float mb_new = m_true * kLog2e;
        const bool move = first || (mb_new - mb > kLazy);
        if (__any_sync(0xffffffffu, move && !first)) {
          const float f = (move && !first) ? exp2f_approx(mb - mb_new) : 1.f;
          l *= f;
#pragma unroll 1
          for (int c0 = 0; c0 < kAttnHd; c0 += 32) {
            uint32_t o[32];
            tc_ld32(tOg + (uint32_t)c0, o);
            tc_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tc_st32(tOg + (uint32_t)c0, o);
          }
          tc_st_wait();
        }
        if (move) mb = mb_new;
        first = false;
        float lq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint4 pk[8];                              // 64 probabilities of this row, 8 per 16-byte chunk
          uint32_t v[2][32];
          tc_ld32(ts + (uint32_t)(half * 64), v[0]);
          tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
          tc_ld_wait();
          if (half == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty + grp);
          }
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int idx = g * 8 + i * 2;
              const float2 s2 = rounded_scores<T>(p.alpha, v[idx >> 5][idx & 31], v[idx >> 5][(idx & 31) + 1]);
              float e0 = exp2f_approx(__fmaf_rn(s2.x, kLog2e, -mb));
              float e1 = exp2f_approx(__fmaf_rn(s2.y, kLog2e, -mb));
              if (j == a.qi) {
                const int c = half * 64 + idx;
                if (c > r) e0 = 0.f;
                if (c + 1 > r) e1 = 0.f;
              }
              lq[i] += e0 + e1;
              w[i] = pack2<T>(e0, e1);
            }
            pk[g] = make_uint4(w[0], w[1], w[2], w[3]);
          }
#pragma unroll
          for (int c = 0; c < 8; ++c)               // chunk c of key half `half`: keys 64 half + 8c .. + 7, 128-byte-swizzled row
            *reinterpret_cast<uint4*>(myP + (size_t)half * 16384 + (size_t)r * 128 + ((c ^ (r & 7)) << 4)) = pk[c];
        }
        l += (lq[0] + lq[1]) + (lq[2] + lq[3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + grp);
      }
      n = n0 + (unsigned)a.ntiles;
      if (!ok && lane == 0) *reinterpret_cast<volatile int*>(abort_flag) = 1;
      // merge the two groups (a group without a tile in this item holds nothing: factor 0, its O rows are not read)
      const bool has0 = a.ntiles >= 2 || (n0 & 1u) == 0u, has1 = a.ntiles >= 2 || (n0 & 1u) == 1u;
      const bool has = grp == 0 ? has0 : has1;
      part[grp * kAttnRows + r] = has ? m_true : -INFINITY;
      named_barrier(1, 256);
      const float m = fmaxf(part[r], part[kAttnRows + r]);
      named_barrier(1, 256);
      const float f_own = has ? exp2f_approx(mb - m * kLog2e) : 0.f;
      part[grp * kAttnRows + r] = has ? l * f_own : 0.f;
      named_barrier(1, 256);
      l = part[r] + part[kAttnRows + r];
      named_barrier(1, 256);
      part[grp * kAttnRows + r] = f_own;
      named_barrier(1, 256);
      const float f0 = part[r], f1 = part[kAttnRows + r];
      const bool fin = ok && mbar_wait_bounded_warp(o_full, it & 1u, kDevErrAttnTimeout);
      if (!fin && lane == 0) *reinterpret_cast<volatile int*>(abort_flag) = 1;
      unsigned char* rowbuf = sP;
      if (fin) {
        tc_fence_after();
        const float rl = 1.f / l;
        const float g0 = f0 * rl, g1 = f1 * rl;
        if (grp == 0) {
          float* st = stats + (((long long)a.b * p.heads + a.h) * p.seq + q0 + r) * 4;
          st[0] = m; st[1] = l;
        }
#pragma unroll 1
        for (int c0 = grp * 64; c0 < grp * 64 + 64 && c0 < p.head_dim; c0 += 32) {
          uint32_t v0[32], v1[32];
          if (has0) tc_ld32(tO + lane_off + (uint32_t)c0, v0);
          if (has1) tc_ld32(tO + 128u + lane_off + (uint32_t)c0, v1);
          tc_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int c = c0 + g * 4;
            if (c + 4 <= p.head_dim) {
              float o[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                o[i] = has0 ? __uint_as_float(v0[g * 4 + i]) * g0 : 0.f;
                if (has1) o[i] = __fmaf_rn(__uint_as_float(v1[g * 4 + i]), g1, o[i]);
              }
              uint2 w;
              w.x = pack2<T>(o[0], o[1]);
              w.y = pack2<T>(o[2], o[3]);
              *reinterpret_cast<uint2*>(rowbuf + ((size_t)r * p.head_dim + c) * sizeof(T)) = w;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_empty);        // the next item's first P V may overwrite the accumulators
      }
      named_barrier(1, 256);
      if (fin) {
        const int cw = warp - 2;                    // 8 softmax warps, 16 rows each
        for (int rr = cw * 16; rr < cw * 16 + 16; ++rr) {
          T* out = ctx + (((long long)a.b * p.seq + q0 + rr) * p.heads + a.h) * p.head_dim;
          if (lane < p.head_dim / 4)
            reinterpret_cast<uint2*>(out)[lane] = *reinterpret_cast<const uint2*>(rowbuf + ((size_t)rr * p.head_dim + lane * 4) * sizeof(T));
        }
      }
      // the staging area is the first probability buffer: nobody writes the next item's probabilities into it before
      // every warp has read its rows.  The same barrier carries the decision to stop: one thread reads the flag and
      // all eight warps act on that one reading (a named barrier has no time limit, so no warp may leave alone)
      if (warp == 2 && lane == 0) *group_stop = *reinterpret_cast<volatile int*>(abort_flag);
      named_barrier(1, 256);
      ++it;
      if (*reinterpret_cast<volatile int*>(group_stop)) break;
    }
    tc_fence_before();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// Two query tiles per CTA, one per softmax group.  In the kernels above the two groups share one query tile and take
// its key tiles in turn: at the tile's start one group idles until a second key tile exists, at its end one idles while
// the other finishes, then both wait for the last P V and merge through shared memory: 6.5 us per query tile that no
// key tile accounts for.  Here group g owns query tile 2 i + g of a (batch, head) outright: its own Q, S buffer, O
// accumulator, running maximum, probability buffer and context rows, nothing to merge; the two groups read the SAME
// K / V tiles, loaded once (K through a single slot: both score matmuls of a key tile are issued back to back; V through
// two).  The tensor-core thread serves whichever group is ready: it looks at the four things it could issue next (a score
// matmul or a P V for either group) without parking on any of them.  Needs an even number of query tiles.
int g_attn_fwd_pair = 1;

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, T* __restrict__ ctx, float* __restrict__ stats,
                      const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = base;                        // 2 x 32 KB (one per group)
  unsigned char* sK = sQ + 2 * kTileBytes;         // 32 KB
  unsigned char* sV = sK + kTileBytes;             // 2 x 32 KB
  unsigned char* sP = sV + 2 * kTileBytes;         // 2 x 32 KB (one per group)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kTileBytes);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // 1
  uint64_t* k_empty = bars + 2;                    // 1
  uint64_t* v_full = bars + 3;                     // 2
  uint64_t* v_empty = bars + 5;                    // 2
  uint64_t* s_full = bars + 7;                     // 2 (per group)
  uint64_t* s_empty = bars + 9;                    // 2
  uint64_t* p_full = bars + 11;                    // 2
  uint64_t* p_empty = bars + 13;                   // 2
  uint64_t* o_full = bars + 15;                    // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // launch order: batch slowest, then the pair of query tiles (heaviest first), then head
  const int npair = p.seq / (2 * kAttnRows);
  const int b = (int)(blockIdx.x / (npair * p.heads));
  const int rem = (int)(blockIdx.x % (npair * p.heads));
  const int qa = 2 * (npair - 1 - rem / p.heads);  // group 0's query tile; group 1 has qa + 1
  const int h = rem % p.heads;
  const int nkv = qa + 2;                          // key tiles 0 .. qa + 1 (the last one for group 1 only)

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(k_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1);
      mbar_init(s_full + s, 1); mbar_init(s_empty + s, 4); mbar_init(p_full + s, 4); mbar_init(p_empty + s, 1);
      mbar_init(o_full + s, 1);
    }
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
  const uint32_t tmem_base = *tmem_slot;           // S of group g at 128 g, O of group g at 256 + 128 g

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    mbar_expect_tx(q_full, 2 * kTileBytes);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      tma_load_4d(sQ + (size_t)g * kTileBytes, &tmQ, q_full, 0, (qa + g) * kAttnRows, h, b);
      tma_load_4d(sQ + (size_t)g * kTileBytes + 16384, &tmQ, q_full, 64, (qa + g) * kAttnRows, h, b);
    }
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait_bounded(k_empty, (unsigned)(j & 1) ^ 1u, kDevErrAttnTimeout)) goto done;
      mbar_expect_tx(k_full, kTileBytes);
      tma_load_4d(sK, &tmK, k_full, 0, j * kAttnRows, h, b);
      tma_load_4d(sK + 16384, &tmK, k_full, 64, j * kAttnRows, h, b);
      const int vs = j & 1;
      if (!mbar_wait_bounded(v_empty + vs, (unsigned)((j >> 1) & 1) ^ 1u, kDevErrAttnTimeout)) goto done;
      unsigned char* dv = sV + (size_t)vs * kTileBytes;
      mbar_expect_tx(v_full + vs, kTileBytes);
#pragma unroll
      for (int kh = 0; kh < 2; ++kh)
#pragma unroll
        for (int nh = 0; nh < 2; ++nh)
          tma_load_4d(dv + kh * 16384 + nh * 8192, &tmV, v_full + vs, nh * 64, j * kAttnRows + kh * 64, h, b);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer: serves whichever group is ready ----------------
    if (!mbar_wait_bounded(q_full, 0, kDevErrAttnTimeout)) goto done;
    const int nt[2] = {qa + 1, qa + 2};             // key tiles of each group
    int sN[2] = {0, 0}, pN[2] = {0, 0};             // score matmuls and P V issued so far, per group
    int kdone = 0;                                  // key tiles whose slot has been handed back
    unsigned idle = 0;
    const uint32_t aK = smem_u32(sK);
    while (pN[0] < nt[0] || pN[1] < nt[1]) {
      bool progress = false;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const int j = sN[g];
        if (j < nt[g] && j == kdone && mbar_test(k_full, (unsigned)(j & 1)) && mbar_test(s_empty + g, (unsigned)(j & 1) ^ 1u)) {
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQ + (size_t)g * kTileBytes);
#pragma unroll
          for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
            tc_mma_f16(tmem_base + (uint32_t)g * 128u, kmajor_desc(aQ, k16), kmajor_desc(aK, k16), p.idesc_s, k16 ? 1u : 0u);
          tc_commit(s_full + g);
          sN[g] = j + 1;
          progress = true;
          if ((sN[0] > j || j >= nt[0]) && (sN[1] > j || j >= nt[1])) { tc_commit(k_empty); kdone = j + 1; }
        }
        const int t = pN[g];
        if (t < sN[g] && mbar_test(p_full + g, (unsigned)(t & 1)) && mbar_test(v_full + (t & 1), (unsigned)((t >> 1) & 1))) {
          tc_fence_after();
          const uint32_t aV = smem_u32(sV + (size_t)(t & 1) * kTileBytes), aP = smem_u32(sP + (size_t)g * kTileBytes);
#pragma unroll
          for (int k16 = 0; k16 < kAttnRows / 16; ++k16)
            tc_mma_f16(tmem_base + 256u + (uint32_t)g * 128u, kmajor_desc(aP, k16), v_desc(aV, k16), p.idesc_pv, (t | k16) ? 1u : 0u);
          tc_commit(p_empty + g);
          pN[g] = t + 1;
          progress = true;
          if ((pN[0] > t || t >= nt[0]) && (pN[1] > t || t >= nt[1])) tc_commit(v_empty + (t & 1));
          if (pN[g] == nt[g]) tc_commit(o_full + g);
        }
      }
      if (progress) {
        idle = 0;
      } else if (++idle > (1u << 24)) {             // nothing became ready for far longer than any healthy wait
        atomicMax(&g_dev_error, kDevErrAttnTimeout);
        goto done;
      }
    }
  } else if (warp >= 2) {
    // ---------------- softmax groups: group g = query tile qa + g, thread = query row ----------------
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;                        // TMEM lane quarter this warp may read
    const int r = qq * 32 + lane;                   // row inside the tile
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kLazy = 8.f;
    const bool neg = p.alpha < 0.f;
    const int qi = qa + grp, ntiles = qi + 1, q0 = qi * kAttnRows;
    unsigned char* myP = sP + (size_t)grp * kTileBytes;
    const uint32_t ts = tmem_base + (uint32_t)grp * 128u + lane_off;
    const uint32_t tOg = tmem_base + 256u + (uint32_t)grp * 128u + lane_off;
    float m_true = -INFINITY, mb = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const unsigned ph = (unsigned)(j & 1);
      if (!mbar_wait_bounded_warp(s_full + grp, ph, kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t v[2][32];
        tc_ld32(ts + (uint32_t)(half * 64), v[0]);
        tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
        tc_ld_wait();
        if (j != qi) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float x = __uint_as_float(v[i >> 5][i & 31]);
            mq[i & 3] = fmaxf(mq[i & 3], neg ? -x : x);
          }
        } else {                                    // diagonal tile: columns c <= r are unmasked
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float x = __uint_as_float(v[i >> 5][i & 31]);
            if (half * 64 + i <= r) mq[i & 3] = fmaxf(mq[i & 3], neg ? -x : x);
          }
        }
      }
      float tm = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
      tm = Elem<T>::to_f32(Elem<T>::from_f32(p.alpha * (neg ? -tm : tm)));
      m_true = fmaxf(m_true, tm);
      const bool first = j == 0;
      const float mb_new = m_true * kLog2e;
      const bool move = first || (mb_new - mb > kLazy);
      // the group's previous P V must have completed before its O rows are scaled and before its probability buffer
      // is written again (a score matmul may overtake the P V before it, so s_full does not imply it)
      bool waited = false;
      if (__any_sync(0xffffffffu, move && !first)) {
        if (!mbar_wait_bounded_warp(p_empty + grp, ph ^ 1u, kDevErrAttnTimeout)) { ok = false; break; }
        waited = true;
        tc_fence_after();
        const float f = (move && !first) ? exp2f_approx(mb - mb_new) : 1.f;
        l *= f;
#pragma unroll 1
        for (int c0 = 0; c0 < kAttnHd; c0 += 32) {
          uint32_t o[32];
          tc_ld32(tOg + (uint32_t)c0, o);
          tc_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tc_st32(tOg + (uint32_t)c0, o);
        }
        tc_st_wait();
      }
      if (move) mb = mb_new;
      float lq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint4 pk[8];
        uint32_t v[2][32];
        tc_ld32(ts + (uint32_t)(half * 64), v[0]);
        tc_ld32(ts + (uint32_t)(half * 64 + 32), v[1]);
        tc_ld_wait();
        if (half == 1) {                            // the accumulator is in registers: the next S may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + grp);
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int idx = g * 8 + i * 2;
            const float2 s2 = rounded_scores<T>(p.alpha, v[idx >> 5][idx & 31], v[idx >> 5][(idx & 31) + 1]);
            float e0 = exp2f_approx(__fmaf_rn(s2.x, kLog2e, -mb));
            float e1 = exp2f_approx(__fmaf_rn(s2.y, kLog2e, -mb));
            if (j == qi) {
              const int c = half * 64 + idx;
              if (c > r) e0 = 0.f;
              if (c + 1 > r) e1 = 0.f;
            }
            lq[i] += e0 + e1;
            w[i] = pack2<T>(e0, e1);
          }
          pk[g] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (!waited) {
          if (!mbar_wait_bounded_warp(p_empty + grp, ph ^ 1u, kDevErrAttnTimeout)) { ok = false; break; }
          waited = true;
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)                 // chunk c of key half `half`, 128-byte-swizzled row
          *reinterpret_cast<uint4*>(myP + (size_t)half * 16384 + (size_t)r * 128 + ((c ^ (r & 7)) << 4)) = pk[c];
      }
      if (!ok) break;
      l += (lq[0] + lq[1]) + (lq[2] + lq[3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + grp);
    }
    // context rows = O / l, through the group's own probability buffer (free once its last P V has completed) so that
    // whole rows leave with consecutive lanes on consecutive 8-byte pieces
    const bool fin = ok && mbar_wait_bounded_warp(o_full + grp, 0, kDevErrAttnTimeout);
    unsigned char* rowbuf = myP;
    if (fin) {
      tc_fence_after();
      const float rl = 1.f / l;
      float* st = stats + (((long long)b * p.heads + h) * p.seq + q0 + r) * 4;
      st[0] = m_true;
      st[1] = l * exp2f_approx(mb - m_true * kLog2e);       // the sum relative to the true maximum
#pragma unroll 1
      for (int c0 = 0; c0 < p.head_dim; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tOg + (uint32_t)c0, v);
        tc_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {               // 4 elements = 8 bytes (head_dim % 4 == 0)
          const int c = c0 + g * 4;
          if (c + 4 <= p.head_dim) {
            uint2 w;
            w.x = pack2<T>(__uint_as_float(v[g * 4]) * rl, __uint_as_float(v[g * 4 + 1]) * rl);
            w.y = pack2<T>(__uint_as_float(v[g * 4 + 2]) * rl, __uint_as_float(v[g * 4 + 3]) * rl);
            *reinterpret_cast<uint2*>(rowbuf + ((size_t)r * p.head_dim + c) * sizeof(T)) = w;
          }
        }
      }
      tc_fence_before();
    }
    named_barrier(1 + grp, 128);
    if (fin) {
      const int cw = (warp - 2) & 3;                // the group's 4 warps, 32 rows each
      for (int rr = cw * 32; rr < cw * 32 + 32; ++rr) {
        T* out = ctx + (((long long)b * p.seq + q0 + rr) * p.heads + h) * p.head_dim;
        if (lane < p.head_dim / 4)
          reinterpret_cast<uint2*>(out)[lane] = *reinterpret_cast<const uint2*>(rowbuf + ((size_t)rr * p.head_dim + lane * 4) * sizeof(T));
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

// c[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d] in f32, written to word 2 of the row's statistics.  Eight lanes per
// (b, s, h) row, four rows per warp, each lane on 8-byte pieces 8 apart: both tensors stream coalesced and every lane
// has up to eight loads in flight.
template <typename T>
__global__ void __launch_bounds__(256)
attention_rowdot_kernel(float* __restrict__ stats, const T* __restrict__ ctx, const T* __restrict__ dctx_pad, long long rows,
                        int seq, int heads, int head_dim) {
  const int lane = threadIdx.x & 31, sub = lane >> 3, l8 = lane & 7;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  const int pieces = head_dim / 4;
  for (long long row0 = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 4; row0 < rows; row0 += warps * 4) {
    const long long row = row0 + sub;
    float acc = 0.f;
    if (row < rows) {
      const uint2* o2 = reinterpret_cast<const uint2*>(ctx + row * head_dim);
      const uint2* g2 = reinterpret_cast<const uint2*>(dctx_pad + row * kAttnHd);
#pragma unroll 4
      for (int i = l8; i < pieces; i += 8) {
        const uint2 a = __ldg(o2 + i), g = __ldg(g2 + i);
        float2 a0, a1, g0, g1;
        if constexpr (std::is_same<T, __half>::value) {
          a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x)); a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
          g0 = __half22float2(*reinterpret_cast<const __half2*>(&g.x)); g1 = __half22float2(*reinterpret_cast<const __half2*>(&g.y));
        } else {
          a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x)); a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
          g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.x)); g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.y));
        }
        acc = __fmaf_rn(a0.x, g0.x, __fmaf_rn(a0.y, g0.y, __fmaf_rn(a1.x, g1.x, __fmaf_rn(a1.y, g1.y, acc))));
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (l8 == 0 && row < rows) {
      const long long bs = row / heads;              // row = (b * seq + s) * heads + h
      const int h = (int)(row - bs * heads);
      const long long b = bs / seq;
      const int sq = (int)(bs - b * seq);
      stats[((b * heads + h) * seq + sq) * 4 + 2] = acc;
    }
  }
}

// ---- backward: probabilities and score adjoints, rebuilt tile by tile -------------------------------------------
// The adjoint of the chain needs P (for dV = P^T dO) and dS (for dQ = dS K, dK = dS^T Q).  The reference keeps the
// scores and recomputes the softmax from them inside InnerSoftmaxPostAdj (src/thunk/op.rs:3376-3457) after a block
// matmul has produced dP = dO V^T.  Here neither scores nor dP exist in HBM: per 128 x 128 tile two MMAs rebuild
// S = Q K^T and dP = dO V^T in tensor memory and the softmax threads turn them into
//   y = exp(s - m) / l   (m, l: the forward's row statistics),   P = T(y),   dS = T(y * T(dP) - c * y)
// with the reference's rounding points (s and dP rounded to the storage type first).  c = sum_j y_j dP_j is taken as
// D = dO . O (equal in exact arithmetic; O is the stored context row), so no pass over the whole row is needed
// before the first tile can be written; a small streaming kernel computes it per row into the statistics first.  Tiles above the diagonal are not written, except the one zero tile that
// completes the last written pair of tiles to 256 columns (what a CACTI_B200_TRI_A_* consumer may read).
template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_bwd_prep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                          const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmdS,
                          const T* __restrict__ ctx, const T* __restrict__ dctx_pad,
                          const float* __restrict__ stats, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = base;                        // 32 KB
  unsigned char* sdO = sQ + kTileBytes;            // 32 KB
  unsigned char* sK = sdO + kTileBytes;            // 2 x 32 KB
  unsigned char* sV = sK + 2 * kTileBytes;         // 2 x 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kTileBytes);
  uint64_t* q_full = bars;                         // 1: Q and dO
  uint64_t* kv_full = bars + 1;                    // 2
  uint64_t* kv_empty = bars + 3;                   // 2
  uint64_t* t_full = bars + 5;                     // 2: S and dP of one tile are complete
  uint64_t* t_empty = bars + 7;                    // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  // output staging: per softmax warp one [32 rows][64 columns] box in the 128-byte-swizzled layout of a TMA store
  unsigned char* stage = sV + 2 * kTileBytes + 1024;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int nq = p.seq / kAttnRows;                // launch order as in the forward kernel
  const int b = (int)(blockIdx.x / (nq * p.heads));
  const int rem = (int)(blockIdx.x % (nq * p.heads));
  const int qi = nq - 1 - rem / p.heads;
  const int h = rem % p.heads;
  const int ntiles = qi + 1;
  const int q0 = qi * kAttnRows;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); mbar_init(t_full + s, 1); mbar_init(t_empty + s, 4);
    }
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
  const uint32_t tmem_base = *tmem_slot;           // columns: S0 0, dP0 128, S1 256, dP1 384

  if (warp == 0 && lane == 0) {
    mbar_expect_tx(q_full, 2 * kTileBytes);
    tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
    tma_load_4d(sQ + 16384, &tmQ, q_full, 64, q0, h, b);
    tma_load_4d(sdO, &tmdO, q_full, 0, q0, h, b);
    tma_load_4d(sdO + 16384, &tmdO, q_full, 64, q0, h, b);
    for (int j = 0; j < ntiles; ++j) {
      const int sl = j & 1;
      if (!mbar_wait_bounded(kv_empty + sl, (unsigned)((j >> 1) & 1) ^ 1, kDevErrAttnTimeout)) goto done;
      unsigned char* dk = sK + (size_t)sl * kTileBytes;
      unsigned char* dv = sV + (size_t)sl * kTileBytes;
      mbar_expect_tx(kv_full + sl, 2 * kTileBytes);
      tma_load_4d(dk, &tmK, kv_full + sl, 0, j * kAttnRows, h, b);
      tma_load_4d(dk + 16384, &tmK, kv_full + sl, 64, j * kAttnRows, h, b);
      tma_load_4d(dv, &tmV, kv_full + sl, 0, j * kAttnRows, h, b);
      tma_load_4d(dv + 16384, &tmV, kv_full + sl, 64, j * kAttnRows, h, b);
    }
  } else if (warp == 1 && lane == 0) {
    if (!mbar_wait_bounded(q_full, 0, kDevErrAttnTimeout)) goto done;
    const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO);
    for (int j = 0; j < ntiles; ++j) {
      const int sl = j & 1;
      const unsigned ph = (unsigned)((j >> 1) & 1);
      if (!mbar_wait_bounded(kv_full + sl, ph, kDevErrAttnTimeout)) goto done;
      if (!mbar_wait_bounded(t_empty + sl, ph ^ 1, kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      const uint32_t aK = smem_u32(sK + (size_t)sl * kTileBytes), aV = smem_u32(sV + (size_t)sl * kTileBytes);
      const uint32_t tS = tmem_base + (uint32_t)sl * 256u, tdP = tS + 128u;
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
        tc_mma_f16(tS, kmajor_desc(aQ, k16), kmajor_desc(aK, k16), p.idesc_s, k16 ? 1u : 0u);
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
        tc_mma_f16(tdP, kmajor_desc(adO, k16), kmajor_desc(aV, k16), p.idesc_s, k16 ? 1u : 0u);
      tc_commit(kv_empty + sl);
      tc_commit(t_full + sl);
    }
  } else if (warp >= 2) {
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;
    const int r = qq * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    const float* st = stats + (((long long)b * p.heads + h) * p.seq + q0 + r) * 4;
    // y = exp(s - m) / l as one exponential: 2^(s log2e - (m log2e + log2 l))
    const float mb = __fmaf_rn(st[0], kLog2e, __log2f(st[1]));
    const float cdot = st[2];                       // c = dO . O, from attention_rowdot_kernel
    // Output staging: the warp's 4 KB hold one [32 rows][32 columns] box of P and one of dS (2 KB each, 64-byte rows in
    // the TMA unit's 64-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3)).  Both stores of a
    // quarter tile are issued together, and the wait for the TMA unit to have read them comes a quarter tile of
    // arithmetic later.
    unsigned char* boxP = stage + (size_t)(warp - 2) * 4096;
    unsigned char* boxD = boxP + 2048;
    const int row0 = q0 + qq * 32;                  // first query row of this warp
    const int sw = (lane >> 1) & 3;
    auto store_quarter = [&](const uint4 (&pc)[4], const uint4 (&dc)[4], int col0) {
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4*>(boxP + lane * 64 + ((c ^ sw) << 4)) = pc[c];
        *reinterpret_cast<uint4*>(boxD + lane * 64 + ((c ^ sw) << 4)) = dc[c];
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(&tmP, boxP, col0, row0, h, b);
        tma_store_4d(&tmdS, boxD, col0, row0, h, b);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    };
    for (int j = grp; j < ntiles; j += 2) {
      const int sl = j & 1;
      if (!mbar_wait_bounded_warp(t_full + sl, (unsigned)((j >> 1) & 1), kDevErrAttnTimeout)) goto done;
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)sl * 256u + lane_off;
#pragma unroll 1
      for (int qt = 0; qt < 4; ++qt) {              // 32 key columns at a time
        uint32_t sv[32], gv[32];
        tc_ld32(ts + (uint32_t)(qt * 32), sv);
        tc_ld32(ts + 128u + (uint32_t)(qt * 32), gv);
        tc_ld_wait();
        if (qt == 3) {                              // S and dP of this tile are in registers
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(t_empty + sl);
        }
        uint4 pc[4], dc[4];
        // two bodies, chosen per tile: only the tile on the diagonal carries the compares and selects of the mask
        auto quarter_math = [&](auto diag_tag) {
          constexpr bool DIAG = decltype(diag_tag)::value;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t pw[4], dw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int idx = g * 8 + i * 2;
              const float2 s2 = rounded_scores<T>(p.alpha, sv[idx], sv[idx + 1]);
              const float2 g2 = rounded_pair<T>(gv[idx], gv[idx + 1]);
              float y0 = exp2f_approx(__fmaf_rn(s2.x, kLog2e, -mb));
              float y1 = exp2f_approx(__fmaf_rn(s2.y, kLog2e, -mb));
              if (DIAG) {
                const int c = qt * 32 + idx;
                if (c > r) y0 = 0.f;
                if (c + 1 > r) y1 = 0.f;
              }
              pw[i] = pack2<T>(y0, y1);
              dw[i] = pack2<T>(__fmaf_rn(y0, g2.x, -__fmul_rn(cdot, y0)), __fmaf_rn(y1, g2.y, -__fmul_rn(cdot, y1)));
            }
            pc[g] = make_uint4(pw[0], pw[1], pw[2], pw[3]);
            dc[g] = make_uint4(dw[0], dw[1], dw[2], dw[3]);
          }
        };
        if (j == qi) quarter_math(std::true_type{}); else quarter_math(std::false_type{});
        store_quarter(pc, dc, j * kAttnRows + qt * 32);
      }
    }
    // zero tile that completes an odd count of written tiles to a multiple of 256 columns
    if ((ntiles & 1) && ntiles * kAttnRows < p.seq && grp == (ntiles & 1)) {
      uint4 z[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) z[g] = make_uint4(0, 0, 0, 0);
      for (int qt = 0; qt < 4; ++qt) store_quarter(z, z, ntiles * kAttnRows + qt * 32);
    }
    tc_fence_before();
  }
done:
  if (warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- backward, fully fused: dQ, dK, dV without P or dS in HBM ------------------------------------------------------
// attention_bwd_prep writes P and dS (2 x 2 bytes per unmasked score) for three block matmuls to read back.  The two
// kernels below keep them on chip instead.  Both rebuild S = Q K^T and dP = dO V^T per tile on the tensor cores and form
//   y = exp(s - m) / l,   P = T(y),   dS = T(y * T(dP) - c * y)       (s, dP rounded to the storage type; c = dO . O)
// exactly as attention_bwd_prep does (same rounding points), stage the 16-bit P / dS in shared memory in the layout
// of an MMA operand, and contract them at once:
//   attention_bwd_dq_kernel   one CTA per 128 query rows, over the key tiles at or before it:  dQ  = alpha dS K
//   attention_bwd_dkv_kernel  one CTA per 128 keys, over the query rows at or after it:        dV  = P^T dO,
//                                                                                              dK  = alpha dS^T Q
// Each output element is accumulated by one CTA in a fixed order (no floating-point atomics; dQ is not scattered from
// the key-tile kernel but recomputed per query tile, which costs S and dP a second time).  The f32 accumulators of the
// products live in tensor memory for the whole CTA; their operands differ from the block matmuls' only in that P and
// dS never left the SM, so the results agree with the three hinted block matmuls over attention_bwd_prep's output up
// to the summation order inside the tensor cores.
//
// Work is cut in units of 128 x 64 scores so that two softmax groups (4 warps each, one thread per TMEM lane) alternate
// and 512 tensor-memory columns hold everything: per group S (64) and dP (64), plus the 128-column accumulators (one in
// the dQ kernel, two in the dK / dV kernel).
constexpr int kBwdCols = 64;                                  // scores per TMEM lane and unit
constexpr uint32_t kUnitBytes = kAttnRows * kBwdCols * 2;     // 16 KB: a [128][64] 16-bit operand tile (128-byte rows)

// K-major operand with 128-byte rows stored as boxes of `box_bytes` (one per 64 contraction elements): step k16 of 16
__device__ __forceinline__ uint64_t kmajor_box_desc(uint32_t base, int k16, uint32_t box_bytes) {
  return make_desc(base + (uint32_t)(k16 >> 2) * box_bytes + (uint32_t)(k16 & 3) * 32u, 1, 64);
}
// The same stored tile read as an MN-major B operand [64 contraction rows][128 columns]: rows 128 bytes apart, the
// second 64 columns one box further (leading-dimension offset), 16 rows per step
__device__ __forceinline__ uint64_t mnmajor_box_desc(uint32_t base, int k16, uint32_t box_bytes) {
  return make_desc(base + (uint32_t)k16 * 2048u, box_bytes >> 4, 64);
}

// One thread's 32 scores of a unit: y and dS from the accumulators sv (S) and gv (dP).  col0: key (dQ kernel) or query
// (dK / dV kernel) index of element 0 relative to the thread's own row index `self`; masked when key > query.
template <typename T, bool WANT_P, bool ROW_IS_QUERY>
__device__ __forceinline__ void bwd_unit_math(const uint32_t (&sv)[32], const uint32_t (&gv)[32], float alpha, const float2* colstat,
                                              float mb_row, float c_row, bool diag, int col0, int self,
                                              uint4 (&pc)[4], uint4 (&dc)[4]) {
  constexpr float kLog2e = 1.4426950408889634f;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t pw[4], dw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = g * 8 + i * 2;
      const float2 s2 = rounded_scores<T>(alpha, sv[idx], sv[idx + 1]);
      const float2 g2 = rounded_pair<T>(gv[idx], gv[idx + 1]);
      // statistics belong to the query: the thread's own row, or the column's (shared memory: one 16-byte broadcast
      // load brings (mb, c) of two neighbouring queries)
      float mb0 = mb_row, mb1 = mb_row, c0 = c_row, c1 = c_row;
      if (!ROW_IS_QUERY) {
        const float4 st2 = *reinterpret_cast<const float4*>(colstat + idx);
        mb0 = st2.x; c0 = st2.y; mb1 = st2.z; c1 = st2.w;
      }
      float y0 = exp2f_approx(__fmaf_rn(s2.x, kLog2e, -mb0));
      float y1 = exp2f_approx(__fmaf_rn(s2.y, kLog2e, -mb1));
      if (diag) {
        const int c = col0 + idx;
        // ROW_IS_QUERY: column = key, masked when key > query (self); else column = query, masked when key (self) > query
        if (ROW_IS_QUERY ? (c > self) : (self > c)) y0 = 0.f;
        if (ROW_IS_QUERY ? (c + 1 > self) : (self > c + 1)) y1 = 0.f;
      }
      if (WANT_P) pw[i] = pack2<T>(y0, y1);
      dw[i] = pack2<T>(__fmaf_rn(y0, g2.x, -__fmul_rn(c0, y0)), __fmaf_rn(y1, g2.y, -__fmul_rn(c1, y1)));
    }
    if (WANT_P) pc[g] = make_uint4(pw[0], pw[1], pw[2], pw[3]);
    dc[g] = make_uint4(dw[0], dw[1], dw[2], dw[3]);
  }
}

// ---- dQ: one CTA per (batch, head, 128 query rows) -------------------------------------------------------------------
// warp 0 producer (Q and dO once, then K and V tiles through a two-slot ring), warp 1 MMA issuer, warps 2..9 two
// softmax groups; group g works on keys [64 g, 64 g + 64) of every 128-key tile.
// Tensor memory: group g: S at columns 128 g, dP at 128 g + 64; dQ at 256.
template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                        T* __restrict__ dq, const float* __restrict__ stats, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = base;                        // 32 KB
  unsigned char* sdO = sQ + kTileBytes;            // 32 KB
  unsigned char* sK = sdO + kTileBytes;            // 2 x 32 KB
  unsigned char* sV = sK + 2 * kTileBytes;         // 2 x 32 KB
  unsigned char* sDS = sV + 2 * kTileBytes;        // 2 x 16 KB, one per group: dS [128 queries][64 keys], K-major
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * kUnitBytes);
  uint64_t* q_full = bars;                         // 1
  uint64_t* kv_full = bars + 1;                    // 2
  uint64_t* kv_empty = bars + 3;                   // 2
  uint64_t* t_full = bars + 5;                     // 2 (per group): S and dP of the group's unit are complete
  uint64_t* t_empty = bars + 7;                    // 2: the group has them in registers
  uint64_t* ds_full = bars + 9;                    // 2: the group's dS is staged
  uint64_t* ds_empty = bars + 11;                  // 2: the dQ product has read it
  uint64_t* acc_full = bars + 13;                  // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int nq = p.seq / kAttnRows;                // launch order as in the forward kernel
  const int b = (int)(blockIdx.x / (nq * p.heads));
  const int rem = (int)(blockIdx.x % (nq * p.heads));
  const int qi = nq - 1 - rem / p.heads;
  const int h = rem % p.heads;
  const int ntiles = qi + 1;
  const int q0 = qi * kAttnRows;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(acc_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1);
      mbar_init(t_full + s, 1); mbar_init(t_empty + s, 4); mbar_init(ds_full + s, 4); mbar_init(ds_empty + s, 1);
    }
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
  const uint32_t tAcc = tmem_base + 256u;

  if (warp == 0 && lane == 0) {
    mbar_expect_tx(q_full, 2 * kTileBytes);
    tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
    tma_load_4d(sQ + 16384, &tmQ, q_full, 64, q0, h, b);
    tma_load_4d(sdO, &tmdO, q_full, 0, q0, h, b);
    tma_load_4d(sdO + 16384, &tmdO, q_full, 64, q0, h, b);
    for (int j = 0; j < ntiles; ++j) {
      const int sl = j & 1;
      if (!mbar_wait_bounded(kv_empty + sl, (unsigned)((j >> 1) & 1) ^ 1, kDevErrAttnTimeout)) break;
      unsigned char* dk = sK + (size_t)sl * kTileBytes;
      unsigned char* dv = sV + (size_t)sl * kTileBytes;
      mbar_expect_tx(kv_full + sl, 2 * kTileBytes);
      tma_load_4d(dk, &tmK, kv_full + sl, 0, j * kAttnRows, h, b);
      tma_load_4d(dk + 16384, &tmK, kv_full + sl, 64, j * kAttnRows, h, b);
      tma_load_4d(dv, &tmV, kv_full + sl, 0, j * kAttnRows, h, b);
      tma_load_4d(dv + 16384, &tmV, kv_full + sl, 64, j * kAttnRows, h, b);
    }
  } else if (warp == 1 && lane == 0) {
    bool ok = mbar_wait_bounded(q_full, 0, kDevErrAttnTimeout);
    const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO);
    // dQ += dS_g K[64 g ..] of tile jj, for both groups; then the tile's K / V slot is free
    auto finish = [&](int jj) -> bool {
      const int sl = jj & 1;
      const uint32_t aK = smem_u32(sK + (size_t)sl * kTileBytes);
      for (int g = 0; g < 2; ++g) {
        if (!mbar_wait_bounded(ds_full + g, (unsigned)(jj & 1), kDevErrAttnTimeout)) return false;
        tc_fence_after();
        const uint32_t aDS = smem_u32(sDS + (size_t)g * kUnitBytes);
#pragma unroll
        for (int k16 = 0; k16 < kBwdCols / 16; ++k16)
          tc_mma_f16(tAcc, kmajor_box_desc(aDS, k16, kUnitBytes), mnmajor_box_desc(aK + (uint32_t)g * 8192u, k16, 16384u), p.idesc_pv,
                     (jj | g | k16) ? 1u : 0u);
        tc_commit(ds_empty + g);
      }
      tc_commit(kv_empty + sl);
      return true;
    };
    for (int j = 0; ok && j < ntiles; ++j) {
      const int sl = j & 1;
      if (!mbar_wait_bounded(kv_full + sl, (unsigned)((j >> 1) & 1), kDevErrAttnTimeout)) { ok = false; break; }
      const uint32_t aK = smem_u32(sK + (size_t)sl * kTileBytes), aV = smem_u32(sV + (size_t)sl * kTileBytes);
      for (int g = 0; g < 2; ++g) {
        if (!mbar_wait_bounded(t_empty + g, (unsigned)(j & 1) ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tS = tmem_base + (uint32_t)g * 128u, tdP = tS + 64u;
#pragma unroll
        for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
          tc_mma_f16(tS, kmajor_desc(aQ, k16), kmajor_box_desc(aK + (uint32_t)g * 8192u, k16, 16384u), p.idesc_s, k16 ? 1u : 0u);
#pragma unroll
        for (int k16 = 0; k16 < kAttnHd / 16; ++k16)
          tc_mma_f16(tdP, kmajor_desc(adO, k16), kmajor_box_desc(aV + (uint32_t)g * 8192u, k16, 16384u), p.idesc_s, k16 ? 1u : 0u);
        tc_commit(t_full + g);
      }
      if (ok && j > 0) ok = finish(j - 1);
    }
    if (ok) ok = finish(ntiles - 1);
    if (ok) tc_commit(acc_full);
  } else if (warp >= 2) {
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;
    const int r = qq * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    const float* st = stats + (((long long)b * p.heads + h) * p.seq + q0 + r) * 4;
    const float mb = __fmaf_rn(st[0], kLog2e, __log2f(st[1]));      // y = 2^(s log2e - mb)
    const float cdot = st[2];
    unsigned char* myDS = sDS + (size_t)grp * kUnitBytes;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      if (!mbar_wait_bounded_warp(t_full + grp, (unsigned)(j & 1), kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)grp * 128u + lane_off;
      // the dQ product of the previous tile has read this group's staging buffer (issued a whole unit ago)
      if (!mbar_wait_bounded_warp(ds_empty + grp, (unsigned)(j & 1) ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {              // 32 keys at a time
        uint32_t sv[32], gv[32];
        tc_ld32(ts + (uint32_t)(hh * 32), sv);
        tc_ld32(ts + 64u + (uint32_t)(hh * 32), gv);
        tc_ld_wait();
        if (hh == 1) {                              // the unit is in registers: the next S / dP may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(t_empty + grp);
        }
        uint4 unused[4], dc[4];
        bwd_unit_math<T, false, true>(sv, gv, p.alpha, nullptr, mb, cdot, j == qi, grp * kBwdCols + hh * 32, r, unused, dc);
#pragma unroll
        for (int c = 0; c < 4; ++c)                 // chunk hh * 4 + c: keys 8 (hh * 4 + c) .. + 7 of the unit
          *reinterpret_cast<uint4*>(myDS + (size_t)r * 128 + ((((hh * 4 + c) ^ (r & 7))) << 4)) = dc[c];
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full + grp);
    }
    // dQ rows: alpha * accumulator, rounded once; staged packed [128][head_dim] (the K ring is free by then) and
    // written with consecutive lanes on consecutive 8-byte pieces
    const bool fin = ok && mbar_wait_bounded_warp(acc_full, 0, kDevErrAttnTimeout);
    unsigned char* rowbuf = sK;
    if (fin) {
      tc_fence_after();
#pragma unroll 1
      for (int c0 = grp * 64; c0 < grp * 64 + 64 && c0 < p.head_dim; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tAcc + lane_off + (uint32_t)c0, v);
        tc_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int c = c0 + g * 4;
          if (c + 4 <= p.head_dim) {
            uint2 w;
            w.x = pack2<T>(__uint_as_float(v[g * 4]) * p.alpha, __uint_as_float(v[g * 4 + 1]) * p.alpha);
            w.y = pack2<T>(__uint_as_float(v[g * 4 + 2]) * p.alpha, __uint_as_float(v[g * 4 + 3]) * p.alpha);
            *reinterpret_cast<uint2*>(rowbuf + ((size_t)r * p.head_dim + c) * sizeof(T)) = w;
          }
        }
      }
      tc_fence_before();
    }
    named_barrier(1, 256);
    if (fin) {
      const int cw = warp - 2;
      for (int rr = cw * 16; rr < cw * 16 + 16; ++rr) {
        T* out = dq + (((long long)b * p.seq + q0 + rr) * p.heads + h) * p.head_dim;
        if (lane < p.head_dim / 4)
          reinterpret_cast<uint2*>(out)[lane] = *reinterpret_cast<const uint2*>(rowbuf + ((size_t)rr * p.head_dim + lane * 4) * sizeof(T));
      }
    }
    tc_fence_before();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- dK, dV: one CTA per (batch, head, 128 keys) -------------------------------------------------------------------
// K and V of the tile stay in shared memory; Q, dO (64 query rows at a time) and those rows' statistics come through a
// two-slot ring.  The scores are built transposed, S^T = K Q^T (TMEM lane = key, column = query), so that P^T and dS^T
// come out of the softmax threads in the layout of an A operand.  Unit t (query rows 128 j + 64 t ...) belongs to group
// t & 1 and ring slot t & 1.  Tensor memory: group g: S^T at 128 g, dP^T at 128 g + 64; dV at 256, dK at 384.
template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO64,
                         T* __restrict__ dk, T* __restrict__ dv, const float* __restrict__ stats, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sK = base;                        // 32 KB
  unsigned char* sV = sK + kTileBytes;             // 32 KB
  unsigned char* sQ = sV + kTileBytes;             // 2 x 16 KB: [64 queries][128 hd] as two boxes of 8 KB
  unsigned char* sdO = sQ + 2 * kUnitBytes;        // 2 x 16 KB
  unsigned char* sPT = sdO + 2 * kUnitBytes;       // 2 x 16 KB, one per group: P^T [128 keys][64 queries], K-major
  unsigned char* sDST = sPT + 2 * kUnitBytes;      // 2 x 16 KB: dS^T likewise
  float2* sStat = reinterpret_cast<float2*>(sDST + 2 * kUnitBytes);       // 2 x 64 x (mb, c)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 2 * kBwdCols);
  uint64_t* kv_full = bars;                        // 1
  uint64_t* qd_full = bars + 1;                    // 2
  uint64_t* qd_empty = bars + 3;                   // 2
  uint64_t* t_full = bars + 5;                     // 2 (per group)
  uint64_t* t_empty = bars + 7;                    // 2
  uint64_t* st_full = bars + 9;                    // 2: the group's P^T and dS^T are staged
  uint64_t* st_empty = bars + 11;                  // 2
  uint64_t* acc_full = bars + 13;                  // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // launch order: batch slowest, then key tile (tile 0 has the most query rows after it: heaviest first), then head
  const int nk = p.seq / kAttnRows;
  const int b = (int)(blockIdx.x / (nk * p.heads));
  const int rem = (int)(blockIdx.x % (nk * p.heads));
  const int kj = rem / p.heads;
  const int h = rem % p.heads;
  const int k0 = kj * kAttnRows;
  const int nunits = (p.seq - k0) / kBwdCols;      // query rows k0 .. seq in steps of 64

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(acc_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(qd_full + s, 1); mbar_init(qd_empty + s, 1);
      mbar_init(t_full + s, 1); mbar_init(t_empty + s, 4); mbar_init(st_full + s, 4); mbar_init(st_empty + s, 1);
    }
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
  const uint32_t tdV = tmem_base + 256u, tdK = tmem_base + 384u;

  if (warp == 0) {
    // ---------------- producer warp: lane 0 issues the bulk copies, all lanes stage the rows' statistics ----------------
    constexpr float kLog2e = 1.4426950408889634f;
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kTileBytes);
      tma_load_4d(sK, &tmK, kv_full, 0, k0, h, b);
      tma_load_4d(sK + 16384, &tmK, kv_full, 64, k0, h, b);
      tma_load_4d(sV, &tmV, kv_full, 0, k0, h, b);
      tma_load_4d(sV + 16384, &tmV, kv_full, 64, k0, h, b);
    }
    for (int t = 0; t < nunits; ++t) {
      const int sl = t & 1;
      const int qrow = k0 + t * kBwdCols;
      if (!mbar_wait_bounded_warp(qd_empty + sl, (unsigned)((t >> 1) & 1) ^ 1, kDevErrAttnTimeout)) break;
      // y = 2^(s log2e - mb) with mb = m log2e + log2 l; c = dO . O (word 2, from attention_rowdot_kernel)
      for (int i = lane; i < kBwdCols; i += 32) {
        const float4 sv = *reinterpret_cast<const float4*>(stats + (((long long)b * p.heads + h) * p.seq + qrow + i) * 4);
        sStat[sl * kBwdCols + i] = make_float2(__fmaf_rn(sv.x, kLog2e, __log2f(sv.y)), sv.z);
      }
      __syncwarp();
      if (lane == 0) {
        unsigned char* dq_ = sQ + (size_t)sl * kUnitBytes;
        unsigned char* do_ = sdO + (size_t)sl * kUnitBytes;
        mbar_expect_tx(qd_full + sl, 2 * kUnitBytes);            // its release also publishes the statistics above
        tma_load_4d(dq_, &tmQ64, qd_full + sl, 0, qrow, h, b);
        tma_load_4d(dq_ + 8192, &tmQ64, qd_full + sl, 64, qrow, h, b);
        tma_load_4d(do_, &tmdO64, qd_full + sl, 0, qrow, h, b);
        tma_load_4d(do_ + 8192, &tmdO64, qd_full + sl, 64, qrow, h, b);
      }
    }
  } else if (warp == 1 && lane == 0) {
    bool ok = mbar_wait_bounded(kv_full, 0, kDevErrAttnTimeout);
    const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
    // dV += P^T dO, dK += dS^T Q for unit u; then its ring slot and staging buffers are free
    auto finish = [&](int u) -> bool {
      const int g = u & 1;
      if (!mbar_wait_bounded(st_full + g, (unsigned)((u >> 1) & 1), kDevErrAttnTimeout)) return false;
      tc_fence_after();
      const uint32_t aPT = smem_u32(sPT + (size_t)g * kUnitBytes), aDST = smem_u32(sDST + (size_t)g * kUnitBytes);
      const uint32_t aQ = smem_u32(sQ + (size_t)g * kUnitBytes), adO = smem_u32(sdO + (size_t)g * kUnitBytes);
#pragma unroll
      for (int k16 = 0; k16 < kBwdCols / 16; ++k16)
        tc_mma_f16(tdV, kmajor_box_desc(aPT, k16, kUnitBytes), mnmajor_box_desc(adO, k16, 8192u), p.idesc_pv, (u | k16) ? 1u : 0u);
#pragma unroll
      for (int k16 = 0; k16 < kBwdCols / 16; ++k16)
        tc_mma_f16(tdK, kmajor_box_desc(aDST, k16, kUnitBytes), mnmajor_box_desc(aQ, k16, 8192u), p.idesc_pv, (u | k16) ? 1u : 0u);
      tc_commit(st_empty + g);
      tc_commit(qd_empty + g);
      return true;
    };
    for (int t = 0; ok && t < nunits; ++t) {
      const int g = t & 1;
      const unsigned ph = (unsigned)((t >> 1) & 1);
      if (!mbar_wait_bounded(qd_full + g, ph, kDevErrAttnTimeout)) { ok = false; break; }
      if (!mbar_wait_bounded(t_empty + g, ph ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      const uint32_t aQ = smem_u32(sQ + (size_t)g * kUnitBytes), adO = smem_u32(sdO + (size_t)g * kUnitBytes);
      const uint32_t tS = tmem_base + (uint32_t)g * 128u, tdP = tS + 64u;
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)       // S^T = K Q^T: 128 keys x 64 queries
        tc_mma_f16(tS, kmajor_desc(aK, k16), kmajor_box_desc(aQ, k16, 8192u), p.idesc_s, k16 ? 1u : 0u);
#pragma unroll
      for (int k16 = 0; k16 < kAttnHd / 16; ++k16)       // dP^T = V dO^T
        tc_mma_f16(tdP, kmajor_desc(aV, k16), kmajor_box_desc(adO, k16, 8192u), p.idesc_s, k16 ? 1u : 0u);
      tc_commit(t_full + g);
      if (t > 0) ok = finish(t - 1);
    }
    if (ok) ok = finish(nunits - 1);
    if (ok) tc_commit(acc_full);
  } else if (warp >= 2) {
    const int grp = (warp - 2) >> 2;
    const int qq = warp & 3;
    const int r = qq * 32 + lane;                   // key row inside the tile
    const uint32_t lane_off = (uint32_t)(qq * 32) << 16;
    unsigned char* myPT = sPT + (size_t)grp * kUnitBytes;
    unsigned char* myDST = sDST + (size_t)grp * kUnitBytes;
    bool ok = true;
    for (int t = grp; t < nunits; t += 2) {
      const unsigned ph = (unsigned)((t >> 1) & 1);
      if (!mbar_wait_bounded_warp(t_full + grp, ph, kDevErrAttnTimeout)) { ok = false; break; }
      // complete long since (the products waited for it); taken here for the statistics the producer warp staged with it
      if (!mbar_wait_bounded_warp(qd_full + grp, ph, kDevErrAttnTimeout)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + (uint32_t)grp * 128u + lane_off;
      const float2* stq = sStat + grp * kBwdCols;   // slot = group: this unit's 64 query rows
      // the products of the group's previous unit have read its staging buffers (issued a whole unit ago)
      if (!mbar_wait_bounded_warp(st_empty + grp, ph ^ 1, kDevErrAttnTimeout)) { ok = false; break; }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {              // 32 queries at a time
        uint32_t sv[32], gv[32];
        tc_ld32(ts + (uint32_t)(hh * 32), sv);
        tc_ld32(ts + 64u + (uint32_t)(hh * 32), gv);
        tc_ld_wait();
        if (hh == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(t_empty + grp);
        }
        // queries of units 0 and 1 overlap the key tile's own rows: key k0 + r is masked for query k0 + 64 t + c when r > 64 t + c
        uint4 pc[4], dc[4];
        bwd_unit_math<T, true, false>(sv, gv, p.alpha, stq + hh * 32, 0.f, 0.f, t < 2, t * kBwdCols + hh * 32, r, pc, dc);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const size_t off = (size_t)r * 128 + ((((hh * 4 + c) ^ (r & 7))) << 4);
          *reinterpret_cast<uint4*>(myPT + off) = pc[c];
          *reinterpret_cast<uint4*>(myDST + off) = dc[c];
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(st_full + grp);
    }
    // group 0 writes dV, group 1 alpha * dK: rows staged packed [128][head_dim] (P^T / dS^T buffers are free), then
    // consecutive lanes on consecutive 8-byte pieces
    const bool fin = ok && mbar_wait_bounded_warp(acc_full, 0, kDevErrAttnTimeout);
    unsigned char* rowbuf = grp == 0 ? sPT : sDST;          // 32 KB each: 128 rows x up to 256 bytes
    const float scale = grp == 0 ? 1.f : p.alpha;
    if (fin) {
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < p.head_dim; c0 += 32) {
        uint32_t v[32];
        tc_ld32((grp == 0 ? tdV : tdK) + lane_off + (uint32_t)c0, v);
        tc_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int c = c0 + g * 4;
          if (c + 4 <= p.head_dim) {
            uint2 w;
            w.x = pack2<T>(__uint_as_float(v[g * 4]) * scale, __uint_as_float(v[g * 4 + 1]) * scale);
            w.y = pack2<T>(__uint_as_float(v[g * 4 + 2]) * scale, __uint_as_float(v[g * 4 + 3]) * scale);
            *reinterpret_cast<uint2*>(rowbuf + ((size_t)r * p.head_dim + c) * sizeof(T)) = w;
          }
        }
      }
      tc_fence_before();
    }
    named_barrier(1 + grp, 128);                    // the group's 128 rows are staged
    if (fin) {
      T* outp = grp == 0 ? dv : dk;
      const int cw = qq;                            // 4 warps of the group, 32 rows each
      for (int rr = cw * 32; rr < cw * 32 + 32; ++rr) {
        T* out = outp + (((long long)b * p.seq + k0 + rr) * p.heads + h) * p.head_dim;
        if (lane < p.head_dim / 4)
          reinterpret_cast<uint2*>(out)[lane] = *reinterpret_cast<const uint2*>(rowbuf + ((size_t)rr * p.head_dim + lane * 4) * sizeof(T));
      }
    }
    tc_fence_before();
  }
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

// Fast path: cols % 4 == 0, cols_pad % 8 == 0, 8-byte aligned source, 16-byte aligned destination.  One thread per
// 16-byte chunk of the destination: two 8-byte loads (a source row is only 8-byte aligned), one 16-byte store.
__global__ void __launch_bounds__(256)
block_pad_vec_kernel(uint4* __restrict__ dst, const uint2* __restrict__ src, long long groups, int cols_u /* 8-byte units */,
                     int chunks /* 16-byte chunks per destination row */) {
  const long long total = groups * chunks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long gidx = i / chunks;
    const int c = (int)(i - gidx * chunks);
    const uint2* row = src + gidx * cols_u;
    uint2 lo = make_uint2(0, 0), hi = make_uint2(0, 0);
    if (2 * c < cols_u) lo = __ldcs(row + 2 * c);
    if (2 * c + 1 < cols_u) hi = __ldcs(row + 2 * c + 1);
    dst[i] = make_uint4(lo.x, lo.y, hi.x, hi.y);      // plain store: the padded copy is read next, from L2
  }
}

static int encode_bshd(CUtensorMap* map, uint64_t ptr, int batch, int seq, int heads, int hdp, int box_inner, int box_rows,
                       bool bf16, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CACTI_B200_ERR_LAUNCH;
  cuuint64_t dims[4] = {(cuuint64_t)hdp, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)heads * hdp * 2, (cuuint64_t)hdp * 2, (cuuint64_t)seq * heads * hdp * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  reinterpret_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return CACTI_B200_ERR_LAUNCH; }
  return CACTI_B200_OK;
}

constexpr size_t kAttnFwdSmem = 1024 + 7 * (size_t)kTileBytes + 256 + 2 * kAttnRows * sizeof(float);

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
  const long long grid = (long long)batch * heads * (seq / kAttnRows);
  // The persistent walk pays where items are short (measured against one tile per CTA: 11 to 18 % at seq <= 512, nothing
  // at seq = 2048, where the hardware's dynamic placement of one-item CTAs balances better than dealing the items out):
  // 1 = short sequences only, 2 = always, 0 = never.
  // Two query tiles per CTA wherever their number is even (measured fastest at every length: 185 / 227 / 313 / 464 us at
  // seq = 256 / 512 / 1024 / 2048 against 196 / 257 / 356 / 562 us persistent and 233 / 289 / 389 / 568 us one tile per
  // CTA, 28 one-tile CTAs per SM each); otherwise the persistent walk for short sequences, one tile per CTA for long.
  const bool pair = g_attn_fwd_pair && (seq / kAttnRows) % 2 == 0 && g_attn_fwd_persistent != 2;
  const bool persistent = g_attn_fwd_persistent == 2 || (g_attn_fwd_persistent == 1 && seq / kAttnRows <= 4);
  if (g_attn_fwd_single && pair) {
    auto kern = attention_fwd2_kernel<T>;
    static bool attr_set[kMaxDevices] = {};
    ensure_dynamic_smem(kern, kAttnFwdSmem, attr_set);
    kern<<<(unsigned)(grid / 2), kAttnThreads, kAttnFwdSmem, st>>>(tmQ, tmK, tmV, reinterpret_cast<T*>(ctx),
                                                                   reinterpret_cast<float*>(stats), p);
  } else if (g_attn_fwd_single && persistent) {
    auto kern = attention_fwd1p_kernel<T>;
    static bool attr_set[kMaxDevices] = {};
    ensure_dynamic_smem(kern, kAttnFwdSmem, attr_set);
    const unsigned pgrid = (unsigned)(grid < kNumSMs ? grid : kNumSMs);
    kern<<<pgrid, kAttnThreads, kAttnFwdSmem, st>>>(tmQ, tmK, tmV, reinterpret_cast<T*>(ctx),
                                                    reinterpret_cast<float*>(stats), p);
  } else if (g_attn_fwd_single) {
    auto kern = attention_fwd1_kernel<T>;
    static bool attr_set[kMaxDevices] = {};
    ensure_dynamic_smem(kern, kAttnFwdSmem, attr_set);
    kern<<<(unsigned)grid, kAttnThreads, kAttnFwdSmem, st>>>(tmQ, tmK, tmV, reinterpret_cast<T*>(ctx),
                                                             reinterpret_cast<float*>(stats), p);
  } else {
    auto kern = attention_fwd_kernel<T>;
    static bool attr_set[kMaxDevices] = {};
    ensure_dynamic_smem(kern, kAttnFwdSmem, attr_set);
    kern<<<(unsigned)grid, kAttnThreads, kAttnFwdSmem, st>>>(tmQ, tmK, tmV, reinterpret_cast<T*>(ctx),
                                                             reinterpret_cast<float*>(stats), p);
  }
  return check_launch();
}

constexpr size_t kAttnBwdSmem = 1024 + 6 * (size_t)kTileBytes + 1024 + 8 * 4096;

template <typename T>
static int attention_bwd_prep_run(uint64_t pp, uint64_t ds, uint64_t q, uint64_t k, uint64_t v, uint64_t dctx, uint64_t ctx,
                                  uint64_t stats, int batch, int seq, int heads, int head_dim, float alpha, cudaStream_t st) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  CUtensorMap tmQ, tmK, tmV, tmdO;
  int rc = encode_bshd(&tmQ, q, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmK, k, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmV, v, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmdO, dctx, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  // P and dS: [batch, seq, heads, seq] written as [32 rows][32 columns] boxes (64-byte rows, 64-byte swizzle)
  CUtensorMap tmP, tmdS;
  if (!rc) rc = encode_bshd(&tmP, pp, batch, seq, heads, seq, 32, 32, bf16, CU_TENSOR_MAP_SWIZZLE_64B);
  if (!rc) rc = encode_bshd(&tmdS, ds, batch, seq, heads, seq, 32, 32, bf16, CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc) return rc;
  AttnParams p;
  p.batch = batch; p.seq = seq; p.heads = heads; p.head_dim = head_dim; p.alpha = alpha;
  p.idesc_s = (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(128 >> 3) << 17) |
              ((uint32_t)(128 >> 4) << 24);
  p.idesc_pv = p.idesc_s;
  {
    const long long rows = (long long)batch * seq * heads;
    long long grid = (rows + 31) / 32;
    if (grid > (long long)kNumSMs * 16) grid = (long long)kNumSMs * 16;
    attention_rowdot_kernel<T><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<float*>(stats), reinterpret_cast<const T*>(ctx),
                                                               reinterpret_cast<const T*>(dctx), rows, seq, heads, head_dim);
    rc = check_launch();
    if (rc) return rc;
  }
  auto kern = attention_bwd_prep_kernel<T>;
  static bool attr_set[kMaxDevices] = {};
  ensure_dynamic_smem(kern, kAttnBwdSmem, attr_set);
  const long long grid = (long long)batch * heads * (seq / kAttnRows);
  kern<<<(unsigned)grid, kAttnThreads, kAttnBwdSmem, st>>>(tmQ, tmK, tmV, tmdO, tmP, tmdS,
                                                           reinterpret_cast<const T*>(ctx), reinterpret_cast<const T*>(dctx),
                                                           reinterpret_cast<const float*>(stats), p);
  return check_launch();
}

constexpr size_t kAttnBwdDqSmem = 1024 + 6 * (size_t)kTileBytes + 2 * (size_t)kUnitBytes + 256;
constexpr size_t kAttnBwdDkvSmem = 1024 + 2 * (size_t)kTileBytes + 8 * (size_t)kUnitBytes + 2 * kBwdCols * sizeof(float2) + 256;

template <typename T>
static int attention_bwd_run(uint64_t dq, uint64_t dk, uint64_t dv, uint64_t q, uint64_t k, uint64_t v, uint64_t dctx, uint64_t ctx,
                             uint64_t stats, int batch, int seq, int heads, int head_dim, float alpha, cudaStream_t st) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  CUtensorMap tmQ, tmK, tmV, tmdO, tmQ64, tmdO64;
  int rc = encode_bshd(&tmQ, q, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmK, k, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmV, v, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmdO, dctx, batch, seq, heads, kAttnHd, 64, kAttnRows, bf16);
  if (!rc) rc = encode_bshd(&tmQ64, q, batch, seq, heads, kAttnHd, 64, kBwdCols, bf16);
  if (!rc) rc = encode_bshd(&tmdO64, dctx, batch, seq, heads, kAttnHd, 64, kBwdCols, bf16);
  if (rc) return rc;
  AttnParams p;
  p.batch = batch; p.seq = seq; p.heads = heads; p.head_dim = head_dim; p.alpha = alpha;
  const uint32_t kind = (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(128 >> 4) << 24);
  p.idesc_s = kind | ((uint32_t)(kBwdCols >> 3) << 17);                  // 128 x 64, both operands K-major
  p.idesc_pv = kind | ((uint32_t)(128 >> 3) << 17) | (1u << 16);        // 128 x 128, B MN-major
  {
    const long long rows = (long long)batch * seq * heads;
    long long grid = (rows + 31) / 32;
    if (grid > (long long)kNumSMs * 16) grid = (long long)kNumSMs * 16;
    attention_rowdot_kernel<T><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<float*>(stats), reinterpret_cast<const T*>(ctx),
                                                               reinterpret_cast<const T*>(dctx), rows, seq, heads, head_dim);
    rc = check_launch();
    if (rc) return rc;
  }
  const long long grid = (long long)batch * heads * (seq / kAttnRows);
  {
    auto kern = attention_bwd_dkv_kernel<T>;
    static bool attr_set[kMaxDevices] = {};
    ensure_dynamic_smem(kern, kAttnBwdDkvSmem, attr_set);
    kern<<<(unsigned)grid, kAttnThreads, kAttnBwdDkvSmem, st>>>(tmQ64, tmK, tmV, tmdO64, reinterpret_cast<T*>(dk), reinterpret_cast<T*>(dv),
                                                                reinterpret_cast<const float*>(stats), p);
    rc = check_launch();
    if (rc) return rc;
  }
  auto kern = attention_bwd_dq_kernel<T>;
  static bool attr_set[kMaxDevices] = {};
  ensure_dynamic_smem(kern, kAttnBwdDqSmem, attr_set);
  kern<<<(unsigned)grid, kAttnThreads, kAttnBwdDqSmem, st>>>(tmQ, tmK, tmV, tmdO, reinterpret_cast<T*>(dq),
                                                             reinterpret_cast<const float*>(stats), p);
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
  // rows of whole blocks that are multiples of 16 bytes on both sides: staged copy (rows in by bulk copy, spread to the
  // padded pitch in shared memory, out by bulk store)
  if (cols > 0 && ncol > 0) {
    const int staged = pitched_rows_staged(false, dst, src, 0, 0, nrow * rows, ncol, cols, cols_pad, 1, 0, dtype, st);
    if (staged >= 0) return staged;
  }
  if (cols % 4 == 0 && cols_pad % 8 == 0 && dst % 16 == 0 && src % 8 == 0) {
    const long long total = groups * (cols_pad / 8);
    long long grid = (total + 255) / 256;
    if (grid > (long long)kNumSMs * 64) grid = (long long)kNumSMs * 64;
    block_pad_vec_kernel<<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint2*>(src),
                                                         groups, (int)(cols / 4), (int)(cols_pad / 8));
    return check_launch();
  }
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
  if (!ctx || !stats || !q || !k || !v || (q & 15) || (k & 15) || (v & 15) || (ctx & 7) || (stats & 15))
    return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == CACTI_B200_R_16F)
    return attention_fwd_run<__half>(ctx, stats, q, k, v, (int)batch, (int)seq, (int)heads, (int)head_dim, alpha, st);
  return attention_fwd_run<__nv_bfloat16>(ctx, stats, q, k, v, (int)batch, (int)seq, (int)heads, (int)head_dim, alpha, st);
}

int cacti_b200_attention_bwd(cacti_b200_dptr dq, cacti_b200_dptr dk, cacti_b200_dptr dv, cacti_b200_dptr q, cacti_b200_dptr k,
                             cacti_b200_dptr v, cacti_b200_dptr dctx, cacti_b200_dptr ctx, cacti_b200_dptr stats, int64_t batch,
                             int64_t seq, int64_t heads, int64_t head_dim, float alpha, int dtype, cacti_b200_stream stream) {
  using namespace cb;
  if (batch < 0 || seq < 0 || heads < 0 || head_dim <= 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (head_dim > kAttnHd || head_dim % 4 || seq % kAttnRows || batch * heads * (seq / kAttnRows) > 0x7fffffffLL)
    return CACTI_B200_ERR_SHAPE;
  if (batch == 0 || seq == 0 || heads == 0) return CACTI_B200_OK;
  if (!dq || !dk || !dv || !q || !k || !v || !dctx || !ctx || !stats || ((q | k | v | dctx) & 15) || ((dq | dk | dv | ctx) & 7) ||
      (stats & 15))
    return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == CACTI_B200_R_16F)
    return attention_bwd_run<__half>(dq, dk, dv, q, k, v, dctx, ctx, stats, (int)batch, (int)seq, (int)heads, (int)head_dim, alpha, st);
  return attention_bwd_run<__nv_bfloat16>(dq, dk, dv, q, k, v, dctx, ctx, stats, (int)batch, (int)seq, (int)heads, (int)head_dim, alpha,
                                          st);
}

int cacti_b200_attention_bwd_prep(cacti_b200_dptr p, cacti_b200_dptr ds, cacti_b200_dptr q, cacti_b200_dptr k,
                                  cacti_b200_dptr v, cacti_b200_dptr dctx, cacti_b200_dptr ctx, cacti_b200_dptr stats,
                                  int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, float alpha, int dtype,
                                  cacti_b200_stream stream) {
  using namespace cb;
  if (batch < 0 || seq < 0 || heads < 0 || head_dim <= 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (head_dim > kAttnHd || head_dim % 4 || seq % kAttnRows || batch * heads * (seq / kAttnRows) > 0x7fffffffLL)
    return CACTI_B200_ERR_SHAPE;
  if (batch == 0 || seq == 0 || heads == 0) return CACTI_B200_OK;
  if (!p || !ds || !q || !k || !v || !dctx || !ctx || !stats || ((p | ds | q | k | v | dctx) & 15) || (ctx & 7) || (stats & 7))
    return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == CACTI_B200_R_16F)
    return attention_bwd_prep_run<__half>(p, ds, q, k, v, dctx, ctx, stats, (int)batch, (int)seq, (int)heads, (int)head_dim,
                                          alpha, st);
  return attention_bwd_prep_run<__nv_bfloat16>(p, ds, q, k, v, dctx, ctx, stats, (int)batch, (int)seq, (int)heads,
                                               (int)head_dim, alpha, st);
}
}
