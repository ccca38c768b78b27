// K3: rotary position embedding, forward / backward / fused forward+backward, and its tables.
//
// Replaces symplectic_embed (src/librarium/llama.rs:463-465): BroadcastMul (x*cos) +
// InnerSymplecticMap (rotate-half, :975-1049) + BroadcastMul (rot*sin) + Add
// (src/thunk/op.rs:1480-1535) -- four programs and three full-size temporaries forward, two
// memcpys, two Futhark-vjp programs and an accumulate backward.  The backward does not depend on
// x: dx = dy*cos + R(dy*sin), so the fused form streams x and dy in and y and dx out.
//
// head_dim 100 makes a head 200 bytes, so heads are not 16-byte aligned; token rows
// (heads*head_dim elements) are.  Three kernels, chosen per call:
//  * rope_staged_kernel (16-byte aligned rows, Apply mode): whole token rows travel by bulk copies
//    into and out of shared memory, where (unit, partner) pairs are rotated in place;
//  * rope_vec_kernel (16-byte aligned rows, Accumulate mode): 16-byte vectors over the flat token
//    row; the rotate-half partner of each 4-byte unit (a half2 / bf162 / float) sits
//    +-head_dim/2 elements away and is fetched with a 4-byte load that hits lines the CTA already
//    streams;
//  * rope_generic_kernel: element-wise, any shape and alignment.
// All three give the same bits.
//
// f16 follows the reference's f16 arithmetic (both operands f16 => f16 ops, one rounding per
// primitive, src/thunk/op.rs:2126-2133) using the non-contracting *_rn intrinsics; f32 uses
// separately rounded f32 ops; bf16 (no reference chain: Futhark has no bf16) computes in f32 and
// rounds once.
#include "common.cuh"
#include <type_traits>

namespace cb {

int g_rope_threads = 256;
int g_rope_ctas_per_sm = 8;
int g_rope_staged = 1;             // 1: staged kernel where it applies; 0: vector kernel (measurement knob)
int g_rope_staged_g = 160;         // staged kernel: threads per row group
int g_rope_staged_groups = 2;      // staged kernel: row groups per CTA
int g_rope_staged_stages = 3;      // staged kernel: rows in the ring of a group

template <typename T> struct Unit;         // one 4-byte unit
template <> struct Unit<__half> { static constexpr int UPV = 2; };
template <> struct Unit<__nv_bfloat16> { static constexpr int UPV = 2; };
template <> struct Unit<float> { static constexpr int UPV = 1; };

// Division by a run-time constant as multiply-high + shift (round-up method), exact for dividends below 2^31.  The
// index arithmetic of the vector kernels (vector -> token -> position, offset inside the head) otherwise costs two
// emulated 64-bit divisions per 16-byte vector, which showed as issue-slot pressure in a kernel that should only wait
// on memory.
struct FastDiv { uint32_t d, magic, shift; };
static FastDiv make_fastdiv(uint32_t d) {
  FastDiv f; f.d = d; f.shift = 0;
  while ((1ull << f.shift) < d) ++f.shift;
  f.magic = (uint32_t)(((((1ull << f.shift) - d) << 32) / d) + 1);
  return f;
}
__device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv& f) { return (__umulhi(n, f.magic) + n) >> f.shift; }
__device__ __forceinline__ uint32_t fmod_(uint32_t n, const FastDiv& f) { return n - fdiv(n, f) * f.d; }

template <typename T> __device__ __forceinline__ uint32_t ldu(const T* p) {      // 4-byte aligned
  return __ldg(reinterpret_cast<const unsigned int*>(p));
}

// y = x*c + r*s with r = first ? -xp : xp   (forward)
// d = g*c + (first ? z : -z), z = gp*sp     (backward)
template <typename T>
__device__ __forceinline__ uint32_t rope_unit(uint32_t own, uint32_t partner, uint32_t c, uint32_t s_for_partner_term,
                                              bool first, bool backward) {
  if constexpr (std::is_same<T, __half>::value) {
    const __half2 o = *reinterpret_cast<__half2*>(&own), p = *reinterpret_cast<__half2*>(&partner);
    const __half2 cc = *reinterpret_cast<__half2*>(&c), ss = *reinterpret_cast<__half2*>(&s_for_partner_term);
    const __half2 a = __hmul2_rn(o, cc);
    __half2 b;
    if (!backward) b = __hmul2_rn(first ? __hneg2(p) : p, ss);
    else { b = __hmul2_rn(p, ss); if (!first) b = __hneg2(b); }
    const __half2 y = __hadd2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&y);
  } else if constexpr (std::is_same<T, float>::value) {
    const float o = __uint_as_float(own), p = __uint_as_float(partner);
    const float cc = __uint_as_float(c), ss = __uint_as_float(s_for_partner_term);
    const float a = __fmul_rn(o, cc);
    float b = __fmul_rn(p, ss);
    if (first != backward) b = -b;
    return __float_as_uint(__fadd_rn(a, b));
  } else {
    float r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float o = __uint_as_float(i ? (own & 0xffff0000u) : (own << 16));
      const float p = __uint_as_float(i ? (partner & 0xffff0000u) : (partner << 16));
      const float cc = __uint_as_float(i ? (c & 0xffff0000u) : (c << 16));
      const float ss = __uint_as_float(i ? (s_for_partner_term & 0xffff0000u) : (s_for_partner_term << 16));
      const float b = p * ss;
      r[i] = fmaf(o, cc, (first != backward) ? -b : b);
    }
    __nv_bfloat162 y = __floats2bfloat162_rn(r[0], r[1]);
    return *reinterpret_cast<const uint32_t*>(&y);
  }
}

// Accumulate mode: out = old + new in T.
template <typename T> __device__ __forceinline__ uint32_t add_unit(uint32_t old, uint32_t v) {
  if constexpr (std::is_same<T, __half>::value) {
    const __half2 y = __hadd2_rn(*reinterpret_cast<__half2*>(&old), *reinterpret_cast<__half2*>(&v));
    return *reinterpret_cast<const uint32_t*>(&y);
  } else if constexpr (std::is_same<T, float>::value) {
    return __float_as_uint(__fadd_rn(__uint_as_float(old), __uint_as_float(v)));
  } else {
    __nv_bfloat162 y = __floats2bfloat162_rn(__uint_as_float(old << 16) + __uint_as_float(v << 16),
                                              __uint_as_float(old & 0xffff0000u) + __uint_as_float(v & 0xffff0000u));
    return *reinterpret_cast<const uint32_t*>(&y);
  }
}

// I32: every index fits 31 bits, divisions go through FastDiv (fd_vpr, fd_hd, fd_pos); otherwise plain 64-bit division.
template <typename T, bool FWD, bool BWD, bool I32>
__global__ void __launch_bounds__(256)
rope_vec_kernel(T* __restrict__ Y, T* __restrict__ dX, const T* __restrict__ X, const T* __restrict__ dY,
                const T* __restrict__ cosT, const T* __restrict__ sinT, int64_t nvec, int vpr /* vectors per token row */,
                int hd, int64_t pos_mod, int64_t pos_off, int beta, FastDiv fd_vpr, FastDiv fd_hd, FastDiv fd_pos) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int UPV = Unit<T>::UPV;
  constexpr int NU = 4;                       // units per vector
  const int half = hd >> 1;
  // UNR vectors per thread per trip.  Measured on B200: 4 per trip lowered occupancy and ran slower; a per-token-row
  // variant that reused the table units across the batch and exchanged partners through shared memory was also
  // slower (86-119 us against 82 us at [16384, 32, 100]); a same-size device copy takes 71 us.
  constexpr int UNR = 1;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += UNR * stride) {
    uint4 xo[UNR], go[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t v = v0 + u * stride;
      if (v < nvec) {
        if (FWD) xo[u] = ld_stream(X + v * VEC);
        if (BWD) go[u] = ld_stream(dY + v * VEC);
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t v = v0 + u * stride;
      if (v >= nvec) break;
      int64_t pos;
      int r;                                               // element offset inside the token row
      int j;                                               // element offset inside the head
      if (I32) {
        const uint32_t tok = fdiv((uint32_t)v, fd_vpr);
        r = (int)((uint32_t)v - tok * (uint32_t)vpr) * VEC;
        pos = fmod_(tok + (uint32_t)pos_off, fd_pos);
        j = (int)fmod_((uint32_t)r, fd_hd);
      } else {
        const int64_t tok = v / vpr;
        r = (int)(v - tok * vpr) * VEC;
        pos = (tok + pos_off) % pos_mod;
        j = r % hd;
      }
      const int64_t e0 = v * VEC;                          // flat element index
      const T* ct = cosT + pos * hd;
      const T* stb = sinT + pos * hd;
      uint32_t yo[NU], dout[NU];
      const uint32_t xw[NU] = {xo[u].x, xo[u].y, xo[u].z, xo[u].w};
      const uint32_t gw[NU] = {go[u].x, go[u].y, go[u].z, go[u].w};
#pragma unroll
      for (int p = 0; p < NU; ++p) {
        if (j >= hd) j -= hd;
        const bool first = j < half;
        const int jp = first ? j + half : j - half;        // partner index inside the head
        const int64_t ep = e0 + p * UPV + (first ? half : -half);
        const uint32_t c = ldu(ct + j);
        if (FWD) yo[p] = rope_unit<T>(xw[p], ldu(X + ep), c, ldu(stb + j), first, false);
        if (BWD) dout[p] = rope_unit<T>(gw[p], ldu(dY + ep), c, ldu(stb + jp), first, true);
        j += UPV;
      }
      if (FWD) st_stream(Y + e0, make_uint4(yo[0], yo[1], yo[2], yo[3]));
      if (BWD) {
        if (beta) {
          const uint4 o = ld_stream(dX + e0);
          dout[0] = add_unit<T>(o.x, dout[0]); dout[1] = add_unit<T>(o.y, dout[1]);
          dout[2] = add_unit<T>(o.z, dout[2]); dout[3] = add_unit<T>(o.w, dout[3]);
        }
        st_stream(dX + e0, make_uint4(dout[0], dout[1], dout[2], dout[3]));
      }
    }
  }
}

// Staged form of the fused kernel, for 16-byte aligned token rows.  A group of G threads owns one token row at a
// time: the x row and the dy row arrive in shared memory by bulk copies behind an mbarrier (a ring of rows per
// group, so the next rows are in flight while one is computed); each thread rotates (head, unit) pairs in place --
// consecutive threads take consecutive 4-byte units, so every shared-memory access of a warp is conflict-free, and
// a pair is read and written by one thread only -- and the finished rows leave by bulk stores from the same
// buffer.  The load/store units then carry only the table loads; global memory traffic is moved by the copy engine.
// A slot is refilled one row late, once the bulk store that read it has finished reading.

template <typename T, bool FWD, bool BWD>
__global__ void __launch_bounds__(512)
rope_staged_kernel(T* __restrict__ Y, T* __restrict__ dX, const T* __restrict__ X, const T* __restrict__ dY,
                   const T* __restrict__ cosT, const T* __restrict__ sinT, int64_t tokens, int row_len, int hd,
                   int items, FastDiv fd_uh, int G, int nstages, int64_t pos_mod, int64_t pos_off) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int UPV = Unit<T>::UPV;
  const int groups = blockDim.x / G;
  const int gid = threadIdx.x / G, lane = threadIdx.x - gid * G;
  const unsigned row_bytes = (unsigned)row_len * sizeof(T);
  const unsigned stage_bytes = row_bytes * ((FWD && BWD) ? 2 : 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)groups * nstages * stage_bytes);
  unsigned char* stage0 = smem_raw + (size_t)gid * nstages * stage_bytes;
  uint64_t* bar0 = bars + gid * nstages;
  if (lane < nstages) mbar_init(bar0 + lane, 1);
  mbar_fence_init();
  __syncthreads();
  const int half = hd >> 1;
  const int64_t stride = (int64_t)gridDim.x * groups;
  const int64_t row0 = (int64_t)blockIdx.x * groups + gid;
  const int64_t pstep = stride % pos_mod;
  int64_t pos = (row0 + pos_off) % pos_mod;

  auto issue = [&](int64_t r, int sl) {       // lane 0 only
    unsigned char* dst = stage0 + (size_t)sl * stage_bytes;
    mbar_expect_tx(bar0 + sl, stage_bytes);
    if (FWD) bulk_g2s(dst, X + r * row_len, row_bytes, bar0 + sl);
    if (BWD) bulk_g2s(dst + (FWD ? row_bytes : 0), dY + r * row_len, row_bytes, bar0 + sl);
  };
  if (lane == 0)
    for (int sl = 0; sl < nstages; ++sl)
      if (row0 + sl * stride < tokens) issue(row0 + sl * stride, sl);

  int slot = 0;
  unsigned phase = 0;
  int prev_slot = -1;
  int64_t prev_row = 0;
  for (int64_t row = row0; row < tokens; row += stride) {
    const bool gave_up = !mbar_wait_bounded(bar0 + slot, phase, kDevErrStageTimeout);
    T* sx = reinterpret_cast<T*>(stage0 + (size_t)slot * stage_bytes);
    T* sg = reinterpret_cast<T*>(stage0 + (size_t)slot * stage_bytes + (FWD ? row_bytes : 0));
    const T* ct = cosT + pos * hd;
    const T* stb = sinT + pos * hd;
#pragma unroll 5
    for (int n = lane; n < items; n += G) {
      const uint32_t h = fdiv((uint32_t)n, fd_uh);
      const int i = (int)((uint32_t)n - h * fd_uh.d) * UPV;          // element offset inside the half head
      const int e = (int)h * hd + i;                                 // element offset inside the token row
      const uint32_t c1 = ldu(ct + i), c2 = ldu(ct + i + half), s1 = ldu(stb + i), s2 = ldu(stb + i + half);
      if (FWD) {
        uint32_t* p1 = reinterpret_cast<uint32_t*>(sx + e);
        uint32_t* p2 = reinterpret_cast<uint32_t*>(sx + e + half);
        const uint32_t x1 = *p1, x2 = *p2;
        *p1 = rope_unit<T>(x1, x2, c1, s1, true, false);
        *p2 = rope_unit<T>(x2, x1, c2, s2, false, false);
      }
      if (BWD) {
        uint32_t* p1 = reinterpret_cast<uint32_t*>(sg + e);
        uint32_t* p2 = reinterpret_cast<uint32_t*>(sg + e + half);
        const uint32_t g1 = *p1, g2 = *p2;
        *p1 = rope_unit<T>(g1, g2, c1, s2, true, true);
        *p2 = rope_unit<T>(g2, g1, c2, s1, false, true);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the bulk store reads what was just written
    // the group's barrier also carries the vote on a wait that ran out: the group stops together, nothing is stored
    {
      GroupCtx gc; gc.G = G; gc.gid = gid;
      if (group_any(gc, gave_up)) break;
    }
    if (lane == 0) {
      if (FWD) bulk_s2g(Y + row * row_len, sx, row_bytes);
      if (BWD) bulk_s2g(dX + row * row_len, sg, row_bytes);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      if (prev_slot >= 0) {
        // the store of the previous row has finished reading its slot: refill it
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        const int64_t next = prev_row + (int64_t)nstages * stride;
        if (next < tokens) issue(next, prev_slot);
      }
    }
    prev_slot = slot; prev_row = row;
    if (++slot == nstages) { slot = 0; phase ^= 1; }
    pos += pstep;
    if (pos >= pos_mod) pos -= pos_mod;
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory stays valid until read
}

// Staged form of the head-pitched forward (below), for 16-byte aligned token rows: the x row arrives by a bulk copy;
// each thread rotates (head, unit) pairs as in rope_staged_kernel but writes them straight to their place in an output
// row of `pitch` elements per head (the zeros after head_dim are written once, before the first row) in a second
// shared-memory buffer, and the padded row leaves by one bulk store.  Two output buffers per group: a buffer is written
// again two rows later, after the store that read it has finished reading.  Same bits as the per-thread kernel.
// ROTATE = false: the copy alone (8 bytes per thread and step), which is block_pad on rows of whole heads.
template <typename T, bool ROTATE>
__global__ void __launch_bounds__(512)
rope_pitched_staged_kernel(T* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ cosT, const T* __restrict__ sinT,
                           int64_t tokens, int row_len, int hd, int pitch, int items, FastDiv fd_uh, FastDiv fd_iu, int G,
                           int nstages, int64_t pos_mod, int64_t pos_off) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int UPV = Unit<T>::UPV;
  const int groups = blockDim.x / G;
  const int gid = threadIdx.x / G, lane = threadIdx.x - gid * G;
  const int heads = row_len / hd;
  const unsigned row_bytes = (unsigned)row_len * sizeof(T);
  const unsigned out_bytes = (unsigned)heads * (unsigned)pitch * sizeof(T);
  const size_t per_group = (size_t)nstages * row_bytes + 2 * (size_t)out_bytes;
  unsigned char* stage0 = smem_raw + (size_t)gid * per_group;
  unsigned char* out0 = stage0 + (size_t)nstages * row_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)groups * per_group);
  uint64_t* bar0 = bars + gid * nstages;
  if (lane < nstages) mbar_init(bar0 + lane, 1);
  mbar_fence_init();
  __syncthreads();
  const int half = hd >> 1;
  const int64_t stride = (int64_t)gridDim.x * groups;
  const int64_t row0 = (int64_t)blockIdx.x * groups + gid;
  const int64_t pstep = stride % pos_mod;
  int64_t pos = (row0 + pos_off) % pos_mod;
  const int in_u8 = hd >> 2, out_u8 = pitch >> 2;        // 8-byte units per head, stored and pitched
  const int out_units = heads * out_u8;
  GroupCtx gc; gc.G = G; gc.gid = gid;

  auto issue = [&](int64_t r, int sl) {       // lane 0 only
    mbar_expect_tx(bar0 + sl, row_bytes);
    bulk_g2s(stage0 + (size_t)sl * row_bytes, X + r * row_len, row_bytes, bar0 + sl);
  };
  if (lane == 0)
    for (int sl = 0; sl < nstages; ++sl)
      if (row0 + sl * stride < tokens) issue(row0 + sl * stride, sl);

  // the zeros after head_dim never change: write them once into both output buffers
  {
    const int tail_u8 = out_u8 - in_u8;
    for (int u = lane; u < 2 * heads * tail_u8; u += G) {
      const int bh = u / tail_u8;                              // buffer * heads + head
      const int k = u - bh * tail_u8;
      reinterpret_cast<uint2*>(out0)[(size_t)bh * out_u8 + in_u8 + k] = make_uint2(0u, 0u);
    }
  }
  group_barrier(gc);

  int slot = 0;
  unsigned phase = 0, it = 0;
  for (int64_t row = row0; row < tokens; row += stride, ++it) {
    const bool gave_up = !mbar_wait_bounded(bar0 + slot, phase, kDevErrStageTimeout);
    const T* sx = reinterpret_cast<const T*>(stage0 + (size_t)slot * row_bytes);
    // this row's output buffer is free: lane 0 saw the store that read it finish before the previous row's barrier
    unsigned char* ob = out0 + (size_t)(it & 1) * out_bytes;
    if (ROTATE) {
      // rotated pairs go straight to their pitched place: no pass of their own for the spreading
      T* so = reinterpret_cast<T*>(ob);
      const T* ct = cosT + pos * hd;
      const T* stb = sinT + pos * hd;
#pragma unroll 5
      for (int n = lane; n < items; n += G) {
        const uint32_t h = fdiv((uint32_t)n, fd_uh);
        const int i = (int)((uint32_t)n - h * fd_uh.d) * UPV;
        const int e = (int)h * hd + i;
        const int o = (int)h * pitch + i;
        const uint32_t c1 = ldu(ct + i), c2 = ldu(ct + i + half), s1 = ldu(stb + i), s2 = ldu(stb + i + half);
        const uint32_t x1 = *reinterpret_cast<const uint32_t*>(sx + e);
        const uint32_t x2 = *reinterpret_cast<const uint32_t*>(sx + e + half);
        *reinterpret_cast<uint32_t*>(so + o) = rope_unit<T>(x1, x2, c1, s1, true, false);
        *reinterpret_cast<uint32_t*>(so + o + half) = rope_unit<T>(x2, x1, c2, s2, false, false);
      }
    } else {
      const uint2* in8 = reinterpret_cast<const uint2*>(sx);
      uint2* out8 = reinterpret_cast<uint2*>(ob);
      const int in_units = heads * in_u8;
#pragma unroll 5
      for (int u = lane; u < in_units; u += G) {
        const uint32_t h = fdiv((uint32_t)u, fd_iu);             // 8-byte units per stored head
        out8[u + (int)h * (out_u8 - in_u8)] = in8[u];
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the bulk store reads what was just written
    // the store of the previous row has read the other buffer: the next row may fill it right after this barrier
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    // one barrier per row: output row complete, input slot read by every lane, and the vote on a wait that ran out
    // (the group stops together, nothing is stored)
    if (group_any(gc, gave_up)) break;
    if (lane == 0) {
      bulk_s2g(Y + row * (int64_t)heads * pitch, ob, out_bytes);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      const int64_t next = row + (int64_t)nstages * stride;
      if (next < tokens) issue(next, slot);
    }
    if (++slot == nstages) { slot = 0; phase ^= 1; }
    pos += pstep;
    if (pos >= pos_mod) pos -= pos_mod;
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory stays valid until read
}

// Forward RoPE whose output rows are head-pitched: y[tok][h][0 .. pitch) with the head's head_dim rotated values
// followed by zeros, the layout cacti_b200_block_pad would produce from the packed result (the fused attention reads
// q and k that way).  One thread per 8-byte unit of the output; 16-bit types only (two 4-byte rope units per thread).
template <typename T>
__global__ void __launch_bounds__(256)
rope_fwd_pitched_kernel(T* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ cosT, const T* __restrict__ sinT,
                        int64_t units /* tokens * heads * pitch / 4 */, int heads, int hd, int pitch, int64_t pos_mod,
                        int64_t pos_off) {
  const int upr = pitch >> 2, half = hd >> 1;
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (int64_t)gridDim.x * blockDim.x) {
    const int64_t th = u / upr;                   // token * heads + head
    const int d = (int)(u - th * upr) * 4;        // first element of this unit inside the head
    uint2 out = make_uint2(0, 0);
    if (d < hd) {
      const int64_t tok = th / heads;
      const int64_t pos = (tok + pos_off) % pos_mod;
      const T* xh = X + th * hd;
      const T* ct = cosT + pos * hd;
      const T* stb = sinT + pos * hd;
      uint32_t w[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int j = d + 2 * q;
        const bool first = j < half;
        w[q] = rope_unit<T>(ldu(xh + j), ldu(xh + (first ? j + half : j - half)), ldu(ct + j), ldu(stb + j), first, false);
      }
      out = make_uint2(w[0], w[1]);
    }
    *reinterpret_cast<uint2*>(Y + u * 4) = out;     // plain store: the attention kernel reads it next, from L2
  }
}

// Element-wise fallback for shapes/alignments the vector kernel does not take (head_dim not a
// multiple of 4 for 16-bit types, token rows not a multiple of 16 bytes, unaligned views).
template <typename T> __device__ __forceinline__ T rope_scalar(T own, T partner, T c, T s, bool first, bool backward) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const float b = __bfloat162float(partner) * __bfloat162float(s);
    return __float2bfloat16_rn(fmaf(__bfloat162float(own), __bfloat162float(c), (first != backward) ? -b : b));
  } else {
    const float a = round_to<T>(Elem<T>::to_f32(own) * Elem<T>::to_f32(c));     // exact product, one rounding
    float b = round_to<T>(Elem<T>::to_f32(partner) * Elem<T>::to_f32(s));
    if (first != backward) b = -b;
    return Elem<T>::from_f32(__fadd_rn(a, b));
  }
}

template <typename T, bool FWD, bool BWD>
__global__ void __launch_bounds__(256)
rope_generic_kernel(T* __restrict__ Y, T* __restrict__ dX, const T* __restrict__ X, const T* __restrict__ dY,
                    const T* __restrict__ cosT, const T* __restrict__ sinT, int64_t n, int64_t row_len, int hd,
                    int64_t pos_mod, int64_t pos_off, int beta) {
  const int half = hd >> 1;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t tok = e / row_len;
    const int j = (int)((e - tok * row_len) % hd);
    const int64_t pos = (tok + pos_off) % pos_mod;
    const bool first = j < half;
    const int jp = first ? j + half : j - half;
    const int64_t ep = e + (jp - j);
    const T c = cosT[pos * hd + j];
    if (FWD) Y[e] = rope_scalar<T>(X[e], X[ep], c, sinT[pos * hd + j], first, false);
    if (BWD) {
      T d = rope_scalar<T>(dY[e], dY[ep], c, sinT[pos * hd + jp], first, true);
      if (beta) d = Elem<T>::from_f32(Elem<T>::to_f32(dX[e]) + Elem<T>::to_f32(d));
      dX[e] = d;
    }
  }
}

template <typename T>
__global__ void rope_tables_kernel(T* __restrict__ cosT, T* __restrict__ sinT, int64_t seq, int hd, float theta,
                                   float exp_scale) {
  const int half = hd >> 1;
  const int64_t n = seq * half;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = t / half;
    const int i = (int)(t - p * half);
    const float e = __fmul_rn((float)i, exp_scale);      // f32(i) * (-2/hd)
    const float w = powf(theta, e);
    const float phi = __fmul_rn((float)p, w);
    const T c = Elem<T>::from_f32(cosf(phi)), s = Elem<T>::from_f32(sinf(phi));
    cosT[p * hd + i] = c; cosT[p * hd + i + half] = c;
    sinT[p * hd + i] = s; sinT[p * hd + i + half] = s;
  }
}

template <typename T, bool FWD, bool BWD>
static int launch_rope(uint64_t y, uint64_t dx, uint64_t x, uint64_t dy, uint64_t c, uint64_t s, int64_t tokens,
                       int64_t heads, int64_t hd, int64_t pos_mod, int64_t pos_off, int beta, cudaStream_t st) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int UPV = Unit<T>::UPV;
  T* Y = reinterpret_cast<T*>(y); T* dX = reinterpret_cast<T*>(dx);
  const T* X = reinterpret_cast<const T*>(x); const T* dY = reinterpret_cast<const T*>(dy);
  const T* C = reinterpret_cast<const T*>(c); const T* S = reinterpret_cast<const T*>(s);
  const int64_t row_len = heads * hd, n = tokens * row_len;
  const bool vec_ok = (row_len % VEC == 0) && (hd % (2 * UPV) == 0) && hd >= VEC && (c % 4 == 0) && (s % 4 == 0) &&
                      (!FWD || (aligned16(x) && aligned16(y))) && (!BWD || (aligned16(dy) && aligned16(dx))) &&
                      row_len / VEC <= 0x7fffffffLL;
  const int threads = g_rope_threads;
  const int64_t units_half = (hd / 2) / UPV;
  const int64_t items = heads * units_half;
  const bool staged_ok = g_rope_staged && vec_ok && !beta && items <= 0x7fffffffLL && row_len <= 0x3fffffffLL &&
                         ((c | s) % 4 == 0);
  if (staged_ok) {
    int G = g_rope_staged_g;
    if (G > items) G = (int)((items + 31) / 32 * 32);
    int groups = g_rope_staged_groups;
    if (G * groups > 512) groups = 512 / G;
    if (groups > kMaxGroupsPerCta) groups = kMaxGroupsPerCta;
    const size_t stage = (size_t)row_len * sizeof(T) * ((FWD && BWD) ? 2 : 1);
    int nst = g_rope_staged_stages;
    auto smem_for = [&](int ns) { return (size_t)groups * ns * (stage + sizeof(uint64_t)); };
    while (nst > 2 && smem_for(nst) > kMaxDynSmem) --nst;
    while (groups > 1 && smem_for(nst) > kMaxDynSmem) --groups;
    const size_t smem = smem_for(nst);
    if (groups >= 1 && smem <= kMaxDynSmem && G <= 512) {
      auto kern = rope_staged_kernel<T, FWD, BWD>;
      const int threads_s = G * groups;
      int64_t grid = (int64_t)kNumSMs * resident_ctas(kern, threads_s, smem);
      const int64_t want = (tokens + groups - 1) / groups;
      if (grid > want) grid = want;
      kern<<<(unsigned)grid, threads_s, smem, st>>>(Y, dX, X, dY, C, S, tokens, (int)row_len, (int)hd, (int)items,
                                                   make_fastdiv((uint32_t)units_half), G, nst, pos_mod, pos_off);
      return check_launch();
    }
  }
  if (vec_ok) {
    const int64_t nvec = n / VEC;
    int64_t grid = (nvec + threads - 1) / threads;
    const int64_t cap = (int64_t)kNumSMs * g_rope_ctas_per_sm;
    if (grid > cap) grid = cap;
    const int vpr = (int)(row_len / VEC);
    const bool i32 = nvec < 0x7fffffffLL && pos_mod < 0x7fffffffLL && tokens + pos_off < 0x7fffffffLL;
    if (i32)
      rope_vec_kernel<T, FWD, BWD, true><<<(unsigned)grid, threads, 0, st>>>(
          Y, dX, X, dY, C, S, nvec, vpr, (int)hd, pos_mod, pos_off, beta, make_fastdiv((uint32_t)vpr),
          make_fastdiv((uint32_t)hd), make_fastdiv((uint32_t)pos_mod));
    else
      rope_vec_kernel<T, FWD, BWD, false><<<(unsigned)grid, threads, 0, st>>>(
          Y, dX, X, dY, C, S, nvec, vpr, (int)hd, pos_mod, pos_off, beta, FastDiv{}, FastDiv{}, FastDiv{});
    return check_launch();
  }
  int64_t grid = (n + threads - 1) / threads;
  const int64_t cap = (int64_t)kNumSMs * 16;
  if (grid > cap) grid = cap;
  rope_generic_kernel<T, FWD, BWD><<<(unsigned)grid, threads, 0, st>>>(Y, dX, X, dY, C, S, n, row_len, (int)hd,
                                                                      pos_mod, pos_off, beta);
  return check_launch();
}

static int rope_entry(bool fwd, bool bwd, uint64_t y, uint64_t dx, uint64_t x, uint64_t dy, uint64_t c, uint64_t s,
                      int64_t tokens, int64_t heads, int64_t hd, int64_t pos_mod, int64_t pos_off, int dtype, int beta,
                      void* stream) {
  if (tokens < 0 || heads < 0 || hd < 0 || hd > 0x3fffffffLL) return CACTI_B200_ERR_INVALID_VALUE;
  if (beta & ~1) return CACTI_B200_ERR_INVALID_VALUE;
  if (tokens == 0 || heads == 0 || hd == 0) return CACTI_B200_OK;
  if (hd & 1) return CACTI_B200_ERR_SHAPE;     // rotate-half splits the head in two equal parts
  if (pos_mod <= 0 || pos_off < 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (!c || !s || (fwd && (!x || !y)) || (bwd && (!dy || !dx))) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    if (fwd && bwd) return launch_rope<T, true, true>(y, dx, x, dy, c, s, tokens, heads, hd, pos_mod, pos_off, beta, st);
    if (fwd) return launch_rope<T, true, false>(y, dx, x, dy, c, s, tokens, heads, hd, pos_mod, pos_off, beta, st);
    return launch_rope<T, false, true>(y, dx, x, dy, c, s, tokens, heads, hd, pos_mod, pos_off, beta, st);
  });
}

}  // namespace cb

namespace cb {
// Launches rope_pitched_staged_kernel when the shape allows it (16-byte aligned rows on both sides, head and pitch in
// whole 8-byte units); returns -1 when it does not, else the launch's return code.  rotate = false: the padded copy
// alone (cos, sin unused).
int pitched_rows_staged(bool rotate, uint64_t y, uint64_t x, uint64_t cos, uint64_t sin, int64_t n_tokens, int64_t heads,
                        int64_t head_dim, int64_t head_pitch, int64_t pos_mod, int64_t pos_offset, int dtype, cudaStream_t st) {
  const int64_t row_len = heads * head_dim;
  if (!g_rope_staged || head_dim <= 0 || (head_dim & 3) || (head_pitch & 3) || (x & 15) || (y & 15) || (row_len * 2) % 16 ||
      (heads * head_pitch * 2) % 16 || row_len > 0x3fffffffLL || heads * head_pitch > 0x3fffffffLL)
    return -1;
  const int64_t items = heads * ((head_dim / 2) / 2);
  int G = g_rope_staged_g;
  if (G > items) G = (int)((items + 31) / 32 * 32);
  int groups = g_rope_staged_groups;
  if (G * groups > 512) groups = 512 / G;
  if (groups > kMaxGroupsPerCta) groups = kMaxGroupsPerCta;
  int nst = g_rope_staged_stages;
  auto smem_for = [&](int gr, int ns) {
    return (size_t)gr * ((size_t)ns * row_len * 2 + 2 * (size_t)heads * head_pitch * 2 + (size_t)ns * sizeof(uint64_t));
  };
  while (nst > 2 && smem_for(groups, nst) > kMaxDynSmem) --nst;
  while (groups > 1 && smem_for(groups, nst) > kMaxDynSmem) --groups;
  const size_t smem = smem_for(groups, nst);
  if (G < 32 || G > 512 || smem > kMaxDynSmem) return -1;
  const int threads_s = G * groups;
  const int64_t want = (n_tokens + groups - 1) / groups;
#define CB_ROPE_PITCHED(T_, R_)                                                                                               \
  do {                                                                                                                        \
    auto kern = rope_pitched_staged_kernel<T_, R_>;                                                                           \
    int64_t grid_s = (int64_t)kNumSMs * resident_ctas(kern, threads_s, smem);                                                 \
    if (grid_s > want) grid_s = want;                                                                                         \
    kern<<<(unsigned)grid_s, threads_s, smem, st>>>(reinterpret_cast<T_*>(y), reinterpret_cast<const T_*>(x),                 \
        reinterpret_cast<const T_*>(cos), reinterpret_cast<const T_*>(sin), n_tokens, (int)row_len, (int)head_dim,            \
        (int)head_pitch, (int)items, make_fastdiv((uint32_t)((head_dim / 2) / 2)), make_fastdiv((uint32_t)(head_dim / 4)),  \
        G, nst, pos_mod, pos_offset);                                                                                         \
  } while (0)
  if (dtype == CACTI_B200_R_16F) { if (rotate) CB_ROPE_PITCHED(__half, true); else CB_ROPE_PITCHED(__half, false); }
  else { if (rotate) CB_ROPE_PITCHED(__nv_bfloat16, true); else CB_ROPE_PITCHED(__nv_bfloat16, false); }
#undef CB_ROPE_PITCHED
  return check_launch();
}
}  // namespace cb

extern "C" {
int cacti_b200_rope_tables(cacti_b200_dptr cos, cacti_b200_dptr sin, int64_t seq, int64_t head_dim, float theta,
                           int dtype, cacti_b200_stream stream) {
  using namespace cb;
  if (seq < 0 || head_dim < 0 || head_dim > 0x3fffffffLL) return CACTI_B200_ERR_INVALID_VALUE;
  if (seq == 0 || head_dim == 0) return CACTI_B200_OK;
  if (head_dim & 1) return CACTI_B200_ERR_SHAPE;
  if (!cos || !sin) return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float exp_scale = -2.0f / (float)head_dim;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    const int64_t n = seq * (head_dim / 2);
    int64_t grid = (n + 255) / 256;
    if (grid > kNumSMs * 8) grid = kNumSMs * 8;
    rope_tables_kernel<T><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<T*>(cos), reinterpret_cast<T*>(sin), seq,
                                                         (int)head_dim, theta, exp_scale);
    return check_launch();
  });
}
int cacti_b200_rope_fwd(cacti_b200_dptr y, cacti_b200_dptr x, cacti_b200_dptr cos, cacti_b200_dptr sin, int64_t tokens,
                        int64_t heads, int64_t head_dim, int64_t pos_mod, int64_t pos_off, int dtype,
                        cacti_b200_stream stream) {
  return cb::rope_entry(true, false, y, 0, x, 0, cos, sin, tokens, heads, head_dim, pos_mod, pos_off, dtype, 0, stream);
}
int cacti_b200_rope_bwd(cacti_b200_dptr dx, cacti_b200_dptr dy, cacti_b200_dptr cos, cacti_b200_dptr sin, int64_t tokens,
                        int64_t heads, int64_t head_dim, int64_t pos_mod, int64_t pos_off, int dtype, int beta_dx,
                        cacti_b200_stream stream) {
  return cb::rope_entry(false, true, 0, dx, 0, dy, cos, sin, tokens, heads, head_dim, pos_mod, pos_off, dtype, beta_dx,
                        stream);
}
int cacti_b200_rope_fwd_bwd(cacti_b200_dptr y, cacti_b200_dptr dx, cacti_b200_dptr x, cacti_b200_dptr dy,
                            cacti_b200_dptr cos, cacti_b200_dptr sin, int64_t tokens, int64_t heads, int64_t head_dim,
                            int64_t pos_mod, int64_t pos_off, int dtype, int beta_dx, cacti_b200_stream stream) {
  return cb::rope_entry(true, true, y, dx, x, dy, cos, sin, tokens, heads, head_dim, pos_mod, pos_off, dtype, beta_dx,
                        stream);
}
int cacti_b200_rope_fwd_pitched(cacti_b200_dptr y, cacti_b200_dptr x, cacti_b200_dptr cos, cacti_b200_dptr sin,
                                int64_t n_tokens, int64_t heads, int64_t head_dim, int64_t head_pitch, int64_t pos_mod,
                                int64_t pos_offset, int dtype, cacti_b200_stream stream) {
  using namespace cb;
  if (n_tokens < 0 || heads < 0 || head_dim < 0 || head_pitch < head_dim || head_pitch > 0x3fffffffLL)
    return CACTI_B200_ERR_INVALID_VALUE;
  if (dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (n_tokens == 0 || heads == 0 || head_pitch == 0) return CACTI_B200_OK;
  // 8-byte units: the head and its half must be multiples of 4 and 2 elements
  if ((head_dim & 3) || (head_pitch & 3) || heads > 0x7fffffffLL) return CACTI_B200_ERR_SHAPE;
  if (pos_mod <= 0 || pos_offset < 0) return CACTI_B200_ERR_INVALID_VALUE;
  if (!y || (head_dim > 0 && (!x || !cos || !sin)) || (y & 7) || (x & 3) || (cos & 3) || (sin & 3))
    return CACTI_B200_ERR_INVALID_VALUE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int staged = pitched_rows_staged(true, y, x, cos, sin, n_tokens, heads, head_dim, head_pitch, pos_mod, pos_offset, dtype, st);
  if (staged >= 0) return staged;
  const int64_t units = n_tokens * heads * (head_pitch / 4);
  int64_t grid = (units + 255) / 256;
  if (grid > (int64_t)kNumSMs * 32) grid = (int64_t)kNumSMs * 32;
  if (dtype == CACTI_B200_R_16F)
    rope_fwd_pitched_kernel<__half><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<__half*>(y), reinterpret_cast<const __half*>(x),
        reinterpret_cast<const __half*>(cos), reinterpret_cast<const __half*>(sin), units, (int)heads, (int)head_dim,
        (int)head_pitch, pos_mod, pos_offset);
  else
    rope_fwd_pitched_kernel<__nv_bfloat16><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(y),
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(cos),
        reinterpret_cast<const __nv_bfloat16*>(sin), units, (int)heads, (int)head_dim, (int)head_pitch, pos_mod, pos_offset);
  return check_launch();
}
}
