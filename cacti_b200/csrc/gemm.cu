// G1 / G2: dense and block (strided-batched) matmul on the 5th-generation tensor cores.
//
// Replaces MatrixMulF16F32GpuThunkImpl (cublasGemmEx, src/thunk/op.rs:4413-4716) and
// BlockMatrixMulF16F32GpuThunkImpl (cublasGemmBatchedEx over host-built pointer arrays,
// src/thunk/op.rs:5025-5471): C = f16(alpha * op(A) op(B) + beta * C), 16-bit operands, fp32
// accumulation, no split-K and no atomics (cacti_gpu_cu_ffi/src/lib.rs:749,766-767), row-major with
// leading dimensions, all four transpose combinations (src/thunk/op.rs:4336-4365, :4883-4911).
// The block form addresses block (i, j) by two affine strides per operand, which is what the
// reference computes on the host for its pointer arrays (src/thunk/op.rs:5174-5189); a stride of 0
// broadcasts the block.
//
// Kernel: one persistent CTA per SM, 192 threads.
//   warp 0      : TMA producer.  Operand tiles are fetched with cp.async.bulk.tensor (4-D tensor maps:
//                 inner, outer, block j, block i) into a ring of 128-byte-swizzled shared-memory stages;
//                 out-of-range rows/columns/K are zero-filled by the TMA unit.
//   warp 1      : allocates TMEM and issues tcgen05.mma (UMMA 128 x BN x 16, kind::f16) from one thread;
//                 tcgen05.commit releases shared-memory stages and publishes finished accumulators.
//   warps 2..5  : epilogue.  tcgen05.ld brings the fp32 accumulator out of TMEM, alpha/beta are applied,
//                 the result is rounded once to the 16-bit type and stored.
// Two accumulators (2 x BN of the 512 TMEM columns) let the epilogue of one tile overlap the main
// loop of the next.  Operands may be K-major or MN-major in memory; the transpose flags only change
// the tensor-map box and the "major" bits of the descriptors, never the data.  No load uses cluster
// multicast.  Every wait is bounded; on a timeout the CTA records kDevErrGemmTimeout, drains, frees
// its TMEM and returns.
//
// Operands that TMA cannot address (base or a stride not a multiple of 16 bytes, e.g. head_dim 100
// slices at 200-byte offsets) are first repacked into the caller's workspace with the inner
// dimension zero-padded to a multiple of 64 elements; the reference pads the same operands to 16 bytes
// with a separate thunk before calling cuBLAS (src/op.rs:1454-1482).  Outputs need no alignment.
#include "tc_common.cuh"
#include <atomic>
#include <type_traits>

namespace cb {

constexpr int kBM = 128, kBK = 64;
constexpr int kGemmThreads = 192;

struct GemmParams {
  int M, N, K;
  int nb_inner, nb_outer;                 // block grid: j (inner) and i (outer)
  int tiles_m, tiles_n;
  int a_j, a_i, b_j, b_i;                 // 1: operand has that block dimension, 0: broadcast
  long long ldc, c_stride_inner, c_stride_outer;
  float alpha, beta;
  uint32_t idesc;
  int c_align;                            // bytes every output row chunk is aligned to: 16, 8, 4 or 2
  int c_tma;                              // 1: C is written with TMA stores from a swizzled staging buffer
  int group_m;                            // tile rasterisation: m-tiles per group (L2 reuse of the B panel)
  int tri, diag;                          // triangular-structure hint (CACTI_B200_TRI_*) and its diagonal offset
  // k-split schedule of the two-SM kernel (see WorkIter); sk_tiles == 0: every tile is computed whole
  long long sk_tiles, sk_units;           // tiles [0, sk_tiles) are shared out in k-blocks: sk_units = sk_tiles * k-blocks
  float* sk_part;                         // [workers][2 CTAs][256 columns][128 rows] f32 partial accumulators
  int sk_slot;                            // which row of g_sk_flags this launch signals through
  int dyn;                                // 1: tiles beyond a worker's first come from g_tile_next[sk_slot] (dynamic schedule)
};

// ---- k-split ("stream-K") schedule ------------------------------------------------------------------------------
// A persistent grid of W workers over T tiles runs ceil(T / W) waves; when T is not a multiple of W the last wave is
// partly idle (104 tiles on 74 SM pairs: 2 waves for 1.4 waves of work).  Here the first sk_tiles tiles are treated
// as one run of sk_tiles * nkb k-blocks that is cut into W equal consecutive ranges; worker w computes range w and
// then whole tiles sk_tiles + w, sk_tiles + w + W, ...  A range starts inside at most one tile.  That first piece is
// a *contribution*: its f32 accumulator goes to the worker's slot of `sk_part` and a flag is raised.  The worker
// whose range holds a tile's first k-block *owns* the tile: it computes its piece last, then adds the
// contributions in increasing k order and runs the normal epilogue.  Every output element is therefore summed in
// an order fixed by (shape, W): results do not change from run to run.  Contributions are the first thing a worker
// computes and owned pieces the last thing of its range, so an owner finds them ready unless the contributing CTA
// has not been scheduled yet; the wait for it is bounded (kDevErrGemmSplitTimeout).  Waits only ever point from
// worker w to workers > w, so no cycle exists.
enum { kItemFull = 0, kItemContrib = 1, kItemOwner = 2 };
constexpr unsigned kDevErrGemmSplitTimeout = 4u;
constexpr int kSkSlots = 128;                       // launches in flight at once share flags only 128 launches apart
constexpr int kSkMaxWorkers = kNumSMs / 2;
constexpr size_t kSkPartFloats = 256 * 128;         // per (worker, CTA of the pair)
__device__ unsigned g_sk_flags[kSkSlots][kSkMaxWorkers][2][4];    // zero at load; every flag is cleared by its reader

struct WorkItem { long long tile; int kb0, kb1, kind; };
struct WorkIter {
  long long pos, end, dp_next, dp_step, total;
  int nkb;
  __device__ __forceinline__ static long long range_begin(const GemmParams& p, long long w, long long nworkers) {
    return p.sk_units * w / nworkers;
  }
  __device__ __forceinline__ void init(const GemmParams& p, long long w, long long nworkers, long long total_tiles, int nkb_) {
    nkb = nkb_; total = total_tiles; dp_step = nworkers;
    pos = range_begin(p, w, nworkers); end = range_begin(p, w + 1, nworkers);
    dp_next = p.sk_tiles + w;
  }
  __device__ __forceinline__ bool next(WorkItem& it) {
    if (pos < end) {
      const long long t = pos / nkb, tile_end = (t + 1) * nkb;
      const long long e = end < tile_end ? end : tile_end;
      it.tile = t; it.kb0 = (int)(pos - t * nkb); it.kb1 = (int)(e - t * nkb);
      it.kind = it.kb0 ? kItemContrib : (it.kb1 == nkb ? kItemFull : kItemOwner);
      pos = e;
      return true;
    }
    if (dp_next < total) {
      it.tile = dp_next; it.kb0 = 0; it.kb1 = nkb; it.kind = kItemFull;
      dp_next += dp_step;
      return true;
    }
    return false;
  }
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Lane 0 polls the flag (acquire) for at most about a second; the whole warp gets the same answer.
__device__ __forceinline__ bool sk_wait_flag(const unsigned* flag, int lane) {
  unsigned ok = 1;
  if (lane == 0) {
    ok = 0;
    const unsigned long long t0 = global_timer_ns();
    for (unsigned it = 1;; ++it) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v) { ok = 1; break; }
      __nanosleep(100);
      if ((it & 255u) == 0 && global_timer_ns() - t0 > 1000000000ull) break;
    }
    if (!ok) atomicMax(&g_dev_error, kDevErrGemmSplitTimeout);
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---- dynamic tile schedule ---------------------------------------------------------------------------------------
// A persistent grid that walks tiles with a fixed stride (worker w takes tiles w, w + W, ...) assumes all W workers
// run at once.  When another kernel holds some SMs (the gradient all-reduce beside the backward pass) the CTAs that
// find no SM start only when others have finished, and then still compute their whole share: the matmul takes two
// rounds instead of one and a fraction.  Here a worker's first tile is its own index and every further tile comes
// from a global counter, so the tiles go to whichever workers are running; a worker that starts late finds the
// counter exhausted and leaves.  Every tile is still computed whole by one worker in the same k order, so the
// results are bit-identical to the fixed-stride walk.
// The producer thread draws the tile indices and hands them to the other roles of its CTA (and, in the two-SM
// kernel, of the peer CTA) through a ring of kSchedDepth entries in shared memory guarded by mbarriers; -1 ends the
// walk.  The counter of a launch is g_tile_next[slot]; the last worker to finish (g_tile_done[slot]) puts both back
// to zero for the next launch that uses the slot.
constexpr int kSchedDepth = 4;
__device__ unsigned g_tile_next[kSkSlots];
__device__ unsigned g_tile_done[kSkSlots];

struct SchedSmem {
  uint64_t full[kSchedDepth];          // an entry has been published (1 arrival: the scheduling thread)
  uint64_t empty[kSchedDepth];         // this CTA's consumers have read it
  uint64_t empty_peer[kSchedDepth];    // two-SM kernel, leader only: the peer CTA's consumers have read theirs
  int ring[kSchedDepth];
};

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, unsigned parity) {   // acquire at cluster scope
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(g_mbar_suspend_ns) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, unsigned parity, unsigned err_code) {
  for (unsigned it = 0; it < kMbarPolls; ++it)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  atomicMax(&g_dev_error, err_code);
  return false;
}
// Consumer side of the ring for one thread (n: entries read so far).  Returns the tile, -1 at the end of the walk, -2
// when the wait ran out.  `arrive`: this thread reports the read (one thread per consuming warp does).
// CLUSTER: the entry was written by the other CTA of the pair, and the read is reported to that CTA's barrier.
template <bool CLUSTER>
__device__ __forceinline__ int sched_take(SchedSmem* sm, unsigned& n, bool arrive, uint32_t leader_empty_peer0) {
  const int sl = (int)(n % kSchedDepth);
  const unsigned ph = (n / kSchedDepth) & 1u;
  const bool ok = CLUSTER ? mbar_wait_bounded_cluster(sm->full + sl, ph, kDevErrGemmTimeout)
                          : mbar_wait_bounded(sm->full + sl, ph, kDevErrGemmTimeout);
  if (!ok) return -2;
  const int tile = *reinterpret_cast<volatile int*>(&sm->ring[sl]);
  if (arrive) {
    if (CLUSTER) mbar_arrive_cluster(leader_empty_peer0 + (uint32_t)sl * 8u);
    else mbar_arrive(sm->empty + sl);
  }
  ++n;
  return tile;
}
// The same for a whole warp (all lanes get the tile; lane 0 reports the read after every lane has it).
template <bool CLUSTER>
__device__ __forceinline__ int sched_take_warp(SchedSmem* sm, unsigned& n, int lane, uint32_t leader_empty_peer0) {
  const int sl = (int)(n % kSchedDepth);
  const unsigned ph = (n / kSchedDepth) & 1u;
  const bool ok = CLUSTER ? mbar_wait_bounded_cluster(sm->full + sl, ph, kDevErrGemmTimeout)
                          : mbar_wait_bounded(sm->full + sl, ph, kDevErrGemmTimeout);
  if (!__all_sync(0xffffffffu, ok)) return -2;
  const int tile = *reinterpret_cast<volatile int*>(&sm->ring[sl]);
  __syncwarp();
  if (lane == 0) {
    if (CLUSTER) mbar_arrive_cluster(leader_empty_peer0 + (uint32_t)sl * 8u);
    else mbar_arrive(sm->empty + sl);
  }
  ++n;
  return tile;
}
// Scheduling thread: publish `tile` (or -1) as entry n.  PAIR: also into the peer CTA's ring.
template <bool PAIR>
__device__ __forceinline__ bool sched_publish(SchedSmem* sm, unsigned& n, int tile) {
  const int sl = (int)(n % kSchedDepth);
  const unsigned ph = (n / kSchedDepth) & 1u;
  if (!mbar_wait_bounded(sm->empty + sl, ph ^ 1u, kDevErrGemmTimeout)) return false;
  if (PAIR && !mbar_wait_bounded_cluster(sm->empty_peer + sl, ph ^ 1u, kDevErrGemmTimeout)) return false;
  sm->ring[sl] = tile;
  mbar_arrive(sm->full + sl);                                  // release: the entry is visible to who sees the arrival
  if (PAIR) {
    uint32_t peer_ring, peer_full;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_ring) : "r"(smem_u32(&sm->ring[sl])), "r"(1u));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_full) : "r"(smem_u32(sm->full + sl)), "r"(1u));
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_ring), "r"((uint32_t)tile) : "memory");
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_full) : "memory");
  }
  ++n;
  return true;
}
// Next tile for the scheduling thread: workers' first tiles are their own indices, the rest come from the counter.
__device__ __forceinline__ long long sched_draw(int slot, long long nworkers, long long total) {
  const long long t = nworkers + (long long)atomicAdd(&g_tile_next[slot], 1u);
  return t < total ? t : -1;
}
// Called once per worker by its scheduling thread when it is done drawing.
__device__ __forceinline__ void sched_retire(int slot, long long nworkers) {
  __threadfence();
  if (atomicAdd(&g_tile_done[slot], 1u) == (unsigned)(nworkers - 1)) {
    __threadfence();
    g_tile_next[slot] = 0;
    g_tile_done[slot] = 0;
  }
}

// What the epilogue does with one accumulator (two-SM kernel).
struct SkEpi {
  int kind;                 // kItemFull: normal epilogue; kItemContrib: store the accumulator; kItemOwner: add, then normal
  float* my_part;           // contribution: this CTA's slot
  unsigned* my_flags;       // contribution: this CTA's four flags (one per epilogue warp)
  const float* part0;       // owner: slot of the first contributor (the next worker), same CTA rank; next worker 2 slots on
  unsigned* flags0;         // owner: flags of the first contributor; next worker 8 words on
  int ncontrib;
};

// Tile order inside one block: groups of `group_m` m-tiles; inside a group the m index runs fastest, so
// the CTAs that run at the same time share a few B (weight) panels and a bounded set of A rows in L2.
__device__ __forceinline__ void decode_tile(long long tile, long long tiles_per_block, const GemmParams& p, int& blk,
                                            int& tm, int& tn) {
  blk = (int)(tile / tiles_per_block);
  const int r = (int)(tile - (long long)blk * tiles_per_block);
  const int per_group = p.group_m * p.tiles_n;
  const int grp = r / per_group, in = r - grp * per_group;
  const int m0 = grp * p.group_m;
  const int gm = p.tiles_m - m0 < p.group_m ? p.tiles_m - m0 : p.group_m;
  tn = in / gm;
  tm = m0 + (in - tn * gm);
  // With a triangular hint the work of a tile depends on tm; rotating tm by the block index makes the tiles a
  // CTA meets (tile, tile + grid, ...) run through all row positions instead of a few residues.
  if (p.tri) tm = (tm + blk) % p.tiles_m;
}

// Instruction descriptor with the N extent replaced (edge tiles issue narrower MMAs instead of multiplying zeros).
__device__ __forceinline__ uint32_t idesc_with_n(uint32_t idesc, int n) {
  return (idesc & ~(0x3Fu << 17)) | ((uint32_t)(n >> 3) << 17);
}

// Triangular hints, per output tile whose rows are [row0, row0 + rows) and whose first column is col0.
//   C_LOWER: only C[r, c] with c <= r + diag is wanted; a tile wholly beyond that is skipped (not written).
//   A_LOWER: op(A)[r, k] == 0 for k > r + diag; k-blocks wholly beyond the tile's last row are skipped.
//   A_UPPER: op(A)[r, k] == 0 for k < r - diag; k-blocks wholly before the tile's first row are skipped.
// Skipped products are exact zeros, so the result is bit-identical to the full computation.
__device__ __forceinline__ bool tile_skipped(const GemmParams& p, int row0, int rows, int col0) {
  return p.tri == CACTI_B200_TRI_C_LOWER && (long long)col0 > (long long)row0 + rows - 1 + p.diag;
}
__device__ __forceinline__ void k_block_range(const GemmParams& p, int row0, int rows, int nkb, int& kb0, int& kb1) {
  kb0 = 0; kb1 = nkb;
  if (p.tri == CACTI_B200_TRI_A_LOWER) {
    const long long last = (long long)row0 + rows - 1 + p.diag;
    const long long e = last < 0 ? 1 : last / kBK + 1;
    kb1 = e < 1 ? 1 : (e < nkb ? (int)e : nkb);
  } else if (p.tri == CACTI_B200_TRI_A_UPPER) {
    const long long first = (long long)row0 - p.diag;
    const long long b = first < 0 ? 0 : first / kBK;
    kb0 = b > nkb - 1 ? nkb - 1 : (int)b;
  }
}

// Epilogue of one accumulator for one warp: TMEM lanes [q*32, q*32+32) x BN columns of accumulator `acc` become
// rows row0 .. row0+31 of the output tile whose first column is tn * BN.  `tempty_addr` is the shared::cluster
// address of the barrier that frees the accumulator: the warp arrives on it once, as soon as its last
// tcgen05.ld has completed.  `cbar` / `cpar`: this warp's barrier and phase for the TMA loads that bring the old
// C boxes into the staging buffers when beta != 0 (Accumulate mode, src/thunk/mod.rs:347-351).
template <typename T, int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const CUtensorMap& tmC, T* __restrict__ C,
                                              uint32_t tmem_base, int acc, int row0, int tn, int bj, int bi, int q, int lane,
                                              unsigned char* mybuf, uint32_t tempty_addr, uint64_t* cbar, unsigned& cpar,
                                              const SkEpi sk = SkEpi{}) {
  const int prow = q * 32 + lane;             // this thread's row inside its CTA's 128 rows (partial-slot index)
  if (sk.kind == kItemContrib) {
    // this CTA's piece of a tile another worker owns: accumulator -> f32 slot (column-major, so a warp's stores of
    // one column are 128 contiguous bytes), then the flag
#pragma unroll 1
    for (int c = 0; c < BN / 64; ++c) {
      if (tn * BN + c * 64 >= p.N) break;
      uint32_t v[2][32];
      tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 64), v[0]);
      tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 64 + 32), v[1]);
      tc_ld_wait();
      float* dst = sk.my_part + (size_t)(c * 64) * kBM + prow;
#pragma unroll
      for (int i = 0; i < 64; ++i) __stcg(dst + (size_t)i * kBM, __uint_as_float(v[i >> 5][i & 31]));
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(tempty_addr);
    __threadfence();
    __syncwarp();
    if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sk.my_flags + q), "r"(1u) : "memory");
    return;
  }
  if (sk.kind == kItemOwner) {
    // the contributions were computed first by their workers; a wait that runs out is recorded and the tile is
    // finished with what is there (the device error word tells the caller the result is void)
    for (int ci = 0; ci < sk.ncontrib; ++ci) sk_wait_flag(sk.flags0 + ci * 8 + q, lane);
  }
  if (p.c_tma) {
    // TMEM -> registers -> swizzled shared staging -> TMA store (clips rows/columns past M, N)
    // 128 accumulator columns per trip: four tcgen05.ld in flight, one wait, two 64-column TMA stores
    const bool scale = p.alpha != 1.f;
    const bool accum = p.beta != 0.f;
    constexpr int TRIPS = (BN + 127) / 128;
#pragma unroll 1
    for (int c = 0; c < TRIPS; ++c) {
      const int col0 = tn * BN + c * 128;
      if (col0 >= p.N) break;               // warp-uniform
      const int ncols = BN - c * 128 < 128 ? BN - c * 128 : 128;      // columns of this tile in this trip (128 or 64)
      uint32_t v[4][32];
#pragma unroll
      for (int hh = 0; hh < 4; ++hh)
        if (hh * 32 < ncols)
          tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 128 + hh * 32), v[hh]);
      // both staging buffers must have been read by the stores of the previous trip
      if (lane == 0) {
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (accum) {
          // old C: the same boxes the stores below write, into the same (swizzled) places of the staging buffers;
          // rows and columns past M, N arrive as zeros and are clipped again by the store
          const bool two = col0 + 64 < p.N && ncols > 64;
          mbar_expect_tx(cbar, two ? 8192u : 4096u);
          tma_load_4d(mybuf, &tmC, cbar, col0, row0, bj, bi);
          if (two) tma_load_4d(mybuf + 4096, &tmC, cbar, col0 + 64, row0, bj, bi);
        }
      }
      tc_ld_wait();
      if (c == TRIPS - 1 || col0 + 128 >= p.N) {         // last trip of this tile: the accumulator is free
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_addr);
      } else {
        __syncwarp();
      }
      if (sk.kind == kItemOwner) {                       // + the other workers' pieces, in increasing k
        for (int ci = 0; ci < sk.ncontrib; ++ci) {
          const float* src = sk.part0 + (size_t)ci * 2 * kSkPartFloats + (size_t)(c * 128) * kBM + prow;
#pragma unroll
          for (int hh = 0; hh < 4; ++hh) {
            if (hh * 32 < ncols && col0 + hh * 32 < p.N) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                v[hh][i] = __float_as_uint(__uint_as_float(v[hh][i]) + __ldcg(src + (size_t)(hh * 32 + i) * kBM));
            }
          }
        }
      }
      if (accum) {
        // the warp decides together: a wait that ran out leaves the tile unwritten (device error word set)
        const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(cbar, cpar, kDevErrGemmTimeout));
        cpar ^= 1u;
        if (!ok) return;
      }
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {
        if (hb * 64 >= ncols) break;
        unsigned char* buf = mybuf + hb * 4096;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float t8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float a = __uint_as_float(v[hb * 2 + hh][g * 8 + i]);
              t8[i] = scale ? p.alpha * a : a;
            }
            const int chunk = hh * 4 + g;       // 16-byte chunk inside the 128-byte row
            uint4* slot = reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4));
            if (accum && (hb == 0 || col0 + 64 < p.N)) {
              float o8[8];
              unpack<T>(*slot, o8);
#pragma unroll
              for (int i = 0; i < 8; ++i) t8[i] = fmaf(p.beta, o8[i], t8[i]);
            }
            *slot = pack<T>(t8);
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(&tmC, mybuf, col0, row0, bj, bi);
        if (col0 + 64 < p.N && ncols > 64) tma_store_4d(&tmC, mybuf + 4096, col0 + 64, row0, bj, bi);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    if (sk.kind == kItemOwner && lane == 0)
      for (int ci = 0; ci < sk.ncontrib; ++ci) sk.flags0[ci * 8 + q] = 0;       // ready for the next launch
    return;                                   // the accumulator was released inside the loop
  }
  const int row = row0 + lane;
  T* crow = C + (long long)bi * p.c_stride_outer + (long long)bj * p.c_stride_inner + (long long)row * p.ldc;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    const int col0 = tn * BN + c * 32;
    if (col0 >= p.N) break;               // warp-uniform
    uint32_t v[32];
    tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 32), v);
    tc_ld_wait();
    if (sk.kind == kItemOwner) {
      for (int ci = 0; ci < sk.ncontrib; ++ci) {
        const float* src = sk.part0 + (size_t)ci * 2 * kSkPartFloats + (size_t)(c * 32) * kBM + prow;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __ldcg(src + (size_t)i * kBM));
      }
    }
    if (row < p.M) {
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = p.alpha * __uint_as_float(v[i]);
      const int nvalid = p.N - col0 < 32 ? p.N - col0 : 32;
      T* out = crow + col0;
      if (p.beta != 0.f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (i < nvalid) f[i] = fmaf(p.beta, Elem<T>::to_f32(out[i]), f[i]);
      }
      if (nvalid == 32 && p.c_align >= 16) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float t8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) t8[i] = f[g * 8 + i];
          *reinterpret_cast<uint4*>(out + g * 8) = pack<T>(t8);
        }
      } else if (p.c_align >= 8) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (g * 4 + 4 <= nvalid) {
            uint2 w;
            if constexpr (std::is_same<T, __half>::value) {
              __half2 a = __floats2half2_rn(f[g * 4], f[g * 4 + 1]), b = __floats2half2_rn(f[g * 4 + 2], f[g * 4 + 3]);
              w.x = *reinterpret_cast<uint32_t*>(&a); w.y = *reinterpret_cast<uint32_t*>(&b);
            } else {
              __nv_bfloat162 a = __floats2bfloat162_rn(f[g * 4], f[g * 4 + 1]), b = __floats2bfloat162_rn(f[g * 4 + 2], f[g * 4 + 3]);
              w.x = *reinterpret_cast<uint32_t*>(&a); w.y = *reinterpret_cast<uint32_t*>(&b);
            }
            *reinterpret_cast<uint2*>(out + g * 4) = w;
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) if (g * 4 + i < nvalid) out[g * 4 + i] = Elem<T>::from_f32(f[g * 4 + i]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (i < nvalid) out[i] = Elem<T>::from_f32(f[i]);
      }
    }
  }
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive_cluster(tempty_addr);
  if (sk.kind == kItemOwner && lane == 0)
    for (int ci = 0; ci < sk.ncontrib; ++ci) sk.flags0[ci * 8 + q] = 0;
}

template <typename T, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, T* __restrict__ C, const GemmParams p) {
  constexpr int STAGES = BN >= 192 ? 4 : 6;
  constexpr uint32_t A_BYTES = kBM * kBK * 2, B_BYTES = BN * kBK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  SchedSmem* sched = reinterpret_cast<SchedSmem*>(tmem_slot + 4);
  uint64_t* cbar = reinterpret_cast<uint64_t*>(sched + 1);        // one per epilogue warp: old C boxes have arrived
  // epilogue staging: per epilogue warp two [32 rows][64 cols] buffers in the 128-byte-swizzled layout of a
  // TMA box (4 KB each), 1024-byte aligned
  unsigned char* cstage = tiles + (size_t)STAGES * STAGE_BYTES + 1024;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull + a, 1); mbar_init(tempty + a, 4); }
    // schedule ring: read by the MMA thread and by the four epilogue warps
    for (int i = 0; i < kSchedDepth; ++i) { mbar_init(sched->full + i, 1); mbar_init(sched->empty + i, 5); mbar_init(sched->empty_peer + i, 5); }
    for (int w = 0; w < 4; ++w) mbar_init(cbar + w, 1);
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

  const int nkb = (p.K + kBK - 1) / kBK;
  const long long tiles_per_block = (long long)p.tiles_m * p.tiles_n;
  const long long total = tiles_per_block * p.nb_inner * p.nb_outer;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer (and, with the dynamic schedule, the thread that draws the tiles) ----------------
    int s = 0; unsigned ph = 0;
    auto produce = [&](long long tile) -> bool {
      int blk, tm, tn;
      decode_tile(tile, tiles_per_block, p, blk, tm, tn);
      const int bi = blk / p.nb_inner, bj = blk - bi * p.nb_inner;
      const int aj = p.a_j ? bj : 0, ai = p.a_i ? bi : 0, bjj = p.b_j ? bj : 0, bii = p.b_i ? bi : 0;
      if (tile_skipped(p, tm * kBM, kBM, tn * BN)) return true;
      int kb0, kb1;
      k_block_range(p, tm * kBM, kBM, nkb, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(empty + s, ph ^ 1, kDevErrGemmTimeout)) return false;
        unsigned char* sa = tiles + (size_t)s * STAGE_BYTES;
        unsigned char* sb = sa + A_BYTES;
        mbar_expect_tx(full + s, STAGE_BYTES);
        if (!A_MN) tma_load_4d(sa, &tmA, full + s, kb * kBK, tm * kBM, aj, ai);
        else {
#pragma unroll
          for (int h = 0; h < kBM / 64; ++h) tma_load_4d(sa + h * 8192, &tmA, full + s, tm * kBM + h * 64, kb * kBK, aj, ai);
        }
        if (!B_MN) tma_load_4d(sb, &tmB, full + s, kb * kBK, tn * BN, bjj, bii);
        else {
#pragma unroll
          for (int h = 0; h < BN / 64; ++h) tma_load_4d(sb + h * 8192, &tmB, full + s, tn * BN + h * 64, kb * kBK, bjj, bii);
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      return true;
    };
    if (p.dyn) {
      unsigned sn = 0;
      long long tile = blockIdx.x;                       // the grid never exceeds the tile count
      for (;;) {
        if (!sched_publish<false>(sched, sn, (int)tile)) break;
        if (tile < 0) break;
        const long long nxt = sched_draw(p.sk_slot, gridDim.x, total);     // in flight while this tile's loads are issued
        if (!produce(tile)) break;
        tile = nxt;
      }
    } else {
      for (long long tile = blockIdx.x; tile < total; tile += gridDim.x)
        if (!produce(tile)) break;
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    int s = 0; unsigned ph = 0;
    long long local = 0;
    auto mma_tile = [&](long long tile) -> bool {
      int kb0 = 0, kb1 = nkb;
      int blk, tm, tn;
      decode_tile(tile, tiles_per_block, p, blk, tm, tn);
      if (p.tri) {
        if (tile_skipped(p, tm * kBM, kBM, tn * BN)) return true;
        k_block_range(p, tm * kBM, kBM, nkb, kb0, kb1);
      }
      // the last column tile multiplies only the columns that exist (rounded up to the MMA's granularity of 16)
      const int nvalid = p.N - tn * BN;
      const uint32_t idesc = nvalid >= BN ? p.idesc : idesc_with_n(p.idesc, (nvalid + 15) & ~15);
      const int acc = (int)(local & 1);
      if (!mbar_wait_bounded(tempty + acc, (unsigned)((local >> 1) & 1) ^ 1, kDevErrGemmTimeout)) return false;
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(full + s, ph, kDevErrGemmTimeout)) return false;
        tc_fence_after();
        const uint32_t sa = smem_u32(tiles + (size_t)s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4) {
          const uint64_t da = A_MN ? make_desc(sa + k4 * 2048, 512, 64) : make_desc(sa + k4 * 32, 1, 64);
          const uint64_t db = B_MN ? make_desc(sb + k4 * 2048, 512, 64) : make_desc(sb + k4 * 32, 1, 64);
          tc_mma_f16(tacc, da, db, idesc, (kb > kb0 || k4) ? 1u : 0u);
        }
        tc_commit(empty + s);                 // stage free once these MMAs have read it
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      tc_commit(tfull + acc);                 // accumulator complete
      ++local;
      return true;
    };
    if (p.dyn) {
      unsigned sn = 0;
      for (;;) {
        const int tile = sched_take<false>(sched, sn, true, 0);
        if (tile < 0 || !mma_tile(tile)) break;
      }
    } else {
      for (long long tile = blockIdx.x; tile < total; tile += gridDim.x)
        if (!mma_tile(tile)) break;
    }
  } else if (warp >= 2) {
    // ---------------- epilogue ----------------
    const int q = warp & 3;                   // TMEM lane quarter this warp may read
    long long local = 0;
    unsigned cpar = 0;                        // phase of this warp's old-C barrier
    auto epi_tile = [&](long long tile) -> bool {
      int blk, tm, tn;
      decode_tile(tile, tiles_per_block, p, blk, tm, tn);
      if (tile_skipped(p, tm * kBM, kBM, tn * BN)) return true;
      const int bi = blk / p.nb_inner, bj = blk - bi * p.nb_inner;
      const int acc = (int)(local & 1);
      // all 32 lanes leave together: a wait that ran out on some lanes only must not split the warp before the
      // warp-wide tcgen05.ld of the epilogue
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(tfull + acc, (unsigned)((local >> 1) & 1), kDevErrGemmTimeout))) return false;
      tc_fence_after();
      epilogue_tile<T, BN>(p, tmC, C, tmem_base, acc, tm * kBM + q * 32, tn, bj, bi, q, lane,
                           cstage + (size_t)(warp - 2) * 8192, smem_u32(tempty + acc), cbar + (warp - 2), cpar);
      ++local;
      return true;
    };
    if (p.dyn) {
      unsigned sn = 0;
      for (;;) {
        const int tile = sched_take_warp<false>(sched, sn, lane, 0);
        if (tile < 0 || !epi_tile(tile)) break;
      }
    } else {
      for (long long tile = blockIdx.x; tile < total; tile += gridDim.x)
        if (!epi_tile(tile)) break;
    }
  }
  if (p.dyn && warp == 0 && lane == 0) sched_retire(p.sk_slot, gridDim.x);     // on every path, or the counter stays dirty
  if (warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- two-SM variant (cta_group::2) -------------------------------------------------------------------------
// A cluster of two CTAs on one SM pair computes a 256 x 256 output tile.  Each CTA stages its own 128 rows of A
// and one half (128 rows) of the B tile; the leader CTA (cluster rank 0) issues tcgen05.mma.cta_group::2 with
// M = 256, which reads A from both CTAs, both halves of B, and accumulates rows 0..127 into the leader's TMEM and
// rows 128..255 into the peer's.  Per flop each SM reads a third less shared memory and L2 than the
// one-SM 128 x 256 tile.  Signalling:
//   full[s]   (leader only) : 1 arrival (the leader's expect_tx for both CTAs' bytes); both CTAs' TMA loads
//                             complete their bytes on it (the load's cta_group::2 form allows a peer barrier)
//   empty[s]  (both CTAs)   : the leader's tcgen05.commit, multicast to both CTAs
//   tfull[a]  (both CTAs)   : same, when an accumulator is complete
//   tempty[a] (leader only) : 8 arrivals, one per epilogue warp of either CTA
// No load uses cluster multicast.  Every wait is bounded; all threads of both CTAs meet on the cluster barrier
// before TMEM is freed, and the producers wait for the last stage releases, so neither CTA exits while the other
// can still signal into its shared memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(void* dst, const CUtensorMap* map, uint32_t bar_addr, int c0, int c1, int c2,
                                                 int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {       // arrives on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((unsigned short)3)
               : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accum)
      : "memory");
}

constexpr int kPairBM = 256, kPairBN = 256, kPairStages = 6;
constexpr size_t kPairSmem = (size_t)kPairStages * (kBM * kBK * 2 + (kPairBN / 2) * kBK * 2) + 1024 + 1024 + 4 * 8192;

template <typename T, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, T* __restrict__ C, const GemmParams p) {
  constexpr int BN = kPairBN, HB = BN / 2, STAGES = kPairStages;
  constexpr uint32_t A_BYTES = kBM * kBK * 2, B_BYTES = HB * kBK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  SchedSmem* sched = reinterpret_cast<SchedSmem*>(tmem_slot + 4);
  uint64_t* cbar = reinterpret_cast<uint64_t*>(sched + 1);        // one per epilogue warp: old C boxes have arrived
  unsigned char* cstage = tiles + (size_t)STAGES * STAGE_BYTES + 1024;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const long long pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull + a, 1); mbar_init(tempty + a, 8); }
    // schedule ring: in the leader read by the MMA thread and four epilogue warps (empty), in the peer by the producer
    // thread and four epilogue warps, which report to the leader's empty_peer
    for (int i = 0; i < kSchedDepth; ++i) { mbar_init(sched->full + i, 1); mbar_init(sched->empty + i, 5); mbar_init(sched->empty_peer + i, 5); }
    for (int w = 0; w < 4; ++w) mbar_init(cbar + w, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                         // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nkb = (p.K + kBK - 1) / kBK;
  const long long tiles_per_block = (long long)p.tiles_m * p.tiles_n;
  const long long total = tiles_per_block * p.nb_inner * p.nb_outer;

  // the leader's barriers on which the peer CTA's consumers report their reads of the schedule ring
  const uint32_t leader_empty_peer0 = map_to_rank(smem_u32(sched->empty_peer), 0);

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer (both CTAs); the leader's also draws the tiles of the dynamic schedule ----------------
    int s = 0; unsigned ph = 0;
    const int row_off = (int)rank * kBM;
    auto produce = [&](const WorkItem& wi) -> bool {
      int blk, tm, tn;
      decode_tile(wi.tile, tiles_per_block, p, blk, tm, tn);
      const int bi = blk / p.nb_inner, bj = blk - bi * p.nb_inner;
      const int aj = p.a_j ? bj : 0, ai = p.a_i ? bi : 0, bjj = p.b_j ? bj : 0, bii = p.b_i ? bi : 0;
      // a last column tile with at most 128 columns runs as an N = 128 MMA: each CTA then supplies 64 rows of B
      // (the first 64 of the box it loads), so the CTAs' boxes start 64 rows apart instead of 128
      const int hb = (p.N - tn * BN <= HB) ? HB / 2 : HB;
      const int m0 = tm * kPairBM + row_off, n0 = tn * BN + (int)rank * hb;
      if (tile_skipped(p, tm * kPairBM, kPairBM, tn * BN)) return true;
      int kb0 = wi.kb0, kb1 = wi.kb1;
      if (p.tri) k_block_range(p, tm * kPairBM, kPairBM, nkb, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(empty + s, ph ^ 1, kDevErrGemmTimeout)) return false;
        unsigned char* sa = tiles + (size_t)s * STAGE_BYTES;
        unsigned char* sb = sa + A_BYTES;
        const uint32_t fb = map_to_rank(smem_u32(full + s), 0);
        if (rank == 0) mbar_expect_tx(full + s, 2 * STAGE_BYTES);
        if (!A_MN) tma_load_4d_pair(sa, &tmA, fb, kb * kBK, m0, aj, ai);
        else {
#pragma unroll
          for (int h = 0; h < kBM / 64; ++h) tma_load_4d_pair(sa + h * 8192, &tmA, fb, m0 + h * 64, kb * kBK, aj, ai);
        }
        if (!B_MN) tma_load_4d_pair(sb, &tmB, fb, kb * kBK, n0, bjj, bii);
        else {
#pragma unroll
          for (int h = 0; h < HB / 64; ++h) tma_load_4d_pair(sb + h * 8192, &tmB, fb, n0 + h * 64, kb * kBK, bjj, bii);
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      return true;
    };
    bool ok = true;
    WorkItem wi;
    if (p.dyn) {
      unsigned sn = 0;
      wi.kb0 = 0; wi.kb1 = nkb; wi.kind = kItemFull;
      if (rank == 0) {
        long long tile = pair;                             // the grid never has more pairs than tiles
        for (;;) {
          if (!sched_publish<true>(sched, sn, (int)tile)) { ok = false; break; }
          if (tile < 0) break;
          const long long nxt = sched_draw(p.sk_slot, npairs, total);    // in flight while this tile's loads are issued
          wi.tile = tile;
          if (!produce(wi)) { ok = false; break; }
          tile = nxt;
        }
      } else {
        for (;;) {
          const int tile = sched_take<true>(sched, sn, true, leader_empty_peer0);
          if (tile < 0) { ok = tile == -1; break; }
          wi.tile = tile;
          if (!produce(wi)) { ok = false; break; }
        }
      }
    } else {
      WorkIter it;
      it.init(p, pair, npairs, total, nkb);
      while (ok && it.next(wi)) ok = produce(wi);
    }
    // the leader's last commits still arrive on this CTA's empty barriers: wait for them before leaving
    for (int i = 0; ok && i < STAGES; ++i) {
      ok = mbar_wait_bounded(empty + s, ph ^ 1, kDevErrGemmTimeout);
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------- MMA issuer (leader CTA) ----------------
    int s = 0; unsigned ph = 0;
    long long local = 0;
    auto mma_item = [&](const WorkItem& wi) -> bool {
      int kb0 = wi.kb0, kb1 = wi.kb1;
      int blk, tm, tn;
      decode_tile(wi.tile, tiles_per_block, p, blk, tm, tn);
      if (p.tri) {
        if (tile_skipped(p, tm * kPairBM, kPairBM, tn * BN)) return true;
        k_block_range(p, tm * kPairBM, kPairBM, nkb, kb0, kb1);
      }
      const uint32_t idesc = (p.N - tn * BN <= HB) ? idesc_with_n(p.idesc, HB) : p.idesc;      // see the producer
      const int acc = (int)(local & 1);
      if (!mbar_wait_bounded(tempty + acc, (unsigned)((local >> 1) & 1) ^ 1, kDevErrGemmTimeout)) return false;
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(full + s, ph, kDevErrGemmTimeout)) return false;
        tc_fence_after();
        const uint32_t sa = smem_u32(tiles + (size_t)s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4) {
          const uint64_t da = A_MN ? make_desc(sa + k4 * 2048, 512, 64) : make_desc(sa + k4 * 32, 1, 64);
          const uint64_t db = B_MN ? make_desc(sb + k4 * 2048, 512, 64) : make_desc(sb + k4 * 32, 1, 64);
          tc_mma_f16_pair(tacc, da, db, idesc, (kb > kb0 || k4) ? 1u : 0u);
        }
        tc_commit_pair(empty + s);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      tc_commit_pair(tfull + acc);
      ++local;
      return true;
    };
    WorkItem wi;
    if (p.dyn) {
      unsigned sn = 0;
      wi.kb0 = 0; wi.kb1 = nkb; wi.kind = kItemFull;
      for (;;) {
        const int tile = sched_take<false>(sched, sn, true, 0);
        if (tile < 0) break;
        wi.tile = tile;
        if (!mma_item(wi)) break;
      }
    } else {
      WorkIter it;
      it.init(p, pair, npairs, total, nkb);
      while (it.next(wi))
        if (!mma_item(wi)) break;
    }
  } else if (warp >= 2) {
    // ---------------- epilogue (both CTAs, each on its own 128 rows) ----------------
    const int q = warp & 3;
    long long local = 0;
    unsigned cpar = 0;                        // phase of this warp's old-C barrier
    auto epi_item = [&](const WorkItem& wi) -> bool {
      int blk, tm, tn;
      decode_tile(wi.tile, tiles_per_block, p, blk, tm, tn);
      if (tile_skipped(p, tm * kPairBM, kPairBM, tn * BN)) return true;
      const int bi = blk / p.nb_inner, bj = blk - bi * p.nb_inner;
      const int acc = (int)(local & 1);
      SkEpi sk{};
      sk.kind = wi.kind;
      if (wi.kind == kItemContrib) {
        sk.my_part = p.sk_part + ((size_t)pair * 2 + rank) * kSkPartFloats;
        sk.my_flags = &g_sk_flags[p.sk_slot][pair][rank][0];
      } else if (wi.kind == kItemOwner) {
        // the rest of this tile lies in the ranges of the next workers
        const long long tile_end = (wi.tile + 1) * nkb;
        int n = 0;
        for (long long w2 = pair + 1; w2 < npairs && WorkIter::range_begin(p, w2, npairs) < tile_end; ++w2) ++n;
        sk.ncontrib = n;
        sk.part0 = p.sk_part + ((size_t)(pair + 1) * 2 + rank) * kSkPartFloats;
        sk.flags0 = &g_sk_flags[p.sk_slot][pair + 1][rank][0];
      }
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(tfull + acc, (unsigned)((local >> 1) & 1), kDevErrGemmTimeout))) return false;
      tc_fence_after();
      epilogue_tile<T, BN>(p, tmC, C, tmem_base, acc, tm * kPairBM + (int)rank * kBM + q * 32, tn, bj, bi, q, lane,
                           cstage + (size_t)(warp - 2) * 8192, map_to_rank(smem_u32(tempty + acc), 0), cbar + (warp - 2), cpar, sk);
      ++local;
      return true;
    };
    WorkItem wi;
    if (p.dyn) {
      unsigned sn = 0;
      wi.kb0 = 0; wi.kb1 = nkb; wi.kind = kItemFull;
      for (;;) {
        const int tile = rank == 0 ? sched_take_warp<false>(sched, sn, lane, 0) : sched_take_warp<true>(sched, sn, lane, leader_empty_peer0);
        if (tile < 0) break;
        wi.tile = tile;
        if (!epi_item(wi)) break;
      }
    } else {
      WorkIter it;
      it.init(p, pair, npairs, total, nkb);
      while (it.next(wi))
        if (!epi_item(wi)) break;
    }
  }
  if (p.dyn && warp == 0 && lane == 0 && rank == 0) sched_retire(p.sk_slot, npairs);   // on every path, or the counter stays dirty
  if (warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                         // both CTAs have finished reading TMEM and signalling each other
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// Repack blocks [nbo][nbi] of a stored matrix [rows x cols] (leading dimension ld, block strides so/si)
// into a dense [nbo*nbi][rows][cols_pad] buffer, zero-filling the padding columns.  One thread per unit of
// UNIT bytes (8 when every row start is 8-byte aligned and cols % 4 == 0, else 4 or 2); consecutive threads
// take consecutive units of a row, so both sides are coalesced.
template <typename U>
__global__ void __launch_bounds__(256)
pack_blocks_kernel(U* __restrict__ dst, const U* __restrict__ src, unsigned rows, unsigned upr_src /* units per source row */,
                   unsigned upr_dst, long long ld_units, unsigned nbi, long long so_units, long long si_units,
                   long long total_units) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_units; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / upr_dst;                      // destination row
    const unsigned c = (unsigned)(i - t * upr_dst);
    const unsigned blk = (unsigned)(t / rows);
    const unsigned r = (unsigned)(t - (long long)blk * rows);
    const unsigned bo = blk / nbi, bi = blk - bo * nbi;
    U v{};
    if (c < upr_src) v = src[bo * so_units + bi * si_units + (long long)r * ld_units + c];
    dst[i] = v;
  }
}

// One operand as stored: `rows` x `cols` elements, cols contiguous, leading dimension ld, block strides.
struct Operand {
  uint64_t ptr; long long rows, cols, ld, stride_inner, stride_outer; int has_j, has_i;
  long long map_cols = 0;     // inner extent given to the tensor map (0: cols); > cols for zero-padded repacked operands
};

static bool tma_ok(const Operand& o, int nbi, int nbo) {
  if (o.ptr & 15) return false;
  if ((o.ld * 2) & 15) return false;
  if (o.has_j && nbi > 1 && ((o.stride_inner * 2) & 15)) return false;
  if (o.has_i && nbo > 1 && ((o.stride_outer * 2) & 15)) return false;
  return true;
}

static int encode_operand(CUtensorMap* map, const Operand& o, int nbi, int nbo, int box_inner, int box_outer, bool bf16) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CACTI_B200_ERR_LAUNCH;
  const cuuint64_t dj = (o.has_j && nbi > 1) ? (cuuint64_t)nbi : 1, di = (o.has_i && nbo > 1) ? (cuuint64_t)nbo : 1;
  cuuint64_t dims[4] = {(cuuint64_t)(o.map_cols ? o.map_cols : o.cols), (cuuint64_t)o.rows, dj, di};
  const cuuint64_t row_bytes = (cuuint64_t)o.ld * 2;
  const cuuint64_t dflt = row_bytes * (cuuint64_t)o.rows;      // any legal value for an extent-1 dimension
  cuuint64_t strides[3] = {row_bytes, dj > 1 ? (cuuint64_t)o.stride_inner * 2 : dflt,
                           di > 1 ? (cuuint64_t)o.stride_outer * 2 : dflt};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  reinterpret_cast<void*>(o.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return CACTI_B200_ERR_LAUNCH; }
  return CACTI_B200_OK;
}

// Repacked operands are padded to a multiple of 64 columns (one 128-byte swizzle span) with zeros, so that no
// TMA box of theirs is partly out of range: measured on B200, boxes that needed out-of-range fill made the
// head_dim-100 block matmuls 1.45x slower than the same kernel on head_dim 128.
static long long packed_cols(long long cols) { return (cols + 63) / 64 * 64; }
static size_t packed_bytes(long long rows, long long cols, long long nblk) {
  const long long cp = packed_cols(cols);
  return ((size_t)nblk * rows * cp * 2 + 255) / 256 * 256;
}

int g_gemm_bn = 0;   // 0: choose by N; 128 or 256 forces the tile width (measurement knob)
int g_gemm_group_m = 0;
int g_gemm_sms = 0;   // 0: all 148
int g_gemm_pair = 1;  // 1: 256-wide tiles may run as two-SM (cta_group::2) 256 x 256 tiles; 0: one-SM tiles only
// 1: the two-SM kernel may share tiles out in k-blocks when a workspace is given (see WorkIter).  Off unless asked
// for: timed alone at one sequence per GPU (M = 2048) the schedule brought the forward and input-gradient matmuls to
// the per-flop rate they have at M = 16384 (2048 x 3200 x 8640: 124 -> 107 us), but a whole training step ran 5 %
// slower with it (50.8 -> 53.6 ms at M = 2048): these matmuls are power-limited, the SMs a partly filled last wave
// leaves idle let the others clock higher, and the partial sums displace 19 MB of the L2 per matmul.
int g_gemm_split = 0;
int g_gemm_dynamic = 1;  // 1: tiles beyond a worker's first are drawn from a global counter (see "dynamic tile schedule")

// Workers and k-split tiles for `tiles` two-SM tiles of `nkb` k-blocks on at most `max_workers` SM pairs.  Splitting
// pays when the last wave of whole tiles would leave more than about 5 % of the grid idle.
struct SplitPlan { long long workers, sk_tiles; };
// `tiles_n`, `group_m`, `N`, `K`: to bound the operand bytes the split tiles touch.  Whole tiles that run at the same
// time walk k together, so each operand panel is fetched from HBM once and shared through L2; workers of the k-split
// region sit at different k, and the region's operands must stay in L2 (126 MB) as a whole or every panel is fetched
// again per tile (measured: the 2048 x 3200 x 32000 input-gradient matmul of the output head, 336 MB of operands,
// ran 14 % slower split than whole; the 90 MB of the 8640-deep projections 8 to 15 % faster).
static SplitPlan plan_split(long long tiles, int nkb, long long max_workers, long long tiles_n, long long group_m, long long M,
                            long long N, long long K) {
  SplitPlan s{tiles < max_workers ? tiles : max_workers, 0};
  if (max_workers < 2 || tiles * 2 < max_workers) return s;          // a handful of tiles: not worth the partial traffic
  const long long rem = tiles % max_workers;
  if (rem == 0) return s;
  const long long waves = (tiles + max_workers - 1) / max_workers;
  if ((double)(max_workers - rem) / (double)(waves * max_workers) <= 0.05) return s;
  const long long sk_tiles = tiles < max_workers ? tiles : max_workers + rem;
  if (sk_tiles * nkb / max_workers < 4) return s;                    // pieces shorter than the operand ring
  const long long per_group = (group_m > 0 ? group_m : 1) * tiles_n;
  long long rows = (sk_tiles + per_group - 1) / per_group * group_m * 256;
  if (rows > M) rows = M;
  if ((rows + N) * K * 2 > 100ll * 1024 * 1024) return s;
  s.workers = max_workers; s.sk_tiles = sk_tiles;
  return s;
}
static long long pair_group_m(long long tiles_m) {
  const long long g = g_gemm_group_m > 0 ? g_gemm_group_m : 8;
  return g > tiles_m ? tiles_m : g;
}
static size_t split_bytes() { return (size_t)kSkMaxWorkers * 2 * kSkPartFloats * sizeof(float); }

template <typename T>
static int gemm_run(uint64_t c, Operand A, Operand B, bool a_mn, bool b_mn, long long M, long long N, long long K,
                    long long ldc, long long cso, long long csi, int nbi, int nbo, float alpha, float beta,
                    int tri, long long diag, int opflags, uint64_t ws, size_t ws_bytes, cudaStream_t st) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  size_t ws_off = 0;
  // repack what TMA cannot address
  for (Operand* o : {&A, &B}) {
    if (tma_ok(*o, nbi, nbo)) {
      // rows stored zero-padded to a multiple of 64 elements: let the tensor map cover the padding, so that no box
      // is partly out of range (the slow path of the TMA unit) and nothing has to be repacked
      if (opflags & (o == &A ? CACTI_B200_OPERAND_A_PADDED : CACTI_B200_OPERAND_B_PADDED)) {
        if (o->ld < packed_cols(o->cols)) return CACTI_B200_ERR_INVALID_VALUE;
        o->map_cols = packed_cols(o->cols);
      }
      continue;
    }
    const long long nblk = (long long)((o->has_j ? nbi : 1)) * (o->has_i ? nbo : 1);
    const size_t need = packed_bytes(o->rows, o->cols, nblk);
    if (!ws || (ws & 255) || ws_off + need > ws_bytes) return CACTI_B200_ERR_WORKSPACE;
    const long long cp = packed_cols(o->cols);
    const int eff_nbi = o->has_j ? nbi : 1;
    const long long so_ = o->has_i ? o->stride_outer : 0, si_ = o->has_j ? o->stride_inner : 0;
    // widest unit (in elements) that divides every offset involved
    const unsigned long long all = (unsigned long long)(o->ptr / 2) | (unsigned long long)o->ld | (unsigned long long)so_ |
                                   (unsigned long long)si_ | (unsigned long long)o->cols;
    const int ue = (all & 3) == 0 ? 4 : (all & 1) == 0 ? 2 : 1;       // elements per unit
    const long long total_units = nblk * o->rows * (cp / ue);
    long long grid = (total_units + 255) / 256;
    if (grid > (long long)kNumSMs * 32) grid = (long long)kNumSMs * 32;
#define CB_PACK(U_)                                                                                              \
  pack_blocks_kernel<U_><<<(unsigned)grid, 256, 0, st>>>(reinterpret_cast<U_*>(ws + ws_off),                     \
      reinterpret_cast<const U_*>(o->ptr), (unsigned)o->rows, (unsigned)(o->cols / ue), (unsigned)(cp / ue),     \
      o->ld / ue, (unsigned)eff_nbi, so_ / ue, si_ / ue, total_units)
    if (ue == 4) CB_PACK(uint2); else if (ue == 2) CB_PACK(uint32_t); else CB_PACK(uint16_t);
#undef CB_PACK
    int rc = check_launch();
    if (rc) return rc;
    o->ptr = ws + ws_off; o->ld = cp; o->map_cols = cp;
    o->stride_inner = o->rows * cp;
    o->stride_outer = o->rows * cp * eff_nbi;
    ws_off += need;
  }
  // Tile shape: the persistent grid runs ceil(tiles / CTAs) waves; pick the shape with the least wave-time.
  // Per-flop cost relative to the one-SM 256-wide tile with K-major operands, from sustained interleaved runs of
  // the projection shapes: 1.08 for 192-wide and 1.3 for 128-wide tiles; one-SM tiles with an MN-major operand
  // 1.25 (their shared-memory reads conflict more); the two-SM 256 x 256 tile 0.93 with either operand layout (the
  // 3200 x 3200 x 16384 weight-gradient matmul: 1041 TFLOP/s in 3 waves of 256 x 256 against 963 in 3 waves of 128 x 192).
  int BN = g_gemm_bn;
  bool pair = false;
  const int sms = g_gemm_sms > 0 && g_gemm_sms < kNumSMs ? g_gemm_sms : kNumSMs;
  const long long pair_workers = sms / 2;
  const int nkb_host = (int)((K + kBK - 1) / kBK);
  // the k-split schedule needs room for the partial accumulators behind whatever was repacked; dense matmuls only
  // (block matmuls bring hundreds of tiles, and their hinted forms promise bits equal to the unhinted ones)
  const size_t split_off = (ws_off + 255) / 256 * 256;
  const bool split_ok = g_gemm_split && tri == 0 && nbi == 1 && nbo == 1 && ws && !(ws & 255) &&
                        split_off + split_bytes() <= ws_bytes;
  if (!BN) {
    if (N <= 128) BN = 128;
    else {
      const bool mn = a_mn || b_mn;
      double best = 1e300;
      for (int bn : {256, 192, 128}) {
        const long long tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn) * nbi * nbo;
        const double cost = (double)((tiles + kNumSMs - 1) / kNumSMs) * bn * (bn == 128 ? 1.3 : bn == 192 ? 1.08 : 1.0) *
                            (mn ? 1.25 : 1.0);
        if (cost < best * 0.999) { best = cost; BN = bn; }
      }
      if (g_gemm_pair && M > kBM) {
        const long long tiles2 = ((M + kPairBM - 1) / kPairBM) * ((N + kPairBN - 1) / kPairBN) * nbi * nbo;
        double cost = (double)((tiles2 + kNumSMs / 2 - 1) / (kNumSMs / 2)) * kPairBN * 0.93;
        // with the k-split schedule the two-SM grid has no idle last wave (3 % for the partial sums)
        const long long tm2 = (M + kPairBM - 1) / kPairBM, tn2 = (N + kPairBN - 1) / kPairBN;
        if (split_ok && plan_split(tiles2, nkb_host, pair_workers, tn2, pair_group_m(tm2), M, N, K).sk_tiles)
          cost = (double)tiles2 / (double)pair_workers * kPairBN * 0.93 * 1.03;
        if (cost < best) { best = cost; BN = kPairBN; pair = true; }
      }
    }
  } else {
    pair = g_gemm_pair != 0 && BN == kPairBN && M > kBM;
  }
  const int tile_m = pair ? kPairBM : kBM;
  CUtensorMap tmA, tmB;
  // K-major operand: stored [mn][k] -> box {64 k, tile mn}; MN-major: stored [k][mn] -> box {64 mn, 64 k}
  int rc = encode_operand(&tmA, A, nbi, nbo, 64, a_mn ? 64 : kBM, bf16);
  if (rc) return rc;
  rc = encode_operand(&tmB, B, nbi, nbo, 64, b_mn ? 64 : (pair ? BN / 2 : BN), bf16);
  if (rc) return rc;
  GemmParams p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.nb_inner = nbi; p.nb_outer = nbo;
  p.tiles_m = (int)((M + tile_m - 1) / tile_m); p.tiles_n = (int)((N + BN - 1) / BN);
  p.a_j = A.has_j && nbi > 1; p.a_i = A.has_i && nbo > 1; p.b_j = B.has_j && nbi > 1; p.b_i = B.has_i && nbo > 1;
  p.ldc = ldc; p.c_stride_inner = csi; p.c_stride_outer = cso;
  p.alpha = alpha; p.beta = beta;
  p.tri = tri; p.diag = (int)diag;
  p.idesc = (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn ? 1u : 0u) << 15) |
            ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(tile_m >> 4) << 24);
  const uint64_t all = c | (uint64_t)(ldc * 2) | (uint64_t)(nbi > 1 ? csi * 2 : 0) | (uint64_t)(nbo > 1 ? cso * 2 : 0);
  p.c_align = (all & 15) == 0 ? 16 : (all & 7) == 0 ? 8 : (all & 3) == 0 ? 4 : 2;
  // TMA store (and, with beta != 0, TMA load) of C needs a 16-byte aligned base and strides
  CUtensorMap tmC = tmA;
  p.c_tma = 0;
  {
    Operand Co{c, M, N, ldc, csi, cso, nbi > 1, nbo > 1};
    if (tma_ok(Co, nbi, nbo) && (nbi == 1 || csi != 0) && (nbo == 1 || cso != 0)) {
      rc = encode_operand(&tmC, Co, nbi, nbo, 64, 32, bf16);
      if (rc) return rc;
      p.c_tma = 1;
    }
  }
  // about 16 m-tiles of A (2048 rows) stay hot in L2 while the B panels stream
  p.group_m = pair ? (int)pair_group_m(p.tiles_m) : (g_gemm_group_m > 0 ? g_gemm_group_m : 16);
  if (p.group_m > p.tiles_m) p.group_m = p.tiles_m;
  const long long total = (long long)p.tiles_m * p.tiles_n * nbi * nbo;
  // g_gemm_sms < 148 leaves SMs free for a concurrent kernel (the gradient all-reduce): a persistent grid that
  // cannot be fully resident would otherwise run its last CTAs as a second wave
  const int grid = (int)(total < sms ? total : sms);
  p.sk_tiles = 0; p.sk_units = 0; p.sk_part = nullptr; p.sk_slot = 0;
  static std::atomic<unsigned> launch_seq{0};       // flag / counter slot of a launch: consecutive launches use different ones
  p.dyn = (g_gemm_dynamic && total < 0x7fffffffLL) ? 1 : 0;
  if (p.dyn) p.sk_slot = (int)(launch_seq.fetch_add(1) % kSkSlots);
  const int stages = BN >= 192 ? 4 : 6;
  const size_t smem = (size_t)stages * (kBM * kBK * 2 + BN * kBK * 2) + 1024 /*align*/ + 1024 /*barriers*/ + 4 * 8192;
  T* C = reinterpret_cast<T*>(c);
  if (pair) {
    long long pairs = total < sms / 2 ? total : sms / 2;
    if (split_ok) {
      const SplitPlan sp = plan_split(total, nkb_host, pair_workers, p.tiles_n, p.group_m, M, N, K);
      if (sp.sk_tiles) {                                // the k-split walk is static: it replaces the dynamic one
        pairs = sp.workers;
        p.sk_tiles = sp.sk_tiles; p.sk_units = sp.sk_tiles * nkb_host;
        p.sk_part = reinterpret_cast<float*>(ws + split_off);
        if (!p.dyn) p.sk_slot = (int)(launch_seq.fetch_add(1) % kSkSlots);
        p.dyn = 0;
      }
    }
#define CB_GEMM2(AM_, BM_)                                                                             \
  do {                                                                                                 \
    auto kern = gemm_tc_pair_kernel<T, AM_, BM_>;                                                      \
    static bool attr_set[kMaxDevices] = {};                                                                      \
    ensure_dynamic_smem(kern, kPairSmem, attr_set); \
    kern<<<(unsigned)(2 * pairs), kGemmThreads, kPairSmem, st>>>(tmA, tmB, tmC, C, p);                 \
  } while (0)
    if (!a_mn && !b_mn) CB_GEMM2(false, false); else if (!a_mn && b_mn) CB_GEMM2(false, true);
    else if (a_mn && !b_mn) CB_GEMM2(true, false); else CB_GEMM2(true, true);
#undef CB_GEMM2
    return check_launch();
  }
#define CB_GEMM(BN_, AM_, BM_)                                                                         \
  do {                                                                                                 \
    auto kern = gemm_tc_kernel<T, BN_, AM_, BM_>;                                                      \
    static bool attr_set[kMaxDevices] = {};                                                                      \
    ensure_dynamic_smem(kern, smem, attr_set); \
    kern<<<grid, kGemmThreads, smem, st>>>(tmA, tmB, tmC, C, p);                                            \
  } while (0)
  if (BN == 256) {
    if (!a_mn && !b_mn) CB_GEMM(256, false, false); else if (!a_mn && b_mn) CB_GEMM(256, false, true);
    else if (a_mn && !b_mn) CB_GEMM(256, true, false); else CB_GEMM(256, true, true);
  } else if (BN == 192) {
    if (!a_mn && !b_mn) CB_GEMM(192, false, false); else if (!a_mn && b_mn) CB_GEMM(192, false, true);
    else if (a_mn && !b_mn) CB_GEMM(192, true, false); else CB_GEMM(192, true, true);
  } else {
    if (!a_mn && !b_mn) CB_GEMM(128, false, false); else if (!a_mn && b_mn) CB_GEMM(128, false, true);
    else if (a_mn && !b_mn) CB_GEMM(128, true, false); else CB_GEMM(128, true, true);
  }
#undef CB_GEMM
  return check_launch();
}

static int gemm_entry(uint64_t c, uint64_t a, uint64_t b, long long m, long long n, long long k, long long lda,
                      long long ldb, long long ldc, int ta, int tb, const float* alpha, const float* beta, int nbo, int nbi,
                      long long sao, long long sai, long long sbo, long long sbi, long long sco, long long sci, int tri,
                      long long diag, int opflags, int dtype, uint64_t ws, size_t ws_bytes, void* stream) {
  if (m < 0 || n < 0 || k < 0 || nbo < 0 || nbi < 0 || !alpha || !beta) return CACTI_B200_ERR_INVALID_VALUE;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return CACTI_B200_ERR_SHAPE;
  if ((ta & ~1) || (tb & ~1)) return CACTI_B200_ERR_INVALID_VALUE;
  if (tri < CACTI_B200_TRI_NONE || tri > CACTI_B200_TRI_A_UPPER || diag > 0x3fffffffLL || diag < -0x3fffffffLL)
    return CACTI_B200_ERR_INVALID_VALUE;
  if (dtype != CACTI_B200_R_16F && dtype != CACTI_B200_R_16BF) return CACTI_B200_ERR_DTYPE;
  if (m == 0 || n == 0 || nbo == 0 || nbi == 0) return CACTI_B200_OK;
  if (!c || (k > 0 && (!a || !b))) return CACTI_B200_ERR_INVALID_VALUE;
  // stored shapes: A is [m,k] (ta = 0) or [k,m]; B is [k,n] (tb = 0) or [n,k]
  const long long a_rows = ta ? k : m, a_cols = ta ? m : k, b_rows = tb ? n : k, b_cols = tb ? k : n;
  if (lda < a_cols || ldb < b_cols || ldc < n) return CACTI_B200_ERR_INVALID_VALUE;
  if (k == 0) return CACTI_B200_ERR_SHAPE;      // the reference never stages an empty contraction
  Operand A{a, a_rows, a_cols, lda, sai, sao, sai != 0, sao != 0};
  Operand B{b, b_rows, b_cols, ldb, sbi, sbo, sbi != 0, sbo != 0};
  if (nbi == 1) { A.has_j = B.has_j = 0; }
  if (nbo == 1) { A.has_i = B.has_i = 0; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // A as [m][k] is K-major; as [k][m] it is MN-major.  B as [n][k] (tb = 1) is K-major; as [k][n] MN-major.
  const bool a_mn = ta != 0, b_mn = tb == 0;
  if (dtype == CACTI_B200_R_16F)
    return gemm_run<__half>(c, A, B, a_mn, b_mn, m, n, k, ldc, sco, sci, nbi, nbo, *alpha, *beta, tri, diag, opflags, ws, ws_bytes, st);
  return gemm_run<__nv_bfloat16>(c, A, B, a_mn, b_mn, m, n, k, ldc, sco, sci, nbi, nbo, *alpha, *beta, tri, diag, opflags, ws, ws_bytes, st);
}

}  // namespace cb

extern "C" {

size_t cacti_b200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch_outer, int64_t batch_inner) {
  if (m < 0 || n < 0 || k < 0 || batch_outer < 0 || batch_inner < 0) return 0;
  const long long nb = (batch_outer ? batch_outer : 1) * (batch_inner ? batch_inner : 1);
  // worst case: both operands repacked, either orientation
  auto worst = [&](long long r, long long c) {
    const size_t x = cb::packed_bytes(r, c, nb), y = cb::packed_bytes(c, r, nb);
    return x > y ? x : y;
  };
  return worst(m, k) + worst(k, n) + 512 + cb::split_bytes() + 256;
}

int cacti_b200_gemm(cacti_b200_dptr c, cacti_b200_dptr a, cacti_b200_dptr b, int64_t m, int64_t n, int64_t k, int64_t lda,
                    int64_t ldb, int64_t ldc, int trans_a, int trans_b, const float* alpha, const float* beta, int dtype,
                    cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_stream stream) {
  return cb::gemm_entry(c, a, b, m, n, k, lda, ldb, ldc, trans_a, trans_b, alpha, beta, 1, 1, 0, 0, 0, 0, 0, 0,
                        CACTI_B200_TRI_NONE, 0, 0, dtype, workspace, workspace_bytes, stream);
}

int cacti_b200_gemm_strided_batched(cacti_b200_dptr c, cacti_b200_dptr a, cacti_b200_dptr b, int64_t m, int64_t n,
                                    int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                                    const float* alpha, const float* beta, int64_t batch_outer, int64_t batch_inner,
                                    int64_t stride_a_outer, int64_t stride_a_inner, int64_t stride_b_outer,
                                    int64_t stride_b_inner, int64_t stride_c_outer, int64_t stride_c_inner, int dtype,
                                    cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_stream stream) {
  if (batch_outer > 0x7fffffffLL || batch_inner > 0x7fffffffLL) return CACTI_B200_ERR_SHAPE;
  return cb::gemm_entry(c, a, b, m, n, k, lda, ldb, ldc, trans_a, trans_b, alpha, beta, (int)batch_outer, (int)batch_inner,
                        stride_a_outer, stride_a_inner, stride_b_outer, stride_b_inner, stride_c_outer, stride_c_inner,
                        CACTI_B200_TRI_NONE, 0, 0, dtype, workspace, workspace_bytes, stream);
}

int cacti_b200_gemm_strided_batched_tri(cacti_b200_dptr c, cacti_b200_dptr a, cacti_b200_dptr b, int64_t m, int64_t n,
                                        int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                                        const float* alpha, const float* beta, int64_t batch_outer, int64_t batch_inner,
                                        int64_t stride_a_outer, int64_t stride_a_inner, int64_t stride_b_outer,
                                        int64_t stride_b_inner, int64_t stride_c_outer, int64_t stride_c_inner, int tri_mode,
                                        int64_t diag, int operand_flags, int dtype, cacti_b200_dptr workspace,
                                        size_t workspace_bytes,
                                        cacti_b200_stream stream) {
  if (batch_outer > 0x7fffffffLL || batch_inner > 0x7fffffffLL) return CACTI_B200_ERR_SHAPE;
  return cb::gemm_entry(c, a, b, m, n, k, lda, ldb, ldc, trans_a, trans_b, alpha, beta, (int)batch_outer, (int)batch_inner,
                        stride_a_outer, stride_a_inner, stride_b_outer, stride_b_inner, stride_c_outer, stride_c_inner,
                        tri_mode, diag, operand_flags, dtype, workspace, workspace_bytes, stream);
}
}
