// Warp-specialised batched GEMM skeleton for sm_100a:  C[b] = A[b] * Bt[b]^T
//
//   A  is (batch, m, k) row-major  -> "K-major" operand tile of 128 rows
//   Bt is (batch, n, k) row-major  -> rows of B^T, also K-major
//
// One CTA produces one 128 x 128 output tile.
//   warp 0      TMA producer: cp.async.bulk.tensor 3-D boxes {128 bytes of K, 128 rows, 1 batch}
//               with the 128-byte swizzle into a STAGES-deep shared-memory ring
//   warp 1      allocates tensor memory and issues tcgen05.mma (one elected thread)
//   warps 2..5  epilogue: tcgen05.ld the accumulator rows and run the fused epilogue
//
// Two accumulator disciplines:
//   * whole-K accumulation (floating point and global-scale INT8): one 128-column
//     accumulator, epilogue runs once after the last K block;
//   * per-K-block promotion (128x128 block-quantised INT8 / E4M3): every 128-deep
//     K block lands in a fresh accumulator (two TMEM buffers, ping-pong) and the
//     epilogue warps fold it into FP32 registers with the block scales while the
//     tensor core works on the next block.
//
// A debug core (geom.debug_simt) replaces TMA/tcgen05 by plain global-memory dot
// products inside the epilogue threads, so that epilogue logic can be validated
// independently of the tensor pipeline.  It is selected only by tests.
#pragma once
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace i8m {

constexpr int TILE = 128;            // CTA tile is TILE x TILE
constexpr int TILE_BYTES = TILE * 128;  // one operand tile of one stage (128 rows x 128 B)
constexpr int GEMM_THREADS = 192;  // default: 2 control warps + 4 epilogue warps

// Error codes written to the status word (first error wins).
enum StatusCode : unsigned {
  ST_OK = 0,
  ST_PRODUCER_TIMEOUT = 0x100,
  ST_MMA_TIMEOUT = 0x200,
  ST_EPILOGUE_TIMEOUT = 0x300,
  ST_TAIL_TIMEOUT = 0x400,
};

struct GemmGeom {
  int batch;
  int m, n, k;          // padded operand extents (elements)
  int lm, ln;           // logical output extent
  int tiles_m, tiles_n;
  int sym;              // 1: only tiles with tm >= tn are computed
  int tiles_per_batch;
  int num_kb;           // K blocks of 128 bytes
  int debug_simt;
  int group;            // row blocks per group of the tile / unit order (even, >= 8; set by the launcher)
  const void* a_raw;    // raw operand pointers (debug core and epilogue reads)
  const void* b_raw;
  unsigned* status;
};

struct alignas(16) Ctrl {
  unsigned long long full[8];
  unsigned long long empty[8];
  unsigned long long acc_full[4];
  unsigned long long acc_empty[4];
  uint32_t tmem_base;
  uint32_t abort;
  float red[8];
  int redi[8];
  float diag[TILE];
  float red2[2][8];
  // split-tail kernel: the tile's FP32 totals parked in shared memory (full: 8 fold warps arrive,
  // empty: 4 tail warps arrive), and the tail warps' own rendezvous (4 arrivals)
  unsigned long long park_full, park_empty, tail_sync, pad_;
};

struct TileCtx {
  int b, tm, tn, row0, col0;
  int r;        // row inside the tile owned by this epilogue thread
  int row;      // global row
  int q;        // TMEM lane quarter of this warp
  int half;     // column slice of this warp when a row is split over several warps
  int ew;       // epilogue warp index (0 .. EPI_WARPS-1)
  int lane;
  int c_begin, c_end;  // 32-column chunks of the tile row that this thread handles (whole-K epilogues)
  Ctrl* ctrl;
  float* red;   // shared scratch for the tile-wide reduction (one float per epilogue warp)
  float* diag;  // shared scratch: TILE floats
  uint8_t* tsm; // shared staging tile for transposed stores, or nullptr
  uint8_t* wsm; // this warp's own WARP_PATCH_BYTES of shared memory (32 x 32 transposes), or nullptr
};

// A warp's private patch of shared memory: 32 rows of 64 bytes, the 16-byte pieces of a row
// XOR-swizzled with the row number (see WarpPatch) so that the three access patterns of the
// epilogues are all free of bank conflicts.
constexpr int WARP_PATCH_BYTES = 32 * 64;

__host__ __device__ __forceinline__ void decode_tile(const GemmGeom& g, int linear, int& b, int& tm,
                                                     int& tn) {
  b = linear / g.tiles_per_batch;
  int t = linear - b * g.tiles_per_batch;
  if (g.sym) {
    int i = int((sqrtf(float(8 * t + 1)) - 1.f) * 0.5f);
    while ((i + 1) * (i + 2) / 2 <= t) ++i;
    while (i * (i + 1) / 2 > t) --i;
    tm = i;
    tn = t - i * (i + 1) / 2;
  } else {
    // Row blocks are taken in groups and walked column-major inside a group, so
    // that the tiles in flight at one time (one or two per SM, consecutive indices) share few
    // row blocks of both operands: with row-major order the 296 tiles of a wave spanned every
    // column block and the right operand was re-read from DRAM once per 2.6 row blocks
    // (1.4 GB read for 0.27 GB of operands on the 4096 x 14336 FP16 update).
    // g.group row blocks per group: as many as keep the group's left row blocks in L2 (at least 8).
    const int group = g.group;
    const int per_group = group * g.tiles_n;
    const int grp = t / per_group;
    const int in_group = t - grp * per_group;
    const int left = g.tiles_m - grp * group;
    const int rows = left < group ? left : group;
    tn = in_group / rows;
    tm = grp * group + (in_group - tn * rows);
  }
}

// ----------------------------------------------------- element conversions
template <int KIND, typename Elem>
struct ElemOps;
template <>
struct ElemOps<KIND_F16, __half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
};
template <>
struct ElemOps<KIND_F16, __nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
};

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(__half(h));
}

// Debug core: direct dot product over K range [k0, k1) of row `row` of A and
// row `col` of Bt, returned as the raw 32-bit accumulator pattern.
template <int KIND, typename Elem>
__device__ inline uint32_t simt_dot(const GemmGeom& g, int b, int row, int col, int k0, int k1) {
  if (row >= g.m || col >= g.n) return 0u;
  const Elem* a = static_cast<const Elem*>(g.a_raw) + (size_t(b) * g.m + row) * g.k;
  const Elem* bt = static_cast<const Elem*>(g.b_raw) + (size_t(b) * g.n + col) * g.k;
  if (k1 > g.k) k1 = g.k;
  if constexpr (KIND == KIND_I8) {
    int acc = 0;
    for (int kk = k0; kk < k1; ++kk) acc += int(int8_t(a[kk])) * int(int8_t(bt[kk]));
    return uint32_t(acc);
  } else if constexpr (KIND == KIND_F8) {
    float acc = 0.f;
    for (int kk = k0; kk < k1; ++kk)
      acc = fmaf(e4m3_to_float(uint8_t(a[kk])), e4m3_to_float(uint8_t(bt[kk])), acc);
    return __float_as_uint(acc);
  } else if constexpr (KIND == KIND_TF32) {
    float acc = 0.f;
    for (int kk = k0; kk < k1; ++kk) acc = fmaf(float(a[kk]), float(bt[kk]), acc);
    return __float_as_uint(acc);
  } else {
    float acc = 0.f;
    for (int kk = k0; kk < k1; ++kk) acc = fmaf(float(a[kk]), float(bt[kk]), acc);
    return __float_as_uint(acc);
  }
}

// ------------------------------------------------------------ accumulators
// Whole-K accumulator: chunk c = columns [32c, 32c+32) of this thread's row.
template <int KIND, typename Elem, bool DEBUG>
struct AccWholeK {
  static constexpr bool IN_REGS = false;
  const GemmGeom& g;
  const TileCtx& t;
  uint32_t taddr;  // TMEM address of (lane quarter base, column 0)
  __device__ __forceinline__ void load(int c, uint32_t (&v)[32]) const {
    if constexpr (DEBUG) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        v[j] = simt_dot<KIND, Elem>(g, t.b, t.row, t.col0 + c * 32 + j, 0, g.k);
    } else {
      __syncwarp();  // tcgen05.ld is warp-collective: reconverge after masked stores
      tmem_ld32(taddr + uint32_t(c * 32), v);
      tmem_wait_ld();
    }
  }
};

// Accumulator already folded into registers (chunked promotion): same chunk
// interface, compile-time indexing so that the array stays in registers.
struct AccRegs {
  static constexpr bool IN_REGS = true;
  const float (&total)[TILE];
  __device__ __forceinline__ void load(int c, uint32_t (&v)[32]) const {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(total[c * 32 + j]);
  }
};

// ------------------------------------------------------------------ kernel
// Epi supplies:
//   KIND, Elem, PARTS (operand planes per side: 1, or 2 for split-TF32),
//   PROMOTE_KB (0: the whole K extent accumulates in tensor memory; n > 0: every n
//   K blocks the partial accumulator is folded into FP32 registers by the epilogue
//   warps while the tensor core fills the other TMEM buffer), BLOCKQ (block-quantised
//   epilogue: only its debug core runs here), STAGES, MIN_CTAS, IDESC, struct Args,
//   static __device__ void run(g, args, t, acc)   (whole-K and chunked promotion)
//   static __device__ void run_debug(g, args, t)  (BLOCKQ)
// DEBUG = true is the test-only core: no TMA / tcgen05, the epilogue threads compute
// plain dot products.  It is a separate instantiation so that the product kernels
// carry none of its code or register pressure.
// Warp layout: warp 0 producer, warp 1 MMA issuer, then the epilogue warps: four of them
// are warps 2..5; eight start at warp 4 so that every epilogue warp w reads the TMEM lane
// quarter w % 4.  The block-quantised epilogues (eight warps) run in this skeleton only with
// the debug core; their product kernel is bq_persistent_kernel.
template <class Epi>
struct WarpLayout {
  static constexpr int EPI_WARP0 = Epi::EPI_WARPS > 4 ? 4 : 2;
  static constexpr int THREADS = 32 * (EPI_WARP0 + Epi::EPI_WARPS);
};

template <class Epi, bool DEBUG>
__global__ void __launch_bounds__(WarpLayout<Epi>::THREADS, Epi::MIN_CTAS)
ns_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
               GemmGeom g, typename Epi::Args args) {
  constexpr int STAGES = Epi::STAGES;
  constexpr int PARTS = Epi::PARTS;
  constexpr int STAGE_BYTES = 2 * PARTS * TILE_BYTES;
  constexpr int PROMOTE = Epi::PROMOTE_KB;
  constexpr int NBUF = Epi::NBUF;          // TMEM accumulators of 128 columns
  constexpr int TMEM_COLS = 128 * NBUF;
  static_assert(NBUF == 1 || NBUF == 2 || NBUF == 4, "TMEM allocations are powers of two");
  constexpr int BKE = 128 / int(sizeof(typename Epi::Elem));  // elements per 128-byte K block

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int b, tm, tn;
  decode_tile(g, blockIdx.x, b, tm, tn);
  const int row0 = tm * TILE, col0 = tn * TILE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&ctrl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[i]), Epi::EPI_WARPS);  // one arrival per epilogue warp
    }
    ctrl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  volatile uint32_t* abort_flag = &ctrl->abort;
  const uint32_t smem_base = smem_u32(smem);
  constexpr int EPI_WARP0 = WarpLayout<Epi>::EPI_WARP0;

  static_assert(!Epi::BLOCKQ || DEBUG, "block-quantised GEMMs run in bq_persistent_kernel");
  if (warp < EPI_WARP0) {
  if (!DEBUG && warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int issued = 0;
    bool ok = true;
    for (int kb = 0; kb < g.num_kb; ++kb) {
      const int s = kb % STAGES;
      if (kb >= STAGES) {
        ok = mbar_wait(smem_u32(&ctrl->empty[s]), uint32_t((kb / STAGES) - 1) & 1u, abort_flag);
        if (!ok) break;
      }
      const uint32_t bar = smem_u32(&ctrl->full[s]);
      const uint32_t dst = smem_base + uint32_t(s * STAGE_BYTES);
      mbar_arrive_expect_tx(bar, STAGE_BYTES);
      tma_load_3d(dst, &map_a, bar, kb * BKE, row0, b);
      tma_load_3d(dst + PARTS * TILE_BYTES, &map_b, bar, kb * BKE, col0, b);
      if constexpr (PARTS == 2) {
        tma_load_3d(dst + TILE_BYTES, &map_a2, bar, kb * BKE, row0, b);
        tma_load_3d(dst + 3 * TILE_BYTES, &map_b2, bar, kb * BKE, col0, b);
      }
      issued = kb + 1;
    }
    if (!ok) {
      atomicCAS(g.status, 0u, unsigned(ST_PRODUCER_TIMEOUT) | unsigned(blockIdx.x & 0xff));
      // Let the copies that were issued land before shared memory is released.
      int first = issued > STAGES ? issued - STAGES : 0;
      for (int kb = first; kb < issued; ++kb) {
        uint32_t bar = smem_u32(&ctrl->full[kb % STAGES]);
        uint32_t parity = uint32_t(kb / STAGES) & 1u;
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, parity); ++spin) {
        }
      }
    }
  } else if (!DEBUG && warp == 1 && lane == 0) {
    // ---------------------------------------------------------- MMA issuer
    bool ok = true;
    for (int kb = 0; kb < g.num_kb; ++kb) {
      const int s = kb % STAGES;
      ok = mbar_wait(smem_u32(&ctrl->full[s]), uint32_t(kb / STAGES) & 1u, abort_flag);
      if (!ok) break;
      uint32_t d = tmem_base;
      bool chunk_first = kb == 0, chunk_last = false;
      int buf = 0;
      if constexpr (PROMOTE > 0) {
        const int chunk = kb / PROMOTE;
        buf = chunk % NBUF;
        const int use = chunk / NBUF;  // how often this buffer has been filled before
        chunk_first = (kb % PROMOTE) == 0;
        chunk_last = (kb % PROMOTE) == PROMOTE - 1 || kb == g.num_kb - 1;
        if (chunk_first) {
          // a buffer is free until its first reuse
          if (use >= 1)
            ok = mbar_wait(smem_u32(&ctrl->acc_empty[buf]), uint32_t(use - 1) & 1u, abort_flag);
          if (!ok) break;
        }
        d = tmem_base + uint32_t(buf * TILE);
      }
      tc_fence_after();
      const uint32_t sa = smem_base + uint32_t(s * STAGE_BYTES);
      const uint32_t sb = sa + PARTS * TILE_BYTES;
      const uint64_t adesc = make_smem_desc_sw128(sa);
      const uint64_t bdesc = make_smem_desc_sw128(sb);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        // 32 bytes of K per instruction: advance the start address inside the
        // 128-byte swizzle row (address field is in 16-byte units).
        const uint64_t adv = uint64_t(ks * 2);
        uint32_t accumulate = (chunk_first && ks == 0) ? 0u : 1u;
        umma<Epi::KIND>(d, adesc + adv, bdesc + adv, Epi::IDESC, accumulate);
        if constexpr (PARTS == 2) {
          // split-TF32: hi*hi (above) + hi*lo + lo*hi
          const uint64_t a2 = make_smem_desc_sw128(sa + TILE_BYTES) + adv;
          const uint64_t b2 = make_smem_desc_sw128(sb + TILE_BYTES) + adv;
          umma<Epi::KIND>(d, adesc + adv, b2, Epi::IDESC, 1u);
          umma<Epi::KIND>(d, a2, bdesc + adv, Epi::IDESC, 1u);
#ifdef I8M_TF32_LOLO
          umma<Epi::KIND>(d, a2, b2, Epi::IDESC, 1u);
#endif
        }
      }
      umma_commit(smem_u32(&ctrl->empty[s]));
      if constexpr (PROMOTE > 0) {
        if (chunk_last) umma_commit(smem_u32(&ctrl->acc_full[buf]));
      }
    }
    if constexpr (PROMOTE == 0) {
      if (ok) umma_commit(smem_u32(&ctrl->acc_full[0]));
    }
    if (!ok) atomicCAS(g.status, 0u, unsigned(ST_MMA_TIMEOUT) | unsigned(blockIdx.x & 0xff));
  }
  } else {
    // ------------------------------------------------------------ epilogue
    TileCtx t;
    t.b = b; t.tm = tm; t.tn = tn; t.row0 = row0; t.col0 = col0;
    t.q = warp & 3; t.lane = lane;
    t.ew = warp - EPI_WARP0; t.half = (warp - EPI_WARP0) >> 2;
    t.r = t.q * 32 + lane;
    t.row = row0 + t.r;
    t.ctrl = ctrl;
    t.red = ctrl->red; t.diag = ctrl->diag; t.tsm = nullptr; t.wsm = nullptr;
    t.c_begin = 0; t.c_end = TILE / 32;
    const uint32_t taddr = tmem_base + (uint32_t(t.q * 32) << 16);
    if constexpr (Epi::BLOCKQ) {
      Epi::run_debug(g, args, t);
    } else if constexpr (PROMOTE > 0) {
      if constexpr (DEBUG) {
        AccWholeK<Epi::KIND, typename Epi::Elem, true> acc{g, t, taddr};
        Epi::run(g, args, t, acc);
      } else {
        // Chunked promotion: the tensor core accumulates with truncation, so a
        // long K extent is folded into registers (round-to-nearest adds) every
        // PROMOTE K blocks.
        float total[TILE];
#pragma unroll
        for (int j = 0; j < TILE; ++j) total[j] = 0.f;
        const int chunks = (g.num_kb + PROMOTE - 1) / PROMOTE;
        bool ok = true;
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          const int buf = c % NBUF;
          ok = mbar_wait(smem_u32(&ctrl->acc_full[buf]), uint32_t(c / NBUF) & 1u, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < TILE / 32; ++cc) {
            uint32_t v[32];
            tmem_ld32(taddr + uint32_t(buf * TILE + cc * 32), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) total[cc * 32 + j] = __fadd_rn(total[cc * 32 + j], __uint_as_float(v[j]));
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty[buf]));
        }
        if (ok) {
          AccRegs acc{total};
          Epi::run(g, args, t, acc);
        } else if (lane == 0) {
          atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
        }
      }
    } else {
      bool ok = true;
      if constexpr (!DEBUG) {
        ok = mbar_wait(smem_u32(&ctrl->acc_full[0]), 0u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);  // keep the warp together for tcgen05.ld
        tc_fence_after();
      }
      if (ok) {
        AccWholeK<Epi::KIND, typename Epi::Elem, DEBUG> acc{g, t, taddr};
        Epi::run(g, args, t, acc);
      } else if (lane == 0) {
        atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------ store helpers
// Store `count` (<= 32) consecutive elements; vectorised when the destination
// is 16-byte aligned and the chunk is complete.
template <typename T>
__device__ __forceinline__ void store_row(T* dst, const T (&vals)[32], int count) {
  if (count == 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
    constexpr int VEC = 16 / int(sizeof(T));
    const uint4* src = reinterpret_cast<const uint4*>(vals);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 32 / VEC; ++i) d4[i] = src[i];
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < count) dst[j] = vals[j];
  }
}

// A 32 x 64-byte block (32 x 32 values of 16 bits, or 32 x 16 of 32 bits) that a warp re-shapes
// through its patch, so that every global access of an epilogue is coalesced:
//   own rows      lane r reads / writes row r, four 16-byte pieces (the layout the accumulator
//                 arrives in: one tile row per lane);
//   row sweep j   lanes 4 s .. 4 s + 3 hold the four pieces of row 8 j + s: one request covers
//                 eight rows of 64 contiguous bytes (instead of 32 rows of 16 bytes);
//   column sweep i (16-bit values) lane (s, a) = (lane >> 2, lane & 3) gathers rows 8 a .. 8 a + 7
//                 of column 8 i + s: 16 bytes of the transposed block, again eight segments of 64
//                 contiguous bytes per request.
// Piece p of row r lives at r * 64 + ((p ^ (r >> 1) ^ (r >> 3)) & 3) * 16.
struct WarpPatch {
  uint32_t base;
  int lane;
  __device__ __forceinline__ uint32_t piece(int r, int p) const {
    return base + uint32_t(r * 64 + (((p ^ (r >> 1) ^ (r >> 3)) & 3) << 4));
  }
  __device__ __forceinline__ void write_own_row(const uint32_t (&p)[16]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) sts128u(piece(lane, i), make_uint4(p[4 * i], p[4 * i + 1], p[4 * i + 2], p[4 * i + 3]));
  }
  __device__ __forceinline__ void read_own_row(uint32_t (&p)[16]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = lds128u(piece(lane, i));
      p[4 * i] = v.x; p[4 * i + 1] = v.y; p[4 * i + 2] = v.z; p[4 * i + 3] = v.w;
    }
  }
  // row sweep: this lane's 16 bytes of request j (row 8 j + (lane >> 2), piece lane & 3)
  __device__ __forceinline__ int sweep_row(int j) const { return 8 * j + (lane >> 2); }
  __device__ __forceinline__ uint4 read_sweep(int j) const { return lds128u(piece(sweep_row(j), lane & 3)); }
  __device__ __forceinline__ void write_sweep(int j, uint4 v) const { sts128u(piece(sweep_row(j), lane & 3), v); }
  // column sweep of 16-bit values: rows 8 (lane & 3) .. + 7 of column 8 i + (lane >> 2)
  __device__ __forceinline__ uint4 read_column(int i) const {
    const int r0 = 8 * (lane & 3);
    const uint32_t within = uint32_t((lane >> 2) * 2);
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t lo = lds16u(piece(r0 + 2 * k, i) + within);
      const uint32_t hi = lds16u(piece(r0 + 2 * k + 1, i) + within);
      w[k] = lo | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Row-major store of a warp's 32 x 64-byte block held one row per lane: through the patch, as four
// requests of eight 64-byte row segments.  dst = address of the block's first byte, pitch in bytes.
__device__ __forceinline__ void store_block_rows(const WarpPatch& wp, uint8_t* dst, size_t pitch) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(dst + size_t(wp.sweep_row(j)) * pitch + 16 * (wp.lane & 3)) = wp.read_sweep(j);
}
// Transposed store of a block of 16-bit values that sits in the patch: column c of the block
// becomes 64 contiguous bytes at dst + c * pitch.
__device__ __forceinline__ void store_block_columns16(const WarpPatch& wp, uint8_t* dst, size_t pitch) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(dst + size_t(8 * i + (wp.lane >> 2)) * pitch + 16 * (wp.lane & 3)) = wp.read_column(i);
}
// Row-major load of a 32 x 32-byte block (int8 companions) into pieces 0 and 1 of the patch rows:
// two requests of sixteen 32-byte row segments; afterwards lane r finds its row in pieces 0, 1.
__device__ __forceinline__ void load_block_rows32(const WarpPatch& wp, const uint8_t* src, size_t pitch) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = 16 * j + (wp.lane >> 1);
    sts128u(wp.piece(r, wp.lane & 1), *reinterpret_cast<const uint4*>(src + size_t(r) * pitch + 16 * (wp.lane & 1)));
  }
}
// Row-major load of a 32 x 64-byte block into the patch (four coalesced requests).
__device__ __forceinline__ void load_block_rows(const WarpPatch& wp, const uint8_t* src, size_t pitch) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    wp.write_sweep(j, *reinterpret_cast<const uint4*>(src + size_t(wp.sweep_row(j)) * pitch + 16 * (wp.lane & 3)));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_max_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Finite non-negative floats order like their bit patterns.
__device__ __forceinline__ void atomic_max_nonneg(float* p, float v) {
  atomicMax(reinterpret_cast<int*>(p), __float_as_int(v));
}

}  // namespace i8m
