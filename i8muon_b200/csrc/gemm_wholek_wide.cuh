// Whole-K GEMM kernel with 128 x 256 work units.
//
// A 128 x 128 tcgen05.mma tile reads 8 KB of shared memory per 64 tensor cycles and the producer
// writes as much: wholek_persistent_kernel keeps the tensor pipe 65 % busy and shared memory is the
// unit that saturates.  Here one work unit is a pair of output tiles (tm, tn) and (tm, tn + 1):
// one 128-row left tile and two adjacent 128-row right tiles per K block, one N = 256 instruction
// per 32 bytes of K, so a quarter less shared-memory traffic per multiply-add.  A row of tiles with
// an odd count ends in a unit of one tile (N = 128).
//
//   warp 0          TMA producer: {left, right, right + 1} tiles into a four-stage ring (48 KB each)
//   warp 1          tcgen05.mma issuer: all K blocks of a unit into one 256-column accumulator,
//                   in order, by one thread (fixed floating accumulation order)
//   warps 4..11     epilogue: the unit's tiles one after the other through the same fused
//                   epilogues as wholek_persistent_kernel (two warps per TMEM lane quarter)
// Two 256-column accumulators (all of tensor memory) ping-pong between the issuer and the epilogue
// warps.  Every wait is bounded; a role that gives up posts its code in the status word, sets the
// abort flag and the other roles leave at their next poll.
#pragma once
#include "gemm_wholek_persistent.cuh"

namespace i8m {

constexpr int WKW_STAGES = 4;
constexpr int WKW_STAGE_BYTES = 3 * TILE_BYTES;
constexpr int WKW_THREADS = 384;
constexpr int WKW_NBUF = 2;
constexpr int WKW_ACC_COLS = 2 * TILE;

// Units of one batch element.  Symmetric products: row i of the lower triangle holds tiles 0..i,
// (i + 2) / 2 units; before row i there are p (p + 1) units for i = 2 p and (p + 1)^2 for i = 2 p + 1.
__host__ __device__ inline int wide_units_before_row(int i) {
  const int p = i >> 1;
  return (i & 1) ? (p + 1) * (p + 1) : p * (p + 1);
}
__host__ __device__ inline int wide_units_per_batch(int tiles_m, int tiles_n, int sym) {
  return sym ? wide_units_before_row(tiles_m) : tiles_m * ((tiles_n + 1) / 2);
}

// Order of the units.  Row blocks are taken in groups of g.group and a group is walked column by
// column, so the units in flight (one per SM, consecutive indices) share the group's left row
// blocks, which stay in L2 for the whole sweep, and the right operand streams through once per
// group.  (In plain row-major order of the triangle, row i of a symmetric product re-reads row
// blocks 0..i of the right operand, a cyclic pattern that an LRU cache larger than L2 never hits.)
// In a symmetric product a group of rows r0 .. r0 + R - 1 has r0 / 2 + 1 full columns of units and
// then columns of R - 2, R - 4, ... units (rows tm >= 2 tw only).
__host__ __device__ __forceinline__ void decode_unit(const GemmGeom& g, int units_per_batch, int linear, int& b,
                                                     int& tm, int& tn, int& width) {
  b = linear / units_per_batch;
  int u = linear - b * units_per_batch;
  const int group = g.group;   // even, >= 2
  if (g.sym) {
    // the group that holds u: groups are whole rows, so the row search of the triangle finds it
    int i = int(2.f * sqrtf(float(u)));
    if (i > g.tiles_m - 1) i = g.tiles_m - 1;
    while (i + 1 < g.tiles_m && wide_units_before_row(i + 1) <= u) ++i;
    while (i > 0 && wide_units_before_row(i) > u) --i;
    const int r0 = i / group * group;
    const int rows = g.tiles_m - r0 < group ? g.tiles_m - r0 : group;
    u -= wide_units_before_row(r0);
    const int full = r0 / 2 + 1;
    int tw;
    if (u < full * rows) {
      tw = u / rows;
      tm = r0 + (u - tw * rows);
    } else {
      u -= full * rows;
      tw = full;
      int n = rows - 2;
      while (u >= n && n > 0) { u -= n; n -= 2; ++tw; }
      tm = 2 * tw + u;
    }
    tn = 2 * tw;
    width = tn + 1 <= tm ? 2 : 1;
  } else {
    const int cols = (g.tiles_n + 1) / 2;
    const int per_group = group * cols;
    const int grp = u / per_group;
    const int in_group = u - grp * per_group;
    const int rows = g.tiles_m - grp * group < group ? g.tiles_m - grp * group : group;
    const int tw = in_group / rows;
    tm = grp * group + (in_group - tw * rows);
    tn = 2 * tw;
    width = tn + 1 < g.tiles_n ? 2 : 1;
  }
}

template <class Epi>
constexpr size_t wholek_wide_smem_bytes() {
  // after the control block: the staging tile of an epilogue with a tile tail, or one transpose
  // patch per epilogue warp
  size_t tail = 8 * WARP_PATCH_BYTES;
  if constexpr (WholekTileSync<Epi>::value) tail = Epi::TSM_BYTES;
  return size_t(WKW_STAGES) * WKW_STAGE_BYTES + sizeof(Ctrl) + tail + 1024;
}

template <class Epi>
__global__ void __launch_bounds__(WKW_THREADS, 1)
wholek_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   GemmGeom g, typename Epi::Args args) {
  constexpr int STAGES = WKW_STAGES;
  constexpr int STAGE_BYTES = WKW_STAGE_BYTES;
  constexpr int NBUF = WKW_NBUF;
  constexpr int BKE = 128 / int(sizeof(typename Epi::Elem));  // elements per 128-byte K block
  static_assert(Epi::PARTS == 1 && Epi::PROMOTE_KB == 0 && !Epi::BLOCKQ, "whole-K epilogues only");
  // the same instruction descriptor with N = 256
  constexpr uint32_t IDESC_WIDE = (Epi::IDESC & ~(0x3Fu << 17)) | (uint32_t(WKW_ACC_COLS >> 3) << 17);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * STAGE_BYTES);
  uint8_t* tsm = reinterpret_cast<uint8_t*>(ctrl + 1);   // staging tile of epilogues that have a tile tail
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int i = 0; i < NBUF; ++i) {
      mbar_init(smem_u32(&ctrl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[i]), 8);  // one arrival per epilogue warp
    }
    ctrl->abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), WKW_ACC_COLS * NBUF);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  volatile uint32_t* abort_flag = &ctrl->abort;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
  const uint32_t accf0 = smem_u32(&ctrl->acc_full[0]), acce0 = smem_u32(&ctrl->acc_empty[0]);

  const int upb = wide_units_per_batch(g.tiles_m, g.tiles_n, g.sym);
  const int total_units = upb * g.batch;
  const int my_units = (total_units - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
  const int nkb = g.num_kb;

  if (warp < 4) {
    setmaxnreg_dec<WKP_CTRL_REGS>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------ producer
      int ring = 0;
      uint32_t wrap = 0;
      int issued = 0;
      bool ok = true;
      // test hook (i8m_set_debug_core(2)): issue nothing, so that every consumer's bounded wait runs out
      const int units = (g.debug_simt & 0x100) ? 0 : my_units;
      for (int j = 0; j < units && ok; ++j) {
        int b, tm, tn, width;
        decode_unit(g, upb, int(blockIdx.x) + j * int(gridDim.x), b, tm, tn, width);
        const uint32_t bytes = uint32_t(1 + width) * TILE_BYTES;
        for (int kb = 0; kb < nkb; ++kb) {
          if (wrap > 0) {
            ok = mbar_wait(empty0 + 8u * uint32_t(ring), (wrap - 1) & 1u, abort_flag);
            if (!ok) break;
          }
          const uint32_t bar = full0 + 8u * uint32_t(ring);
          const uint32_t dst = smem_base + uint32_t(ring * STAGE_BYTES);
          mbar_arrive_expect_tx(bar, bytes);
          tma_load_3d(dst, &map_a, bar, kb * BKE, tm * TILE, b);
          tma_load_3d(dst + TILE_BYTES, &map_b, bar, kb * BKE, tn * TILE, b);
          if (width == 2) tma_load_3d(dst + 2 * TILE_BYTES, &map_b, bar, kb * BKE, (tn + 1) * TILE, b);
          ++issued;
          if (++ring == STAGES) { ring = 0; ++wrap; }
        }
      }
      if (!ok) {
        atomicCAS(g.status, 0u, unsigned(ST_PRODUCER_TIMEOUT) | unsigned(blockIdx.x & 0xff));
        // let the copies that were issued land before shared memory is released
        for (int back = 0; back < STAGES && back < issued; ++back) {
          const int n = issued - 1 - back;
          const uint32_t parity = uint32_t(n / STAGES) & 1u;
          const uint32_t bar = full0 + 8u * uint32_t(n % STAGES);
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, parity); ++spin) {
          }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------- MMA issuer
      int ring = 0;
      uint32_t wrap = 0;
      bool ok = true;
      for (int j = 0; j < my_units && ok; ++j) {
        int b, tm, tn, width;
        decode_unit(g, upb, int(blockIdx.x) + j * int(gridDim.x), b, tm, tn, width);
        const uint32_t idesc = width == 2 ? IDESC_WIDE : Epi::IDESC;
        const int buf = j & 1;
        const uint32_t use = uint32_t(j >> 1);  // how often this accumulator was filled before
        if (use >= 1) {
          ok = mbar_wait(acce0 + 8u * uint32_t(buf), (use - 1) & 1u, abort_flag);
          if (!ok) break;
        }
        const uint32_t d = tmem_base + uint32_t(buf * WKW_ACC_COLS);
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(full0 + 8u * uint32_t(ring), wrap & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + uint32_t(ring * STAGE_BYTES);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + TILE_BYTES);   // 128 or 256 rows, 8-row groups 1 KB apart
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t accumulate = (kb == 0 && ks == 0) ? 0u : 1u;
            umma<Epi::KIND>(d, adesc + uint64_t(ks * 2), bdesc + uint64_t(ks * 2), idesc, accumulate);
          }
          umma_commit(empty0 + 8u * uint32_t(ring));
          if (++ring == STAGES) { ring = 0; ++wrap; }
        }
        if (ok) umma_commit(accf0 + 8u * uint32_t(buf));
      }
      if (!ok) atomicCAS(g.status, 0u, unsigned(ST_MMA_TIMEOUT) | unsigned(blockIdx.x & 0xff));
    }
  } else {
    // -------------------------------------------------------------- epilogue
    setmaxnreg_inc<WKP_EPI_REGS>();
    TileCtx t;
    t.q = warp & 3; t.lane = lane;
    t.ew = warp - 4; t.half = (warp - 4) >> 2;
    t.r = t.q * 32 + lane;
    t.ctrl = ctrl;
    t.red = ctrl->red; t.diag = ctrl->diag;
    t.tsm = WholekTileSync<Epi>::value ? tsm : nullptr;
    t.wsm = WholekTileSync<Epi>::value ? nullptr : tsm + t.ew * WARP_PATCH_BYTES;
    t.c_begin = t.half * 2; t.c_end = t.half * 2 + 2;
    bool ok = true;
    uint32_t tiles_done = 0;
    for (int j = 0; j < my_units; ++j) {
      int tn0, width;
      decode_unit(g, upb, int(blockIdx.x) + j * int(gridDim.x), t.b, t.tm, tn0, width);
      t.row0 = t.tm * TILE;
      t.row = t.row0 + t.r;
      const int buf = j & 1;
      if (ok) ok = mbar_wait_warp(accf0 + 8u * uint32_t(buf), uint32_t(j >> 1) & 1u, abort_flag);
      if (ok) tc_fence_after();
      for (int sub = 0; sub < width; ++sub, ++tiles_done) {
        t.tn = tn0 + sub;
        t.col0 = t.tn * TILE;
        const uint32_t taddr = tmem_base + (uint32_t(t.q * 32) << 16) + uint32_t(buf * WKW_ACC_COLS + sub * TILE);
        AccWholeK<Epi::KIND, typename Epi::Elem, false> acc{g, t, taddr};
        if constexpr (WholekTileSync<Epi>::value) {
          // this epilogue's tile tail meets on named barriers: a warp that gave up walks through
          // them too (without loading or storing), so the others can never wait for it
          t.red = ctrl->red2[tiles_done & 1u];
          Epi::run_sync(g, args, t, acc, ok);
        } else {
          if (ok) Epi::run(g, args, t, acc);
        }
      }
      if (ok) {
        tc_fence_before();
        __syncwarp();
        mbar_arrive_if(acce0 + 8u * uint32_t(buf), lane == 0 ? 1u : 0u);
      }
    }
    if (!ok && lane == 0)
      atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, WKW_ACC_COLS * NBUF);
}

}  // namespace i8m
