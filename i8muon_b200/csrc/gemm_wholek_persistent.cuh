// Persistent kernel for the GEMMs whose whole K extent accumulates in tensor memory:
// FP16 / BF16 products (regular and Gram-space Newton-Schulz, the FP16 first iteration of
// the quantised routes) and the global-scale INT8 products.
//
// One CTA per SM walks a static round-robin list of 128x128 output tiles.
//   Two independent streams of tiles (tiles 0, 2, 4, ... and 1, 3, 5, ... of this CTA's list),
//   each with its own producer, issuer, three shared-memory stages and two accumulators:
//   warps 0 / 2     TMA producer of stream 0 / 1
//   warps 1 / 3     tcgen05.mma issuer of stream 0 / 1: all K blocks of a tile into one
//                   128-column accumulator, in order, by one thread, so that the floating
//                   accumulation order is fixed.  One issuing thread cannot keep the tensor
//                   pipe busy (issue is nearly synchronous with execution, and every wait or
//                   address computation in its loop is dead time for the pipe: 800 cycles
//                   per K block measured); two threads on different accumulators fill each
//                   other's gaps.
//   warps 4..11     epilogue: two warps per TMEM lane quarter, 64 columns each; they take
//                   the tiles in list order, alternating between the streams
// Two accumulators per stream ping-pong between the tensor core and the epilogue warps, so the fused
// epilogue of tile i (rounding, polynomial, mirror / transpose, stores) runs under the K loop
// of tile i+1, and per tile there is no launch, barrier initialisation or TMEM allocation.
// With one CTA per tile and two CTAs per SM the K loops of both CTAs compete for the same
// shared-memory bandwidth, and a third of the time per tile was fill, drain and epilogue.
#pragma once
#include "gemm_core.cuh"
#include <type_traits>

namespace i8m {

constexpr int WKP_STAGES = 6;
constexpr int WKP_THREADS = 384;
constexpr int WKP_NBUF = 4;      // two streams x two accumulators
constexpr int WKP_CTRL_REGS = 56;
constexpr int WKP_EPI_REGS = 224;

// Epilogues with a tile-wide tail (a maximum over the tile, a staged transposed store) declare TILE_SYNC.
template <class Epi, class = void>
struct WholekTileSync { static constexpr bool value = false; };
template <class Epi>
struct WholekTileSync<Epi, std::enable_if_t<Epi::TILE_SYNC>> { static constexpr bool value = true; };

template <class Epi>
__global__ void __launch_bounds__(WKP_THREADS, 1)
wholek_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         GemmGeom g, typename Epi::Args args) {
  constexpr int STAGES = WKP_STAGES;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int NBUF = WKP_NBUF;
  constexpr int BKE = 128 / int(sizeof(typename Epi::Elem));  // elements per 128-byte K block
  static_assert(Epi::PARTS == 1 && Epi::PROMOTE_KB == 0 && !Epi::BLOCKQ, "whole-K epilogues only");
  static_assert(STAGES % 2 == 0, "each stream owns half of the stages");
  constexpr int SSTAGES = STAGES / 2;  // stages of one stream: stream, stream + 2, ...

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
    tmem_alloc(smem_u32(&ctrl->tmem_base), 128 * NBUF);
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

  const int total_tiles = g.tiles_per_batch * g.batch;
  const int my_tiles = (total_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
  const int nkb = g.num_kb;

  if (warp < 4) {
    setmaxnreg_dec<WKP_CTRL_REGS>();
    const int stream = warp >> 1;
    // tiles of this stream: list positions stream, stream + 2, ...
    const int stream_tiles = (my_tiles - stream + 1) / 2;
    if ((warp & 1) == 0 && lane == 0) {
      // ------------------------------------------------------------ producer
      int ring = 0;             // position in this stream's ring of SSTAGES stages
      uint32_t wrap = 0;
      int issued = 0;
      bool ok = true;
      for (int j = 0; j < stream_tiles && ok; ++j) {
        int b, tm, tn;
        decode_tile(g, int(blockIdx.x) + (2 * j + stream) * int(gridDim.x), b, tm, tn);
        for (int kb = 0; kb < nkb; ++kb) {
          const int s = stream + 2 * ring;
          if (wrap > 0) {
            ok = mbar_wait(empty0 + 8u * uint32_t(s), (wrap - 1) & 1u, abort_flag);
            if (!ok) break;
          }
          const uint32_t bar = full0 + 8u * uint32_t(s);
          const uint32_t dst = smem_base + uint32_t(s * STAGE_BYTES);
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          tma_load_3d(dst, &map_a, bar, kb * BKE, tm * TILE, b);
          tma_load_3d(dst + TILE_BYTES, &map_b, bar, kb * BKE, tn * TILE, b);
          ++issued;
          if (++ring == SSTAGES) { ring = 0; ++wrap; }
        }
      }
      if (!ok) {
        atomicCAS(g.status, 0u, unsigned(ST_PRODUCER_TIMEOUT) | unsigned(blockIdx.x & 0xff));
        // let the copies that were issued land before shared memory is released
        for (int back = 0; back < SSTAGES && back < issued; ++back) {
          const int n = issued - 1 - back;   // copy number within this stream
          const uint32_t parity = uint32_t(n / SSTAGES) & 1u;
          const uint32_t bar = full0 + 8u * uint32_t(stream + 2 * (n % SSTAGES));
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, parity); ++spin) {
          }
        }
      }
    } else if ((warp & 1) == 1 && lane == 0) {
      // ---------------------------------------------------------- MMA issuer
      int ring = 0;
      uint32_t wrap = 0;
      bool ok = true;
      for (int j = 0; j < stream_tiles && ok; ++j) {
        const int buf = 2 * stream + (j & 1);
        const uint32_t use = uint32_t(j >> 1);  // how often this accumulator was filled before
        if (use >= 1) {
          ok = mbar_wait(acce0 + 8u * uint32_t(buf), (use - 1) & 1u, abort_flag);
          if (!ok) break;
        }
        const uint32_t d = tmem_base + uint32_t(buf * TILE);
        for (int kb = 0; kb < nkb; ++kb) {
          const int s = stream + 2 * ring;
          ok = mbar_wait(full0 + 8u * uint32_t(s), wrap & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + uint32_t(s * STAGE_BYTES);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t accumulate = (kb == 0 && ks == 0) ? 0u : 1u;
            umma<Epi::KIND>(d, adesc + uint64_t(ks * 2), bdesc + uint64_t(ks * 2), Epi::IDESC, accumulate);
          }
          umma_commit(empty0 + 8u * uint32_t(s));
          if (++ring == SSTAGES) { ring = 0; ++wrap; }
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
    t.red = ctrl->red; t.diag = ctrl->diag; t.tsm = WholekTileSync<Epi>::value ? tsm : nullptr; t.wsm = nullptr;
    t.c_begin = t.half * 2; t.c_end = t.half * 2 + 2;
    bool ok = true;
    for (int it = 0; it < my_tiles; ++it) {
      decode_tile(g, int(blockIdx.x) + it * int(gridDim.x), t.b, t.tm, t.tn);
      t.row0 = t.tm * TILE; t.col0 = t.tn * TILE;
      t.row = t.row0 + t.r;
      const int buf = 2 * (it & 1) + ((it >> 1) & 1);   // stream it & 1, its tile number it >> 1
      if (ok) ok = mbar_wait_warp(accf0 + 8u * uint32_t(buf), uint32_t(it >> 2) & 1u, abort_flag);
      const uint32_t taddr = tmem_base + (uint32_t(t.q * 32) << 16) + uint32_t(buf * TILE);
      AccWholeK<Epi::KIND, typename Epi::Elem, false> acc{g, t, taddr};
      if constexpr (WholekTileSync<Epi>::value) {
        // this epilogue's tile tail meets on named barriers: a warp that gave up walks through them
        // too (without loading or storing), so the others can never wait for it
        t.red = ctrl->red2[it & 1];
        if (ok) tc_fence_after();
        Epi::run_sync(g, args, t, acc, ok);
        if (ok) {
          tc_fence_before();
          __syncwarp();
          mbar_arrive_if(acce0 + 8u * uint32_t(buf), lane == 0 ? 1u : 0u);
        }
        continue;
      } else {
      if (!ok) continue;  // a warp that gave up skips the remaining tiles; the status word says so
      tc_fence_after();
      Epi::run(g, args, t, acc);
      }
      tc_fence_before();
      __syncwarp();
      mbar_arrive_if(acce0 + 8u * uint32_t(buf), lane == 0 ? 1u : 0u);
    }
    if (!ok && lane == 0)
      atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 128 * NBUF);
}

}  // namespace i8m
