// Block-quantised GEMM kernel with the tile tail on its own warps.
//
// In bq_persistent_kernel the eight epilogue warps fold every K block AND run the tile tail
// (tile maximum, quantisation, two stores).  During that tail, about 6400 cycles per tile, the
// tensor core runs the four K blocks ahead that tensor memory can hold and then idles: a quarter
// of a K = 4096 tile.  Here the fold warps only park the tile's 128 x 128 FP32 totals in shared
// memory (16 vector stores per thread) and go straight into the next tile's K loop, and a fourth
// warpgroup does the tail from the parked tile while that K loop runs.
//
//   warpgroup 0   warps 0/2 TMA producers, warps 1/3 tcgen05.mma issuers      (40 registers)
//   warpgroups 1-2  eight fold warps, as in bq_persistent_kernel               (200 registers)
//   warpgroup 3   four tail warps: EpiBq::split_tail                           (72 registers)
//
// Shared memory: a four-stage operand ring (128 KB), the parked tile (66 KB), the scale ring.
// Hand-over: park_full (8 fold-warp arrivals) / park_empty (4 tail-warp arrivals), both mbarriers
// with bounded waits; a role that gives up sets the abort flag and every other role leaves at its
// next poll.  The final update (cast to the caller's dtype, no quantisation) has its own tail
// (EpiBq::split_tail_final).
#pragma once
#include "gemm_bq_persistent.cuh"

namespace i8m {

constexpr int BQS_STAGES = 4;
constexpr int BQS_THREADS = 512;
constexpr int BQS_CTRL_REGS = 40;
constexpr int BQS_FOLD_REGS = 200;
constexpr int BQS_TAIL_REGS = 72;
static_assert(128 * BQS_CTRL_REGS + 256 * BQS_FOLD_REGS + 128 * BQS_TAIL_REGS <= 65536, "register file");


template <class Epi>
constexpr size_t bq_split_smem_bytes() {
  return size_t(BQS_STAGES) * 2 * TILE_BYTES + sizeof(Ctrl) + 2 * BQP_MAX_KB * sizeof(float) +
         size_t(TILE) * Epi::PARK_PITCH * sizeof(float) + 1024;
}

template <class Epi>
__global__ void __launch_bounds__(BQS_THREADS, 1)
bq_split_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                GemmGeom g, typename Epi::Args args) {
  constexpr int STAGES = BQS_STAGES;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int NBUF = 4;
  constexpr int Q = TILE;
  constexpr int CPT = 64;  // columns per fold thread
  static_assert(Epi::CPT == CPT && Epi::EPI_WARPS == 8 && Epi::NBUF == NBUF, "layout mismatch with the epilogue");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * STAGE_BYTES);
  float* scale_ring = reinterpret_cast<float*>(ctrl + 1);  // [2][BQP_MAX_KB] products sA*sB per K block
  float* park_tile = scale_ring + 2 * BQP_MAX_KB;          // [TILE][PARK_PITCH] FP32 totals of one tile
  static_assert(sizeof(Ctrl) % 16 == 0 && (2 * BQP_MAX_KB * sizeof(float)) % 16 == 0 && (Epi::PARK_PITCH * 4) % 16 == 0,
                "the parked tile is accessed with 16-byte loads and stores");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int i = 0; i < NBUF; ++i) {
      mbar_init(smem_u32(&ctrl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[i]), 8);  // one arrival per fold warp
    }
    mbar_init(smem_u32(&ctrl->park_full), 8);       // one arrival per fold warp
    mbar_init(smem_u32(&ctrl->park_empty), 4);      // one arrival per tail warp
    mbar_init(smem_u32(&ctrl->tail_sync), 4);
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
  const uint32_t park_full = smem_u32(&ctrl->park_full), park_empty = smem_u32(&ctrl->park_empty);
  const uint32_t park = smem_u32(park_tile);

  const int total_tiles = g.tiles_per_batch * g.batch;
  const int my_tiles = (total_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
  const int nkb = g.num_kb;
  const int my_kb = my_tiles * nkb;
  const int mq = g.m / Q, nq = g.n / Q, kq = g.k / Q;

  if (warp < 4) {
    setmaxnreg_dec<BQS_CTRL_REGS>();
    const int par = warp >> 1;
    if ((warp & 1) == 0 && lane == 0)
      bq_produce<STAGES>(&map_a, &map_b, g, par, my_tiles, nkb, my_kb, smem_base, full0, empty0, abort_flag);
    else if ((warp & 1) == 1 && lane == 0)
      bq_issue<Epi, STAGES>(g, par, my_kb, tmem_base, smem_base, full0, empty0, accf0, acce0, abort_flag);
  } else if (warp < 12) {
    // ------------------------------------------------------------------ fold warps
    setmaxnreg_inc<BQS_FOLD_REGS>();
    TileCtx t;
    t.q = warp & 3; t.lane = lane;
    t.ew = warp - 4; t.half = (warp - 4) >> 2;
    t.r = t.q * 32 + lane;
    t.ctrl = ctrl;
    const int c0 = t.half * CPT;
    const uint32_t taddr = tmem_base + (uint32_t(t.q * 32) << 16) + uint32_t(c0);
    const uint32_t park_mine = park + uint32_t(t.r * Epi::PARK_PITCH + c0) * 4u;
    uint32_t magic[32];
    bq_fold_begin<Epi>(taddr, acce0, lane, magic);
    BqFoldState st;
    const bool staged = nkb <= BQP_MAX_KB;
    float next_fa = 0.f, next_fb = 0.f;
    for (int it = 0; it < my_tiles; ++it) {
      decode_tile(g, int(blockIdx.x) + it * int(gridDim.x), t.b, t.tm, t.tn);
      float* sc = scale_ring + (it & 1) * BQP_MAX_KB;
      const int ek = int(threadIdx.x) - 128;
      if (staged) {
        if (ek < nkb) sc[ek] = (it == 0) ? Epi::block_scale(g, args, t, ek, mq, nq, kq) : __fmul_rn(next_fa, next_fb);
        for (int k = ek + 256; k < nkb; k += 256) sc[k] = Epi::block_scale(g, args, t, k, mq, nq, kq);
        named_bar_sync(2, 256);
      }
      if (staged && it + 1 < my_tiles && ek < nkb) {
        TileCtx nt = t;
        decode_tile(g, int(blockIdx.x) + (it + 1) * int(gridDim.x), nt.b, nt.tm, nt.tn);
        Epi::block_scale_factors(g, args, nt, ek, mq, nq, kq, next_fa, next_fb);
      }
      unsigned long long tot2[CPT / 2];
#pragma unroll
      for (int j = 0; j < CPT / 2; ++j) tot2[j] = 0ull;
      bq_fold_tile<Epi>(st, tot2, magic, taddr, accf0, acce0, nkb, staged, sc, lane, abort_flag,
                        [&](int kb) { return Epi::block_scale(g, args, t, kb, mq, nq, kq); });
      // hand the totals over: the parked tile is free once the tail warps have read tile it - 1
      if (st.ok) st.ok = mbar_wait_warp(park_empty, (uint32_t(it) & 1u) ^ 1u, abort_flag);
      if (st.ok) {
#pragma unroll
        for (int j = 0; j < CPT / 4; ++j) sts128_pairs(park_mine + uint32_t(j) * 16u, tot2[2 * j], tot2[2 * j + 1]);
        __syncwarp();
        mbar_arrive_if(park_full, lane == 0 ? 1u : 0u);
      } else if (lane == 0) {
        atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
      }
    }
  } else {
    // ------------------------------------------------------------------ tail warps
    setmaxnreg_dec<BQS_TAIL_REGS>();
    const int tid = int(threadIdx.x) - 384;
    for (int it = 0; it < my_tiles; ++it) {
      int b, tm, tn;
      decode_tile(g, int(blockIdx.x) + it * int(gridDim.x), b, tm, tn);
      bool ok = mbar_wait_warp_inline(park_full, uint32_t(it) & 1u, abort_flag);
      if (ok) ok = Epi::split_tail(g, args, b, tm, tn, tid, it, park, ctrl, abort_flag, mq, nq, kq);
      if (!ok) {
        if (lane == 0) atomicCAS(g.status, 0u, unsigned(ST_TAIL_TIMEOUT) | unsigned(blockIdx.x & 0xff));
        break;
      }
      __syncwarp();
      mbar_arrive_if(park_empty, lane == 0 ? 1u : 0u);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 128 * NBUF);
}

}  // namespace i8m
