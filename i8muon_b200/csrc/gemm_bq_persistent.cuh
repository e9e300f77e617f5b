// Persistent kernel for the 128x128 block-quantised GEMMs (the dominant kernels of
// the INT8-BQ / FP8-BQ Newton-Schulz step).
//
// One CTA per SM walks a static round-robin list of output tiles.  Three warpgroups:
//   warpgroup 0  warps 0 and 2 = TMA producers, warps 1 and 3 = tcgen05.mma issuers;
//                registers trimmed with setmaxnreg
//   warpgroups 1-2  eight epilogue warps; thread = one accumulator row x 64 columns
// The shared-memory ring and the four TMEM accumulators are indexed by a K-block
// counter that runs across tiles, so the producers and the tensor core move on to the
// next tile while the epilogue warps still quantise and store the previous one; per
// tile there is no launch, no barrier initialisation and no TMEM allocation.
//
// Measured facts behind the structure (B200, update GEMM 4096 x 14336, K = 4096):
//   * every K block has its own accumulator, so K blocks are independent work items for
//     the tensor core; two producers and two issuers work on alternate K blocks;
//   * a 128-byte K block of a 128x128 tile is 256 cycles of tensor work; the K loop sits at
//     about 550 cycles per K block: the epilogue drains and refills a 64 KB accumulator every
//     K block (the MMA itself slows to ~390 cycles per K block while eight warps read TMEM),
//     and 32 KB go into and out of shared memory;
//   * the epilogue loop is written for instruction count (see the step lambda): with the
//     first, straightforward loop the kernel spent 800 cycles per K block, two to three
//     bookkeeping instructions per useful one;
//   * the per-K-block scale products are staged in shared memory per tile; one mbarrier
//     arrival per epilogue warp, not per thread.
#pragma once
#include "epi_bq.cuh"

namespace i8m {

constexpr int BQP_STAGES = 6;        // default ring depth; the tuner may pick BQP_STAGES_ALT
constexpr int BQP_STAGES_ALT = 4;
constexpr int BQP_THREADS = 384;
constexpr int BQP_MAX_KB = 512;  // K blocks whose scales are staged in shared memory (K <= 65536)
constexpr int BQP_CTRL_REGS = 56;
constexpr int BQP_EPI_REGS = 224;

// ---------------------------------------------------------------- roles shared by both kernels
// One producer thread: K blocks gk = par, par + 2, ... of this CTA's tile list go into stages
// s = par, par + 2, ... (modulo STAGES) of the operand ring.
template <int STAGES>
__device__ __forceinline__ void bq_produce(const CUtensorMap* map_a, const CUtensorMap* map_b, const GemmGeom& g,
                                           const int par, const int my_tiles, const int nkb, const int my_kb,
                                           const uint32_t smem_base, const uint32_t full0, const uint32_t empty0,
                                           volatile uint32_t* abort_flag) {
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int Q = TILE;
  // Test hook (i8m_set_debug_core(2)): the producers issue nothing, so every consumer's bounded wait runs
  // out, each role records its code in the status word and leaves, and the CTA frees its tensor memory.
  // Nothing is in flight when that happens: no copy was issued and no MMA could start.
  if (g.debug_simt & 0x100) return;
  int it = 0, kb = par, b = 0, tm = 0, tn = 0;
  while (kb >= nkb && it < my_tiles) { kb -= nkb; ++it; }
  if (it < my_tiles) decode_tile(g, int(blockIdx.x) + it * int(gridDim.x), b, tm, tn);
  int s = par;              // stage of the current K block, advances by 2 modulo STAGES
  uint32_t wrap = 0;        // how often this stage has been used before
  int issued = 0;
  bool ok = true;
  for (int gk = par; gk < my_kb; gk += 2) {
    if (wrap > 0) {
      ok = mbar_wait(empty0 + 8u * uint32_t(s), (wrap - 1) & 1u, abort_flag);
      if (!ok) break;
    }
    const uint32_t bar = full0 + 8u * uint32_t(s);
    const uint32_t dst = smem_base + uint32_t(s * STAGE_BYTES);
    mbar_arrive_expect_tx(bar, STAGE_BYTES);
    tma_load_3d(dst, map_a, bar, kb * Q, tm * Q, b);
    tma_load_3d(dst + TILE_BYTES, map_b, bar, kb * Q, tn * Q, b);
    ++issued;
    s += 2;
    if (s >= STAGES) { s -= STAGES; ++wrap; }
    kb += 2;
    if (kb >= nkb) {
      do { kb -= nkb; ++it; } while (kb >= nkb && it < my_tiles);
      if (it < my_tiles) decode_tile(g, int(blockIdx.x) + it * int(gridDim.x), b, tm, tn);
    }
  }
  if (!ok) {
    atomicCAS(g.status, 0u, unsigned(ST_PRODUCER_TIMEOUT) | unsigned(blockIdx.x & 0xff));
    // let the copies that were issued land before shared memory is released
    for (int back = 0; back < STAGES / 2 && back < issued; ++back) {
      const int n = par + 2 * (issued - 1 - back);     // global K block index
      const uint32_t parity = uint32_t(n / STAGES) & 1u;
      for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(full0 + 8u * uint32_t(n % STAGES), parity); ++spin) {
      }
    }
  }
}

// One issuing thread: the K blocks of the same parity, each into its own accumulator.
template <class Epi, int STAGES>
__device__ __forceinline__ void bq_issue(const GemmGeom& g, const int par, const int my_kb, const uint32_t tmem_base,
                                         const uint32_t smem_base, const uint32_t full0, const uint32_t empty0,
                                         const uint32_t accf0, const uint32_t acce0,
                                         volatile uint32_t* abort_flag) {
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int NBUF = 4;
  constexpr int Q = TILE;
  int s = par, buf = par;   // both advance by 2 (modulo STAGES / NBUF)
  uint32_t wrap = 0, use = 0;
  bool ok = true;
  for (int gk = par; gk < my_kb; gk += 2) {
    // PRESET: every use waits for the epilogue's refill (completion 0 = initial fill);
    // otherwise a buffer is free until its first reuse
    if (Epi::PRESET) ok = mbar_wait(acce0 + 8u * uint32_t(buf), use & 1u, abort_flag);
    else if (use >= 1) ok = mbar_wait(acce0 + 8u * uint32_t(buf), (use - 1) & 1u, abort_flag);
    if (!ok) break;
    ok = mbar_wait(full0 + 8u * uint32_t(s), wrap & 1u, abort_flag);
    if (!ok) break;
    tc_fence_after();
    const uint32_t d = tmem_base + uint32_t(buf * Q);
    const uint32_t sa = smem_base + uint32_t(s * STAGE_BYTES);
    const uint64_t adesc = make_smem_desc_sw128(sa);
    const uint64_t bdesc = make_smem_desc_sw128(sa + TILE_BYTES);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t accumulate = (!Epi::PRESET && ks == 0) ? 0u : 1u;
      umma<Epi::KIND>(d, adesc + uint64_t(ks * 2), bdesc + uint64_t(ks * 2), Epi::IDESC, accumulate);
    }
    umma_commit(empty0 + 8u * uint32_t(s));
    umma_commit(accf0 + 8u * uint32_t(buf));
    s += 2;
    if (s >= STAGES) { s -= STAGES; ++wrap; }
    buf += 2;
    if (buf >= NBUF) { buf -= NBUF; ++use; }
  }
  if (!ok) atomicCAS(g.status, 0u, unsigned(ST_MMA_TIMEOUT) | unsigned(blockIdx.x & 0xff));
}

// State that a fold (epilogue) warp carries from tile to tile.
struct BqFoldState {
  int buf = 0;
  uint32_t use = 0;
  bool ok = true;
};

// Preset the four accumulators (INT8) and keep the 32 registers that every refill stores from.
template <class Epi>
__device__ __forceinline__ void bq_fold_begin(const uint32_t taddr, const uint32_t acce0, const int lane,
                                              uint32_t (&magic)[32]) {
  constexpr int NBUF = 4;
  constexpr int Q = TILE;
  if constexpr (Epi::PRESET) {
#pragma unroll
    for (int i = 0; i < NBUF; ++i) {
      tmem_st32_fill(taddr + uint32_t(i * Q), I8_MAGIC_BITS);
      tmem_st32_fill(taddr + uint32_t(i * Q + 32), I8_MAGIC_BITS);
    }
    tmem_wait_st();
    // Every refill stores from these 32 registers.  A store of one replicated register
    // makes the compiler copy it into 32 consecutive registers before every store (64
    // moves per K block on the FP32 pipe); values read back from tensor memory are opaque
    // to it and stay where the load put them.
    tmem_ld32(taddr, magic);
    tmem_wait_ld();
    tc_fence_before();
    __syncwarp();
    if (lane == 0)
      for (int i = 0; i < NBUF; ++i) mbar_arrive(acce0 + 8u * uint32_t(i));
  }
}

// The K loop of one tile for one fold warp: every K block's accumulator is pulled into
// registers, refilled with the bias constant (INT8), folded into the FP32 totals and handed
// back.  Written for few instructions: the loop runs 8 warps x K/128 times per tile and its
// bookkeeping competes with the arithmetic for issue slots.  Every K block refills, also the
// last ones of the launch whose buffers are not used again: no predicate.
template <class Epi, class ScaleFn>
__device__ __forceinline__ void bq_fold_tile(BqFoldState& st, unsigned long long (&tot2)[32], const uint32_t (&magic)[32],
                                             const uint32_t taddr, const uint32_t accf0, const uint32_t acce0,
                                             const int nkb, const bool staged, const float* sc, const int lane,
                                             volatile uint32_t* abort_flag, ScaleFn&& unstaged_scale) {
  constexpr int NBUF = 4;
  constexpr int Q = TILE;
  const uint32_t is_lane0 = lane == 0 ? 1u : 0u;
  auto step = [&](const uint32_t full_bar, const uint32_t empty_bar, const uint32_t tbuf,
                  const uint32_t parity, const float s) -> bool {
    if (!mbar_wait_warp(full_bar, parity, abort_flag)) return false;
    tc_fence_after();
    uint32_t v[2][32];
    tmem_ld32(tbuf, v[0]);
    tmem_ld32(tbuf + 32u, v[1]);
    tmem_wait_ld();
    if constexpr (Epi::PRESET) {
      tmem_st32(tbuf, magic);
      tmem_st32(tbuf + 32u, magic);
    }
    Epi::fold64p(tot2, v, s);
    if constexpr (Epi::PRESET) tmem_wait_st();
    tc_fence_before();
    __syncwarp();
    mbar_arrive_if(empty_bar, is_lane0);
    return true;
  };
  bool ok = st.ok;
  if (staged && (nkb & 3) == 0 && st.buf == 0) {
    // every tile starts on accumulator 0: buffers and barriers are compile-time offsets,
    // four scale products come with one shared-memory load
    const uint32_t sc_s = smem_u32(sc);
    uint32_t parity = st.use & 1u;
#pragma unroll 1
    for (int kb = 0; kb < nkb && ok; kb += 4) {
      const float4 s4 = lds128(sc_s + uint32_t(kb) * 4u);
      ok = step(accf0, acce0, taddr, parity, s4.x) &&
           step(accf0 + 8u, acce0 + 8u, taddr + uint32_t(Q), parity, s4.y) &&
           step(accf0 + 16u, acce0 + 16u, taddr + uint32_t(2 * Q), parity, s4.z) &&
           step(accf0 + 24u, acce0 + 24u, taddr + uint32_t(3 * Q), parity, s4.w);
      parity ^= 1u;
    }
    st.use += uint32_t(nkb >> 2);
  } else {
#pragma unroll 1
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const float s = staged ? sc[kb] : unstaged_scale(kb);
      ok = step(accf0 + 8u * uint32_t(st.buf), acce0 + 8u * uint32_t(st.buf), taddr + uint32_t(st.buf * Q),
                st.use & 1u, s);
      if (++st.buf == NBUF) { st.buf = 0; ++st.use; }
    }
  }
  st.ok = ok;
}

template <class Epi, int STAGES_T>
__global__ void __launch_bounds__(BQP_THREADS, 1)
bq_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     GemmGeom g, typename Epi::Args args) {
  constexpr int STAGES = STAGES_T;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int NBUF = 4;
  constexpr int Q = TILE;
  constexpr int CPT = 64;  // columns per epilogue thread
  static_assert(Epi::CPT == CPT && Epi::EPI_WARPS == 8 && Epi::NBUF == NBUF, "layout mismatch with the epilogue");
  static_assert(STAGES % 2 == 0, "two producers alternate stages");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * STAGE_BYTES);
  float* scale_ring = reinterpret_cast<float*>(ctrl + 1);  // [2][BQP_MAX_KB] products sA*sB per K block
  uint8_t* tsm = reinterpret_cast<uint8_t*>(scale_ring + 2 * BQP_MAX_KB);  // transposed staging tile
  static_assert(sizeof(Ctrl) % 16 == 0 && (2 * BQP_MAX_KB * sizeof(float)) % 16 == 0 && Epi::TSM_PITCH % 16 == 0,
                "the staging tile is read with 16-byte loads");
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
  const int my_kb = my_tiles * nkb;  // K blocks this CTA pushes through the pipeline

  if (warp < 4) {
    setmaxnreg_dec<BQP_CTRL_REGS>();
    const int par = warp >> 1;  // this thread takes K blocks gk = par, par + 2, ...
    if ((warp & 1) == 0 && lane == 0)
      bq_produce<STAGES>(&map_a, &map_b, g, par, my_tiles, nkb, my_kb, smem_base, full0, empty0, abort_flag);
    else if ((warp & 1) == 1 && lane == 0)
      bq_issue<Epi, STAGES>(g, par, my_kb, tmem_base, smem_base, full0, empty0, accf0, acce0, abort_flag);
  } else {
    // -------------------------------------------------------------- epilogue
    setmaxnreg_inc<BQP_EPI_REGS>();
    TileCtx t;
    t.q = warp & 3; t.lane = lane;
    t.ew = warp - 4; t.half = (warp - 4) >> 2;
    t.r = t.q * 32 + lane;
    t.ctrl = ctrl;
    t.diag = ctrl->diag;
    t.tsm = tsm; t.wsm = nullptr;
    const int c0 = t.half * CPT;
    const uint32_t taddr = tmem_base + (uint32_t(t.q * 32) << 16) + uint32_t(c0);
    const int mq = g.m / Q, nq = g.n / Q, kq = g.k / Q;
    uint32_t magic[32];
    bq_fold_begin<Epi>(taddr, acce0, lane, magic);
    BqFoldState st;
    const bool staged = nkb <= BQP_MAX_KB;
    float next_fa = 0.f, next_fb = 0.f;  // factors of the next tile's first scale products
    for (int it = 0; it < my_tiles; ++it) {
      decode_tile(g, int(blockIdx.x) + it * int(gridDim.x), t.b, t.tm, t.tn);
      t.row0 = t.tm * Q; t.col0 = t.tn * Q;
      t.row = t.row0 + t.r;
      t.red = ctrl->red2[it & 1];
      // scale products of this tile -> shared memory (a slow warp of tile it-1 cannot still
      // be reading this half of the ring: it passed this barrier of tile it-1 after that)
      float* sc = scale_ring + (it & 1) * BQP_MAX_KB;
      const int ek = int(threadIdx.x) - 128;  // this thread's first K block of the scale staging
      if (staged) {
        // the first 256 products were fetched into a register during the previous tile
        if (ek < nkb) sc[ek] = (it == 0) ? Epi::block_scale(g, args, t, ek, mq, nq, kq) : __fmul_rn(next_fa, next_fb);
        for (int k = ek + 256; k < nkb; k += 256) sc[k] = Epi::block_scale(g, args, t, k, mq, nq, kq);
        named_bar_sync(2, 256);
      }
      const typename Epi::Pre pre = Epi::tail_prefetch(g, args, t, mq, nq, kq);
      if (staged && it + 1 < my_tiles && int(threadIdx.x) - 128 < nkb) {
        // the factors of the next tile's scale products: fetched here so that the address
        // arithmetic and the loads' latency lie under this tile's K loop, not in its tail
        TileCtx nt = t;
        decode_tile(g, int(blockIdx.x) + (it + 1) * int(gridDim.x), nt.b, nt.tm, nt.tn);
        Epi::block_scale_factors(g, args, nt, int(threadIdx.x) - 128, mq, nq, kq, next_fa, next_fb);
      }
      unsigned long long tot2[CPT / 2];
#pragma unroll
      for (int j = 0; j < CPT / 2; ++j) tot2[j] = 0ull;
      bq_fold_tile<Epi>(st, tot2, magic, taddr, accf0, acce0, nkb, staged, sc, lane, abort_flag,
                        [&](int kb) { return Epi::block_scale(g, args, t, kb, mq, nq, kq); });
      if (!st.ok && lane == 0)
        atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
      float tot[CPT];
#pragma unroll
      for (int j = 0; j < CPT / 2; ++j) { tot[2 * j] = lane0(tot2[j]); tot[2 * j + 1] = lane1(tot2[j]); }
      // a warp that gave up still walks through the tail's barriers, without storing
      Epi::tail(g, args, t, tot, st.ok, pre, mq, nq, kq);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 128 * NBUF);
}

}  // namespace i8m
