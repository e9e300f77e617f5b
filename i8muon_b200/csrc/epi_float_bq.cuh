// Epilogue that ends the FP16 first iteration of an fp16-first block-quantised call: the update
// product Q * A of that iteration is rounded the way the floating route rounds its result (to the
// compute type, then to the caller's dtype: src/i8muon/csrc/prec.cu:159-164 and
// src/i8muon/_cutlass.py:137-142) and handed, still in registers, to the block quantiser's tile tail
// (src/i8muon/csrc/bq.cu:41-101 with inv = 1): the 128 x 128 CTA tile IS the quantisation block, so
// the tile maximum, the scale, the INT8 codes of A and of A^T leave from here.  The standalone
// quantisation pass and the round trip of the 16-bit intermediate through HBM disappear; the integer
// artefacts are bit-identical to the two-kernel sequence.
#pragma once
#include "epi_bq.cuh"

namespace i8m {

struct FloatToBqArgs {
  uint8_t* q;      // (batch, lp, hp) codes, lp and hp multiples of 128
  uint8_t* qt;     // (batch, hp, lp)
  float* scale;    // (batch, lp / 128, hp / 128)
  int lp, hp;
  int user_dtype;  // DType the floating route would have written
};

template <typename E>
struct EpiFloatToBq {
  static constexpr int KIND = KIND_F16;
  using Elem = E;
  static constexpr int PARTS = 1;
  static constexpr bool BLOCKQ = false;
  static constexpr int PROMOTE_KB = 0;
  static constexpr bool TILE_SYNC = true;    // the tile tail meets on named barriers: no warp may skip a tile
  static constexpr uint32_t FMT = std::is_same<E, __nv_bfloat16>::value ? 1u : 0u;
  static constexpr uint32_t IDESC = make_idesc(1u, FMT, FMT, TILE, TILE);
  static constexpr int TSM_BYTES = EpiBq<false, BQ_PLAIN>::TSM_BYTES;
  using Args = FloatToBqArgs;
  using Tail = EpiBq<false, BQ_PLAIN>;

  template <class Acc>
  static __device__ __forceinline__ void run_sync(const GemmGeom& g, const Args& a, const TileCtx& t, const Acc& acc,
                                                  const bool live) {
    float vals[Tail::CPT];
#pragma unroll
    for (int j = 0; j < Tail::CPT; ++j) vals[j] = 0.f;
    if (live) {
#pragma unroll
      for (int c = 0; c < Tail::CPT / 32; ++c) {
        uint32_t v[32];
        acc.load(t.c_begin + c, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = t.col0 + (t.c_begin + c) * 32 + j;
          float x = widen<E>(round_to<E>(__uint_as_float(v[j])));
          if (a.user_dtype == DT_BF16) x = widen<__nv_bfloat16>(round_to<__nv_bfloat16>(x));
          else if (a.user_dtype == DT_F16) x = widen<__half>(round_to<__half>(x));
          vals[c * 32 + j] = (t.row < g.lm && col < g.ln) ? x : 0.f;
        }
      }
    }
    GemmGeom gb = g;
    gb.m = a.lp; gb.n = a.hp;
    BqArgs b{};
    b.out = a.q; b.out_t = a.qt; b.so = a.scale;
    typename Tail::Pre pre{};
    Tail::tail(gb, b, t, vals, live, pre, a.lp / TILE, a.hp / TILE, 0);
  }
};

}  // namespace i8m
