// Fused epilogues of the 128x128 block-quantised Newton-Schulz GEMMs (INT8 via
// tcgen05 kind::i8, E4M3 via kind::f8f6f4).
//
// Every 128-deep K block is accumulated on its own in tensor memory and then
// promoted:  total = fmaf(float(partial), sA[tm,kb] * sB[.,kb], total)  in ascending
// kb order, as in the reference (src/i8muon/csrc/bq.cu:190-195).  The tile tail
// restates bq.cu:204-299 with un-fused FP32 operations:
//   BQ_GRAM    diagonal -> dout (zero beyond the logical size), diagonal entry zeroed
//   BQ_POLY    v = g_ij * sG[tm,tn];  val = (total + (d_i + d_j) * v) * cc + v * cb;
//              diagonal: dout_i = val + (ca + d_i * (cb + d_i * cc)), entry zeroed
//   BQ_UPDATE  val = total + (a_ij * dP_i) * sA[tm,tn]
// then (non-final) tile max (floor 1e-8) -> scale, quantise (INT8 truncates toward
// zero, E4M3 rounds to nearest even and saturates), store the tile and its
// mirror / transpose; the final update casts to the user's dtype instead.
#pragma once
#include "epi_float.cuh"

namespace i8m {

enum BqMode : int { BQ_GRAM = 0, BQ_POLY = 1, BQ_UPDATE = 2, BQ_UPDATE_FINAL = 3 };

struct BqArgs {
  const float* sa;        // scales of the left operand  (batch, m/128, k/128)
  const float* sb;        // scales of the right operand (gram/poly: (batch, n/128, k/128);
                          //                              update:    (batch, k/128, n/128))
  const float* da;        // (batch, m) diagonal: dG (poly) or dP (update)
  const uint8_t* row_b;   // update: A (batch, m, n) row-major
  void* out;              // quantised (batch, m, n) | final: user tensor
  void* out_t;            // update: quantised transpose (batch, n, m)
  float* so;              // output block scales (batch, m/128, n/128)
  float* dout;            // gram/poly: (batch, m) diagonal out
  float ca, cb, cc;
  int out_dtype, transpose;
};

template <bool FP8>
__device__ __forceinline__ float bq_decode(uint8_t v) {
  if constexpr (FP8) return e4m3_to_float(v);
  else return float(int(int8_t(v)));
}
template <bool FP8>
__device__ __forceinline__ uint8_t bq_quant(float v, float multiplier) {
  float x = __fmul_rn(v, multiplier);
  if constexpr (FP8) {
    return uint8_t(__nv_cvt_float_to_fp8(fmaxf(-448.f, x), __NV_SATFINITE, __NV_E4M3));
  } else {
    return uint8_t(int8_t(max(-127, min(127, __float2int_rz(x)))));
  }
}

template <bool FP8, int MODE>
struct EpiBq {
  static constexpr int KIND = FP8 ? KIND_F8 : KIND_I8;
  using Elem = uint8_t;
  static constexpr int PARTS = 1;
  static constexpr bool BLOCKQ = true;
  static constexpr int PROMOTE_KB = 1;
  static constexpr int STAGES = 4;
  static constexpr int MIN_CTAS = 1;
  static constexpr uint32_t IDESC =
      FP8 ? make_idesc(1u, 0u, 0u, TILE, TILE) : make_idesc(2u, 1u, 1u, TILE, TILE);
  using Args = BqArgs;
  static constexpr float QMAX = FP8 ? 448.f : 127.f;

  static __device__ __forceinline__ void run_blockq(const GemmGeom& g, const Args& a,
                                                    const TileCtx& t, uint32_t taddr,
                                                    volatile uint32_t* abort_flag) {
    constexpr int Q = TILE;
    const int mq = g.m / Q, nq = g.n / Q, kq = g.k / Q;
    float total[Q];
#pragma unroll
    for (int j = 0; j < Q; ++j) total[j] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int kb = 0; kb < g.num_kb; ++kb) {
      const int buf = kb & 1;
      if (!g.debug_simt) {
        ok = mbar_wait(smem_u32(&t.ctrl->acc_full[buf]), uint32_t(kb >> 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);  // keep the warp together for tcgen05.ld
        if (!ok) break;
        tc_fence_after();
      }
      float bs;
      if constexpr (MODE == BQ_UPDATE || MODE == BQ_UPDATE_FINAL)
        bs = a.sb[(size_t(t.b) * kq + kb) * nq + t.tn];
      else
        bs = a.sb[(size_t(t.b) * nq + t.tn) * kq + kb];
      const float s = __fmul_rn(a.sa[(size_t(t.b) * mq + t.tm) * kq + kb], bs);
#pragma unroll
      for (int c = 0; c < Q / 32; ++c) {
        uint32_t v[32];
        if (g.debug_simt) {
#pragma unroll 1
          for (int j = 0; j < 32; ++j)
            v[j] = simt_dot<KIND, uint8_t>(g, t.b, t.row, t.col0 + c * 32 + j, kb * Q, kb * Q + Q);
        } else {
          tmem_ld32(taddr + uint32_t(buf * Q + c * 32), v);
          tmem_wait_ld();
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float p = FP8 ? __uint_as_float(v[j]) : float(int(v[j]));
          total[c * 32 + j] = __fmaf_rn(p, s, total[c * 32 + j]);
        }
      }
      if (!g.debug_simt) {
        tc_fence_before();
        mbar_arrive(smem_u32(&t.ctrl->acc_empty[buf]));
      }
    }
    if (!ok) {
      if (t.lane == 0)
        atomicCAS(g.status, 0u, unsigned(ST_EPILOGUE_TIMEOUT) | unsigned(blockIdx.x & 0xff));
      return;
    }

    // ------------------------------------------------------------ tile tail
    const bool in_rows = t.row < g.lm;
    float drow = 0.f, stile = 0.f;
    if constexpr (MODE != BQ_GRAM) drow = a.da[size_t(t.b) * g.m + t.row];
    if constexpr (MODE == BQ_POLY) stile = a.sa[(size_t(t.b) * mq + t.tm) * kq + t.tn];
    if constexpr (MODE == BQ_UPDATE || MODE == BQ_UPDATE_FINAL)
      stile = a.sb[(size_t(t.b) * kq + t.tm) * nq + t.tn];
    float mx = 1e-8f;
#pragma unroll
    for (int j = 0; j < Q; ++j) {
      const int col = t.col0 + j;
      float val = total[j];
      if constexpr (MODE == BQ_GRAM) {
        if (col == t.row) {
          a.dout[size_t(t.b) * g.m + t.row] = in_rows ? val : 0.f;
          val = 0.f;
        }
      } else if constexpr (MODE == BQ_POLY) {
        const uint8_t gq = static_cast<const uint8_t*>(g.a_raw)[(size_t(t.b) * g.m + t.row) * g.k + col];
        const float v = __fmul_rn(bq_decode<FP8>(gq), stile);
        const float dcol = a.da[size_t(t.b) * g.m + col];
        val = __fadd_rn(val, __fmul_rn(__fadd_rn(drow, dcol), v));
        val = __fmul_rn(val, a.cc);
        val = __fadd_rn(val, __fmul_rn(v, a.cb));
        if (col == t.row) {
          const float dpoly =
              __fadd_rn(a.ca, __fmul_rn(drow, __fadd_rn(a.cb, __fmul_rn(drow, a.cc))));
          a.dout[size_t(t.b) * g.m + t.row] = in_rows ? __fadd_rn(val, dpoly) : 0.f;
          val = 0.f;
        }
      } else {
        const uint8_t aq = a.row_b[(size_t(t.b) * g.m + t.row) * g.n + col];
        val = __fadd_rn(val, __fmul_rn(__fmul_rn(bq_decode<FP8>(aq), drow), stile));
      }
      if (!in_rows || col >= g.ln) val = 0.f;  // padding never contributes to a block scale
      total[j] = val;
      mx = fmaxf(mx, fabsf(val));
    }

    if constexpr (MODE == BQ_UPDATE_FINAL) {
      if (in_rows) {
#pragma unroll
        for (int j = 0; j < Q; ++j) {
          const int col = t.col0 + j;
          if (col < g.ln) {
            size_t idx = a.transpose ? (size_t(t.b) * g.ln + col) * g.lm + t.row
                                     : (size_t(t.b) * g.lm + t.row) * g.ln + col;
            store_user(a.out, a.out_dtype, idx, total[j]);
          }
        }
      }
      return;
    } else {
      mx = warp_max(mx);
      if (t.lane == 0) t.ctrl->red[t.q] = mx;
      named_bar_sync(1, 128);
      mx = fmaxf(fmaxf(t.ctrl->red[0], t.ctrl->red[1]), fmaxf(t.ctrl->red[2], t.ctrl->red[3]));
      const float multiplier = QMAX / mx;
      const float scale = 1.f / multiplier;
      if (t.r == 0) {
        a.so[(size_t(t.b) * mq + t.tm) * nq + t.tn] = scale;
        if constexpr (MODE != BQ_UPDATE) a.so[(size_t(t.b) * mq + t.tn) * nq + t.tm] = scale;
      }
      uint8_t* out = static_cast<uint8_t*>(a.out);
      const bool diag_tile = (MODE != BQ_UPDATE) && t.tm == t.tn;
      if (!diag_tile) {
        uint32_t packed[Q / 4];
#pragma unroll
        for (int j = 0; j < Q; j += 4) {
          packed[j / 4] = uint32_t(bq_quant<FP8>(total[j], multiplier)) |
                          (uint32_t(bq_quant<FP8>(total[j + 1], multiplier)) << 8) |
                          (uint32_t(bq_quant<FP8>(total[j + 2], multiplier)) << 16) |
                          (uint32_t(bq_quant<FP8>(total[j + 3], multiplier)) << 24);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t(t.b) * g.m + t.row) * g.n + t.col0);
#pragma unroll
        for (int i = 0; i < Q / 16; ++i)
          dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        // transpose (update) or mirror (gram / poly off-diagonal tile)
        uint8_t* tdst = (MODE == BQ_UPDATE) ? static_cast<uint8_t*>(a.out_t) : out;
        const int trows = (MODE == BQ_UPDATE) ? g.n : g.m;
        const int tld = (MODE == BQ_UPDATE) ? g.m : g.n;
#pragma unroll
        for (int j = 0; j < Q; ++j) {
          const uint8_t qv = uint8_t(packed[j / 4] >> (8 * (j & 3)));
          tdst[(size_t(t.b) * trows + (t.col0 + j)) * tld + t.row] = qv;
        }
      } else {
#pragma unroll
        for (int j = 0; j < Q; ++j) {
          if (j > t.r) continue;
          const uint8_t qv = bq_quant<FP8>(total[j], multiplier);
          out[(size_t(t.b) * g.m + t.row) * g.n + t.col0 + j] = qv;
          out[(size_t(t.b) * g.m + t.col0 + j) * g.n + t.row] = qv;
        }
      }
    }
  }
};

}  // namespace i8m
