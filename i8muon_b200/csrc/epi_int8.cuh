// Fused epilogues of the global-scale INT8 Newton-Schulz GEMMs (tcgen05 kind::i8,
// int32 accumulation in tensor memory).
//
// Arithmetic restates the reference's INT8 GEMM modes (src/i8muon/csrc/int8.cu:254-352).
// The reference is compiled with --fmad=true, so its unannotated expressions contain fused
// multiply-adds; which ones was established against tensors recorded from the reference's own
// build for sm_100a (tests/golden/reference_ns_i8_*.npz).  This library is compiled with
// --fmad=false and writes every rounding explicitly, so that a CPU restatement reproduces it:
//   I8_GRAM    G32 = A8 * A8^T  (lower tiles), gmax = max_{i != j} |G32_ij|   (int32, exact)
//   I8_SQUARE  P_ij = fma((g8*g8)_ij, gs*gs*c, g8_ij * t_ij),
//              t_ij = fma(fma(dG_i, c, b), gs, (dG_j*gs)*c)
//              (the reference's binary uses this form for about three quarters of the elements and
//              fma(dG_j*gs, c, (fma(dG_i,c,b))*gs) for the rest, by unrolled instance: 1 ulp apart);
//              pmax = max |P_ij| over i != j, floor(i/128) >= floor(j/128)
//   I8_UPDATE  Y_ij = fma(a8_ij, dP_i, (p8*a8)_ij * ps) * as  (the reference's binary, every element);
//              non-final keeps FP32 + max, final casts to the user's dtype, un-pads, optionally transposes.
#pragma once
#include "epi_float.cuh"

namespace i8m {

enum I8Mode : int { I8_GRAM = 0, I8_SQUARE = 1, I8_UPDATE = 2, I8_UPDATE_FINAL = 3 };

struct I8Args {
  void* out;              // int32 (gram) / fp32 (square, update) (batch, m, n); final: user tensor
  void* maximum;          // per-batch reduction slot: int32 (gram) or fp32 bits
  const float* a_scale;   // per-batch scale of the left operand (square: gs, update: ps)
  const float* b_scale;   // update: per-batch scale of A8 (as)
  const float* diag;      // (batch, m): dG (square) or dP (update)
  const int8_t* row_b;    // update: A8 (batch, m, n) row-major
  float alpha, beta;      // square: b and c coefficients
  float gain;             // update: multiplies b_scale when use_gain (completed-square / cubic rows)
  int use_gain;
  int out_dtype, transpose;
};

template <int MODE>
struct EpiI8 {
  static constexpr int KIND = KIND_I8;
  using Elem = int8_t;
  static constexpr int PARTS = 1;
  static constexpr bool BLOCKQ = false;
  static constexpr int PROMOTE_KB = 0;
  static constexpr int NBUF = 1;
  static constexpr int EPI_WARPS = 4;
  static constexpr int STAGES = 3;
  static constexpr int MIN_CTAS = 2;
  static constexpr uint32_t IDESC = make_idesc(2u, 1u, 1u, TILE, TILE);  // s32 <- s8 * s8
  using Args = I8Args;

  // Fast path for a tile inside the logical extent: every global access of a warp's 32-row block
  // goes through the warp's shared-memory patch in coalesced requests, the column diagonal is
  // loaded once per chunk (one column per lane) and handed round by shuffles.
  // Every element goes through the same operations, in the same order, as in the general path.
  static __device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
  static __device__ __forceinline__ bool fast_ok(const GemmGeom& g, const Args& a, const TileCtx& t) {
    if (t.wsm == nullptr || t.row0 + TILE > g.lm || t.col0 + TILE > g.ln || !aligned16(a.out)) return false;
    if constexpr (MODE == I8_UPDATE_FINAL) {
      if (a.out_dtype == DT_F32) { if (a.transpose || (g.ln & 3)) return false; }
      else if ((a.transpose ? g.lm : g.ln) & 7) return false;
    } else if (g.n & 3) {
      return false;
    }
    if constexpr (MODE == I8_SQUARE) return aligned16(g.a_raw) && (g.k & 15) == 0;
    if constexpr (MODE == I8_UPDATE || MODE == I8_UPDATE_FINAL) return aligned16(a.row_b) && (g.n & 15) == 0;
    return true;
  }
  static __device__ __forceinline__ float byte_to_float(uint32_t word, int k) {
    return float(int(int8_t(word >> (8 * k))));
  }

  // 32 columns of 32-bit results per lane row: two halves of 64 bytes through the patch
  static __device__ __forceinline__ void store_rows32(const WarpPatch& wp, uint8_t* dst, size_t pitch,
                                                      const uint32_t (&r)[32]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t half[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) half[k] = r[16 * h + k];
      wp.write_own_row(half);
      __syncwarp();
      store_block_rows(wp, dst + 64 * h, pitch);
      __syncwarp();
    }
  }

  template <class Acc>
  static __device__ __forceinline__ void run_fast(const GemmGeom& g, const Args& a, const TileCtx& t,
                                                  const Acc& acc) {
    int imax = 0;
    float fmax_ = 0.f;
    float sa = 0.f, sb = 0.f, sq = 0.f, drow = 0.f, xrow = 0.f;
    if constexpr (MODE != I8_GRAM) {
      sa = a.a_scale[t.b];
      drow = a.diag[size_t(t.b) * g.m + t.row];
    }
    if constexpr (MODE == I8_SQUARE) {
      sq = __fmul_rn(__fmul_rn(sa, sa), a.beta);
      xrow = __fmaf_rn(drow, a.beta, a.alpha);
    }
    if constexpr (MODE == I8_UPDATE || MODE == I8_UPDATE_FINAL) {
      sb = a.b_scale[t.b];
      if (a.use_gain) sb = __fmul_rn(sb, a.gain);
    }
    const WarpPatch wp{smem_u32(t.wsm), t.lane};
    const int wrow0 = t.row0 + 32 * t.q;   // first row of this warp's block
#pragma unroll 1
    for (int c = t.c_begin; c < t.c_end; ++c) {
      uint32_t v[32];
      acc.load(c, v);
      const int colb = t.col0 + c * 32;
      const size_t wbase = (size_t(t.b) * g.m + wrow0) * g.n + colb;   // first element of the warp's block
      const int dcol = t.row - colb;   // this row's diagonal column inside the chunk when 0 <= dcol < 32
      if constexpr (MODE == I8_GRAM) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j != dcol) imax = max(imax, abs(int(v[j])));
        store_rows32(wp, reinterpret_cast<uint8_t*>(static_cast<int*>(a.out) + wbase), size_t(g.n) * 4, v);
      } else {
        // the int8 companion block (g8 for the square, a8 for the update): coalesced into the patch
        const int8_t* comp = (MODE == I8_SQUARE)
            ? static_cast<const int8_t*>(g.a_raw) + (size_t(t.b) * g.m + wrow0) * g.k + colb
            : a.row_b + wbase;
        load_block_rows32(wp, reinterpret_cast<const uint8_t*>(comp), size_t(MODE == I8_SQUARE ? g.k : g.n));
        __syncwarp();
        const uint4 c0 = lds128u(wp.piece(t.lane, 0)), c1 = lds128u(wp.piece(t.lane, 1));
        __syncwarp();
        const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float cj_lane = 0.f;
        if constexpr (MODE == I8_SQUARE)
          cj_lane = __fmul_rn(__fmul_rn(a.diag[size_t(t.b) * g.m + colb + t.lane], sa), a.beta);
        uint32_t res[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float accf = float(int(v[j]));
          const float e = byte_to_float(cw[j >> 2], j & 3);
          float r;
          if constexpr (MODE == I8_SQUARE) {
            const float cj = __shfl_sync(0xffffffffu, cj_lane, j);
            r = __fmaf_rn(accf, sq, __fmul_rn(e, __fmaf_rn(xrow, sa, cj)));
            if (j != dcol) fmax_ = fmaxf(fmax_, fabsf(r));
          } else {
            r = __fmul_rn(__fmaf_rn(e, drow, __fmul_rn(accf, sa)), sb);
            if constexpr (MODE == I8_UPDATE) fmax_ = fmaxf(fmax_, fabsf(r));
          }
          res[j] = __float_as_uint(r);
        }
        if constexpr (MODE == I8_UPDATE_FINAL) {
          uint8_t* out = static_cast<uint8_t*>(a.out);
          if (a.out_dtype == DT_F32) {
            store_rows32(wp, out + ((size_t(t.b) * g.lm + wrow0) * g.ln + colb) * 4, size_t(g.ln) * 4, res);
          } else {
            uint32_t p[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float lo = __uint_as_float(res[2 * k]), hi = __uint_as_float(res[2 * k + 1]);
              p[k] = a.out_dtype == DT_F16 ? pack2<__half>(lo, hi) : pack2<__nv_bfloat16>(lo, hi);
            }
            wp.write_own_row(p);
            __syncwarp();
            if (!a.transpose)
              store_block_rows(wp, out + ((size_t(t.b) * g.lm + wrow0) * g.ln + colb) * 2, size_t(g.ln) * 2);
            else
              store_block_columns16(wp, out + ((size_t(t.b) * g.ln + colb) * g.lm + wrow0) * 2, size_t(g.lm) * 2);
            __syncwarp();
          }
        } else {
          store_rows32(wp, reinterpret_cast<uint8_t*>(static_cast<float*>(a.out) + wbase), size_t(g.n) * 4, res);
        }
      }
    }
    __syncwarp();
    if constexpr (MODE == I8_GRAM) {
      imax = warp_max_i(imax);
      if (t.lane == 0 && imax > 0) atomicMax(static_cast<int*>(a.maximum) + t.b, imax);
    } else if constexpr (MODE != I8_UPDATE_FINAL) {
      fmax_ = warp_max(fmax_);
      if (t.lane == 0 && fmax_ > 0.f) atomic_max_nonneg(static_cast<float*>(a.maximum) + t.b, fmax_);
    }
  }

  template <class Acc>
  static __device__ __forceinline__ void run(const GemmGeom& g, const Args& a, const TileCtx& t,
                                             const Acc& acc) {
    if constexpr (!Acc::IN_REGS) {
      if (fast_ok(g, a, t)) {   // uniform over the tile's warps
        run_fast(g, a, t, acc);
        return;
      }
    }
    const bool row_ok = t.row < g.m;
    int imax = 0;
    float fmax_ = 0.f;
    float sa = 0.f, sb = 0.f, sq = 0.f, drow = 0.f, xrow = 0.f;
    if constexpr (MODE != I8_GRAM) {
      sa = a.a_scale[t.b];
      if (row_ok) drow = a.diag[size_t(t.b) * g.m + t.row];
    }
    if constexpr (MODE == I8_SQUARE) {
      sq = __fmul_rn(__fmul_rn(sa, sa), a.beta);
      xrow = __fmaf_rn(drow, a.beta, a.alpha);
    }
    if constexpr (MODE == I8_UPDATE || MODE == I8_UPDATE_FINAL) {
      sb = a.b_scale[t.b];
      if (a.use_gain) sb = __fmul_rn(sb, a.gain);   // int8.cu:258
    }
#pragma unroll 1
    for (int c = t.c_begin; c < t.c_end; ++c) {
      uint32_t v[32];
      acc.load(c, v);
      const int colb = t.col0 + c * 32;
      if (colb >= g.n || !row_ok) continue;
      const int ncol = min(32, g.n - colb);
      const size_t rbase = (size_t(t.b) * g.m + t.row) * g.n + colb;
      if constexpr (MODE == I8_GRAM) {
        int iv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          iv[j] = int(v[j]);
          const int col = colb + j;
          if (t.row < g.lm && col < g.ln && col != t.row) imax = max(imax, abs(iv[j]));
        }
        store_row<int>(static_cast<int*>(a.out) + rbase, iv, ncol);
      } else {
        float res[32];
        // Row-major int8 companion of this row chunk (g8 for square, a8 for update).
        const int8_t* comp = (MODE == I8_SQUARE)
            ? static_cast<const int8_t*>(g.a_raw) + (size_t(t.b) * g.m + t.row) * g.k + colb
            : a.row_b + rbase;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = colb + j;
          float accf = float(int(v[j]));
          float e = (col < g.n) ? float(comp[j]) : 0.f;
          float r;
          if constexpr (MODE == I8_SQUARE) {
            float dcol = (col < g.n) ? a.diag[size_t(t.b) * g.m + col] : 0.f;
            float cj = __fmul_rn(__fmul_rn(dcol, sa), a.beta);
            r = __fmaf_rn(accf, sq, __fmul_rn(e, __fmaf_rn(xrow, sa, cj)));
            if (col != t.row && (t.row >> 7) >= (col >> 7) && t.row < g.lm && col < g.ln)
              fmax_ = fmaxf(fmax_, fabsf(r));
          } else {
            r = __fmul_rn(__fmaf_rn(e, drow, __fmul_rn(accf, sa)), sb);
            if (MODE == I8_UPDATE && t.row < g.lm && col < g.ln) fmax_ = fmaxf(fmax_, fabsf(r));
          }
          res[j] = r;
        }
        if constexpr (MODE == I8_UPDATE_FINAL) {
          const size_t fbase = (size_t(t.b) * g.lm + t.row) * g.ln + colb;
          const int esz = a.out_dtype == DT_F32 ? 4 : 2;
          const bool wide = !a.transpose && t.row < g.lm && colb + 32 <= g.ln &&
                            ((reinterpret_cast<uintptr_t>(a.out) + fbase * esz) & 15u) == 0;
          if (wide) {
            if (a.out_dtype == DT_F32) {
              store_row<float>(static_cast<float*>(a.out) + fbase, res, 32);
            } else if (a.out_dtype == DT_F16) {
              alignas(16) __half hv[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) hv[j] = __float2half_rn(res[j]);
              store_row<__half>(static_cast<__half*>(a.out) + fbase, hv, 32);
            } else {
              alignas(16) __nv_bfloat16 bv[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) bv[j] = __float2bfloat16_rn(res[j]);
              store_row<__nv_bfloat16>(static_cast<__nv_bfloat16*>(a.out) + fbase, bv, 32);
            }
          } else if (t.row < g.lm) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = colb + j;
              if (col < g.ln) {
                size_t idx = a.transpose ? (size_t(t.b) * g.ln + col) * g.lm + t.row
                                         : (size_t(t.b) * g.lm + t.row) * g.ln + col;
                store_user(a.out, a.out_dtype, idx, res[j]);
              }
            }
          }
        } else {
          store_row<float>(static_cast<float*>(a.out) + rbase, res, ncol);
        }
      }
    }
    __syncwarp();
    if constexpr (MODE == I8_GRAM) {
      imax = warp_max_i(imax);
      if (t.lane == 0 && imax > 0) atomicMax(static_cast<int*>(a.maximum) + t.b, imax);
    } else if constexpr (MODE != I8_UPDATE_FINAL) {
      fmax_ = warp_max(fmax_);
      if (t.lane == 0 && fmax_ > 0.f) atomic_max_nonneg(static_cast<float*>(a.maximum) + t.b, fmax_);
    }
  }
};

}  // namespace i8m
