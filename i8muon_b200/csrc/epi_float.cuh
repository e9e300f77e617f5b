// Fused epilogues of the floating-point Newton-Schulz GEMMs (FP16 / BF16 with
// FP32 accumulation; FP32 as split-TF32 with two operand planes).
//
// Arithmetic follows the reference's floating path (src/i8muon/csrc/prec.cu:122-190):
//   MODE_PLAIN  out = E(acc)                                    (Gram, products, update)
//   MODE_QUAD   out = E(cb * R_ij + cc * acc  [+ ca on the diagonal])   R = the left operand
//   MODE_FINAL  user = Output(float(E(acc))), un-padded, optionally transposed
// with explicit un-fused multiplies and adds in MODE_QUAD.  Symmetric products
// compute tiles with tm >= tn and mirror them; a diagonal tile mirrors its own
// strictly-lower half so that the stored matrix is exactly symmetric.
#pragma once
#include "gemm_core.cuh"
#include <type_traits>

namespace i8m {

enum FloatMode : int { MODE_PLAIN = 0, MODE_QUAD = 1, MODE_FINAL = 2 };
enum DType : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_I8 = 3, DT_E4M3 = 4 };

struct FloatArgs {
  void* out;        // (batch, m, n) in E   | final: user tensor
  void* out_t;      // (batch, n, m) in E or nullptr
  void* out_lo;     // split-TF32 only: low planes of out / out_t
  void* out_t_lo;
  const void* src;  // MODE_QUAD: the left operand R (batch, m, k) in E (k == n)
  const void* src_lo;
  int out_dtype;    // MODE_FINAL: DType of the user tensor
  int transpose;    // MODE_FINAL: store (ln x lm)
  float ca, cb, cc;
};

template <typename E>
__device__ __forceinline__ E round_to(float v);
template <>
__device__ __forceinline__ __half round_to<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 round_to<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <typename E>
__device__ __forceinline__ float widen(E v);
template <>
__device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float widen<float>(float v) { return v; }

// FP32 values travel between GEMMs as two TF32-representable planes.
__device__ __forceinline__ float tf32_hi(float v) {
  return __uint_as_float(__float_as_uint(v) & 0xffffe000u);
}

__device__ __forceinline__ void store_user(void* out, int dtype, size_t index, float v) {
  if (dtype == DT_F32) static_cast<float*>(out)[index] = v;
  else if (dtype == DT_F16) static_cast<__half*>(out)[index] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(out)[index] = __float2bfloat16_rn(v);
}

template <typename E, int MODE>
struct EpiFloat {
  static constexpr bool IS_F32 = sizeof(E) == 4;
  static constexpr int KIND = IS_F32 ? KIND_TF32 : KIND_F16;
  using Elem = E;
  static constexpr int PARTS = IS_F32 ? 2 : 1;
  static constexpr bool BLOCKQ = false;
  static constexpr int STAGES = IS_F32 ? 3 : 3;
  static constexpr int MIN_CTAS = IS_F32 ? 1 : 2;
  static constexpr uint32_t FMT = IS_F32 ? 2u : (std::is_same<E, __nv_bfloat16>::value ? 1u : 0u);
  static constexpr uint32_t IDESC = make_idesc(1u, FMT, FMT, TILE, TILE);
  using Args = FloatArgs;

  template <class Acc>
  static __device__ __forceinline__ void run(const GemmGeom& g, const Args& a, const TileCtx& t,
                                             const Acc& acc) {
    const bool row_ok = t.row < g.m;
    const bool diag_tile = g.sym && t.tm == t.tn;
    const bool mirror = g.sym && t.tm != t.tn;
#pragma unroll 1
    for (int c = 0; c < TILE / 32; ++c) {
      uint32_t v[32];
      acc.load(c, v);
      const int colb = t.col0 + c * 32;
      if (colb >= g.n) continue;  // uniform per CTA
      float val[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float x = __uint_as_float(v[j]);
        const int col = colb + j;
        if constexpr (MODE == MODE_QUAD) {
          float rij = 0.f;
          if (row_ok && col < g.n) {
            size_t si = (size_t(t.b) * g.m + t.row) * g.k + col;
            rij = widen<E>(static_cast<const E*>(a.src)[si]);
            if constexpr (IS_F32) rij = __fadd_rn(rij, static_cast<const float*>(a.src_lo)[si]);
          }
          x = __fadd_rn(__fmul_rn(a.cb, rij), __fmul_rn(a.cc, x));
          if (t.row == col) x = __fadd_rn(x, a.ca);
        }
        // Values outside the logical extent are stored as zero padding.
        val[j] = (t.row < g.lm && col < g.ln) ? widen<E>(round_to<E>(x)) : 0.f;
      }
      if (!row_ok) continue;
      const int ncol = min(32, g.n - colb);
      if constexpr (MODE == MODE_FINAL) {
        if (t.row < g.lm) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = colb + j;
            if (col < g.ln) {
              size_t idx = a.transpose ? (size_t(t.b) * g.ln + col) * g.lm + t.row
                                       : (size_t(t.b) * g.lm + t.row) * g.ln + col;
              store_user(a.out, a.out_dtype, idx, val[j]);
            }
          }
        }
      } else {
        E* out = static_cast<E*>(a.out);
        float* out_lo = static_cast<float*>(a.out_lo);
        const size_t rbase = (size_t(t.b) * g.m + t.row) * g.n + colb;
        if (!diag_tile) {
          if constexpr (IS_F32) {
            float hi[32], lo[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) { hi[j] = tf32_hi(val[j]); lo[j] = val[j] - hi[j]; }
            store_row<float>(reinterpret_cast<float*>(out) + rbase, hi, ncol);
            store_row<float>(out_lo + rbase, lo, ncol);
          } else {
            E ev[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) ev[j] = round_to<E>(val[j]);
            store_row<E>(out + rbase, ev, ncol);
          }
        }
        // Transposed copy: mirrored half of a symmetric product, or the
        // (n x m) transpose that the next update GEMM consumes.
        E* tdst = mirror ? out : static_cast<E*>(a.out_t);
        float* tdst_lo = mirror ? out_lo : static_cast<float*>(a.out_t_lo);
        const int tld = mirror ? g.n : g.m;  // row length of the transposed target
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = colb + j;
          if (col >= g.n) continue;
          if (diag_tile) {
            if (col > t.row) continue;
            size_t d0 = (size_t(t.b) * g.m + t.row) * g.n + col;
            size_t d1 = (size_t(t.b) * g.m + col) * g.n + t.row;
            if constexpr (IS_F32) {
              float hi = tf32_hi(val[j]);
              reinterpret_cast<float*>(out)[d0] = hi; out_lo[d0] = val[j] - hi;
              reinterpret_cast<float*>(out)[d1] = hi; out_lo[d1] = val[j] - hi;
            } else {
              out[d0] = round_to<E>(val[j]);
              out[d1] = round_to<E>(val[j]);
            }
          } else if (tdst != nullptr) {
            size_t d1 = (size_t(t.b) * (mirror ? g.m : g.n) + col) * tld + t.row;
            if constexpr (IS_F32) {
              float hi = tf32_hi(val[j]);
              reinterpret_cast<float*>(tdst)[d1] = hi; tdst_lo[d1] = val[j] - hi;
            } else {
              tdst[d1] = round_to<E>(val[j]);
            }
          }
        }
      }
    }
  }
};

}  // namespace i8m
