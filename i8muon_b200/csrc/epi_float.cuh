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
  float* amax;      // MODE_FINAL, optional: [batch] maximum magnitude of the stored values (zeroed by the caller)
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

// FP32 values travel between GEMMs as two planes: hi = v rounded to the nearest
// TF32 value (ties to even), lo = v - hi exactly.  Rounding instead of truncating
// keeps |lo| <= 2^-11 |v| with no sign bias, so the dropped lo*lo term of the
// three-product expansion stays near 2^-24 relative.
__device__ __forceinline__ float tf32_hi(float v) {
  uint32_t u = __float_as_uint(v);
  u += 0xfffu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xffffe000u);
}
// Low plane of the split.  The tensor core reads only the upper 19 bits of an
// operand, so the remainder is rounded (not truncated) to that width here.
__device__ __forceinline__ float tf32_lo(float v, float hi) {
#ifdef I8M_TF32_EXACT_LO
  return v - hi;
#else
  return tf32_hi(v - hi);
#endif
}

__device__ __forceinline__ void store_user(void* out, int dtype, size_t index, float v) {
  if (dtype == DT_F32) static_cast<float*>(out)[index] = v;
  else if (dtype == DT_F16) static_cast<__half*>(out)[index] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(out)[index] = __float2bfloat16_rn(v);
}

// Packed pairs of 16-bit values: rounding (to nearest even, as round_to) and widening.
template <typename E>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <typename E>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

template <typename E, int MODE>
struct EpiFloat {
  static constexpr bool IS_F32 = sizeof(E) == 4;
  static constexpr int E_CODE = std::is_same<E, __half>::value ? DT_F16 : (IS_F32 ? DT_F32 : DT_BF16);
  static constexpr int KIND = IS_F32 ? KIND_TF32 : KIND_F16;
  using Elem = E;
  static constexpr int PARTS = IS_F32 ? 2 : 1;
  static constexpr bool BLOCKQ = false;
  // FP32: fold the TMEM accumulator into registers after every K block (32 elements of
  // K, 12 tensor-core accumulations).  The tensor core accumulates with truncation:
  // measured bias of a whole-K Gram diagonal is about -1e-8 * K relative, which at
  // K = 4096 alone would exceed the 1e-5 bar of this path.
  static constexpr int PROMOTE_KB = IS_F32 ? 1 : 0;
  static constexpr int NBUF = IS_F32 ? 2 : 1;
  static constexpr int EPI_WARPS = 4;
  static constexpr int STAGES = 3;
  static constexpr int MIN_CTAS = IS_F32 ? 1 : 2;
  static constexpr uint32_t FMT = IS_F32 ? 2u : (std::is_same<E, __nv_bfloat16>::value ? 1u : 0u);
  static constexpr uint32_t IDESC = make_idesc(1u, FMT, FMT, TILE, TILE);
  using Args = FloatArgs;

  // Fast path of the 16-bit types for a tile that lies inside the logical extent: packed
  // conversions, 16-byte loads and stores only, the transposed copy through a 32 x 32 transpose in
  // the warp's own shared-memory patch (64 contiguous bytes per lane instead of 32 scattered
  // 2-byte stores).  Same roundings and the same un-fused arithmetic as the general path below.
  static __device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
  static __device__ __forceinline__ bool fast_ok(const GemmGeom& g, const Args& a, const TileCtx& t) {
    if (t.wsm == nullptr || t.row0 + TILE > g.lm || t.col0 + TILE > g.ln) return false;
    if constexpr (MODE == MODE_FINAL) {
      if (a.out_dtype != DT_F16 && a.out_dtype != DT_BF16) return false;
      return aligned16(a.out) && ((a.transpose ? g.lm : g.ln) & 7) == 0;
    } else {
      bool ok = aligned16(a.out) && (g.n & 7) == 0 && (g.m & 7) == 0 && (a.out_t == nullptr || aligned16(a.out_t));
      if constexpr (MODE == MODE_QUAD) ok = ok && aligned16(a.src) && (g.k & 7) == 0;
      return ok;
    }
  }

  template <class Acc>
  static __device__ __forceinline__ void run_fast(const GemmGeom& g, const Args& a, const TileCtx& t,
                                                  const Acc& acc) {
    const bool diag_tile = g.sym && t.tm == t.tn;
    const bool mirror = g.sym && t.tm != t.tn;
    const WarpPatch wp{smem_u32(t.wsm), t.lane};
    const int wrow0 = t.row0 + 32 * t.q;   // first row of this warp's block
    float stored_max = 0.f;
#pragma unroll 1
    for (int c = t.c_begin; c < t.c_end; ++c) {
      uint32_t v[32];
      acc.load(c, v);
      const int colb = t.col0 + c * 32;
      uint32_t p[16];
      if constexpr (MODE == MODE_QUAD) {
        // the left operand's block R[wrow0 .. + 31][colb .. + 31]: coalesced into the patch, then one row per lane
        load_block_rows(wp, reinterpret_cast<const uint8_t*>(static_cast<const E*>(a.src) +
                                                             (size_t(t.b) * g.m + wrow0) * g.k + colb),
                        size_t(g.k) * 2);
        __syncwarp();
        uint32_t rr[16];
        wp.read_own_row(rr);
        __syncwarp();
        const int dcol = t.tm == t.tn ? t.row - colb : -1;   // this row's diagonal column inside the chunk, if any
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const float2 r = unpack2<E>(rr[k]);
          float x0 = __fadd_rn(__fmul_rn(a.cb, r.x), __fmul_rn(a.cc, __uint_as_float(v[2 * k])));
          float x1 = __fadd_rn(__fmul_rn(a.cb, r.y), __fmul_rn(a.cc, __uint_as_float(v[2 * k + 1])));
          if (dcol == 2 * k) x0 = __fadd_rn(x0, a.ca);
          if (dcol == 2 * k + 1) x1 = __fadd_rn(x1, a.ca);
          p[k] = pack2<E>(x0, x1);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 16; ++k) p[k] = pack2<E>(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
      }
      if constexpr (MODE == MODE_FINAL) {
        // E -> the user's 16-bit type (a second rounding when they differ, as in the general path)
        if (a.out_dtype != E_CODE) {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float2 f = unpack2<E>(p[k]);
            p[k] = a.out_dtype == DT_F16 ? pack2<__half>(f.x, f.y) : pack2<__nv_bfloat16>(f.x, f.y);
          }
        }
        if (a.amax != nullptr) {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float2 f = a.out_dtype == DT_F16 ? unpack2<__half>(p[k]) : unpack2<__nv_bfloat16>(p[k]);
            stored_max = fmaxf(stored_max, fmaxf(fabsf(f.x), fabsf(f.y)));
          }
        }
        wp.write_own_row(p);
        __syncwarp();
        uint8_t* out = static_cast<uint8_t*>(a.out);
        if (!a.transpose)
          store_block_rows(wp, out + ((size_t(t.b) * g.lm + wrow0) * g.ln + colb) * 2, size_t(g.ln) * 2);
        else
          store_block_columns16(wp, out + ((size_t(t.b) * g.ln + colb) * g.lm + wrow0) * 2, size_t(g.lm) * 2);
        __syncwarp();
      } else {
        wp.write_own_row(p);
        __syncwarp();
        uint8_t* out = static_cast<uint8_t*>(a.out);
        store_block_rows(wp, out + ((size_t(t.b) * g.m + wrow0) * g.n + colb) * 2, size_t(g.n) * 2);
        // transposed copy: the mirrored half of a symmetric product, or the (n x m) transpose
        // that the next update GEMM consumes (a diagonal tile is bitwise symmetric already)
        uint8_t* tdst = mirror ? out : static_cast<uint8_t*>(a.out_t);
        if (tdst != nullptr && !diag_tile) {
          const int tld = mirror ? g.n : g.m;
          store_block_columns16(wp, tdst + ((size_t(t.b) * (mirror ? g.m : g.n) + colb) * tld + wrow0) * 2,
                                size_t(tld) * 2);
        }
        __syncwarp();   // the patch is free for the next chunk
      }
    }
    if constexpr (MODE == MODE_FINAL) {
      if (a.amax != nullptr) {
        stored_max = warp_max(stored_max);
        if (t.lane == 0 && stored_max > 0.f) atomic_max_nonneg(a.amax + t.b, stored_max);
      }
    }
  }

  template <class Acc>
  static __device__ __forceinline__ void run(const GemmGeom& g, const Args& a, const TileCtx& t,
                                             const Acc& acc) {
    if constexpr (!IS_F32 && !Acc::IN_REGS) {
      if (fast_ok(g, a, t)) {   // uniform over the tile's warps
        run_fast(g, a, t, acc);
        return;
      }
    }
    const bool row_ok = t.row < g.m;
    const bool diag_tile = g.sym && t.tm == t.tn;
    const bool mirror = g.sym && t.tm != t.tn;
    float stored_max = 0.f;
    auto body = [&](const int c) {
      uint32_t v[32];
      acc.load(c, v);
      const int colb = t.col0 + c * 32;
      if (colb >= g.n) return;  // uniform per CTA
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
      if (!row_ok) return;
      const int ncol = min(32, g.n - colb);
      if constexpr (MODE == MODE_FINAL) {
        if (a.amax != nullptr && t.row < g.lm) {
          // the value as the user's tensor holds it
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (colb + j < g.ln) {
              const float held = a.out_dtype == DT_F32 ? val[j]
                                 : a.out_dtype == DT_F16 ? __half2float(__float2half_rn(val[j]))
                                                         : __bfloat162float(__float2bfloat16_rn(val[j]));
              stored_max = fmaxf(stored_max, fabsf(held));
            }
          }
        }
        // a thread's 32 consecutive outputs leave as 16-byte stores when the row is aligned
        const size_t fbase = (size_t(t.b) * g.lm + t.row) * g.ln + colb;
        const int esz = a.out_dtype == DT_F32 ? 4 : 2;
        const bool wide = !a.transpose && t.row < g.lm && colb + 32 <= g.ln &&
                          ((reinterpret_cast<uintptr_t>(a.out) + fbase * esz) & 15u) == 0;
        if (wide) {
          if (a.out_dtype == DT_F32) {
            store_row<float>(static_cast<float*>(a.out) + fbase, val, 32);
          } else if (a.out_dtype == DT_F16) {
            alignas(16) __half hv[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) hv[j] = __float2half_rn(val[j]);
            store_row<__half>(static_cast<__half*>(a.out) + fbase, hv, 32);
          } else {
            alignas(16) __nv_bfloat16 bv[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) bv[j] = __float2bfloat16_rn(val[j]);
            store_row<__nv_bfloat16>(static_cast<__nv_bfloat16*>(a.out) + fbase, bv, 32);
          }
        } else if (t.row < g.lm) {
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
        // 16-bit products of a symmetric pair are bitwise symmetric (same products, same
        // accumulation order for (r, c) and (c, r); checked on the device), so a diagonal tile
        // is stored like any other and needs no mirror.  FP32 keeps the explicit mirror.
        if (!diag_tile || !IS_F32) {
          if constexpr (IS_F32) {
            float hi[32], lo[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) { hi[j] = tf32_hi(val[j]); lo[j] = tf32_lo(val[j], hi[j]); }
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
            if (!IS_F32 || col > t.row) continue;
            size_t d0 = (size_t(t.b) * g.m + t.row) * g.n + col;
            size_t d1 = (size_t(t.b) * g.m + col) * g.n + t.row;
            if constexpr (IS_F32) {
              float hi = tf32_hi(val[j]);
              const float lo = tf32_lo(val[j], hi);
              reinterpret_cast<float*>(out)[d0] = hi; out_lo[d0] = lo;
              reinterpret_cast<float*>(out)[d1] = hi; out_lo[d1] = lo;
            } else {
              out[d0] = round_to<E>(val[j]);
              out[d1] = round_to<E>(val[j]);
            }
          } else if (tdst != nullptr) {
            size_t d1 = (size_t(t.b) * (mirror ? g.m : g.n) + col) * tld + t.row;
            if constexpr (IS_F32) {
              float hi = tf32_hi(val[j]);
              reinterpret_cast<float*>(tdst)[d1] = hi; tdst_lo[d1] = tf32_lo(val[j], hi);
            } else {
              tdst[d1] = round_to<E>(val[j]);
            }
          }
        }
      }
    };
    if constexpr (Acc::IN_REGS) {
#pragma unroll
      for (int c = 0; c < TILE / 32; ++c) body(c);
    } else {
#pragma unroll 1
      for (int c = t.c_begin; c < t.c_end; ++c) body(c);
    }
    if constexpr (MODE == MODE_FINAL) {
      if (a.amax != nullptr) {
        __syncwarp();
        stored_max = warp_max(stored_max);
        if (t.lane == 0 && stored_max > 0.f) atomic_max_nonneg(a.amax + t.b, stored_max);
      }
    }
  }
};

}  // namespace i8m
