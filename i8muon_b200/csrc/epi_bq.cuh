// Fused epilogues of the 128x128 block-quantised Newton-Schulz GEMMs (INT8 via
// tcgen05 kind::i8, E4M3 via kind::f8f6f4).
//
// Every 128-deep K block is accumulated on its own in tensor memory and then
// promoted:  total = fmaf(float(partial), sA[tm,kb] * sB[.,kb], total)  in ascending
// kb order, as in the reference (src/i8muon/csrc/bq.cu:190-195).  The tile tail
// restates bq.cu:204-299 with the fused multiply-adds that the reference's --fmad=true build
// contains (established bit for bit, every stage, against tensors recorded from the reference's
// own build for sm_100a: tests/golden/reference_ns_bq_*.npz); every rounding is explicit here:
//   BQ_GRAM    diagonal -> dout (zero beyond the logical size), diagonal entry zeroed
//   BQ_POLY    v = g_ij * sG[tm,tn];  val = fma(v, cb, fma(d_i + d_j, v, total) * cc);
//              diagonal: dout_i = val + fma(d_i, fma(d_i, cc, cb), ca), entry zeroed
//   BQ_UPDATE  val = fma(a_ij * dP_i, sA[tm,tn], total)
// then (non-final) tile max (floor 1e-8) -> scale, quantise (INT8 truncates toward
// zero, E4M3 rounds to nearest even and saturates), store the tile and its
// mirror / transpose; the final update casts to the user's dtype instead.
//
// How the promotion keeps up with the tensor core (one K block is ~270 cycles of
// tcgen05.mma; 128 x 128 partials have to be folded in that time by four warps):
//   * int32 -> FP32 without the conversion unit: each TMEM buffer is preset to the
//     bit pattern of 1.5 * 2^23 and the MMA accumulates on top of it, so what the
//     epilogue loads IS the float 12582912 + partial (|partial| <= 128 * 127^2 < 2^22);
//     one exact subtraction recovers float(partial);
//   * that subtraction and the fmaf run as packed two-lane FP32 instructions
//     (add.rn.f32x2 / fma.rn.f32x2), halving the issue slots;
//   * four TMEM buffers (all 512 columns) decouple the two sides.
#pragma once
#include "epi_float.cuh"

namespace i8m {

// BQ_PLAIN: the tail alone on values that another GEMM's epilogue computed (the FP16 first row of an
// fp16-first call): tile maximum, quantise, store A, A^T and the block scale as BQ_UPDATE does.
enum BqMode : int { BQ_GRAM = 0, BQ_POLY = 1, BQ_UPDATE = 2, BQ_UPDATE_FINAL = 3, BQ_PLAIN = 4 };

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

// int8 <-> float without the conversion unit (its rate is a quarter of the FP32 lanes):
//   decode   float(q) = as_float(0x4B400000 + q) - 12582912    (exact for |q| <= 127)
//   quantise trunc(|x|) = low bits of as_uint(|x| + 8388608 rounded toward zero), |x| < 2^23,
//            then the sign is put back; identical to clamp(cvt.rzi(x), -127, 127).
template <bool FP8>
__device__ __forceinline__ float bq_decode(uint8_t v) {
  if constexpr (FP8) return e4m3_to_float(v);
  else return __fadd_rn(__uint_as_float(0x4B400000u + uint32_t(int(int8_t(v)))), -12582912.0f);
}
template <bool FP8>
__device__ __forceinline__ uint8_t bq_quant(float v, float multiplier) {
  float x = __fmul_rn(v, multiplier);
  if constexpr (FP8) {
    return uint8_t(__nv_cvt_float_to_fp8(fmaxf(-448.f, x), __NV_SATFINITE, __NV_E4M3));
  } else {
    // |x| <= 127 * (1 + 2^-23): the multiplier is 127 / (block maximum), so no clamp is needed
    const uint32_t zb = __float_as_uint(__fadd_rz(fabsf(x), 8388608.0f));   // low byte = trunc(|x|)
    const uint32_t sm = uint32_t(int(__float_as_uint(x)) >> 31);            // 0 or all ones
    return uint8_t(((zb & 0xffu) ^ sm) - sm);                               // two's complement of the sign
  }
}

// packed two-lane FP32 arithmetic (sm_100): one issue slot for two IEEE operations
__device__ __forceinline__ unsigned long long pack2(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ float lane0(unsigned long long v) { return __uint_as_float(uint32_t(v)); }
__device__ __forceinline__ float lane1(unsigned long long v) { return __uint_as_float(uint32_t(v >> 32)); }

constexpr uint32_t I8_MAGIC_BITS = 0x4B400000u;  // 1.5 * 2^23 = 12582912.0f
constexpr float I8_MAGIC = 12582912.0f;

template <bool FP8, int MODE>
struct EpiBq {
  static constexpr int KIND = FP8 ? KIND_F8 : KIND_I8;
  using Elem = uint8_t;
  static constexpr int PARTS = 1;
  static constexpr bool BLOCKQ = true;
  static constexpr int PROMOTE_KB = 1;
  static constexpr int NBUF = 4;           // TMEM accumulators of 128 columns
  static constexpr bool PRESET = !FP8;     // INT8: accumulators start at the bias constant
  static constexpr bool SPLIT_TAIL = MODE != BQ_PLAIN;   // has a split_tail() for bq_split_kernel
  static constexpr int STAGES = 4;
  static constexpr int MIN_CTAS = 1;
  // eight epilogue warps: two per scheduler, each thread owns half a row (64 columns),
  // so one warp's TMEM-load latency hides behind the other's arithmetic
  static constexpr int EPI_WARPS = 8;
  static constexpr int CPT = TILE / (EPI_WARPS / 4);   // columns per thread
  static constexpr int EPI_THREADS = 32 * EPI_WARPS;
  static constexpr int TSM_PITCH = TILE + 16;       // row pitch of the transposed staging tile
  static constexpr int TSM_BYTES = TILE * TSM_PITCH;
  static constexpr uint32_t IDESC =
      FP8 ? make_idesc(1u, 0u, 0u, TILE, TILE) : make_idesc(2u, 1u, 1u, TILE, TILE);
  using Args = BqArgs;
  static constexpr float QMAX = FP8 ? 448.f : 127.f;

  // The two factors of a K block's scale product, for callers that fetch them long before
  // the multiplication (the product itself would wait for both loads where it is written).
  static __device__ __forceinline__ void block_scale_factors(const GemmGeom& g, const Args& a, const TileCtx& t,
                                                             int kb, int mq, int nq, int kq, float& fa, float& fb) {
    if constexpr (MODE == BQ_UPDATE || MODE == BQ_UPDATE_FINAL)
      fb = a.sb[(size_t(t.b) * kq + kb) * nq + t.tn];
    else
      fb = a.sb[(size_t(t.b) * nq + t.tn) * kq + kb];
    fa = a.sa[(size_t(t.b) * mq + t.tm) * kq + kb];
  }
  static __device__ __forceinline__ float block_scale(const GemmGeom& g, const Args& a,
                                                      const TileCtx& t, int kb, int mq, int nq,
                                                      int kq) {
    float bs;
    if constexpr (MODE == BQ_UPDATE || MODE == BQ_UPDATE_FINAL)
      bs = a.sb[(size_t(t.b) * kq + kb) * nq + t.tn];
    else
      bs = a.sb[(size_t(t.b) * nq + t.tn) * kq + kb];
    return __fmul_rn(a.sa[(size_t(t.b) * mq + t.tm) * kq + kb], bs);
  }

  // Fold one K block (this thread's 64 partials) into the FP32 totals:
  //   total = fmaf(float(partial), s, total)
  // INT8 partials arrive biased by 12582912 (preset accumulator); one exact subtraction
  // recovers float(partial).  Packed flavour: two IEEE operations per instruction.
  static __device__ __forceinline__ void fold64p(unsigned long long (&tot)[32], const uint32_t (&v)[2][32],
                                                 const float s) {
    const unsigned long long neg_magic = pack2(__float_as_uint(-I8_MAGIC), __float_as_uint(-I8_MAGIC));
    const unsigned long long s2 = pack2(__float_as_uint(s), __float_as_uint(s));
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        unsigned long long p = pack2(v[c][2 * j], v[c][2 * j + 1]);
        if constexpr (PRESET) p = add2(p, neg_magic);
        tot[c * 16 + j] = fma2(p, s2, tot[c * 16 + j]);
      }
    }
  }
  // Debug core of the one-tile-per-CTA skeleton: plain dot products per K block, the same
  // promotion arithmetic and the same tail.
  static __device__ __forceinline__ void run_debug(const GemmGeom& g, const Args& a, const TileCtx& t) {
    constexpr int Q = TILE;
    const int mq = g.m / Q, nq = g.n / Q, kq = g.k / Q;
    const int c0 = t.half * CPT;  // first tile column of this thread
    float vals[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) vals[j] = 0.f;
#pragma unroll 1
    for (int kb = 0; kb < g.num_kb; ++kb) {
      const float s = block_scale(g, a, t, kb, mq, nq, kq);
#pragma unroll 4
      for (int j = 0; j < CPT; ++j) {
        const uint32_t v = simt_dot<KIND, uint8_t>(g, t.b, t.row, t.col0 + c0 + j, kb * Q, kb * Q + Q);
        const float p = FP8 ? __uint_as_float(v) : float(int(v));
        vals[j] = __fmaf_rn(p, s, vals[j]);
      }
    }
    const Pre pre = tail_prefetch(g, a, t, mq, nq, kq);
    tail(g, a, t, vals, true, pre, mq, nq, kq);
  }

  // What the tail needs from global memory besides the accumulator: the row diagonal,
  // the tile's own block scale and this thread's 64 companion bytes (G for the polynomial,
  // A for the update).  Fetched before the K loop so that their latency is off the tail.
  struct Pre {
    uint4 comp[CPT / 16];
    float drow, stile;
  };
  static __device__ __forceinline__ Pre tail_prefetch(const GemmGeom& g, const Args& a, const TileCtx& t,
                                                      int mq, int nq, int kq) {
    Pre p;
    p.drow = 0.f; p.stile = 0.f;
    const int colbase = t.col0 + t.half * CPT;
    if constexpr (MODE != BQ_GRAM && MODE != BQ_PLAIN) p.drow = a.da[size_t(t.b) * g.m + t.row];
    if constexpr (MODE == BQ_POLY) p.stile = a.sa[(size_t(t.b) * mq + t.tm) * kq + t.tn];
    if constexpr (MODE == BQ_UPDATE || MODE == BQ_UPDATE_FINAL)
      p.stile = a.sb[(size_t(t.b) * kq + t.tm) * nq + t.tn];
    const uint4* comp = nullptr;
    if constexpr (MODE == BQ_POLY)
      comp = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(g.a_raw) +
                                            (size_t(t.b) * g.m + t.row) * g.k + colbase);
    if constexpr (MODE == BQ_UPDATE || MODE == BQ_UPDATE_FINAL)
      comp = reinterpret_cast<const uint4*>(a.row_b + (size_t(t.b) * g.m + t.row) * g.n + colbase);
#pragma unroll
    for (int i = 0; i < CPT / 16; ++i) p.comp[i] = comp ? comp[i] : make_uint4(0u, 0u, 0u, 0u);
    return p;
  }

  // ---------------------------------------------------------------- tile tail, split kernel
  // The same arithmetic as tail() below, run by four dedicated warps on a tile whose FP32 totals
  // the fold warps parked in shared memory (row pitch PARK_PITCH floats), so that the fold warps
  // are already inside the next tile's K loop.  These warps share their schedulers with the fold
  // warps, whose FP32 pipe is the busy one, so the tail is written for few instructions and keeps
  // conversions on the conversion unit (int8 -> float, float -> int8 / e4m3), which is idle here.
  //   pass 0  thread = tile row: value = f(total, companion byte, diagonals) in place, tile maximum
  //           (a Gram tile away from the diagonal and the edges only needs the maximum)
  //   pass 1  thread = tile row: quantise, 16-byte stores of the row-major tile; the codes also go
  //           back over the start of the thread's own parked row
  //   pass 2  thread = 4 columns x 32 rows of the same warp's rows: 4 x 4 byte transposes of the
  //           codes, 16-byte stores of the transposed (update) or mirrored (gram / poly) tile
  // The four warps meet once per tile on an mbarrier (bounded wait), never on bar.sync.
  static constexpr int PARK_PITCH = TILE + 4;   // floats; 16-byte aligned rows, conflict-free 16-byte accesses

  static __device__ __forceinline__ float code_to_float(uint32_t word, int byte) {
    const uint32_t q = (word >> (8 * byte)) & 0xffu;
    if constexpr (FP8) return e4m3_to_float(uint8_t(q));
    else return float(int(int8_t(q)));            // exact; one conversion-unit instruction
  }
  // four values -> four codes in one word (byte i = value i); same results as bq_quant
  static __device__ __forceinline__ uint32_t quant4(float x0, float x1, float x2, float x3, float multiplier) {
    if constexpr (FP8) {
      const float2 lo = make_float2(fmaxf(-448.f, __fmul_rn(x0, multiplier)), fmaxf(-448.f, __fmul_rn(x1, multiplier)));
      const float2 hi = make_float2(fmaxf(-448.f, __fmul_rn(x2, multiplier)), fmaxf(-448.f, __fmul_rn(x3, multiplier)));
      return uint32_t(__nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3)) |
             (uint32_t(__nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3)) << 16);
    } else {
      // |x| <= 127 (1 + 2^-23): truncation toward zero lands in [-127, 127] without a clamp
      const uint32_t i0 = uint32_t(__float2int_rz(__fmul_rn(x0, multiplier)));
      const uint32_t i1 = uint32_t(__float2int_rz(__fmul_rn(x1, multiplier)));
      const uint32_t i2 = uint32_t(__float2int_rz(__fmul_rn(x2, multiplier)));
      const uint32_t i3 = uint32_t(__float2int_rz(__fmul_rn(x3, multiplier)));
      return __byte_perm(__byte_perm(i0, i1, 0x0040), __byte_perm(i2, i3, 0x0040), 0x5410);
    }
  }

  // pass 0 on 16 consecutive columns of this thread's row.  SPECIAL: the tile touches the diagonal or
  // the logical edge of the matrix (tile-uniform), and only then are elements zeroed or set aside.
  template <bool SPECIAL>
  static __device__ __forceinline__ float split_values16(const GemmGeom& g, const Args& a, const int b, const int row,
                                                         const int col0, const int tid, const int j, const bool in_rows,
                                                         const bool diag_tile, const float drow, const float stile,
                                                         const uint8_t* comp, const float* dcols, const uint32_t my_row,
                                                         float mx) {
    float vals[16];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 x = lds128(my_row + uint32_t(16 * j + 4 * q4) * 4u);
      vals[4 * q4] = x.x; vals[4 * q4 + 1] = x.y; vals[4 * q4 + 2] = x.z; vals[4 * q4 + 3] = x.w;
    }
    if constexpr (MODE == BQ_GRAM && !SPECIAL) {
#pragma unroll
      for (int e = 0; e < 16; ++e) mx = fmaxf(mx, fabsf(vals[e]));
      return mx;                                   // nothing changes: no write-back
    }
    uint32_t words[4] = {0u, 0u, 0u, 0u};
    if constexpr (MODE != BQ_GRAM) {
      const uint4 cw = *reinterpret_cast<const uint4*>(comp + 16 * j);
      words[0] = cw.x; words[1] = cw.y; words[2] = cw.z; words[3] = cw.w;
    }
    float dc[16];
    if constexpr (MODE == BQ_POLY) {
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float4 d4 = *reinterpret_cast<const float4*>(dcols + 16 * j + 4 * q4);
        dc[4 * q4] = d4.x; dc[4 * q4 + 1] = d4.y; dc[4 * q4 + 2] = d4.z; dc[4 * q4 + 3] = d4.w;
      }
    }
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const int c = 16 * j + e;            // column inside the tile
      float val = vals[e];
      if constexpr (MODE == BQ_GRAM) {
        if (SPECIAL && diag_tile && c == tid) {
          a.dout[size_t(b) * g.m + row] = in_rows ? val : 0.f;
          val = 0.f;
        }
      } else if constexpr (MODE == BQ_POLY) {
        const float v = __fmul_rn(code_to_float(words[e >> 2], e & 3), stile);
        val = __fmaf_rn(__fadd_rn(drow, dc[e]), v, val);
        val = __fmaf_rn(v, a.cb, __fmul_rn(val, a.cc));
        if (SPECIAL && diag_tile && c == tid) {
          const float dpoly = __fmaf_rn(drow, __fmaf_rn(drow, a.cc, a.cb), a.ca);
          a.dout[size_t(b) * g.m + row] = in_rows ? __fadd_rn(val, dpoly) : 0.f;
          val = 0.f;
        }
      } else {
        val = __fmaf_rn(__fmul_rn(code_to_float(words[e >> 2], e & 3), drow), stile, val);
      }
      if (SPECIAL && (!in_rows || col0 + c >= g.ln)) val = 0.f;   // padding never contributes to a block scale
      mx = fmaxf(mx, fabsf(val));
      vals[e] = val;
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4)
      sts128(my_row + uint32_t(16 * j + 4 * q4) * 4u,
             make_float4(vals[4 * q4], vals[4 * q4 + 1], vals[4 * q4 + 2], vals[4 * q4 + 3]));
    return mx;
  }

  // eight consecutive values -> the caller's 16-bit dtype, one 16-byte vector
  static __device__ __forceinline__ uint4 pack8_16bit(const float* v, int dtype) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (dtype == DT_BF16)
        w[e] = uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(v[2 * e]))) |
               (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(v[2 * e + 1]))) << 16);
      else
        w[e] = uint32_t(__half_as_ushort(__float2half_rn(v[2 * e]))) |
               (uint32_t(__half_as_ushort(__float2half_rn(v[2 * e + 1]))) << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }

  // The last update of a call: value = fma(a * dP, sA, total) cast to the caller's dtype, un-padded, in the
  // caller's orientation.  Row-major results leave straight from pass 0; a transposed result (rows > cols
  // inputs) goes back into the parked tile and leaves column by column after the four warps have met.
  static __device__ __forceinline__ bool split_tail_final(const GemmGeom& g, const Args& a, const int b, const int tm,
                                                          const int tn, const int tid, const int it, const uint32_t park,
                                                          Ctrl* ctrl, volatile uint32_t* abort_flag, const int nq,
                                                          const int kq) {
    const int lane = tid & 31;
    const int row0 = tm * TILE, col0 = tn * TILE;
    const int row = row0 + tid;
    const bool in_rows = row < g.lm;
    const float drow = a.da[size_t(b) * g.m + row];
    const float stile = a.sb[(size_t(b) * kq + tm) * nq + tn];
    const uint8_t* comp = a.row_b + (size_t(b) * g.m + row) * g.n + col0;
    const uint32_t my_row = park + uint32_t(tid * PARK_PITCH) * 4u;
    const int esz = a.out_dtype == DT_F32 ? 4 : 2;
    const bool vec_rows = !a.transpose && in_rows && (g.ln % 8) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
#pragma unroll 1
    for (int j = 0; j < TILE / 16; ++j) {
      const uint4 cw = *reinterpret_cast<const uint4*>(comp + 16 * j);
      const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
      float vals[16];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float4 x = lds128(my_row + uint32_t(16 * j + 4 * q4) * 4u);
        vals[4 * q4] = x.x; vals[4 * q4 + 1] = x.y; vals[4 * q4 + 2] = x.z; vals[4 * q4 + 3] = x.w;
      }
#pragma unroll
      for (int e = 0; e < 16; ++e)
        vals[e] = __fmaf_rn(__fmul_rn(code_to_float(words[e >> 2], e & 3), drow), stile, vals[e]);
      if (a.transpose) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          sts128(my_row + uint32_t(16 * j + 4 * q4) * 4u,
                 make_float4(vals[4 * q4], vals[4 * q4 + 1], vals[4 * q4 + 2], vals[4 * q4 + 3]));
      } else if (in_rows) {
        const int col = col0 + 16 * j;
        const size_t idx = (size_t(b) * g.lm + row) * g.ln + col;
        if (vec_rows && col + 16 <= g.ln) {
          if (esz == 2) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + idx);
            dst[0] = pack8_16bit(vals, a.out_dtype);
            dst[1] = pack8_16bit(vals + 8, a.out_dtype);
          } else {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(a.out) + idx);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              dst[q4] = make_float4(vals[4 * q4], vals[4 * q4 + 1], vals[4 * q4 + 2], vals[4 * q4 + 3]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            if (col + e < g.ln) store_user(a.out, a.out_dtype, idx + e, vals[e]);
        }
      }
    }
    if (!a.transpose) return true;
    // transposed result: the warps meet (rows of other warps are read below), then thread = tile column
    __syncwarp();
    const uint32_t meet = smem_u32(&ctrl->tail_sync);
    mbar_arrive_if(meet, lane == 0 ? 1u : 0u);
    if (!mbar_wait_warp_inline(meet, uint32_t(it) & 1u, abort_flag)) return false;
    const int col = col0 + tid;
    if (col >= g.ln) return true;
    const uint32_t my_col = park + uint32_t(tid) * 4u;
    const size_t tbase = (size_t(b) * g.ln + col) * g.lm + row0;      // out is (batch, ln, lm)
    const bool vec_cols = (g.lm % 8) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
#pragma unroll 1
    for (int j = 0; j < TILE / 8; ++j) {
      if (row0 + 8 * j >= g.lm) break;
      float vals[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) vals[e] = lds32(my_col + uint32_t((8 * j + e) * PARK_PITCH) * 4u);
      if (vec_cols && row0 + 8 * j + 8 <= g.lm) {
        if (esz == 2) {
          *reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + tbase + 8 * j) = pack8_16bit(vals, a.out_dtype);
        } else {
          float4* dst = reinterpret_cast<float4*>(static_cast<float*>(a.out) + tbase + 8 * j);
          dst[0] = make_float4(vals[0], vals[1], vals[2], vals[3]);
          dst[1] = make_float4(vals[4], vals[5], vals[6], vals[7]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (row0 + 8 * j + e < g.lm) store_user(a.out, a.out_dtype, tbase + 8 * j + e, vals[e]);
      }
    }
    return true;
  }

  static __device__ __forceinline__ bool split_tail(const GemmGeom& g, const Args& a, const int b, const int tm,
                                                    const int tn, const int tid, const int it, const uint32_t park,
                                                    Ctrl* ctrl, volatile uint32_t* abort_flag, const int mq,
                                                    const int nq, const int kq) {
    if constexpr (MODE == BQ_UPDATE_FINAL) return split_tail_final(g, a, b, tm, tn, tid, it, park, ctrl, abort_flag, nq, kq);
    const int lane = tid & 31, w = tid >> 5;
    const int row0 = tm * TILE, col0 = tn * TILE;
    const int row = row0 + tid;
    const bool in_rows = row < g.lm;
    const bool diag_tile = (MODE != BQ_UPDATE) && tm == tn;
    const bool special = diag_tile || row0 + TILE > g.lm || col0 + TILE > g.ln;
    float drow = 0.f, stile = 0.f;
    if constexpr (MODE != BQ_GRAM) drow = a.da[size_t(b) * g.m + row];
    if constexpr (MODE == BQ_POLY) stile = a.sa[(size_t(b) * mq + tm) * kq + tn];
    if constexpr (MODE == BQ_UPDATE) stile = a.sb[(size_t(b) * kq + tm) * nq + tn];
    const uint8_t* comp = nullptr;
    if constexpr (MODE == BQ_POLY)
      comp = static_cast<const uint8_t*>(g.a_raw) + (size_t(b) * g.m + row) * g.k + col0;
    if constexpr (MODE == BQ_UPDATE) comp = a.row_b + (size_t(b) * g.m + row) * g.n + col0;
    const float* dcols = (MODE == BQ_POLY) ? a.da + size_t(b) * g.m + col0 : nullptr;
    const uint32_t my_row = park + uint32_t(tid * PARK_PITCH) * 4u;

    // ---- pass 0
    float mx = 1e-8f;
    if (special) {
#pragma unroll 1
      for (int j = 0; j < TILE / 16; ++j)
        mx = split_values16<true>(g, a, b, row, col0, tid, j, in_rows, diag_tile, drow, stile, comp, dcols, my_row, mx);
    } else {
#pragma unroll 1
      for (int j = 0; j < TILE / 16; ++j)
        mx = split_values16<false>(g, a, b, row, col0, tid, j, in_rows, diag_tile, drow, stile, comp, dcols, my_row, mx);
    }
    mx = warp_max(mx);
    if (lane == 0) ctrl->red[w] = mx;
    __syncwarp();
    const uint32_t meet = smem_u32(&ctrl->tail_sync);
    mbar_arrive_if(meet, lane == 0 ? 1u : 0u);
    if (!mbar_wait_warp_inline(meet, uint32_t(it) & 1u, abort_flag)) return false;
    mx = fmaxf(fmaxf(ctrl->red[0], ctrl->red[1]), fmaxf(ctrl->red[2], ctrl->red[3]));
    const float multiplier = QMAX / mx;
    if (tid == 0) {
      const float scale = 1.f / multiplier;
      a.so[(size_t(b) * mq + tm) * nq + tn] = scale;
      if constexpr (MODE != BQ_UPDATE) a.so[(size_t(b) * mq + tn) * nq + tm] = scale;
    }

    // ---- pass 1: the row-major tile (a diagonal tile takes its upper half from the lower one)
    uint8_t* out = static_cast<uint8_t*>(a.out);
    uint4* orow = reinterpret_cast<uint4*>(out + (size_t(b) * g.m + row) * g.n + col0);
    const uint32_t my_col = park + uint32_t(tid) * 4u;
#pragma unroll 1
    for (int j = 0; j < TILE / 16; ++j) {
      float vals[16];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float4 x = lds128(my_row + uint32_t(16 * j + 4 * q4) * 4u);
        vals[4 * q4] = x.x; vals[4 * q4 + 1] = x.y; vals[4 * q4 + 2] = x.z; vals[4 * q4 + 3] = x.w;
      }
      if (diag_tile && 16 * j + 15 > tid) {
#pragma unroll
        for (int e = 0; e < 16; ++e)
          if (16 * j + e > tid) vals[e] = lds32(my_col + uint32_t((16 * j + e) * PARK_PITCH) * 4u);
      }
      uint4 codes;
      codes.x = quant4(vals[0], vals[1], vals[2], vals[3], multiplier);
      codes.y = quant4(vals[4], vals[5], vals[6], vals[7], multiplier);
      codes.z = quant4(vals[8], vals[9], vals[10], vals[11], multiplier);
      codes.w = quant4(vals[12], vals[13], vals[14], vals[15], multiplier);
      orow[j] = codes;
      // the codes of columns 16j .. 16j+15 go over floats 4j .. 4j+3 of this row, which this thread has
      // read already (chunk j / 4); a diagonal tile has no third pass and other rows still read its floats
      if (!diag_tile) sts128u(my_row + uint32_t(16 * j), codes);
    }
    // ---- pass 2: codes of rows 32w .. 32w+31 (this warp's own), columns 4 lane .. 4 lane + 3, transposed
    if (!diag_tile) {
      __syncwarp();
      uint8_t* tdst = (MODE == BQ_UPDATE) ? static_cast<uint8_t*>(a.out_t) : out;
      const int trows = (MODE == BQ_UPDATE) ? g.n : g.m;
      const int tld = (MODE == BQ_UPDATE) ? g.m : g.n;
      uint8_t* tbase = tdst + (size_t(b) * trows + col0 + 4 * lane) * tld + row0 + 32 * w;
      const uint32_t src = park + uint32_t(32 * w * PARK_PITCH) * 4u + uint32_t(4 * lane);
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t o[4][4];       // [column][four rows each]
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          uint32_t r4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) r4[i] = lds32u(src + uint32_t((16 * half + 4 * blk + i) * PARK_PITCH) * 4u);
          const uint32_t t0 = __byte_perm(r4[0], r4[1], 0x5140), t1 = __byte_perm(r4[2], r4[3], 0x5140);
          const uint32_t t2 = __byte_perm(r4[0], r4[1], 0x7362), t3 = __byte_perm(r4[2], r4[3], 0x7362);
          o[0][blk] = __byte_perm(t0, t1, 0x5410);
          o[1][blk] = __byte_perm(t0, t1, 0x7632);
          o[2][blk] = __byte_perm(t2, t3, 0x5410);
          o[3][blk] = __byte_perm(t2, t3, 0x7632);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(tbase + size_t(c) * tld + 16 * half) = make_uint4(o[c][0], o[c][1], o[c][2], o[c][3]);
      }
    }
    return true;
  }

  // ---------------------------------------------------------------- tile tail
  static __device__ __forceinline__ void tail(const GemmGeom& g, const Args& a, const TileCtx& t,
                                              float (&vals)[CPT], const bool live, const Pre& pre,
                                              int mq, int nq, int kq) {
    const int c0 = t.half * CPT;           // first tile column of this thread
    const int colbase = t.col0 + c0;       // first global column of this thread
    const bool in_rows = t.row < g.lm;
    // thread-uniform shortcuts: most threads own no padding and no diagonal element
    const bool inside = in_rows && colbase + CPT <= g.ln;
    constexpr bool RECT = MODE == BQ_UPDATE || MODE == BQ_PLAIN;   // rectangular result with a transposed copy
    const bool has_diag = (MODE == BQ_GRAM || MODE == BQ_POLY) && t.tm == t.tn;
    const float drow = pre.drow, stile = pre.stile;
    if constexpr (MODE == BQ_POLY) {
      // the column diagonals of this tile, shared through shared memory
      if (t.half == 0) t.diag[t.r] = a.da[size_t(t.b) * g.m + t.col0 + t.r];
      named_bar_sync(1, EPI_THREADS);
    }

    float mx = 1e-8f;
#pragma unroll
    for (int c16 = 0; c16 < CPT / 16; ++c16) {
      uint32_t words[4] = {0u, 0u, 0u, 0u};
      if constexpr (MODE != BQ_GRAM && MODE != BQ_PLAIN) {
        const uint4 w = pre.comp[c16];
        words[0] = w.x; words[1] = w.y; words[2] = w.z; words[3] = w.w;
      }
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const int j = c16 * 16 + jj;
        const int col = colbase + j;
        float val = vals[j];
        if constexpr (MODE == BQ_PLAIN) {
          // nothing to add: the caller's values are the result
        } else if constexpr (MODE == BQ_GRAM) {
          if (has_diag && col == t.row) {
            if (live) a.dout[size_t(t.b) * g.m + t.row] = in_rows ? val : 0.f;
            val = 0.f;
          }
        } else {
          const uint8_t q = uint8_t(words[jj >> 2] >> (8 * (jj & 3)));
          if constexpr (MODE == BQ_POLY) {
            const float v = __fmul_rn(bq_decode<FP8>(q), stile);
            const float dcol = t.diag[c0 + j];
            val = __fmaf_rn(__fadd_rn(drow, dcol), v, val);
            val = __fmaf_rn(v, a.cb, __fmul_rn(val, a.cc));
            if (has_diag && col == t.row) {
              const float dpoly = __fmaf_rn(drow, __fmaf_rn(drow, a.cc, a.cb), a.ca);
              if (live) a.dout[size_t(t.b) * g.m + t.row] = in_rows ? __fadd_rn(val, dpoly) : 0.f;
              val = 0.f;
            }
          } else {
            val = __fmaf_rn(__fmul_rn(bq_decode<FP8>(q), drow), stile, val);
          }
        }
        if (!inside && (!in_rows || col >= g.ln)) val = 0.f;  // padding never contributes to a block scale
        mx = fmaxf(mx, fabsf(val));
        vals[j] = val;
      }
    }

    if constexpr (MODE == BQ_UPDATE_FINAL) {
      if (!live || !in_rows) return;
      const size_t rbase = (size_t(t.b) * g.lm + t.row) * g.ln + colbase;
      const bool wide16 = !a.transpose && a.out_dtype != DT_F32 && (g.ln % 8) == 0 && colbase + CPT <= g.ln &&
                          (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
      if (wide16) {
        // this thread's consecutive 16-bit outputs as 16-byte stores
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + rbase);
#pragma unroll
        for (int c8 = 0; c8 < CPT / 8; ++c8) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = vals[c8 * 8 + 2 * e], hi = vals[c8 * 8 + 2 * e + 1];
            if (a.out_dtype == DT_BF16) {
              w[e] = uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
                     (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
            } else {
              w[e] = uint32_t(__half_as_ushort(__float2half_rn(lo))) |
                     (uint32_t(__half_as_ushort(__float2half_rn(hi))) << 16);
            }
          }
          dst[c8] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        return;
      }
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        const int col = colbase + j;
        if (col < g.ln) {
          size_t idx = a.transpose ? (size_t(t.b) * g.ln + col) * g.lm + t.row : rbase + j;
          store_user(a.out, a.out_dtype, idx, vals[j]);
        }
      }
      return;
    } else {
      mx = warp_max(mx);
      // A warp whose wait ran out publishes a negative value (a maximum is >= 1e-8), so that all
      // eight warps take the same decision: either every warp stores this tile or none does, and
      // every warp walks through the same barriers below whatever it decided.
      if (t.lane == 0) t.red[t.ew] = live ? mx : -1.f;
      named_bar_sync(1, EPI_THREADS);
      bool store = true;
#pragma unroll
      for (int i = 0; i < EPI_WARPS; ++i) {
        const float other = t.red[i];
        store = store && other >= 0.f;
        mx = fmaxf(mx, other);
      }
      const float multiplier = QMAX / mx;
      const float scale = 1.f / multiplier;
      if (store && t.r == 0 && t.half == 0) {
        a.so[(size_t(t.b) * mq + t.tm) * nq + t.tn] = scale;
        if constexpr (!RECT) a.so[(size_t(t.b) * mq + t.tn) * nq + t.tm] = scale;
      }
      uint8_t* out = static_cast<uint8_t*>(a.out);
      const bool diag_tile = !RECT && t.tm == t.tn;
      // transposed target: A^T (update) or the mirrored tile (gram / poly)
      uint8_t* tdst = RECT ? static_cast<uint8_t*>(a.out_t) : out;
      const int trows = RECT ? g.n : g.m;
      const int tld = RECT ? g.m : g.n;
      uint4* dst = reinterpret_cast<uint4*>(out + (size_t(t.b) * g.m + t.row) * g.n + colbase);
      // With a staging tile in shared memory the transposed copy is written there byte by
      // byte (conflict free: a warp's lanes are consecutive rows) and then leaves as
      // coalesced 16-byte stores; without one, each byte goes to global memory directly.
      // A diagonal tile (gram / poly) is its own mirror: its lower half goes to the staging
      // tile at both positions and the whole tile leaves through the same copy-out.
      uint8_t* tsm = t.tsm;
      const bool staged_t = tsm != nullptr;
      const uint32_t tsm_s = tsm ? smem_u32(tsm) + uint32_t(c0 * TSM_PITCH + t.r) : 0u;      // (column, row)
      const uint32_t tsm_own = tsm ? smem_u32(tsm) + uint32_t(t.r * TSM_PITCH + c0) : 0u;    // (row, column)
      if (store)
#pragma unroll
      for (int c16 = 0; c16 < CPT / 16; ++c16) {
        uint32_t w[4];
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          uint32_t word = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = c16 * 16 + k4 * 4 + e;
            const uint32_t qv = bq_quant<FP8>(vals[j], multiplier);
            word |= qv << (8 * e);
            if (staged_t) {
              if (!diag_tile) {
                sts8(tsm_s + uint32_t(j * TSM_PITCH), qv);
              } else if (c0 + j <= t.r) {
                sts8(tsm_s + uint32_t(j * TSM_PITCH), qv);
                sts8(tsm_own + uint32_t(j), qv);
              }
            } else if (!diag_tile) {
              tdst[(size_t(t.b) * trows + (colbase + j)) * tld + t.row] = uint8_t(qv);
            } else if (c0 + j <= t.r) {
              // a diagonal tile stores its lower half and mirrors it
              out[(size_t(t.b) * g.m + t.row) * g.n + colbase + j] = uint8_t(qv);
              out[(size_t(t.b) * g.m + colbase + j) * g.n + t.row] = uint8_t(qv);
            }
          }
          w[k4] = word;
        }
        if (!diag_tile) dst[c16] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (tsm != nullptr) {
        named_bar_sync(1, EPI_THREADS);  // uniform per tile: every epilogue warp takes this branch
        // 128 staged rows of 128 bytes = 1024 chunks of 16 bytes over 256 threads; a staged row
        // is a column of this tile, i.e. a row of the transposed / mirrored tile
        const int tid = t.ew * 32 + t.lane;
        if (store)
#pragma unroll
        for (int i = 0; i < (TILE * TILE / 16) / EPI_THREADS; ++i) {
          const int chunk = tid + i * EPI_THREADS;
          const int trow = chunk >> 3, part = chunk & 7;
          const uint4 v4 = lds128u(smem_u32(tsm) + uint32_t(trow * TSM_PITCH + part * 16));
          *reinterpret_cast<uint4*>(tdst + (size_t(t.b) * trows + (t.col0 + trow)) * tld + t.row0 + part * 16) = v4;
        }
      }
    }
  }
};

}  // namespace i8m
