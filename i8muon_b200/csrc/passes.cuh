// Memory-bound passes around the Newton-Schulz GEMMs: input statistics
// (Frobenius norm + abs-max in one read), normalise / quantise prologues with a
// fused transpose, the symmetric and output re-quantisers of the global-scale
// INT8 path, and the two fused optimizer kernels (momentum, decay + update).
//
// All of them are HBM-bound: one coalesced read of the input, one coalesced
// write of each output, 32x32 or 128x128 shared-memory tiles for the transposed
// copies.  FP32 expressions are written un-fused (the library is also compiled
// with --fmad=false) so that the CPU restatement reproduces them bit for bit.
#pragma once
#include "epi_bq.cuh"

namespace i8m {

template <typename T>
__device__ __forceinline__ float load_f(const T* p, size_t i) { return widen<T>(p[i]); }

__device__ __forceinline__ int8_t quant_rn(float x, float multiplier) {
  return int8_t(max(-127, min(127, __float2int_rn(__fmul_rn(x, multiplier)))));
}

// ------------------------------------------------------------------ stats
// Pass 1: each block reduces STATS_CHUNK elements of one matrix to a partial
// sum of squares and a partial abs-max.  Pass 2: one block per matrix folds the
// partials in a fixed order (deterministic) into norm[b] = sqrt(sum), amax[b].
// Restates src/i8muon/csrc/int8.cu:41-62 plus the torch Frobenius norm of
// src/i8muon/_cutlass.py:190 as one read of the input.
constexpr int STATS_THREADS = 256;
constexpr int STATS_CHUNK = STATS_THREADS * 32;

__device__ __forceinline__ float block_sum_256(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x < 32) {
    r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  __syncthreads();
  return r;  // valid in warp 0
}
__device__ __forceinline__ float block_max_256(float v, float* sh) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x < 32) {
    r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    r = warp_max(r);
  }
  __syncthreads();
  return r;
}

// The partial of one chunk is defined by ONE mapping, shared with the momentum kernel (which computes the
// partials of the update it writes, so that the statistics pass over it disappears): thread t takes the
// elements 8 (t + 256 i) + e of the chunk, i = 0..3 outer, e = 0..7 inner, s = fma(v, v, s) in that order,
// then the block tree.  Same mapping => bit-identical norms whichever kernel produced the partials.
template <typename In>
__global__ void __launch_bounds__(STATS_THREADS)
stats_partial_kernel(const In* x, float* partial_sum, float* partial_max, long long count,
                     int chunks) {
  __shared__ float sh[8];
  const int b = blockIdx.y, chunk = blockIdx.x;
  const In* src = x + size_t(b) * count;
  const long long base = (long long)chunk * STATS_CHUNK;
  float s = 0.f, mx = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const long long idx = base + 8 * (threadIdx.x + STATS_THREADS * i) + e;
      const float v = idx < count ? load_f(src, size_t(idx)) : 0.f;
      s = __fmaf_rn(v, v, s);
      mx = fmaxf(mx, fabsf(v));
    }
  }
  s = block_sum_256(s, sh);
  mx = block_max_256(mx, sh);
  if (threadIdx.x == 0) {
    partial_sum[size_t(b) * chunks + chunk] = s;
    partial_max[size_t(b) * chunks + chunk] = mx;
  }
}

__global__ void __launch_bounds__(STATS_THREADS)
stats_final_kernel(const float* partial_sum, const float* partial_max, float* norm, float* amax,
                   int chunks) {
  __shared__ float sh[8];
  const int b = blockIdx.x;
  float s = 0.f, mx = 0.f;
  for (int i = threadIdx.x; i < chunks; i += STATS_THREADS) {
    s += partial_sum[size_t(b) * chunks + i];
    mx = fmaxf(mx, partial_max[size_t(b) * chunks + i]);
  }
  s = block_sum_256(s, sh);
  mx = block_max_256(mx, sh);
  if (threadIdx.x == 0) {
    if (norm) norm[b] = sqrtf(s);
    if (amax) amax[b] = mx;
  }
}

// One-pass flavour for callers that do not ask for a reproducible summation order
// (``deterministic=False``; the reference's fused path, src/i8muon/csrc/int8.cu:41-62 with
// src/i8muon/_cutlass.py:189-194): every block adds its partial sum of squares to sumsq[b] with an
// atomic, and the block that arrives last for a matrix writes norm[b] = sqrt(sum) and amax[b].
// sumsq / amax_bits / arrived (3 x batch words) must be zero when the kernel starts.
template <typename In>
__global__ void __launch_bounds__(STATS_THREADS)
stats_onepass_kernel(const In* x, float* sumsq, unsigned* amax_bits, unsigned* arrived, float* norm, float* amax,
                     long long count, int chunks) {
  __shared__ float sh[8];
  const int b = blockIdx.y, chunk = blockIdx.x;
  const In* src = x + size_t(b) * count;
  long long base = (long long)chunk * STATS_CHUNK;
  float s = 0.f, mx = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const long long idx = base + 8 * (threadIdx.x + STATS_THREADS * i) + e;
      const float v = idx < count ? load_f(src, size_t(idx)) : 0.f;
      s = __fmaf_rn(v, v, s);
      mx = fmaxf(mx, fabsf(v));
    }
  }
  s = block_sum_256(s, sh);
  mx = block_max_256(mx, sh);
  if (threadIdx.x == 0) {
    atomicAdd(sumsq + b, s);
    atomicMax(amax_bits + b, __float_as_uint(mx));     // non-negative floats order like their bit patterns
    __threadfence();
    if (atomicAdd(arrived + b, 1u) == unsigned(chunks) - 1u) {
      __threadfence();
      if (norm) norm[b] = sqrtf(atomicAdd(sumsq + b, 0.f));
      if (amax) amax[b] = __uint_as_float(atomicMax(amax_bits + b, 0u));
    }
  }
}

// norm[b] <- max(norm[b], eps) / gain: folds an input gain into the dequantisation scale of the
// grouped-cubic route (src/i8muon/_cutlass_cubic.py:38-40).
__global__ void clamp_divide_kernel(float* norm, int batch, float eps, float gain) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch) norm[b] = __fdiv_rn(fmaxf(norm[b], eps), gain);
}

// -------------------------------------------------------------- normalise
// A = E(x * inv), A^T, zero padded to (m x n); restates src/i8muon/csrc/prec.cu:46-68.
// For E = float the value is split into two TF32-representable planes.
template <typename In, typename E>
__global__ void __launch_bounds__(256)
normalize_kernel(const In* x, const float* norm, E* out, E* out_t, float* out_lo, float* out_t_lo,
                 int rows, int cols, int m, int n, int transpose, float eps) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  const float nb = norm ? norm[b] : 1.f;
  const float inv = nb == 0.f ? 0.f : 1.f / fmaxf(nb, eps);
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  // Tiles are taken in the INPUT's orientation so that reads are coalesced.
  // Without transpose A = x; with transpose A^T has the input's orientation.
  const int prow = transpose ? n : m, pcol = transpose ? m : n;
  E* primary = transpose ? out_t : out;
  float* primary_lo = transpose ? out_t_lo : out_lo;
  E* secondary = transpose ? out : out_t;
  float* secondary_lo = transpose ? out_lo : out_t_lo;
  auto put = [](E* dst, float* dst_lo, size_t o, float v) {
    if constexpr (sizeof(E) == 4) {
      const float hi = tf32_hi(v);
      dst[o] = hi;
      dst_lo[o] = tf32_lo(v, hi);
    } else {
      dst[o] = round_to<E>(v);
    }
  };
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = blockIdx.y * 32 + r, col = blockIdx.x * 32 + tx;
    float v = 0.f;
    if (row < rows && col < cols) v = __fmul_rn(load_f(x, (size_t(b) * rows + row) * cols + col), inv);
    tile[r][tx] = v;
    if (primary != nullptr && row < prow && col < pcol) put(primary, primary_lo, (size_t(b) * prow + row) * pcol + col, v);
  }
  __syncthreads();
  if (secondary == nullptr) return;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = blockIdx.x * 32 + r, col = blockIdx.y * 32 + tx;
    if (row < pcol && col < prow) put(secondary, secondary_lo, (size_t(b) * pcol + row) * prow + col, tile[tx][r]);
  }
}

// Vectorised flavours of the two prologues for 16-bit inputs whose rows are a multiple of
// eight elements and 16-byte aligned: every global access is a 16-byte (8-byte for the INT8
// row-major output) coalesced vector, and the transposed copy goes through a shared tile that
// is already stored transposed.  The tile rows are 128 bytes; their 16-byte units are XOR-ed
// with (column / 8) % 8, which spreads the column-wise element stores of a warp over all banks
// and keeps the row-wise 16-byte loads of the copy-out conflict free.  Same arithmetic, same
// results as the scalar kernels above.
__device__ __forceinline__ uint32_t swz16(int c) { return uint32_t((c >> 3) & 7) << 4; }

template <typename In>
__device__ __forceinline__ void unpack8(const uint4 raw, float (&v)[8]) {
  const In* e = reinterpret_cast<const In*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = widen<In>(e[j]);
}
// eight consecutive input elements (16-byte aligned): one vector load for 16-bit types, two for FP32
template <typename In>
__device__ __forceinline__ void load8(const In* p, float (&v)[8]) {
  if constexpr (sizeof(In) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    unpack8<In>(*reinterpret_cast<const uint4*>(p), v);
  }
}

// 64 x 64 tile of the input per block of 256 threads; E is a 16-bit type, In any floating type.
template <typename In, typename E>
__global__ void __launch_bounds__(256)
normalize_vec_kernel(const In* x, const float* norm, E* out, E* out_t, int rows, int cols, int m, int n,
                     int transpose, float eps) {
  __shared__ __align__(16) uint8_t tile_t[64 * 128];   // [input column][input row] of E, swizzled
  const int b = blockIdx.z;
  const float nb = norm ? norm[b] : 1.f;
  const float inv = nb == 0.f ? 0.f : 1.f / fmaxf(nb, eps);
  const int prow = transpose ? n : m, pcol = transpose ? m : n;
  E* primary = transpose ? out_t : out;
  E* secondary = transpose ? out : out_t;
  const int row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int id = int(threadIdx.x) + 256 * i;
    const int r = id >> 3, part = id & 7;
    const int row = row0 + r, col = col0 + part * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (row < rows && col < cols) {
      load8<In>(x + (size_t(b) * rows + row) * cols + col, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], inv);
    }
    alignas(16) E e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = round_to<E>(v[j]);
    if (primary != nullptr && row < prow && col < pcol)
      *reinterpret_cast<uint4*>(primary + (size_t(b) * prow + row) * pcol + col) = *reinterpret_cast<const uint4*>(e);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = part * 8 + j;
      *reinterpret_cast<E*>(tile_t + c * 128 + ((uint32_t(r) * 2u) ^ swz16(c))) = e[j];
    }
  }
  __syncthreads();
  if (secondary == nullptr) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int id = int(threadIdx.x) + 256 * i;
    const int c = id >> 3, p = id & 7;   // transposed row = input column, 16-byte unit = 8 input rows
    const int trow = col0 + c, tcol = row0 + p * 8;
    if (trow < pcol && tcol < prow)
      *reinterpret_cast<uint4*>(secondary + (size_t(b) * pcol + trow) * prow + tcol) =
          *reinterpret_cast<const uint4*>(tile_t + c * 128 + ((uint32_t(p) * 16u) ^ swz16(c)));
  }
}

// One 128 x 128 quantisation block per block of 256 threads; In is a 16-bit type.
template <typename In, bool FP8>
__global__ void __launch_bounds__(256)
bq_quant_vec_kernel(const In* x, const float* norm, uint8_t* out, uint8_t* out_t, float* scale,
                    int rows, int cols, int m, int n, int transpose, float eps) {
  __shared__ float sh[8];
  __shared__ float s_mult;
  __shared__ __align__(16) uint8_t tile_t[128 * 128];   // [input column][input row] bytes, swizzled
  const int tmb = blockIdx.x, tnb = blockIdx.y, b = blockIdx.z;
  const float nb = norm ? norm[b] : 1.f;
  float inv = 1.f / fmaxf(nb, eps);
  if (nb == 0.f) inv = 0.f;
  // the patch in the INPUT's orientation: without transpose its rows are the block's rows
  const int ir0 = transpose ? tnb * 128 : tmb * 128, ic0 = transpose ? tmb * 128 : tnb * 128;
  float vals[8][8];
  float mx = 1e-8f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int id = int(threadIdx.x) + 256 * i;
    const int r = id >> 4, part = id & 15;
    const int ir = ir0 + r, ic = ic0 + part * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
    if (ir < rows && ic < cols) {
      unpack8<In>(*reinterpret_cast<const uint4*>(x + (size_t(b) * rows + ir) * cols + ic), vals[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) vals[i][j] = __fmul_rn(vals[i][j], inv);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(vals[i][j]));
  }
  mx = block_max_256(mx, sh);
  if (threadIdx.x == 0) {
    const float multiplier = (FP8 ? 448.f : 127.f) / mx;
    s_mult = multiplier;
    scale[(size_t(b) * (m / 128) + tmb) * (n / 128) + tnb] = 1.f / multiplier;
  }
  __syncthreads();
  const float multiplier = s_mult;
  uint8_t* same = transpose ? out_t : out;     // shares the input's orientation
  uint8_t* other = transpose ? out : out_t;
  const int sld = transpose ? m : n, srows = transpose ? n : m;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int id = int(threadIdx.x) + 256 * i;
    const int r = id >> 4, part = id & 15;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t q = bq_quant<FP8>(vals[i][j], multiplier);
      w[j >> 2] |= q << (8 * (j & 3));
      const int c = part * 8 + j;
      tile_t[c * 128 + (uint32_t(r) ^ swz16(c))] = uint8_t(q);
    }
    *reinterpret_cast<uint2*>(same + (size_t(b) * srows + ir0 + r) * sld + ic0 + part * 8) = make_uint2(w[0], w[1]);
  }
  __syncthreads();
  const int old = transpose ? n : m, orows = transpose ? m : n;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = int(threadIdx.x) + 256 * i;
    const int c = id >> 3, p = id & 7;   // transposed row = input column, 16 input rows per unit
    *reinterpret_cast<uint4*>(other + (size_t(b) * orows + ic0 + c) * old + ir0 + p * 16) =
        *reinterpret_cast<const uint4*>(tile_t + c * 128 + ((uint32_t(p) * 16u) ^ swz16(c)));
  }
}

// ------------------------------------------------------------ input quant
// Global-scale INT8 quantisation of the input (round half to even), its
// transpose, and a_scale[b] = amax / (127 * max(norm, eps)); restates
// src/i8muon/csrc/int8.cu:64-100.  use_norm == 0 means norm = 1 and eps = 0.
template <typename In>
__global__ void __launch_bounds__(256)
input_quant_kernel(const In* x, const float* amax, const float* norm, int8_t* out, int8_t* out_t,
                   float* scale, int rows, int cols, int m, int n, int transpose, float eps) {
  __shared__ int8_t tile[32][33];
  const int b = blockIdx.z;
  const float mx = amax[b];
  const float nb = norm ? norm[b] : 1.f;
  const float multiplier = mx > 0.f ? 127.f / mx : 0.f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
    scale[b] = mx > 0.f ? mx / __fmul_rn(127.f, fmaxf(nb, eps)) : 0.f;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  // Tile origin in the INPUT: rows blockIdx.y*32, cols blockIdx.x*32.
  // Without transpose A = x (m x n padded); with transpose A^T has the input's
  // layout (n x m padded) and A is written through the shared tile.
  const int prow = transpose ? n : m, pcol = transpose ? m : n;
  int8_t* primary = transpose ? out_t : out;
  int8_t* secondary = transpose ? out : out_t;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = blockIdx.y * 32 + r, col = blockIdx.x * 32 + tx;
    int8_t q = 0;
    if (row < rows && col < cols) q = quant_rn(load_f(x, (size_t(b) * rows + row) * cols + col), multiplier);
    tile[r][tx] = q;
    if (row < prow && col < pcol) primary[(size_t(b) * prow + row) * pcol + col] = q;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = blockIdx.x * 32 + r, col = blockIdx.y * 32 + tx;
    if (row < pcol && col < prow) secondary[(size_t(b) * pcol + row) * prow + col] = tile[tx][r];
  }
}

// -------------------------------------------------------- symmetric quant
// Reads the lower-triangular 32x32 tiles of the int32 Gram (QUAD = false) or of
// the FP32 polynomial (QUAD = true), quantises with the global scale and a
// zeroed diagonal, mirrors to a full symmetric int8 matrix, and writes the FP32
// diagonal and the new scale; restates src/i8muon/csrc/int8.cu:363-420.
template <typename In, bool QUAD>
__global__ void __launch_bounds__(256)
symmetric_quant_kernel(const In* input, const void* maximum, const float* orig_scale,
                       const float* orig_diag, int8_t* output, float* scale, float* diag, int m,
                       float c0, float c1, float c2) {
  __shared__ int8_t tile[32][33];
  const int b = blockIdx.y, pid = blockIdx.x;
  int tm = int((sqrtf(float(8 * pid + 1)) - 1.f) * 0.5f);
  while ((tm + 1) * (tm + 2) / 2 <= pid) ++tm;
  while (tm * (tm + 1) / 2 > pid) --tm;
  const int tn = pid - tm * (tm + 1) / 2;
  float mx;
  if constexpr (QUAD) mx = static_cast<const float*>(maximum)[b];
  else mx = float(static_cast<const int*>(maximum)[b]);
  const float multiplier = mx > 0.f ? 127.f / mx : 0.f;
  const float os = orig_scale[b];
  const float sa = QUAD ? 1.f : __fmul_rn(os, os);
  if (pid == 0 && threadIdx.x == 0) scale[b] = mx > 0.f ? sa / multiplier : 0.f;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = tm * 32 + r, col = tn * 32 + tx;
    float v = (row < m && col < m) ? float(input[(size_t(b) * m + row) * m + col]) : 0.f;
    int8_t q = (row == col) ? int8_t(0) : quant_rn(v, multiplier);
    if (row == col && row < m) {
      if constexpr (QUAD) {
        const float d = orig_diag[size_t(b) * m + row];
        // the reference's binary (--fmad=true) fuses both products of v + (c2*d + c1)*d + c0
        diag[size_t(b) * m + row] = __fadd_rn(__fmaf_rn(__fmaf_rn(c2, d, c1), d, v), c0);
      } else {
        // c0 shifts the Gram diagonal (completed-square rows, int8.cu:396); it is 0 otherwise
        diag[size_t(b) * m + row] = __fmaf_rn(v, sa, c0);
      }
    }
    tile[r][tx] = q;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    int row = tm * 32 + r, col = tn * 32 + tx;
    if (row < m && col < m) {
      // a diagonal tile takes its upper half from the mirrored lower half
      int8_t q = (tm == tn && r < tx) ? tile[tx][r] : tile[r][tx];
      output[(size_t(b) * m + row) * m + col] = q;
    }
    if (tm != tn) {
      row = tn * 32 + r; col = tm * 32 + tx;
      if (row < m && col < m) output[(size_t(b) * m + row) * m + col] = tile[tx][r];
    }
  }
}

// ------------------------------------------- 128 x 128 tiles of int8 codes
// The two re-quantisers below work on 128 x 128 tiles when the matrix extents are multiples of
// 128: 16-byte loads of the FP32 / int32 input, the codes of a row chunk packed into one word per
// lane (128 contiguous bytes per warp store), and the transposed tile written as 16-byte stores
// after 4 x 4 byte transposes in registers.  Same roundings as the 32 x 32 kernels.
constexpr int QT_PITCH = 33;   // words per row of the staged tile of codes

__device__ __forceinline__ uint32_t quant4_rn(float4 v, float multiplier) {
  const uint32_t a = uint8_t(quant_rn(v.x, multiplier)), b = uint8_t(quant_rn(v.y, multiplier));
  const uint32_t c = uint8_t(quant_rn(v.z, multiplier)), d = uint8_t(quant_rn(v.w, multiplier));
  return a | (b << 8) | (c << 16) | (d << 24);
}
__device__ __forceinline__ float4 load4f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4f(const int* p) {
  const int4 v = *reinterpret_cast<const int4*>(p);
  return make_float4(float(v.x), float(v.y), float(v.z), float(v.w));
}
// 4 x 4 byte transpose: w[k] = four consecutive bytes of row k; t[j] = byte j of rows 0..3.
__device__ __forceinline__ void transpose4x4(const uint32_t (&w)[4], uint32_t (&t)[4]) {
  const uint32_t x0 = __byte_perm(w[0], w[1], 0x5140), x1 = __byte_perm(w[2], w[3], 0x5140);
  const uint32_t x2 = __byte_perm(w[0], w[1], 0x7362), x3 = __byte_perm(w[2], w[3], 0x7362);
  t[0] = __byte_perm(x0, x1, 0x5410); t[1] = __byte_perm(x0, x1, 0x7632);
  t[2] = __byte_perm(x2, x3, 0x5410); t[3] = __byte_perm(x2, x3, 0x7632);
}
// This thread's 16 rows x 4 columns of the staged tile, transposed: tr[j][g] = bytes of column
// 4 cb + j at rows r0 + 4 g .. r0 + 4 g + 3.  Thread layout of a 256-thread block: warp w covers
// rows 32 (w >> 1) .. + 31 and word columns 16 (w & 1) .. + 15; lane: rows + 16 (lane >> 4), word
// column + (lane & 15).  Shared-memory reads are free of bank conflicts at a pitch of 33 words.
__device__ __forceinline__ void tile_block_transposed(const uint32_t* tile, int r0, int cb, uint32_t (&tr)[4][4]) {
#pragma unroll
  for (int gq = 0; gq < 4; ++gq) {
    uint32_t w[4], t4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = tile[(r0 + 4 * gq + k) * QT_PITCH + cb];
    transpose4x4(w, t4);
#pragma unroll
    for (int j = 0; j < 4; ++j) tr[j][gq] = t4[j];
  }
}

template <typename In>
__device__ __forceinline__ float4 load4any(const In* p) {
  if constexpr (sizeof(In) == 4) {
    return load4f(p);
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const In* e = reinterpret_cast<const In*>(&raw);
    return make_float4(widen<In>(e[0]), widen<In>(e[1]), widen<In>(e[2]), widen<In>(e[3]));
  }
}

// Global-scale quantisation of an unpadded input whose extents are multiples of 128 (the tiles
// are taken in the input's orientation; `same` has that orientation, `other` is its transpose).
template <typename In>
__global__ void __launch_bounds__(256)
input_quant128_kernel(const In* x, const float* amax, const float* norm, int8_t* same, int8_t* other, float* scale,
                      int rows, int cols, float eps) {
  __shared__ uint32_t tile[128 * QT_PITCH];
  const int b = blockIdx.z;
  const float mx = amax[b];
  const float nb = norm ? norm[b] : 1.f;
  const float multiplier = mx > 0.f ? 127.f / mx : 0.f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
    scale[b] = mx > 0.f ? mx / __fmul_rn(127.f, fmaxf(nb, eps)) : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.y * 128, col0 = blockIdx.x * 128;
  const In* src = x + (size_t(b) * rows + row0) * cols + col0 + 4 * lane;
  uint32_t* dst = reinterpret_cast<uint32_t*>(same + (size_t(b) * rows + row0) * cols + col0) + lane;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = warp * 16 + i;
    const uint32_t q = quant4_rn(load4any<In>(src + size_t(r) * cols), multiplier);
    dst[size_t(r) * (cols / 4)] = q;
    tile[r * QT_PITCH + lane] = q;
  }
  __syncthreads();
  const int r0 = 32 * (warp >> 1) + 16 * (lane >> 4), cb = 16 * (warp & 1) + (lane & 15);
  uint32_t tr[4][4];
  tile_block_transposed(tile, r0, cb, tr);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(other + (size_t(b) * cols + col0 + 4 * cb + j) * rows + row0 + r0) =
        make_uint4(tr[j][0], tr[j][1], tr[j][2], tr[j][3]);
}

// FP32 (m x n) -> int8 and transposed int8, m and n multiples of 128, 16-byte aligned pointers.
__global__ void __launch_bounds__(256)
output_quant128_kernel(const float* input, const float* maximum, int8_t* out, int8_t* out_t, float* scale, int m,
                       int n) {
  __shared__ uint32_t tile[128 * QT_PITCH];
  const int b = blockIdx.z;
  const float mx = maximum[b];
  const float multiplier = mx > 0.f ? 127.f / mx : 0.f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) scale[b] = mx > 0.f ? 1.f / multiplier : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.y * 128, col0 = blockIdx.x * 128;
  const float* src = input + (size_t(b) * m + row0) * n + col0 + 4 * lane;
  uint32_t* dst = reinterpret_cast<uint32_t*>(out + (size_t(b) * m + row0) * n + col0) + lane;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = warp * 16 + i;
    const uint32_t q = quant4_rn(load4f(src + size_t(r) * n), multiplier);
    dst[size_t(r) * (n / 4)] = q;
    tile[r * QT_PITCH + lane] = q;
  }
  __syncthreads();
  const int r0 = 32 * (warp >> 1) + 16 * (lane >> 4), cb = 16 * (warp & 1) + (lane & 15);
  uint32_t tr[4][4];
  tile_block_transposed(tile, r0, cb, tr);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(out_t + (size_t(b) * n + col0 + 4 * cb + j) * m + row0 + r0) =
        make_uint4(tr[j][0], tr[j][1], tr[j][2], tr[j][3]);
}

// Lower 128 x 128 tiles of the int32 Gram / FP32 polynomial -> full symmetric int8 matrix with a
// zero diagonal, the FP32 diagonal and the scale; m a multiple of 128.
template <typename In, bool QUAD>
__global__ void __launch_bounds__(256)
symmetric_quant128_kernel(const In* input, const void* maximum, const float* orig_scale, const float* orig_diag,
                          int8_t* output, float* scale, float* diag, int m, float c0, float c1, float c2) {
  __shared__ uint32_t tile[128 * QT_PITCH];
  const int b = blockIdx.y, pid = blockIdx.x;
  int tm = int((sqrtf(float(8 * pid + 1)) - 1.f) * 0.5f);
  while ((tm + 1) * (tm + 2) / 2 <= pid) ++tm;
  while (tm * (tm + 1) / 2 > pid) --tm;
  const int tn = pid - tm * (tm + 1) / 2;
  float mx;
  if constexpr (QUAD) mx = static_cast<const float*>(maximum)[b];
  else mx = float(static_cast<const int*>(maximum)[b]);
  const float multiplier = mx > 0.f ? 127.f / mx : 0.f;
  const float os = orig_scale[b];
  const float sa = QUAD ? 1.f : __fmul_rn(os, os);
  if (pid == 0 && threadIdx.x == 0) scale[b] = mx > 0.f ? sa / multiplier : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = tm * 128, col0 = tn * 128;
  const bool diagonal = tm == tn;
  const In* src = input + (size_t(b) * m + row0) * m + col0 + 4 * lane;
  uint32_t* dst = reinterpret_cast<uint32_t*>(output + (size_t(b) * m + row0) * m + col0) + lane;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int r = warp * 16 + i;
    const float4 v = load4f(src + size_t(r) * m);
    uint32_t q = quant4_rn(v, multiplier);
    if (diagonal) {
      const int k = r - 4 * lane;   // position of the diagonal element inside this lane's four columns
      if (k >= 0 && k < 4) {
        q &= ~(0xffu << (8 * k));
        const float dv = k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w));
        const size_t di = size_t(b) * m + row0 + r;
        if constexpr (QUAD) {
          const float d = orig_diag[di];
          diag[di] = __fadd_rn(__fmaf_rn(__fmaf_rn(c2, d, c1), d, dv), c0);
        } else {
          diag[di] = __fmaf_rn(dv, sa, c0);
        }
      }
    } else {
      dst[size_t(r) * (m / 4)] = q;
    }
    tile[r * QT_PITCH + lane] = q;
  }
  __syncthreads();
  const int r0 = 32 * (warp >> 1) + 16 * (lane >> 4), cb = 16 * (warp & 1) + (lane & 15);
  uint32_t tr[4][4];
  tile_block_transposed(tile, r0, cb, tr);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int orow = 4 * cb + j;       // row of the transposed tile, columns r0 .. r0 + 15
    if (diagonal) {
      // lower half (column <= row) from the tile itself, upper half from its transpose
#pragma unroll
      for (int gq = 0; gq < 4; ++gq) {
        const int d = orow - (r0 + 4 * gq);
        const uint32_t keep = d >= 3 ? 0xffffffffu : (d < 0 ? 0u : (1u << (8 * (d + 1))) - 1u);
        const uint32_t own = tile[orow * QT_PITCH + (r0 >> 2) + gq];
        tr[j][gq] = (own & keep) | (tr[j][gq] & ~keep);
      }
    }
    *reinterpret_cast<uint4*>(output + (size_t(b) * m + col0 + orow) * m + row0 + r0) =
        make_uint4(tr[j][0], tr[j][1], tr[j][2], tr[j][3]);
  }
}

// R[i][i] <- E(R[i][i] + shift) on every matrix of the batch: the diagonal shift of a
// completed-square row in the floating first iteration (src/i8muon/_cutlass_prec.py:97-99).
template <typename E>
__global__ void __launch_bounds__(256)
diag_add_kernel(E* r, int batch, int m, int logical, float shift) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)batch * logical) return;
  const int b = int(i / logical), d = int(i - (long long)b * logical);
  E* e = r + (size_t(b) * m + d) * m + d;
  *e = round_to<E>(__fadd_rn(widen<E>(*e), shift));
}

// ----------------------------------------------------------- output quant
// FP32 (m x n) -> int8 and transposed int8 with the global scale 1/(127/max);
// restates src/i8muon/csrc/int8.cu:422-450.
__global__ void __launch_bounds__(256)
output_quant_kernel(const float* input, const float* maximum, int8_t* out, int8_t* out_t,
                    float* scale, int m, int n) {
  __shared__ int8_t tile[32][33];
  const int b = blockIdx.z;
  const float mx = maximum[b];
  const float multiplier = mx > 0.f ? 127.f / mx : 0.f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
    scale[b] = mx > 0.f ? 1.f / multiplier : 0.f;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = blockIdx.y * 32 + r, col = blockIdx.x * 32 + tx;
    int8_t q = 0;
    if (row < m && col < n) {
      q = quant_rn(input[(size_t(b) * m + row) * n + col], multiplier);
      out[(size_t(b) * m + row) * n + col] = q;
    }
    tile[r][tx] = q;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = ty + j;
    const int row = blockIdx.x * 32 + r, col = blockIdx.y * 32 + tx;
    if (row < n && col < m) out_t[(size_t(b) * n + row) * m + col] = tile[tx][r];
  }
}

// --------------------------------------------------------------- BQ quant
// Per-128x128-block quantisation of x * inv: block max (floor 1e-8) -> scale,
// INT8 truncating or E4M3 round-to-nearest-even saturating; writes A, A^T and
// the scale grid; restates src/i8muon/csrc/bq.cu:60-101.
// A 128x128 block is processed as sixteen 32x32 sub-tiles by 256 threads.
template <typename In, bool FP8>
__global__ void __launch_bounds__(256)
bq_quant_kernel(const In* x, const float* norm, uint8_t* out, uint8_t* out_t, float* scale,
                int rows, int cols, int m, int n, int transpose, float eps) {
  __shared__ float sh[8];
  __shared__ uint8_t qt[128][132];
  const int tmb = blockIdx.x, tnb = blockIdx.y, b = blockIdx.z;
  const float nb = norm ? norm[b] : 1.f;
  float inv = 1.f / fmaxf(nb, eps);
  if (nb == 0.f) inv = 0.f;
  // Thread layout chosen for coalesced INPUT reads: without transpose the block
  // rows are input rows; with transpose the block rows are input columns.
  float vals[64];
  float mx = 1e-8f;
  const int tx = threadIdx.x & 127, ty = threadIdx.x >> 7;  // 128 x 2
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    // element (p, tx) of the 128x128 patch in INPUT orientation
    const int p = ty + 2 * i;
    int ir, ic;
    if (!transpose) { ir = tmb * 128 + p; ic = tnb * 128 + tx; }
    else { ir = tnb * 128 + p; ic = tmb * 128 + tx; }
    float v = (ir < rows && ic < cols) ? __fmul_rn(load_f(x, (size_t(b) * rows + ir) * cols + ic), inv) : 0.f;
    vals[i] = v;
    mx = fmaxf(mx, fabsf(v));
  }
  mx = block_max_256(mx, sh);
  __shared__ float s_mult;
  if (threadIdx.x == 0) {
    const float multiplier = (FP8 ? 448.f : 127.f) / mx;
    s_mult = multiplier;
    scale[(size_t(b) * (m / 128) + tmb) * (n / 128) + tnb] = 1.f / multiplier;
  }
  __syncthreads();
  const float multiplier = s_mult;
  // The matrix that shares the input's orientation is written directly.
  uint8_t* same = transpose ? out_t : out;     // rows = input rows
  uint8_t* other = transpose ? out : out_t;
  const int srow0 = transpose ? tnb * 128 : tmb * 128, scol0 = transpose ? tmb * 128 : tnb * 128;
  const int sld = transpose ? m : n;
  const int srows = transpose ? n : m;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    const int p = ty + 2 * i;
    uint8_t q = bq_quant<FP8>(vals[i], multiplier);
    qt[p][tx] = q;
    same[(size_t(b) * srows + srow0 + p) * sld + scol0 + tx] = q;
  }
  __syncthreads();
  const int old = transpose ? n : m;
  const int orows = transpose ? m : n;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    const int p = ty + 2 * i;  // row of the transposed patch
    other[(size_t(b) * orows + scol0 + p) * old + srow0 + tx] = qt[tx][p];
  }
}

// ----------------------------------------------------- optimizer kernels
// Up to MT_MAX same-shaped tensors per launch; pointers travel as kernel
// arguments so that no device-side pointer table (and no host-to-device copy)
// is needed and the launch can be captured in a CUDA graph.
constexpr int MT_MAX = 32;
struct MomentumTable {
  const void* grad[MT_MAX];
  void* buf[MT_MAX];
};
struct ApplyTable {
  void* param[MT_MAX];
};

__device__ __forceinline__ float lerp_f(float start, float end, float w) {
  // torch.lerp: two-sided formula selected by |w| < 0.5
  const float d = end - start;
  return fabsf(w) < 0.5f ? __fmaf_rn(w, d, start) : __fmaf_rn(-d, 1.f - w, end);
}

// buf <- lerp(buf, g, 1 - mu2) (rounded to the buffer's dtype), then
// u = nesterov ? lerp(g, buf, mu) : buf, written to the stacked update tensor
// (count x numel) in the gradient's dtype; restates src/i8muon/_optimizer.py:472-474.
template <typename T>
__global__ void __launch_bounds__(256)
momentum_kernel(MomentumTable tab, T* update, long long numel, float w_buf, float mu,
                int nesterov, float* partial_sum, float* partial_max, int chunks, int first_tensor) {
  __shared__ float sh[8];
  const int t = blockIdx.y;
  const T* g = static_cast<const T*>(tab.grad[t]);
  T* buf = static_cast<T*>(tab.buf[t]);
  T* u = update + size_t(t) * numel;
  constexpr int VEC = 16 / int(sizeof(T));       // elements per 16-byte vector: 8 (16-bit) or 4 (FP32)
  constexpr int PER8 = 8 / VEC;                   // vectors per group of eight elements
  const bool aligned = ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(buf) |
                         reinterpret_cast<uintptr_t>(u)) & 15u) == 0;
  // One chunk of STATS_CHUNK elements at a time, in the element order of stats_partial_kernel, so that the
  // partial sums of squares and maxima of the update written here are the ones that kernel would compute.
  for (int chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    const long long base = (long long)chunk * STATS_CHUNK;
    float s = 0.f, mx = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long e0 = base + 8 * (threadIdx.x + STATS_THREADS * i);   // first of this thread's eight elements
      if (aligned && e0 + 8 <= numel) {
#pragma unroll
        for (int v = 0; v < PER8; ++v) {
          const long long vi = e0 / VEC + v;
          uint4 gv = reinterpret_cast<const uint4*>(g)[vi];
          uint4 bv = reinterpret_cast<uint4*>(buf)[vi];
          uint4 uv;
          const T* ge = reinterpret_cast<const T*>(&gv);
          T* be = reinterpret_cast<T*>(&bv);
          T* ue = reinterpret_cast<T*>(&uv);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float gf = widen<T>(ge[e]);
            const T nb = round_to<T>(lerp_f(widen<T>(be[e]), gf, w_buf));
            be[e] = nb;
            ue[e] = nesterov ? round_to<T>(lerp_f(gf, widen<T>(nb), mu)) : nb;
            const float uf = widen<T>(ue[e]);
            s = __fmaf_rn(uf, uf, s);
            mx = fmaxf(mx, fabsf(uf));
          }
          reinterpret_cast<uint4*>(buf)[vi] = bv;
          reinterpret_cast<uint4*>(u)[vi] = uv;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const long long idx = e0 + e;
          if (idx < numel) {
            const float gf = widen<T>(g[idx]);
            const T nb = round_to<T>(lerp_f(widen<T>(buf[idx]), gf, w_buf));
            buf[idx] = nb;
            const T un = nesterov ? round_to<T>(lerp_f(gf, widen<T>(nb), mu)) : nb;
            u[idx] = un;
            const float uf = widen<T>(un);
            s = __fmaf_rn(uf, uf, s);
            mx = fmaxf(mx, fabsf(uf));
          }
        }
      }
    }
    if (partial_sum) {   // uniform per launch
      s = block_sum_256(s, sh);
      mx = block_max_256(mx, sh);
      if (threadIdx.x == 0) {
        partial_sum[size_t(first_tensor + t) * chunks + chunk] = s;
        partial_max[size_t(first_tensor + t) * chunks + chunk] = mx;
      }
    }
  }
}

// decay_mode 0: none; 1: param *= decay (then rounded) ; 2: update += wd * param
// (rounded to the update dtype).  Then param += (-lr) * update.  Restates
// src/i8muon/_optimizer.py:503-511 including its intermediate roundings.
template <typename P, typename U>
__global__ void __launch_bounds__(256)
apply_kernel(ApplyTable tab, const U* update, long long numel, int decay_mode, float decay,
             float neg_lr) {
  const int t = blockIdx.y;
  P* p = static_cast<P*>(tab.param[t]);
  const U* u = update + size_t(t) * numel;
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int VEC = 8;
  const long long nvec = numel / VEC;
  const bool aligned = ((reinterpret_cast<uintptr_t>(p) % (VEC * sizeof(P))) == 0) &&
                       ((reinterpret_cast<uintptr_t>(u) % (VEC * sizeof(U))) == 0);
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  auto one = [&](float pf, float uf) -> float {
    if (decay_mode == 1) pf = widen<P>(round_to<P>(__fmul_rn(pf, decay)));
    else if (decay_mode == 2) uf = widen<U>(round_to<U>(__fmaf_rn(decay, pf, uf)));
    return __fmaf_rn(neg_lr, uf, pf);
  };
  if (aligned) {
    struct alignas(VEC * sizeof(P)) PV { P e[VEC]; };
    struct alignas(VEC * sizeof(U)) UV { U e[VEC]; };
    for (; i < nvec; i += stride) {
      PV pv = reinterpret_cast<PV*>(p)[i];
      const UV uv = reinterpret_cast<const UV*>(u)[i];
#pragma unroll
      for (int e = 0; e < VEC; ++e) pv.e[e] = round_to<P>(one(widen<P>(pv.e[e]), widen<U>(uv.e[e])));
      reinterpret_cast<PV*>(p)[i] = pv;
    }
    i = nvec * VEC + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  }
  for (; i < numel; i += stride) p[i] = round_to<P>(one(widen<P>(p[i]), widen<U>(u[i])));
}

// ----------------------------------------------------------------- AdamW
// Multi-tensor AdamW for the parameters Muon does not take (embeddings, heads, vectors):
// up to ADAM_MAX tensors of different sizes per launch, FP32 moments, decoupled decay.
// Per element, in this order (the statements of torch.optim.AdamW's single-tensor path):
//   p  = p * (1 - lr * wd)
//   m  = lerp(m, g, 1 - beta1);   v = beta2 * v + (1 - beta2) * g * g
//   p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps)
constexpr int ADAM_MAX = 24;
struct AdamTable {
  void* param[ADAM_MAX];
  const void* grad[ADAM_MAX];
  float* exp_avg[ADAM_MAX];
  float* exp_avg_sq[ADAM_MAX];
  long long numel[ADAM_MAX];
};

template <typename P, typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(AdamTable tab, float decay, float beta1, float beta2, float eps, float step_size,
             float inv_bc2_sqrt) {
  const int t = blockIdx.y;
  P* p = static_cast<P*>(tab.param[t]);
  const G* g = static_cast<const G*>(tab.grad[t]);
  float* m = tab.exp_avg[t];
  float* v = tab.exp_avg_sq[t];
  const long long n = tab.numel[t];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gf = widen<G>(g[i]);
    float pf = __fmul_rn(widen<P>(p[i]), decay);
    const float mf = lerp_f(m[i], gf, 1.f - beta1);
    const float vf = __fmaf_rn(__fmul_rn(gf, gf), 1.f - beta2, __fmul_rn(v[i], beta2));
    m[i] = mf;
    v[i] = vf;
    const float denom = __fadd_rn(__fmul_rn(sqrtf(vf), inv_bc2_sqrt), eps);
    pf = __fmaf_rn(-step_size, __fdiv_rn(mf, denom), pf);
    p[i] = round_to<P>(pf);
  }
}

}  // namespace i8m
