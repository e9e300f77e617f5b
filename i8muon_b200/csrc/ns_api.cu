// Host side of the C ABI: argument checks, TMA descriptor encoding, kernel
// launches, and the C++ drivers that sequence one whole Newton-Schulz call out
// of the stage kernels.  No device memory is allocated here; the caller's
// workspace is carved up by a bump allocator.
#include "../../include/i8muon_b200.h"
#include "epi_bq.cuh"
#include "epi_float.cuh"
#include "epi_float_bq.cuh"
#include "epi_int8.cuh"
#include "gemm_bq_persistent.cuh"
#include "gemm_bq_split.cuh"
#include "gemm_wholek_persistent.cuh"
#include "gemm_wholek_wide.cuh"
#include "passes.cuh"

#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

using namespace i8m;

namespace {

thread_local char g_error[512] = "";
// Kernel selection is per calling thread: two engines on two threads (or two devices driven
// from two threads) never see each other's choice.  i8m_ns_run additionally takes the
// selection as an argument and restores the thread's own setting when it returns.
thread_local int g_debug_simt = 0;
thread_local int g_starve_producers = 0;   // test hook: see bq_produce
thread_local float* g_final_amax = nullptr;  // set by run_float around its final product: [batch] maximum of the stored result
constexpr int WHOLEK_VARIANTS = 3;
thread_local int g_wholek_variant = 0;   // "wholek_gemm": 0 units of 128 x 256, 1 two streams of 128 x 128 tiles, 2 one CTA per tile
// block-quantised GEMMs: 0 = split kernel (tail on its own warps, four-stage ring), 1 = fused tail with a
// six-stage ring, 2 = fused tail with a four-stage ring; the host-side tuner chooses per shape
thread_local int g_cta_limit = 0;   // persistent GEMM kernels launch at most this many CTAs (0: one per SM)
thread_local int g_bq_variant = 0;
constexpr int BQ_VARIANTS = 3;
std::atomic<unsigned long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}
#define CUDA_TRY(expr)                                                              \
  do {                                                                              \
    cudaError_t e_ = (expr);                                                        \
    if (e_ != cudaSuccess)                                                          \
      return fail(I8M_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));      \
  } while (0)
#define LAUNCH_CHECK(name)                                                          \
  do {                                                                              \
    cudaError_t e_ = cudaGetLastError();                                            \
    if (e_ != cudaSuccess)                                                          \
      return fail(I8M_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e_)); \
    g_launches.fetch_add(1, std::memory_order_relaxed);                             \
  } while (0)

inline cudaStream_t S(i8m_stream_t s) { return static_cast<cudaStream_t>(s); }
inline int cdiv(long long a, long long b) { return int((a + b - 1) / b); }
inline int pad_to(int v, int a) { return (v + a - 1) / a * a; }
inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// ------------------------------------------------------- tensor map encode
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_encode_once;

int load_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeFn>(fn);
  });
  return g_encode ? 0 : fail(I8M_E_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
}

// 3-D map {k, rows, batch} over a (batch, rows, k) row-major operand; the box
// is {128 bytes of K, 128 rows, 1}; rows or K beyond the tensor read as zero.
int make_operand_map(CUtensorMap* map, const void* ptr, int esize, int k, int rows, int batch) {
  if (int rc = load_encode()) return rc;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0)
    return fail(I8M_E_ARGUMENT, "GEMM operand is not 16-byte aligned");
  if ((size_t(k) * esize) % 16 != 0)
    return fail(I8M_E_ARGUMENT, "GEMM operand row pitch (%d x %d bytes) is not a multiple of 16", k, esize);
  CUtensorMapDataType dt = esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                         : esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                      : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  cuuint64_t dims[3] = {cuuint64_t(k), cuuint64_t(rows), cuuint64_t(batch)};
  cuuint64_t strides[2] = {cuuint64_t(k) * esize, cuuint64_t(k) * esize * rows};
  cuuint32_t box[3] = {cuuint32_t(128 / esize), 128u, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = g_encode(map, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(I8M_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", int(r));
  return 0;
}

// ------------------------------------------------------------ GEMM launch
int sm_count();

// Row blocks per group of the wide-unit order: as many as keep the group's left row blocks
// (128 rows x k bytes each) within 32 MB of L2; even, 8 to 64.
int wide_group(long long k_bytes) {
  const long long fit = (32LL << 20) / std::max<long long>(1, 128 * k_bytes);
  return int(std::min<long long>(64, std::max<long long>(8, fit))) & ~1;
}

template <class Epi>
int launch_gemm(const void* a, const void* a_lo, const void* bt, const void* bt_lo, int batch,
                int m, int n, int k, int lm, int ln, int sym, unsigned* status,
                const typename Epi::Args& args, cudaStream_t stream, const char* name) {
  if (batch < 1 || m < 1 || n < 1 || k < 1) return fail(I8M_E_ARGUMENT, "%s: empty problem", name);
  if (!a || !bt || !status) return fail(I8M_E_ARGUMENT, "%s: null operand or status pointer", name);
  if (sym && m != n) return fail(I8M_E_ARGUMENT, "%s: symmetric product needs m == n", name);
  constexpr int ES = int(sizeof(typename Epi::Elem));
  constexpr int STAGE_BYTES = 2 * Epi::PARTS * TILE_BYTES;
  constexpr size_t SMEM = size_t(Epi::STAGES) * STAGE_BYTES + sizeof(Ctrl) + 1024;
  GemmGeom g;
  g.batch = batch; g.m = m; g.n = n; g.k = k; g.lm = lm; g.ln = ln;
  g.tiles_m = cdiv(m, TILE); g.tiles_n = cdiv(n, TILE);
  g.sym = sym;
  g.tiles_per_batch = sym ? g.tiles_m * (g.tiles_m + 1) / 2 : g.tiles_m * g.tiles_n;
  g.num_kb = cdiv((long long)k * ES, 128);
  g.debug_simt = g_debug_simt | (g_starve_producers ? 0x100 : 0);
  g.group = wide_group((long long)k * ES);
  g.a_raw = a; g.b_raw = bt; g.status = status;
  long long blocks = (long long)g.tiles_per_batch * batch;
  if (blocks > 0x7fffffffLL) return fail(I8M_E_LIMIT, "%s: too many tiles", name);
  CUtensorMap ma, mb, ma2, mb2;
  if (int rc = make_operand_map(&ma, a, ES, k, m, batch)) return rc;
  if (int rc = make_operand_map(&mb, bt, ES, k, n, batch)) return rc;
  if (Epi::PARTS == 2) {
    if (!a_lo || !bt_lo) return fail(I8M_E_ARGUMENT, "%s: missing low planes", name);
    if (int rc = make_operand_map(&ma2, a_lo, ES, k, m, batch)) return rc;
    if (int rc = make_operand_map(&mb2, bt_lo, ES, k, n, batch)) return rc;
  } else {
    ma2 = ma; mb2 = mb;
  }
  // products that accumulate their whole K extent in tensor memory: persistent kernel
  if constexpr (!Epi::BLOCKQ && Epi::PARTS == 1 && Epi::PROMOTE_KB == 0) {
    if (!g_debug_simt && g_wholek_variant == 0) {
      constexpr size_t WSMEM = wholek_wide_smem_bytes<Epi>();
      auto wk = wholek_wide_kernel<Epi>;
      CUDA_TRY(cudaFuncSetAttribute(wk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(WSMEM)));
      const long long units = (long long)wide_units_per_batch(g.tiles_m, g.tiles_n, sym) * batch;
      wk<<<unsigned(std::min<long long>(units, sm_count())), WKW_THREADS, WSMEM, stream>>>(ma, mb, g, args);
      LAUNCH_CHECK(name);
      return 0;
    }
    if (!g_debug_simt && g_wholek_variant == 1) {
      constexpr size_t PSMEM = size_t(WKP_STAGES) * 2 * TILE_BYTES + sizeof(Ctrl) + 1024;
      auto pk = wholek_persistent_kernel<Epi>;
      CUDA_TRY(cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PSMEM)));
      const unsigned grid = unsigned(std::min<long long>(blocks, sm_count()));
      pk<<<grid, WKP_THREADS, PSMEM, stream>>>(ma, mb, g, args);
      LAUNCH_CHECK(name);
      return 0;
    }
  }
  auto kernel = ns_gemm_kernel<Epi, true>;
  if constexpr (!Epi::BLOCKQ) {
    if (!g_debug_simt) kernel = ns_gemm_kernel<Epi, false>;
  }
  CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
  kernel<<<dim3(unsigned(blocks)), WarpLayout<Epi>::THREADS, SMEM, stream>>>(ma, mb, ma2, mb2, g, args);
  LAUNCH_CHECK(name);
  return 0;
}

// Block-quantised GEMMs: persistent kernel, one CTA per SM (the debug core keeps the
// one-tile-per-CTA skeleton).
int sm_count() {
  static int counts[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (counts[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    counts[device] = n;
  }
  return g_cta_limit > 0 ? std::min(counts[device], g_cta_limit) : counts[device];
}

template <class Epi>
int launch_bq(const void* a, const void* bt, int batch, int m, int n, int k, int lm, int ln, int sym,
              unsigned* status, const typename Epi::Args& args, cudaStream_t stream, const char* name) {
  if (g_debug_simt)
    return launch_gemm<Epi>(a, nullptr, bt, nullptr, batch, m, n, k, lm, ln, sym, status, args, stream, name);
  if (batch < 1 || m < 1 || n < 1 || k < 1) return fail(I8M_E_ARGUMENT, "%s: empty problem", name);
  if (!a || !bt || !status) return fail(I8M_E_ARGUMENT, "%s: null operand or status pointer", name);
  if (sym && m != n) return fail(I8M_E_ARGUMENT, "%s: symmetric product needs m == n", name);
  GemmGeom g;
  g.batch = batch; g.m = m; g.n = n; g.k = k; g.lm = lm; g.ln = ln;
  g.tiles_m = cdiv(m, TILE); g.tiles_n = cdiv(n, TILE);
  g.sym = sym;
  g.tiles_per_batch = sym ? g.tiles_m * (g.tiles_m + 1) / 2 : g.tiles_m * g.tiles_n;
  g.num_kb = cdiv(k, 128);
  g.debug_simt = g_starve_producers ? 0x100 : 0;
  g.group = wide_group(k);
  g.a_raw = a; g.b_raw = bt; g.status = status;
  const long long tiles = (long long)g.tiles_per_batch * batch;
  if (tiles > 0x7fffffffLL / 2) return fail(I8M_E_LIMIT, "%s: too many tiles", name);
  if ((long long)g.num_kb * ((tiles + 1) / 1) > 0x7fffffffLL) return fail(I8M_E_LIMIT, "%s: too many K blocks", name);
  CUtensorMap ma, mb;
  if (int rc = make_operand_map(&ma, a, 1, k, m, batch)) return rc;
  if (int rc = make_operand_map(&mb, bt, 1, k, n, batch)) return rc;
  const unsigned grid = unsigned(std::min<long long>(tiles, sm_count()));
  if constexpr (Epi::SPLIT_TAIL) {
    if (g_bq_variant == 0) {
      constexpr size_t SMEM = bq_split_smem_bytes<Epi>();
      auto kernel = bq_split_kernel<Epi>;
      CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
      kernel<<<grid, BQS_THREADS, SMEM, stream>>>(ma, mb, g, args);
      LAUNCH_CHECK(name);
      return 0;
    }
  }
  const bool four = g_bq_variant == 2;
  const int stages = four ? BQP_STAGES_ALT : BQP_STAGES;
  const size_t SMEM = size_t(stages) * 2 * TILE_BYTES + sizeof(Ctrl) + 2 * BQP_MAX_KB * sizeof(float) +
                      Epi::TSM_BYTES + 1024;
  auto kernel = four ? bq_persistent_kernel<Epi, BQP_STAGES_ALT> : bq_persistent_kernel<Epi, BQP_STAGES>;
  CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
  kernel<<<grid, BQP_THREADS, SMEM, stream>>>(ma, mb, g, args);
  LAUNCH_CHECK(name);
  return 0;
}

bool float_dtype_ok(int d) { return d == I8M_F32 || d == I8M_F16 || d == I8M_BF16; }
size_t dtype_size(int d) { return d == I8M_F32 ? 4 : 2; }

template <typename E>
int float_gemm_typed(const void* left, const void* left_lo, const void* right_t,
                     const void* right_t_lo, void* out, void* out_t, void* out_lo, void* out_t_lo,
                     int mode, int batch, int m, int n, int k, int lm, int ln, int symmetric,
                     int final, int transpose, int out_dtype, float ca, float cb, float cc,
                     unsigned* status, cudaStream_t stream) {
  FloatArgs a;
  a.out = out; a.out_t = out_t; a.out_lo = out_lo; a.out_t_lo = out_t_lo;
  a.src = left; a.src_lo = left_lo;
  a.out_dtype = out_dtype; a.transpose = transpose;
  a.ca = ca; a.cb = cb; a.cc = cc;
  a.amax = final ? g_final_amax : nullptr;
  if (mode == 1) {
    if (final) return fail(I8M_E_ARGUMENT, "float_gemm: the polynomial mode has no final variant");
    if (k != n) return fail(I8M_E_ARGUMENT, "float_gemm: polynomial mode needs a square left operand");
    return launch_gemm<EpiFloat<E, MODE_QUAD>>(left, left_lo, right_t, right_t_lo, batch, m, n, k,
                                               lm, ln, symmetric, status, a, stream, "float_gemm(poly)");
  }
  if (final) {
    if (!float_dtype_ok(out_dtype)) return fail(I8M_E_ARGUMENT, "float_gemm: bad out_dtype %d", out_dtype);
    return launch_gemm<EpiFloat<E, MODE_FINAL>>(left, left_lo, right_t, right_t_lo, batch, m, n, k,
                                                lm, ln, 0, status, a, stream, "float_gemm(final)");
  }
  return launch_gemm<EpiFloat<E, MODE_PLAIN>>(left, left_lo, right_t, right_t_lo, batch, m, n, k, lm,
                                              ln, symmetric, status, a, stream, "float_gemm");
}

// dtype dispatch helpers for the memory-bound passes
#define DISPATCH_IN(dtype, In, ...)                                  \
  do {                                                               \
    if ((dtype) == I8M_F32) { using In = float; __VA_ARGS__; }       \
    else if ((dtype) == I8M_F16) { using In = __half; __VA_ARGS__; } \
    else { using In = __nv_bfloat16; __VA_ARGS__; }                  \
  } while (0)

}  // namespace

// =========================================================== library state
extern "C" int i8m_version(void) { return 100; }
extern "C" const char* i8m_build_info(void) {
  static char info[256];
  snprintf(info, sizeof(info),
           "i8muon_b200 arch=sm_100a cudart=%d tile=128x128x128B threads=%d mma=tcgen05 copy=tma "
           "fmad=off",
           CUDART_VERSION, GEMM_THREADS);
  return info;
}
extern "C" const char* i8m_last_error(void) { return g_error; }
extern "C" unsigned long long i8m_launch_count(void) { return g_launches.load(); }
extern "C" int i8m_set_debug_core(int simt) {
  g_debug_simt = simt == 1 ? 1 : 0;
  g_starve_producers = simt == 2 ? 1 : 0;
  return 0;
}
extern "C" int i8m_set_cta_limit(int max_ctas) {
  if (max_ctas < 0) return fail(I8M_E_ARGUMENT, "set_cta_limit: negative limit");
  g_cta_limit = max_ctas;
  return 0;
}
extern "C" int i8m_variant_count(const char* operation) {
  if (operation && std::strcmp(operation, "bq_gemm") == 0) return BQ_VARIANTS;
  if (operation && std::strcmp(operation, "wholek_gemm") == 0) return WHOLEK_VARIANTS;
  return 0;
}
extern "C" int i8m_set_variant(const char* operation, int variant) {
  if (!operation || (std::strcmp(operation, "bq_gemm") != 0 && std::strcmp(operation, "wholek_gemm") != 0))
    return fail(I8M_E_ARGUMENT, "set_variant: unknown operation");
  if (variant < 0 || variant >= i8m_variant_count(operation))
    return fail(I8M_E_ARGUMENT, "set_variant: %s has variants 0 to %d", operation, i8m_variant_count(operation) - 1);
  if (operation[0] == 'b') g_bq_variant = variant;
  else g_wholek_variant = variant;
  return 0;
}

// ================================================================== stats
extern "C" int i8m_stats_scratch_bytes(int batch, long long count, size_t* bytes) {
  if (batch < 1 || count < 1 || !bytes) return fail(I8M_E_ARGUMENT, "stats_scratch_bytes: bad argument");
  if (count / STATS_CHUNK >= 0x7fffffffLL) return fail(I8M_E_LIMIT, "stats_scratch_bytes: count %lld is too large", count);
  *bytes = size_t(2) * batch * size_t(count / STATS_CHUNK + (count % STATS_CHUNK != 0)) * sizeof(float);
  return 0;
}
extern "C" int i8m_stats(const void* x, int dtype, int batch, long long count, void* scratch,
                         size_t scratch_bytes, float* norm, float* amax, i8m_stream_t stream) {
  if (!x || !scratch || batch < 1 || batch > 65535 || count < 1 || !float_dtype_ok(dtype))
    return fail(I8M_E_ARGUMENT, "stats: bad argument");
  if (count / STATS_CHUNK >= 0x7fffffffLL) return fail(I8M_E_LIMIT, "stats: count %lld is too large", count);
  const int chunks = int(count / STATS_CHUNK + (count % STATS_CHUNK != 0));
  size_t need = size_t(2) * batch * chunks * sizeof(float);
  if (scratch_bytes < need) return fail(I8M_E_WORKSPACE, "stats: scratch %zu < %zu bytes", scratch_bytes, need);
  float* psum = static_cast<float*>(scratch);
  float* pmax = psum + size_t(batch) * chunks;
  DISPATCH_IN(dtype, In, (stats_partial_kernel<In><<<dim3(chunks, batch), STATS_THREADS, 0, S(stream)>>>(
                             static_cast<const In*>(x), psum, pmax, count, chunks)));
  LAUNCH_CHECK("stats_partial");
  stats_final_kernel<<<batch, STATS_THREADS, 0, S(stream)>>>(psum, pmax, norm, amax, chunks);
  LAUNCH_CHECK("stats_final");
  return 0;
}

// One launch, atomics, summation order not reproducible (the reference's deterministic=False path).
extern "C" int i8m_stats_onepass(const void* x, int dtype, int batch, long long count, void* scratch,
                                 size_t scratch_bytes, float* norm, float* amax, i8m_stream_t stream) {
  if (!x || !scratch || batch < 1 || batch > 65535 || count < 1 || !float_dtype_ok(dtype))
    return fail(I8M_E_ARGUMENT, "stats_onepass: bad argument");
  if (count / STATS_CHUNK >= 0x7fffffffLL) return fail(I8M_E_LIMIT, "stats_onepass: count %lld is too large", count);
  const int chunks = int(count / STATS_CHUNK + (count % STATS_CHUNK != 0));
  const size_t need = size_t(3) * batch * sizeof(float);
  if (scratch_bytes < need) return fail(I8M_E_WORKSPACE, "stats_onepass: scratch %zu < %zu bytes", scratch_bytes, need);
  CUDA_TRY(cudaMemsetAsync(scratch, 0, need, S(stream)));
  float* sumsq = static_cast<float*>(scratch);
  unsigned* bits = reinterpret_cast<unsigned*>(sumsq + batch);
  unsigned* arrived = bits + batch;
  DISPATCH_IN(dtype, In, (stats_onepass_kernel<In><<<dim3(chunks, batch), STATS_THREADS, 0, S(stream)>>>(
                             static_cast<const In*>(x), sumsq, bits, arrived, norm, amax, count, chunks)));
  LAUNCH_CHECK("stats_onepass");
  return 0;
}

// ------------------------------------------------------ stats without allocation
// Scratch for i8m_stats_static lives in the library image: 2^20 floats (4 MiB) per GPU
// that loads the library, held until the process exits.
constexpr size_t STATIC_SCRATCH_FLOATS = size_t(1) << 20;
static __device__ __align__(256) float g_static_stats_scratch[STATIC_SCRATCH_FLOATS];
namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {};
std::mutex g_static_scratch_mutex;
}  // namespace

extern "C" int i8m_stats_static(const void* x, int dtype, int batch, long long count, float* norm,
                                float* amax, i8m_stream_t stream) {
  if (!x || batch < 1 || batch > 65535 || count < 1 || !float_dtype_ok(dtype))
    return fail(I8M_E_ARGUMENT, "stats_static: bad argument");
  // no sum or product here can wrap: chunks is compared with the limit before it is multiplied
  const long long chunks = count / STATS_CHUNK + (count % STATS_CHUNK != 0);
  if (chunks > (long long)(STATIC_SCRATCH_FLOATS / 2) / batch)
    return fail(I8M_E_LIMIT,
                "stats_static: batch * ceil(count / 8192) = %lld exceeds the built-in scratch of %zu "
                "partials; use i8m_stats with caller scratch",
                (long long)batch * chunks, STATIC_SCRATCH_FLOATS / 2);
  int device = -1;
  CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= MAX_DEVICES) return fail(I8M_E_LIMIT, "stats_static: device index %d", device);
  float* scratch = nullptr;
  {
    // First call on this device: resolve the device address of the array.  In host
    // code the array's name is only a handle, never a pointer a kernel may use.
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_ptr[device]) {
      void* address = nullptr;
      CUDA_TRY(cudaGetSymbolAddress(&address, g_static_stats_scratch));
      g_static_scratch_ptr[device] = static_cast<float*>(address);
    }
    scratch = g_static_scratch_ptr[device];
  }
  // Every partial that the second pass reads is written by the first pass of the
  // same call, so nothing left over from an earlier call needs clearing.
  float* psum = scratch;
  float* pmax = scratch + size_t(batch) * chunks;
  DISPATCH_IN(dtype, In, (stats_partial_kernel<In><<<dim3(unsigned(chunks), batch), STATS_THREADS, 0, S(stream)>>>(
                             static_cast<const In*>(x), psum, pmax, count, int(chunks))));
  LAUNCH_CHECK("stats_partial(static)");
  stats_final_kernel<<<batch, STATS_THREADS, 0, S(stream)>>>(psum, pmax, norm, amax, int(chunks));
  LAUNCH_CHECK("stats_final(static)");
  return 0;
}

// ========================================================== floating path
extern "C" int i8m_normalize(const void* x, int in_dtype, const float* norm, void* a, void* a_t,
                             void* a_lo, void* a_t_lo, int compute, int batch, int rows, int cols,
                             int lp, int hp, int transpose, float eps, i8m_stream_t stream) {
  if (!x || !a || !float_dtype_ok(in_dtype) || !float_dtype_ok(compute) || batch < 1 || batch > 65535)
    return fail(I8M_E_ARGUMENT, "normalize: bad argument");
  if (compute == I8M_F32 && (!a_lo || (a_t && !a_t_lo)))
    return fail(I8M_E_ARGUMENT, "normalize: FP32 compute needs the low planes");
  // grid in the input's orientation, covering the padded extent
  const int prow = transpose ? hp : lp, pcol = transpose ? lp : hp;
  dim3 grid(cdiv(pcol, 32), cdiv(prow, 32), batch);
#define NORM_LAUNCH(E)                                                                         \
  DISPATCH_IN(in_dtype, In, (normalize_kernel<In, E><<<grid, 256, 0, S(stream)>>>(             \
                                static_cast<const In*>(x), norm, static_cast<E*>(a),           \
                                static_cast<E*>(a_t), static_cast<float*>(a_lo),               \
                                static_cast<float*>(a_t_lo), rows, cols, lp, hp, transpose, eps)))
  // 16-bit out, rows of whole 16-byte vectors: the vectorised kernel
  const bool vec = compute != I8M_F32 && cols % 8 == 0 && lp % 8 == 0 && hp % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a) |
                     reinterpret_cast<uintptr_t>(a_t)) & 15u) == 0;
  if (vec) {
    dim3 vgrid(cdiv(pcol, 64), cdiv(prow, 64), batch);
#define NORM_VEC(In, E)                                                                              \
  normalize_vec_kernel<In, E><<<vgrid, 256, 0, S(stream)>>>(static_cast<const In*>(x), norm,         \
                                                            static_cast<E*>(a), static_cast<E*>(a_t), \
                                                            rows, cols, lp, hp, transpose, eps)
    if (in_dtype == I8M_F32 && compute == I8M_F16) NORM_VEC(float, __half);
    else if (in_dtype == I8M_F32) NORM_VEC(float, __nv_bfloat16);
    else if (in_dtype == I8M_F16 && compute == I8M_F16) NORM_VEC(__half, __half);
    else if (in_dtype == I8M_F16) NORM_VEC(__half, __nv_bfloat16);
    else if (compute == I8M_F16) NORM_VEC(__nv_bfloat16, __half);
    else NORM_VEC(__nv_bfloat16, __nv_bfloat16);
#undef NORM_VEC
  } else if (compute == I8M_F32) NORM_LAUNCH(float);
  else if (compute == I8M_F16) NORM_LAUNCH(__half);
  else NORM_LAUNCH(__nv_bfloat16);
#undef NORM_LAUNCH
  LAUNCH_CHECK("normalize");
  return 0;
}

extern "C" int i8m_float_gemm(const void* left, const void* left_lo, const void* right_t,
                              const void* right_t_lo, void* out, void* out_t, void* out_lo,
                              void* out_t_lo, int compute, int mode, int batch, int m, int n, int k,
                              int lm, int ln, int symmetric, int final, int transpose,
                              int out_dtype, float ca, float cb, float cc, uint32_t* status,
                              i8m_stream_t stream) {
  if (!out || (mode != 0 && mode != 1)) return fail(I8M_E_ARGUMENT, "float_gemm: bad argument");
  if (compute == I8M_F32)
    return float_gemm_typed<float>(left, left_lo, right_t, right_t_lo, out, out_t, out_lo, out_t_lo,
                                   mode, batch, m, n, k, lm, ln, symmetric, final, transpose,
                                   out_dtype, ca, cb, cc, status, S(stream));
  if (compute == I8M_F16)
    return float_gemm_typed<__half>(left, left_lo, right_t, right_t_lo, out, out_t, out_lo, out_t_lo,
                                    mode, batch, m, n, k, lm, ln, symmetric, final, transpose,
                                    out_dtype, ca, cb, cc, status, S(stream));
  if (compute == I8M_BF16)
    return float_gemm_typed<__nv_bfloat16>(left, left_lo, right_t, right_t_lo, out, out_t, out_lo,
                                           out_t_lo, mode, batch, m, n, k, lm, ln, symmetric, final,
                                           transpose, out_dtype, ca, cb, cc, status, S(stream));
  return fail(I8M_E_ARGUMENT, "float_gemm: bad compute dtype %d", compute);
}

// FP16 / BF16 product whose result leaves as block-quantised INT8 operands (the end of the FP16 first
// iteration of an fp16-first INT8-BQ call): persistent kernel only.
template <typename E>
static int float_gemm_to_bq_typed(const void* left, const void* right_t, const FloatToBqArgs& args, int batch, int m,
                                  int n, int k, int lm, int ln, unsigned* status, cudaStream_t stream) {
  using Epi = EpiFloatToBq<E>;
  GemmGeom g;
  g.batch = batch; g.m = m; g.n = n; g.k = k; g.lm = lm; g.ln = ln;
  g.tiles_m = cdiv(m, TILE); g.tiles_n = cdiv(n, TILE);
  g.sym = 0;
  g.tiles_per_batch = g.tiles_m * g.tiles_n;
  g.num_kb = cdiv((long long)k * 2, 128);
  g.debug_simt = 0;
  g.group = wide_group(2LL * k);
  g.a_raw = left; g.b_raw = right_t; g.status = status;
  const long long blocks = (long long)g.tiles_per_batch * batch;
  if (blocks > 0x7fffffffLL) return fail(I8M_E_LIMIT, "float_gemm_to_bq: too many tiles");
  CUtensorMap ma, mb;
  if (int rc = make_operand_map(&ma, left, 2, k, m, batch)) return rc;
  if (int rc = make_operand_map(&mb, right_t, 2, k, n, batch)) return rc;
  if (g_wholek_variant == 0) {
    constexpr size_t WSMEM = wholek_wide_smem_bytes<Epi>();
    auto wk = wholek_wide_kernel<Epi>;
    CUDA_TRY(cudaFuncSetAttribute(wk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(WSMEM)));
    const long long units = (long long)wide_units_per_batch(g.tiles_m, g.tiles_n, 0) * batch;
    wk<<<unsigned(std::min<long long>(units, sm_count())), WKW_THREADS, WSMEM, stream>>>(ma, mb, g, args);
    LAUNCH_CHECK("float_gemm_to_bq");
    return 0;
  }
  constexpr size_t SMEM = size_t(WKP_STAGES) * 2 * TILE_BYTES + sizeof(Ctrl) + Epi::TSM_BYTES + 1024;
  auto kernel = wholek_persistent_kernel<Epi>;
  CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
  const unsigned grid = unsigned(std::min<long long>(blocks, sm_count()));
  kernel<<<grid, WKP_THREADS, SMEM, stream>>>(ma, mb, g, args);
  LAUNCH_CHECK("float_gemm_to_bq");
  return 0;
}

extern "C" int i8m_float_gemm_to_bq(const void* left, const void* right_t, void* q, void* q_t, float* scale,
                                    int compute, int user_dtype, int batch, int m, int n, int k, int lm, int ln,
                                    int lp, int hp, uint32_t* status, i8m_stream_t stream) {
  if (!left || !right_t || !q || !q_t || !scale || !status) return fail(I8M_E_ARGUMENT, "float_gemm_to_bq: null pointer");
  if (batch < 1 || m < 1 || n < 1 || k < 1 || lm < 1 || ln < 1 || lm > m || ln > n)
    return fail(I8M_E_ARGUMENT, "float_gemm_to_bq: bad extents");
  if (lp % 128 || hp % 128 || lp < m || hp < n || cdiv(lp, 128) != cdiv(m, 128) || cdiv(hp, 128) != cdiv(n, 128))
    return fail(I8M_E_ARGUMENT, "float_gemm_to_bq: lp, hp must be m, n rounded up to multiples of 128");
  if (!float_dtype_ok(user_dtype)) return fail(I8M_E_ARGUMENT, "float_gemm_to_bq: bad user dtype");
  FloatToBqArgs a;
  a.q = static_cast<uint8_t*>(q); a.qt = static_cast<uint8_t*>(q_t); a.scale = scale;
  a.lp = lp; a.hp = hp; a.user_dtype = user_dtype;
  if (compute == I8M_F16)
    return float_gemm_to_bq_typed<__half>(left, right_t, a, batch, m, n, k, lm, ln, status, S(stream));
  if (compute == I8M_BF16)
    return float_gemm_to_bq_typed<__nv_bfloat16>(left, right_t, a, batch, m, n, k, lm, ln, status, S(stream));
  return fail(I8M_E_ARGUMENT, "float_gemm_to_bq: compute must be a 16-bit type");
}

// ====================================================== global INT8 path
extern "C" int i8m_input_quant(const void* x, int in_dtype, const float* amax, const float* norm,
                               int8_t* a8, int8_t* a8_t, float* a_scale, int batch, int rows,
                               int cols, int lp, int hp, int transpose, float eps,
                               i8m_stream_t stream) {
  if (!x || !amax || !a8 || !a8_t || !a_scale || !float_dtype_ok(in_dtype) || batch < 1 || batch > 65535)
    return fail(I8M_E_ARGUMENT, "input_quant: bad argument");
  const int prow = transpose ? hp : lp, pcol = transpose ? lp : hp;
  if (rows == prow && cols == pcol && rows % 128 == 0 && cols % 128 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a8) | reinterpret_cast<uintptr_t>(a8_t)) & 15u) == 0) {
    // unpadded input of whole 128 x 128 tiles: vector loads, packed stores, transposes in registers
    int8_t* same = transpose ? a8_t : a8;
    int8_t* other = transpose ? a8 : a8_t;
    DISPATCH_IN(in_dtype, In, (input_quant128_kernel<In><<<dim3(cols / 128, rows / 128, batch), 256, 0, S(stream)>>>(
                                  static_cast<const In*>(x), amax, norm, same, other, a_scale, rows, cols,
                                  norm ? eps : 0.f)));
    LAUNCH_CHECK("input_quant");
    return 0;
  }
  dim3 grid(cdiv(pcol, 32), cdiv(prow, 32), batch);
  DISPATCH_IN(in_dtype, In, (input_quant_kernel<In><<<grid, 256, 0, S(stream)>>>(
                                static_cast<const In*>(x), amax, norm, a8, a8_t, a_scale, rows, cols,
                                lp, hp, transpose, norm ? eps : 0.f)));
  LAUNCH_CHECK("input_quant");
  return 0;
}

extern "C" int i8m_i8_gemm(int mode, const int8_t* a, const int8_t* b_t, const int8_t* row_b,
                           void* out, void* maximum, const float* a_scale, const float* b_scale,
                           const float* diag, int batch, int m, int n, int k, int lm, int ln,
                           float alpha, float beta, int final, int transpose, int out_dtype,
                           uint32_t* status, i8m_stream_t stream) {
  if (!out) return fail(I8M_E_ARGUMENT, "i8_gemm: null output");
  I8Args g;
  g.out = out; g.maximum = maximum; g.a_scale = a_scale; g.b_scale = b_scale; g.diag = diag;
  g.row_b = row_b; g.alpha = alpha; g.beta = beta; g.out_dtype = out_dtype; g.transpose = transpose;
  g.gain = alpha; g.use_gain = mode == 4;
  if (mode == 4) mode = 2;   // update whose right-hand scale is multiplied by alpha
  if (mode == 0) {
    if (!maximum) return fail(I8M_E_ARGUMENT, "i8_gemm: gram needs a maximum slot");
    return launch_gemm<EpiI8<I8_GRAM>>(a, nullptr, b_t, nullptr, batch, m, n, k, lm, ln, 1, status, g,
                                       S(stream), "i8_gemm(gram)");
  }
  if (mode == 1) {
    if (!maximum || !a_scale || !diag) return fail(I8M_E_ARGUMENT, "i8_gemm: square needs scale, diag, maximum");
    return launch_gemm<EpiI8<I8_SQUARE>>(a, nullptr, b_t, nullptr, batch, m, n, k, lm, ln, 1, status,
                                         g, S(stream), "i8_gemm(square)");
  }
  if (mode == 2) {
    if (!a_scale || !b_scale || !diag || !row_b) return fail(I8M_E_ARGUMENT, "i8_gemm: update needs scales, diag, row_b");
    if (final) {
      if (!float_dtype_ok(out_dtype)) return fail(I8M_E_ARGUMENT, "i8_gemm: bad out_dtype");
      return launch_gemm<EpiI8<I8_UPDATE_FINAL>>(a, nullptr, b_t, nullptr, batch, m, n, k, lm, ln, 0,
                                                 status, g, S(stream), "i8_gemm(final update)");
    }
    if (!maximum) return fail(I8M_E_ARGUMENT, "i8_gemm: update needs a maximum slot");
    return launch_gemm<EpiI8<I8_UPDATE>>(a, nullptr, b_t, nullptr, batch, m, n, k, lm, ln, 0, status, g,
                                         S(stream), "i8_gemm(update)");
  }
  return fail(I8M_E_ARGUMENT, "i8_gemm: bad mode %d", mode);
}

extern "C" int i8m_symmetric_quant(const void* input, const void* maximum, const float* orig_scale,
                                   const float* orig_diag, int8_t* output, float* scale, float* diag,
                                   int batch, int m, int quad, float c0, float c1, float c2,
                                   i8m_stream_t stream) {
  if (!input || !maximum || !orig_scale || !output || !scale || !diag || batch < 1 || batch > 65535 || m < 1)
    return fail(I8M_E_ARGUMENT, "symmetric_quant: bad argument");
  if (quad && !orig_diag) return fail(I8M_E_ARGUMENT, "symmetric_quant: quad needs the previous diagonal");
  if (m % 128 == 0 && ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(output)) & 15u) == 0) {
    const int t128 = m / 128;
    dim3 grid128(t128 * (t128 + 1) / 2, batch);
    if (quad)
      symmetric_quant128_kernel<float, true><<<grid128, 256, 0, S(stream)>>>(
          static_cast<const float*>(input), maximum, orig_scale, orig_diag, output, scale, diag, m, c0, c1, c2);
    else
      symmetric_quant128_kernel<int, false><<<grid128, 256, 0, S(stream)>>>(
          static_cast<const int*>(input), maximum, orig_scale, orig_diag, output, scale, diag, m, c0, c1, c2);
    LAUNCH_CHECK("symmetric_quant");
    return 0;
  }
  const int t = cdiv(m, 32);
  dim3 grid(t * (t + 1) / 2, batch);
  if (quad)
    symmetric_quant_kernel<float, true><<<grid, 256, 0, S(stream)>>>(
        static_cast<const float*>(input), maximum, orig_scale, orig_diag, output, scale, diag, m, c0, c1, c2);
  else
    symmetric_quant_kernel<int, false><<<grid, 256, 0, S(stream)>>>(
        static_cast<const int*>(input), maximum, orig_scale, orig_diag, output, scale, diag, m, c0, c1, c2);
  LAUNCH_CHECK("symmetric_quant");
  return 0;
}

extern "C" int i8m_output_quant(const float* input, const float* maximum, int8_t* out, int8_t* out_t,
                                float* scale, int batch, int m, int n, i8m_stream_t stream) {
  if (!input || !maximum || !out || !out_t || !scale || batch < 1 || batch > 65535)
    return fail(I8M_E_ARGUMENT, "output_quant: bad argument");
  if (m % 128 == 0 && n % 128 == 0 &&
      ((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out_t)) & 15u) == 0) {
    output_quant128_kernel<<<dim3(n / 128, m / 128, batch), 256, 0, S(stream)>>>(input, maximum, out, out_t, scale, m, n);
    LAUNCH_CHECK("output_quant");
    return 0;
  }
  dim3 grid(cdiv(n, 32), cdiv(m, 32), batch);
  output_quant_kernel<<<grid, 256, 0, S(stream)>>>(input, maximum, out, out_t, scale, m, n);
  LAUNCH_CHECK("output_quant");
  return 0;
}

// ================================================= block-quantised path
extern "C" int i8m_bq_quant(const void* x, int in_dtype, const float* norm, void* a, void* a_t,
                            float* scale, int fp8, int batch, int rows, int cols, int lp, int hp,
                            int transpose, float eps, i8m_stream_t stream) {
  if (!x || !a || !a_t || !scale || !float_dtype_ok(in_dtype) || batch < 1 || batch > 65535 ||
      lp % 128 || hp % 128)
    return fail(I8M_E_ARGUMENT, "bq_quant: bad argument");
  dim3 grid(lp / 128, hp / 128, batch);
  if (grid.y > 65535) return fail(I8M_E_LIMIT, "bq_quant: matrix too wide");
  const float e = norm ? eps : 0.f;
  const bool vec = in_dtype != I8M_F32 && cols % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a) |
                     reinterpret_cast<uintptr_t>(a_t)) & 15u) == 0;
  if (vec) {
#define BQ_VEC(In, F8)                                                                                  \
  bq_quant_vec_kernel<In, F8><<<grid, 256, 0, S(stream)>>>(static_cast<const In*>(x), norm,             \
                                                           static_cast<uint8_t*>(a),                    \
                                                           static_cast<uint8_t*>(a_t), scale, rows, cols, \
                                                           lp, hp, transpose, e)
    if (in_dtype == I8M_F16) { if (fp8) BQ_VEC(__half, true); else BQ_VEC(__half, false); }
    else { if (fp8) BQ_VEC(__nv_bfloat16, true); else BQ_VEC(__nv_bfloat16, false); }
#undef BQ_VEC
  } else if (fp8)
    DISPATCH_IN(in_dtype, In, (bq_quant_kernel<In, true><<<grid, 256, 0, S(stream)>>>(
                                  static_cast<const In*>(x), norm, static_cast<uint8_t*>(a),
                                  static_cast<uint8_t*>(a_t), scale, rows, cols, lp, hp, transpose, e)));
  else
    DISPATCH_IN(in_dtype, In, (bq_quant_kernel<In, false><<<grid, 256, 0, S(stream)>>>(
                                  static_cast<const In*>(x), norm, static_cast<uint8_t*>(a),
                                  static_cast<uint8_t*>(a_t), scale, rows, cols, lp, hp, transpose, e)));
  LAUNCH_CHECK("bq_quant");
  return 0;
}

template <bool FP8>
static int bq_gemm_typed(int mode, const void* a, const float* sa, const float* da, const void* b_t,
                         const float* sb, const void* row_b, void* out, void* out_t, float* so,
                         float* dout, int batch, int m, int n, int k, int lm, int ln, float ca,
                         float cb, float cc, int final, int transpose, int out_dtype,
                         unsigned* status, cudaStream_t stream) {
  BqArgs g;
  g.sa = sa; g.sb = sb; g.da = da; g.row_b = static_cast<const uint8_t*>(row_b);
  g.out = out; g.out_t = out_t; g.so = so; g.dout = dout;
  g.ca = ca; g.cb = cb; g.cc = cc; g.out_dtype = out_dtype; g.transpose = transpose;
  if (mode == 0) {
    if (!so || !dout) return fail(I8M_E_ARGUMENT, "bq_gemm: gram needs scale and diagonal outputs");
    return launch_bq<EpiBq<FP8, BQ_GRAM>>(a, b_t, batch, m, n, k, lm, ln, 1, status, g, stream, "bq_gemm(gram)");
  }
  if (mode == 1) {
    if (!so || !dout || !da) return fail(I8M_E_ARGUMENT, "bq_gemm: poly needs scale, diagonal in and out");
    return launch_bq<EpiBq<FP8, BQ_POLY>>(a, b_t, batch, m, n, k, lm, ln, 1, status, g, stream, "bq_gemm(poly)");
  }
  if (mode == 2) {
    if (!da || !row_b) return fail(I8M_E_ARGUMENT, "bq_gemm: update needs the diagonal and row_b");
    if (final) {
      if (!float_dtype_ok(out_dtype)) return fail(I8M_E_ARGUMENT, "bq_gemm: bad out_dtype");
      return launch_bq<EpiBq<FP8, BQ_UPDATE_FINAL>>(a, b_t, batch, m, n, k, lm, ln, 0, status, g, stream,
                                                   "bq_gemm(final update)");
    }
    if (!so || !out_t) return fail(I8M_E_ARGUMENT, "bq_gemm: update needs scale and transposed outputs");
    return launch_bq<EpiBq<FP8, BQ_UPDATE>>(a, b_t, batch, m, n, k, lm, ln, 0, status, g, stream, "bq_gemm(update)");
  }
  return fail(I8M_E_ARGUMENT, "bq_gemm: bad mode %d", mode);
}

extern "C" int i8m_bq_gemm(int fp8, int mode, const void* a, const float* sa, const float* da,
                           const void* b_t, const float* sb, const void* row_b, void* out,
                           void* out_t, float* so, float* dout, int batch, int m, int n, int k,
                           int lm, int ln, float ca, float cb, float cc, int final, int transpose,
                           int out_dtype, uint32_t* status, i8m_stream_t stream) {
  if (!out || !sa || !sb) return fail(I8M_E_ARGUMENT, "bq_gemm: null pointer");
  if (m % 128 || n % 128 || k % 128) return fail(I8M_E_ARGUMENT, "bq_gemm: extents must be multiples of 128");
  if (fp8)
    return bq_gemm_typed<true>(mode, a, sa, da, b_t, sb, row_b, out, out_t, so, dout, batch, m, n, k,
                               lm, ln, ca, cb, cc, final, transpose, out_dtype, status, S(stream));
  return bq_gemm_typed<false>(mode, a, sa, da, b_t, sb, row_b, out, out_t, so, dout, batch, m, n, k,
                              lm, ln, ca, cb, cc, final, transpose, out_dtype, status, S(stream));
}

// ====================================================== optimizer kernels
extern "C" int i8m_momentum(const void* const* grads, void* const* bufs, int count, void* update,
                            long long numel, int dtype, float buf_weight, float mu, int nesterov,
                            float* stats_partials, i8m_stream_t stream) {
  if (!grads || !bufs || !update || count < 1 || numel < 1 || !float_dtype_ok(dtype))
    return fail(I8M_E_ARGUMENT, "momentum: bad argument");
  if (numel / STATS_CHUNK >= 0x7fffffffLL) return fail(I8M_E_LIMIT, "momentum: tensor too large");
  const size_t es = dtype_size(dtype);
  const int chunks = int(numel / STATS_CHUNK + (numel % STATS_CHUNK != 0));
  const int blocks_x = std::min(chunks, 148 * 16);
  // stats_partials (optional): the scratch layout of i8m_stats over the stacked update,
  // [count][chunks] sums of squares followed by [count][chunks] maxima
  float* psum = stats_partials;
  float* pmax = stats_partials ? stats_partials + size_t(count) * chunks : nullptr;
  for (int first = 0; first < count; first += MT_MAX) {
    const int c = std::min(MT_MAX, count - first);
    MomentumTable tab;
    for (int i = 0; i < c; ++i) {
      if (!grads[first + i] || !bufs[first + i]) return fail(I8M_E_ARGUMENT, "momentum: null tensor");
      tab.grad[i] = grads[first + i];
      tab.buf[i] = bufs[first + i];
    }
    char* u = static_cast<char*>(update) + size_t(first) * numel * es;
    dim3 grid(blocks_x, c);
    DISPATCH_IN(dtype, T, (momentum_kernel<T><<<grid, 256, 0, S(stream)>>>(
                              tab, reinterpret_cast<T*>(u), numel, buf_weight, mu, nesterov, psum, pmax, chunks, first)));
    LAUNCH_CHECK("momentum");
  }
  return 0;
}

extern "C" int i8m_apply(void* const* params, int count, const void* update, long long numel,
                         int param_dtype, int update_dtype, int decay_mode, float decay,
                         float neg_lr, i8m_stream_t stream) {
  if (!params || !update || count < 1 || numel < 1 || !float_dtype_ok(param_dtype) ||
      !float_dtype_ok(update_dtype) || decay_mode < 0 || decay_mode > 2)
    return fail(I8M_E_ARGUMENT, "apply: bad argument");
  const size_t es = dtype_size(update_dtype);
  const int blocks_x = int(std::min<long long>(cdiv(numel, 256 * 8), 148 * 16));
  for (int first = 0; first < count; first += MT_MAX) {
    const int c = std::min(MT_MAX, count - first);
    ApplyTable tab;
    for (int i = 0; i < c; ++i) {
      if (!params[first + i]) return fail(I8M_E_ARGUMENT, "apply: null tensor");
      tab.param[i] = params[first + i];
    }
    const char* u = static_cast<const char*>(update) + size_t(first) * numel * es;
    dim3 grid(blocks_x, c);
#define APPLY_LAUNCH(P)                                                                        \
  DISPATCH_IN(update_dtype, U, (apply_kernel<P, U><<<grid, 256, 0, S(stream)>>>(               \
                                   tab, reinterpret_cast<const U*>(u), numel, decay_mode, decay, neg_lr)))
    if (param_dtype == I8M_F32) APPLY_LAUNCH(float);
    else if (param_dtype == I8M_F16) APPLY_LAUNCH(__half);
    else APPLY_LAUNCH(__nv_bfloat16);
#undef APPLY_LAUNCH
    LAUNCH_CHECK("apply");
  }
  return 0;
}

// AdamW companion for the parameters outside Muon; FP32 moments, parameters and gradients in
// any of the three floating types.  bias corrections are passed by the host (1 - beta^step).
extern "C" int i8m_adamw(void* const* params, const void* const* grads, float* const* exp_avg,
                         float* const* exp_avg_sq, const long long* numel, int count, int param_dtype,
                         int grad_dtype, float lr, float beta1, float beta2, float eps,
                         float weight_decay, float bias_correction1, float bias_correction2,
                         i8m_stream_t stream) {
  if (!params || !grads || !exp_avg || !exp_avg_sq || !numel || count < 1 || !float_dtype_ok(param_dtype) ||
      !float_dtype_ok(grad_dtype) || !(bias_correction1 > 0.f) || !(bias_correction2 > 0.f))
    return fail(I8M_E_ARGUMENT, "adamw: bad argument");
  const float decay = 1.f - lr * weight_decay;
  const float step_size = lr / bias_correction1;
  const float inv_bc2_sqrt = 1.f / sqrtf(bias_correction2);
  for (int first = 0; first < count; first += ADAM_MAX) {
    const int c = std::min(ADAM_MAX, count - first);
    AdamTable tab;
    long long longest = 0;
    for (int i = 0; i < c; ++i) {
      const int k = first + i;
      if (!params[k] || !grads[k] || !exp_avg[k] || !exp_avg_sq[k] || numel[k] < 1)
        return fail(I8M_E_ARGUMENT, "adamw: null tensor or empty tensor");
      tab.param[i] = params[k]; tab.grad[i] = grads[k];
      tab.exp_avg[i] = exp_avg[k]; tab.exp_avg_sq[i] = exp_avg_sq[k];
      tab.numel[i] = numel[k];
      longest = std::max(longest, numel[k]);
    }
    dim3 grid(unsigned(std::min<long long>(cdiv(longest, 256 * 4), 148 * 16)), c);
#define ADAM_LAUNCH(P)                                                                              \
  DISPATCH_IN(grad_dtype, G, (adamw_kernel<P, G><<<grid, 256, 0, S(stream)>>>(tab, decay, beta1, beta2, eps, \
                                                                              step_size, inv_bc2_sqrt)))
    if (param_dtype == I8M_F32) ADAM_LAUNCH(float);
    else if (param_dtype == I8M_F16) ADAM_LAUNCH(__half);
    else ADAM_LAUNCH(__nv_bfloat16);
#undef ADAM_LAUNCH
    LAUNCH_CHECK("adamw");
  }
  return 0;
}

// ============================================== whole Newton-Schulz drivers
namespace {

struct Bump {
  char* base;
  size_t used = 0, cap;
  bool dry;
  Bump(void* p, size_t c, bool d) : base(static_cast<char*>(p)), cap(c), dry(d) {}
  void* take(size_t bytes) {
    size_t off = align256(used);
    used = off + bytes;
    return dry ? nullptr : base + off;
  }
  template <typename T>
  T* take_n(size_t n) { return static_cast<T*>(take(n * sizeof(T))); }
};

struct NsCall {
  int route, dtype, batch, rows, cols, compute, steps, fp16_first;
  int factored = 0;   // coefficient rows are (c, p, q) of c * ((G + p I)^2 + q I)
  int deterministic = 1;   // 0: one-pass statistics with atomics (summation order not reproducible)
  const float* stats_partials = nullptr;   // partials of the statistics over x, computed by the caller (i8m_momentum)
  int fuse_first_row = 1;   // fp16-first INT8-BQ: the first row's update quantises its own result
  int wholek[3] = {-1, -1, -1};   // global INT8: kernel variant of the Gram / square / update product (-1: thread's)
  const void* x;
  void* out;
  const double* coeffs;
  float eps;
  const char* gram_order;
  unsigned* status;
  cudaStream_t stream;
};

int call_stats(const NsCall& c, const void* x, int B, long long count, void* scratch, size_t sbytes, float* norm,
               float* amax) {
  if (c.stats_partials && x == c.x) {
    // the producer of x left the per-chunk partials: only the final fold remains
    const int chunks = int(count / STATS_CHUNK + (count % STATS_CHUNK != 0));
    stats_final_kernel<<<B, STATS_THREADS, 0, c.stream>>>(c.stats_partials, c.stats_partials + size_t(B) * chunks, norm,
                                                          amax, chunks);
    LAUNCH_CHECK("stats_final");
    return 0;
  }
  if (c.deterministic) return i8m_stats(x, c.dtype, B, count, scratch, sbytes, norm, amax, c.stream);
  return i8m_stats_onepass(x, c.dtype, B, count, scratch, sbytes, norm, amax, c.stream);
}
size_t stats_bytes(int B, long long count) {
  size_t sbytes = 0;
  i8m_stats_scratch_bytes(B, count, &sbytes);
  return std::max(sbytes, size_t(3) * B * sizeof(float));   // either flavour fits
}

// A matrix in the floating compute dtype: one plane, or (hi, lo) for FP32.
struct FMat {
  void* p = nullptr;
  void* lo = nullptr;
};
FMat take_fmat(Bump& ws, size_t elems, int compute) {
  FMat m;
  m.p = ws.take(elems * dtype_size(compute));
  if (compute == I8M_F32) m.lo = ws.take(elems * 4);
  return m;
}

// floating NS (regular and Gram); with plan == true only the workspace is sized.
struct BqOperands {   // where a floating first row leaves its result for the block-quantised rows
  uint8_t* a = nullptr;
  uint8_t* at = nullptr;
  float* sa = nullptr;
  int lp = 0, hp = 0;
};

int run_float(const NsCall& c, Bump& ws, bool plan, bool gram, const void* x, void* out,
              int out_dtype, int steps, const double* coeffs, int compute, bool normalize_input,
              bool factored = false, const BqOperands* to_bq = nullptr, float* final_amax = nullptr) {
  const int B = c.batch, rows = c.rows, cols = c.cols;
  const int l = std::min(rows, cols), h = std::max(rows, cols);
  const int lp = pad_to(l, 16), hp = pad_to(h, 16);
  const int transpose = rows > cols;
  const size_t wide = size_t(B) * lp * hp, sq = size_t(B) * lp * lp;
  FMat a = take_fmat(ws, wide, compute), at = take_fmat(ws, wide, compute);
  FMat y = take_fmat(ws, wide, compute), yt = take_fmat(ws, wide, compute);
  FMat r = take_fmat(ws, sq, compute), q0 = take_fmat(ws, sq, compute);
  FMat z, q1;
  if (gram) { z = take_fmat(ws, sq, compute); q1 = take_fmat(ws, sq, compute); }
  float* norm = ws.take_n<float>(B);
  const size_t sbytes = stats_bytes(B, (long long)rows * cols);
  void* scratch = ws.take(sbytes);
  if (plan) return 0;

  if (normalize_input) {
    if (int rc = call_stats(c, x, B, (long long)rows * cols, scratch, sbytes, norm, nullptr)) return rc;
  }
  if (int rc = i8m_normalize(x, c.dtype, normalize_input ? norm : nullptr, a.p, at.p, a.lo, at.lo,
                             compute, B, rows, cols, lp, hp, transpose, c.eps, c.stream))
    return rc;
  auto gemm = [&](const FMat& left, const FMat& right, const FMat& o, const FMat& ot, int mode, int n,
                  int k, int ln, int sym, int final, int tr, void* user, double ca, double cb,
                  double cc) -> int {
    // the final product can leave the maximum magnitude of what it stores (the global-INT8 rows that
    // follow an FP16 first row quantise it with that scale: no statistics pass over the result)
    struct Handover { ~Handover() { g_final_amax = nullptr; } } reset;
    g_final_amax = final ? final_amax : nullptr;
    return i8m_float_gemm(left.p, left.lo, right.p, right.lo, final ? user : o.p, ot.p, o.lo, ot.lo,
                          compute, mode, B, lp, n, k, l, ln, sym, final, tr, out_dtype, float(ca),
                          float(cb), float(cc), c.status, c.stream);
  };
  const FMat none;
  if (!gram) {
    for (int it = 0; it < steps; ++it) {
      double ca = coeffs[3 * it], cb = coeffs[3 * it + 1], cc = coeffs[3 * it + 2];
      if (int rc = gemm(a, a, r, none, 0, lp, hp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
      if (factored) {
        // completed-square row (c, p, q): shift the Gram diagonal by p, then c*q I + c R'^2
        // (src/i8muon/_cutlass_prec.py:97-100); 16-bit compute types only
        const double fc = ca, fp = cb, fq = cc;
        const long long n = (long long)B * l;
        if (compute == I8M_F16)
          diag_add_kernel<__half><<<unsigned(cdiv(n, 256)), 256, 0, c.stream>>>(static_cast<__half*>(r.p), B, lp, l, float(fp));
        else
          diag_add_kernel<__nv_bfloat16><<<unsigned(cdiv(n, 256)), 256, 0, c.stream>>>(static_cast<__nv_bfloat16*>(r.p), B, lp, l, float(fp));
        LAUNCH_CHECK("diag_add");
        ca = fc * fq; cb = 0.0; cc = fc;
      }
      if (int rc = gemm(r, r, q0, none, 1, lp, lp, l, 1, 0, 0, nullptr, ca, cb, cc)) return rc;
      const bool final = it == steps - 1;
      if (final && to_bq) {
        // the result stays in the wide orientation and leaves as INT8 blocks (no transposition back)
        if (int rc = i8m_float_gemm_to_bq(q0.p, at.p, to_bq->a, to_bq->at, to_bq->sa, compute, out_dtype, B, lp, hp, lp,
                                          l, h, to_bq->lp, to_bq->hp, c.status, c.stream))
          return rc;
        return 0;
      }
      if (int rc = gemm(q0, at, y, yt, 0, hp, lp, h, 0, final, final && transpose, out, 0, 0, 0)) return rc;
      if (!final) { std::swap(a, y); std::swap(at, yt); }
    }
    return 0;
  }
  // Gram-space iteration with restarts (src/i8muon/_cutlass_prec.py:107-130).
  std::string order = c.gram_order ? c.gram_order : "00100";
  if (order.empty() || order[0] != '0' || order.find_first_not_of("01") != std::string::npos)
    return fail(I8M_E_ARGUMENT, "gram_order must be a binary string starting with 0");
  if (int(order.size()) < steps) order.append(size_t(steps) - order.size(), '0');
  for (int it = 0; it < steps; ++it) {
    const double ca = coeffs[3 * it], cb = coeffs[3 * it + 1], cc = coeffs[3 * it + 2];
    const char kind = order[size_t(it)];
    const bool refresh = it + 1 < steps && order[size_t(it) + 1] == '0';
    if (kind == '1') {
      if (int rc = gemm(q0, at, y, yt, 0, hp, lp, h, 0, 0, 0, nullptr, 0, 0, 0)) return rc;
      std::swap(a, y); std::swap(at, yt);
    }
    if (kind == '1' || it == 0) {
      if (int rc = gemm(a, a, r, none, 0, lp, hp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
      if (int rc = gemm(r, r, q0, none, 1, lp, lp, l, 1, 0, 0, nullptr, ca, cb, cc)) return rc;
      if (refresh) {
        if (int rc = gemm(r, q0, q1, none, 0, lp, lp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
        if (int rc = gemm(q0, q1, r, none, 0, lp, lp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
      }
    } else {
      if (int rc = gemm(r, r, z, none, 1, lp, lp, l, 1, 0, 0, nullptr, ca, cb, cc)) return rc;
      if (int rc = gemm(z, q0, q1, none, 0, lp, lp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
      std::swap(q0, q1);
      if (refresh) {
        if (int rc = gemm(r, z, q1, none, 0, lp, lp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
        if (int rc = gemm(z, q1, r, none, 0, lp, lp, l, 1, 0, 0, nullptr, 0, 0, 0)) return rc;
      }
    }
  }
  return gemm(q0, at, y, yt, 0, hp, lp, h, 0, 1, transpose, out, 0, 0, 0);
}

// global-scale INT8 NS (src/i8muon/_cutlass.py:162-251)
int run_int8(const NsCall& c, Bump& ws, bool plan, const void* x, int steps, const double* coeffs,
             bool normalize_input, bool factored = false, const float* given_amax = nullptr) {
  const int B = c.batch, rows = c.rows, cols = c.cols;
  const int l = std::min(rows, cols), h = std::max(rows, cols);
  const int lp = pad_to(l, 16), hp = pad_to(h, 16);
  const int transpose = rows > cols;
  const size_t wide = size_t(B) * lp * hp, sq = size_t(B) * lp * lp;
  int8_t* a8 = ws.take_n<int8_t>(wide);
  int8_t* a8t = ws.take_n<int8_t>(wide);
  float* work = ws.take_n<float>(wide);      // int32 Gram / fp32 polynomial / fp32 update
  int8_t* s8 = ws.take_n<int8_t>(sq);         // quantised Gram, then quantised polynomial
  float* a_scale = ws.take_n<float>(B);
  float* g_scale = ws.take_n<float>(B);
  float* p_scale = ws.take_n<float>(B);
  float* g_diag = ws.take_n<float>(size_t(B) * lp);
  float* p_diag = ws.take_n<float>(size_t(B) * lp);
  float* maxima = ws.take_n<float>(size_t(3) * steps * B);
  float* norm = ws.take_n<float>(B);
  float* amax = ws.take_n<float>(B);
  const size_t sbytes = stats_bytes(B, (long long)rows * cols);
  void* scratch = ws.take(sbytes);
  if (plan) return 0;
  if ((long long)hp * 127 * 127 > 0x7fffffffLL)
    return fail(I8M_E_LIMIT, "inner dimension can overflow the int32 accumulator");

  CUDA_TRY(cudaMemsetAsync(maxima, 0, size_t(3) * steps * B * sizeof(float), c.stream));
  if (given_amax == nullptr) {
    if (int rc = call_stats(c, x, B, (long long)rows * cols, scratch, sbytes, normalize_input ? norm : nullptr, amax))
      return rc;
  }
  if (int rc = i8m_input_quant(x, c.dtype, given_amax ? given_amax : amax, normalize_input ? norm : nullptr, a8, a8t, a_scale, B,
                               rows, cols, lp, hp, transpose, c.eps, c.stream))
    return rc;
  for (int it = 0; it < steps; ++it) {
    // A completed-square row (c, p, q) is the same five stages with the Gram diagonal shifted
    // by p, the polynomial G'^2 + q I (b = 0, c = 1, a = q: bit-identical expressions to the
    // reference's unscaled modes) and c folded into the update's right-hand scale
    // (src/i8muon/_cutlass.py:196-246).
    float ca = float(coeffs[3 * it]), cb = float(coeffs[3 * it + 1]), cc = float(coeffs[3 * it + 2]);
    float shift = 0.f, gain = 0.f;
    if (factored) { gain = ca; shift = cb; ca = cc; cb = 0.f; cc = 1.f; }
    float* gmax = maxima + size_t(3 * it) * B;
    float* pmax = gmax + B;
    float* ymax = pmax + B;
    const int thread_wholek = g_wholek_variant;
    auto pick = [&](int op) { g_wholek_variant = c.wholek[op] < 0 ? thread_wholek : c.wholek[op]; };
    struct Restore { int v; ~Restore() { g_wholek_variant = v; } } restore{thread_wholek};
    pick(0);
    if (int rc = i8m_i8_gemm(0, a8, a8, nullptr, work, gmax, nullptr, nullptr, nullptr, B, lp, lp, hp, l,
                             l, 0, 0, 0, 0, 0, c.status, c.stream))
      return rc;
    if (int rc = i8m_symmetric_quant(work, gmax, a_scale, nullptr, s8, g_scale, g_diag, B, lp, 0, shift, 0, 0, c.stream))
      return rc;
    pick(1);
    if (int rc = i8m_i8_gemm(1, s8, s8, nullptr, work, pmax, g_scale, nullptr, g_diag, B, lp, lp, lp, l, l,
                             cb, cc, 0, 0, 0, c.status, c.stream))
      return rc;
    if (int rc = i8m_symmetric_quant(work, pmax, g_scale, g_diag, s8, p_scale, p_diag, B, lp, 1, ca, cb, cc, c.stream))
      return rc;
    const bool final = it == steps - 1;
    pick(2);
    if (int rc = i8m_i8_gemm(factored ? 4 : 2, s8, a8t, a8, final ? c.out : static_cast<void*>(work), ymax, p_scale,
                             a_scale, p_diag, B, lp, hp, lp, l, h, gain, 0, final, transpose, c.dtype,
                             c.status, c.stream))
      return rc;
    if (!final)
      if (int rc = i8m_output_quant(work, ymax, a8, a8t, a_scale, B, lp, hp, c.stream)) return rc;
  }
  return 0;
}

// grouped cubics with a terminal quintic, all INT8 (src/i8muon/_cutlass_cubic.py:8-71): per cubic the
// Gram product, its quantisation with the shifted FP32 diagonal, the update with -gain folded into
// the right-hand scale, and the output quantisation; then the regular five stages of the last row.
int run_int8_cubic(const NsCall& c, Bump& ws, bool plan) {
  const int B = c.batch, rows = c.rows, cols = c.cols;
  const int l = std::min(rows, cols), h = std::max(rows, cols);
  const int lp = pad_to(l, 16), hp = pad_to(h, 16);
  const int transpose = rows > cols;
  const int cubics = c.steps - 2;
  const size_t wide = size_t(B) * lp * hp, sq = size_t(B) * lp * lp;
  int8_t* a8 = ws.take_n<int8_t>(wide);
  int8_t* a8t = ws.take_n<int8_t>(wide);
  float* work = ws.take_n<float>(wide);
  int8_t* s8 = ws.take_n<int8_t>(sq);
  float* a_scale = ws.take_n<float>(B);
  float* g_scale = ws.take_n<float>(B);
  float* p_scale = ws.take_n<float>(B);
  float* g_diag = ws.take_n<float>(size_t(B) * lp);
  float* p_diag = ws.take_n<float>(size_t(B) * lp);
  const size_t slots = size_t(2) * std::max(cubics, 0) + 3;
  float* maxima = ws.take_n<float>(slots * B);
  float* norm = ws.take_n<float>(B);
  float* amax = ws.take_n<float>(B);
  const size_t sbytes = stats_bytes(B, (long long)rows * cols);
  void* scratch = ws.take(sbytes);
  if (plan) return 0;
  if (cubics < 1) return fail(I8M_E_ARGUMENT, "the cubic route needs an input-gain row, cubic rows and a terminal row");
  if ((long long)hp * 127 * 127 > 0x7fffffffLL)
    return fail(I8M_E_LIMIT, "inner dimension can overflow the int32 accumulator");
  const float input_gain = float(c.coeffs[0]);
  if (!(input_gain > 0.f) || !(c.eps > 0.f)) return fail(I8M_E_ARGUMENT, "the cubic route needs positive input_gain and eps");
  CUDA_TRY(cudaMemsetAsync(maxima, 0, slots * B * sizeof(float), c.stream));
  if (int rc = call_stats(c, c.x, B, (long long)rows * cols, scratch, sbytes, norm, amax)) return rc;
  clamp_divide_kernel<<<cdiv(B, 256), 256, 0, c.stream>>>(norm, B, c.eps, input_gain);
  LAUNCH_CHECK("clamp_divide");
  if (int rc = i8m_input_quant(c.x, c.dtype, amax, norm, a8, a8t, a_scale, B, rows, cols, lp, hp, transpose, 0.f, c.stream))
    return rc;
  for (int i = 0; i < cubics; ++i) {
    const float gain = float(c.coeffs[3 * (i + 1)]), shift = float(c.coeffs[3 * (i + 1) + 1]);
    float* gmax = maxima + size_t(2 * i) * B;
    float* ymax = gmax + B;
    if (int rc = i8m_i8_gemm(0, a8, a8, nullptr, work, gmax, nullptr, nullptr, nullptr, B, lp, lp, hp, l, l, 0, 0, 0, 0, 0,
                             c.status, c.stream))
      return rc;
    if (int rc = i8m_symmetric_quant(work, gmax, a_scale, nullptr, s8, g_scale, g_diag, B, lp, 0, shift, 0, 0, c.stream))
      return rc;
    if (int rc = i8m_i8_gemm(4, s8, a8t, a8, work, ymax, g_scale, a_scale, g_diag, B, lp, hp, lp, l, h, -gain, 0, 0, 0, 0,
                             c.status, c.stream))
      return rc;
    if (int rc = i8m_output_quant(work, ymax, a8, a8t, a_scale, B, lp, hp, c.stream)) return rc;
  }
  const double* abc = c.coeffs + 3 * (c.steps - 1);
  float* gmax = maxima + size_t(2 * cubics) * B;
  float* pmax = gmax + B;
  if (int rc = i8m_i8_gemm(0, a8, a8, nullptr, work, gmax, nullptr, nullptr, nullptr, B, lp, lp, hp, l, l, 0, 0, 0, 0, 0,
                           c.status, c.stream))
    return rc;
  if (int rc = i8m_symmetric_quant(work, gmax, a_scale, nullptr, s8, g_scale, g_diag, B, lp, 0, 0, 0, 0, c.stream)) return rc;
  if (int rc = i8m_i8_gemm(1, s8, s8, nullptr, work, pmax, g_scale, nullptr, g_diag, B, lp, lp, lp, l, l, float(abc[1]),
                           float(abc[2]), 0, 0, 0, c.status, c.stream))
    return rc;
  if (int rc = i8m_symmetric_quant(work, pmax, g_scale, g_diag, s8, p_scale, p_diag, B, lp, 1, float(abc[0]), float(abc[1]),
                                   float(abc[2]), c.stream))
    return rc;
  return i8m_i8_gemm(2, s8, a8t, a8, c.out, nullptr, p_scale, a_scale, p_diag, B, lp, hp, lp, l, h, 0, 0, 1, transpose,
                     c.dtype, c.status, c.stream);
}

// block-quantised NS (src/i8muon/_cutlass_bq.py:15-70)
int run_bq(const NsCall& c, Bump& ws, bool plan, bool fp8, const void* x, int steps,
           const double* coeffs, bool normalize_input, const BqOperands* given = nullptr) {
  const int B = c.batch, rows = c.rows, cols = c.cols;
  const int l = std::min(rows, cols), h = std::max(rows, cols);
  const int lp = pad_to(l, 128), hp = pad_to(h, 128);
  const int transpose = rows > cols;
  const size_t wide = size_t(B) * lp * hp, sq = size_t(B) * lp * lp;
  const int lq = lp / 128, hq = hp / 128;
  // `given`: the operands were quantised already (by the floating first row's epilogue)
  uint8_t* a = given ? given->a : ws.take_n<uint8_t>(wide);
  uint8_t* at = given ? given->at : ws.take_n<uint8_t>(wide);
  uint8_t* y = ws.take_n<uint8_t>(wide);
  uint8_t* yt = ws.take_n<uint8_t>(wide);
  uint8_t* gq = ws.take_n<uint8_t>(sq);
  uint8_t* pq = ws.take_n<uint8_t>(sq);
  float* sa = given ? given->sa : ws.take_n<float>(size_t(B) * lq * hq);
  float* sy = ws.take_n<float>(size_t(B) * lq * hq);
  float* sg = ws.take_n<float>(size_t(B) * lq * lq);
  float* sp = ws.take_n<float>(size_t(B) * lq * lq);
  float* dg = ws.take_n<float>(size_t(B) * lp);
  float* dp = ws.take_n<float>(size_t(B) * lp);
  float* norm = ws.take_n<float>(B);
  const size_t sbytes = stats_bytes(B, (long long)rows * cols);
  void* scratch = ws.take(sbytes);
  if (plan) return 0;

  if (!given) {
    if (normalize_input)
      if (int rc = call_stats(c, x, B, (long long)rows * cols, scratch, sbytes, norm, nullptr)) return rc;
    if (int rc = i8m_bq_quant(x, c.dtype, normalize_input ? norm : nullptr, a, at, sa, fp8, B, rows, cols,
                              lp, hp, transpose, c.eps, c.stream))
      return rc;
  }
  for (int it = 0; it < steps; ++it) {
    const float ca = float(coeffs[3 * it]), cb = float(coeffs[3 * it + 1]), cc = float(coeffs[3 * it + 2]);
    if (int rc = i8m_bq_gemm(fp8, 0, a, sa, nullptr, a, sa, nullptr, gq, nullptr, sg, dg, B, lp, lp, hp, l,
                             l, 0, 0, 0, 0, 0, 0, c.status, c.stream))
      return rc;
    if (int rc = i8m_bq_gemm(fp8, 1, gq, sg, dg, gq, sg, nullptr, pq, nullptr, sp, dp, B, lp, lp, lp, l, l,
                             ca, cb, cc, 0, 0, 0, c.status, c.stream))
      return rc;
    const bool final = it == steps - 1;
    if (int rc = i8m_bq_gemm(fp8, 2, pq, sp, dp, at, sa, a, final ? c.out : static_cast<void*>(y),
                             final ? nullptr : yt, final ? nullptr : sy, nullptr, B, lp, hp, lp, l, h, 0,
                             0, 0, final, transpose, c.dtype, c.status, c.stream))
      return rc;
    if (!final) { std::swap(a, y); std::swap(at, yt); std::swap(sa, sy); }
  }
  return 0;
}

int ns_dispatch(const NsCall& c, Bump& ws, bool plan) {
  if (c.batch < 1 || c.batch > 65535) return fail(I8M_E_ARGUMENT, "batch size must be between 1 and 65535");
  if (c.rows < 1 || c.cols < 1) return fail(I8M_E_ARGUMENT, "matrix dimensions must be positive");
  if (!float_dtype_ok(c.dtype)) return fail(I8M_E_ARGUMENT, "input must be float32, float16 or bfloat16");
  if (c.steps < 1) return fail(I8M_E_ARGUMENT, "at least one coefficient row is required");
  switch (c.route) {
    case I8M_ROUTE_FLOAT:
    case I8M_ROUTE_GRAM:
      if (!float_dtype_ok(c.compute)) return fail(I8M_E_ARGUMENT, "bad compute dtype %d", c.compute);
      return run_float(c, ws, plan, c.route == I8M_ROUTE_GRAM, c.x, c.out, c.dtype, c.steps, c.coeffs,
                       c.compute, true);
    case I8M_ROUTE_INT8_FACTORED: {
      // completed-square rows (c, p, q), src/i8muon/_cutlass.py:93-128
      if (!c.fp16_first) return run_int8(c, ws, plan, c.x, c.steps, c.coeffs, true, true);
      if (c.steps == 1)
        return run_float(c, ws, plan, false, c.x, c.out, c.dtype, 1, c.coeffs, I8M_F16, true, true);
      void* first = ws.take(size_t(c.batch) * c.rows * c.cols * dtype_size(c.dtype));
      size_t mark = ws.used;
      if (int rc = run_float(c, ws, plan, false, c.x, first, c.dtype, 1, c.coeffs, I8M_F16, true, true)) return rc;
      size_t after_float = ws.used;
      ws.used = mark;
      int rc = run_int8(c, ws, plan, first, c.steps - 1, plan ? nullptr : c.coeffs + 3, false, true);
      ws.used = std::max(ws.used, after_float);
      return rc;
    }
    case I8M_ROUTE_INT8:
    case I8M_ROUTE_BQ_INT8: {
      const bool bq = c.route == I8M_ROUTE_BQ_INT8;
      if (!c.fp16_first)
        return bq ? run_bq(c, ws, plan, false, c.x, c.steps, c.coeffs, true)
                  : run_int8(c, ws, plan, c.x, c.steps, c.coeffs, true);
      // First row in FP16 with its result rounded to the input dtype, then the
      // quantised rows without re-normalising (src/i8muon/_cutlass.py:137-142).
      if (c.steps == 1)
        return run_float(c, ws, plan, false, c.x, c.out, c.dtype, 1, c.coeffs, I8M_F16, true);
      if (bq && c.fuse_first_row) {
        // The first row's update product quantises its own result (the CTA tile is the quantisation
        // block): no 16-bit intermediate in HBM, no standalone quantisation pass.
        const int l = std::min(c.rows, c.cols), h = std::max(c.rows, c.cols);
        BqOperands ops;
        ops.lp = pad_to(l, 128); ops.hp = pad_to(h, 128);
        const size_t wide = size_t(c.batch) * ops.lp * ops.hp;
        ops.a = ws.take_n<uint8_t>(wide);
        ops.at = ws.take_n<uint8_t>(wide);
        ops.sa = ws.take_n<float>(size_t(c.batch) * (ops.lp / 128) * (ops.hp / 128));
        const size_t mark = ws.used;
        if (int rc = run_float(c, ws, plan, false, c.x, nullptr, c.dtype, 1, c.coeffs, I8M_F16, true, false, &ops)) return rc;
        const size_t after_float = ws.used;
        ws.used = mark;  // the quantised rows reuse the floating stage's scratch
        const int rc = run_bq(c, ws, plan, false, nullptr, c.steps - 1, plan ? nullptr : c.coeffs + 3, false, &ops);
        ws.used = std::max(ws.used, after_float);
        return rc;
      }
      void* first = ws.take(size_t(c.batch) * c.rows * c.cols * dtype_size(c.dtype));
      // global INT8: the first row's final store also leaves max |X1| per matrix, the scale of the rows
      // that follow (deterministic: a maximum does not depend on the order of its operands)
      float* first_amax = bq ? nullptr : ws.take_n<float>(c.batch);
      size_t mark = ws.used;
      if (!plan && first_amax) CUDA_TRY(cudaMemsetAsync(first_amax, 0, size_t(c.batch) * sizeof(float), c.stream));
      if (int rc = run_float(c, ws, plan, false, c.x, first, c.dtype, 1, c.coeffs, I8M_F16, true, false, nullptr,
                             first_amax))
        return rc;
      size_t after_float = ws.used;
      ws.used = mark;  // the quantised stage reuses the floating stage's scratch
      int rc = bq ? run_bq(c, ws, plan, false, first, c.steps - 1, plan ? nullptr : c.coeffs + 3, false)
                  : run_int8(c, ws, plan, first, c.steps - 1, plan ? nullptr : c.coeffs + 3, false, false, first_amax);
      ws.used = std::max(ws.used, after_float);
      return rc;
    }
    case I8M_ROUTE_BQ_FP8:
      return run_bq(c, ws, plan, true, c.x, c.steps, c.coeffs, true);
    case I8M_ROUTE_INT8_CUBIC:
      return run_int8_cubic(c, ws, plan);
    default:
      return fail(I8M_E_ARGUMENT, "unknown route %d", c.route);
  }
}

}  // namespace

extern "C" int i8m_ns_workspace_bytes(int route, int batch, int rows, int cols, int dtype,
                                      int compute, int steps, int fp16_first, size_t* bytes) {
  if (!bytes) return fail(I8M_E_ARGUMENT, "ns_workspace_bytes: null result pointer");
  NsCall c{};
  c.route = route; c.dtype = dtype; c.batch = batch; c.rows = rows; c.cols = cols;
  c.compute = compute; c.steps = steps; c.fp16_first = fp16_first;
  Bump ws(nullptr, ~size_t(0), true);
  if (int rc = ns_dispatch(c, ws, true)) return rc;
  *bytes = align256(ws.used);
  return 0;
}

extern "C" int i8m_ns_run(int route, const void* x, void* out, int dtype, int batch, int rows,
                          int cols, int compute, const double* coeffs, int steps, float eps,
                          int fp16_first, int deterministic, int variants, const char* gram_order,
                          const float* stats_partials, void* workspace, size_t workspace_bytes, uint32_t* status,
                          i8m_stream_t stream) {
  if (!x || !out || !coeffs || !workspace || !status) return fail(I8M_E_ARGUMENT, "ns_run: null pointer");
  if (x == out) return fail(I8M_E_ARGUMENT, "ns_run: out may not alias x");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(I8M_E_ARGUMENT, "ns_run: workspace must be 256-byte aligned");
  size_t need = 0;
  if (int rc = i8m_ns_workspace_bytes(route, batch, rows, cols, dtype, compute, steps, fp16_first, &need)) return rc;
  if (workspace_bytes < need)
    return fail(I8M_E_WORKSPACE, "ns_run: workspace %zu < %zu bytes", workspace_bytes, need);
  NsCall c{};
  c.route = route; c.dtype = dtype; c.batch = batch; c.rows = rows; c.cols = cols;
  c.compute = compute; c.steps = steps; c.fp16_first = fp16_first;
  c.x = x; c.out = out; c.coeffs = coeffs; c.eps = eps; c.gram_order = gram_order;
  c.status = status; c.stream = S(stream);
  c.deterministic = deterministic ? 1 : 0;
  c.stats_partials = stats_partials;
  Bump ws(workspace, workspace_bytes, false);
  if (variants < 0) return ns_dispatch(c, ws, false);
  // this call's own kernel selection; the thread's setting comes back whatever happens
  const int bq = variants & 0xff, wholek = (variants >> 8) & 0xff;
  const int wk_square = (variants >> 16) & 0xff, wk_update = (variants >> 24) & 0x7f;
  if (bq >= BQ_VARIANTS || wholek >= WHOLEK_VARIANTS || wk_square >= WHOLEK_VARIANTS || wk_update >= WHOLEK_VARIANTS)
    return fail(I8M_E_ARGUMENT, "ns_run: unknown kernel variant 0x%x", variants);
  const int saved_bq = g_bq_variant, saved_wholek = g_wholek_variant;
  g_bq_variant = bq;
  g_wholek_variant = wholek;
  c.wholek[0] = wholek; c.wholek[1] = wk_square; c.wholek[2] = wk_update;
  const int rc = ns_dispatch(c, ws, false);
  g_bq_variant = saved_bq;
  g_wholek_variant = saved_wholek;
  return rc;
}
