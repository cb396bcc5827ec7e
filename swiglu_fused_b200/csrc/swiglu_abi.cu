// C ABI of libswiglu_b200.so: argument validation, TMA descriptor encoding,
// tile-table lookup and the kernel launches.  Replaces the reference's Python
// launch layer (swiglu/matmul_silu_mul.py:62-95, swiglu/matmul_fused_swiglu.py:71-103),
// its ctypes TMA helper (swiglu/_tma_utils.py:69-111) and its nvcc JIT loader
// (swiglu/_pycuda_loader.py:128-144; this library is built ahead of time).
//
// No function here allocates device memory or synchronises, except
// sgl_device_status, which is a debugging aid and says so, and the host-buffer
// pipeline (swiglu_host_pipeline.cuh), whose job is to own device buffers.

#include "../../include/swiglu_b200.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include <cuda.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>   // header-only; a no-op unless a profiler is attached

#include "swiglu_elementwise.cuh"
#include "swiglu_kernel.cuh"

namespace {

thread_local std::string t_last_error;
std::atomic<int64_t> g_launches{0};
std::atomic<uint64_t> g_wait_limit_ns{2000000000ull};
// Self-checking builds only (sgl_debug_cluster_sum_missing_arrivals): arrivals the barrier of
// the cluster sum expects on top of those that will come, so that its bounded wait runs out.
std::atomic<int> g_debug_missing_arrivals{0};

// Tracing, off by default (the reference prints from its tuner and loader unconditionally,
// swiglu/matmul_silu_mul.py:135,156,159).  SGL_LOG=1 writes one line per kernel launch to
// stderr; SGL_NVTX=1 wraps every launch in an NVTX range named after the form and the shape,
// which shows up in timeline profilers.  Both are read once.
bool env_flag(const char* name) {
  const char* v = getenv(name);
  return v && v[0] != '\0' && v[0] != '0';
}
bool log_enabled() {
  static const bool on = env_flag("SGL_LOG");
  return on;
}
bool nvtx_enabled() {
  static const bool on = env_flag("SGL_NVTX");
  return on;
}
const char* form_name(int form) {
  switch (form) {
    case SGL_FORM_SILU_MUL: return "silu_mul";
    case SGL_FORM_FUSED_SWIGLU: return "fused_swiglu";
    case SGL_FORM_MATMUL: return "matmul";
    case SGL_FORM_FUSED_SWIGLU_SAVE: return "fused_swiglu_save";
    default: return "?";
  }
}

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_last_error = buf;
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  // Clear the sticky-free error so later calls are not poisoned by this one.
  cudaGetLastError();
  return fail(static_cast<int>(e), "%s: %s (%s)", what, cudaGetErrorName(e),
              cudaGetErrorString(e));
}

// ---------------------------------------------------------------- driver entry point

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// A tensor map is a pure function of these parameters, so encoded maps are kept in a small
// per-thread cache (the reference caches its maps too, keyed by pointers only:
// swiglu/matmul_silu_mul.py:62-75).  Saves the driver call on repeated launches over the
// same buffers, which is what a decode loop or a CUDA-graph-free serving step does.
struct MapKey {
  const void* base;
  int64_t rows, cols, ld;
  int32_t box_rows, box_cols, promo, swizzle, f32;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && box_cols == o.box_cols && promo == o.promo &&
           swizzle == o.swizzle && f32 == o.f32;
  }
};
struct MapCacheEntry {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapCacheSize = 64;   // direct mapped

// Rank-2 bf16 (or fp32) map over a row-major [rows, cols] tensor with row pitch `ld`
// elements; box = box_cols (one swizzle row: <= 128 bytes, or <= 64 with the 64B swizzle)
// x box_rows.
int make_map(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld,
             int box_rows, int box_cols, CUtensorMapL2promotion promo, const char* name,
             bool f32 = false, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  thread_local MapCacheEntry cache[kMapCacheSize] = {};
  const MapKey key{base, rows, cols, ld, box_rows, box_cols, static_cast<int32_t>(promo),
                   static_cast<int32_t>(swizzle), f32 ? 1 : 0};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h ^= static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(cols) * 0xC2B2AE3D27D4EB4Full;
  h ^= static_cast<uint64_t>(box_rows * 131 + box_cols * 7 + static_cast<int>(swizzle));
  MapCacheEntry& e = cache[(h ^ (h >> 29)) % kMapCacheSize];
  if (e.valid && e.key == key) {
    *out = e.map;
    return SGL_OK;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(SGL_ERR_NO_DRIVER, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(SGL_ERR_TENSOR_MAP,
                "cuTensorMapEncodeTiled(%s) failed with CUresult %d (rows=%lld cols=%lld ld=%lld)",
                name, static_cast<int>(r), static_cast<long long>(rows),
                static_cast<long long>(cols), static_cast<long long>(ld));
  }
  e.key = key;
  e.map = *out;
  e.valid = true;
  return SGL_OK;
}

// ---------------------------------------------------------------- kernel variants

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap,
                          const sgl::OutMaps, const sgl::KernelParams);

struct Variant {
  KernelFn fn;
  int out_cols;
  int max_stages;
  int (*smem_bytes)(int);
};

template <int F, int G, int BK, bool W = false>
int smem_bytes_of(int stages) {
  return sgl::KernelTraits<F, G, BK, W>::smem_bytes(stages);
}

template <int F, int G, int BK, bool W = false>
Variant make_variant() {
  using T = sgl::KernelTraits<F, G, BK, W>;
  Variant v;
  v.fn = sgl::swiglu_kernel<F, G, BK, W>;
  v.out_cols = T::kOutCols;
  v.max_stages = T::max_stages();
  v.smem_bytes = smem_bytes_of<F, G, BK, W>;
  return v;
}

// Index: form * 4 + (cta_group - 1) * 2 + (block_k == 128); 16 = the wide-tile fused variant.
constexpr int kNumVariants = 17;
constexpr int kWideVariant = 16;
int variant_index(int form, int cta_group, int block_k, int wide = 0) {
  if (wide) return kWideVariant;
  return form * 4 + (cta_group - 1) * 2 + (block_k == 128 ? 1 : 0);
}
const Variant& variant(int form, int cta_group, int block_k, int wide = 0) {
  static const Variant table[kNumVariants] = {
      make_variant<sgl::FORM_SILU_MUL, 1, 64>(),  make_variant<sgl::FORM_SILU_MUL, 1, 128>(),
      make_variant<sgl::FORM_SILU_MUL, 2, 64>(),  make_variant<sgl::FORM_SILU_MUL, 2, 128>(),
      make_variant<sgl::FORM_FUSED, 1, 64>(),     make_variant<sgl::FORM_FUSED, 1, 128>(),
      make_variant<sgl::FORM_FUSED, 2, 64>(),     make_variant<sgl::FORM_FUSED, 2, 128>(),
      make_variant<sgl::FORM_GEMM, 1, 64>(),      make_variant<sgl::FORM_GEMM, 1, 128>(),
      make_variant<sgl::FORM_GEMM, 2, 64>(),      make_variant<sgl::FORM_GEMM, 2, 128>(),
      make_variant<sgl::FORM_FUSED_SAVE, 1, 64>(), make_variant<sgl::FORM_FUSED_SAVE, 1, 128>(),
      make_variant<sgl::FORM_FUSED_SAVE, 2, 64>(), make_variant<sgl::FORM_FUSED_SAVE, 2, 128>(),
      make_variant<sgl::FORM_FUSED, 2, 64, true>(),
  };
  return table[variant_index(form, cta_group, block_k, wide)];
}

bool config_fields_ok(const sgl_config& c) {
  return (c.cta_group == 1 || c.cta_group == 2) && (c.block_k == 64 || c.block_k == 128) &&
         c.stages >= 0 && c.stages <= sgl::kMaxStages && c.group_m >= 1 && c.max_ctas >= 0 &&
         c.group_n >= 0 && (c.wide == 0 || c.wide == 1) &&
         c.l2_hints >= 0 && c.l2_hints < 256 && (c.l2_hints & 3) != 3 &&
         ((c.l2_hints >> 2) & 3) != 3 && ((c.l2_hints >> 4) & 3) != 3 && ((c.l2_hints >> 6) & 3) != 3;
}

// Built-in tile table (cta_group, block_k, stages (0 = deepest), group_m, max_ctas, l2_hints).
const sgl_config kTable[] = {
    {2, 64, 0, 8, 0, 0, 0, 0},  {2, 64, 0, 4, 0, 0, 0, 0},  {2, 64, 0, 16, 0, 0, 0, 0},
    {2, 64, 0, 1, 0, 0, 0, 0},  {2, 64, 0, 32, 0, 0, 0, 0}, {2, 128, 0, 8, 0, 0, 0, 0},
    {2, 128, 0, 16, 0, 0, 0, 0}, {1, 64, 0, 8, 0, 0, 0, 0}, {1, 64, 0, 16, 0, 0, 0, 0},
    {1, 64, 0, 1, 0, 0, 0, 0},  {1, 128, 0, 8, 0, 0, 0, 0},
    // x loads evict-last + output stores evict-first (l2_hints = 2 | 1 << 4)
    {2, 128, 0, 16, 0, 18, 0, 0}, {2, 64, 0, 16, 0, 18, 0, 0}, {2, 128, 0, 12, 0, 18, 0, 0},
};
constexpr int kTableSize = static_cast<int>(sizeof(kTable) / sizeof(kTable[0]));

// Entries of kTable a form can run: at least a two-stage ring must fit.
int form_entries(int form, int* idx) {
  int n = 0;
  for (int i = 0; i < kTableSize; ++i) {
    if (variant(form, kTable[i].cta_group, kTable[i].block_k).max_stages >= 2) idx[n++] = i;
  }
  return n;
}

// ---------------------------------------------------------------- per-device state

struct DeviceInfo {
  int sm_count = 0;
  int cc = 0;
  int max_smem_optin = 0;
  int max_clusters[20] = {};  // per variant, 0 = not yet queried
  int smem_set[20] = {};      // dynamic smem attribute already raised to
  // split-K summed in the cluster: clusters of n single-CTA tiles that can be resident at once,
  // per variant and n (0 = not yet asked, -1 = such clusters cannot be launched here)
  int max_k_clusters[20][17] = {};
};

std::mutex g_dev_mutex;
std::map<int, DeviceInfo> g_devices;

int device_info(int* dev_out, DeviceInfo** info_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  auto it = g_devices.find(dev);
  if (it == g_devices.end()) {
    DeviceInfo d;
    int major = 0, minor = 0;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) !=
            cudaSuccess ||
        (e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev)) !=
            cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) !=
            cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                    dev)) != cudaSuccess) {
      return fail_cuda(e, "cudaDeviceGetAttribute");
    }
    d.cc = major * 10 + minor;
    it = g_devices.emplace(dev, d).first;
  }
  *dev_out = dev;
  *info_out = &it->second;
  return SGL_OK;
}

int validate_ptr(const void* p, const char* name) {
  if (!p) return fail(SGL_ERR_NULL_POINTER, "%s is NULL", name);
  if (reinterpret_cast<uintptr_t>(p) & 15u)
    return fail(SGL_ERR_MISALIGNED, "%s is not 16-byte aligned", name);
  return SGL_OK;
}

int validate_ld(int64_t ld, int64_t min_cols, const char* name) {
  if (ld < min_cols)
    return fail(SGL_ERR_BAD_STRIDE, "%s=%lld is smaller than the %lld columns it must hold", name,
                static_cast<long long>(ld), static_cast<long long>(min_cols));
  if (ld % 8 != 0)
    return fail(SGL_ERR_BAD_STRIDE, "%s=%lld is not a multiple of 8 elements (16 bytes)", name,
                static_cast<long long>(ld));
  if (ld > 0x7fffffffll)
    return fail(SGL_ERR_BAD_STRIDE, "%s=%lld does not fit 31 bits", name,
                static_cast<long long>(ld));
  return SGL_OK;
}

int validate_shape(int64_t M, int64_t N, int64_t K) {
  if (M < 1 || N < 1 || K < 1)
    return fail(SGL_ERR_BAD_SHAPE, "M=%lld N=%lld K=%lld must all be >= 1",
                static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K));
  if (N % 8 != 0 || K % 8 != 0)
    return fail(SGL_ERR_BAD_SHAPE, "N=%lld and K=%lld must be multiples of 8",
                static_cast<long long>(N), static_cast<long long>(K));
  if (M > 0x7fffff00ll || N > 0x7fffff00ll || K > 0x7fffff00ll)
    return fail(SGL_ERR_BAD_SHAPE, "M, N and K must fit 31 bits");
  return SGL_OK;
}

// Built-in choice when the caller passes no configuration.  Measured on B200
// under a sustained (power-capped) load: both activation forms run best with CTA
// pairs, BLOCK_K = 128 (3-stage ring) and bands of 16 tile rows once there are
// at least 2048 rows; shorter problems as the branches below say.  A single
// 128-row tile cannot use a pair.
void default_config(int form, int64_t M, sgl_config* c) {
  std::memset(c, 0, sizeof(*c));
  c->stages = 0;
  if (M <= sgl::kBlockM) {
    c->cta_group = 1;
    c->block_k = 64;
    c->group_m = 8;
  } else if (form == SGL_FORM_FUSED_SWIGLU_SAVE) {
    c->cta_group = 2;
    c->block_k = (M >= 2048) ? 128 : 64;
    c->group_m = 16;
    c->l2_hints = 2 | (1 << 4);   // x evict-last, h and factor stores evict-first (measured)
  } else if (form != SGL_FORM_SILU_MUL && M >= 2048) {
    c->cta_group = 2;
    c->block_k = 128;
    c->group_m = 16;
    // x and weight loads evict-last, h stores evict-first: 1-3 % at the 32768 x 3072 x 12288
    // and 16384 x 4096 x 14336 fused problems (the GEMM form keeps the plain policy)
    if (form == SGL_FORM_FUSED_SWIGLU) c->l2_hints = 2 | (2 << 2) | (1 << 4);
  } else if (form == SGL_FORM_FUSED_SWIGLU && M <= 2 * sgl::kBlockM) {
    // one pair-tile row: tiles of 256 output columns (x fetched once per 256 columns, half as
    // many tiles to spread over the CTA pairs).  Measured under sustained load at 256 x 4096 x
    // 14336: 65 us against 69 (BLOCK_K 128) and 79 (BLOCK_K 64) with 128-column tiles.
    c->cta_group = 2;
    c->block_k = 64;
    c->group_m = 8;
    c->wide = 1;
  } else if (form == SGL_FORM_FUSED_SWIGLU) {
    // a few tile rows: the BLOCK_K = 128 ring (half as many barrier round trips per tile);
    // measured 115 against 148 us at 512 x 4096 x 14336, 195 against 256 us at 1024 rows
    c->cta_group = 2;
    c->block_k = 128;
    c->group_m = 8;
  } else if (M >= 2048) {
    c->cta_group = 2;
    c->block_k = 128;
    c->group_m = 16;   // silu_mul at 32768 x 3072 x 12288: 1.96 ms against 2.00 with bands of 8
  } else if (form == SGL_FORM_SILU_MUL && M >= 1024) {
    c->cta_group = 2;
    c->block_k = 128;  // silu_mul at 1024 x 4096 x 14336: 111 against 116 us
    c->group_m = 8;
  } else {
    c->cta_group = 2;
    c->block_k = 64;
    c->group_m = 8;
  }
}

// Resolves stages == 0 and checks that the configuration fits.
int resolve_config(int form, const sgl_config* in, int64_t M, sgl_config* out) {
  if (in) {
    *out = *in;
  } else {
    default_config(form, M, out);
  }
  if (!config_fields_ok(*out))
    return fail(SGL_ERR_BAD_CONFIG,
                "unsupported tile configuration: cta_group=%d block_k=%d stages=%d group_m=%d",
                out->cta_group, out->block_k, out->stages, out->group_m);
  if (out->wide && (form != SGL_FORM_FUSED_SWIGLU || out->cta_group != 2 || out->block_k != 64))
    return fail(SGL_ERR_BAD_CONFIG,
                "wide tiles need the fused_swiglu form with cta_group=2 and block_k=64");
  const Variant& v = variant(form, out->cta_group, out->block_k, out->wide);
  if (out->stages == 0) out->stages = v.max_stages;
  if (out->stages < 2 || out->stages > v.max_stages)
    return fail(SGL_ERR_BAD_CONFIG, "stages=%d outside [2, %d] for cta_group=%d block_k=%d",
                out->stages, v.max_stages, out->cta_group, out->block_k);
  return SGL_OK;
}

// Everything one kernel launch needs besides the tile configuration.
struct LaunchSpec {
  int form = SGL_FORM_FUSED_SWIGLU;
  const CUtensorMap* x = nullptr;    // A operand
  const CUtensorMap* w = nullptr;    // B operand
  const CUtensorMap* up = nullptr;   // silu_mul form only (any valid map otherwise)
  const sgl::OutMaps* out = nullptr;
  int64_t M = 0, N = 0, K = 0;
  int64_t col0 = 0, col1 = 0;        // B column (or row) offsets: see KernelParams
  int n_dst = 1;
  int a_mnmajor = 0;
  int b_kmajor = 0;
  int out_f32 = 0;
  int reduce_rows = 0, reduce_add = 0, first_dst = 0;     // reduce-scatter epilogue
  int splits = 1, k_per_split = 0, slot_rows = 0;         // split-K
  int acc_cols = 0;                                       // GEMM form: tile width (0 = choose)
  int a_rows = sgl::kBlockM;                              // rows of the A box (see a_box_rows)
  int peer_mode = 0, n_peer = 0;                          // gather by thread stores
  int64_t peer_ld = 0;
  const void* peer_ptr[sgl::kMaxDst] = {};
  // split-K: where the K ranges may be summed inside the launch (KernelParams::cluster_sum)
  void* sum_out = nullptr;           // bf16 result, row pitch sum_ld
  int64_t sum_ld = 0;
  bool* summed = nullptr;            // set to true when the launch wrote the result itself
  const void* up_raw = nullptr;      // silu_mul form summed in clusters: up, row pitch up_ld
  int64_t up_ld = 0;
  bool cluster_only = false;         // launch only if the K ranges can be summed in clusters,
                                     // else return kClustersNotPlaced without launching
};

constexpr int kClustersNotPlaced = 1;   // internal to this file, never returned to a caller

// Split-K problems whose K ranges can form thread-block clusters are summed inside the GEMM
// launch through distributed shared memory.  sgl_set_splitk_cluster_sum(0) switches that off
// (partial tiles through scratch memory and a second kernel, as for every other problem);
// SGL_SPLITK_CLUSTER_SUM=0 in the environment does the same from outside.
std::atomic<int> g_splitk_cluster_sum{-1};   // -1 = not yet read from the environment

bool splitk_cluster_sum_enabled() {
  int v = g_splitk_cluster_sum.load();
  if (v < 0) {
    const char* e = getenv("SGL_SPLITK_CLUSTER_SUM");
    v = (e && e[0] == '0') ? 0 : 1;
    g_splitk_cluster_sum.store(v);
  }
  return v != 0;
}

// Rows of the A operand's TMA box.  A problem shorter than one 128-row tile loads only the rows
// it has (rounded up to the 8-row swizzle atom): the rest of the tile's rows in shared memory
// keep whatever they held, the MMA turns them into accumulator rows nobody stores, and the
// SM is spared fetching zero fill for them on every k-block.
int a_box_rows(int64_t M, int cta_group) {
  if (cta_group == 1 && M < sgl::kBlockM) return static_cast<int>((M + 7) / 8 * 8);
  return sgl::kBlockM;
}

// Clusters of this variant that can be resident at once (1 CTA or CTA pair per SM).
int query_max_clusters(const Variant& v, int cta_group, int sm_count) {
  int n = sm_count / cta_group;
  if (cta_group == 2) {
    cudaLaunchConfig_t qc = {};
    qc.gridDim = dim3(static_cast<unsigned>(sm_count / 2 * 2), 1, 1);
    qc.blockDim = dim3(sgl::kNumThreads, 1, 1);
    qc.dynamicSmemBytes = static_cast<size_t>(v.smem_bytes(v.max_stages));
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    qc.attrs = qa;
    qc.numAttrs = 1;
    int q = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&q, reinterpret_cast<const void*>(v.fn), &qc);
    if (e == cudaSuccess && q > 0) {
      if (q < n) n = q;
    } else {
      cudaGetLastError();   // keep the SM-count estimate
    }
  }
  return n > 0 ? n : 1;
}

// Clusters of n CTAs of a single-CTA variant that can be resident at once with `smem` bytes
// each (sizes above 8 need the kernel's consent to a non-portable cluster size).  Negative:
// the driver cannot place such clusters.  Call with g_dev_mutex held.
int query_k_clusters(const Variant& v, int n, int smem) {
  cudaError_t e;
  if (n > 8) {
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(v.fn),
                             cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
  }
  cudaLaunchConfig_t qc = {};
  qc.gridDim = dim3(static_cast<unsigned>(n), 1, 1);
  qc.blockDim = dim3(sgl::kNumThreads, 1, 1);
  qc.dynamicSmemBytes = static_cast<size_t>(smem);
  cudaLaunchAttribute qa[1];
  qa[0].id = cudaLaunchAttributeClusterDimension;
  qa[0].val.clusterDim.x = static_cast<unsigned>(n);
  qa[0].val.clusterDim.y = 1;
  qa[0].val.clusterDim.z = 1;
  qc.attrs = qa;
  qc.numAttrs = 1;
  int q = 0;
  e = cudaOccupancyMaxActiveClusters(&q, reinterpret_cast<const void*>(v.fn), &qc);
  if (e != cudaSuccess || q < 1) {
    cudaGetLastError();
    return -1;
  }
  return q;
}

// First use of this variant on this device: raise its dynamic shared-memory limit to the
// deepest ring and ask how many clusters fit.
int prepare_variant(DeviceInfo* info, const Variant& v, int vi, int cta_group) {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  const int smem_max = v.smem_bytes(v.max_stages);
  if (info->smem_set[vi] < smem_max) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(v.fn),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
    if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(max dynamic smem)");
    info->smem_set[vi] = smem_max;
  }
  if (info->max_clusters[vi] == 0)
    info->max_clusters[vi] = query_max_clusters(v, cta_group, info->sm_count);
  return SGL_OK;
}

// Clusters of n CTAs of single-CTA variant vi that fit at once (cached; <= 0: none).
int k_clusters(DeviceInfo* info, const Variant& v, int vi, int n, int smem) {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  int& q = info->max_k_clusters[vi][n];
  if (q == 0) q = query_k_clusters(v, n, smem);
  return q;
}

// Whether this configuration's ring can hold a partial tile for the cluster sum.
bool ring_holds_partial_tile(const Variant& v, int stages) {
  return static_cast<int64_t>(stages) * (v.smem_bytes(2) - v.smem_bytes(1)) >=
         static_cast<int64_t>(sgl::kRedBytes);
}

int launch(const LaunchSpec& s, const sgl_config& cfg, DeviceInfo* info, void* stream) {
  const int wide = (cfg.wide && !s.b_kmajor) ? 1 : 0;   // the [n, k] layout has no wide form
  const int vi = variant_index(s.form, cfg.cta_group, cfg.block_k, wide);
  const Variant& v = variant(s.form, cfg.cta_group, cfg.block_k, wide);
  const int smem = v.smem_bytes(cfg.stages);
  if (smem > info->max_smem_optin)
    return fail(SGL_ERR_BAD_CONFIG, "configuration needs %d bytes of shared memory, device has %d",
                smem, info->max_smem_optin);

  const int rows_per_tile = sgl::kBlockM * cfg.cta_group;
  const int64_t tiles_m = (s.M + rows_per_tile - 1) / rows_per_tile;
  // GEMM form on single-CTA tiles ([k, n] weight, no split-K, no reduce-scatter): a short
  // problem with few 256-column tiles leaves most SMs idle while a handful stream all of B;
  // halve the tile width (down to 64) while the tiles still fit half the SMs.
  int acc_cols = sgl::kAccCols;
  if (s.acc_cols > 0 && s.form == SGL_FORM_MATMUL && cfg.cta_group == 1 && !s.b_kmajor) {
    acc_cols = s.acc_cols;   // the caller's plan (split-K summed in clusters)
  } else if (s.form == SGL_FORM_MATMUL && cfg.cta_group == 1 && !s.b_kmajor && s.splits == 1 &&
      s.reduce_rows == 0) {
    while (acc_cols > 64 && tiles_m * ((s.N + acc_cols - 1) / acc_cols) * 2 <= info->sm_count)
      acc_cols /= 2;
  }
  const int tile_cols = s.form == SGL_FORM_MATMUL ? acc_cols : v.out_cols;
  const int64_t tiles_n = (s.N + tile_cols - 1) / tile_cols;
  const int64_t units = tiles_m * tiles_n * s.splits;
  if (units > 0x7fffffffll) return fail(SGL_ERR_BAD_SHAPE, "too many tiles");

  cudaError_t e;
  int rc_ready = prepare_variant(info, v, vi, cfg.cta_group);
  if (rc_ready) return rc_ready;
  // Split-K summed in the cluster: the K ranges of a tile are the CTAs of one cluster, every
  // unit has its own CTA, all clusters fit at once, and the ring holds a partial tile.
  bool cluster_sum = false;
  const bool form_splits = s.form == SGL_FORM_MATMUL ||
                           (s.form == SGL_FORM_FUSED_SWIGLU && !wide && !s.b_kmajor &&
                            s.n_dst == 1 && s.peer_mode == 0) ||
                           (s.form == SGL_FORM_SILU_MUL && s.up_raw && s.n_dst == 1);
  if (s.sum_out && form_splits && cfg.cta_group == 1 && s.splits >= 2 &&
      s.splits <= 16 && cfg.max_ctas == 0 && splitk_cluster_sum_enabled() &&
      ring_holds_partial_tile(v, cfg.stages)) {
    cluster_sum = tiles_m * tiles_n <= k_clusters(info, v, vi, s.splits, smem);
  }
  if (s.summed) *s.summed = cluster_sum;
  if (s.cluster_only && !cluster_sum) return kClustersNotPlaced;

  int64_t clusters = info->max_clusters[vi];
  if (cfg.max_ctas > 0 && cfg.max_ctas / cfg.cta_group < clusters)
    clusters = cfg.max_ctas / cfg.cta_group;
  if (clusters < 1) clusters = 1;
  if (units < clusters) clusters = units;
  if (cluster_sum) clusters = units;   // one unit per CTA

  sgl::KernelParams p;
  p.M = static_cast<int>(s.M);
  p.N = static_cast<int>(s.N);
  p.K = static_cast<int>(s.K);
  p.b_col0 = static_cast<int>(s.col0);
  p.b_col1 = static_cast<int>(s.col1);
  p.tiles_m = static_cast<int>(tiles_m);
  p.tiles_n = static_cast<int>(tiles_n);
  p.group_m = cfg.group_m;
  p.group_n = cfg.group_n;
  p.stages = cfg.stages;
  p.l2_hints = cfg.l2_hints;
  p.n_dst = s.n_dst;
  p.a_mnmajor = s.a_mnmajor;
  p.b_kmajor = s.b_kmajor;
  p.reduce_rows = s.reduce_rows;
  p.reduce_add = s.reduce_add;
  p.acc_cols = acc_cols;
  p.out_f32 = s.out_f32;
  p.splits = s.splits;
  p.k_per_split = s.k_per_split;
  p.slot_rows = s.slot_rows;
  p.a_rows = s.a_rows;
  p.peer_mode = s.peer_mode;
  p.n_peer = s.n_peer;
  p.peer_ld = s.peer_ld;
  for (int d = 0; d < sgl::kMaxDst; ++d)
    p.peer_ptr[d] = reinterpret_cast<unsigned long long>(s.peer_ptr[d]);
  p.m_shift = 0;
  if (s.reduce_rows > 0 && s.first_dst > 0) {
    // start at the first tile row owned by destination first_dst
    p.m_shift = static_cast<int>(
        (static_cast<int64_t>(s.first_dst) * s.reduce_rows / rows_per_tile) % tiles_m);
  }
  p.wait_limit_ns = g_wait_limit_ns.load();
  p.cluster_sum = cluster_sum ? 1 + 2 * g_debug_missing_arrivals.load() : 0;
  p.sum_out = reinterpret_cast<unsigned long long>(s.sum_out);
  p.sum_ld = s.sum_ld;
  p.up_raw = reinterpret_cast<unsigned long long>(s.up_raw);
  p.up_ld = s.up_ld;

  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(static_cast<unsigned>(clusters * cfg.cta_group), 1, 1);
  lc.blockDim = dim3(sgl::kNumThreads, 1, 1);
  lc.dynamicSmemBytes = static_cast<size_t>(smem);
  lc.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = static_cast<unsigned>(cluster_sum ? s.splits : cfg.cta_group);
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  // the kernel orders itself behind its predecessor with griddepcontrol.wait, so its set-up
  // may overlap the predecessor's tail
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attrs;
  lc.numAttrs = 2;
  char label[160];
  if (log_enabled() || nvtx_enabled()) {
    snprintf(label, sizeof(label),
             "sgl %s %lldx%lldx%lld cta_group=%d block_k=%d stages=%d group_m=%d group_n=%d "
             "wide=%d splits=%d%s n_dst=%d grid=%lld smem=%d",
             form_name(s.form), static_cast<long long>(s.M), static_cast<long long>(s.N),
             static_cast<long long>(s.K), cfg.cta_group, cfg.block_k, cfg.stages, cfg.group_m,
             cfg.group_n, wide, s.splits, cluster_sum ? " (summed in the cluster)" : "", s.n_dst,
             static_cast<long long>(clusters * cfg.cta_group), smem);
    if (log_enabled()) fprintf(stderr, "[libswiglu_b200] launch %s\n", label);
    if (nvtx_enabled()) nvtxRangePushA(label);
  }
  e = cudaLaunchKernelEx(&lc, v.fn, *s.x, *s.w, *s.up, *s.out, p);
  if (nvtx_enabled()) nvtxRangePop();
  if (e != cudaSuccess && cluster_sum) {
    // The driver would not place clusters of this size after all (the occupancy query said it
    // could): remember that for this variant and size and take the two-kernel form instead.
    cudaGetLastError();
    {
      std::lock_guard<std::mutex> lock(g_dev_mutex);
      info->max_k_clusters[vi][s.splits] = -1;
    }
    return launch(s, cfg, info, stream);
  }
  if (e != cudaSuccess) return fail_cuda(e, "cudaLaunchKernelEx");
  g_launches.fetch_add(1);
  return SGL_OK;
}

// A short, deep activation-form problem with few tiles (the gate/up stage of a narrow FFN at
// decode batch sizes) under the library's own configuration: cut K into as many ranges as still
// form clusters that all fit at once; each CTA sums its share of the tile and applies the
// activation.  Every range then loads 1/n of what the whole-K tile loads.  Returns
// kClustersNotPlaced if nothing was launched (the caller then launches whole-K tiles).
int launch_in_clusters_if_narrow(LaunchSpec ks, const sgl_config& c, DeviceInfo* info,
                                 void* stream, void* out, int64_t ld_out) {
  if (ks.M > sgl::kBlockM || c.cta_group != 1 || c.wide || ks.K < 4096 || c.max_ctas != 0 ||
      !splitk_cluster_sum_enabled())
    return kClustersNotPlaced;
  const Variant& v = variant(ks.form, c.cta_group, c.block_k, 0);
  const int vi = variant_index(ks.form, c.cta_group, c.block_k, 0);
  int rc;
  if ((rc = prepare_variant(info, v, vi, c.cta_group))) return rc;
  if (!ring_holds_partial_tile(v, c.stages)) return kClustersNotPlaced;
  const int64_t tiles = (ks.N + v.out_cols - 1) / v.out_cols;
  for (int n = 8; n >= 2; --n) {
    int64_t per = (ks.K + n - 1) / n;
    per = (per + 127) / 128 * 128;
    if ((ks.K + per - 1) / per != n || per < 512) continue;
    if (tiles > k_clusters(info, v, vi, n, v.smem_bytes(c.stages))) continue;
    ks.splits = n;
    ks.k_per_split = static_cast<int>(per);
    ks.sum_out = out;
    ks.sum_ld = ld_out;
    ks.cluster_only = true;
    return launch(ks, c, info, stream);
  }
  return kClustersNotPlaced;
}

int check_device(DeviceInfo** info) {
  int dev = 0;
  int rc = device_info(&dev, info);
  if (rc != SGL_OK) return rc;
  // The driver entry point used for the tensor maps needs a context bound to THIS host
  // thread; a thread that has only inherited the process-wide current device has none yet.
  thread_local int bound_device = -1;
  if (bound_device != dev) {
    cudaError_t e = cudaSetDevice(dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
    bound_device = dev;
  }
  if ((*info)->cc / 10 != 10)
    return fail(SGL_ERR_UNSUPPORTED_DEVICE,
                "device %d has compute capability %d.%d; this library is built for sm_100a only",
                dev, (*info)->cc / 10, (*info)->cc % 10);
  return SGL_OK;
}

}  // namespace

extern "C" {

int sgl_matmul_silu_mul(const void* x, const void* w_gate, const void* up, void* h, int64_t M,
                        int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldup, int64_t ldh,
                        const sgl_config* cfg, void* stream) {
  int rc;
  if ((rc = validate_ptr(x, "x")) || (rc = validate_ptr(w_gate, "w_gate")) ||
      (rc = validate_ptr(up, "up")) || (rc = validate_ptr(h, "h")))
    return rc;
  if ((rc = validate_shape(M, N, K))) return rc;
  if ((rc = validate_ld(ldx, K, "ldx")) || (rc = validate_ld(ldw, N, "ldw")) ||
      (rc = validate_ld(ldup, N, "ldup")) || (rc = validate_ld(ldh, N, "ldh")))
    return rc;
  sgl_config c;
  if ((rc = resolve_config(SGL_FORM_SILU_MUL, cfg, M, &c))) return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;

  CUtensorMap tx, tw, tup;
  sgl::OutMaps th;
  std::memset(&th, 0, sizeof(th));
  if ((rc = make_map(&tx, x, M, K, ldx, a_box_rows(M, c.cta_group), 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     "x")) ||
      (rc = make_map(&tw, w_gate, K, N, ldw, c.block_k, 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     "w_gate")) ||
      (rc = make_map(&tup, up, M, N, ldup, 32, 64, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "up")) ||
      (rc = make_map(&th.m[0], h, M, N, ldh, 32, 64, CU_TENSOR_MAP_L2_PROMOTION_NONE, "h")))
    return rc;
  LaunchSpec spec;
  spec.form = SGL_FORM_SILU_MUL;
  spec.x = &tx;
  spec.w = &tw;
  spec.up = &tup;
  spec.out = &th;
  spec.M = M;
  spec.N = N;
  spec.K = K;
  spec.a_rows = a_box_rows(M, c.cta_group);
  if (!cfg) {
    LaunchSpec ks = spec;
    ks.up_raw = up;
    ks.up_ld = ldup;
    rc = launch_in_clusters_if_narrow(ks, c, info, stream, h, ldh);
    if (rc != kClustersNotPlaced) return rc;
  }
  return launch(spec, c, info, stream);
}

struct PeerStores {
  int mode = 0;                 // 1 = ordinary stores to n raw pointers, 2 = one multicast pointer
  int n = 0;
  void* const* ptrs = nullptr;
};

static int fused_swiglu_impl(const void* x, const void* w, int w_is_nk, void* const* h_dsts,
                            int n_dsts, void* factors, int64_t ldf, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                            int64_t ldh, int64_t up_col0, int64_t gate_col0,
                            const sgl_config* cfg, void* stream,
                            const PeerStores* peers = nullptr) {
  int rc;
  if ((rc = validate_ptr(x, "x")) || (rc = validate_ptr(w, "w"))) return rc;
  for (int d = 0; d < n_dsts; ++d) {
    if ((rc = validate_ptr(h_dsts[d], "h"))) return rc;
  }
  if ((rc = validate_shape(M, N, K))) return rc;
  if (up_col0 < 0 || gate_col0 < 0)
    return fail(SGL_ERR_BAD_ARGUMENT, "up_col0=%lld and gate_col0=%lld must be >= 0",
                static_cast<long long>(up_col0), static_cast<long long>(gate_col0));
  if (up_col0 % 8 != 0 || gate_col0 % 8 != 0)
    return fail(SGL_ERR_MISALIGNED,
                "up_col0=%lld and gate_col0=%lld must be multiples of 8 columns (16 bytes)",
                static_cast<long long>(up_col0), static_cast<long long>(gate_col0));
  // [k, n] storage: ldw is the pitch of a row of all columns; [n, k] storage: of one
  // feature's K weights, and the tensor has (max offset + N) rows.
  const int64_t w_span = (up_col0 > gate_col0 ? up_col0 : gate_col0) + N;
  if ((rc = validate_ld(ldx, K, "ldx")) ||
      (rc = validate_ld(ldw, w_is_nk ? K : w_span, "ldw")) || (rc = validate_ld(ldh, N, "ldh")))
    return rc;
  const int form = factors ? SGL_FORM_FUSED_SWIGLU_SAVE : SGL_FORM_FUSED_SWIGLU;
  if (factors) {
    if ((rc = validate_ptr(factors, "factors")) || (rc = validate_ld(ldf, 2 * N, "ldf")))
      return rc;
  }
  sgl_config c;
  if ((rc = resolve_config(form, cfg, M, &c))) return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;

  CUtensorMap tx, tw;
  sgl::OutMaps th;
  std::memset(&th, 0, sizeof(th));
  if ((rc = make_map(&tx, x, M, K, ldx, a_box_rows(M, c.cta_group), 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     "x")) ||
      (rc = w_is_nk ? make_map(&tw, w, w_span, K, ldw, 128, 64,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "w")
                    : make_map(&tw, w, K, ldw, ldw, c.block_k, 64,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "w")))
    return rc;
  for (int d = 0; d < n_dsts; ++d) {
    // the side-store form stages 32-column half chunks (64-byte rows, 64B swizzle)
    if ((rc = factors ? make_map(&th.m[d], h_dsts[d], M, N, ldh, 32, 32,
                                 CU_TENSOR_MAP_L2_PROMOTION_NONE, "h", false,
                                 CU_TENSOR_MAP_SWIZZLE_64B)
                      : make_map(&th.m[d], h_dsts[d], M, N, ldh, 32, 64,
                                 CU_TENSOR_MAP_L2_PROMOTION_NONE, "h")))
      return rc;
  }
  if (factors) {
    // m[1]: the silu block, columns [0, N); m[2]: the gate-factor block, columns [N, 2N).
    // Separate maps so a ragged last tile is clipped at N, not at 2N.
    char* f = static_cast<char*>(factors);
    if ((rc = make_map(&th.m[1], f, M, N, ldf, 32, 32, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       "factors", false, CU_TENSOR_MAP_SWIZZLE_64B)) ||
        (rc = make_map(&th.m[2], f + 2 * N, M, N, ldf, 32, 32, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       "factors", false, CU_TENSOR_MAP_SWIZZLE_64B)))
      return rc;
    n_dsts = 3;
  }
  LaunchSpec spec;
  spec.form = form;
  spec.x = &tx;
  spec.w = &tw;
  spec.up = &th.m[0];
  spec.out = &th;
  spec.M = M;
  spec.N = N;
  spec.K = K;
  spec.col0 = up_col0;
  spec.col1 = gate_col0;
  spec.n_dst = n_dsts;
  spec.b_kmajor = w_is_nk;
  spec.a_rows = a_box_rows(M, c.cta_group);
  if (peers && peers->mode != 0) {
    for (int d = 0; d < peers->n; ++d) {
      if ((rc = validate_ptr(peers->ptrs[d], "peer destination"))) return rc;
      spec.peer_ptr[d] = peers->ptrs[d];
    }
    spec.peer_mode = peers->mode;
    spec.n_peer = peers->n;
    spec.peer_ld = ldh;
  }
  if (!cfg && form == SGL_FORM_FUSED_SWIGLU && !w_is_nk && n_dsts == 1 && !peers) {
    rc = launch_in_clusters_if_narrow(spec, c, info, stream, h_dsts[0], ldh);
    if (rc != kClustersNotPlaced) return rc;
  }
  return launch(spec, c, info, stream);
}

int sgl_matmul_fused_swiglu(const void* x, const void* w, void* h, int64_t M, int64_t N, int64_t K,
                            int64_t ldx, int64_t ldw, int64_t ldh, int64_t up_col0,
                            int64_t gate_col0, const sgl_config* cfg, void* stream) {
  void* dst[1] = {h};
  return fused_swiglu_impl(x, w, 0, dst, 1, nullptr, 0, M, N, K, ldx, ldw, ldh, up_col0, gate_col0, cfg,
                           stream);
}

int sgl_matmul_fused_swiglu_nk(const void* x, const void* w_nk, void* h, int64_t M, int64_t N,
                               int64_t K, int64_t ldx, int64_t ldw, int64_t ldh, int64_t up_row0,
                               int64_t gate_row0, const sgl_config* cfg, void* stream) {
  void* dst[1] = {h};
  return fused_swiglu_impl(x, w_nk, 1, dst, 1, nullptr, 0, M, N, K, ldx, ldw, ldh, up_row0, gate_row0, cfg,
                           stream);
}

int sgl_matmul_fused_swiglu_save_factors(const void* x, const void* w, void* h, void* factors,
                                         int64_t M, int64_t N, int64_t K, int64_t ldx,
                                         int64_t ldw, int64_t ldh, int64_t ldf, int64_t up_col0,
                                         int64_t gate_col0, const sgl_config* cfg,
                                         void* stream) {
  if (!factors) return fail(SGL_ERR_NULL_POINTER, "factors is NULL");
  void* dst[1] = {h};
  return fused_swiglu_impl(x, w, 0, dst, 1, factors, ldf, M, N, K, ldx, ldw, ldh, up_col0,
                           gate_col0, cfg, stream);
}

int sgl_swiglu_grad_preact(const void* dy, const void* factors, void* grad_preact, int64_t M,
                           int64_t N, int64_t lddy, int64_t ldf, int64_t ldo, void* stream) {
  int rc;
  if ((rc = validate_ptr(dy, "dy")) || (rc = validate_ptr(factors, "factors")) ||
      (rc = validate_ptr(grad_preact, "grad_preact")))
    return rc;
  if ((rc = validate_shape(M, N, 8))) return rc;
  if ((rc = validate_ld(lddy, N, "lddy")) || (rc = validate_ld(ldf, 2 * N, "ldf")) ||
      (rc = validate_ld(ldo, 2 * N, "ldo")))
    return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;
  const int64_t vecs = M * (N / 8);
  int64_t blocks = (vecs + 255) / 256;
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 8;   // 8 resident CTAs of 256 per SM
  if (blocks > cap) blocks = cap;
  sgl::grad_preact_kernel<<<static_cast<unsigned>(blocks), 256, 0,
                            static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(dy), static_cast<const uint4*>(factors),
      static_cast<uint4*>(grad_preact), static_cast<int>(M), static_cast<int>(N / 8), lddy / 8,
      ldf / 8, ldo / 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "grad_preact_kernel launch");
  g_launches.fetch_add(1);
  return SGL_OK;
}

namespace {

// Split-K plan: K ranges are multiples of 128 (both BLOCK_K values divide it) and every
// range is non-empty; slots are padded to whole 32-row store boxes.
struct SplitPlan {
  int splits;
  int k_per_split;
  int slot_rows;
  int64_t scratch_bytes;
  bool automatic;          // the caller left the number of ranges to the library
};

int plan_splitk(int64_t M, int64_t N, int64_t K, int splits, int sm_count, SplitPlan* out,
                int64_t max_scratch = 0) {
  if (splits < 0 || splits > 64)
    return fail(SGL_ERR_BAD_ARGUMENT, "splits=%d outside [0, 64] (0 = choose)", splits);
  const bool automatic = splits == 0;
  out->automatic = automatic;
  if (automatic) {
    // As many K ranges as fill ONE wave of workers (a second, partly filled wave would cost
    // as much as a full one), at least 512 of K each.  Up to 128 rows the default
    // configuration runs one CTA per 128-row tile, above that a CTA pair per 256-row tile.
    const bool single = M <= 128;
    const int64_t workers = single ? sm_count : sm_count / 2;
    const int64_t row_tile = single ? 128 : 256;
    const int64_t tiles = ((M + row_tile - 1) / row_tile) * ((N + 255) / 256);
    int64_t want = workers / tiles;
    const int64_t by_k = K / 512 > 0 ? K / 512 : 1;
    if (want > by_k) want = by_k;
    if (want > 16) want = 16;
    splits = want < 1 ? 1 : static_cast<int>(want);
  }
  out->slot_rows = static_cast<int>((M + 31) / 32 * 32);
  for (;;) {
    int64_t per = (K + splits - 1) / splits;
    per = (per + 127) / 128 * 128;
    out->k_per_split = static_cast<int>(per);
    out->splits = static_cast<int>((K + per - 1) / per);
    out->scratch_bytes = static_cast<int64_t>(out->splits) * out->slot_rows * N * 4;
    // an automatic choice gives way to a fixed scratch size; an explicit one does not
    if (!automatic || max_scratch <= 0 || out->scratch_bytes <= max_scratch || splits <= 1) break;
    --splits;
  }
  return SGL_OK;
}

// Split-K plan whose K ranges can be summed in thread-block clusters, for a problem of one or
// two rows of single-CTA tiles: tile width (whole 64-column slabs of b), number of ranges and
// K extent of a range.  Clusters have to be placed whole, so fewer of the larger ones fit; only
// plans whose clusters all fit at once are considered.  ctas = 0: no such plan.
struct ClusterPlan {
  int cols = 0, ranges = 0, k_per_range = 0;
  int64_t ctas = 0;
};

// The choice itself, given how many clusters of n CTAs fit at once (fit[n], n = 2..8).  These
// problems are bound by what one SM can pull in, so the plan whose CTAs each load the fewest
// operand bytes wins: K extent of a range x (rows of a + columns of b); a_rows = rows of a
// that a tile loads.  On a tie the wider tile, which comes first.
void choose_cluster_plan(int64_t tiles_m, int a_rows, int64_t N, int64_t K, const int* fit,
                         ClusterPlan* out) {
  *out = ClusterPlan();
  int64_t best = 0;
  for (int cols = 256; cols >= 64; cols -= 64) {   // whole 64-column slabs of b
    const int64_t tiles = tiles_m * ((N + cols - 1) / cols);
    for (int n = 8; n >= 2; --n) {
      int64_t per = (K + n - 1) / n;
      per = (per + 127) / 128 * 128;
      const int ranges = static_cast<int>((K + per - 1) / per);
      if (ranges != n || per < 512) continue;   // empty or very short ranges
      if (tiles > fit[n]) continue;
      const int64_t load = per * (a_rows + cols);
      if (best == 0 || load < best) {
        best = load;
        out->ctas = tiles * n;
        out->cols = cols;
        out->ranges = n;
        out->k_per_range = static_cast<int>(per);
      }
      break;   // fewer ranges of the same width only make every range longer
    }
  }
}

int plan_cluster_splitk(DeviceInfo* info, const sgl_config& cf, int64_t tiles_m, int a_rows,
                        int64_t N, int64_t K, ClusterPlan* out) {
  *out = ClusterPlan();
  if (cf.cta_group != 1 || cf.max_ctas != 0 || !splitk_cluster_sum_enabled()) return SGL_OK;
  const Variant& v = variant(SGL_FORM_MATMUL, cf.cta_group, cf.block_k, 0);
  const int vi = variant_index(SGL_FORM_MATMUL, cf.cta_group, cf.block_k, 0);
  // A decode loop asks for the same problem over and over: remember the last answer.
  struct Memo {
    const DeviceInfo* info = nullptr;
    int vi = -1, stages = 0;
    int64_t tiles_m = 0, N = 0, K = 0;
    int a_rows = 0;
    ClusterPlan plan;
  };
  thread_local Memo memo;
  if (memo.info == info && memo.vi == vi && memo.stages == cf.stages &&
      memo.tiles_m == tiles_m && memo.a_rows == a_rows && memo.N == N && memo.K == K) {
    *out = memo.plan;
    return SGL_OK;
  }
  int rc;
  if ((rc = prepare_variant(info, v, vi, cf.cta_group))) return rc;
  if (!ring_holds_partial_tile(v, cf.stages)) return SGL_OK;
  const int smem = v.smem_bytes(cf.stages);
  int fit[9] = {};
  for (int n = 2; n <= 8; ++n) fit[n] = k_clusters(info, v, vi, n, smem);
  choose_cluster_plan(tiles_m, a_rows, N, K, fit, out);
  memo.info = info;
  memo.vi = vi;
  memo.stages = cf.stages;
  memo.tiles_m = tiles_m;
  memo.a_rows = a_rows;
  memo.N = N;
  memo.K = K;
  memo.plan = *out;
  return SGL_OK;
}

// a @ b through `plan.splits` fp32 partial tiles in `scratch`, then the fp32 slot sum into c.
int matmul_splitk_run(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, const SplitPlan& plan,
                      void* scratch, const sgl_config* cfg, DeviceInfo* info, void* stream) {
  int rc;
  sgl_config cf;
  if ((rc = resolve_config(SGL_FORM_MATMUL, cfg, M, &cf))) return rc;
  CUtensorMap ta, tb;
  sgl::OutMaps tc;
  std::memset(&tc, 0, sizeof(tc));
  if ((rc = make_map(&ta, a, M, K, lda, a_box_rows(M, cf.cta_group), 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     "a")) ||
      (rc = make_map(&tb, b, K, N, ldb, cf.block_k, 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     "b")) ||
      (rc = make_map(&tc.m[0], scratch, static_cast<int64_t>(plan.splits) * plan.slot_rows, N, N,
                     32, 32, CU_TENSOR_MAP_L2_PROMOTION_NONE, "scratch", true)))
    return rc;
  LaunchSpec spec;
  spec.form = SGL_FORM_MATMUL;
  spec.x = &ta;
  spec.w = &tb;
  spec.up = &tc.m[0];
  spec.out = &tc;
  spec.M = M;
  spec.N = N;
  spec.K = K;
  spec.out_f32 = 1;
  spec.splits = plan.splits;
  spec.k_per_split = plan.k_per_split;
  spec.slot_rows = plan.slot_rows;
  spec.a_rows = a_box_rows(M, cf.cta_group);
  // Left to choose, and on single-CTA tiles: prefer a plan whose K ranges can meet in a
  // thread-block cluster (no scratch traffic, no second kernel).
  if (plan.automatic && cf.cta_group == 1 && M <= sgl::kBlockM) {
    ClusterPlan cp;
    if ((rc = plan_cluster_splitk(info, cf, 1, a_box_rows(M, 1), N, K, &cp))) return rc;
    if (cp.ctas > 0) {
      spec.acc_cols = cp.cols;
      spec.splits = cp.ranges;
      spec.k_per_split = cp.k_per_range;
    }
  }
  bool summed = false;
  spec.sum_out = c;
  spec.sum_ld = ldc;
  spec.summed = &summed;
  if ((rc = launch(spec, cf, info, stream))) return rc;
  if (summed) return SGL_OK;   // the K ranges met in their cluster: c is written
  // (spec.splits <= plan.splits: a plan made for clusters that then could not be launched has
  // fewer ranges than the scratch was sized for)
  const int64_t vecs = M * (N / 8);
  int64_t blocks = (vecs + 255) / 256;
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 8;
  if (blocks > cap) blocks = cap;
  // The slot sum is launched with programmatic stream serialisation: its grid is set up while
  // the GEMM's last tiles still run and waits (griddepcontrol.wait) for the GEMM to finish,
  // which takes the launch gap between the two kernels off a 30 us problem.
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  lc.blockDim = dim3(256, 1, 1);
  lc.dynamicSmemBytes = 0;
  lc.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = pdl;
  lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(
      &lc, sgl::sum_slots_f32_kernel, static_cast<const float4*>(scratch),
      static_cast<uint4*>(c), spec.splits, static_cast<int64_t>(plan.slot_rows) * N / 4,
      static_cast<int>(M), static_cast<int>(N / 8), static_cast<int64_t>(N / 4),
      static_cast<int64_t>(ldc / 8));
  if (e != cudaSuccess) return fail_cuda(e, "sum_slots_f32_kernel launch");
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "sum_slots_f32_kernel launch");
  g_launches.fetch_add(1);
  return SGL_OK;
}

int validate_matmul(const void* a, const void* b, const void* c, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc) {
  int rc;
  if ((rc = validate_ptr(a, "a")) || (rc = validate_ptr(b, "b")) || (rc = validate_ptr(c, "c")))
    return rc;
  if ((rc = validate_shape(M, N, K))) return rc;
  if ((rc = validate_ld(lda, K, "lda")) || (rc = validate_ld(ldb, N, "ldb")) ||
      (rc = validate_ld(ldc, N, "ldc")))
    return rc;
  return SGL_OK;
}

}  // namespace

int64_t sgl_matmul_bf16_splitk_scratch_bytes(int64_t M, int64_t N, int64_t K, int splits) {
  if (validate_shape(M, N, K)) return SGL_ERR_BAD_SHAPE;
  SplitPlan plan;
  // The automatic choice depends on the SM count: the current device's, as the launch will
  // use; where no device can be asked (a host without a GPU) a B200's 148.
  int sm_count = 148;
  int dev = 0;
  DeviceInfo* info = nullptr;
  if (device_info(&dev, &info) == SGL_OK && info->sm_count > 0) sm_count = info->sm_count;
  cudaGetLastError();
  int rc = plan_splitk(M, N, K, splits, sm_count, &plan);
  if (rc) return rc;
  return plan.scratch_bytes;
}

int sgl_matmul_bf16_splitk(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                           int64_t lda, int64_t ldb, int64_t ldc, int splits, void* scratch,
                           int64_t scratch_bytes, const sgl_config* cfg, void* stream) {
  int rc;
  if ((rc = validate_matmul(a, b, c, M, N, K, lda, ldb, ldc))) return rc;
  if ((rc = validate_ptr(scratch, "scratch"))) return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;
  SplitPlan plan;
  if ((rc = plan_splitk(M, N, K, splits, info->sm_count, &plan))) return rc;
  if (scratch_bytes < plan.scratch_bytes)
    return fail(SGL_ERR_BAD_ARGUMENT, "scratch holds %lld bytes, %lld needed (%d K ranges)",
                static_cast<long long>(scratch_bytes), static_cast<long long>(plan.scratch_bytes),
                plan.splits);
  return matmul_splitk_run(a, b, c, M, N, K, lda, ldb, ldc, plan, scratch, cfg, info, stream);
}

int sgl_splitk_cluster_plan(int64_t M, int64_t N, int64_t K, const int* clusters_that_fit,
                            int* tile_cols, int* ranges, int* k_per_range) {
  if (!clusters_that_fit || !tile_cols || !ranges || !k_per_range)
    return fail(SGL_ERR_NULL_POINTER, "NULL argument");
  if (M < 1 || M > 2 * sgl::kBlockM)
    return fail(SGL_ERR_BAD_SHAPE, "M=%lld: the cluster plan covers 1 to 256 rows",
                static_cast<long long>(M));
  int rc;
  if ((rc = validate_shape(M, N, K))) return rc;
  ClusterPlan cp;
  choose_cluster_plan((M + sgl::kBlockM - 1) / sgl::kBlockM,
                      M > sgl::kBlockM ? sgl::kBlockM : a_box_rows(M, 1), N, K,
                      clusters_that_fit, &cp);
  *tile_cols = cp.cols;
  *ranges = cp.ranges;
  *k_per_range = cp.k_per_range;
  return static_cast<int>(cp.ctas);
}

int sgl_set_splitk_cluster_sum(int enabled) {
  const bool before = splitk_cluster_sum_enabled();
  g_splitk_cluster_sum.store(enabled ? 1 : 0);
  return before ? 1 : 0;
}

// ---------------------------------------------------------------- no-allocation split-K
//
// Scratch for sgl_matmul_bf16_splitk_static.  Every GPU that loads this library carries
// these 8 MiB until the process exits.  In HOST code the name below is only a stand-in for
// the symbol, not a device address: the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
constexpr int64_t kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) unsigned char g_splitk_static_scratch[kStaticScratchBytes];

namespace {
std::mutex g_static_scratch_mutex;
std::map<int, void*> g_static_scratch_ptr;   // device ordinal -> device address of the array

// Device address of the static scratch on the CURRENT device (resolved on first use).
int static_scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  auto it = g_static_scratch_ptr.find(dev);
  if (it == g_static_scratch_ptr.end()) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_splitk_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static split-K scratch)");
    if (!ptr) return fail(SGL_ERR_NULL_POINTER, "static split-K scratch resolved to NULL");
    it = g_static_scratch_ptr.emplace(dev, ptr).first;
  }
  *out = it->second;
  return SGL_OK;
}
}  // namespace

int sgl_matmul_bf16_splitk_static(const void* a, const void* b, void* c, int64_t M, int64_t N,
                                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int splits,
                                  const sgl_config* cfg, void* stream) {
  int rc;
  if ((rc = validate_matmul(a, b, c, M, N, K, lda, ldb, ldc))) return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;
  SplitPlan plan;
  if ((rc = plan_splitk(M, N, K, splits, info->sm_count, &plan, kStaticScratchBytes))) return rc;
  if (plan.scratch_bytes > kStaticScratchBytes)
    return fail(SGL_ERR_BAD_ARGUMENT,
                "this problem needs %lld bytes of split-K scratch (%d K ranges x %d rows x %lld "
                "columns x 4), the built-in scratch holds %lld: use fewer splits or "
                "sgl_matmul_bf16_splitk with your own scratch",
                static_cast<long long>(plan.scratch_bytes), plan.splits, plan.slot_rows,
                static_cast<long long>(N), static_cast<long long>(kStaticScratchBytes));
  void* scratch = nullptr;
  if ((rc = static_scratch_for_current_device(&scratch))) return rc;
  return matmul_splitk_run(a, b, c, M, N, K, lda, ldb, ldc, plan, scratch, cfg, info, stream);
}

int sgl_sum_bf16_slots(const void* slots, int n_slots, int64_t slot_stride, void* out,
                       int64_t rows, int64_t cols, int64_t lds, int64_t ldo, void* stream) {
  int rc;
  if ((rc = validate_ptr(slots, "slots")) || (rc = validate_ptr(out, "out"))) return rc;
  if (n_slots < 1 || n_slots > 64)
    return fail(SGL_ERR_BAD_ARGUMENT, "n_slots=%d outside [1, 64]", n_slots);
  if ((rc = validate_shape(rows, cols, 8))) return rc;
  if ((rc = validate_ld(lds, cols, "lds")) || (rc = validate_ld(ldo, cols, "ldo"))) return rc;
  if (slot_stride % 8 != 0 || slot_stride < (rows - 1) * lds + cols)
    return fail(SGL_ERR_BAD_STRIDE, "slot_stride=%lld too small or not a multiple of 8",
                static_cast<long long>(slot_stride));
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;
  const int64_t vecs = rows * (cols / 8);
  int64_t blocks = (vecs + 255) / 256;
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 8;
  if (blocks > cap) blocks = cap;
  sgl::sum_slots_kernel<<<static_cast<unsigned>(blocks), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(slots), static_cast<uint4*>(out), n_slots, slot_stride / 8,
      static_cast<int>(rows), static_cast<int>(cols / 8), lds / 8, ldo / 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "sum_slots_kernel launch");
  g_launches.fetch_add(1);
  return SGL_OK;
}

int sgl_matmul_fused_swiglu_multi_dst(const void* x, const void* w, void* const* h_dsts,
                                      int n_dsts, int64_t M, int64_t N, int64_t K, int64_t ldx,
                                      int64_t ldw, int64_t ldh, int64_t up_col0,
                                      int64_t gate_col0, const sgl_config* cfg, void* stream) {
  if (!h_dsts) return fail(SGL_ERR_NULL_POINTER, "h_dsts is NULL");
  if (n_dsts < 1 || n_dsts > sgl::kMaxDst)
    return fail(SGL_ERR_BAD_ARGUMENT, "n_dsts=%d outside [1, %d]", n_dsts, sgl::kMaxDst);
  return fused_swiglu_impl(x, w, 0, h_dsts, n_dsts, nullptr, 0, M, N, K, ldx, ldw, ldh, up_col0, gate_col0,
                           cfg, stream);
}

int sgl_matmul_fused_swiglu_gather(const void* x, const void* w, void* h_local,
                                   void* const* h_peers, int n_peers, void* h_multicast,
                                   int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                                   int64_t ldh, int64_t up_col0, int64_t gate_col0,
                                   const sgl_config* cfg, void* stream) {
  if (n_peers < 0 || n_peers > sgl::kMaxDst)
    return fail(SGL_ERR_BAD_ARGUMENT, "n_peers=%d outside [0, %d]", n_peers, sgl::kMaxDst);
  if (n_peers > 0 && !h_peers && !h_multicast)
    return fail(SGL_ERR_NULL_POINTER, "h_peers is NULL");
  void* dst[1] = {h_local};
  PeerStores ps;
  void* mc[1] = {h_multicast};
  if (h_multicast) {
    ps.mode = 2;
    ps.n = 1;
    ps.ptrs = mc;
  } else if (n_peers > 0) {
    ps.mode = 1;
    ps.n = n_peers;
    ps.ptrs = h_peers;
  }
  return fused_swiglu_impl(x, w, 0, dst, 1, nullptr, 0, M, N, K, ldx, ldw, ldh, up_col0,
                           gate_col0, cfg, stream, &ps);
}

static int matmul_impl(const void* a, const void* b, void* const* dsts, int n_dsts,
                       int64_t reduce_rows, int dst_is_f32, int accumulate, int first_dst,
                       int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, const sgl_config* cfg,
                       void* stream) {
  int rc;
  if ((rc = validate_ptr(a, "a")) || (rc = validate_ptr(b, "b"))) return rc;
  for (int d = 0; d < n_dsts; ++d) {
    if ((rc = validate_ptr(dsts[d], "c"))) return rc;
  }
  if ((rc = validate_shape(M, N, K))) return rc;
  if ((rc = validate_ld(lda, K, "lda")) || (rc = validate_ld(ldb, N, "ldb")) ||
      (rc = validate_ld(ldc, N, "ldc")))
    return rc;
  if (reduce_rows < 0 || (reduce_rows > 0 && reduce_rows % 32 != 0))
    return fail(SGL_ERR_BAD_ARGUMENT, "rows_per_dst=%lld must be a positive multiple of 32",
                static_cast<long long>(reduce_rows));
  if (reduce_rows > 0 && reduce_rows * n_dsts < M)
    return fail(SGL_ERR_BAD_ARGUMENT, "%d destinations of %lld rows do not cover M=%lld", n_dsts,
                static_cast<long long>(reduce_rows), static_cast<long long>(M));
  sgl_config c;
  if ((rc = resolve_config(SGL_FORM_MATMUL, cfg, M, &c))) return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;

  CUtensorMap ta, tb;
  sgl::OutMaps tc;
  std::memset(&tc, 0, sizeof(tc));
  if ((rc = make_map(&ta, a, M, K, lda, a_box_rows(M, c.cta_group), 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     "a")) ||
      (rc = make_map(&tb, b, K, N, ldb, c.block_k, 64, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "b")))
    return rc;
  const bool f32 = dst_is_f32 != 0;
  for (int d = 0; d < n_dsts; ++d) {
    int64_t rows = M;
    if (reduce_rows > 0) {
      rows = M - d * reduce_rows;
      if (rows > reduce_rows) rows = reduce_rows;
      if (rows < 1) rows = 1;   // a destination past the end is never addressed
    }
    if ((rc = make_map(&tc.m[d], dsts[d], rows, N, ldc, 32, f32 ? 32 : 64,
                       CU_TENSOR_MAP_L2_PROMOTION_NONE, "c", f32)))
      return rc;
  }
  LaunchSpec spec;
  spec.form = SGL_FORM_MATMUL;
  spec.x = &ta;
  spec.w = &tb;
  spec.up = &tc.m[0];
  spec.out = &tc;
  spec.M = M;
  spec.N = N;
  spec.K = K;
  spec.n_dst = n_dsts;
  spec.out_f32 = f32 ? 1 : 0;
  spec.reduce_rows = static_cast<int>(reduce_rows);
  spec.reduce_add = accumulate;
  spec.first_dst = first_dst;
  spec.a_rows = a_box_rows(M, c.cta_group);
  return launch(spec, c, info, stream);
}

int sgl_matmul_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, const sgl_config* cfg, void* stream) {
  return sgl_matmul_bf16_ex(a, b, c, M, N, K, lda, ldb, ldc, 0, 0, cfg, stream);
}

int sgl_matmul_bf16_ex(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, int a_transposed,
                       int b_transposed, const sgl_config* cfg, void* stream) {
  int rc;
  if ((rc = validate_ptr(a, "a")) || (rc = validate_ptr(b, "b")) || (rc = validate_ptr(c, "c")))
    return rc;
  // With a stored [K, M] and b stored [K, N] the reduction index is only a ROW count of both
  // operands: no row pitch depends on it and rows past K read as zero, so any K >= 1 is fine
  // (the weight gradient x^T @ g of a ragged token count).  In every other layout K is the
  // contiguous extent of a row and must keep it 16-byte sized.
  const bool k_is_row_count = a_transposed && !b_transposed;
  if ((rc = validate_shape(M, N, k_is_row_count ? (K + 7) / 8 * 8 : K))) return rc;
  if (a_transposed && M % 8 != 0)
    return fail(SGL_ERR_BAD_SHAPE, "M=%lld must be a multiple of 8 when a is stored [K, M]",
                static_cast<long long>(M));
  if ((rc = validate_ld(lda, a_transposed ? M : K, "lda")) ||
      (rc = validate_ld(ldb, b_transposed ? K : N, "ldb")) || (rc = validate_ld(ldc, N, "ldc")))
    return rc;
  sgl_config cf;
  if ((rc = resolve_config(SGL_FORM_MATMUL, cfg, M, &cf))) return rc;
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;
  CUtensorMap ta, tb;
  sgl::OutMaps tc;
  std::memset(&tc, 0, sizeof(tc));
  if ((rc = a_transposed ? make_map(&ta, a, K, M, lda, cf.block_k, 64,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "a")
                         : make_map(&ta, a, M, K, lda, a_box_rows(M, cf.cta_group), 64,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "a")) ||
      (rc = b_transposed ? make_map(&tb, b, N, K, ldb, 128, 64,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "b")
                         : make_map(&tb, b, K, N, ldb, cf.block_k, 64,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "b")) ||
      (rc = make_map(&tc.m[0], c, M, N, ldc, 32, 64, CU_TENSOR_MAP_L2_PROMOTION_NONE, "c")))
    return rc;
  LaunchSpec spec;
  spec.form = SGL_FORM_MATMUL;
  spec.x = &ta;
  spec.w = &tb;
  spec.up = &tc.m[0];
  spec.out = &tc;
  spec.M = M;
  spec.N = N;
  spec.K = K;
  spec.a_mnmajor = a_transposed ? 1 : 0;
  spec.b_kmajor = b_transposed ? 1 : 0;
  spec.a_rows = a_transposed ? sgl::kBlockM : a_box_rows(M, cf.cta_group);
  // A short, deep problem with the library's own configuration (the down projection at decode
  // batch sizes): cut K into ranges that run as thread-block clusters and sum themselves, if
  // a CTA then has clearly less to load than a CTA of the whole-K grid.  Needs no scratch, so
  // the plain entry point can do it; the result is deterministic, and differs from the whole-K
  // kernel's only in the order of the fp32 additions.
  // (Up to 256 rows - two rows of single-CTA tiles instead of one row of CTA pairs - the same
  // holds: 256 x 14336 x 4096 takes 90 us on 16 whole-K pair tiles.)
  if (!cfg && !a_transposed && !b_transposed && M <= 2 * sgl::kBlockM && K >= 4096) {
    sgl_config cf1;   // the library's configuration for single-CTA tiles
    if ((rc = resolve_config(SGL_FORM_MATMUL, nullptr, sgl::kBlockM, &cf1))) return rc;
    const int64_t tiles_m = (M + sgl::kBlockM - 1) / sgl::kBlockM;
    ClusterPlan cp;
    const int rows_a = tiles_m > 1 ? sgl::kBlockM : a_box_rows(M, 1);
    if ((rc = plan_cluster_splitk(info, cf1, tiles_m, rows_a, N, K, &cp))) return rc;
    // what launch() does for whole-K tiles: CTA pairs on 256 x 256 tiles above 128 rows, else
    // single-CTA tiles narrowed while they fit half the SMs
    int whole_cols = sgl::kAccCols;
    while (tiles_m == 1 && whole_cols > 64 &&
           ((N + whole_cols - 1) / whole_cols) * 2 <= info->sm_count)
      whole_cols /= 2;
    // operand bytes one CTA loads either way (a pair member loads 128 rows of a and half of
    // the pair's 256 columns of b): the cluster plan has to be a quarter lighter to be taken
    const int64_t whole_load = K * (rows_a + (tiles_m > 1 ? whole_cols / 2 : whole_cols));
    const int64_t plan_load = static_cast<int64_t>(cp.k_per_range) * (rows_a + cp.cols);
    if (cp.ctas > 0 && plan_load * 5 <= whole_load * 4) {
      CUtensorMap ta1, tb1;
      if (tiles_m > 1) {
        // operand boxes of the single-CTA configuration
        if ((rc = make_map(&ta1, a, M, K, lda, sgl::kBlockM, 64,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "a")) ||
            (rc = make_map(&tb1, b, K, N, ldb, cf1.block_k, 64,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "b")))
          return rc;
      }
      LaunchSpec ks = spec;
      if (tiles_m > 1) {
        ks.x = &ta1;
        ks.w = &tb1;
        ks.a_rows = sgl::kBlockM;
      }
      ks.acc_cols = cp.cols;
      ks.splits = cp.ranges;
      ks.k_per_split = cp.k_per_range;
      ks.slot_rows = static_cast<int>((M + 31) / 32 * 32);
      ks.sum_out = c;
      ks.sum_ld = ldc;
      ks.cluster_only = true;
      rc = launch(ks, tiles_m > 1 ? cf1 : cf, info, stream);
      if (rc != kClustersNotPlaced) return rc;
    }
  }
  return launch(spec, cf, info, stream);
}

int sgl_matmul_bf16_reduce_scatter(const void* a, const void* b, void* const* dsts, int n_dsts,
                                   int64_t rows_per_dst, int dst_is_f32, int accumulate,
                                   int first_dst, int64_t M, int64_t N,
                                   int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                   const sgl_config* cfg, void* stream) {
  if (!dsts) return fail(SGL_ERR_NULL_POINTER, "dsts is NULL");
  if (n_dsts < 1 || n_dsts > sgl::kMaxDst)
    return fail(SGL_ERR_BAD_ARGUMENT, "n_dsts=%d outside [1, %d]", n_dsts, sgl::kMaxDst);
  if (rows_per_dst < 1) return fail(SGL_ERR_BAD_ARGUMENT, "rows_per_dst must be >= 1");
  if (first_dst < 0 || first_dst >= n_dsts)
    return fail(SGL_ERR_BAD_ARGUMENT, "first_dst=%d outside [0, %d)", first_dst, n_dsts);
  return matmul_impl(a, b, dsts, n_dsts, rows_per_dst, dst_is_f32, accumulate ? 1 : 0, first_dst,
                     M, N, K, lda, ldb, ldc, cfg, stream);
}

int sgl_config_count(int form) {
  if (form < SGL_FORM_SILU_MUL || form > SGL_FORM_FUSED_SWIGLU_SAVE)
    return fail(SGL_ERR_BAD_ARGUMENT, "unknown form %d", form);
  int idx[kTableSize];
  return form_entries(form, idx);
}

int sgl_config_get(int form, int index, sgl_config* out) {
  if (!out) return fail(SGL_ERR_NULL_POINTER, "out is NULL");
  if (form < SGL_FORM_SILU_MUL || form > SGL_FORM_FUSED_SWIGLU_SAVE)
    return fail(SGL_ERR_BAD_ARGUMENT, "unknown form %d", form);
  int idx[kTableSize];
  const int n = form_entries(form, idx);
  if (index < 0 || index >= n)
    return fail(SGL_ERR_BAD_ARGUMENT, "config index %d outside [0, %d)", index, n);
  *out = kTable[idx[index]];
  out->stages = variant(form, out->cta_group, out->block_k).max_stages;
  return SGL_OK;
}

int sgl_config_default(int form, int64_t M, int64_t N, int64_t K, sgl_config* out) {
  if (!out) return fail(SGL_ERR_NULL_POINTER, "out is NULL");
  if (form < SGL_FORM_SILU_MUL || form > SGL_FORM_FUSED_SWIGLU_SAVE)
    return fail(SGL_ERR_BAD_ARGUMENT, "unknown form %d", form);
  int rc = validate_shape(M, N, K);
  if (rc) return rc;
  return resolve_config(form, nullptr, M, out);
}

int sgl_config_smem_bytes(int form, const sgl_config* cfg) {
  if (!cfg) return fail(SGL_ERR_NULL_POINTER, "cfg is NULL");
  if (form < SGL_FORM_SILU_MUL || form > SGL_FORM_FUSED_SWIGLU_SAVE)
    return fail(SGL_ERR_BAD_ARGUMENT, "unknown form %d", form);
  sgl_config c;
  int rc = resolve_config(form, cfg, 1 << 20, &c);
  if (rc) return rc;
  return variant(form, c.cta_group, c.block_k, c.wide).smem_bytes(c.stages);
}

int sgl_tile_coord(int64_t t, int64_t tiles_m, int64_t tiles_n, int64_t group_m, int64_t* tile_m,
                   int64_t* tile_n) {
  if (!tile_m || !tile_n) return fail(SGL_ERR_NULL_POINTER, "output pointer is NULL");
  if (tiles_m < 1 || tiles_n < 1 || group_m < 1 || t < 0 || t >= tiles_m * tiles_n ||
      tiles_m * tiles_n > 0x7fffffffll)
    return fail(SGL_ERR_BAD_ARGUMENT, "tile index or grid out of range");
  sgl::TileCoord c = sgl::tile_coord(static_cast<int>(t), static_cast<int>(tiles_m),
                                     static_cast<int>(tiles_n), static_cast<int>(group_m));
  *tile_m = c.m;
  *tile_n = c.n;
  return SGL_OK;
}

int sgl_tile_coord_slabs(int64_t t, int64_t tiles_m, int64_t tiles_n, int64_t group_m,
                         int64_t group_n, int64_t* tile_m, int64_t* tile_n) {
  if (!tile_m || !tile_n) return fail(SGL_ERR_NULL_POINTER, "output pointer is NULL");
  if (tiles_m < 1 || tiles_n < 1 || group_m < 1 || group_n < 0 || t < 0 ||
      t >= tiles_m * tiles_n || tiles_m * tiles_n > 0x7fffffffll)
    return fail(SGL_ERR_BAD_ARGUMENT, "tile index or grid out of range");
  sgl::TileCoord c = sgl::tile_coord(static_cast<int>(t), static_cast<int>(tiles_m),
                                     static_cast<int>(tiles_n), static_cast<int>(group_m),
                                     static_cast<int>(group_n > tiles_n ? 0 : group_n));
  *tile_m = c.m;
  *tile_n = c.n;
  return SGL_OK;
}

int sgl_query(int what, int64_t* out) {
  if (!out) return fail(SGL_ERR_NULL_POINTER, "out is NULL");
  if (what == SGL_QUERY_KERNEL_LAUNCHES) {
    *out = g_launches.load();
    return SGL_OK;
  }
  int dev = 0;
  DeviceInfo* info = nullptr;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  switch (what) {
    case SGL_QUERY_SM_COUNT: *out = info->sm_count; return SGL_OK;
    case SGL_QUERY_MAX_SMEM_OPTIN: *out = info->max_smem_optin; return SGL_OK;
    case SGL_QUERY_COMPUTE_CAPABILITY: *out = info->cc; return SGL_OK;
    default: return fail(SGL_ERR_BAD_ARGUMENT, "unknown query %d", what);
  }
}

int sgl_shard_range(int64_t total, int64_t align, int world, int rank, int64_t* begin,
                    int64_t* count) {
  if (!begin || !count) return fail(SGL_ERR_NULL_POINTER, "output pointer is NULL");
  if (total < 0 || align < 1 || world < 1 || rank < 0 || rank >= world)
    return fail(SGL_ERR_BAD_ARGUMENT, "bad shard request: total=%lld align=%lld world=%d rank=%d",
                static_cast<long long>(total), static_cast<long long>(align), world, rank);
  // Distribute whole `align`-sized blocks as evenly as possible; earlier ranks
  // take the extra blocks, the last non-empty shard takes the ragged tail.
  const int64_t blocks = (total + align - 1) / align;
  const int64_t base = blocks / world;
  const int64_t extra = blocks % world;
  const int64_t b0 = rank * base + (rank < extra ? rank : extra);
  const int64_t nb = base + (rank < extra ? 1 : 0);
  int64_t lo = b0 * align;
  int64_t hi = (b0 + nb) * align;
  if (lo > total) lo = total;
  if (hi > total) hi = total;
  *begin = lo;
  *count = hi - lo;
  return SGL_OK;
}

int sgl_device_status(uint32_t* words) {
  unsigned int host[8];
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize");
  e = cudaMemcpyFromSymbol(host, sgl::g_status, sizeof(host));
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyFromSymbol(status)");
  if (words) std::memcpy(words, host, sizeof(host));
  if (host[0] != 0 || host[3] != 0) {
    unsigned int zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    e = cudaMemcpyToSymbol(sgl::g_status, zero, sizeof(zero));
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyToSymbol(status)");
    return fail(SGL_ERR_DEVICE_STATUS,
                "kernel wait timed out: code=0x%x block=%u detail=%u occurrences=%u", host[0],
                host[1], host[2], host[3]);
  }
  return SGL_OK;
}

int sgl_selftest_wait_timeout(uint64_t limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull)
    return fail(SGL_ERR_BAD_ARGUMENT, "limit must be in (0, 1e9] ns");
  DeviceInfo* info = nullptr;
  int rc = check_device(&info);
  if (rc) return rc;
  sgl::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "wait_timeout_selftest_kernel launch");
  return SGL_OK;
}

int sgl_set_wait_limit_ns(uint64_t ns) {
  if (ns == 0) return fail(SGL_ERR_BAD_ARGUMENT, "wait limit must be > 0");
  g_wait_limit_ns.store(ns);
  return SGL_OK;
}

#ifdef SGL_DEBUG
// Self-checking builds only: the per-CTA role counters of the LAST launch (512 x 4 words:
// k-blocks produced, k-blocks consumed, tiles finished by the epilogue, unused).
int sgl_debug_counts(unsigned long long* out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize");
  e = cudaMemcpyFromSymbol(out, sgl::g_debug_counts, sizeof(unsigned long long) * 512 * 4);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyFromSymbol(debug counts)");
  return SGL_OK;
}
#endif

#ifdef SGL_DEBUG
// Self-checking builds only: make the barrier of the split-K cluster sum expect `n` arrivals
// that never come (0 = normal).  Every CTA's wait then runs out after the wait limit, records
// status 0x106 and leaves through the closing cluster barrier: the time-out path is exercised
// without a kernel that stops half way.  Lower the limit first (sgl_set_wait_limit_ns).
int sgl_debug_cluster_sum_missing_arrivals(int n) {
  if (n < 0 || n > 4) return fail(SGL_ERR_BAD_ARGUMENT, "n=%d outside [0, 4]", n);
  g_debug_missing_arrivals.store(n);
  return SGL_OK;
}
#endif

#ifdef SGL_PROFILE
// Profiling builds only: the per-CTA %globaltimer stamps of the LAST launch (512 x 10 words).
int sgl_debug_timeline(unsigned long long* out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize");
  e = cudaMemcpyFromSymbol(out, sgl::g_tl, sizeof(unsigned long long) * 512 * 10);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyFromSymbol(tl)");
  return SGL_OK;
}
#endif

#ifdef SGL_PROFILE
// Profiling builds only: copy the per-CTA cycle counters (512 x 8 words).
int sgl_debug_profile(unsigned long long* out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize");
  e = cudaMemcpyFromSymbol(out, sgl::g_prof, sizeof(unsigned long long) * 512 * 8);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyFromSymbol(prof)");
  return SGL_OK;
}
#endif

const char* sgl_last_error(void) { return t_last_error.c_str(); }

int sgl_version(void) { return 100; }

}  // extern "C"

#include "swiglu_host_pipeline.cuh"
#include "swiglu_mgpu.cuh"
