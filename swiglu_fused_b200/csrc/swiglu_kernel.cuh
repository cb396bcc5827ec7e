// Persistent, warp-specialised fused SwiGLU gate/up kernel for sm_100a.
//
// Four forms share one skeleton:
//   FORM_SILU_MUL  h = silu(x @ W_gate) * up              (up is an input)
//       replaces matmul_silu_mul_impl, swiglu/_matmul_silu_mul.cu:323-652
//   FORM_FUSED     h = silu(x @ W[:, gate cols]) * (x @ W[:, up cols])
//       replaces matmul_fused_swiglu_impl, swiglu/_matmul_fused_swiglu.cu:193-508
//   FORM_FUSED_SAVE  FORM_FUSED that also stores the two factors training needs,
//       silu(gate) and up * silu'(gate), from the same epilogue (the reference does this
//       only in Triton: _fused_swiglu_wide_packed_save_factors_kernel,
//       swiglu/triton/impls.py:384-468)
//   FORM_GEMM      y = a @ b, no activation: the down projection that consumes h.  Its
//       epilogue can send each tile to the rank that owns those rows - stored into that
//       rank's slot for this sender, or ADDED into a shared buffer (TMA reduce) - over
//       NVLink: GEMM + reduce-scatter in one kernel.  It can also cut K into ranges whose
//       partial tiles go to separate slots (split-K).  No counterpart in the reference,
//       which stops at h.
//
// Design (not the reference's):
//   * persistent grid, one CTA (or CTA pair) per SM, static GROUP_SIZE_M-swizzled
//     tile schedule;
//   * warp 0 = TMA producer, warp 1 = tcgen05 MMA issuer, warps 2-5 = epilogue;
//   * one wide 256-column fp32 accumulator per tile.  In the fused form columns
//     [0,128) hold `up` and [128,256) hold `gate` for the same 128 output
//     columns, produced by ONE K loop (x is streamed once, not twice);
//   * two accumulator stages fill the 512 TMEM columns, so the epilogue of tile
//     t (TMEM -> registers -> silu*up in fp32 -> bf16 -> swizzled smem -> TMA
//     store) overlaps the mainloop of tile t+1;
//   * in the silu_mul form each epilogue warp prefetches its own `up` rows with
//     TMA into private shared-memory buffers (coalesced and asynchronous), overwrites
//     them in place with the result and TMA-stores from the same buffer;
//   * with kCtaGroup == 2 a CTA pair computes a 256-row tile with
//     tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of x and its own
//     half of the B operand (no multicast loads anywhere);
//   * the epilogue can write each output tile to several destination buffers
//     (this GPU's and its peers', plain TMA stores over NVLink): the all-gather
//     of a column-parallel launch is fused into the kernel;
//   * every wait is bounded; a timeout raises a CTA-wide abort flag, records an
//     error word in g_status and the kernel drains and exits.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace sgl {

enum : int { FORM_SILU_MUL = 0, FORM_FUSED = 1, FORM_GEMM = 2, FORM_FUSED_SAVE = 3 };

constexpr int kBlockM = 128;        // rows of x per CTA
constexpr int kAccCols = 256;       // accumulator columns per tile (MMA N)
constexpr int kAccStages = 2;       // TMEM accumulator stages
constexpr int kTmemCols = 512;      // kAccCols * kAccStages
constexpr int kMaxStages = 8;       // shared-memory ring depth limit
constexpr int kNumThreads = 192;    // 6 warps
constexpr int kEpiWarps = 4;
constexpr int kChunkCols = 64;      // epilogue works on 64 output columns (128 B rows)
constexpr int kChunkBytes = 32 * kChunkCols * 2;  // one warp's 32 rows x 128 B
constexpr int kOutBufs = 2;         // staging buffers per epilogue warp
constexpr int kUpBufs = 2;          // `up` prefetch buffers per epilogue warp

// Error words written to g_status[0] (first error wins); g_status[1] = block,
// g_status[2] = detail (role-specific: k-block, stage or chunk index).
enum : unsigned {
  kErrProducerEmptyWait = 0x101,
  kErrMmaFullWait = 0x102,
  kErrMmaTmemEmptyWait = 0x103,
  kErrEpiTmemFullWait = 0x104,
  kErrEpiUpWait = 0x105,
  kErrClusterSumWait = 0x106,   // split-K summed in the cluster: a K range never reported
  kErrDebugCoord = 0x301,     // -DSGL_DEBUG builds: a TMA coordinate failed its check
  kErrSelfTestWait = 0x1ff,   // the deliberate timeout of wait_timeout_selftest_kernel
};

// First-error record, readable from the host with cudaMemcpyFromSymbol.
__device__ unsigned int g_status[8];

constexpr int kMaxDst = 8;          // output copies one launch can write (this GPU + 7 peers)

// Tensor maps of the output: one per destination buffer.  A plain call has one;
// the column-parallel gather writes the same tile to every rank's buffer.
struct OutMaps {
  CUtensorMap m[kMaxDst];
};

// Optional cycle accounting (build with -DSGL_PROFILE): per CTA, cycles each role spent
// waiting.  [0] MMA waits for a free accumulator, [1] MMA waits for operands, [2] MMA loop
// total, [3] producer waits for a free ring slot, [4] epilogue waits for an accumulator,
// [5] epilogue waits for `up`, [6] epilogue busy, [7] tiles.
#ifdef SGL_PROFILE
__device__ unsigned long long g_prof[512][8];
#define SGL_PROF_DECL(name) long long name = 0
#define SGL_PROF_BEGIN(t) const long long t = clock64()
#define SGL_PROF_END(acc, t) acc += clock64() - t
#define SGL_PROF_STORE(slot, v) g_prof[blockIdx.x & 511][slot] = static_cast<unsigned long long>(v)
#else
#define SGL_PROF_DECL(name)
#define SGL_PROF_BEGIN(t)
#define SGL_PROF_END(acc, t)
#define SGL_PROF_STORE(slot, v)
#endif

// Self-checking build (-DSGL_DEBUG; compute-sanitizer is not available everywhere): every TMA
// coordinate is checked against the 16-byte rule and the tensor's extent before the copy is
// issued, and every role counts what it did.  A violation is RECORDED (g_status, code
// kErrDebugCoord) and the copy skipped - nothing traps - and the host compares the role
// counters afterwards (sgl_debug_counts): k-blocks produced must equal k-blocks consumed, tiles
// finished by the epilogue must equal tiles issued.  The normal library carries none of this.
#ifdef SGL_DEBUG
__device__ unsigned long long g_debug_counts[512][4];   // [cta]: produced, consumed, tiles, stores
#define SGL_DBG_COUNT(slot, v) g_debug_counts[blockIdx.x & 511][slot] = static_cast<unsigned long long>(v)
// true (after recording the violation) when the coordinate check fails; the caller skips
// the copy.  Always false in the normal build, where the compiler drops the branch.
__device__ __forceinline__ bool debug_coord_bad(bool ok, unsigned detail) {
  if (ok) return false;
  if (atomicCAS(&g_status[0], 0u, 0x301u) == 0u) {
    g_status[1] = blockIdx.x;
    g_status[2] = detail;
  }
  atomicAdd(&g_status[3], 1u);
  return true;
}
#define SGL_DBG_COORD_BAD(ok_expr, detail) debug_coord_bad((ok_expr), static_cast<unsigned>(detail))
#else
#define SGL_DBG_COUNT(slot, v)
#define SGL_DBG_COORD_BAD(ok_expr, detail) false
#endif

// Profiling builds also stamp %globaltimer at points of every CTA's life: [0] CTA start,
// [1] set-up done, [2] past the dependent-launch wait, [3] first operands landed, [4] last MMA
// committed, [5] epilogue sees the last accumulator, [6] epilogue's stores have read their
// staging, [7] teardown done; split-K summed in clusters: [8] partial tile in shared memory,
// [9] all K ranges have reported.  What a single-tile launch spends outside its K loop.
#ifdef SGL_PROFILE
__device__ unsigned long long g_tl[512][10];
#define SGL_TL(slot) g_tl[blockIdx.x & 511][slot] = ptx::globaltimer_ns()
#else
#define SGL_TL(slot)
#endif

struct KernelParams {
  int M, N, K;          // N = output columns of h
  int b_col0;           // first B column: gate (silu_mul form) / up (fused form)
  int b_col1;           // fused form: first gate column of the packed weight
  int tiles_m, tiles_n; // tile grid in cluster-tile units
  int group_m;          // GROUP_SIZE_M
  int group_n;          // column slabs of the tile order (0 = one slab)
  int stages;           // shared-memory ring depth actually used
  int l2_hints;         // 2 bits each: x loads, weight loads, h stores, up loads
  int n_dst;            // destinations in OutMaps actually used (>= 1)
  int a_mnmajor;        // A operand is stored transposed, [k, m] (the reduction index is the row):
                        // x^T @ g products of the backward pass without a transpose copy
  int b_kmajor;         // weight operand is stored [n, k] (nn.Linear layout) instead of [k, n];
                        // b_col0 / b_col1 are then row offsets of that tensor
  int reduce_rows;      // FORM_GEMM: > 0 = add into the destination that owns the row block
                        // (destination d owns rows [d * reduce_rows, (d+1) * reduce_rows))
  int out_f32;          // FORM_GEMM: destination element type is fp32 (else bf16)
  int splits;           // FORM_GEMM: K is cut into `splits` ranges of k_per_split (a multiple
  int k_per_split;      // of BLOCK_K); work unit u = tile u / splits, range u % splits, and
  int slot_rows;        // range s writes its partial tile at row offset s * slot_rows
  int m_shift;          // tile rows are visited starting at this tile row (wrapping): ranks of a
                        // reduce-scatter start at different owners so no owner is swamped
  int reduce_add;       // FORM_GEMM with reduce_rows > 0: 1 = add into the owner's buffer,
                        // 0 = overwrite (the owner's buffer is this rank's private slot)
  int acc_cols;         // FORM_GEMM, single-CTA tiles, [k, n] weight: columns per tile (64, 128
                        // or 256).  Short problems with few 256-wide tiles are cut into
                        // narrower ones so that more SMs stream their own columns of B.
  // Gather by thread stores (fused form): besides the TMA store into OutMaps.m[0], every
  // finished chunk is copied from the staging buffer to n_peer raw destinations with ordinary
  // 16-byte stores (peer_mode 1; peers' buffers over NVLink), or once to a multicast address
  // (peer_mode 2; the switch replicates it into every member's buffer, this GPU's included, and
  // the TMA store is skipped).  TMA stores to peers share the SM's TMA queue with the operand
  // loads, and a store held up by the link then holds up the mainloop; thread stores only
  // ever stall the epilogue warps, which have slack.
  int peer_mode;        // 0 = off
  int n_peer;
  long long peer_ld;    // row pitch of the raw destinations, elements
  unsigned long long peer_ptr[kMaxDst];   // element (0, 0) of this launch's block in each
  int a_rows;           // rows of the A box actually loaded per CTA and k-block: kBlockM, or the
                        // (8-aligned) row count of a problem shorter than one tile, whose
                        // missing rows would otherwise be fetched as zero fill at full cost
  // Split-K summed inside the launch through distributed shared memory (FORM_GEMM, single-CTA
  // tiles, one work unit per CTA): the `splits` K ranges of a tile are the CTAs of one
  // thread-block cluster.  Each CTA puts its fp32 partial tile into its own shared memory (the
  // operand ring, idle by then), tells every CTA of the cluster, waits (bounded) until all of
  // them have done so, sums its share of the tile's elements over the CTAs in K-range order
  // with ld.shared::cluster and writes bf16 straight to the result.  No scratch traffic, no
  // second kernel; the additions are those of the two-launch form, so are the bits.
  int cluster_sum;              // 0 = off; odd = on (out maps are unused, the result goes to
                                // sum_out); bits 1.. = extra arrivals its barrier expects
  unsigned long long up_raw;    // silu_mul form summed in clusters: address of up (0, 0), which
  long long up_ld;              // the CTA that sums a group of columns reads with plain loads
  unsigned long long sum_out;   // address of the bf16 result, element (0, 0)
  long long sum_ld;             // its row pitch, elements
  unsigned long long wait_limit_ns;
};

// Shared-memory layout of a partial tile for the cluster sum: kBlockM rows of 256 fp32 with 16
// bytes of padding, so that 32 lanes storing 16 bytes each at one column of 32 different rows
// spread over all banks.
constexpr uint32_t kRedPitchBytes = 256 * 4 + 16;
constexpr uint32_t kRedBytes = kBlockM * kRedPitchBytes;

// kWide (fused form, CTA pairs): one tile is 256 output columns - two MMAs per k-step into two
// 256-column accumulators, up in TMEM columns [0, 256) and gate in [256, 512) - instead of 128.
// The x tile is then fetched once per 256 output columns instead of once per 128, and the tile
// grid is half as long, which is what problems of a few hundred rows need: they are bound by
// the bytes each SM pulls in and by how evenly few tiles spread over 74 CTA pairs, not by the
// tensor cores.  The price is a single accumulator stage (all 512 TMEM columns hold one tile),
// so the epilogue of a tile no longer overlaps the next tile's mainloop.
template <int kForm, int kCtaGroup, int kBlockK, bool kWide = false>
struct KernelTraits {
  static_assert(!kWide || ((kForm == FORM_FUSED) && kCtaGroup == 2 && kBlockK == 64),
                "wide tiles exist for the fused form on CTA pairs with BLOCK_K 64");
  // silu_mul form: the `up` chunk is overwritten with the result and stored from the same
  // buffer (no separate output staging), which leaves room for one more ring stage.
  static constexpr bool kInPlace = (kForm == FORM_SILU_MUL);
  static constexpr bool kIsFused = (kForm == FORM_FUSED || kForm == FORM_FUSED_SAVE);
  static constexpr int kOutCols = kIsFused ? (kWide ? 256 : 128) : 256;
  static constexpr int kNumAccStages = kWide ? 1 : kAccStages;
  static constexpr int kGateCol = kWide ? 256 : 128;   // first TMEM column of the gate block
  // staging per epilogue warp: two 64-column chunk buffers, or for the side-store form three
  // 32-column buffers (h, silu, gate factor) so that a BLOCK_K = 128 ring still fits
  static constexpr int kNumOutBufs = kOutBufs;
  static constexpr int kSaveBufBytes = 32 * 32 * 2;   // 32 rows x 64 B
  static constexpr int kChunksPerTile = kOutCols / kChunkCols;
  static constexpr int kBColsPerCta = (kWide ? 2 * kAccCols : kAccCols) / kCtaGroup;
  static constexpr int kBSlabs = kBColsPerCta / 64;           // 64-column slabs this CTA loads
  static constexpr int kAStageBytes = kBlockM * kBlockK * 2;
  static constexpr int kBSlabBytes = kBlockK * 128;            // [kBlockK rows][64 cols]
  static constexpr int kBStageBytes = kBSlabs * kBSlabBytes;
  static constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  static constexpr int kOutStagingBytes =
      kInPlace ? 0
               : (kForm == FORM_FUSED_SAVE ? kEpiWarps * 3 * kSaveBufBytes
                                           : kEpiWarps * kNumOutBufs * kChunkBytes);
  static constexpr int kUpStagingBytes =
      (kForm == FORM_SILU_MUL) ? kEpiWarps * kUpBufs * kChunkBytes : 0;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kAlignSlack = 1024;
  static constexpr int kMaxSmem = 227 * 1024;

  __host__ __device__ static constexpr int smem_bytes(int stages) {
    return kAlignSlack + stages * kStageBytes + kOutStagingBytes + kUpStagingBytes +
           kBarrierBytes;
  }
  __host__ __device__ static constexpr int max_stages() {
    int s = (kMaxSmem - kAlignSlack - kOutStagingBytes - kUpStagingBytes - kBarrierBytes) /
            kStageBytes;
    return s > kMaxStages ? kMaxStages : s;
  }
};

struct TileCoord {
  int m;  // cluster-tile row index
  int n;  // cluster-tile column index
};

// GROUP_SIZE_M swizzle: tiles are walked in bands of `group_m` tile rows, rows
// fastest inside a band, so concurrently running tiles share x rows and weight
// columns in L2.  Equivalent in purpose to swiglu/_matmul_silu_mul.cu:357-384,
// applied to the persistent schedule's linear tile index.
//
// group_n > 0 adds an outer level: the tile columns are cut into slabs of group_n tiles and all
// row bands of one slab are walked before the next slab.  A slab of the weight (group_n tile
// columns, every k) then stays in L2 while the bands of x stream past it, instead of the whole
// weight being fetched from DRAM again for every band.
__host__ __device__ inline TileCoord tile_coord(int t, int tiles_m, int tiles_n, int group_m,
                                                int group_n = 0) {
  int first_n = 0, cols = tiles_n;
  if (group_n > 0 && group_n < tiles_n) {
    const int per_slab = tiles_m * group_n;
    const int slab = t / per_slab;
    first_n = slab * group_n;
    cols = (tiles_n - first_n) < group_n ? (tiles_n - first_n) : group_n;
    t -= slab * per_slab;
  }
  const int per_band = group_m * cols;
  const int band = t / per_band;
  const int first_m = band * group_m;
  const int rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const int in_band = t - band * per_band;
  TileCoord c;
  c.m = first_m + in_band % rows;
  c.n = first_n + in_band / rows;
  return c;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// silu(g) * u in fp32 with one MUFU.EX2 and one MUFU.RCP:
//   silu(g) = g / (1 + e^-g) = g * rcp(1 + 2^(-g * log2 e)).
__device__ __forceinline__ float silu_mul(float g, float u) {
  const float e = ex2_approx(g * -1.4426950408889634f);
  const float s = g * rcp_approx(1.0f + e);
  return s * u;
}

// The three values the side-store forward writes for one element:
//   h = silu(g) * u,  s = silu(g),  d = u * silu'(g)  with  silu' = sig + silu * (1 - sig)
// (the same expressions as swiglu/triton/impls.py:455-461), from one ex2 and one rcp.
__device__ __forceinline__ void silu_factors(float g, float u, float& h, float& s, float& d) {
  const float e = ex2_approx(g * -1.4426950408889634f);
  const float sig = rcp_approx(1.0f + e);
  s = g * sig;
  const float sp = sig + s * (1.0f - sig);
  h = s * u;
  d = u * sp;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void report_error(unsigned code, unsigned detail, int* abort_flag) {
  if (atomicCAS(&g_status[0], 0u, code) == 0u) {
    g_status[1] = blockIdx.x;
    g_status[2] = detail;
  }
  atomicAdd(&g_status[3], 1u);
  *reinterpret_cast<volatile int*>(abort_flag) = 1;
}

// Exercises the bounded-wait path on real hardware without any risk of a hang: one thread
// waits on an mbarrier that nobody will ever arrive on, with the given time limit, and must
// come back with a timeout, record kErrSelfTestWait in g_status and exit normally.
__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int flags[2];
  if (threadIdx.x == 0) {
    flags[0] = 0;
    flags[1] = 0;
    const uint32_t b = ptx::smem_u32(&bar);
    ptx::mbar_init(b, 1);
    ptx::fence_mbar_init();
    if (!ptx::mbar_wait(b, 0, limit_ns, flags)) report_error(kErrSelfTestWait, 0, flags);
  }
}

template <int kForm, int kCtaGroup, int kBlockK, bool kWide = false>
__global__ void __launch_bounds__(kNumThreads, 1)
swiglu_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
              const __grid_constant__ CUtensorMap tm_up, const __grid_constant__ OutMaps tm_h,
              const KernelParams p) {
  using T = KernelTraits<kForm, kCtaGroup, kBlockK, kWide>;
  constexpr int kStagesAcc = T::kNumAccStages;
  constexpr bool kInPlace = T::kInPlace;
  static_assert(kBlockK == 64 || kBlockK == 128, "BLOCK_K is 64 or 128");
  static_assert(kCtaGroup == 1 || kCtaGroup == 2, "CTA group is 1 or 2");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { SGL_TL(0); }
  const uint32_t rank = (kCtaGroup == 2) ? ptx::cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / kCtaGroup;
  const int num_clusters = gridDim.x / kCtaGroup;
  // Work units: one per output tile, or (split-K, FORM_GEMM only) one per tile and K range.
  // K may be cut into ranges in the GEMM form and in the fused form on single-CTA tiles
  constexpr bool kCanSplitK =
      (kForm == FORM_GEMM) || (kForm == FORM_FUSED && kCtaGroup == 1 && !kWide) ||
      (kForm == FORM_SILU_MUL && kCtaGroup == 1);
  const int splits = kCanSplitK ? p.splits : 1;
  const int total_tiles = p.tiles_m * p.tiles_n * splits;
  auto shifted_tile = [&](int t) {
    TileCoord tc = tile_coord(t, p.tiles_m, p.tiles_n, p.group_m, p.group_n);
    tc.m += p.m_shift;
    if (tc.m >= p.tiles_m) tc.m -= p.tiles_m;
    return tc;
  };
  // K range of unit u and its length in k-blocks.
  auto unit_k0 = [&](int u) { return (splits > 1) ? (u % splits) * p.k_per_split : 0; };
  auto unit_kb = [&](int u) {
    int len = p.K;
    if (splits > 1) {
      len = p.K - (u % splits) * p.k_per_split;
      len = len < p.k_per_split ? len : p.k_per_split;
      len = len < 0 ? 0 : len;
    }
    return (len + kBlockK - 1) / kBlockK;
  };
  const int stages = p.stages;
  // Output columns per tile: a compile-time constant except in the GEMM form, where
  // single-CTA tiles may be narrower and then load fewer 64-column slabs of B per stage.
  int tile_cols = T::kOutCols;
  int b_slabs = T::kBSlabs;
  if constexpr (kForm == FORM_GEMM) tile_cols = p.acc_cols;
  if constexpr (kForm == FORM_GEMM && kCtaGroup == 1) b_slabs = tile_cols / 64;

  // ---- shared memory carve-up (offsets identical in both CTAs of a pair) ----
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + stages * T::kAStageBytes;
  const uint32_t sOut = sB + stages * T::kBStageBytes;
  const uint32_t sUp = sOut + T::kOutStagingBytes;
  const uint32_t sBar = sUp + T::kUpStagingBytes;
  const uint32_t bar_full = sBar;                       // [kMaxStages]
  const uint32_t bar_empty = bar_full + 8 * kMaxStages; // [kMaxStages]
  const uint32_t bar_tfull = bar_empty + 8 * kMaxStages;  // [kAccStages]
  const uint32_t bar_tempty = bar_tfull + 8 * kAccStages; // [kAccStages]
  const uint32_t bar_up = bar_tempty + 8 * kAccStages;    // [kEpiWarps][kUpBufs]
  const uint32_t tmem_slot = bar_up + 8 * kEpiWarps * kUpBufs;
  const uint32_t abort_slot = tmem_slot + 8;
  const uint32_t bar_sum = abort_slot + 8;   // cluster sum: every epilogue warp of every K range
  const bool cluster_sum = (kCanSplitK && kCtaGroup == 1) && p.cluster_sum != 0;
  // Generic pointers to the two scalar slots.
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
  // abort_flag[0] = CTA-wide abort flag, abort_flag[1] stays zero.
  int* abort_flag = reinterpret_cast<int*>(smem_gen + (abort_slot - smem_base));

  // ---- one-time setup ----
  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, kCtaGroup);  // one arrive.expect_tx per CTA
      ptx::mbar_init(bar_empty + 8 * s, 1);         // one tcgen05.commit
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(bar_tfull + 8 * s, 1);                     // one tcgen05.commit
      ptx::mbar_init(bar_tempty + 8 * s, kEpiWarps * kCtaGroup);  // one arrive per epilogue warp
    }
    for (int i = 0; i < kEpiWarps * kUpBufs; ++i) ptx::mbar_init(bar_up + 8 * i, 1);
    // (p.cluster_sum >> 1: arrivals that never come - the self-checking build's way of making
    // this barrier's bounded wait run out; 0 in every other launch)
    if (cluster_sum) ptx::mbar_init(bar_sum, kEpiWarps * p.splits + (p.cluster_sum >> 1));
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_x);
    ptx::prefetch_tensormap(&tm_w);
    for (int d = 0; d < p.n_dst; ++d) ptx::prefetch_tensormap(&tm_h.m[d]);
    if constexpr (kForm == FORM_SILU_MUL) ptx::prefetch_tensormap(&tm_up);
  }
  if (warp == 1) {
    ptx::tmem_alloc<kCtaGroup>(tmem_slot, kTmemCols);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  // (cluster sum: no CTA may arrive on a peer's barrier before the peer has initialised it)
  if (kCtaGroup == 2 || cluster_sum) ptx::cluster_sync();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // Programmatic dependent launch (the host launches this kernel with programmatic stream
  // serialisation allowed).  Everything above touches no global memory, so it may run while
  // the previous kernel of the stream is still finishing; from here on the previous grid must
  // be complete and its writes visible.  In turn the next kernel of the stream may be set up
  // from now on (it waits at the same point).  Both are no-ops when the neighbour in the
  // stream is an ordinary launch.
  if (threadIdx.x == 0) { SGL_TL(1); }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) { SGL_TL(2); }

  const uint64_t limit = p.wait_limit_ns;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      // Barrier that collects this stage's bytes: the leader CTA's.
      SGL_PROF_DECL(prof_pe);
      const uint64_t pol_x = ptx::make_l2_policy(p.l2_hints & 3);
      const uint64_t pol_w = ptx::make_l2_policy((p.l2_hints >> 2) & 3);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
#ifdef SGL_DEBUG
      unsigned long long dbg_produced = 0;
#endif
      for (int t = cluster_id; t < total_tiles && ok; t += num_clusters) {
        const TileCoord tc = shifted_tile(t / splits);
        const int m0 = (tc.m * kCtaGroup + static_cast<int>(rank)) * kBlockM;
        const int n0 = tc.n * tile_cols;
        const int num_kb = unit_kb(t);
        const int k_base = unit_k0(t);
        // (A stored [k, m] is loaded as whole 64-column slabs; otherwise only a_rows rows)
        const uint32_t a_tx = p.a_mnmajor ? static_cast<uint32_t>(T::kAStageBytes)
                                          : static_cast<uint32_t>(p.a_rows * kBlockK * 2);
        const uint32_t stage_tx = a_tx + static_cast<uint32_t>(b_slabs * T::kBSlabBytes);
        for (int kb = 0; kb < num_kb; ++kb) {
          SGL_PROF_BEGIN(tp0);
          if (!ptx::mbar_wait(bar_empty + 8 * s, ph ^ 1u, limit, abort_flag)) {
            report_error(kErrProducerEmptyWait, kb, abort_flag);
            ok = false;
            break;
          }
          SGL_PROF_END(prof_pe, tp0);
          const uint32_t full_local = bar_full + 8 * s;
          const uint32_t full = (kCtaGroup == 2) ? ptx::mapa(full_local, 0) : full_local;
          const int k0 = k_base + kb * kBlockK;
          if (SGL_DBG_COORD_BAD(k0 >= 0 && k0 < p.K && (k0 & 7) == 0 && m0 >= 0 &&
                                    m0 < p.tiles_m * kCtaGroup * kBlockM && n0 >= 0 &&
                                    (n0 & 7) == 0 && ((p.b_col0 | p.b_col1) & 7) == 0,
                                kb)) {
            // no copy is issued with a bad coordinate: raise the abort flag and leave
            *reinterpret_cast<volatile int*>(abort_flag) = 1;
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx_cluster(full, stage_tx);
#ifdef SGL_DEBUG
          ++dbg_produced;
#endif
          const uint32_t a_dst = sA + s * T::kAStageBytes;
          if (p.a_mnmajor) {
            // A stored [k, m]: two slabs of 64 m-columns x kBlockK k-rows, like the weight.
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j) {
              ptx::tma_load_2d<kCtaGroup == 2>(a_dst + j * (kBlockK * 128), &tm_x, m0 + j * 64, k0,
                                               full, pol_x);
            }
          } else {
#pragma unroll
            for (int j = 0; j < kBlockK / 64; ++j) {
              ptx::tma_load_2d<kCtaGroup == 2>(a_dst + j * (kBlockM * 128), &tm_x, k0 + j * 64,
                                               m0, full, pol_x);
            }
          }
          const uint32_t b_dst = sB + s * T::kBStageBytes;
          if (p.b_kmajor) {
            // Weight stored [n, k]: boxes of 128 n-rows x 64 k, laid out [k box][rows][128 B]
            // so that one 64-k slice of all this CTA's B rows is contiguous.
            constexpr int kRowBoxes = T::kBColsPerCta / 128;
#pragma unroll
            for (int j = 0; j < kBlockK / 64; ++j) {
#pragma unroll
              for (int rb = 0; rb < kRowBoxes; ++rb) {
                const int wdx = static_cast<int>(rank) * kRowBoxes + rb;  // 128-column window
                int row;
                if constexpr (!T::kIsFused) {
                  row = p.b_col0 + n0 + wdx * 128;
                } else {
                  row = (wdx == 0) ? (p.b_col0 + n0) : (p.b_col1 + n0);
                }
                ptx::tma_load_2d<kCtaGroup == 2>(
                    b_dst + j * (T::kBColsPerCta * 128) + rb * (128 * 128), &tm_w, k0 + j * 64,
                    row, full, pol_w);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < T::kBSlabs; ++j) {
              if (j >= b_slabs) break;
              // Slab index inside the 256 accumulator columns of the cluster tile.
              const int g = static_cast<int>(rank) * T::kBSlabs + j;
              int col;
              if constexpr (!T::kIsFused) {
                col = p.b_col0 + n0 + g * 64;
              } else if constexpr (kWide) {
                // this CTA supplies its 128-column half of BOTH MMAs' B operands:
                // slabs 0, 1 = up columns, slabs 2, 3 = gate columns
                const int half0 = n0 + static_cast<int>(rank) * 128 + (j & 1) * 64;
                col = (j < 2) ? (p.b_col0 + half0) : (p.b_col1 + half0);
              } else {
                col = (g < 2) ? (p.b_col0 + n0 + g * 64) : (p.b_col1 + n0 + (g - 2) * 64);
              }
              ptx::tma_load_2d<kCtaGroup == 2>(b_dst + j * T::kBSlabBytes, &tm_w, col, k0, full,
                                               pol_w);
            }
          }
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      SGL_PROF_STORE(3, prof_pe);
      SGL_DBG_COUNT(0, dbg_produced);
      if (!ok) {
        // Give loads that are still in flight time to land before the CTA exits.
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = ptx::make_idesc_bf16(kBlockM * kCtaGroup,
                                                  kForm == FORM_GEMM ? tile_cols : kAccCols,
                                                  /*a_mn_major=*/p.a_mnmajor != 0,
                                                  /*b_mn_major=*/p.b_kmajor == 0);
      const bool b_kmajor = p.b_kmajor != 0;
      const bool a_mnmajor = p.a_mnmajor != 0;
      constexpr uint16_t mask = (kCtaGroup == 2) ? 0x3 : 0x1;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int i = 0;
#ifdef SGL_DEBUG
      unsigned long long dbg_consumed = 0;
#endif
      SGL_PROF_DECL(prof_te);
      SGL_PROF_DECL(prof_fu);
      SGL_PROF_DECL(prof_tot);
      SGL_PROF_BEGIN(tm_all);
      for (int t = cluster_id; t < total_tiles && ok; t += num_clusters, ++i) {
        const int as = i % kStagesAcc;
        const uint32_t aph = (i / kStagesAcc) & 1u;
        SGL_PROF_BEGIN(tm0);
        if (!ptx::mbar_wait(bar_tempty + 8 * as, aph ^ 1u, limit, abort_flag)) {
          report_error(kErrMmaTmemEmptyWait, i, abort_flag);
          ok = false;
          break;
        }
        SGL_PROF_END(prof_te, tm0);
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * kAccCols;
        const int num_kb = unit_kb(t);
        for (int kb = 0; kb < num_kb; ++kb) {
          SGL_PROF_BEGIN(tm1);
          if (!ptx::mbar_wait(bar_full + 8 * s, ph, limit, abort_flag)) {
            report_error(kErrMmaFullWait, kb, abort_flag);
            ok = false;
            break;
          }
          SGL_PROF_END(prof_fu, tm1);
          if (kb == 0 && i == 0) { SGL_TL(3); }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = sA + s * T::kAStageBytes;
          const uint32_t b_base = sB + s * T::kBStageBytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / 16; ++kk) {
            // x tile: K-major, one 128-row x 64-col swizzled box per 64 k;
            // 16 k = 32 bytes inside the 128-byte swizzle row.
            // ([k, m] storage: M-major slabs [kBlockK rows][64 m], 16 k = 16 rows.)
            const uint64_t a_desc =
                a_mnmajor ? ptx::smem_desc_sw128(a_base + kk * 16 * 128, kBlockK * 128, 1024)
                          : ptx::smem_desc_sw128(
                                a_base + (kk >> 2) * (kBlockM * 128) + (kk & 3) * 32, 16, 1024);
            // weight tile, [k, n] storage: N-major slabs [kBlockK rows][64 cols], 16 k = 16
            // rows; [n, k] storage: K-major like x, rows = n, 16 k = 32 bytes.
            const uint64_t b_desc =
                b_kmajor ? ptx::smem_desc_sw128(b_base + (kk >> 2) * (T::kBColsPerCta * 128) +
                                                    (kk & 3) * 32, 16, 1024)
                         : ptx::smem_desc_sw128(b_base + kk * 16 * 128, T::kBSlabBytes, 1024);
            ptx::umma_bf16<kCtaGroup>(d_tmem, a_desc, b_desc, idesc,
                                      (kb > 0 || kk > 0) ? 1u : 0u);
            if constexpr (kWide) {
              // second MMA of the k-step: the gate columns (slabs 2, 3 of the stage)
              const uint64_t b_desc_gate =
                  ptx::smem_desc_sw128(b_base + 2 * T::kBSlabBytes + kk * 16 * 128,
                                       T::kBSlabBytes, 1024);
              ptx::umma_bf16<kCtaGroup>(d_tmem + T::kGateCol, a_desc, b_desc_gate, idesc,
                                        (kb > 0 || kk > 0) ? 1u : 0u);
            }
          }
          ptx::umma_commit<kCtaGroup>(bar_empty + 8 * s, mask);
#ifdef SGL_DEBUG
          ++dbg_consumed;
#endif
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) ptx::umma_commit<kCtaGroup>(bar_tfull + 8 * as, mask);
        SGL_TL(4);
      }
      SGL_PROF_END(prof_tot, tm_all);
      SGL_PROF_STORE(0, prof_te);
      SGL_PROF_STORE(1, prof_fu);
      SGL_PROF_STORE(2, prof_tot);
      SGL_DBG_COUNT(1, dbg_consumed);
    }
  } else {
    // =========================== epilogue ===========================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t out_buf0 =
        sOut + q * (kForm == FORM_FUSED_SAVE ? 3 * T::kSaveBufBytes : T::kNumOutBufs * kChunkBytes);
    const uint32_t up_buf0 = sUp + q * (kUpBufs * kChunkBytes);
    const uint32_t my_bar_up = bar_up + 8 * (q * kUpBufs);
    const uint32_t tempty_leader_base = (kCtaGroup == 2) ? ptx::mapa(bar_tempty, 0) : bar_tempty;
    const uint32_t row_sw = static_cast<uint32_t>(lane & 7);  // 128B-swizzle row phase
    const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;

    // Number of tiles this cluster owns.
    const int my_tiles =
        (cluster_id < total_tiles) ? (total_tiles - cluster_id + num_clusters - 1) / num_clusters : 0;
    const int total_chunks = my_tiles * T::kChunksPerTile;

    // Coordinates of output chunk g (global over this CTA's tile sequence).
    auto chunk_xy = [&](int g, int& x, int& y) {
      const int i = g / T::kChunksPerTile;
      const int c = g - i * T::kChunksPerTile;
      const TileCoord tc = shifted_tile((cluster_id + i * num_clusters) / splits);
      x = tc.n * tile_cols + c * kChunkCols;
      y = (tc.m * kCtaGroup + static_cast<int>(rank)) * kBlockM + q * 32;
      if (SGL_DBG_COORD_BAD(x >= 0 && (x & 7) == 0 && y >= 0 && (y & 31) == 0 &&
                                x < p.tiles_n * tile_cols && y < p.tiles_m * kCtaGroup * kBlockM,
                            g)) {
        x = 0x7fffff00;   // beyond N: every store and `up` load of this chunk is skipped
      }
    };

    const uint64_t pol_h = ptx::make_l2_policy((p.l2_hints >> 4) & 3);
    const uint64_t pol_up = ptx::make_l2_policy((p.l2_hints >> 6) & 3);
    int up_issued = 0;  // `up` chunk loads issued so far (lane 0 only)
    auto issue_up = [&](int g) {
      int x, y;
      chunk_xy(g, x, y);
      const int b = g % kUpBufs;
      ptx::mbar_arrive_expect_tx_cluster(my_bar_up + 8 * b, kChunkBytes);
      ptx::tma_load_2d<false>(up_buf0 + b * kChunkBytes, &tm_up, x, y, my_bar_up + 8 * b,
                              pol_up);
    };
    if constexpr (kForm == FORM_SILU_MUL) {
      if (lane == 0 && !cluster_sum) {
        // In-place staging refills a buffer only after its store has drained, so it runs
        // one chunk ahead; separate staging runs kUpBufs chunks ahead.
        const int ahead = kInPlace ? 1 : kUpBufs;
        for (; up_issued < ahead && up_issued < total_chunks; ++up_issued) issue_up(up_issued);
      }
    }

    // Split-K summed in the cluster (one unit per CTA, cluster = the K ranges of one tile): the
    // epilogue of such a unit.  acc_cols accumulator columns are exchanged; out_cols result
    // columns come out of them (the same in the GEMM form; in the fused form 256 accumulator
    // columns, up | gate, give 128 columns of silu(gate) * up).  Returns false after a
    // time-out, which has been recorded.
    // mode (a std::integral_constant): 0 = plain sum (GEMM form), 1 = fused form, 2 = silu_mul
    // form (256 gate columns summed, up read from global memory by the CTA that sums).
    auto cluster_epilogue = [&](auto mode, int i, int as, uint32_t t_row, int x0, int y,
                                int acc_cols, int out_cols) -> bool {
      (void)i;
      const uint32_t my_range = ptx::cluster_ctarank();
      const uint32_t red = sA;   // the operand ring: every load has landed and been consumed
      const uint32_t my_row = red + static_cast<uint32_t>(q * 32 + lane) * kRedPitchBytes;
      if (SGL_DBG_COORD_BAD(my_tiles == 1 && static_cast<int>(my_range) == cluster_id % splits &&
                                stages * (T::kAStageBytes + T::kBStageBytes) >=
                                    static_cast<int>(kRedBytes),
                            my_range)) {
        // the launch does not have the shape this path relies on (one unit per CTA, cluster
        // rank = K range, a ring that holds a partial tile): record it and leave; the other
        // ranges of the tile run into their bounded wait
        *reinterpret_cast<volatile int*>(abort_flag) = 1;
        return false;
      }
      // (a warp whose 32 rows lie below the last row of the problem keeps nothing; tiles
      // are whole 64-column slabs wide, so the 32-column reads go in pairs: one wait for
      // two TMEM loads)
      if (y < p.M) {
#pragma unroll 1
        for (int u = 0; u < acc_cols / 32; u += 2) {
          float acc0[32], acc1[32];
          ptx::tmem_ld_32x32b_x32(t_row + u * 32, acc0);
          ptx::tmem_ld_32x32b_x32(t_row + u * 32 + 32, acc1);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(
                             my_row + static_cast<uint32_t>(u * 32 + 4 * j) * 4u),
                         "f"(acc0[4 * j]), "f"(acc0[4 * j + 1]), "f"(acc0[4 * j + 2]),
                         "f"(acc0[4 * j + 3])
                         : "memory");
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(
                             my_row + static_cast<uint32_t>(u * 32 + 32 + 4 * j) * 4u),
                         "f"(acc1[4 * j]), "f"(acc1[4 * j + 1]), "f"(acc1[4 * j + 2]),
                         "f"(acc1[4 * j + 3])
                         : "memory");
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader_base + 8 * as);
      // This warp's 32 rows are in place: tell every CTA of the cluster (this one
      // included).  One lane per destination: a cluster-scope release is a fence, and
      // `splits` of them from one lane in turn cost 2 us.
      if (lane < splits)
        ptx::mbar_arrive_release_cluster(ptx::mapa(bar_sum, static_cast<uint32_t>(lane)));
      if (q == 0 && lane == 0) { SGL_TL(8); }
      const bool met = ptx::mbar_wait_acquire_cluster(bar_sum, 0, limit, abort_flag);
      if (q == 0 && lane == 0) { SGL_TL(9); }
      if (!__all_sync(0xffffffffu, met)) {
        if (lane == 0) report_error(kErrClusterSumWait, my_range, abort_flag);
        return false;
      }
      // This CTA's share of the tile, in groups of 4 columns, summed over the K ranges in
      // order starting from 0.f - element by element the additions of sum_slots_f32_kernel.
      // The loads of a batch of ranges for four groups are issued before the first addition.
      // (Sending the rows to their owners with st.shared::cluster instead, so that this sum
      // reads local memory only, measured the same: the exchange itself, about 40 KB per
      // CTA, is what takes the time.)
      const int row0 = y - q * 32;
      const int rows_valid = min(kBlockM, p.M - row0);
      const int n_vec = min(out_cols, p.N - x0) / 4;
      const int total = rows_valid * n_vec;
      const int per = (total + splits - 1) / splits;
      const int hi = min(total, (static_cast<int>(my_range) + 1) * per);
      const int te = q * 32 + lane;
      __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.sum_out);
      // (fused form: the partial tile holds up in columns [0, 128) and gate in [128, 256); a
      // group of the result needs both, so half as many groups are in flight)
      constexpr bool kAct = decltype(mode)::value == 1;
      constexpr bool kUpFromGlobal = decltype(mode)::value == 2;
      constexpr int kItems = kAct ? 2 : 4, kBatch = 8, kEpiThreads = kEpiWarps * 32;
#pragma unroll 1
      for (int e0 = static_cast<int>(my_range) * per + te; e0 < hi;
           e0 += kItems * kEpiThreads) {
        uint32_t src[kItems];
        long long dst_off[kItems];
        bool on[kItems];
        float4 sum[kItems];
        float4 gsum[kItems];   // fused form: the gate columns of the same group
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
          const int e = e0 + k * kEpiThreads;
          on[k] = e < hi;
          const int ee = on[k] ? e : e0;
          const int r = ee / n_vec;
          const int v = ee - r * n_vec;
          src[k] = red + static_cast<uint32_t>(r) * kRedPitchBytes +
                   static_cast<uint32_t>(v) * 16u;
          dst_off[k] = static_cast<long long>(row0 + r) * p.sum_ld + x0 + 4 * v;
          sum[k] = make_float4(0.f, 0.f, 0.f, 0.f);
          gsum[k] = sum[k];
          if constexpr (kUpFromGlobal) {
            // four bf16 of up for this group, fetched now so that they are here when the sum is
            const uint2 u4 = __ldg(reinterpret_cast<const uint2*>(
                reinterpret_cast<const __nv_bfloat16*>(p.up_raw) +
                static_cast<long long>(row0 + r) * p.up_ld + x0 + 4 * v));
            gsum[k] = make_float4(__uint_as_float(u4.x << 16), __uint_as_float(u4.x & 0xffff0000u),
                                  __uint_as_float(u4.y << 16), __uint_as_float(u4.y & 0xffff0000u));
          }
        }
#pragma unroll 1
        for (int s0 = 0; s0 < splits; s0 += kBatch) {
          float4 t[kItems][kBatch];
          float4 tg[kAct ? kItems : 1][kAct ? kBatch : 1];
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
#pragma unroll
            for (int k = 0; k < kItems; ++k) {
              if (s0 + j < splits) {
                const uint32_t remote = ptx::mapa(src[k], static_cast<uint32_t>(s0 + j));
                t[k][j] = ptx::ld_shared_cluster_v4(remote);
                if constexpr (kAct) tg[k][j] = ptx::ld_shared_cluster_v4(remote + T::kGateCol * 4);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
#pragma unroll
            for (int k = 0; k < kItems; ++k) {
              if (s0 + j < splits) {
                sum[k].x += t[k][j].x;
                sum[k].y += t[k][j].y;
                sum[k].z += t[k][j].z;
                sum[k].w += t[k][j].w;
                if constexpr (kAct) {
                  gsum[k].x += tg[k][j].x;
                  gsum[k].y += tg[k][j].y;
                  gsum[k].z += tg[k][j].z;
                  gsum[k].w += tg[k][j].w;
                }
              }
            }
          }
        }
#pragma unroll
        for (int k = 0; k < kItems; ++k) {
          if (on[k]) {
            uint2 o;
            if constexpr (kAct) {
              o.x = pack_bf16x2(silu_mul(gsum[k].x, sum[k].x), silu_mul(gsum[k].y, sum[k].y));
              o.y = pack_bf16x2(silu_mul(gsum[k].z, sum[k].z), silu_mul(gsum[k].w, sum[k].w));
            } else if constexpr (kUpFromGlobal) {
              // sum = the gate pre-activation, gsum = up
              o.x = pack_bf16x2(silu_mul(sum[k].x, gsum[k].x), silu_mul(sum[k].y, gsum[k].y));
              o.y = pack_bf16x2(silu_mul(sum[k].z, gsum[k].z), silu_mul(sum[k].w, gsum[k].w));
            } else {
              o.x = pack_bf16x2(sum[k].x, sum[k].y);
              o.y = pack_bf16x2(sum[k].z, sum[k].w);
            }
            *reinterpret_cast<uint2*>(outp + dst_off[k]) = o;
          }
        }
      }
      return true;
    };

    bool ok = true;
    int g = 0;            // running chunk index
    int gemm_stores = 0;  // FORM_GEMM: staging buffers filled so far
    SGL_PROF_DECL(prof_tf);
    SGL_PROF_DECL(prof_up);
    SGL_PROF_DECL(prof_busy);
    for (int i = 0; i < my_tiles && ok; ++i) {
      const int as = i % kStagesAcc;
      const uint32_t aph = (i / kStagesAcc) & 1u;
      {
        SGL_PROF_BEGIN(te0);
        const bool w = ptx::mbar_wait(bar_tfull + 8 * as, aph, limit, abort_flag);
        SGL_PROF_END(prof_tf, te0);
        if (!__all_sync(0xffffffffu, w)) {
          if (lane == 0) report_error(kErrEpiTmemFullWait, i, abort_flag);
          ok = false;
          break;
        }
      }
      ptx::tc_fence_after_sync();
      if (q == 0 && lane == 0) { SGL_TL(5); }
      SGL_PROF_BEGIN(te_busy);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kAccCols;

      if constexpr (kForm == FORM_FUSED_SAVE) {
        // Side-store epilogue: per 32-column half chunk fill three small staging buffers
        // (h, silu(gate), up * silu'(gate); 64-byte rows, 64B swizzle) and store them with
        // three TMA stores in one bulk group.
        // tm_h.m[0] = h, m[1] = silu block of the factors, m[2] = gate-factor block.
        constexpr uint32_t kSB = T::kSaveBufBytes;
        const uint32_t off_row = static_cast<uint32_t>(lane) * 64u;
        const uint32_t sw64 = (static_cast<uint32_t>(lane) >> 1) & 3u;
#pragma unroll 1
        for (int c = 0; c < T::kChunksPerTile; ++c, ++g) {
          int x, y;
          chunk_xy(g, x, y);
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            const int col = c * kChunkCols + half * 32;
            float gate[32];
            float upv[32];
            ptx::tmem_ld_32x32b_x32(t_row + col, upv);
            ptx::tmem_ld_32x32b_x32(t_row + T::kGateCol + col, gate);
            ptx::tmem_ld_wait();
            if (c == T::kChunksPerTile - 1 && half == 1) {
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader_base + 8 * as);
            }
            if (lane == 0) ptx::bulk_wait_group_read<0>();   // previous half's stores have read
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t wh[4], ws[4], wd[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int idx = j * 8 + 2 * e;
                float h0, s0, d0, h1, s1, d1;
                silu_factors(gate[idx], upv[idx], h0, s0, d0);
                silu_factors(gate[idx + 1], upv[idx + 1], h1, s1, d1);
                wh[e] = pack_bf16x2(h0, h1);
                ws[e] = pack_bf16x2(s0, s1);
                wd[e] = pack_bf16x2(d0, d1);
              }
              const uint32_t off = off_row + ((static_cast<uint32_t>(j) ^ sw64) << 4);
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(out_buf0 + off),
                           "r"(wh[0]), "r"(wh[1]), "r"(wh[2]), "r"(wh[3]) : "memory");
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(out_buf0 + kSB + off),
                           "r"(ws[0]), "r"(ws[1]), "r"(ws[2]), "r"(ws[3]) : "memory");
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(out_buf0 + 2 * kSB + off),
                           "r"(wd[0]), "r"(wd[1]), "r"(wd[2]), "r"(wd[3]) : "memory");
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int xh = x + half * 32;
              if (xh < p.N && y < p.M) {
                ptx::tma_store_2d(&tm_h.m[0], xh, y, out_buf0, pol_h);
                ptx::tma_store_2d(&tm_h.m[1], xh, y, out_buf0 + kSB, pol_h);
                ptx::tma_store_2d(&tm_h.m[2], xh, y, out_buf0 + 2 * kSB, pol_h);
              }
              ptx::bulk_commit_group();
            }
          }
        }
      } else if constexpr (kForm == FORM_GEMM) {
        // Plain GEMM epilogue: fp32 accumulator -> bf16 (or fp32) -> staging -> TMA store, or
        // TMA reduce-add into the buffer of the rank that owns this row block.
        int x0, y;
        chunk_xy(g, x0, y);
        g += T::kChunksPerTile;
        const bool f32 = p.out_f32 != 0;
        int dst = 0, yy = y;
        if (p.reduce_rows > 0) {
          dst = y / p.reduce_rows;
          yy = y - dst * p.reduce_rows;
        } else if (splits > 1) {
          // this unit's K range has its own slot of slot_rows rows in the output tensor
          yy = y + ((cluster_id + i * num_clusters) % splits) * p.slot_rows;
        }
        const int units32 = tile_cols / 32;
        if (cluster_sum) {
          // ---- split-K summed in the cluster (one unit per CTA, cluster = the tile's ranges) ----
          if (!cluster_epilogue(std::integral_constant<int, 0>{}, i, as, t_row, x0, y, tile_cols,
                                tile_cols)) {
            ok = false;
            break;
          }
        } else {
        uint32_t nbuf = out_buf0;
        if (y >= p.M) {
          // rows that do not exist (short or ragged M): hand the accumulator back, store nothing
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader_base + 8 * as);
        }
#pragma unroll 1
        for (int u = (y < p.M) ? 0 : units32; u < units32; ++u) {
          const bool first = f32 || (u & 1) == 0;   // first 32-column unit of a staging buffer
          const bool last = f32 || (u & 1) == 1;    // buffer complete after this unit
          if (first) {
            if (lane == 0) ptx::bulk_wait_group_read<kOutBufs - 1>();
            __syncwarp();
            nbuf = out_buf0 + (gemm_stores & (kOutBufs - 1)) * kChunkBytes;
          }
          float acc[32];
          ptx::tmem_ld_32x32b_x32(t_row + u * 32, acc);
          ptx::tmem_ld_wait();
          if (u == units32 - 1) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader_base + 8 * as);
          }
          if (f32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t addr = nbuf + row_off + ((static_cast<uint32_t>(j) ^ row_sw) << 4);
              asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(acc[4 * j]),
                           "f"(acc[4 * j + 1]), "f"(acc[4 * j + 2]), "f"(acc[4 * j + 3])
                           : "memory");
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t addr =
                  nbuf + row_off + ((static_cast<uint32_t>((u & 1) * 4 + j) ^ row_sw) << 4);
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr),
                           "r"(pack_bf16x2(acc[8 * j], acc[8 * j + 1])),
                           "r"(pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3])),
                           "r"(pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5])),
                           "r"(pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]))
                           : "memory");
            }
          }
          if (last) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int x = x0 + (f32 ? u * 32 : (u >> 1) * 64);
              if (x < p.N && y < p.M) {
                if (p.reduce_rows > 0) {
                  if (p.reduce_add) {
                    ptx::tma_reduce_add_2d(&tm_h.m[dst], x, yy, nbuf);
                  } else {
                    ptx::tma_store_2d(&tm_h.m[dst], x, yy, nbuf, pol_h);
                  }
                } else {
                  for (int d = 0; d < p.n_dst; ++d)
                    ptx::tma_store_2d(&tm_h.m[d], x, yy, nbuf, pol_h);
                }
              }
              ptx::bulk_commit_group();
            }
            ++gemm_stores;
          }
        }
        }  // cluster sum / stores
      } else {
      if constexpr ((kForm == FORM_FUSED || kForm == FORM_SILU_MUL) && kCanSplitK) {
        if (cluster_sum) {
          int x0, y0;
          chunk_xy(g, x0, y0);
          g += T::kChunksPerTile;
          if (!cluster_epilogue(std::integral_constant<int, kForm == FORM_FUSED ? 1 : 2>{}, i, as,
                                t_row, x0, y0, kAccCols, T::kOutCols)) {
            ok = false;
            break;
          }
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < T::kChunksPerTile; ++c, ++g) {
        int x, y;
        chunk_xy(g, x, y);
        const uint32_t ubuf = up_buf0 + (g % kUpBufs) * kChunkBytes;
        const uint32_t obuf = kInPlace ? ubuf : out_buf0 + (g & (kOutBufs - 1)) * kChunkBytes;
        if constexpr (kForm == FORM_FUSED) {
          if (y >= p.M && p.peer_mode == 0) {
            // This warp's 32 rows lie below the last row of the problem (a tile of a short or
            // ragged M): nothing to read, compute or store.  Its share of the accumulator is
            // handed back and the TMEM ports are left to the warps that have rows.
            if (c == T::kChunksPerTile - 1) {
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader_base + 8 * as);
            }
            continue;
          }
        }

        if constexpr (kInPlace) {
          // The other buffer is free once the previous chunk's store has read it:
          // fetch the next `up` chunk into it while this chunk is processed.
          if (lane == 0) {
            ptx::bulk_wait_group_read<0>();
            if (up_issued < total_chunks) {
              issue_up(up_issued);
              ++up_issued;
            }
          }
        }

        if constexpr (kForm == FORM_SILU_MUL) {
          SGL_PROF_BEGIN(te1);
          const bool w = ptx::mbar_wait(my_bar_up + 8 * (g % kUpBufs), (g / kUpBufs) & 1u, limit,
                                        abort_flag);
          SGL_PROF_END(prof_up, te1);
          if (!__all_sync(0xffffffffu, w)) {
            if (lane == 0) report_error(kErrEpiUpWait, g, abort_flag);
            ok = false;
            break;
          }
        }
        // The staging buffer is free once the store issued two chunks ago has
        // finished reading it.
        if constexpr (!kInPlace) {
          if (lane == 0) ptx::bulk_wait_group_read<kOutBufs - 1>();
        }
        __syncwarp();

#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col = c * kChunkCols + half * 32;
          float gate[32];
          float upv[32];
          if constexpr (kForm == FORM_SILU_MUL) {
            ptx::tmem_ld_32x32b_x32(t_row + col, gate);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t addr =
                  ubuf + row_off + ((static_cast<uint32_t>(half * 4 + j) ^ row_sw) << 4);
              uint32_t r0, r1, r2, r3;
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                           : "r"(addr));
              const uint32_t rr[4] = {r0, r1, r2, r3};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                upv[j * 8 + 2 * e] = __uint_as_float(rr[e] << 16);
                upv[j * 8 + 2 * e + 1] = __uint_as_float(rr[e] & 0xffff0000u);
              }
            }
          } else {
            ptx::tmem_ld_32x32b_x32(t_row + col, upv);
            ptx::tmem_ld_32x32b_x32(t_row + T::kGateCol + col, gate);
          }
          ptx::tmem_ld_wait();
          if (c == T::kChunksPerTile - 1 && half == 1) {
            // Last TMEM read of this tile: hand the accumulator stage back to
            // the MMA issuer before finishing the math and the stores.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(tempty_leader_base + 8 * as);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int idx = j * 8 + 2 * e;
              w[e] = pack_bf16x2(silu_mul(gate[idx], upv[idx]),
                                 silu_mul(gate[idx + 1], upv[idx + 1]));
            }
            const uint32_t addr =
                obuf + row_off + ((static_cast<uint32_t>(half * 4 + j) ^ row_sw) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(w[0]),
                         "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (x < p.N && y < p.M && p.peer_mode != 2) {
            // One store per destination buffer (local, then peers over NVLink), all
            // reading the same staging buffer; they form one bulk group.
            for (int d = 0; d < p.n_dst; ++d) ptx::tma_store_2d(&tm_h.m[d], x, y, obuf, pol_h);
          }
          ptx::bulk_commit_group();
          if constexpr (kForm == FORM_SILU_MUL && !kInPlace) {
            // This chunk's `up` buffer has been read by every lane: refill it.
            if (up_issued < total_chunks) {
              issue_up(up_issued);
              ++up_issued;
            }
          }
        }
        if constexpr (kForm == FORM_FUSED) {
          if (p.peer_mode != 0) {
            // Copy the chunk out of the staging buffer with thread stores: 8 lanes cover one
            // 128-byte row, a warp instruction four rows; eight instructions per chunk and
            // destination.  (The buffer is refilled two chunks later, after a __syncwarp.)
            const int sub_row = lane >> 3, piece = lane & 7;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = it * 4 + sub_row;
              const uint32_t addr =
                  obuf + static_cast<uint32_t>(r) * 128u +
                  ((static_cast<uint32_t>(piece) ^ static_cast<uint32_t>(r & 7)) << 4);
              uint32_t v0, v1, v2, v3;
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                           : "r"(addr));
              const int grow = y + r, gcol = x + piece * 8;
              if (grow < p.M && gcol < p.N) {
                const long long off = (static_cast<long long>(grow) * p.peer_ld + gcol) * 2;
                if (p.peer_mode == 2) {
                  ptx::multimem_st_v4(reinterpret_cast<char*>(p.peer_ptr[0]) + off, v0, v1, v2, v3);
                } else {
                  for (int d = 0; d < p.n_peer; ++d)
                    ptx::st_global_v4(reinterpret_cast<char*>(p.peer_ptr[d]) + off, v0, v1, v2, v3);
                }
              }
            }
          }
        }
      }
      }  // form
      SGL_PROF_END(prof_busy, te_busy);
    }
    if (lane == 0 && q == 0) {
      SGL_TL(6);
      SGL_DBG_COUNT(2, ok ? my_tiles : 0);
      SGL_PROF_STORE(4, prof_tf);
      SGL_PROF_STORE(5, prof_up);
      SGL_PROF_STORE(6, prof_busy);
      SGL_PROF_STORE(7, my_tiles);
    }
    if (lane == 0) {
      // Before the CTA exits its staging buffers must have been READ by the last stores (the
      // writes themselves are tracked to completion by the memory system, as for any store);
      // stores or reductions into a peer's memory are waited for in full.
      if (p.n_dst > 1 || p.reduce_rows > 0 || p.peer_mode != 0) {
        ptx::bulk_wait_group<0>();
      } else {
        ptx::bulk_wait_group_read<0>();
      }
      if constexpr (kForm == FORM_SILU_MUL) {
        if (!ok) {
          // Drain `up` loads that were issued but never consumed.
          for (int gg = g; gg < up_issued; ++gg) {
            ptx::mbar_wait(my_bar_up + 8 * (gg % kUpBufs), (gg / kUpBufs) & 1u, 1000000ull,
                           abort_flag + 1 /* stays zero */);
          }
        }
      }
    }
  }

  // ---- teardown ----
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  // (cluster sum: peers may still be reading this CTA's partial tile; every path of every CTA
  // gets here, because every wait above is bounded)
  if (kCtaGroup == 2 || cluster_sum) ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<kCtaGroup>(tmem_base, kTmemCols);
    if (lane == 0) { SGL_TL(7); }
  }
}

}  // namespace sgl
