/*
 * swiglu_b200.h - C ABI of libswiglu_b200.so, the B200 (sm_100a) fused SwiGLU
 * gate/up stage.
 *
 * The library replaces, for one hot path, the launch layer + CUDA kernels of
 * tongzhou8086/swiglu_fused.  Citations are paths inside that project.
 *
 * Conventions
 *   - every tensor is bf16, row-major, addressed by a raw device pointer and a
 *     leading dimension (row pitch) in ELEMENTS;
 *   - pointers must be 16-byte aligned and every leading dimension a multiple
 *     of 8 elements (TMA needs 16-byte rows); K and N must be multiples of 8;
 *     M is arbitrary (ragged tiles are zero-filled on load, clipped on store);
 *   - inputs are borrowed for the duration of the enqueue only; the library
 *     never allocates device memory and never synchronises unless stated;
 *   - `stream` is a cudaStream_t / CUstream passed as void* (NULL = default);
 *   - the first launch of a kernel variant on a device raises its shared-memory limit and
 *     queries the cluster occupancy (cudaFuncSetAttribute, cudaOccupancyMaxActiveClusters);
 *     make that first call outside stream capture - later calls only encode tensor maps on
 *     the host and launch;
 *   - functions return 0 on success, a negative sgl_status on invalid use and a
 *     positive cudaError_t value when the CUDA runtime or driver failed;
 *     sgl_last_error() describes the last failure of the calling thread.
 */
#ifndef SWIGLU_B200_H_
#define SWIGLU_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sgl_status {
  SGL_OK = 0,
  SGL_ERR_NULL_POINTER = -1,
  SGL_ERR_BAD_SHAPE = -2,      /* M,N,K < 1, or K/N not a multiple of 8 */
  SGL_ERR_BAD_STRIDE = -3,     /* leading dimension too small or not a multiple of 8 */
  SGL_ERR_MISALIGNED = -4,     /* pointer or column offset not 16-byte aligned */
  SGL_ERR_BAD_CONFIG = -5,     /* tile configuration not supported / does not fit */
  SGL_ERR_NO_DRIVER = -6,      /* cuTensorMapEncodeTiled could not be resolved */
  SGL_ERR_UNSUPPORTED_DEVICE = -7, /* current device is not compute capability 10.x */
  SGL_ERR_TENSOR_MAP = -8,     /* cuTensorMapEncodeTiled rejected a descriptor */
  SGL_ERR_DEVICE_STATUS = -9,  /* a kernel reported a bounded-wait timeout */
  SGL_ERR_BAD_ARGUMENT = -10
} sgl_status;

/* Operator forms. */
enum {
  SGL_FORM_SILU_MUL = 0,
  SGL_FORM_FUSED_SWIGLU = 1,
  SGL_FORM_MATMUL = 2,
  SGL_FORM_FUSED_SWIGLU_SAVE = 3
};

/*
 * One entry of the tile table.  Replaces the reference's (BN, BK, NS, GSM)
 * tuples, swiglu/matmul_silu_mul.py:30-41 and swiglu/matmul_fused_swiglu.py:34-41.
 * BM is 128 rows per CTA and an accumulator is 256 columns wide in every entry (the `wide`
 * entries of the fused form use two of them per tile).
 */
typedef struct sgl_config {
  int32_t cta_group; /* 1 = one CTA per 128-row tile, 2 = CTA pair per 256-row tile */
  int32_t block_k;   /* 64 or 128 */
  int32_t stages;    /* shared-memory ring depth; 0 = deepest that fits */
  int32_t group_m;   /* GROUP_SIZE_M of the tile order, in cluster-tile rows; >= 1 */
  int32_t max_ctas;  /* cap on the persistent grid (0 = all SMs); for tests and sweeps */
  int32_t l2_hints;  /* L2 eviction priorities, 2 bits each: bits 0-1 x loads, 2-3 weight
                        loads, 4-5 h stores, 6-7 `up` loads; 0 normal, 1 evict-first,
                        2 evict-last.  0 = all normal. */
  int32_t group_n;   /* column slabs of the tile order, in tiles: the tile columns are walked in
                        slabs of group_n, all row bands of one slab before the next slab, so
                        that a slab of the weight stays in L2 while x streams past it;
                        0 = one slab (plain GROUP_SIZE_M order) */
  int32_t wide;      /* 1 = tiles of 256 output columns instead of 128 (fused_swiglu form with
                        cta_group 2, block_k 64 and the [K, 2N] weight layout only): half the x
                        traffic per output and half as many tiles, for problems of a few
                        hundred rows; one accumulator stage, so no epilogue overlap.  0 = off */
} sgl_config;

/*
 * h[M,N] = silu(x[M,K] @ w_gate[K,N]) * up[M,N]
 * Replaces matmul_silu_mul / _launch (swiglu/matmul_silu_mul.py:78-95,142-161)
 * and the kernels matmul_silu_mul_bm128_* (swiglu/_matmul_silu_mul.cu:657-681).
 * cfg may be NULL: the built-in tile table chooses.
  *
 * With cfg == NULL, M <= 128, K >= 4096 and few 256-column tiles, K is cut into ranges that run
 * as thread-block clusters, as described for sgl_matmul_fused_swiglu below; the CTA that sums a
 * group of gate columns reads up for it and applies the activation.
 */
int sgl_matmul_silu_mul(const void* x, const void* w_gate, const void* up, void* h, int64_t M,
                        int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldup, int64_t ldh,
                        const sgl_config* cfg, void* stream);

/*
 * h[M,N] = silu(x @ w[:, gate_col0 : gate_col0+N]) * (x @ w[:, up_col0 : up_col0+N])
 * For the reference's packed weight W[K,2N] = [W_up | W_gate] pass up_col0 = 0,
 * gate_col0 = N, ldw = 2N.  Other offsets let a column-parallel shard address
 * the unsplit weight in place.  Replaces matmul_fused_swiglu / _launch
 * (swiglu/matmul_fused_swiglu.py:85-103,152-172) and the kernels
 * matmul_fused_swiglu_bm128_* (swiglu/_matmul_fused_swiglu.cu:513-533).
 * x is streamed once: both products come from one K loop.
  *
 * With cfg == NULL, M <= 128, K >= 4096 and so few 128-column tiles that two-CTA clusters of
 * them all fit on the GPU at once (a narrow FFN at decode batch sizes) K is cut into 2 to 8
 * ranges that run as thread-block clusters; the CTAs of a cluster exchange their fp32 partial
 * tiles through distributed shared memory and each applies silu(gate) * up to the columns it
 * sums (64 x 4096 x 4096: 18 us instead of 30 us).  Deterministic; against whole-K tiles only the
 * order of the fp32 additions differs.  An explicit cfg, sgl_set_splitk_cluster_sum(0) or
 * SGL_SPLITK_CLUSTER_SUM=0 keep whole-K tiles.
 */
int sgl_matmul_fused_swiglu(const void* x, const void* w, void* h, int64_t M, int64_t N, int64_t K,
                            int64_t ldx, int64_t ldw, int64_t ldh, int64_t up_col0,
                            int64_t gate_col0, const sgl_config* cfg, void* stream);

/*
 * Same computation with the weight in checkpoint (nn.Linear) layout: w_nk[2N, K], row f holds
 * the K weights of output feature f; rows [up_row0, up_row0+N) are the up features and rows
 * [gate_row0, gate_row0+N) the gate features (N and 0.. for the usual [up; gate] stack), ldw
 * the row pitch (>= K).  No transpose or repack: the kernel reads the rows as a K-major B
 * operand.  Counterpart of the reference's pack/unpack helpers
 * (swiglu/triton/impls.py:1898-1917), which convert between the two layouts by copying.
 */
int sgl_matmul_fused_swiglu_nk(const void* x, const void* w_nk, void* h, int64_t M, int64_t N,
                               int64_t K, int64_t ldx, int64_t ldw, int64_t ldh, int64_t up_row0,
                               int64_t gate_row0, const sgl_config* cfg, void* stream);

/*
 * Training forward: h as above, and from the same epilogue the two factors the backward
 * pass needs, factors[M, 2N] = [ silu(gate) | up * silu'(gate) ] (bf16, row pitch ldf).
 * Counterpart of the reference's Triton side-store forward
 * (_fused_swiglu_wide_packed_save_factors_kernel, swiglu/triton/impls.py:384-468); the
 * factors are stored as two plain [M, N] halves, not chunk-interleaved.
 */
int sgl_matmul_fused_swiglu_save_factors(const void* x, const void* w, void* h, void* factors,
                                         int64_t M, int64_t N, int64_t K, int64_t ldx,
                                         int64_t ldw, int64_t ldh, int64_t ldf, int64_t up_col0,
                                         int64_t gate_col0, const sgl_config* cfg, void* stream);

/*
 * Backward elementwise step: grad_preact[M, 2N] = [ dy * factors[:, :N] | dy * factors[:, N:] ]
 * = [ d/d(up) | d/d(gate) ], in the column order of the packed weight, so that
 * grad_x = grad_preact @ W^T and grad_W = x^T @ grad_preact follow directly.  grad_preact may
 * alias factors (in place).  HBM bound: 10 * M * N bytes.  Counterpart of
 * _swiglu_grad_preact_normal_kernel (swiglu/triton/impls.py:3947-3993).
 */
int sgl_swiglu_grad_preact(const void* dy, const void* factors, void* grad_preact, int64_t M,
                           int64_t N, int64_t lddy, int64_t ldf, int64_t ldo, void* stream);

/*
 * Same computation, but every output tile is written to n_dsts (1..8) buffers:
 * h_dsts[i] is the address of element (0, 0) of this launch's [M, N] block inside
 * destination i (all with row pitch ldh).  Destinations may be peer-GPU memory
 * mapped into this process (plain TMA stores over NVLink, no multicast).  This is
 * the all-gather of the column-parallel launch fused into the kernel: rank r
 * computes columns [c0, c0+N) and stores them into that column window of every
 * rank's full-width h.  The caller synchronises the ranks before reading.
 * The reference is single-GPU; no counterpart there.
 */
int sgl_matmul_fused_swiglu_multi_dst(const void* x, const void* w, void* const* h_dsts,
                                      int n_dsts, int64_t M, int64_t N, int64_t K, int64_t ldx,
                                      int64_t ldw, int64_t ldh, int64_t up_col0,
                                      int64_t gate_col0, const sgl_config* cfg, void* stream);

/*
 * sgl_matmul_fused_swiglu whose epilogue also delivers every finished tile to other GPUs: the
 * all-gather of a column-parallel launch inside the kernel, by ordinary stores instead of the
 * TMA stores of sgl_matmul_fused_swiglu_multi_dst.  (TMA stores to a peer queue up behind the
 * link in the same per-SM unit that fetches the operands, and the mainloop then waits with
 * them; stores issued by the epilogue warps only ever hold up those warps.)
 *   h_local      element (0, 0) of this launch's [M, N] block in THIS GPU's buffer (TMA store);
 *   h_peers[i]   the same element in peer i's buffer, mapped into this process, i < n_peers <= 8:
 *                each tile is copied there with 16-byte stores over NVLink;
 *   h_multicast  if not NULL, h_peers is ignored: the address of that element in an NVSwitch
 *                multicast mapping of all the buffers (this GPU's included).  Each tile is then
 *                stored ONCE with multimem.st and the switch replicates it, so the sender's
 *                link carries 1/world of the gathered bytes; h_local is not written separately.
 * All destinations share the row pitch ldh.  The caller owns the buffers and synchronises the
 * ranks before and after (nobody may still read a buffer that is being overwritten, nobody
 * reads before every rank's stores have landed).  The reference is single-GPU; no counterpart.
 */
int sgl_matmul_fused_swiglu_gather(const void* x, const void* w, void* h_local,
                                   void* const* h_peers, int n_peers, void* h_multicast,
                                   int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                                   int64_t ldh, int64_t up_col0, int64_t gate_col0,
                                   const sgl_config* cfg, void* stream);

/*
 * c[M,N] = a[M,K] @ b[K,N], bf16 in, fp32 accumulate, bf16 out: the down projection
 * y = h @ W_down that consumes the stage's output, on the same TMA/tcgen05 pipeline.
 * With cfg == NULL, M <= 256 and K >= 4096 (decode batch sizes) K may be cut into ranges that
 * run as thread-block clusters and sum themselves through distributed shared memory, where a
 * CTA then loads at most 4/5 of the operand bytes a whole-K tile does (64 x 14336 x 4096: 27 us
 * instead of 80 us; 256 x 14336 x 4096: 37 us instead of 82-94 us).  The result stays deterministic; against the whole-K kernel only the
 * order of the fp32 additions differs.  An explicit cfg, sgl_set_splitk_cluster_sum(0) or
 * SGL_SPLITK_CLUSTER_SUM=0 keep whole-K tiles.  The reference stops at h; no counterpart there.
 */
int sgl_matmul_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, const sgl_config* cfg, void* stream);

/*
 * sgl_matmul_bf16 with either operand stored transposed, read in place (no transpose copy):
 *   a_transposed != 0: a is stored [K, M] (row pitch lda >= M, M a multiple of 8);
 *   b_transposed != 0: b is stored [N, K] (row pitch ldb >= K).
 * K must be a multiple of 8 except with a_transposed != 0 and b_transposed == 0, where K only
 * counts rows of both operands and may be any value >= 1 (a ragged token count).
 * These are the two GEMMs of the backward pass over the packed weight W[K, 2N]:
 *   grad_x[M, K]  = grad_preact[M, 2N] @ W^T   -> b = W,  b_transposed = 1
 *   grad_W[K, 2N] = x^T @ grad_preact          -> a = x,  a_transposed = 1
 * (the reference issues them through cuBLAS on two streams,
 * _packed_grad_input_weight, swiglu/triton/impls.py:100-124).
 */
int sgl_matmul_bf16_ex(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, int a_transposed,
                       int b_transposed, const sgl_config* cfg, void* stream);

/*
 * Split-K form of sgl_matmul_bf16 for short, deep problems (few output tiles, large K - the
 * down projection at decode batch sizes): K is cut into `splits` ranges (0 = choose: as many as
 * fill one wave of SMs), each
 * range's partial tile is written in fp32 to its slot of `scratch`, and a second kernel adds
 * the slots in fp32, in order (deterministic), into c (bf16).  `scratch` is device memory the
 * caller owns; sgl_matmul_bf16_splitk_scratch_bytes says how much this problem needs
 * (negative sgl_status on a bad shape).  Contents of scratch are overwritten; two calls that
 * overlap on the GPU must not share it.  No counterpart in the reference.
 *
 * Where the K ranges of a tile can run as one thread-block cluster (single-CTA tiles - M <= 128
 * with the default configuration -, 2 to 16 ranges, all clusters resident at once) neither the
 * scratch nor the second kernel is used: every CTA keeps its fp32 partial tile in shared
 * memory, the CTAs of a cluster read one another's (distributed shared memory) and each sums
 * and stores its share of the tile.  The additions are the same in the same order, so the
 * result is the two-kernel form's bit for bit; a K range that never reports is a bounded
 * wait (code 0x106 in sgl_device_status).  sgl_set_splitk_cluster_sum(0), or
 * SGL_SPLITK_CLUSTER_SUM=0 in the environment, keeps every problem on the two-kernel form;
 * the call returns the previous setting.
 */
int64_t sgl_matmul_bf16_splitk_scratch_bytes(int64_t M, int64_t N, int64_t K, int splits);
int sgl_set_splitk_cluster_sum(int enabled);
/*
 * The plan the library makes for a problem of up to 256 rows whose K ranges are to be summed in
 * thread-block clusters, given how many clusters of n CTAs the GPU can hold at once
 * (clusters_that_fit[n] for n = 2..8; index 0 and 1 unused; what cudaOccupancyMaxActiveClusters
 * says for the GEMM kernel - 74, 45, 33, 26, 22, 15, 15 on a B200).  Among tile widths of 256,
 * 192, 128 and 64 columns and 2 to 8 ranges of at least 512 of K whose clusters all fit, the
 * plan whose CTAs each load the fewest operand bytes (K extent of a range x (rows of a +
 * columns of b)) wins, the wider tile on a tie.  Returns the number of CTAs (0 = no such plan)
 * and writes the tile width, the number of ranges and the K extent of a range (a multiple of
 * 128); negative sgl_status on bad arguments.  No device is touched.
 */
int sgl_splitk_cluster_plan(int64_t M, int64_t N, int64_t K, const int* clusters_that_fit,
                            int* tile_cols, int* ranges, int* k_per_range);
int sgl_matmul_bf16_splitk(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                           int64_t lda, int64_t ldb, int64_t ldc, int splits, void* scratch,
                           int64_t scratch_bytes, const sgl_config* cfg, void* stream);

/*
 * sgl_matmul_bf16_splitk for callers that cannot hand over device memory of their own.
 * (This entry point has no counterpart in the reference.)
 *
 * Who that is: code that runs where every byte of device memory has already been given to
 * somebody else's pool (an inference server that reserves the whole GPU for its KV cache and
 * exposes no allocator to plug-ins), or on a path where cudaMalloc is off limits because it
 * synchronises the device or may fail late (a latency-critical decode loop, a callback from
 * another library).  Such a caller still owns a, b and c, but has nowhere to put the fp32
 * partial tiles.  Here they go into an 8 MiB array that is part of the library image on
 * every GPU that loads it; the call itself performs no allocation of any kind.
 *
 * Limits and rules:
 *   - splits x round_up(M, 32) x N x 4 bytes must fit 8 MiB (8388608); otherwise
 *     SGL_ERR_BAD_ARGUMENT with the sizes in sgl_last_error().  splits = 0 picks the largest
 *     useful number of ranges that fits (down to 1, which must fit too).
 *     Example that just fits: M <= 64, N = 4096, 8 K ranges.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and remembers it; make that first
 *     call before any stream capture begins on the device.
 *   - All calls on one GPU share the one array.  Its contents after a call are that call's
 *     partial tiles; nothing has to be cleared beforehand, because every element the summing
 *     kernel reads is written earlier in the same call.  Two calls that can run at the same
 *     time on one GPU (different streams, different host threads) race on it: serialise them
 *     or use sgl_matmul_bf16_splitk with separate scratch.
 * Results are identical to sgl_matmul_bf16_splitk for the same arguments and the same number
 * of K ranges (pass `splits` explicitly where the two must agree bit for bit: here an
 * automatic choice is lowered until it fits the 8 MiB, there it is not).
 */
int sgl_matmul_bf16_splitk_static(const void* a, const void* b, void* c, int64_t M, int64_t N,
                                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int splits,
                                  const sgl_config* cfg, void* stream);

/*
 * Row-parallel form of the same product with the scatter half of a reduce-scatter fused in:
 * destination d owns rows [d*rows_per_dst, (d+1)*rows_per_dst) of the [M, N] result and
 * dsts[d] is the address of a [rows_per_dst, N] buffer on it (row pitch ldc; element type
 * fp32 if dst_is_f32 else bf16), which may be peer-GPU memory mapped into this process.
 * rows_per_dst must be a multiple of 32.
 *   accumulate = 0: each tile of this rank's partial product a @ b is STORED (plain TMA
 *     stores over NVLink) into the owner's buffer, which is this rank's private slot there;
 *     the owner then adds its slots with sgl_sum_bf16_slots.  Deterministic, fp32 sums.
 *   accumulate = 1: each tile is ADDED (TMA reduce, atomic per element) into a buffer all
 *     ranks share, which must hold its initial value (normally zero) before any rank
 *     launches.  Into fp32 the order of additions does not matter at bf16 output precision;
 *     into bf16 every contribution rounds and the order (hence the last bit) varies run to
 *     run.  Fastest form with a bf16 buffer; an fp32 buffer doubles the NVLink bytes.
 * first_dst: the tile order starts with the rows owned by this destination and wraps around;
 * rank r of a group passes (r + 1) % world (or any rotation) so that at every moment the
 * ranks send to different owners instead of all swamping the same one.
 * The caller synchronises the ranks before and after.  No counterpart in the reference
 * (single GPU, no down projection).
 */
int sgl_matmul_bf16_reduce_scatter(const void* a, const void* b, void* const* dsts, int n_dsts,
                                   int64_t rows_per_dst, int dst_is_f32, int accumulate,
                                   int first_dst, int64_t M, int64_t N, int64_t K, int64_t lda,
                                   int64_t ldb, int64_t ldc, const sgl_config* cfg, void* stream);

/*
 * out[rows, cols] = bf16( sum over s < n_slots of slots[s * slot_stride + r * lds + c] ), summed
 * in fp32 in slot order: the reduce half of the reduce-scatter above (HBM bound).
 * slot_stride, lds and ldo are in elements.  No counterpart in the reference.
 */
int sgl_sum_bf16_slots(const void* slots, int n_slots, int64_t slot_stride, void* out,
                       int64_t rows, int64_t cols, int64_t lds, int64_t ldo, void* stream);

/*
 * Tile table access.  Replaces the module-level config lists and _legal /
 * _legal_for_problem (swiglu/matmul_silu_mul.py:46-51,101-111).
 * sgl_config_count: number of built-in configurations for a form.
 * sgl_config_get:   copy configuration i (stages filled in with the deepest ring).
 * sgl_config_default: the configuration a NULL cfg would use for this problem.
 * sgl_config_smem_bytes: dynamic shared memory a configuration needs, or a
 *                   negative sgl_status if it is not supported.
 */
int sgl_config_count(int form);
int sgl_config_get(int form, int index, sgl_config* out);
int sgl_config_default(int form, int64_t M, int64_t N, int64_t K, sgl_config* out);
int sgl_config_smem_bytes(int form, const sgl_config* cfg);

/*
 * Tile order of the persistent schedule: the (tile row, tile column) that linear
 * tile index t maps to.  Host copy of the device function, exported so the
 * order can be checked without a GPU.  Counterpart of the block-id swizzle in
 * swiglu/_matmul_silu_mul.cu:357-384.
 */
int sgl_tile_coord(int64_t t, int64_t tiles_m, int64_t tiles_n, int64_t group_m, int64_t* tile_m,
                   int64_t* tile_n);
/* The same with column slabs of group_n tiles (sgl_config.group_n; 0 = one slab). */
int sgl_tile_coord_slabs(int64_t t, int64_t tiles_m, int64_t tiles_n, int64_t group_m,
                         int64_t group_n, int64_t* tile_m, int64_t* tile_n);

/* Queries about the current device (no counterpart in the reference). */
enum {
  SGL_QUERY_SM_COUNT = 0,
  SGL_QUERY_MAX_SMEM_OPTIN = 1,
  SGL_QUERY_COMPUTE_CAPABILITY = 2, /* major*10 + minor */
  SGL_QUERY_KERNEL_LAUNCHES = 3     /* kernels launched by this process through this library */
};
int sgl_query(int what, int64_t* out);

/*
 * Contiguous balanced partition used by the multi-GPU launchers: shard `rank`
 * of `world` gets [*begin, *begin + *count) of `total` items, every boundary a
 * multiple of `align` (the last shard takes the ragged tail).  Rows of x/h for
 * the M-sharded launch, columns of W/h for the column-parallel launch.  The
 * reference is single-GPU; this has no counterpart there.
 */
int sgl_shard_range(int64_t total, int64_t align, int world, int rank, int64_t* begin,
                    int64_t* count);

/*
 * Device-side error record.  Every wait inside the kernels is bounded; a wait
 * that runs out records {code, block, detail, count} and the kernel exits.
 * sgl_device_status synchronises the current device, copies the 8 status words
 * to `words` (may be NULL), clears them, and returns SGL_ERR_DEVICE_STATUS if a
 * code was recorded.  The reference's waits spin forever
 * (swiglu/_matmul_silu_mul.cu:152-161).
 */
int sgl_device_status(uint32_t* words);
/*
 * Self-test of the bounded waits: launches one tiny kernel whose only thread waits, with the
 * given limit (<= 1 s), on a barrier nobody signals.  The wait must run out, the kernel must
 * record the time-out and exit normally; the next sgl_device_status then returns
 * SGL_ERR_DEVICE_STATUS with code 0x1ff and the context stays usable.  Nothing faults, traps
 * or hangs.  No counterpart in the reference.
 */
int sgl_selftest_wait_timeout(uint64_t limit_ns, void* stream);
/* Per-wait time limit in nanoseconds for kernels launched afterwards (default 2e9). */
int sgl_set_wait_limit_ns(uint64_t ns);

/*
 * Host-buffer pipeline: the fused_swiglu or silu_mul operator for a caller whose x, weight (and
 * up) and h live in HOST memory.  No counterpart in the reference, whose benchmarks create every
 * tensor on the GPU (bench_fused.py:35-36, bench.py:35-37); this is the work a host-side caller
 * has to do around the launch, overlapped: copies in, launches and copies out run on three
 * streams in row blocks.  Because h is the largest tensor, the schedule starts its copy out as
 * early as it can: the first `first_rows` rows are computed one weight column window at a time
 * while the weight is still arriving (`windows` windows), the rest in blocks of `block_rows`
 * rows over all columns.  0 for any of the three picks a default (3/16 of M, 1/16 of M, 8).
 *
 *   create   allocates the device buffers (x, weight, h, and up for silu_mul), three streams and
 *            the events on the current device; `form` is SGL_FORM_FUSED_SWIGLU (weight [K, 2N],
 *            up columns first) or SGL_FORM_SILU_MUL (weight [K, N], plus up [M, N]).
 *   run      one pass; pitches in elements; up_host is ignored for fused_swiglu.  Returns after
 *            h_host is complete (synchronous).  Host buffers should be page-locked, otherwise
 *            the copies do not overlap.  copy_weight = 0 reuses the weight copied by an earlier
 *            run.  Not re-entrant: one run at a time per pipeline.
 *   query    bytes moved and kernels launched per run, device bytes held.
 *   destroy  frees everything create made; NULL is accepted.  The caller's current device is
 *            restored by run and destroy.
 * These are the only functions of the library that allocate device memory or block the host.
 */
typedef struct sgl_host_pipeline sgl_host_pipeline;
enum {
  SGL_PIPE_H2D_BYTES = 0,           /* per run with copy_weight = 1 */
  SGL_PIPE_H2D_BYTES_NO_WEIGHT = 1, /* per run with copy_weight = 0 */
  SGL_PIPE_D2H_BYTES = 2,
  SGL_PIPE_LAUNCHES = 3,            /* kernels per run with copy_weight = 1 */
  SGL_PIPE_LAUNCHES_NO_WEIGHT = 4,
  SGL_PIPE_DEVICE_BYTES = 5,
  SGL_PIPE_PEER_BYTES = 6           /* shared weight: bytes this rank pushes to peers per run */
};
int sgl_host_pipeline_create(int form, int64_t M, int64_t N, int64_t K, int64_t first_rows,
                             int64_t block_rows, int windows, const sgl_config* cfg,
                             sgl_host_pipeline** out);
/*
 * The pipeline for several GPUs (one process each) that run the SAME weight on different rows:
 * the weight crosses the host link once per group instead of once per rank.  Rank r copies only
 * its column slice of the weight (sgl_shard_range(N, 256, world, r); for fused_swiglu the up and
 * the gate columns of that range) from w_host, pushes it into the other ranks' weight buffers
 * with peer copies over NVLink and then stores a flag word there; a launch over another
 * rank's slice is preceded by a one-thread kernel that waits for that flag, for at most the
 * library's wait limit (a time-out makes run return SGL_ERR_DEVICE_STATUS, nothing hangs).
 * Each rank computes its first rows slice by slice as the slices arrive (its own first), the
 * remaining rows over all columns.
 *
 * regions[q], q in [0, world): device address, valid in THIS process, of rank q's region of
 * sgl_host_pipeline_shared_bytes(form, N, K) bytes (two weight copies, used alternately, and
 * the flag words) - e.g. one symmetric-memory allocation per rank, or buffers of one process
 * with peer access enabled.  The regions must be zero when the pipelines are created, stay
 * valid until they are destroyed, and are not freed by destroy.  Every rank must call run the
 * same number of times with the same copy_weight arguments, and each rank passes its own rows
 * of x and the WHOLE w_host (only its slice of it is read).  No counterpart in the reference.
 */
int64_t sgl_host_pipeline_shared_bytes(int form, int64_t N, int64_t K);
/*
 * The schedule a pipeline of these sizes follows in one run, without creating one (pure host
 * arithmetic, no device needed): step i computes rows [row0, row1) x output columns
 * [col0, col1) after copying in x's rows (copies_rows) and the weight's columns of that window
 * (copies_weight_window); waits_for_rank >= 0 names the rank whose weight slice the step has to
 * wait for, signals_peers marks the step after which this rank raises its flag on the peers.
 * world = 1 gives the single-GPU schedule of sgl_host_pipeline_create, world > 1 rank `rank`'s
 * schedule of sgl_host_pipeline_create_shared; copy_weight as in run.  Writes at most max_steps
 * entries and returns the number of steps of the schedule (negative sgl_status on bad input).
 */
typedef struct sgl_pipe_step {
  int64_t row0, row1, col0, col1;
  int32_t copies_rows, copies_weight_window, waits_for_rank, signals_peers;
} sgl_pipe_step;
int sgl_host_pipeline_plan(int64_t M, int64_t N, int64_t first_rows, int64_t block_rows,
                           int windows, int world, int rank, int copy_weight, int max_steps,
                           sgl_pipe_step* steps);
int sgl_host_pipeline_create_shared(int form, int64_t M, int64_t N, int64_t K, int64_t first_rows,
                                    int64_t block_rows, int windows, const sgl_config* cfg,
                                    int world, int rank, void* const* regions,
                                    sgl_host_pipeline** out);
int sgl_host_pipeline_run(sgl_host_pipeline* p, const void* x_host, int64_t ldx,
                          const void* w_host, int64_t ldw, const void* up_host, int64_t ldup,
                          void* h_host, int64_t ldh, int copy_weight);
int sgl_host_pipeline_query(const sgl_host_pipeline* p, int what, int64_t* out);
int sgl_host_pipeline_destroy(sgl_host_pipeline* p);

/*
 * Single-process multi-GPU launcher for the fused form: one host thread, up to 8 GPUs owned by
 * the calling process.  The reference is single-GPU (one context, swiglu/_pycuda_loader.py:47-55);
 * no counterpart there.  The partition is sgl_shard_range's (rows in multiples of 256, columns
 * in multiples of 128), the same as the one-process-per-GPU launchers use.
 *
 *   create   devices[0..n) are CUDA device ordinals (a device may be listed twice); enables peer
 *            access between them where the hardware allows, creates two events per device;
 *            the caller's current device is restored.
 *   fused_swiglu  x, w, h (and streams, or NULL for the null streams) are arrays of n per-device
 *            pointers; M, N, K are the GLOBAL sizes; pitches in elements, common to all devices.
 *       SGL_MGPU_M_SHARD         x[r]: rows of shard r, [rows_r, K]; w[r]: packed [K, 2N] replica;
 *                                h[r]: [rows_r, N].  No traffic between devices.
 *       SGL_MGPU_N_SHARD         x[r]: full [M, K] replica; w[r]: unsplit packed weight replica,
 *                                column windows read in place; h[r]: local block [M, cols_r]
 *                                (ldh >= cols_r).  No traffic between devices.
 *       SGL_MGPU_N_SHARD_GATHER  as N_SHARD, but each h[d] is a full [M, N] buffer (ldh >= N) and
 *                                device r's epilogue stores its columns into every h[d] (plain TMA
 *                                stores through peer access, no multicast): all-gather fused into
 *                                the kernel.  Before the launches every stream waits for an event
 *                                on every other stream (all h free), and again after them (every
 *                                stream then sees the whole h).  Needs peer access everywhere.
 *            Enqueues only: no host wait, and no kernel waits on another kernel.
 *   size     number of devices in the group (0 for NULL).
 *   destroy  frees the events; peer access stays enabled.  NULL is accepted.
 */
typedef struct sgl_mgpu sgl_mgpu;
enum { SGL_MGPU_M_SHARD = 0, SGL_MGPU_N_SHARD = 1, SGL_MGPU_N_SHARD_GATHER = 2 };
int sgl_mgpu_create(int n, const int* devices, sgl_mgpu** out);
int sgl_mgpu_fused_swiglu(sgl_mgpu* g, int mode, const void* const* x, const void* const* w,
                          void* const* h, int64_t M, int64_t N, int64_t K, int64_t ldx,
                          int64_t ldw, int64_t ldh, const sgl_config* cfg, void* const* streams);
int sgl_mgpu_size(const sgl_mgpu* g);
int sgl_mgpu_destroy(sgl_mgpu* g);

/* Message for the last non-zero return on the calling thread ("" if none). */
const char* sgl_last_error(void);

/* Library version, major*100 + minor. */
int sgl_version(void);

#ifdef __cplusplus
}
#endif

#endif /* SWIGLU_B200_H_ */
