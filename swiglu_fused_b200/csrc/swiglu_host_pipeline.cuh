// Host-buffer pipeline: the operator for callers whose tensors live in HOST memory.
//
// One call copies x and the weight in, runs the fused kernel and copies h out, with the three
// overlapped on three streams.  The reference has no such path (its benchmarks create every
// tensor on the GPU, bench_fused.py:35-36, bench.py:35-37); this is what a host-side caller of
// matmul_fused_swiglu / matmul_silu_mul has to do around the launch, done once, natively.
//
// Schedule.  The device->host copy of h is the longest leg (h is the largest tensor), so the
// schedule is built to start it as early as possible:
//   phase 1  the first `first_rows` rows of x go in, then the weight goes in as column windows;
//            after each window one launch computes h[0:first_rows, window] and its copy out
//            starts at once - the first bytes of h leave after one window, not after the
//            whole weight;
//   phase 2  the remaining rows in blocks of `block_rows`: copy in, launch over all columns,
//            copy out.
// With copy_weight = 0 (weight already resident from an earlier run) only row blocks are used.
//
// Shared weight (several GPUs, one process each, the same weight on all of them).  The weight
// is then the one tensor every rank would copy from the host in full.  Instead each rank
// copies only its own column slice (1/world of the weight) over PCIe and pushes it into the
// other ranks' weight buffers over NVLink (peer copies on a fourth stream, then one flag word
// per slice, stored by a one-thread kernel); a rank's launch over a peer's slice is preceded by
// a one-thread kernel that waits, with the library's time limit, for that flag.  The weight
// buffers are double buffered by run parity, so nobody overwrites a slice a slower rank is
// still computing on.  The buffers live in memory the caller maps into every rank
// (sgl_host_pipeline_create_shared).
//
// Unlike the rest of the library these functions allocate (create), free (destroy) and
// synchronise (run returns when h_host is complete).  Included by swiglu_abi.cu.

#pragma once

#include <vector>

namespace {

struct PipeStep {
  int64_t r0, r1;       // rows of x / h
  int64_t c0, c1;       // output columns
  bool copy_rows;       // x[r0:r1] goes in first
  bool copy_window;     // the weight's columns [c0, c1) go in first
  int wait_owner;       // >= 0: these columns are rank wait_owner's slice, wait for its flag
  bool last_own;        // last window of this rank's own slice: tell the peers afterwards
};

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Restores the caller's current device when a pipeline call returns.
struct DeviceRestore {
  int prev = -1;
  DeviceRestore() {
    if (cudaGetDevice(&prev) != cudaSuccess) {
      prev = -1;
      cudaGetLastError();
    }
  }
  ~DeviceRestore() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Flag protocol of the shared-weight mode.  A flag word lives in the memory of the rank that
// WAITS on it and is stored by the rank that owns the slice, after its peer copies (stream
// order on the owner's push stream).  Values only grow (run counter + 1).
__global__ void pipe_flag_store_kernel(uint32_t* flag, uint32_t value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

constexpr unsigned kErrPipeFlagWait = 0x201;

// One thread polls a flag in this GPU's own memory until it reaches `value`; gives up after
// limit_ns, records the time-out in g_status (the host reads it after the run) and returns.
__global__ void pipe_flag_wait_kernel(const uint32_t* flag, uint32_t value, uint64_t limit_ns,
                                      unsigned owner) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - value) >= 0) return;
    __nanosleep(200);
    if ((it & 63u) == 0u) {
      const uint64_t now = sgl::ptx::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        if (atomicCAS(&sgl::g_status[0], 0u, kErrPipeFlagWait) == 0u) {
          sgl::g_status[1] = owner;
          sgl::g_status[2] = value;
        }
        atomicAdd(&sgl::g_status[3], 1u);
        return;
      }
    }
  }
}

}  // namespace

struct sgl_host_pipeline {
  int device = 0;
  int form = 0;
  int64_t M = 0, N = 0, K = 0;
  bool has_cfg = false;
  sgl_config cfg{};
  char* x_d = nullptr;
  char* w_d = nullptr;          // weight buffer (shared mode: the copy of the current parity)
  char* up_d = nullptr;
  char* h_d = nullptr;
  int64_t device_bytes = 0;
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr, s_peer = nullptr;
  cudaEvent_t ev_peer = nullptr;
  // shared-weight mode (world > 1): every rank's region = two weight copies + flag words
  int world = 1, rank = 0;
  bool shared = false;
  std::vector<char*> region;    // [world] base of each rank's region, as mapped here
  int64_t w_copy_bytes = 0;     // bytes of one weight copy
  uint32_t runs_with_weight = 0;
  int resident_parity = -1;     // parity of the last run that copied the weight
  int64_t own_c0 = 0, own_c1 = 0;
  std::vector<cudaEvent_t> ev_in, ev_run;
  std::vector<PipeStep> with_weight, rows_only;
};

namespace {

int copy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width,
            int64_t rows, cudaMemcpyKind kind, cudaStream_t s, const char* what) {
  cudaError_t e;
  if (dpitch == width && spitch == width)
    e = cudaMemcpyAsync(dst, src, static_cast<size_t>(width * rows), kind, s);
  else
    e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dpitch), src, static_cast<size_t>(spitch),
                          static_cast<size_t>(width), static_cast<size_t>(rows), kind, s);
  if (e != cudaSuccess) return fail_cuda(e, what);
  return SGL_OK;
}

void pipeline_free(sgl_host_pipeline* p) {
  for (cudaEvent_t e : p->ev_in) cudaEventDestroy(e);
  for (cudaEvent_t e : p->ev_run) cudaEventDestroy(e);
  if (p->s_in) cudaStreamDestroy(p->s_in);
  if (p->s_run) cudaStreamDestroy(p->s_run);
  if (p->s_out) cudaStreamDestroy(p->s_out);
  if (p->s_peer) cudaStreamDestroy(p->s_peer);
  if (p->ev_peer) cudaEventDestroy(p->ev_peer);
  cudaFree(p->x_d);
  if (!p->shared) cudaFree(p->w_d);
  cudaFree(p->up_d);
  cudaFree(p->h_d);
  cudaGetLastError();
  delete p;
}

}  // namespace

namespace {

constexpr int64_t kPipeFlagBytes = 1024;    // flag words at the end of a shared region

int64_t pipe_weight_cols(int form, int64_t N) { return form == SGL_FORM_FUSED_SWIGLU ? 2 * N : N; }

// The schedule of one run: which rows and columns each step computes, what it copies in first
// and whose weight slice it has to wait for.  Pure host arithmetic (no device), shared by
// create and by sgl_host_pipeline_plan.
void build_pipe_plan(int64_t M, int64_t N, int64_t first_rows, int64_t block_rows, int windows,
                     bool shared, int world, int rank, std::vector<PipeStep>* with_weight,
                     std::vector<PipeStep>* rows_only, int64_t* own_c0, int64_t* own_c1) {
  *own_c0 = 0;
  *own_c1 = N;
  // Defaults: the first block is 3/16 of the rows (long enough that, per weight window, the
  // output produced keeps the copy-out leg busy), later blocks 1/16; eight weight windows.
  if (first_rows == 0) first_rows = round_up((3 * M + 15) / 16, 256);
  if (block_rows == 0) block_rows = round_up((M + 15) / 16, 256);
  if (block_rows < 1024) block_rows = 1024;
  if (first_rows > M) first_rows = M;
  if (windows == 0) windows = 8;

  // Weight windows of the first block.  Alone: `windows` windows over all columns.  Shared: this
  // rank's own slice first (cut into windows / world windows, each pushed to the peers as soon
  // as it is here), then the peers' slices in the order they arrive (every rank pushes to its
  // successors in turn, so the predecessors' slices land first).
  if (!shared) {
    const int64_t wcols = round_up((N + windows - 1) / windows, 256);
    for (int64_t c = 0; c < N; c += wcols)
      with_weight->push_back({0, first_rows, c, c + wcols < N ? c + wcols : N, c == 0, true, -1,
                                false});
  } else {
    int64_t c0 = 0, cnt = 0;
    sgl_shard_range(N, 256, world, rank, &c0, &cnt);
    *own_c0 = c0;
    *own_c1 = c0 + cnt;
    int sub = windows / world;
    if (sub < 1) sub = 1;
    const int64_t wcols = cnt > 0 ? round_up((cnt + sub - 1) / sub, 128) : 0;
    bool first = true;
    for (int64_t c = c0; c < c0 + cnt; c += wcols) {
      const int64_t e = c + wcols < c0 + cnt ? c + wcols : c0 + cnt;
      with_weight->push_back({0, first_rows, c, e, first, true, -1, e == c0 + cnt});
      first = false;
    }
    if (cnt == 0)   // nothing of its own to send: still owes x's first rows and the flags
      with_weight->push_back({0, first_rows, 0, 0, true, false, -1, true});
    for (int d = 1; d < world; ++d) {
      const int q = (rank - d + world) % world;
      int64_t q0 = 0, qn = 0;
      sgl_shard_range(N, 256, world, q, &q0, &qn);
      if (qn > 0) with_weight->push_back({0, first_rows, q0, q0 + qn, false, false, q, false});
    }
  }
  for (int64_t r = first_rows; r < M; r += block_rows)
    with_weight->push_back({r, r + block_rows < M ? r + block_rows : M, 0, N, true, false, -1,
                              false});
  for (int64_t r = 0; r < M; r += block_rows)
    rows_only->push_back({r, r + block_rows < M ? r + block_rows : M, 0, N, true, false, -1,
                            false});
}

int pipeline_create(int form, int64_t M, int64_t N, int64_t K, int64_t first_rows,
                    int64_t block_rows, int windows, const sgl_config* cfg, int world, int rank,
                    void* const* regions, sgl_host_pipeline** out) {
  if (!out) return fail(SGL_ERR_NULL_POINTER, "out is NULL");
  *out = nullptr;
  if (form != SGL_FORM_FUSED_SWIGLU && form != SGL_FORM_SILU_MUL)
    return fail(SGL_ERR_BAD_ARGUMENT, "form %d: the pipeline runs the fused_swiglu and silu_mul forms",
                form);
  int rc;
  if ((rc = validate_shape(M, N, K))) return rc;
  if (first_rows < 0 || block_rows < 0 || windows < 0 || windows > 64)
    return fail(SGL_ERR_BAD_ARGUMENT,
                "first_rows=%lld, block_rows=%lld must be >= 0 and windows=%d in [0, 64]",
                static_cast<long long>(first_rows), static_cast<long long>(block_rows), windows);
  const bool shared = regions != nullptr;
  if (shared) {
    if (world < 1 || world > 64 || rank < 0 || rank >= world)
      return fail(SGL_ERR_BAD_ARGUMENT, "world=%d rank=%d: need 1 <= world <= 64, 0 <= rank < world",
                  world, rank);
    for (int r = 0; r < world; ++r) {
      if ((rc = validate_ptr(regions[r], "regions[r]"))) return rc;
    }
  }
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;

  sgl_host_pipeline* p = new sgl_host_pipeline;
  cudaGetDevice(&p->device);
  p->form = form;
  p->M = M;
  p->N = N;
  p->K = K;
  p->shared = shared;
  p->world = shared ? world : 1;
  p->rank = shared ? rank : 0;
  if (cfg) {
    p->cfg = *cfg;
    p->has_cfg = true;
  }

  build_pipe_plan(M, N, first_rows, block_rows, windows, shared, p->world, p->rank,
                  &p->with_weight, &p->rows_only, &p->own_c0, &p->own_c1);

  const int64_t w_cols = pipe_weight_cols(form, N);
  p->w_copy_bytes = round_up(2 * K * w_cols, 256);
  cudaError_t e = cudaSuccess;
  auto alloc = [&](char** ptr, int64_t bytes) {
    p->device_bytes += bytes;
    return cudaMalloc(reinterpret_cast<void**>(ptr), static_cast<size_t>(bytes));
  };
  if (shared) {
    for (int r = 0; r < world; ++r) p->region.push_back(static_cast<char*>(regions[r]));
    p->w_d = p->region[rank];
  }
  if ((e = alloc(&p->x_d, 2 * M * K)) != cudaSuccess ||
      (!shared && (e = alloc(&p->w_d, 2 * K * w_cols)) != cudaSuccess) ||
      (e = alloc(&p->h_d, 2 * M * N)) != cudaSuccess ||
      (form == SGL_FORM_SILU_MUL && (e = alloc(&p->up_d, 2 * M * N)) != cudaSuccess) ||
      (e = cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking)) != cudaSuccess ||
      (shared && (e = cudaStreamCreateWithFlags(&p->s_peer, cudaStreamNonBlocking)) != cudaSuccess) ||
      (shared && (e = cudaEventCreateWithFlags(&p->ev_peer, cudaEventDisableTiming)) != cudaSuccess)) {
    pipeline_free(p);
    return fail_cuda(e, "sgl_host_pipeline_create");
  }
  const size_t n_ev = p->with_weight.size() > p->rows_only.size() ? p->with_weight.size()
                                                                  : p->rows_only.size();
  for (size_t i = 0; i < 2 * n_ev; ++i) {
    cudaEvent_t ev = nullptr;
    if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) {
      pipeline_free(p);
      return fail_cuda(e, "cudaEventCreateWithFlags");
    }
    (i < n_ev ? p->ev_in : p->ev_run).push_back(ev);
  }
  *out = p;
  return SGL_OK;
}

}  // namespace

extern "C" {

int sgl_host_pipeline_create(int form, int64_t M, int64_t N, int64_t K, int64_t first_rows,
                             int64_t block_rows, int windows, const sgl_config* cfg,
                             sgl_host_pipeline** out) {
  return pipeline_create(form, M, N, K, first_rows, block_rows, windows, cfg, 1, 0, nullptr, out);
}

int sgl_host_pipeline_plan(int64_t M, int64_t N, int64_t first_rows, int64_t block_rows,
                           int windows, int world, int rank, int copy_weight, int max_steps,
                           sgl_pipe_step* steps) {
  if (M < 1 || N < 1 || N % 8 != 0 || first_rows < 0 || block_rows < 0 || windows < 0 ||
      windows > 64 || world < 1 || world > 64 || rank < 0 || rank >= world || max_steps < 0 ||
      (max_steps > 0 && !steps))
    return fail(SGL_ERR_BAD_ARGUMENT, "bad pipeline plan request");
  std::vector<PipeStep> with_weight, rows_only;
  int64_t c0 = 0, c1 = 0;
  // world == 1 plans the single-GPU schedule (column windows over the whole weight)
  build_pipe_plan(M, N, first_rows, block_rows, windows, world > 1, world, rank, &with_weight,
                  &rows_only, &c0, &c1);
  const std::vector<PipeStep>& plan = copy_weight ? with_weight : rows_only;
  const int n = static_cast<int>(plan.size());
  for (int i = 0; i < n && i < max_steps; ++i) {
    steps[i].row0 = plan[i].r0;
    steps[i].row1 = plan[i].r1;
    steps[i].col0 = plan[i].c0;
    steps[i].col1 = plan[i].c1;
    steps[i].copies_rows = plan[i].copy_rows ? 1 : 0;
    steps[i].copies_weight_window = plan[i].copy_window ? 1 : 0;
    steps[i].waits_for_rank = plan[i].wait_owner;
    steps[i].signals_peers = (plan[i].last_own && world > 1) ? 1 : 0;
  }
  return n;
}

int64_t sgl_host_pipeline_shared_bytes(int form, int64_t N, int64_t K) {
  if (form != SGL_FORM_FUSED_SWIGLU && form != SGL_FORM_SILU_MUL) return SGL_ERR_BAD_ARGUMENT;
  if (validate_shape(8, N, K)) return SGL_ERR_BAD_SHAPE;
  return 2 * round_up(2 * K * pipe_weight_cols(form, N), 256) + kPipeFlagBytes;
}

int sgl_host_pipeline_create_shared(int form, int64_t M, int64_t N, int64_t K, int64_t first_rows,
                                    int64_t block_rows, int windows, const sgl_config* cfg,
                                    int world, int rank, void* const* regions,
                                    sgl_host_pipeline** out) {
  if (!regions) return fail(SGL_ERR_NULL_POINTER, "regions is NULL");
  return pipeline_create(form, M, N, K, first_rows, block_rows, windows, cfg, world, rank,
                         regions, out);
}

int sgl_host_pipeline_run(sgl_host_pipeline* p, const void* x_host, int64_t ldx,
                          const void* w_host, int64_t ldw, const void* up_host, int64_t ldup,
                          void* h_host, int64_t ldh, int copy_weight) {
  if (!p) return fail(SGL_ERR_NULL_POINTER, "pipeline is NULL");
  if (!x_host || !h_host) return fail(SGL_ERR_NULL_POINTER, "x_host or h_host is NULL");
  if (copy_weight && !w_host) return fail(SGL_ERR_NULL_POINTER, "w_host is NULL");
  const bool silu_mul = p->form == SGL_FORM_SILU_MUL;
  if (silu_mul && !up_host) return fail(SGL_ERR_NULL_POINTER, "up_host is NULL");
  const int64_t N = p->N, K = p->K;
  const int64_t w_cols = silu_mul ? N : 2 * N;
  if (ldx < K || ldh < N || (copy_weight && ldw < w_cols) || (silu_mul && ldup < N))
    return fail(SGL_ERR_BAD_STRIDE, "a host pitch is smaller than the row it must hold");
  if (p->shared && !copy_weight && p->resident_parity < 0)
    return fail(SGL_ERR_BAD_ARGUMENT, "copy_weight = 0 before any run has copied the weight");
  DeviceRestore restore;
  cudaError_t e = cudaSetDevice(p->device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");

  // Shared mode: this run's weight copy (by parity) in every rank's region, and the flag
  // words behind the two copies: flags[parity][owner].
  int parity = 0;
  uint32_t flag_value = 0;
  if (p->shared) {
    if (copy_weight) {
      parity = static_cast<int>(p->runs_with_weight & 1u);
      flag_value = p->runs_with_weight + 1;
    } else {
      parity = p->resident_parity;
    }
    p->w_d = p->region[p->rank] + parity * p->w_copy_bytes;
  }
  auto flag_of = [&](int holder, int owner) {
    return reinterpret_cast<uint32_t*>(p->region[holder] + 2 * p->w_copy_bytes) +
           parity * p->world + owner;
  };
  const uint64_t wait_ns = g_wait_limit_ns.load();

  const char* xh = static_cast<const char*>(x_host);
  const char* wh = static_cast<const char*>(w_host);
  const char* uh = static_cast<const char*>(up_host);
  char* hh = static_cast<char*>(h_host);
  const sgl_config* cfg = p->has_cfg ? &p->cfg : nullptr;
  const std::vector<PipeStep>& steps = copy_weight ? p->with_weight : p->rows_only;
  int rc = SGL_OK;
  for (size_t i = 0; i < steps.size() && rc == SGL_OK; ++i) {
    const PipeStep& s = steps[i];
    const int64_t rows = s.r1 - s.r0, cols = s.c1 - s.c0;
    // ---- in
    if (s.copy_rows)
      rc = copy_2d(p->x_d + 2 * s.r0 * K, 2 * K, xh + 2 * s.r0 * ldx, 2 * ldx, 2 * K, rows,
                   cudaMemcpyHostToDevice, p->s_in, "copy of x");
    if (rc == SGL_OK && s.copy_window) {
      rc = copy_2d(p->w_d + 2 * s.c0, 2 * w_cols, wh + 2 * s.c0, 2 * ldw, 2 * cols, K,
                   cudaMemcpyHostToDevice, p->s_in, "copy of the weight");
      if (rc == SGL_OK && !silu_mul)
        rc = copy_2d(p->w_d + 2 * (N + s.c0), 2 * w_cols, wh + 2 * (N + s.c0), 2 * ldw, 2 * cols,
                     K, cudaMemcpyHostToDevice, p->s_in, "copy of the weight");
    }
    if (rc == SGL_OK && silu_mul && cols > 0)
      rc = copy_2d(p->up_d + 2 * (s.r0 * N + s.c0), 2 * N, uh + 2 * (s.r0 * ldup + s.c0),
                   2 * ldup, 2 * cols, rows, cudaMemcpyHostToDevice, p->s_in, "copy of up");
    if (rc != SGL_OK) break;
    if ((e = cudaEventRecord(p->ev_in[i], p->s_in)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(p->s_run, p->ev_in[i], 0)) != cudaSuccess) {
      rc = fail_cuda(e, "event between copy-in and launch");
      break;
    }
    // ---- shared weight: pass this window on to the peers, then (after the last window of the
    // slice) raise this rank's flag on every peer
    if (p->shared && copy_weight && (s.copy_window || s.last_own) && p->world > 1) {
      if ((e = cudaStreamWaitEvent(p->s_peer, p->ev_in[i], 0)) != cudaSuccess) {
        rc = fail_cuda(e, "event between copy-in and the peer copies");
        break;
      }
      for (int d = 1; d < p->world && rc == SGL_OK; ++d) {
        const int q = (p->rank + d) % p->world;
        char* dst = p->region[q] + parity * p->w_copy_bytes;
        if (s.copy_window) {
          rc = copy_2d(dst + 2 * s.c0, 2 * w_cols, p->w_d + 2 * s.c0, 2 * w_cols, 2 * cols, K,
                       cudaMemcpyDeviceToDevice, p->s_peer, "peer copy of the weight");
          if (rc == SGL_OK && !silu_mul)
            rc = copy_2d(dst + 2 * (N + s.c0), 2 * w_cols, p->w_d + 2 * (N + s.c0), 2 * w_cols,
                         2 * cols, K, cudaMemcpyDeviceToDevice, p->s_peer,
                         "peer copy of the weight");
        }
        if (rc == SGL_OK && s.last_own) {
          pipe_flag_store_kernel<<<1, 1, 0, p->s_peer>>>(flag_of(q, p->rank), flag_value);
          if ((e = cudaGetLastError()) != cudaSuccess) rc = fail_cuda(e, "flag store launch");
          g_launches.fetch_add(1);
        }
      }
      if (rc != SGL_OK) break;
    }
    if (cols == 0) continue;   // a rank without columns of its own has nothing to compute here
    // ---- run
    if (s.wait_owner >= 0 && copy_weight) {
      pipe_flag_wait_kernel<<<1, 1, 0, p->s_run>>>(flag_of(p->rank, s.wait_owner), flag_value,
                                                    wait_ns, static_cast<unsigned>(s.wait_owner));
      if ((e = cudaGetLastError()) != cudaSuccess) {
        rc = fail_cuda(e, "flag wait launch");
        break;
      }
      g_launches.fetch_add(1);
    }
    char* h_blk = p->h_d + 2 * (s.r0 * N + s.c0);
    if (silu_mul)
      rc = sgl_matmul_silu_mul(p->x_d + 2 * s.r0 * K, p->w_d + 2 * s.c0,
                               p->up_d + 2 * (s.r0 * N + s.c0), h_blk, rows, cols, K, K, N, N, N,
                               cfg, p->s_run);
    else
      rc = sgl_matmul_fused_swiglu(p->x_d + 2 * s.r0 * K, p->w_d, h_blk, rows, cols, K, K, 2 * N,
                                   N, s.c0, N + s.c0, cfg, p->s_run);
    if (rc != SGL_OK) break;
    if ((e = cudaEventRecord(p->ev_run[i], p->s_run)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(p->s_out, p->ev_run[i], 0)) != cudaSuccess) {
      rc = fail_cuda(e, "event between launch and copy-out");
      break;
    }
    // ---- out
    rc = copy_2d(hh + 2 * (s.r0 * ldh + s.c0), 2 * ldh, h_blk, 2 * N, 2 * cols, rows,
                 cudaMemcpyDeviceToHost, p->s_out, "copy of h");
  }
  // Drain everything that was queued, also after an error, so that no copy is in flight into
  // the caller's buffers when this returns.
  cudaError_t e_in = cudaStreamSynchronize(p->s_in);
  cudaError_t e_run = cudaStreamSynchronize(p->s_run);
  cudaError_t e_out = cudaStreamSynchronize(p->s_out);
  cudaError_t e_peer = p->s_peer ? cudaStreamSynchronize(p->s_peer) : cudaSuccess;
  if (p->shared && copy_weight) {
    // the peers advance their counters whatever happened here: stay in step with them
    p->runs_with_weight += 1;
    if (rc == SGL_OK) p->resident_parity = parity;
  }
  if (rc != SGL_OK) return rc;
  if (e_in != cudaSuccess) return fail_cuda(e_in, "copy-in stream");
  if (e_run != cudaSuccess) return fail_cuda(e_run, "launch stream");
  if (e_out != cudaSuccess) return fail_cuda(e_out, "copy-out stream");
  if (e_peer != cudaSuccess) return fail_cuda(e_peer, "peer-copy stream");
  if (p->shared && copy_weight && p->world > 1) {
    // a flag wait that ran out means some columns were computed from a weight that had not
    // arrived: report it instead of returning a wrong h
    unsigned int st[8];
    e = cudaMemcpyFromSymbol(st, sgl::g_status, sizeof(st));
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyFromSymbol(status)");
    if (st[0] == kErrPipeFlagWait) {
      const unsigned int zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      cudaMemcpyToSymbol(sgl::g_status, zero, sizeof(zero));
      return fail(SGL_ERR_DEVICE_STATUS,
                  "rank %d: the weight slice of rank %u did not arrive within the wait limit "
                  "(every rank of the group must call run the same number of times)",
                  p->rank, st[1]);
    }
  }
  return SGL_OK;
}

int sgl_host_pipeline_query(const sgl_host_pipeline* p, int what, int64_t* out) {
  if (!p || !out) return fail(SGL_ERR_NULL_POINTER, "pipeline or out is NULL");
  const int64_t w_cols = p->form == SGL_FORM_SILU_MUL ? p->N : 2 * p->N;
  const int64_t up = p->form == SGL_FORM_SILU_MUL ? 2 * p->M * p->N : 0;
  // weight bytes THIS rank copies from the host per run: all of it alone, its own slice shared
  const int64_t w_host_bytes =
      p->shared ? 2 * p->K * (p->own_c1 - p->own_c0) * (p->form == SGL_FORM_SILU_MUL ? 1 : 2)
                : 2 * p->K * w_cols;
  int64_t launches = 0;
  for (const PipeStep& s : p->with_weight) {
    if (s.c1 > s.c0) launches += 1 + (s.wait_owner >= 0 ? 1 : 0);
    if (s.last_own && p->shared) launches += p->world - 1;
  }
  switch (what) {
    case SGL_PIPE_H2D_BYTES: *out = 2 * p->M * p->K + w_host_bytes + up; break;
    case SGL_PIPE_H2D_BYTES_NO_WEIGHT: *out = 2 * p->M * p->K + up; break;
    case SGL_PIPE_D2H_BYTES: *out = 2 * p->M * p->N; break;
    case SGL_PIPE_LAUNCHES: *out = launches; break;
    case SGL_PIPE_LAUNCHES_NO_WEIGHT: *out = static_cast<int64_t>(p->rows_only.size()); break;
    case SGL_PIPE_DEVICE_BYTES: *out = p->device_bytes; break;
    case SGL_PIPE_PEER_BYTES:
      *out = p->shared ? w_host_bytes * (p->world - 1) : 0;
      break;
    default: return fail(SGL_ERR_BAD_ARGUMENT, "unknown pipeline query %d", what);
  }
  return SGL_OK;
}

int sgl_host_pipeline_destroy(sgl_host_pipeline* p) {
  if (!p) return SGL_OK;
  DeviceRestore restore;
  cudaError_t e = cudaSetDevice(p->device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
  pipeline_free(p);
  return SGL_OK;
}

}  // extern "C"
