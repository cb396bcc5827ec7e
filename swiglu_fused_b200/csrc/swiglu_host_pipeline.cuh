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
};

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct sgl_host_pipeline {
  int device = 0;
  int form = 0;
  int64_t M = 0, N = 0, K = 0;
  bool has_cfg = false;
  sgl_config cfg{};
  char* x_d = nullptr;
  char* w_d = nullptr;
  char* up_d = nullptr;
  char* h_d = nullptr;
  int64_t device_bytes = 0;
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
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
  cudaFree(p->x_d);
  cudaFree(p->w_d);
  cudaFree(p->up_d);
  cudaFree(p->h_d);
  cudaGetLastError();
  delete p;
}

}  // namespace

extern "C" {

int sgl_host_pipeline_create(int form, int64_t M, int64_t N, int64_t K, int64_t first_rows,
                             int64_t block_rows, int windows, const sgl_config* cfg,
                             sgl_host_pipeline** out) {
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
  DeviceInfo* info = nullptr;
  if ((rc = check_device(&info))) return rc;

  sgl_host_pipeline* p = new sgl_host_pipeline;
  cudaGetDevice(&p->device);
  p->form = form;
  p->M = M;
  p->N = N;
  p->K = K;
  if (cfg) {
    p->cfg = *cfg;
    p->has_cfg = true;
  }

  // Defaults: the first block is 3/16 of the rows (long enough that, per weight window, the
  // output produced keeps the copy-out leg busy), later blocks 1/16; eight weight windows.
  if (first_rows == 0) first_rows = round_up((3 * M + 15) / 16, 256);
  if (block_rows == 0) block_rows = round_up((M + 15) / 16, 256);
  if (block_rows < 1024) block_rows = 1024;
  if (first_rows > M) first_rows = M;
  if (windows == 0) windows = 8;
  int64_t wcols = round_up((N + windows - 1) / windows, 256);
  for (int64_t c = 0; c < N; c += wcols)
    p->with_weight.push_back({0, first_rows, c, c + wcols < N ? c + wcols : N, c == 0, true});
  for (int64_t r = first_rows; r < M; r += block_rows)
    p->with_weight.push_back({r, r + block_rows < M ? r + block_rows : M, 0, N, true, false});
  for (int64_t r = 0; r < M; r += block_rows)
    p->rows_only.push_back({r, r + block_rows < M ? r + block_rows : M, 0, N, true, false});

  const int64_t w_cols = form == SGL_FORM_FUSED_SWIGLU ? 2 * N : N;
  cudaError_t e;
  auto alloc = [&](char** ptr, int64_t bytes) {
    p->device_bytes += bytes;
    return cudaMalloc(reinterpret_cast<void**>(ptr), static_cast<size_t>(bytes));
  };
  if ((e = alloc(&p->x_d, 2 * M * K)) != cudaSuccess ||
      (e = alloc(&p->w_d, 2 * K * w_cols)) != cudaSuccess ||
      (e = alloc(&p->h_d, 2 * M * N)) != cudaSuccess ||
      (form == SGL_FORM_SILU_MUL && (e = alloc(&p->up_d, 2 * M * N)) != cudaSuccess) ||
      (e = cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking)) != cudaSuccess) {
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
  cudaError_t e = cudaSetDevice(p->device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");

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
    if (rc == SGL_OK && silu_mul)
      rc = copy_2d(p->up_d + 2 * (s.r0 * N + s.c0), 2 * N, uh + 2 * (s.r0 * ldup + s.c0),
                   2 * ldup, 2 * cols, rows, cudaMemcpyHostToDevice, p->s_in, "copy of up");
    if (rc != SGL_OK) break;
    if ((e = cudaEventRecord(p->ev_in[i], p->s_in)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(p->s_run, p->ev_in[i], 0)) != cudaSuccess) {
      rc = fail_cuda(e, "event between copy-in and launch");
      break;
    }
    // ---- run
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
  if (rc != SGL_OK) return rc;
  if (e_in != cudaSuccess) return fail_cuda(e_in, "copy-in stream");
  if (e_run != cudaSuccess) return fail_cuda(e_run, "launch stream");
  if (e_out != cudaSuccess) return fail_cuda(e_out, "copy-out stream");
  return SGL_OK;
}

int sgl_host_pipeline_query(const sgl_host_pipeline* p, int what, int64_t* out) {
  if (!p || !out) return fail(SGL_ERR_NULL_POINTER, "pipeline or out is NULL");
  const int64_t w_cols = p->form == SGL_FORM_SILU_MUL ? p->N : 2 * p->N;
  const int64_t up = p->form == SGL_FORM_SILU_MUL ? 2 * p->M * p->N : 0;
  switch (what) {
    case SGL_PIPE_H2D_BYTES: *out = 2 * p->M * p->K + 2 * p->K * w_cols + up; break;
    case SGL_PIPE_H2D_BYTES_NO_WEIGHT: *out = 2 * p->M * p->K + up; break;
    case SGL_PIPE_D2H_BYTES: *out = 2 * p->M * p->N; break;
    case SGL_PIPE_LAUNCHES: *out = static_cast<int64_t>(p->with_weight.size()); break;
    case SGL_PIPE_LAUNCHES_NO_WEIGHT: *out = static_cast<int64_t>(p->rows_only.size()); break;
    case SGL_PIPE_DEVICE_BYTES: *out = p->device_bytes; break;
    default: return fail(SGL_ERR_BAD_ARGUMENT, "unknown pipeline query %d", what);
  }
  return SGL_OK;
}

int sgl_host_pipeline_destroy(sgl_host_pipeline* p) {
  if (!p) return SGL_OK;
  cudaError_t e = cudaSetDevice(p->device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
  pipeline_free(p);
  return SGL_OK;
}

}  // extern "C"
