// Single-process multi-GPU launcher: one host thread drives the fused SwiGLU stage on up to 8
// GPUs that the calling process owns.  The reference is single-GPU (its launch layer binds one
// context, swiglu/_pycuda_loader.py:47-55); this is the C-level counterpart of the
// one-process-per-GPU launchers in the Python package, for hosts that keep all devices in one
// process.  Nothing here waits on the host and no kernel waits on another kernel: ordering
// between devices is expressed with events that the devices' streams wait on.
//
// Modes (the partition is sgl_shard_range's, so it agrees with the per-process launchers):
//   M_SHARD         device r computes its row range; x[r], h[r] hold only those rows; the
//                   packed weight is replicated; no data crosses between devices.
//   N_SHARD         device r computes its column range for all rows, reading the up and gate
//                   column windows of the unsplit weight in place; h[r] is the local
//                   [M, columns of r] block; no data crosses between devices.
//   N_SHARD_GATHER  as N_SHARD, but every h[d] is a full [M, N] buffer and the epilogue of
//                   device r stores each finished tile into the column range of r in EVERY
//                   h[d] (its own first, then the peers' through peer access): the all-gather
//                   rides on the kernel.  Needs peer access between all devices.
// Included by swiglu_abi.cu.

#pragma once

struct sgl_mgpu {
  int n = 0;
  int dev[8] = {};
  bool peer_ok = true;
  cudaEvent_t ev_pre[8] = {};
  cudaEvent_t ev_post[8] = {};
};

namespace {

void mgpu_free(sgl_mgpu* g) {
  for (int r = 0; r < g->n; ++r) {
    if (cudaSetDevice(g->dev[r]) != cudaSuccess) continue;
    if (g->ev_pre[r]) cudaEventDestroy(g->ev_pre[r]);
    if (g->ev_post[r]) cudaEventDestroy(g->ev_post[r]);
  }
  cudaGetLastError();
  delete g;
}

// Every stream waits for an event recorded on every other stream: a barrier in stream order,
// with no host wait and nothing spinning on a device.
int mgpu_stream_barrier(sgl_mgpu* g, cudaEvent_t* ev, void* const* streams) {
  cudaError_t e;
  for (int r = 0; r < g->n; ++r) {
    if ((e = cudaSetDevice(g->dev[r])) != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
    cudaStream_t s = streams ? static_cast<cudaStream_t>(streams[r]) : nullptr;
    if ((e = cudaEventRecord(ev[r], s)) != cudaSuccess) return fail_cuda(e, "cudaEventRecord");
  }
  for (int d = 0; d < g->n; ++d) {
    if ((e = cudaSetDevice(g->dev[d])) != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
    cudaStream_t s = streams ? static_cast<cudaStream_t>(streams[d]) : nullptr;
    for (int r = 0; r < g->n; ++r) {
      if (r == d) continue;
      if ((e = cudaStreamWaitEvent(s, ev[r], 0)) != cudaSuccess)
        return fail_cuda(e, "cudaStreamWaitEvent");
    }
  }
  return SGL_OK;
}

}  // namespace

extern "C" {

int sgl_mgpu_create(int n, const int* devices, sgl_mgpu** out) {
  if (!out) return fail(SGL_ERR_NULL_POINTER, "out is NULL");
  *out = nullptr;
  if (!devices) return fail(SGL_ERR_NULL_POINTER, "devices is NULL");
  if (n < 1 || n > 8) return fail(SGL_ERR_BAD_ARGUMENT, "n=%d devices: must be 1..8", n);
  int count = 0, prev = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDeviceCount");
  for (int r = 0; r < n; ++r) {
    if (devices[r] < 0 || devices[r] >= count)
      return fail(SGL_ERR_BAD_ARGUMENT, "devices[%d]=%d but the process sees %d device(s)", r,
                  devices[r], count);
  }
  if ((e = cudaGetDevice(&prev)) != cudaSuccess) return fail_cuda(e, "cudaGetDevice");

  sgl_mgpu* g = new sgl_mgpu;
  g->n = n;
  int rc = SGL_OK;
  for (int r = 0; r < n && rc == SGL_OK; ++r) {
    g->dev[r] = devices[r];
    if ((e = cudaSetDevice(devices[r])) != cudaSuccess) {
      rc = fail_cuda(e, "cudaSetDevice");
      break;
    }
    DeviceInfo* info = nullptr;
    if ((rc = check_device(&info))) break;
    if ((e = cudaEventCreateWithFlags(&g->ev_pre[r], cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&g->ev_post[r], cudaEventDisableTiming)) != cudaSuccess) {
      rc = fail_cuda(e, "cudaEventCreateWithFlags");
      break;
    }
    for (int j = 0; j < n; ++j) {
      if (devices[j] == devices[r]) continue;
      int can = 0;
      if ((e = cudaDeviceCanAccessPeer(&can, devices[r], devices[j])) != cudaSuccess) {
        rc = fail_cuda(e, "cudaDeviceCanAccessPeer");
        break;
      }
      if (!can) {
        g->peer_ok = false;
        continue;
      }
      e = cudaDeviceEnablePeerAccess(devices[j], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
      } else if (e != cudaSuccess) {
        rc = fail_cuda(e, "cudaDeviceEnablePeerAccess");
        break;
      }
    }
  }
  cudaSetDevice(prev);
  if (rc != SGL_OK) {
    mgpu_free(g);
    cudaSetDevice(prev);
    return rc;
  }
  *out = g;
  return SGL_OK;
}

int sgl_mgpu_fused_swiglu(sgl_mgpu* g, int mode, const void* const* x, const void* const* w,
                          void* const* h, int64_t M, int64_t N, int64_t K, int64_t ldx,
                          int64_t ldw, int64_t ldh, const sgl_config* cfg,
                          void* const* streams) {
  if (!g) return fail(SGL_ERR_NULL_POINTER, "group is NULL");
  if (!x || !w || !h) return fail(SGL_ERR_NULL_POINTER, "x, w or h pointer array is NULL");
  if (mode != SGL_MGPU_M_SHARD && mode != SGL_MGPU_N_SHARD && mode != SGL_MGPU_N_SHARD_GATHER)
    return fail(SGL_ERR_BAD_ARGUMENT, "unknown mode %d", mode);
  int rc;
  if ((rc = validate_shape(M, N, K))) return rc;
  if (mode == SGL_MGPU_N_SHARD_GATHER && !g->peer_ok)
    return fail(SGL_ERR_BAD_ARGUMENT,
                "N_SHARD_GATHER needs peer access between all devices of the group");
  for (int r = 0; r < g->n; ++r) {
    // a device whose shard is empty is skipped, so only the gathered h must exist everywhere
    if (mode == SGL_MGPU_N_SHARD_GATHER && !h[r])
      return fail(SGL_ERR_NULL_POINTER, "h[%d] is NULL", r);
  }
  int prev = 0;
  cudaError_t e = cudaGetDevice(&prev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");

  if (mode == SGL_MGPU_N_SHARD_GATHER && g->n > 1)
    rc = mgpu_stream_barrier(g, g->ev_pre, streams);   // every h[d] is free before any peer writes it
  for (int r = 0; r < g->n && rc == SGL_OK; ++r) {
    int64_t begin = 0, count = 0;
    rc = sgl_shard_range(mode == SGL_MGPU_M_SHARD ? M : N, mode == SGL_MGPU_M_SHARD ? 256 : 128,
                         g->n, r, &begin, &count);
    if (rc != SGL_OK || count == 0) continue;
    if (!x[r] || !w[r] || !h[r]) {
      rc = fail(SGL_ERR_NULL_POINTER, "x[%d], w[%d] or h[%d] is NULL", r, r, r);
      break;
    }
    if ((e = cudaSetDevice(g->dev[r])) != cudaSuccess) {
      rc = fail_cuda(e, "cudaSetDevice");
      break;
    }
    void* stream = streams ? streams[r] : nullptr;
    if (mode == SGL_MGPU_M_SHARD) {
      rc = sgl_matmul_fused_swiglu(x[r], w[r], h[r], count, N, K, ldx, ldw, ldh, 0, N, cfg,
                                   stream);
    } else if (mode == SGL_MGPU_N_SHARD) {
      rc = sgl_matmul_fused_swiglu(x[r], w[r], h[r], M, count, K, ldx, ldw, ldh, begin,
                                   N + begin, cfg, stream);
    } else {
      // own buffer first, then the peers in ring order, so that at any moment the devices
      // are writing to different destinations
      void* dsts[8];
      for (int d = 0; d < g->n; ++d)
        dsts[d] = static_cast<char*>(h[(r + d) % g->n]) + 2 * begin;
      if (ldh < N) {
        rc = fail(SGL_ERR_BAD_STRIDE, "ldh=%lld is smaller than the %lld columns of the gathered h",
                  static_cast<long long>(ldh), static_cast<long long>(N));
        break;
      }
      rc = fused_swiglu_impl(x[r], w[r], 0, dsts, g->n, nullptr, 0, M, count, K, ldx, ldw, ldh,
                             begin, N + begin, cfg, stream);
    }
  }
  if (rc == SGL_OK && mode == SGL_MGPU_N_SHARD_GATHER && g->n > 1)
    rc = mgpu_stream_barrier(g, g->ev_post, streams);  // every stream sees the whole h afterwards
  cudaSetDevice(prev);
  return rc;
}

int sgl_mgpu_size(const sgl_mgpu* g) { return g ? g->n : 0; }

int sgl_mgpu_destroy(sgl_mgpu* g) {
  if (!g) return SGL_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  mgpu_free(g);
  cudaSetDevice(prev);
  cudaGetLastError();
  return SGL_OK;
}

}  // extern "C"
