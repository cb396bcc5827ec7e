// Backward elementwise step of the SwiGLU stage (HBM bound, no tensor cores):
//   grad_preact[:, 0:N]  = dy * silu(gate)            (gradient w.r.t. up   = x @ W_up)
//   grad_preact[:, N:2N] = dy * up * silu'(gate)      (gradient w.r.t. gate = x @ W_gate)
// from the two factors the side-store forward saved, factors = [silu(gate) | up * silu'(gate)].
// Column order matches the packed weight [W_up | W_gate], so grad_x = grad_preact @ W^T and
// grad_W = x^T @ grad_preact need no reshuffle.  Counterpart of
// _swiglu_grad_preact_normal_kernel (swiglu/triton/impls.py:3947-3993), which recomputes
// the sigmoid from saved pre-activations instead.
//
// One thread moves 8 bf16 (16 bytes) per operand; the grid is a multiple of the SM count
// and strides over the rows.  `out` may alias `factors` (each thread reads its elements
// before it writes them).  Algorithmic bytes: 10 * M * N (three reads, two writes).
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace sgl {

__device__ __forceinline__ uint32_t mul_bf16x2_f32(uint32_t a, uint32_t b) {
  const float a0 = __uint_as_float(a << 16), a1 = __uint_as_float(a & 0xffff0000u);
  const float b0 = __uint_as_float(b << 16), b1 = __uint_as_float(b & 0xffff0000u);
  __nv_bfloat162 r = __floats2bfloat162_rn(a0 * b0, a1 * b1);
  return *reinterpret_cast<uint32_t*>(&r);
}

__global__ void __launch_bounds__(256)
grad_preact_kernel(const uint4* __restrict__ dy, const uint4* factors, uint4* out, int M,
                   int n_vec,            // N / 8
                   int64_t lddy_vec, int64_t ldf_vec, int64_t ldo_vec) {
  const int64_t total = static_cast<int64_t>(M) * n_vec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // Two independent 16-byte vectors per thread and iteration: six loads in flight before the
  // first store.
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += 2 * stride) {
    const int64_t j = i + stride;
    const bool two = j < total;
    const int64_t row0 = i / n_vec, v0 = i - row0 * n_vec;
    const int64_t row1 = two ? j / n_vec : row0, v1 = two ? j - row1 * n_vec : v0;
    const uint4 g0 = dy[row0 * lddy_vec + v0];
    const uint4 s0 = factors[row0 * ldf_vec + v0];
    const uint4 d0 = factors[row0 * ldf_vec + n_vec + v0];
    const uint4 g1 = dy[row1 * lddy_vec + v1];
    const uint4 s1 = factors[row1 * ldf_vec + v1];
    const uint4 d1 = factors[row1 * ldf_vec + n_vec + v1];
    uint4 o;
    o.x = mul_bf16x2_f32(g0.x, s0.x); o.y = mul_bf16x2_f32(g0.y, s0.y);
    o.z = mul_bf16x2_f32(g0.z, s0.z); o.w = mul_bf16x2_f32(g0.w, s0.w);
    out[row0 * ldo_vec + v0] = o;
    o.x = mul_bf16x2_f32(g0.x, d0.x); o.y = mul_bf16x2_f32(g0.y, d0.y);
    o.z = mul_bf16x2_f32(g0.z, d0.z); o.w = mul_bf16x2_f32(g0.w, d0.w);
    out[row0 * ldo_vec + n_vec + v0] = o;
    if (two) {
      o.x = mul_bf16x2_f32(g1.x, s1.x); o.y = mul_bf16x2_f32(g1.y, s1.y);
      o.z = mul_bf16x2_f32(g1.z, s1.z); o.w = mul_bf16x2_f32(g1.w, s1.w);
      out[row1 * ldo_vec + v1] = o;
      o.x = mul_bf16x2_f32(g1.x, d1.x); o.y = mul_bf16x2_f32(g1.y, d1.y);
      o.z = mul_bf16x2_f32(g1.z, d1.z); o.w = mul_bf16x2_f32(g1.w, d1.w);
      out[row1 * ldo_vec + n_vec + v1] = o;
    }
  }
}

// out[r, c] = bf16( sum over s of f32(slots[s][r, c]) ): the local half of a reduce-scatter
// whose partial products were written by every rank into its own slot of this GPU's
// buffer.  Summation in fp32 in slot order, so the result is deterministic.  HBM bound:
// (n_slots + 1) * rows * cols * 2 bytes.
__global__ void __launch_bounds__(256)
sum_slots_kernel(const uint4* __restrict__ slots, uint4* __restrict__ out, int n_slots,
                 int64_t slot_stride_vec, int rows, int n_vec, int64_t lds_vec,
                 int64_t ldo_vec) {
  const int64_t total = static_cast<int64_t>(rows) * n_vec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t row = i / n_vec;
    const int64_t v = i - row * n_vec;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f, a5 = 0.f, a6 = 0.f, a7 = 0.f;
    for (int s = 0; s < n_slots; ++s) {
      const uint4 t = slots[s * slot_stride_vec + row * lds_vec + v];
      a0 += __uint_as_float(t.x << 16);
      a1 += __uint_as_float(t.x & 0xffff0000u);
      a2 += __uint_as_float(t.y << 16);
      a3 += __uint_as_float(t.y & 0xffff0000u);
      a4 += __uint_as_float(t.z << 16);
      a5 += __uint_as_float(t.z & 0xffff0000u);
      a6 += __uint_as_float(t.w << 16);
      a7 += __uint_as_float(t.w & 0xffff0000u);
    }
    uint4 o;
    __nv_bfloat162 r;
    r = __floats2bfloat162_rn(a0, a1); o.x = *reinterpret_cast<uint32_t*>(&r);
    r = __floats2bfloat162_rn(a2, a3); o.y = *reinterpret_cast<uint32_t*>(&r);
    r = __floats2bfloat162_rn(a4, a5); o.z = *reinterpret_cast<uint32_t*>(&r);
    r = __floats2bfloat162_rn(a6, a7); o.w = *reinterpret_cast<uint32_t*>(&r);
    out[row * ldo_vec + v] = o;
  }
}

// Same for fp32 slots (split-K partial tiles): out = bf16(sum of fp32 partials).
__global__ void __launch_bounds__(256)
sum_slots_f32_kernel(const float4* __restrict__ slots, uint4* __restrict__ out, int n_slots,
                     int64_t slot_stride_vec4, int rows, int n_vec, int64_t lds_vec4,
                     int64_t ldo_vec) {
  const int64_t total = static_cast<int64_t>(rows) * n_vec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // Launched with programmatic stream serialisation right behind the kernel that writes the
  // slots: this grid may be set up while that kernel is still running, and waits here until it
  // has finished and its writes are visible (a no-op for an ordinary launch).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t row = i / n_vec;
    const int64_t v = i - row * n_vec;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    for (int s = 0; s < n_slots; ++s) {
      const float4* src = slots + s * slot_stride_vec4 + row * lds_vec4 + 2 * v;
      const float4 t0 = src[0], t1 = src[1];
      a0.x += t0.x; a0.y += t0.y; a0.z += t0.z; a0.w += t0.w;
      a1.x += t1.x; a1.y += t1.y; a1.z += t1.z; a1.w += t1.w;
    }
    uint4 o;
    __nv_bfloat162 r;
    r = __floats2bfloat162_rn(a0.x, a0.y); o.x = *reinterpret_cast<uint32_t*>(&r);
    r = __floats2bfloat162_rn(a0.z, a0.w); o.y = *reinterpret_cast<uint32_t*>(&r);
    r = __floats2bfloat162_rn(a1.x, a1.y); o.z = *reinterpret_cast<uint32_t*>(&r);
    r = __floats2bfloat162_rn(a1.z, a1.w); o.w = *reinterpret_cast<uint32_t*>(&r);
    out[row * ldo_vec + v] = o;
  }
}

}  // namespace sgl
