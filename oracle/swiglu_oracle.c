/*
 * Plain-C restatement of the fused SwiGLU gate/up stage.  TEST INFRASTRUCTURE
 * ONLY: built into oracle/libswiglu_oracle.so and called from tests/ to check
 * the torch oracle and the CUDA kernels independently of torch's CPU GEMM.
 * Never linked into, or called by, the product library.
 *
 * Follows the reference's fp32 check expressions:
 *   silu_mul form : bench.py:39-40        ref = silu(x_f32 @ Wg_f32) * up_f32
 *   fused form    : bench_fused.py:39-42  ref = silu((x@W)[:, N:]) * (x@W)[:, :N]
 * with the result rounded once to bf16 (round to nearest even).
 *
 * acc64 != 0 accumulates the dot products and evaluates the activation in
 * double precision (machine-independent values for the golden vectors);
 * acc64 == 0 accumulates in fp32 in plain k order, like a scalar fp32 GEMM.
 *
 * bf16 tensors are passed as uint16_t bit patterns, row-major with a leading
 * dimension in elements.  Single-threaded; callers split rows across threads.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float silu_f32(float g) { return g / (1.0f + expf(-g)); }
static inline double silu_f64(double g) { return g / (1.0 + exp(-g)); }

/* dot(x[row, :], w[:, col]) for one output element. */
static inline double dot64(const uint16_t* xr, const uint16_t* w, int64_t ldw, int64_t col,
                           int64_t K) {
  double acc = 0.0;
  for (int64_t k = 0; k < K; ++k)
    acc += (double)bf16_to_f32(xr[k]) * (double)bf16_to_f32(w[k * ldw + col]);
  return acc;
}

static inline float dot32(const uint16_t* xr, const uint16_t* w, int64_t ldw, int64_t col,
                          int64_t K) {
  float acc = 0.0f;
  for (int64_t k = 0; k < K; ++k) acc += bf16_to_f32(xr[k]) * bf16_to_f32(w[k * ldw + col]);
  return acc;
}

/* h = silu(x @ w_gate) * up */
int oracle_silu_mul(const uint16_t* x, const uint16_t* w_gate, const uint16_t* up, uint16_t* h,
                    int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldup,
                    int64_t ldh, int acc64) {
  if (!x || !w_gate || !up || !h || M < 0 || N < 0 || K < 0) return -1;
  for (int64_t m = 0; m < M; ++m) {
    const uint16_t* xr = x + m * ldx;
    for (int64_t n = 0; n < N; ++n) {
      const float u = bf16_to_f32(up[m * ldup + n]);
      float r;
      if (acc64) {
        r = (float)(silu_f64(dot64(xr, w_gate, ldw, n, K)) * (double)u);
      } else {
        r = silu_f32(dot32(xr, w_gate, ldw, n, K)) * u;
      }
      h[m * ldh + n] = f32_to_bf16_rne(r);
    }
  }
  return 0;
}

/* h = silu(x @ w[:, gate_col0:+N]) * (x @ w[:, up_col0:+N]) */
int oracle_fused_swiglu(const uint16_t* x, const uint16_t* w, uint16_t* h, int64_t M, int64_t N,
                        int64_t K, int64_t ldx, int64_t ldw, int64_t ldh, int64_t up_col0,
                        int64_t gate_col0, int acc64) {
  if (!x || !w || !h || M < 0 || N < 0 || K < 0 || up_col0 < 0 || gate_col0 < 0) return -1;
  for (int64_t m = 0; m < M; ++m) {
    const uint16_t* xr = x + m * ldx;
    for (int64_t n = 0; n < N; ++n) {
      float r;
      if (acc64) {
        const double u = dot64(xr, w, ldw, up_col0 + n, K);
        const double g = dot64(xr, w, ldw, gate_col0 + n, K);
        r = (float)(silu_f64(g) * u);
      } else {
        const float u = dot32(xr, w, ldw, up_col0 + n, K);
        const float g = dot32(xr, w, ldw, gate_col0 + n, K);
        r = silu_f32(g) * u;
      }
      h[m * ldh + n] = f32_to_bf16_rne(r);
    }
  }
  return 0;
}
