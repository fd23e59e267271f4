/* CPU restatement of the deterministic SwiGLU arithmetic (TEST INFRASTRUCTURE, not product code).
 *
 * The reference defines SwiGLU only as an IR node (SwiGlu: converter npu_swiglu.py:8-14; DequantSwigluQuant:
 * third_party/ascend/include/ops/op_proto/inc/experiment_ops.h:3764-3811); its arithmetic is vendor code.  Decision:
 * silu(a) * b = RN(RN(a * RN(1 / (1 + e))) * b) with e = exp(-a) evaluated by the fixed sequence of fp32 operations below
 * (fused multiply-adds, one exponent insertion, one IEEE reciprocal), each of them correctly rounded, so that a CPU and a GPU that run the
 * same sequence agree bit for bit.  e is within 1.3 ulp of exp(-a) for |a| <= 80 apart from the rounded log2(e)
 * (relative error |a| * 1.3e-8); beyond that -a is capped, where 1 + e is 1 or the result is below 1e-33.
 *
 * Build: gcc -O2 -fPIC -shared -fopenmp -ffp-contract=off oracle/silu_exact.c -o oracle/_build/libsilu_exact.so -lm
 * (-ffp-contract=off: products and sums written separately must round separately; fmaf is the only fused form).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define TAB_LOG2E 0x1.715476p+0f       /* RN(log2(e)) */
#define TAB_MAGIC 12582912.0f          /* 1.5 * 2^23: adding it rounds to an integer (half to even) in the low mantissa bits */
/* 2^f on [-0.5, 0.5], degree 6, relative error 7.9e-8 including the fp32 evaluation */
#define TAB_C0 0x1.000000p+0f
#define TAB_C1 0x1.62e430p-1f
#define TAB_C2 0x1.ebfbdap-3f
#define TAB_C3 0x1.c6aed4p-5f
#define TAB_C4 0x1.3b2dbcp-7f
#define TAB_C5 0x1.5f456ap-10f
#define TAB_C6 0x1.41d334p-13f

static inline float silu_mul_exact(float a, float b) {
  const float x = fminf(fmaxf(-a, -80.0f), 80.0f);
  const float nm = fmaf(x, TAB_LOG2E, TAB_MAGIC);
  const float n = nm - TAB_MAGIC;
  const float f = fmaf(x, TAB_LOG2E, -n);
  float p = TAB_C6;
  p = fmaf(p, f, TAB_C5);
  p = fmaf(p, f, TAB_C4);
  p = fmaf(p, f, TAB_C3);
  p = fmaf(p, f, TAB_C2);
  p = fmaf(p, f, TAB_C1);
  p = fmaf(p, f, TAB_C0);
  uint32_t pb, nb;
  memcpy(&pb, &p, 4);
  memcpy(&nb, &nm, 4);
  pb += nb << 23;                      /* 2^n: n sits in the low bits of nm */
  float e;
  memcpy(&e, &pb, 4);
  const float d = 1.0f + e;
  const float y = 1.0f / d;            /* IEEE reciprocal */
  const float s = a * y;
  return s * b;
}

/* out[i] = silu(a[i]) * b[i] */
void tab_oracle_silu_mul(const float* a, const float* b, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = silu_mul_exact(a[i], b[i]);
}
