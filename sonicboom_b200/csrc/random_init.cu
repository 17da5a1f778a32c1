// Seeded normal random tensors that are the same on every device.
//
// Element e of a tensor comes from group g = e / 4: Philox4x32-10 (the generator of the
// reference's sampler, core/src/nn/sampling.cpp:207-227) with counter {g_lo, g_hi, 0x5742, 0}
// and the 64-bit key (key0, key1) gives four words; words 0,1 and words 2,3 each feed one
// Box-Muller transform, whose cosine and sine branches are the group's four values.  Logarithm,
// sine and cosine are short polynomials evaluated with individually rounded float32 operations
// (never fused), and the uniform variates are exact 24-bit fractions, so the host restatement of
// the same steps (weights/random_init.py, numpy float32) produces the same bits.  The result
// mean + std * z is rounded once to the output type.
#include "common.cuh"

namespace {

__device__ __forceinline__ void philox_round10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                               uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// (r cos t, r sin t) with r = sqrt(-2 ln u1), t = 2 pi u2; u1 = (a + 1) / 2^24 in (0, 1],
// u2 = b / 2^24 in [0, 1), a and b the upper 24 bits of two words.
__device__ __forceinline__ void box_muller(uint32_t wa, uint32_t wb, float& z_cos, float& z_sin) {
  // ---- ln u1: u1 = m 2^e with m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh(s), s = (m-1)/(m+1)
  const float u1 = __fmul_rn((float)((wa >> 8) + 1u), 5.9604644775390625e-08f);      // exact
  int e;
  float m = frexpf(u1, &e);                                                          // exact
  if (m < 0.70710678f) { m = __fmul_rn(m, 2.0f); e -= 1; }
  const float s = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
  const float s2 = __fmul_rn(s, s);
  float p = (float)(1.0 / 11.0);
  p = __fadd_rn(__fmul_rn(p, s2), (float)(1.0 / 9.0));
  p = __fadd_rn(__fmul_rn(p, s2), (float)(1.0 / 7.0));
  p = __fadd_rn(__fmul_rn(p, s2), (float)(1.0 / 5.0));
  p = __fadd_rn(__fmul_rn(p, s2), (float)(1.0 / 3.0));
  p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
  const float ln_u1 = __fadd_rn(__fmul_rn((float)e, 0.69314718f), __fmul_rn(__fmul_rn(2.0f, s), p));
  const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u1));
  // ---- the angle: quadrant q and fraction f of a quarter turn, folded into [0, pi/4]
  const uint32_t b = wb >> 8;
  const uint32_t q = b >> 22, fb = b & 0x3fffffu;
  const bool fold = fb > 0x200000u;
  const float f = __fmul_rn((float)(fold ? 0x400000u - fb : fb), 2.384185791015625e-07f);   // exact
  const float x = __fmul_rn(f, 1.57079633f);
  const float x2 = __fmul_rn(x, x);
  float sp = (float)(1.0 / 362880.0);
  sp = __fadd_rn(__fmul_rn(sp, x2), (float)(-1.0 / 5040.0));
  sp = __fadd_rn(__fmul_rn(sp, x2), (float)(1.0 / 120.0));
  sp = __fadd_rn(__fmul_rn(sp, x2), (float)(-1.0 / 6.0));
  sp = __fadd_rn(__fmul_rn(sp, x2), 1.0f);
  float sn = __fmul_rn(x, sp);
  float cp = (float)(-1.0 / 3628800.0);
  cp = __fadd_rn(__fmul_rn(cp, x2), (float)(1.0 / 40320.0));
  cp = __fadd_rn(__fmul_rn(cp, x2), (float)(-1.0 / 720.0));
  cp = __fadd_rn(__fmul_rn(cp, x2), (float)(1.0 / 24.0));
  cp = __fadd_rn(__fmul_rn(cp, x2), (float)(-1.0 / 2.0));
  float cs = __fadd_rn(__fmul_rn(cp, x2), 1.0f);
  if (fold) { const float t = sn; sn = cs; cs = t; }        // sin(pi/2 - x) = cos x
  float c, sgn_s;
  switch (q) {
    case 0: c = cs; sgn_s = sn; break;
    case 1: c = -sn; sgn_s = cs; break;
    case 2: c = -cs; sgn_s = -sn; break;
    default: c = sn; sgn_s = -cs; break;
  }
  z_cos = __fmul_rn(r, c);
  z_sin = __fmul_rn(r, sgn_s);
}

template <typename T>
__global__ void random_normal_kernel(T* out, size_t n, uint32_t key0, uint32_t key1, float mean,
                                     float std) {
  const size_t n_groups = (n + 3) / 4;
  for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups;
       g += (size_t)gridDim.x * blockDim.x) {
    uint32_t w[4];
    philox_round10((uint32_t)g, (uint32_t)(g >> 32), 0x5742u, 0u, key0, key1, w);
    float z[4];
    box_muller(w[0], w[1], z[0], z[1]);
    box_muller(w[2], w[3], z[2], z[3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t e = g * 4 + j;
      if (e < n) out[e] = sb_from_f32<T>(__fadd_rn(mean, __fmul_rn(std, z[j])));
    }
  }
}

}  // namespace

// out[e] = mean + std * z_e for e < n, z standard normal, a function of (key0, key1, e) only.
extern "C" int sb_random_normal(void* out, int out_dtype, size_t n, uint32_t key0, uint32_t key1,
                                float mean, float std, cudaStream_t stream) {
  if (!sb_valid_dtype(out_dtype)) SB_FAIL(SB_ERR_ARG, "sb_random_normal: dtype code %d", out_dtype);
  if (n == 0) return SB_OK;
  if (!out) SB_FAIL(SB_ERR_ARG, "sb_random_normal: no output");
  const size_t groups = (n + 3) / 4;
  const int blocks = (int)((groups + 255) / 256 < 65535 ? (groups + 255) / 256 : 65535);
  SB_DISPATCH_DTYPE(out_dtype, T, {
    sb_launch(random_normal_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out, n, key0, key1,
              mean, std);
  });
  SB_CHECK_LAUNCH("sb_random_normal");
  return SB_OK;
}
