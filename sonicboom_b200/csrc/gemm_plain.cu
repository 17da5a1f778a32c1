// Plain CUDA-core matrix product with float32 accumulation: out[M,N] = A[M,K] . W[N,K]^T.
// It is the true 32-bit path's product (FFMA only, no tensor cores, no reduced-precision
// mode) and takes every size; the same kernel also accepts bfloat16 operands, which the
// tensor-core kernels are checked against.  Each output element is one thread's sum over K in
// ascending order, so a row's result does not depend on what else is in the launch.
//
// Epilogues (the fusions the reference's passes make on its graphs: bias into the product,
// residual add into the product, SiLU*up into the product's consumer;
// core/include/sonicboom/planner/ir_passes.h:35-39):
//   NONE      out = acc
//   BIAS      out = acc + bias[n]
//   RESIDUAL  out = acc + residual[m, n]          (out may be the residual buffer itself)
//   SWIGLU    W holds gate and up rows in alternating blocks of 8; out[m, j] =
//             silu(acc_gate_j) * acc_up_j, out has N/2 columns.
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* A, const TW* __restrict__ W, int M, int N, int K,
                  int epilogue, const void* __restrict__ bias, int bias_dtype,
                  const float* residual, TO* out) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Ws[TK][TN + 1];
  __shared__ float Cs[TM][TN + 1];
  sb_pdl_launch();
  sb_pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;           // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc[4][4] = {};

  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = tid; i < TM * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      const int m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? sb_to_f32<TA>(A[(size_t)m * K + k]) : 0.0f;
    }
    for (int i = tid; i < TN * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      const int n = n0 + r, k = k0 + c;
      Ws[c][r] = (n < N && k < K) ? sb_to_f32<TW>(W[(size_t)n * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }

  if (epilogue == SB_EPI_SWIGLU) {
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < 4; ++j) Cs[ty * 4 + i][tx * 4 + j] = acc[i][j];
    __syncthreads();
    const int half_n = N / 2;
    for (int i = tid; i < TM * (TN / 2); i += 256) {
      const int r = i / (TN / 2), c = i % (TN / 2);       // c: output column within the tile
      const int gate_col = (c / SB_SWIGLU_BLOCK) * 2 * SB_SWIGLU_BLOCK + c % SB_SWIGLU_BLOCK;
      const int m = m0 + r, j = n0 / 2 + c;
      if (m < M && j < half_n)
        out[(size_t)m * half_n + j] =
            sb_from_f32<TO>(sb_silu(Cs[r][gate_col]) * Cs[r][gate_col + SB_SWIGLU_BLOCK]);
    }
    return;
  }
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (epilogue == SB_EPI_BIAS)
        v += bias_dtype == SB_F32 ? ((const float*)bias)[n]
                                  : __bfloat162float(((const __nv_bfloat16*)bias)[n]);
      else if (epilogue == SB_EPI_RESIDUAL)
        v += residual[(size_t)m * N + n];
      out[(size_t)m * N + n] = sb_from_f32<TO>(v);
    }
  }
}

}  // namespace

int sb_check_linear_args(const char* who, int M, int N, int K, int epilogue, const void* bias,
                         const float* residual, int out_dtype) {
  if (M <= 0 || N <= 0 || K <= 0) SB_FAIL(SB_ERR_ARG, "%s: M=%d N=%d K=%d", who, M, N, K);
  if (epilogue < SB_EPI_NONE || epilogue > SB_EPI_SWIGLU)
    SB_FAIL(SB_ERR_ARG, "%s: epilogue %d", who, epilogue);
  if (epilogue == SB_EPI_BIAS && !bias) SB_FAIL(SB_ERR_ARG, "%s: bias epilogue without bias", who);
  if (epilogue == SB_EPI_RESIDUAL && !residual)
    SB_FAIL(SB_ERR_ARG, "%s: residual epilogue without residual", who);
  if (epilogue == SB_EPI_RESIDUAL && out_dtype != SB_F32)
    SB_FAIL(SB_ERR_ARG, "%s: the residual sum is kept in float32", who);
  if (epilogue == SB_EPI_SWIGLU && N % (2 * SB_SWIGLU_BLOCK))
    SB_FAIL(SB_ERR_UNSUPPORTED,
            "%s: fused gate/up needs an intermediate size that is a multiple of %d, got %d", who,
            SB_SWIGLU_BLOCK, N / 2);
  return SB_OK;
}

extern "C" int sb_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
                             int K, int epilogue, const void* bias, int bias_dtype,
                             const float* residual, void* out, int out_dtype,
                             cudaStream_t stream) {
  if (!sb_valid_dtype(a_dtype) || !sb_valid_dtype(w_dtype) || !sb_valid_dtype(out_dtype) ||
      (bias && !sb_valid_dtype(bias_dtype)))
    SB_FAIL(SB_ERR_ARG, "sb_gemm_plain: dtype codes %d %d %d %d", a_dtype, w_dtype, out_dtype,
            bias_dtype);
  if (int rc = sb_check_linear_args("sb_gemm_plain", M, N, K, epilogue, bias, residual, out_dtype))
    return rc;
  const dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
  if (grid.y > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_plain: M=%d is too many rows", M);
  SB_DISPATCH_DTYPE(a_dtype, TA, {
    SB_DISPATCH_DTYPE(w_dtype, TW, {
      SB_DISPATCH_DTYPE(out_dtype, TO, {
        sb_launch(gemm_plain_kernel<TA, TW, TO>, grid, dim3(256), 0, stream,
            (const TA*)A, (const TW*)W, M, N, K, epilogue, bias, bias_dtype, residual, (TO*)out);
      });
    });
  });
  SB_CHECK_LAUNCH("sb_gemm_plain");
  return SB_OK;
}
