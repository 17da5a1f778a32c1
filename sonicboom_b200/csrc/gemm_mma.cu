// bfloat16 matrix products on the warp-level tensor-core path (mma.sync m16n8k16, float32
// accumulation): out[M,N] = A[M,K] . W[N,K]^T with the fused epilogues of gemm_plain.cu.
//
//  * sb_gemm_skinny: up to 64 rows (decode).  The step is bound by reading W once, so W is
//    streamed straight from global memory into MMA A-fragments with 16-byte loads and never
//    touches shared memory; the few activation rows are the B operand.  One block owns 16
//    rows of W, its 8 warps split K, and their partial sums are added in a fixed order, so a
//    result never depends on the batch around it.
//  * sb_gemm_tiled: any number of rows (prefill): 128x128x64 tiles, a 3-stage cp.async
//    pipeline, XOR-swizzled shared memory read with ldmatrix.
//
// Both need K to be a multiple of 8 (16-byte rows) and refuse other K with a clear error.
#include "common.cuh"

int sb_check_linear_args(const char* who, int M, int N, int K, int epilogue, const void* bias,
                         const float* residual, int out_dtype);

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Activations come from the kernel before this one: a coherent load, never the .nc path.
__device__ __forceinline__ uint4 ldg_cached(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <typename TB>
__device__ __forceinline__ float load_bias(const void* bias, int n) {
  return sb_to_f32<TB>(((const TB*)bias)[n]);
}

// ------------------------------------------------------------------------------- skinny
constexpr int SK_WARPS = 8;      // warps of a block; they split K
// 32-wide K blocks a warp has in flight.  Inside the decode step of a 7B-sized model (the q|k|v
// projection at up to 8 rows): batch 1 2.896 ms with two, 2.850 with four, 2.830 with eight,
// 2.847 with twelve, 2.905 with sixteen; batch 8 3.115 / 3.073 / 3.064 / 3.072 / 3.130.
constexpr int SK_UNROLL = 8;

// W is the MMA's A operand (16 rows of W), the activations its B operand (8 rows each).
// Within a 32-wide K block, thread t of a quad loads the 8 consecutive values k0+8t..k0+8t+7
// of its W rows and of its activation row; the four pairs feed two MMAs.  The MMA only needs
// A and B to agree on which k sits in which slot, so this contiguous 16-byte-per-thread
// assignment is as good as the canonical interleaved one.
template <int NT, typename TO>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const bf16* X, const bf16* __restrict__ W, int M, int N, int K,
                   int epilogue, const void* __restrict__ bias, int bias_dtype,
                   const float* residual, TO* out) {
  __shared__ float partial[SK_WARPS][NT][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.x * 16;
  const uint4* w0 = (const uint4*)(W + (size_t)min(m0 + g, N - 1) * K) + t;
  const uint4* w1 = (const uint4*)(W + (size_t)min(m0 + g + 8, N - 1) * K) + t;
  const uint4* xp[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int row = nt * 8 + g;
    xok[nt] = row < M;
    xp[nt] = (const uint4*)(X + (size_t)min(row, M - 1) * K) + t;
  }
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

  const int n_blocks = (K + 31) >> 5;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int kb = warp; kb < n_blocks; kb += SK_WARPS * SK_UNROLL) {
    uint4 wa[SK_UNROLL], wb[SK_UNROLL];
    bool ok[SK_UNROLL];
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = kb + u * SK_WARPS;
      ok[u] = k < n_blocks && (k * 32 + 8 * t + 8 <= K);
      wa[u] = ok[u] ? ldg_stream(w0 + k * 4) : zero;
      wb[u] = ok[u] ? ldg_stream(w1 + k * 4) : zero;
    }
    // the weights above do not depend on the kernel before this one; everything below does
    if (kb == warp) sb_pdl_wait();
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = kb + u * SK_WARPS;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 x = (ok[u] && xok[nt]) ? ldg_cached(xp[nt] + k * 4) : zero;
        mma_bf16(acc[nt], wa[u].x, wb[u].x, wa[u].y, wb[u].y, x.x, x.y);
        mma_bf16(acc[nt], wa[u].z, wb[u].z, wa[u].w, wb[u].w, x.z, x.w);
      }
    }
  }
  if (warp >= n_blocks) sb_pdl_wait();          // a warp without K blocks never waited above
  sb_pdl_launch();                              // the weights have been read
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) partial[warp][nt][lane][i] = acc[nt][i];
  __syncthreads();

  // Epilogue: thread e takes W row r = e % 16 of batch row b = e / 16, sums the warps'
  // partial results in warp order, and applies the epilogue.
  for (int e = threadIdx.x; e < 16 * 8 * NT; e += SK_WARPS * 32) {
    const int r = e & 15, b = e >> 4;
    if (b >= M) continue;
    const int nt = b >> 3, src_lane = (r & 7) * 4 + ((b & 7) >> 1), reg = (r >> 3) * 2 + (b & 1);
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) v += partial[w][nt][src_lane][reg];
    const int n = m0 + r;
    if (epilogue == SB_EPI_SWIGLU) {
      if (r >= 8 || n >= N) continue;           // rows 0..7 are gates, 8..15 their up rows
      float up = 0.0f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) up += partial[w][nt][src_lane][reg + 2];
      out[(size_t)b * (N / 2) + (m0 / 2 + r)] = sb_from_f32<TO>(sb_silu(v) * up);
      continue;
    }
    if (n >= N) continue;
    if (epilogue == SB_EPI_BIAS)
      v += bias_dtype == SB_F32 ? load_bias<float>(bias, n) : load_bias<bf16>(bias, n);
    else if (epilogue == SB_EPI_RESIDUAL)
      v += residual[(size_t)b * N + n];
    out[(size_t)b * N + n] = sb_from_f32<TO>(v);
  }
}

template <int NT>
int launch_skinny(const bf16* X, const bf16* W, int M, int N, int K, int epilogue,
                  const void* bias, int bias_dtype, const float* residual, void* out,
                  int out_dtype, cudaStream_t stream) {
  const int blocks = (N + 15) / 16;
  SB_DISPATCH_DTYPE(out_dtype, TO, {
    sb_launch<SB_K_SKINNY>(gemm_skinny_kernel<NT, TO>, dim3(blocks), dim3(SK_WARPS * 32), 0, stream,
        X, W, M, N, K, epilogue, bias, bias_dtype, residual, (TO*)out);
  });
  SB_CHECK_LAUNCH("sb_gemm_skinny");
  return SB_OK;
}

// -------------------------------------------------------------------------------- tiled
constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3, TILED_THREADS = 256;
constexpr int TILE_BYTES = BM * BK * 2;                       // one operand tile of a stage
constexpr int TILED_SMEM = STAGES * 2 * TILE_BYTES;           // 96 KiB

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;                            // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                            uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// A tile row holds BK = 64 values = 8 chunks of 16 bytes; chunk c of row r is stored at chunk
// c ^ (r & 7), which makes both the cp.async stores and the ldmatrix reads conflict-free.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return (uint32_t)(row * (BK * 2) + ((chunk ^ (row & 7)) << 4));
}

template <typename TO>
__global__ void __launch_bounds__(TILED_THREADS)
gemm_tiled_kernel(const bf16* A, const bf16* __restrict__ W, int M, int N, int K,
                  int epilogue, const void* __restrict__ bias, int bias_dtype,
                  const float* residual, TO* out) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
  sb_pdl_launch();
  sb_pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp >> 2, warp_n = warp & 3;             // 2 x 4 warps, 64 x 32 each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int n_k = (K + BK - 1) / BK;

  auto load_stage = [&](int stage, int kt) {
    const int k0 = kt * BK;
    const uint32_t a_base = smem_base + stage * 2 * TILE_BYTES, b_base = a_base + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < (BM * 8) / TILED_THREADS; ++i) {       // 1024 chunks per operand
      const int idx = tid + i * TILED_THREADS, row = idx >> 3, chunk = idx & 7;
      const int k = k0 + chunk * 8;
      const bool kv = k + 8 <= K;
      const int am = m0 + row, bn = n0 + row;
      cp_async16(a_base + tile_offset(row, chunk),
                 A + (size_t)min(am, M - 1) * K + (kv ? k : 0), kv && am < M);
      cp_async16(b_base + tile_offset(row, chunk),
                 W + (size_t)min(bn, N - 1) * K + (kv ? k : 0), kv && bn < N);
    }
  };

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_k) load_stage(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < n_k; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (kt + STAGES - 1 < n_k) load_stage((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
    cp_async_commit();
    const uint32_t a_base = smem_base + (kt % STAGES) * 2 * TILE_BYTES, b_base = a_base + TILE_BYTES;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t af[4][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // matrices: (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
        const int row = warp_m * 64 + i * 16 + (lane & 15), chunk = ks * 2 + (lane >> 4);
        ldmatrix_x4(a_base + tile_offset(row, chunk), af[i][0], af[i][1], af[i][2], af[i][3]);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        // matrices: (n 0-7, k lo), (n 0-7, k hi), (n 8-15, k lo), (n 8-15, k hi)
        const int row = warp_n * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b_base + tile_offset(row, chunk), bfr[2 * j][0], bfr[2 * j][1],
                    bfr[2 * j + 1][0], bfr[2 * j + 1][1]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma_bf16(acc[i][j], af[i][0], af[i][1], af[i][2], af[i][3], bfr[j][0], bfr[j][1]);
    }
  }
  cp_async_wait<0>();

  // Epilogue straight from the accumulators: thread holds rows g, g+8 and columns 2t, 2t+1
  // of every 16x8 tile.  With gate/up in blocks of 8, tiles 2j and 2j+1 are a gate/up pair.
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = m0 + warp_m * 64 + i * 16 + g + half * 8;
      if (m >= M) continue;
      if (epilogue == SB_EPI_SWIGLU) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col = (n0 + warp_n * 32) / 2 + j * 8 + 2 * t;       // output column
#pragma unroll
          for (int c = 0; c < 2; ++c)
            if (col + c < N / 2)
              out[(size_t)m * (N / 2) + col + c] = sb_from_f32<TO>(
                  sb_silu(acc[i][2 * j][half * 2 + c]) * acc[i][2 * j + 1][half * 2 + c]);
        }
        continue;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + warp_n * 32 + j * 8 + 2 * t + c;
          if (n >= N) continue;
          float v = acc[i][j][half * 2 + c];
          if (epilogue == SB_EPI_BIAS)
            v += bias_dtype == SB_F32 ? load_bias<float>(bias, n) : load_bias<bf16>(bias, n);
          else if (epilogue == SB_EPI_RESIDUAL)
            v += residual[(size_t)m * N + n];
          out[(size_t)m * N + n] = sb_from_f32<TO>(v);
        }
      }
    }
  }
}

int check_bf16_product(const char* who, int a_dtype, int w_dtype, int K, const void* A,
                       const void* W) {
  if (a_dtype != SB_BF16 || w_dtype != SB_BF16)
    SB_FAIL(SB_ERR_UNSUPPORTED, "%s: takes bfloat16 operands (got dtype codes %d, %d)", who,
            a_dtype, w_dtype);
  if (K % 8)
    SB_FAIL(SB_ERR_UNSUPPORTED,
            "%s: the inner size must be a multiple of 8 for 16-byte rows, got %d", who, K);
  if (((uintptr_t)A | (uintptr_t)W) & 15)
    SB_FAIL(SB_ERR_ARG, "%s: operands must be 16-byte aligned", who);
  return SB_OK;
}

}  // namespace

extern "C" int sb_gemm_skinny(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
                              int K, int epilogue, const void* bias, int bias_dtype,
                              const float* residual, void* out, int out_dtype,
                              cudaStream_t stream) {
  if (int rc = sb_check_linear_args("sb_gemm_skinny", M, N, K, epilogue, bias, residual, out_dtype))
    return rc;
  if (int rc = check_bf16_product("sb_gemm_skinny", a_dtype, w_dtype, K, A, W)) return rc;
  if (M > 64) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_skinny: at most 64 rows, got %d", M);
  if (!sb_valid_dtype(out_dtype)) SB_FAIL(SB_ERR_ARG, "sb_gemm_skinny: out dtype %d", out_dtype);
  const bf16 *x = (const bf16*)A, *w = (const bf16*)W;
  if (M <= 8)
    return launch_skinny<1>(x, w, M, N, K, epilogue, bias, bias_dtype, residual, out, out_dtype, stream);
  if (M <= 16)
    return launch_skinny<2>(x, w, M, N, K, epilogue, bias, bias_dtype, residual, out, out_dtype, stream);
  if (M <= 32)
    return launch_skinny<4>(x, w, M, N, K, epilogue, bias, bias_dtype, residual, out, out_dtype, stream);
  return launch_skinny<8>(x, w, M, N, K, epilogue, bias, bias_dtype, residual, out, out_dtype, stream);
}

extern "C" int sb_gemm_tiled(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
                             int K, int epilogue, const void* bias, int bias_dtype,
                             const float* residual, void* out, int out_dtype,
                             cudaStream_t stream) {
  if (int rc = sb_check_linear_args("sb_gemm_tiled", M, N, K, epilogue, bias, residual, out_dtype))
    return rc;
  if (int rc = check_bf16_product("sb_gemm_tiled", a_dtype, w_dtype, K, A, W)) return rc;
  if (!sb_valid_dtype(out_dtype)) SB_FAIL(SB_ERR_ARG, "sb_gemm_tiled: out dtype %d", out_dtype);
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tiled: M=%d is too many rows", M);
  static bool configured[2] = {false, false};
  SB_DISPATCH_DTYPE(out_dtype, TO, {
    if (!configured[out_dtype]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tiled_kernel<TO>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, TILED_SMEM);
      if (e != cudaSuccess)
        SB_FAIL(SB_ERR_CUDA, "sb_gemm_tiled: shared memory opt-in failed: %s", cudaGetErrorString(e));
      configured[out_dtype] = true;
    }
    sb_launch<SB_K_SKINNY>(gemm_tiled_kernel<TO>, grid, dim3(TILED_THREADS), TILED_SMEM, stream,
        (const bf16*)A, (const bf16*)W, M, N, K, epilogue, bias, bias_dtype, residual, (TO*)out);
  });
  SB_CHECK_LAUNCH("sb_gemm_tiled");
  return SB_OK;
}
