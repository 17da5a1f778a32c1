// bfloat16 matrix product on the fifth-generation tensor cores: TMA-fed shared-memory ring,
// tcgen05.mma issued by one thread with the accumulator in tensor memory, epilogue read back
// with tcgen05.ld.  out[M,N] = A[M,K] . W[N,K]^T with the fused epilogues of gemm_plain.cu.
//
// One block computes a 128 x BN tile.  Warp 0 is the TMA producer, warp 1 allocates tensor
// memory and issues the MMAs, warps 2-5 run the epilogue (one TMEM lane quarter each; the decode
// form from 32 tokens on has warps 6-9 as a second group).  Both
// operands are K-major; tiles are 64 values (128 bytes) wide in K and stored with the 128-byte
// swizzle that the tensor maps write and the MMA descriptors read.  Rows and columns beyond
// M, N and K are zero-filled by TMA, so any M and N and any K that is a multiple of 8 work.
//
// Two forms share the kernel:
//   normal   A = activations (rows are tokens), B = weights: the prefill product.  With many
//            rows it is a persistent kernel (further down), from 129 rows on one on pairs of SMs
//            (gemm_tc5_pair.cuh); their epilogue keeps a thread's row and writes 16 bytes at a
//            time along it (store_chunk_rowwise);
//   swapped  A = weights (128 weight rows per tile), B = activations (up to 64 rows): the
//            decode product, which is bound by reading the weights once.  K may be split over
//            several blocks; their partial tiles go to scratch memory and a second kernel adds
//            them in split order and runs the epilogue, so the sum's order is fixed.  That
//            second kernel can also apply the RMSNorm that follows the product
//            (tc5_reduce_norm_kernel: a cluster of blocks per row, the sum of squares over
//            distributed shared memory), or the rotation and the cache write that follow a
//            q|k|v product (tc5_reduce_rope_kernel).
//
// Every wait on an mbarrier is bounded; when a bound is hit the kernel records a code in a
// status word, stops issuing work and leaves normally (sb_tc5_status reads the word).
#include <cooperative_groups.h>
#include <stdlib.h>

#include "tc5.cuh"

int sb_check_linear_args(const char* who, int M, int N, int K, int epilogue, const void* bias,
                         const float* residual, int out_dtype);

namespace {

typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
// The decode form with 32 or 64 tokens has two groups of four epilogue warps: a warp reaches only
// its own quarter of the tensor memory's lanes (weight rows), so the second group takes the
// second half of the columns (tokens).  With one group the epilogue of the last wave of blocks,
// beside which nothing else runs, took 5 of the fused gate/up product's 46 microseconds at 64
// tokens (at 32 tokens the second group is worth 0.2 % of the decode step).
constexpr int epilogue_groups(int bn, bool swapped) { return swapped && bn >= 32 ? 2 : 1; }
constexpr int kernel_threads(int bn, bool swapped) { return 64 + 128 * epilogue_groups(bn, swapped); }
// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// SiLU of a value that is rounded to TO afterwards: for bfloat16 outputs with the hardware's
// exponential (relative error about 1e-6 against bfloat16's 4e-3; a gate so negative that the
// exponential overflows gives 1 / inf = 0, as it should); for float32 outputs the accurate one.
template <typename TO>
__device__ __forceinline__ float sb_silu_out(float x) {
  if (sizeof(TO) == 2) return x * __frcp_rn(1.0f + __expf(-x));
  return sb_silu(x);
}

template <typename TB>
__device__ __forceinline__ float bias_at(const void* bias, int n) {
  return sb_to_f32<TB>(((const TB*)bias)[n]);
}

struct Tc5Params {
  int M, N, K;                 // the product's sizes as the caller sees them (rows, features, inner)
  int epilogue, bias_dtype;
  const void* bias;
  const float* residual;
  void* out;
  int tiles_a, tiles_b;        // tiles along the A rows and along the B rows
  int k_splits;                // swapped form: blocks that share one output tile
  float* scratch;              // swapped form with k_splits > 1: partial tiles [tile][split][BN][128]
  const char* warm;            // asked into L2 by every block as it ends (or null)
  size_t warm_bytes;
  int rowwise;                 // the many-rows epilogue may use 16-byte accesses along a row
};

constexpr int stage_bytes(int bn) { return (BM + bn) * BK * 2; }
constexpr int smem_bytes(int bn, int stages) { return stages * stage_bytes(bn) + 1024 + 256; }

// Epilogue of one 32-row x 32-column chunk of the normal form.  The accumulator chunk (a thread
// holds one row) is passed through a 32 x 33 shared-memory tile of the warp and written out row
// by row with a lane per column, so that global accesses coalesce.
// NC = 32, or 16 for the last chunk of a tile whose width is an odd multiple of 16.
// Sixteen-byte stores of `n` consecutive values of one row (n a multiple of 4 for float32, of 8
// for bfloat16; `dst` 16-byte aligned).
__device__ __forceinline__ void store_row(float* dst, const float* v, int n) {
#pragma unroll
  for (int j = 0; j < 32; j += 4)
    if (j < n) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
}
__device__ __forceinline__ void store_row(bf16* dst, const float* v, int n) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    if (j >= n) break;
    uint4 o;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(v[j], v[j + 1]); o.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[j + 2], v[j + 3]); o.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[j + 4], v[j + 5]); o.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[j + 6], v[j + 7]); o.w = *reinterpret_cast<uint32_t*>(&t);
    *reinterpret_cast<uint4*>(dst + j) = o;
  }
}

// The same epilogue without the transpose: the thread keeps its row.  Its 32 columns are 128
// consecutive bytes of a float32 output (64 of a bfloat16 one, 16 fused gate/up outputs), read
// and written with 16-byte accesses: an eighth of the instructions of the transposed form and
// no shared memory, which measured 53.5 against 66.1 us for the 2,048 x 3,584 x 3,584 product
// with the residual (the last tile's epilogue is not hidden behind anything).  Needs the whole
// chunk inside the matrix and rows that start on 16-byte boundaries (p.rowwise).
template <typename TO>
__device__ __forceinline__ void store_chunk_rowwise(const Tc5Params& p, const uint32_t (&r)[32], int m, int n0) {
  if (m >= p.M) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (p.epilogue == SB_EPI_SWIGLU) {
    // columns come as 8 gates, then their 8 up values
    float o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j] = sb_silu_out<TO>(v[j]) * v[j + 8];
      o[j + 8] = sb_silu_out<TO>(v[j + 16]) * v[j + 24];
    }
    store_row((TO*)p.out + (size_t)m * (p.N / 2) + n0 / 2, o, 16);
    return;
  }
  if (p.epilogue == SB_EPI_BIAS) {
    if (p.bias_dtype == SB_F32) {
      const float4* b = reinterpret_cast<const float4*>((const float*)p.bias + n0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 x = b[j];
        v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
      }
    } else {
      const uint4* b = reinterpret_cast<const uint4*>((const bf16*)p.bias + n0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 x = b[j];
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
          v[8 * j + 2 * k] += f.x;
          v[8 * j + 2 * k + 1] += f.y;
        }
      }
    }
  } else if (p.epilogue == SB_EPI_RESIDUAL) {
    // every residual value is loaded before any store: the output may be the residual itself
    const float4* res = reinterpret_cast<const float4*>(p.residual + (size_t)m * p.N + n0);
    float4 x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = res[j];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[4 * j] += x[j].x; v[4 * j + 1] += x[j].y; v[4 * j + 2] += x[j].z; v[4 * j + 3] += x[j].w;
    }
  }
  store_row((TO*)p.out + (size_t)m * p.N + n0, v, 32);
}

template <typename TO, int NC = 32>
__device__ __forceinline__ void store_chunk(const Tc5Params& p, float* stage, const uint32_t (&r)[32],
                                            int m_base, int n0, int lane) {
  if (NC == 32 && p.rowwise && n0 + 32 <= p.N) {
    store_chunk_rowwise<TO>(p, r, m_base + lane, n0);
    return;
  }
  __syncwarp();
#pragma unroll
  for (int j = 0; j < NC; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]);
  __syncwarp();
  if (p.epilogue == SB_EPI_SWIGLU) {
    // 16 outputs per row (8 of a 16-column chunk): lanes 0-15 take an even row, lanes 16-31 the next one
    const int o = lane & 15, src = (o >> 3) * 16 + (o & 7);
    const bool live = n0 / 2 + o < p.N / 2 && o < NC / 2;
#pragma unroll 4
    for (int rr = 0; rr < 32; rr += 2) {
      const int row = rr + (lane >> 4), m = m_base + row;
      if (m < p.M && live)
        ((TO*)p.out)[(size_t)m * (p.N / 2) + n0 / 2 + o] =
            sb_from_f32<TO>(sb_silu_out<TO>(stage[row * 33 + src]) * stage[row * 33 + src + 8]);
    }
    return;
  }
  const int n = n0 + lane;
  const bool live = n < p.N && lane < NC;
  float add = 0.0f;
  if (p.epilogue == SB_EPI_BIAS && live)
    add = p.bias_dtype == SB_F32 ? bias_at<float>(p.bias, n) : bias_at<bf16>(p.bias, n);
  if (p.epilogue == SB_EPI_RESIDUAL) {
    // every residual value is loaded before any store: the output may be the residual
    // buffer itself (each element is read and written by the same lane), and loads
    // that had to stay behind stores would run one at a time
    float resv[32];
#pragma unroll
    for (int rr = 0; rr < 32; ++rr)
      resv[rr] = (live && m_base + rr < p.M) ? p.residual[(size_t)(m_base + rr) * p.N + n] : 0.0f;
#pragma unroll
    for (int rr = 0; rr < 32; ++rr)
      if (live && m_base + rr < p.M)
        ((TO*)p.out)[(size_t)(m_base + rr) * p.N + n] = sb_from_f32<TO>(stage[rr * 33 + lane] + resv[rr]);
    return;
  }
#pragma unroll 8
  for (int rr = 0; rr < 32; ++rr) {
    const int m = m_base + rr;
    if (m < p.M && live)
      ((TO*)p.out)[(size_t)m * p.N + n] = sb_from_f32<TO>(stage[rr * 33 + lane] + add);
  }
}

// ----------------------------------------------------------------------------- the kernel
// SWAPPED = false: A rows are tokens (m), B rows are features (n).
// SWAPPED = true:  A rows are features (n), B rows are tokens (m <= BN).
template <int BN, int STAGES, bool SWAPPED, typename TO>
__global__ void __launch_bounds__(kernel_threads(BN, SWAPPED))
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Tc5Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;                       // 1024-byte aligned ring
  const uint32_t bars = tiles + STAGES * stage_bytes(BN);
  // full[s] at bars + 8 s, empty[s] at bars + 8 (STAGES + s), accumulator-full after them
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, acc_bar = bars + 16 * STAGES;
  const uint32_t tmem_slot = acc_bar + 8;
  volatile uint32_t* tmem_slot_ptr =
      (volatile uint32_t*)(smem_raw + (tmem_slot - raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // consecutive blocks walk the A tiles of one B tile (or K splits first, in the swapped form),
  // so that a wave of blocks shares its operand tiles through L2
  int tile_a, tile_b, split = 0;
  if (SWAPPED) {
    split = blockIdx.x % p.k_splits;
    tile_a = blockIdx.x / p.k_splits;
    tile_b = 0;
  } else {
    tile_a = blockIdx.x % p.tiles_a;
    tile_b = blockIdx.x / p.tiles_a;
  }
  const int n_k_total = (p.K + BK - 1) / BK;
  const int k_per = (n_k_total + p.k_splits - 1) / p.k_splits;
  const int k_begin = split * k_per, k_end = min(n_k_total, k_begin + k_per);
  const int n_k = max(0, k_end - k_begin);
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0 && lane == 0) {
    // ---- producer.  The weight operand (A when swapped, else B) does not depend on the
    // kernel before this one, so the first ring of weight tiles is requested before the wait
    // on that kernel; the activation tiles follow after it.
    int issued = 0;
    bool ok = true;
    const int head = min(n_k, STAGES);
    for (int i = 0; i < head; ++i) {
      mbar_expect_tx(full0 + 8 * i, stage_bytes(BN));
      const uint32_t a_dst = tiles + i * stage_bytes(BN), b_dst = a_dst + BM * BK * 2;
      if (SWAPPED) tma_load_2d(a_dst, &map_a, (k_begin + i) * BK, tile_a * BM, full0 + 8 * i);
      else         tma_load_2d(b_dst, &map_b, (k_begin + i) * BK, tile_b * BN, full0 + 8 * i);
    }
    sb_pdl_wait();
    for (int i = 0; i < head; ++i) {
      const uint32_t a_dst = tiles + i * stage_bytes(BN), b_dst = a_dst + BM * BK * 2;
      if (SWAPPED) tma_load_2d(b_dst, &map_b, (k_begin + i) * BK, tile_b * BN, full0 + 8 * i);
      else         tma_load_2d(a_dst, &map_a, (k_begin + i) * BK, tile_a * BM, full0 + 8 * i);
      issued = i + 1;
    }
    for (int i = head; i < n_k && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(empty0 + 8 * s, ((i / STAGES) & 1) ^ 1, 1);
      if (!ok) break;
      mbar_expect_tx(full0 + 8 * s, stage_bytes(BN));
      const uint32_t a_dst = tiles + s * stage_bytes(BN), b_dst = a_dst + BM * BK * 2;
      tma_load_2d(a_dst, &map_a, (k_begin + i) * BK, tile_a * BM, full0 + 8 * s);
      tma_load_2d(b_dst, &map_b, (k_begin + i) * BK, tile_b * BN, full0 + 8 * s);
      issued = i + 1;
    }
    sb_pdl_launch();                        // every load of this block is on its way
    if (!ok) {
      // let copies that are still in flight land before the block's memory goes away
      for (int i = max(0, issued - STAGES); i < issued; ++i)
        mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, 2);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer
    constexpr uint32_t idesc = instr_desc(BN);
    bool ok = true;
    for (int i = 0; i < n_k && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(full0 + 8 * s, (i / STAGES) & 1, 3);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_addr = tiles + s * stage_bytes(BN), b_addr = a_addr + BM * BK * 2;
      const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(b_addr);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        umma_bf16(tmem_base, adesc + (uint64_t)(k * UMMA_K * 2 >> 4),
                  bdesc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, (i > 0 || k > 0) ? 1u : 0u);
      umma_commit(empty0 + 8 * s);          // the stage is free once these MMAs have read it
    }
    umma_commit(acc_bar);                   // arrives when every MMA above has finished
  } else if (warp >= 2) {
    // ---- epilogue: this warp reads TMEM lanes [32 q, 32 q + 32)
    sb_pdl_wait();                          // the residual, and the scratch of an earlier product
    const int q = warp & 3;
    const bool ok = mbar_wait(acc_bar, 0, 4);
    tc_fence_after();
    const int a_row = tile_a * BM + q * 32 + lane;            // this thread's row of A
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
    if (ok && n_k > 0) {
      if (!SWAPPED) {
        float* stage = reinterpret_cast<float*>(smem_raw + (tiles - raw)) + (warp - 2) * 32 * 33;
        const int m_base = tile_a * BM + q * 32;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          const int n0 = tile_b * BN + c * 32;
          if (n0 >= p.N) break;
          store_chunk<TO>(p, stage, r, m_base, n0, lane);
        }
      } else {
        // swapped: this thread owns feature n = a_row and holds its value for the CN tokens
        // from t0 on (all BN of them unless the epilogue warps come in two groups)
        constexpr int CN = BN / epilogue_groups(BN, SWAPPED);
        const int t0 = ((warp - 2) >> 2) * CN;
        const int n = a_row;
        uint32_t r[32];
        float acc[CN];
#pragma unroll
        for (int c = 0; c < (CN + 31) / 32; ++c) {
          if (CN >= 32) tmem_ld32(t_row + t0 + c * 32, r); else tmem_ld16(t_row + t0, r);
#pragma unroll
          for (int j = 0; j < (CN < 32 ? CN : 32); ++j) acc[c * 32 + j] = __uint_as_float(r[j]);
        }
        if (p.k_splits > 1) {
          // partial tile to scratch: [tile][split][token][128 features]
          float* dst = p.scratch + (((size_t)tile_a * p.k_splits + split) * BN + t0) * BM + q * 32 + lane;
#pragma unroll
          for (int j = 0; j < CN; ++j)
            if (t0 + j < p.M) dst[(size_t)j * BM] = acc[j];
        } else if (p.epilogue == SB_EPI_SWIGLU) {
          // Features come in groups of 8 gates then their 8 up values, so lane l of a gate
          // group and lane l + 8 hold the two factors of one output.  They take a token each
          // of every two: the gate lane hands over its gate of the odd token and gets the up
          // value of the even one, so that every lane computes and stores one output per
          // exchange.  Nothing leaves the loop early: tokens beyond M are zero rows whose
          // results are not stored, and without branches the exchanges, exponentials and
          // divisions of different tokens overlap (with 64 tokens the epilogue of the last wave
          // of blocks was a chain of their latencies, and nothing else runs beside it).
          const bool gate = (lane & 15) < 8;
          const int col = (n >> 4) * 8 + (n & 7);               // the same for both lanes of an output
          const bool live = n < p.N;                            // N is a multiple of 16 here
#pragma unroll
          for (int j = 0; j < CN; j += 2) {
            const float a0 = acc[j], a1 = acc[j + 1];
            const float other = __shfl_xor_sync(0xffffffffu, gate ? a1 : a0, 8);
            const int tok = t0 + (gate ? j : j + 1);
            const float g = gate ? a0 : other, up = gate ? other : a1;
            if (live && tok < p.M)
              ((TO*)p.out)[(size_t)tok * (p.N / 2) + col] = sb_from_f32<TO>(sb_silu_out<TO>(g) * up);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CN; ++j) {
            const int tok = t0 + j;
            if (tok >= p.M) break;
            float v = acc[j];
            if (n >= p.N) continue;
            if (p.epilogue == SB_EPI_BIAS)
              v += p.bias_dtype == SB_F32 ? bias_at<float>(p.bias, n) : bias_at<bf16>(p.bias, n);
            else if (p.epilogue == SB_EPI_RESIDUAL)
              v += p.residual[(size_t)tok * p.N + n];
            ((TO*)p.out)[(size_t)tok * p.N + n] = sb_from_f32<TO>(v);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  // The block has read and written all it had to.  If the caller named weights that a later
  // kernel streams but cannot request early itself (one launched without programmatic
  // dependent launch), ask for them now: they arrive while the partial tiles are added.
  if (p.warm_bytes && threadIdx.x == 0) sb_warm_l2(p.warm, p.warm_bytes, blockIdx.x, gridDim.x);
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);

}

// ------------------------------------------------------------------ the persistent kernel
// Normal form only.  One block per SM walks its tiles (block b takes tiles b, b + grid, ...; a
// tile index walks the A tiles of one B tile first, so that the blocks of a wave share operand
// tiles through L2).  Tiles are 128 x BN with BN up to 256, which halves the operand traffic per
// flop of the 128 x 128 kernel; tensor memory holds two accumulators, so the epilogue of a tile
// runs while the MMAs of the block's next tile are already being issued.
constexpr int PERSIST_STAGING = 4 * 32 * 33 * 4;     // the epilogue warps' transpose tiles
constexpr int persist_smem_bytes(int bn, int stages) {
  return stages * stage_bytes(bn) + PERSIST_STAGING + 1024 + 256;
}

template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(THREADS)
gemm_tc5_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_b, const Tc5Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t staging = tiles + STAGES * stage_bytes(BN);
  const uint32_t bars = staging + PERSIST_STAGING;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;
  const uint32_t acc_full0 = bars + 16 * STAGES, acc_empty0 = acc_full0 + 16;
  const uint32_t tmem_slot = acc_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(smem_raw + (tmem_slot - raw));
  constexpr uint32_t ACC_COLS = 256;                   // column offset of the second accumulator

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  sb_pdl_launch();
  const int n_tiles = p.tiles_a * p.tiles_b;
  const int n_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, 4);                // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0 && lane == 0) {
    // ---- producer
    sb_pdl_wait();
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
      for (int kt = 0; kt < n_k; ++kt, ++it) {
        const uint32_t s = it % STAGES;
        ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, 1);
        if (!ok) break;
        mbar_expect_tx(full0 + 8 * s, stage_bytes(BN));
        const uint32_t a_dst = tiles + s * stage_bytes(BN), b_dst = a_dst + BM * BK * 2;
        tma_load_2d(a_dst, &map_a, kt * BK, tile_a * BM, full0 + 8 * s);
        tma_load_2d(b_dst, &map_b, kt * BK, tile_b * BN, full0 + 8 * s);
      }
    }
    if (!ok) {
      // let copies that are still in flight land before the block's memory goes away
      for (uint32_t i = it > STAGES ? it - STAGES : 0; i < it; ++i)
        mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, 2);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer
    constexpr uint32_t idesc = instr_desc(BN);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
      const uint32_t acc = lt & 1;
      ok = mbar_wait(acc_empty0 + 8 * acc, ((lt >> 1) & 1) ^ 1, 5);   // the epilogue has drained it
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
      for (int kt = 0; kt < n_k; ++kt, ++it) {
        const uint32_t s = it % STAGES;
        ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, 3);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = tiles + s * stage_bytes(BN), b_addr = a_addr + BM * BK * 2;
        const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(b_addr);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(d_tmem, adesc + (uint64_t)(k * UMMA_K * 2 >> 4),
                    bdesc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, (kt > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);
      }
      umma_commit(acc_full0 + 8 * acc);
    }
  } else if (warp >= 2) {
    // ---- epilogue: this warp reads TMEM lanes [32 q, 32 q + 32) of the finished accumulator
    sb_pdl_wait();
    const int q = warp & 3;
    float* stage = reinterpret_cast<float*>(smem_raw + (staging - raw)) + (warp - 2) * 32 * 33;
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++lt) {
      const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
      const uint32_t acc = lt & 1;
      if (!mbar_wait(acc_full0 + 8 * acc, (lt >> 1) & 1, 4)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
      const int m_base = tile_a * BM + q * 32;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        const int n0 = tile_b * BN + c * 32;
        if (n0 < p.N) store_chunk<TO>(p, stage, r, m_base, n0, lane);
      }
      if (BN % 32) {                                   // a last chunk of 16 columns
        uint32_t r[32];
        tmem_ld16(t_row + (BN / 32) * 32, r);
        const int n0 = tile_b * BN + (BN / 32) * 32;
        if (n0 < p.N) store_chunk<TO, 16>(p, stage, r, m_base, n0, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

#include "gemm_tc5_pair.cuh"

namespace {

// Adds the partial tiles of a split-K swapped product in split order and applies the epilogue.
// One thread takes four consecutive features of one token (for the fused gate/up: four gates and
// their four up values).  A second, fully parallel kernel measured faster here than letting the
// block that finishes a tile last add its partials.
template <typename TO>
__global__ void __launch_bounds__(256)
tc5_reduce_kernel(const Tc5Params p, int bn) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int n_out = p.epilogue == SB_EPI_SWIGLU ? p.N / 2 : p.N;
  const int groups = (n_out + 3) / 4;
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)groups * p.M) return;
  const int j = (int)(idx / groups), o0 = (int)(idx % groups) * 4;      // token, first output
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // first feature of the group in W's row order
  const int n0 = p.epilogue == SB_EPI_SWIGLU ? (o0 / 8) * 16 + (o0 % 8) : o0;
  const int tile = n0 / BM, f = n0 % BM;
  const float* base = p.scratch + (((size_t)tile * p.k_splits) * bn + j) * BM + f;
  for (int s = 0; s < p.k_splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(base + (size_t)s * bn * BM);
    acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    if (p.epilogue == SB_EPI_SWIGLU) {
      const float4 u = *reinterpret_cast<const float4*>(base + (size_t)s * bn * BM + 8);
      up[0] += u.x; up[1] += u.y; up[2] += u.z; up[3] += u.w;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int o = o0 + i;
    if (o >= n_out) break;
    float v = acc[i];
    if (p.epilogue == SB_EPI_SWIGLU) v = sb_silu(v) * up[i];
    else if (p.epilogue == SB_EPI_BIAS)
      v += p.bias_dtype == SB_F32 ? bias_at<float>(p.bias, o) : bias_at<bf16>(p.bias, o);
    else if (p.epilogue == SB_EPI_RESIDUAL) v += p.residual[(size_t)j * p.N + o];
    ((TO*)p.out)[(size_t)j * n_out + o] = sb_from_f32<TO>(v);
  }
}

// The same sum for a fused q|k|v product, followed by the rotation and the cache write that
// rope_store_vec_kernel (elementwise.cu) does on the finished row: the float32 row is neither
// written nor read again, and the step has one kernel less.  The same sums in the same order and
// the same rotation formulas as the two kernels.  A block takes a
// token and a share of its heads; a task is four pairs (e, e + half) of one head, or four of the
// values beyond the rotated part.  cos and sin of the token's position are worked out once a
// block (from the step's plan, before the wait for the product).
constexpr int RR_THREADS = 256;
__global__ void __launch_bounds__(RR_THREADS)
tc5_reduce_rope_kernel(const Tc5Params p, int bn, const SbRopeStore r) {
  extern __shared__ float rr_cs[];                   // cos[rot/2], then sin[rot/2]
  sb_pdl_launch();
  const int t = blockIdx.x;
  const int pos = r.row_pos[t];
  const int half = r.rot >> 1, hd = r.hd;
  for (int i = threadIdx.x; i < half; i += RR_THREADS) {
    const float theta = (float)pos * r.inv_freq[i];
    rr_cs[i] = cosf(theta);
    rr_cs[half + i] = sinf(theta);
  }
  const bool has_kv = r.cache != nullptr;
  const int n_heads = r.n_q_heads + (has_kv ? 2 * r.n_kv_heads : 0);
  size_t k_base = 0, v_base = 0;
  bool stores = has_kv;
  if (has_kv) {
    // a position without a page in its own sequence's list writes no key and no value
    const int seq = r.row_seq[t], first = r.page_off[seq], n_pages = r.page_off[seq + 1] - first;
    const int pi = pos / r.page_size;
    const int page = (pos >= 0 && pi < n_pages) ? r.page_ids[first + pi] : -1;
    stores = page >= 0;
    k_base = (((size_t)(stores ? page : 0) * 2) * r.n_kv_heads * r.page_size + pos % r.page_size) * hd;
    v_base = (((size_t)(stores ? page : 0) * 2 + 1) * r.n_kv_heads * r.page_size + pos % r.page_size) * hd;
  }
  __syncthreads();
  sb_pdl_wait();
  const int pair_tasks = half >> 2, per_head = pair_tasks + ((hd - r.rot) >> 2);
  const int heads_per = (n_heads + (int)gridDim.y - 1) / (int)gridDim.y;
  const int head_lo = blockIdx.y * heads_per, head_hi = min(n_heads, head_lo + heads_per);
  bf16* q_out = (bf16*)r.q_out;
  bf16* cache = (bf16*)r.cache;
  // the sum over the splits of four consecutive features starting at feature n of token t, + bias
  auto sum4 = [&](int n, float (&acc)[4]) {
    const int tile = n / BM, f = n % BM;
    const float* base = p.scratch + (((size_t)tile * p.k_splits) * bn + t) * BM + f;
    acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
    for (int s = 0; s < p.k_splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(base + (size_t)s * bn * BM);
      acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    }
    if (p.epilogue == SB_EPI_BIAS) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        acc[i] += p.bias_dtype == SB_F32 ? bias_at<float>(p.bias, n + i) : bias_at<bf16>(p.bias, n + i);
    }
  };
  auto store4 = [](bf16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
  };
  for (int task = threadIdx.x; task < (head_hi - head_lo) * per_head; task += RR_THREADS) {
    const int head = head_lo + task / per_head, k = task % per_head;      // q heads, then k heads, then v heads
    const bool is_v = head >= r.n_q_heads + r.n_kv_heads;
    if (head >= r.n_q_heads && !stores) continue;
    bf16* dst = head < r.n_q_heads ? q_out + ((size_t)t * r.n_q_heads + head) * hd
                : is_v ? cache + v_base + (size_t)(head - r.n_q_heads - r.n_kv_heads) * r.page_size * hd
                       : cache + k_base + (size_t)(head - r.n_q_heads) * r.page_size * hd;
    float a[4], b[4];
    if (k >= pair_tasks) {                           // beyond the rotated part: a copy
      const int e = r.rot + 4 * (k - pair_tasks);
      sum4(head * hd + e, a);
      store4(dst + e, a[0], a[1], a[2], a[3]);
      continue;
    }
    const int e = 4 * k;
    sum4(head * hd + e, a);
    sum4(head * hd + e + half, b);
    if (is_v) {
      store4(dst + e, a[0], a[1], a[2], a[3]);
      store4(dst + e + half, b[0], b[1], b[2], b[3]);
    } else {
      const float4 c = *reinterpret_cast<const float4*>(rr_cs + e);
      const float4 sn = *reinterpret_cast<const float4*>(rr_cs + half + e);
      store4(dst + e, sb_rot_lo(a[0], b[0], c.x, sn.x), sb_rot_lo(a[1], b[1], c.y, sn.y),
             sb_rot_lo(a[2], b[2], c.z, sn.z), sb_rot_lo(a[3], b[3], c.w, sn.w));
      store4(dst + e + half, sb_rot_hi(a[0], b[0], c.x, sn.x), sb_rot_hi(a[1], b[1], c.y, sn.y),
             sb_rot_hi(a[2], b[2], c.z, sn.z), sb_rot_hi(a[3], b[3], c.w, sn.w));
    }
  }
}

// The same sum for a row-wise epilogue, followed by the RMSNorm of the finished rows: what a
// pre-norm block's next product reads.  A cluster of RN_CLUSTER blocks takes one token; a block
// adds the partial tiles of its part of the row, writes the float32 result, and the blocks
// exchange their sums of squares through each other's shared memory, so that the row is neither
// written and read again for the norm nor waits for another launch.  The sum of squares is added
// in a fixed order (threads, warps, blocks), so the result does not depend on timing.
constexpr int RN_CLUSTER = 4, RN_THREADS = 256, RN_VEC = 4;
constexpr int RN_MAX_WIDTH = RN_CLUSTER * RN_THREADS * RN_VEC * 4;

__device__ __forceinline__ void rn_load4(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void rn_load4(const bf16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void rn_store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void rn_store4(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TW, typename TN>
__global__ void __launch_bounds__(RN_THREADS)
tc5_reduce_norm_kernel(const Tc5Params p, int bn, const TW* __restrict__ norm_w, float eps,
                       TN* __restrict__ norm_out) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float warp_sums[RN_THREADS / 32];
  __shared__ float block_sums[RN_CLUSTER];          // slot c is written by block c of the cluster
  sb_pdl_launch();
  const int j = blockIdx.y;                                             // token
  const int c = (int)cluster.block_rank();
  const int groups = p.N / 4, per = (groups + RN_CLUSTER - 1) / RN_CLUSTER;
  const int g0 = c * per, g1 = min(groups, g0 + per);
  float wv[RN_VEC][4];
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {                 // the norm's weights wait for nobody
    const int g = g0 + threadIdx.x + i * RN_THREADS;
    if (g < g1) rn_load4(norm_w + (size_t)g * 4, wv[i]);
  }
  sb_pdl_wait();
  float v[RN_VEC][4];
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int g = g0 + threadIdx.x + i * RN_THREADS;
    if (g >= g1) continue;
    const int e = g * 4, tile = e / BM, f = e % BM;
    const float* base = p.scratch + (((size_t)tile * p.k_splits) * bn + j) * BM + f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s = 0; s < p.k_splits; ++s) {
      const float4 t = *reinterpret_cast<const float4*>(base + (size_t)s * bn * BM);
      acc[0] += t.x; acc[1] += t.y; acc[2] += t.z; acc[3] += t.w;
    }
    if (p.epilogue == SB_EPI_BIAS) {
      float b[4];
      if (p.bias_dtype == SB_F32) rn_load4((const float*)p.bias + e, b);
      else rn_load4((const bf16*)p.bias + e, b);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += b[k];
    } else if (p.epilogue == SB_EPI_RESIDUAL) {
      float r[4];
      rn_load4(p.residual + (size_t)j * p.N + e, r);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += r[k];
    }
    rn_store4((float*)p.out + (size_t)j * p.N + e, acc);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[i][k] = acc[k];
      sq = fmaf(acc[k], acc[k], sq);
    }
  }
  sq = sb_warp_sum(sq);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < RN_CLUSTER) {                    // thread t tells block t of the cluster
    float total = 0.0f;
    for (int i = 0; i < RN_THREADS / 32; ++i) total += warp_sums[i];
    *cluster.map_shared_rank(&block_sums[c], threadIdx.x) = total;
  }
  cluster.sync();                                    // after it nobody touches another block's memory
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < RN_CLUSTER; ++i) total += block_sums[i];
  const float inv = 1.0f / sqrtf(total / (float)p.N + eps);
#pragma unroll
  for (int i = 0; i < RN_VEC; ++i) {
    const int g = g0 + threadIdx.x + i * RN_THREADS;
    if (g >= g1) continue;
    float y[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) y[k] = (v[i][k] * inv) * wv[i][k];
    rn_store4(norm_out + (size_t)j * p.N + (size_t)g * 4, y);
  }
}

// --------------------------------------------------------------------------- host side
// A [rows, K] bfloat16 row-major matrix as a tensor map with boxes of box_rows x 64.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, bool SWAPPED, typename TO>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Tc5Params& p, int blocks,
           cudaStream_t stream) {
  static bool configured = false;
  constexpr int smem = smem_bytes(BN, STAGES);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<BN, STAGES, SWAPPED, TO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess)
      SB_FAIL(SB_ERR_CUDA, "sb_gemm_tc5: shared memory opt-in failed: %s", cudaGetErrorString(e));
    configured = true;
  }
  sb_launch<SB_K_TC5>(gemm_tc5_kernel<BN, STAGES, SWAPPED, TO>, dim3(blocks), dim3(kernel_threads(BN, SWAPPED)), smem, stream,
                  ma, mb, p);
  SB_CHECK_LAUNCH("sb_gemm_tc5");
  return SB_OK;
}

template <int BN, int STAGES, typename TO>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const Tc5Params& p, int blocks,
                      cudaStream_t stream) {
  static bool configured = false;
  constexpr int smem = persist_smem_bytes(BN, STAGES);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc5_persistent_kernel<BN, STAGES, TO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess)
      SB_FAIL(SB_ERR_CUDA, "sb_gemm_tc5: shared memory opt-in failed: %s", cudaGetErrorString(e));
    configured = true;
  }
  sb_launch<SB_K_TC5>(gemm_tc5_persistent_kernel<BN, STAGES, TO>, dim3(blocks), dim3(THREADS), smem, stream, ma,
            mb, p);
  SB_CHECK_LAUNCH("sb_gemm_tc5 (persistent)");
  return SB_OK;
}

// Tile width of the persistent kernel.  A product takes about (waves of tiles over the SMs) x
// (tile width) units of time, so the candidate with the smallest product wins, the wider one
// on a tie (fewer tiles, fewer epilogues).  Any multiple of 16 up to 256 is a legal MMA width
// at 128 rows; the candidates are the ones that fit a four-stage ring.  For 2,048 rows and
// 3,584 features on 148 SMs: 256 wide gives 224 tiles (2 waves, the second half empty: 512
// units), 224 wide 256 tiles (448), 208 wide 288 tiles (1.95 waves: 416).
constexpr int PERSIST_BNS[] = {256, 240, 224, 208, 192};
// One tile width for every many-rows product, for measurements and tests: sb_gemm_tc5_force_width
// sets it (0: by the sizes), SB_TC5_BN=<width> in the environment is its first value.
int g_forced_bn = -1;
int valid_bn(int v) {
  for (int bn : PERSIST_BNS) if (bn == v) return v;
  return 0;
}
int forced_bn() {
  if (g_forced_bn < 0) {
    const char* e = getenv("SB_TC5_BN");
    g_forced_bn = valid_bn(e ? atoi(e) : 0);
  }
  return g_forced_bn;
}
int persistent_bn(int M, int N, int n_sms) {
  if (const int forced = forced_bn()) return forced;
  const int tiles_m = (M + BM - 1) / BM;
  int best = 0;
  long best_cost = 0;
  for (int bn : PERSIST_BNS) {
    const long tiles = (long)tiles_m * ((N + bn - 1) / bn);
    const long cost = ((tiles + n_sms - 1) / n_sms) * bn;
    if (!best || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}

// The pair kernel: clusters of two blocks, as many as the device runs at once (cached per kernel).
template <int BN, typename TO>
int pair_clusters() {
  static int clusters = -1;
  if (clusters >= 0) return clusters;
  constexpr int smem = pair_smem_bytes(BN, PAIR_STAGES);
  clusters = 0;
  if (cudaFuncSetAttribute(gemm_tc5_pair_kernel<BN, PAIR_STAGES, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           smem) != cudaSuccess) {
    cudaGetLastError();
    return clusters;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2);
  cfg.blockDim = dim3(PAIR_THREADS);
  cfg.dynamicSmemBytes = smem;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tc5_pair_kernel<BN, PAIR_STAGES, TO>, &cfg) == cudaSuccess && n > 0)
    clusters = n;
  else
    cudaGetLastError();
  return clusters;
}

template <int BN, typename TO>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const Tc5Params& p, int clusters,
                cudaStream_t stream) {
  sb_launch<SB_K_TC5>(gemm_tc5_pair_kernel<BN, PAIR_STAGES, TO>, dim3(2 * clusters), dim3(PAIR_THREADS),
                      pair_smem_bytes(BN, PAIR_STAGES), stream, ma, mb, p);
  SB_CHECK_LAUNCH("sb_gemm_tc5 (pairs)");
  return SB_OK;
}

// Whether products of more than 128 rows run on pairs of SMs: sb_gemm_tc5_pairs(0 or 1) decides,
// else the environment (SB_TC5_PAIR=0 keeps every product on the one-block kernels).
int g_pair_mode = -1;
bool pair_enabled() {
  if (g_pair_mode >= 0) return g_pair_mode != 0;
  static const bool on = [] {
    const char* e = getenv("SB_TC5_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Tile width of the pair kernel.  The prefill products run at the GPU's power limit, where a
// partly filled last wave of tiles costs next to nothing (the idle SMs' share of the power lets
// the busy ones clock higher) and what counts is the work per flop: the columns computed beyond
// N in the last tile, and the operand traffic, which grows as the tile narrows (per flop as
// 1/width + 1/256; about a third of the energy).  Measured at 2,048 rows, pairs of SMs, widths
// 256 / 240 / 224 / 208 / 192: 3,584 x 3,584 57 / 70 / 65 / 65 / 71 us, 37,888 x 3,584 415 / 435 /
// 426 / 438 / 439 us, 4,608 x 3,584 54 / 69 / 80 / 77 / 66 us.  So the widest tile, unless a
// narrower one leaves clearly fewer columns outside the matrix.
int pair_bn(int M, int N, int clusters) {
  if (const int forced = forced_bn()) return forced;
  // Few rows: when even the widest tiles do not give every pair of SMs one, the product takes as
  // long as one tile does, and the narrowest width that still fits one wave wins (512 rows,
  // 3,584 x 18,944: 122 us at 256 columns, 108 us at 192).
  const long tiles_m = (M + PAIR_M - 1) / PAIR_M;
  if (clusters > 0 && tiles_m * ((N + 255) / 256) <= clusters) {
    int narrow = 256;
    for (int bn : PERSIST_BNS)
      if (tiles_m * ((N + bn - 1) / bn) <= clusters && bn < narrow) narrow = bn;
    return narrow;
  }
  int best = 0;
  double best_cost = 0.0;
  for (int bn : PERSIST_BNS) {
    const double padded = (double)((N + bn - 1) / bn) * bn;
    const double cost = padded * (1.0 + 0.3 * ((256.0 / bn + 1.0) / 2.0 - 1.0));
    if (!best || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}

}  // namespace

namespace {
int pair_splits(int M, int N, int K, int clusters);
// Whether the many-rows product runs on pairs of SMs: from 129 rows on, and from 65 rows on when
// it would split K there (one row tile either way, but the pairs share a tile's K blocks out,
// while one block per tile would leave most SMs without work).
bool pair_form(int M, int N, int K, int n_sms) {
  if (N < 192 || n_sms <= 1 || !pair_enabled()) return false;
  return M > BM || (M > 64 && pair_splits(M, N, K, n_sms / 2) > 1);
}
// K splits of the pair kernel.  When even 256-column tiles leave at least half of the pairs of
// SMs without one and the inner dimension is long enough, every tile's K blocks are shared out
// over as many pairs as there are to spare (at most eight, at least eight K blocks each); the
// tiles are then 256 columns wide.  1: no split.
int pair_splits(int M, int N, int K, int clusters) {
  if (forced_bn() || N % 16) return 1;
  const long tiles = (long)((M + PAIR_M - 1) / PAIR_M) * ((N + 255) / 256);
  const int n_k = (K + BK - 1) / BK;
  if (clusters <= 0 || 2 * tiles > clusters) return 1;
  int splits = (int)(clusters / tiles);
  if (splits > 8) splits = 8;
  if (splits > n_k / 8) splits = n_k / 8;
  if (splits < 2) return 1;
  const int k_per = (n_k + splits - 1) / splits;
  return (n_k + k_per - 1) / k_per;
}
}  // namespace

// 0 when no kernel has given up on a wait since the last call; else the code of the wait
// (1 producer/empty, 2 producer drain, 3 MMA/full, 4 epilogue/accumulator).  Reading
// synchronizes with the device.
extern "C" int sb_tc5_status() { return tc5_read_status(); }

// 1: products of more than 128 rows run on pairs of SMs, 0: on single SMs, -1: by the environment.
extern "C" void sb_gemm_tc5_pairs(int mode) { g_pair_mode = mode; }

// One of 256, 240, 224, 208, 192: every many-rows product uses that tile width; anything else:
// the width is chosen by the sizes again.
extern "C" void sb_gemm_tc5_force_width(int bn) { g_forced_bn = valid_bn(bn); }

// The tile width the product of these sizes runs with in its many-rows form (for tests that
// want every width covered); 0 when that form does not run.
extern "C" int sb_gemm_tc5_tile_width(int M, int N, int n_sms) {
  if (M <= 64 || N < 192 || n_sms <= 0) return 0;
  if (n_sms > 1 && M > BM && pair_enabled()) return pair_bn(M, N, n_sms / 2);
  return persistent_bn(M, N, n_sms);
}

namespace {

int swapped_bn(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

// How many blocks share one output tile of the swapped form: enough to give every SM two
// blocks, at least four K tiles each, and no block without work.
int choose_splits(int N, int K, int n_sms) {
  const int tiles = (N + BM - 1) / BM, n_k = (K + BK - 1) / BK;
  int splits = n_sms > 0 ? 2 * n_sms / tiles : 1;       // two blocks fit an SM
  if (splits > 16) splits = 16;
  if (splits > n_k / 4) splits = n_k / 4;
  if (splits < 1) splits = 1;
  const int k_per = (n_k + splits - 1) / splits;
  return (n_k + k_per - 1) / k_per;
}

}  // namespace

// Bytes of scratch (partial tiles) the swapped form needs for these sizes; 0 when K is not split.
extern "C" size_t sb_gemm_tc5_scratch_bytes(int M, int N, int K, int n_sms) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 64 && pair_form(M, N, K, n_sms)) {
    // the many-rows form on pairs of SMs, when it splits K: [split][row][column]
    const int splits = pair_splits(M, N, K, n_sms / 2);
    return splits > 1 ? (size_t)splits * M * N * sizeof(float) : 0;
  }
  if (M > 64) return 0;
  const int splits = choose_splits(N, K, n_sms);
  if (splits <= 1) return 0;
  const int tiles = (N + BM - 1) / BM;
  return (size_t)tiles * splits * swapped_bn(M) * BM * sizeof(float);
}

// Whether the swapped split-K form can finish these rows with the fused reduce + norm kernel.
static bool norm_fuses(int M, int N, int K, int n_sms, int epilogue, int out_dtype, int form) {
  const bool normal = form == 1 || (form == 0 && M > 64);
  return !normal && M <= 64 && choose_splits(N, K, n_sms) > 1 && epilogue != SB_EPI_SWIGLU &&
         out_dtype == SB_F32 && N % 4 == 0 && N <= RN_MAX_WIDTH;
}

extern "C" int sb_gemm_tc5_fuses_norm(int M, int N, int K, int n_sms, int epilogue, int out_dtype,
                                      int form) {
  return norm_fuses(M, N, K, n_sms, epilogue, out_dtype, form) ? 1 : 0;
}

// Whether the swapped split-K form can finish these rows with the rotation and the cache write.
static bool rope_fuses(int M, int N, int K, int n_sms, int n_q_heads, int n_kv_heads, int hd, int rot,
                       int has_kv) {
  if (M <= 0 || M > 64 || N <= 0 || K <= 0 || n_q_heads <= 0 || hd <= 0 || (has_kv && n_kv_heads <= 0)) return false;
  if (N != (n_q_heads + (has_kv ? 2 * n_kv_heads : 0)) * hd) return false;
  if (rot < 0 || rot > hd || (rot & 7) || ((hd - rot) & 3) || (hd & 3)) return false;
  return choose_splits(N, K, n_sms) > 1;
}

extern "C" int sb_gemm_tc5_fuses_rope(int M, int N, int K, int n_sms, int n_q_heads, int n_kv_heads,
                                      int hd, int rot, int has_kv) {
  return rope_fuses(M, N, K, n_sms, n_q_heads, n_kv_heads, hd, rot, has_kv) ? 1 : 0;
}

static int tc5_run(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
                   int K, int epilogue, const void* bias, int bias_dtype,
                   const float* residual, void* out, int out_dtype, void* scratch,
                   size_t scratch_bytes, int n_sms, int form, const SbLinearExtras* extras,
                   cudaStream_t stream) {
  const SbLinearExtras* norm = extras && extras->norm_weight ? extras : nullptr;
  const SbRopeStore* rope = extras ? extras->rope : nullptr;
  if (rope) {
    // the product's rows go through the rotation into q_out and the cache; `out` is not written
    if (norm || (epilogue != SB_EPI_BIAS && epilogue != SB_EPI_NONE) || form == 1 ||
        !rope_fuses(M, N, K, n_sms, rope->n_q_heads, rope->n_kv_heads, rope->hd, rope->rot, rope->cache != nullptr))
      SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: these sizes do not take the fused rotation "
              "(see sb_gemm_tc5_fuses_rope)");
    if (!rope->q_out || !rope->inv_freq || !rope->row_pos || (rope->cache && (!rope->row_seq || !rope->page_off ||
        !rope->page_ids || rope->page_size <= 0)))
      SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: rotation arguments missing");
    if ((((uintptr_t)rope->q_out | (uintptr_t)rope->cache) & 7) || ((uintptr_t)rope->inv_freq & 15))
      SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: unaligned rotation operands");
    if (epilogue == SB_EPI_BIAS && !bias) SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: bias epilogue without a bias");
  } else if (int rc = sb_check_linear_args("sb_gemm_tc5", M, N, K, epilogue, bias, residual, out_dtype))
    return rc;
  if (norm) {
    if (epilogue == SB_EPI_SWIGLU || out_dtype != SB_F32)
      SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: a norm follows a float32 product without SwiGLU");
    if (!norm->norm_out || !sb_valid_dtype(norm->norm_weight_dtype) ||
        !sb_valid_dtype(norm->norm_out_dtype) || !(norm->norm_eps >= 0.0f))
      SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: norm output, dtype codes %d %d or eps %g",
              norm->norm_weight_dtype, norm->norm_out_dtype, norm->norm_eps);
    if (!norm_fuses(M, N, K, n_sms, epilogue, out_dtype, form) ||
        (((uintptr_t)norm->norm_weight | (uintptr_t)norm->norm_out | (uintptr_t)out |
          (uintptr_t)residual | (uintptr_t)bias) & 15)) {
      // the product as usual, then the norm as a kernel of its own
      if (int rc = tc5_run(A, a_dtype, W, w_dtype, M, N, K, epilogue, bias, bias_dtype, residual,
                           out, out_dtype, scratch, scratch_bytes, n_sms, form, nullptr, stream))
        return rc;
      return sb_rmsnorm((const float*)out, nullptr, M, N, norm->norm_weight, norm->norm_weight_dtype,
                        norm->norm_eps, norm->norm_out, norm->norm_out_dtype, stream);
    }
  }
  if (a_dtype != SB_BF16 || w_dtype != SB_BF16)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: takes bfloat16 operands (got dtype codes %d, %d)",
            a_dtype, w_dtype);
  if (K % 8)
    SB_FAIL(SB_ERR_UNSUPPORTED,
            "sb_gemm_tc5: the inner size must be a multiple of 8 for 16-byte rows, got %d", K);
  if (((uintptr_t)A | (uintptr_t)W) & 15) SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: operands must be 16-byte aligned");
  if (!sb_valid_dtype(out_dtype)) SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: out dtype %d", out_dtype);

  Tc5Params p;
  p.M = M; p.N = N; p.K = K; p.epilogue = epilogue; p.bias = bias; p.bias_dtype = bias_dtype;
  p.residual = residual; p.out = out; p.k_splits = 1; p.scratch = nullptr;
  // rows of the output, the residual and the bias chunks start on 16-byte boundaries
  // (SB_TC5_ROWWISE=0: never, for measurements)
  static const bool rowwise_on = [] { const char* e = getenv("SB_TC5_ROWWISE"); return !(e && e[0] == '0'); }();
  p.rowwise = rowwise_on && N % 16 == 0 && (((uintptr_t)out | (uintptr_t)residual | (uintptr_t)bias) & 15) == 0;
  p.warm = extras ? (const char*)extras->warm : nullptr;
  p.warm_bytes = extras ? sb_warm_bytes(extras->warm, extras->warm_bytes) : 0;
  CUtensorMap ma, mb;
  // form: 0 picks by the number of rows, 1 forces the normal form, 2 the swapped form
  const bool normal = form == 1 || (form == 0 && M > 64);
  if (form == 2 && M > 64) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: the swapped form takes at most 64 rows");
  if (normal && M > 64 && pair_form(M, N, K, n_sms)) {
    // at least two row tiles, wide output: the persistent kernel on pairs of SMs
    int splits = p.rowwise ? pair_splits(M, N, K, n_sms / 2) : 1;
    if (splits > 1 && (!scratch || scratch_bytes < (size_t)splits * M * N * sizeof(float) || ((uintptr_t)scratch & 255)))
      splits = 1;                                       // no room for the partial sums: the whole K per tile
    const int bn = splits > 1 ? 256 : pair_bn(M, N, n_sms / 2);
    p.k_splits = splits;
    p.scratch = splits > 1 ? (float*)scratch : nullptr;
    p.tiles_a = (M + PAIR_M - 1) / PAIR_M;
    p.tiles_b = (N + bn - 1) / bn;
    const long n_tiles = (long)p.tiles_a * p.tiles_b * splits;
    if (n_tiles > 2147483647L) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: too many tiles");
    int clusters = 0;
#define SB_TC5_PAIR_CLUSTERS(BN_)                                                                  \
    if (bn == BN_) clusters = out_dtype == SB_F32 ? pair_clusters<BN_, float>() : pair_clusters<BN_, bf16>();
    SB_TC5_PAIR_CLUSTERS(256) SB_TC5_PAIR_CLUSTERS(240) SB_TC5_PAIR_CLUSTERS(224) SB_TC5_PAIR_CLUSTERS(208)
    SB_TC5_PAIR_CLUSTERS(192)
#undef SB_TC5_PAIR_CLUSTERS
    if (splits > 1) clusters = pair_clusters<256, float>();   // the kernel that writes the partial sums
    if (clusters > 0) {                               // else: the one-block kernel below
      if (!make_map(&ma, A, M, K, BM) || !make_map(&mb, W, N, K, bn / 2))
        SB_FAIL(SB_ERR_CUDA, "sb_gemm_tc5: cuTensorMapEncodeTiled failed");
      if (n_tiles < clusters) clusters = (int)n_tiles;
      if (splits > 1) {
        // the partial sums, then their sum in split order with the epilogue
        if (int rc = launch_pair<256, float>(ma, mb, p, clusters, stream)) return rc;
        const long work = (long)M * (N / 16);
        const dim3 rgrid((unsigned)((work + 255) / 256));
        if (out_dtype == SB_F32) sb_launch<SB_K_REDUCE>(tc5_splitk_reduce_kernel<float>, rgrid, dim3(256), 0, stream, p);
        else sb_launch<SB_K_REDUCE>(tc5_splitk_reduce_kernel<bf16>, rgrid, dim3(256), 0, stream, p);
        SB_CHECK_LAUNCH("sb_gemm_tc5 (pairs, sum of the K splits)");
        return SB_OK;
      }
#define SB_TC5_PAIR_LAUNCH(BN_)                                                                    \
      if (bn == BN_)                                                                               \
        return out_dtype == SB_F32 ? launch_pair<BN_, float>(ma, mb, p, clusters, stream)          \
                                   : launch_pair<BN_, bf16>(ma, mb, p, clusters, stream);
      SB_TC5_PAIR_LAUNCH(256) SB_TC5_PAIR_LAUNCH(240) SB_TC5_PAIR_LAUNCH(224) SB_TC5_PAIR_LAUNCH(208)
      SB_TC5_PAIR_LAUNCH(192)
#undef SB_TC5_PAIR_LAUNCH
    }
    p.k_splits = 1;
    p.scratch = nullptr;
  }
  if (normal && N >= 192 && n_sms > 0) {
    // many rows, wide output: the persistent kernel
    const int bn = persistent_bn(M, N, n_sms);
    p.tiles_a = (M + BM - 1) / BM;
    p.tiles_b = (N + bn - 1) / bn;
    if (!make_map(&ma, A, M, K, BM) || !make_map(&mb, W, N, K, bn))
      SB_FAIL(SB_ERR_CUDA, "sb_gemm_tc5: cuTensorMapEncodeTiled failed");
    const long n_tiles = (long)p.tiles_a * p.tiles_b;
    if (n_tiles > 2147483647L) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: too many tiles");
    const int blocks = (int)(n_tiles < n_sms ? n_tiles : n_sms);
#define SB_TC5_PERSIST(BN_)                                                                        \
    if (bn == BN_)                                                                                 \
      return out_dtype == SB_F32 ? launch_persistent<BN_, 4, float>(ma, mb, p, blocks, stream)     \
                                 : launch_persistent<BN_, 4, bf16>(ma, mb, p, blocks, stream);
    SB_TC5_PERSIST(256) SB_TC5_PERSIST(240) SB_TC5_PERSIST(224) SB_TC5_PERSIST(208) SB_TC5_PERSIST(192)
#undef SB_TC5_PERSIST
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: no persistent kernel of width %d", bn);
  }
  if (normal) {
    constexpr int BN = 128;
    p.tiles_a = (M + BM - 1) / BM;
    p.tiles_b = (N + BN - 1) / BN;
    if (!make_map(&ma, A, M, K, BM) || !make_map(&mb, W, N, K, BN))
      SB_FAIL(SB_ERR_CUDA, "sb_gemm_tc5: cuTensorMapEncodeTiled failed");
    const long blocks = (long)p.tiles_a * p.tiles_b;
    if (blocks > 2147483647L) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_gemm_tc5: too many tiles");
    if (out_dtype == SB_F32) return launch<BN, 3, false, float>(ma, mb, p, (int)blocks, stream);
    return launch<BN, 3, false, bf16>(ma, mb, p, (int)blocks, stream);
  }
  // swapped form: weights are the A operand
  const int bn = swapped_bn(M);
  p.tiles_a = (N + BM - 1) / BM;
  p.tiles_b = 1;
  const int splits = choose_splits(N, K, n_sms);
  p.k_splits = splits;
  if (splits > 1) {
    const size_t need = sb_gemm_tc5_scratch_bytes(M, N, K, n_sms);
    if (!scratch || scratch_bytes < need)
      SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: %zu bytes of scratch needed, %zu given", need, scratch_bytes);
    if ((uintptr_t)scratch & 255) SB_FAIL(SB_ERR_ARG, "sb_gemm_tc5: scratch must be 256-byte aligned");
    p.scratch = (float*)scratch;
  }
  if (!make_map(&ma, W, N, K, BM) || !make_map(&mb, A, M, K, bn))
    SB_FAIL(SB_ERR_CUDA, "sb_gemm_tc5: cuTensorMapEncodeTiled failed");
  const int blocks = p.tiles_a * splits;
  // an L2 hint pays only when many blocks share it (each block's share goes through its SM's
  // copy engine): at most 48 prefetches of 16 KB a block
  if ((size_t)blocks * 48 * SB_WARM_CHUNK < p.warm_bytes) p.warm_bytes = 0;
  int rc;
  // Stages are chosen so that two blocks fit an SM (at most about 100 KB of shared memory each).
  // At up to 16 rows four stages (72 KB) do as well as six when the kernel runs alone, and leave
  // room on every SM for a block of the next product, which starts early and requests its first
  // weight tiles while this one ends: the decode step at batch 8 took 3.073 ms with four stages,
  // 3.097 with five, 3.104 with six, 3.124 with three (alternating runs on one GPU).  At 32 and
  // 64 rows fewer stages were slower (batch 64: 5.445 ms with three, 5.380 with four).
#define SB_TC5_SWAPPED(BN_, ST_)                                                             \
  rc = out_dtype == SB_F32 ? launch<BN_, ST_, true, float>(ma, mb, p, blocks, stream)         \
                           : launch<BN_, ST_, true, bf16>(ma, mb, p, blocks, stream);
  if (bn == 16) { SB_TC5_SWAPPED(16, 4) }
  else if (bn == 32) { SB_TC5_SWAPPED(32, 5) }
  else { SB_TC5_SWAPPED(64, 4) }
#undef SB_TC5_SWAPPED
  if (rc != SB_OK || splits <= 1) return rc;
  if (rope) {
    const size_t smem = (size_t)(rope->rot > 0 ? rope->rot : 2) * sizeof(float);
    // the heads of a token are shared out over enough blocks for two per SM, at least four
    const int n_heads = rope->n_q_heads + (rope->cache ? 2 * rope->n_kv_heads : 0);
    int shares = n_sms > 0 ? (2 * n_sms + M - 1) / M : 4;
    shares = shares < 4 ? 4 : (shares > n_heads ? n_heads : shares);
    sb_launch<SB_K_REDUCE>(tc5_reduce_rope_kernel, dim3((unsigned)M, (unsigned)shares), dim3(RR_THREADS), smem,
                           stream, p, bn, *rope);
    SB_CHECK_LAUNCH("sb_gemm_tc5 (reduce + rotation)");
    return SB_OK;
  }
  if (norm) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(RN_CLUSTER, (unsigned)M);
    cfg.blockDim = dim3(RN_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = RN_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (sb_pdl_enabled() & SB_K_REDUCE) ? 2 : 1;
    SB_DISPATCH_DTYPE(norm->norm_weight_dtype, TW, {
      SB_DISPATCH_DTYPE(norm->norm_out_dtype, TN, {
        cudaLaunchKernelEx(&cfg, tc5_reduce_norm_kernel<TW, TN>, p, bn, (const TW*)norm->norm_weight,
                           norm->norm_eps, (TN*)norm->norm_out);
      });
    });
    SB_CHECK_LAUNCH("sb_gemm_tc5 (reduce + norm)");
    return SB_OK;
  }
  const int n_out = epilogue == SB_EPI_SWIGLU ? N / 2 : N;
  const long work = (long)((n_out + 3) / 4) * M;
  const dim3 rgrid((unsigned)((work + 255) / 256));
  if (out_dtype == SB_F32) sb_launch<SB_K_REDUCE>(tc5_reduce_kernel<float>, rgrid, dim3(256), 0, stream, p, bn);
  else sb_launch<SB_K_REDUCE>(tc5_reduce_kernel<bf16>, rgrid, dim3(256), 0, stream, p, bn);
  SB_CHECK_LAUNCH("sb_gemm_tc5 (reduce)");
  return SB_OK;
}

extern "C" int sb_gemm_tc5(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
                           int K, int epilogue, const void* bias, int bias_dtype,
                           const float* residual, void* out, int out_dtype, void* scratch,
                           size_t scratch_bytes, int n_sms, int form, cudaStream_t stream) {
  return tc5_run(A, a_dtype, W, w_dtype, M, N, K, epilogue, bias, bias_dtype, residual, out,
                 out_dtype, scratch, scratch_bytes, n_sms, form, nullptr, stream);
}

// The product with what may accompany it (see SbLinearExtras).  norm_out = RMSNorm(out) *
// norm_weight over the rows of the float32 result comes from one kernel with the split-K sum
// where that form runs, else from a norm kernel after the product.  The L2 hint is taken by
// the non-persistent kernel.
extern "C" int sb_gemm_tc5_ex(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
                              int K, int epilogue, const void* bias, int bias_dtype,
                              const float* residual, void* out, int out_dtype, void* scratch,
                              size_t scratch_bytes, int n_sms, int form,
                              const SbLinearExtras* extras, cudaStream_t stream) {
  return tc5_run(A, a_dtype, W, w_dtype, M, N, K, epilogue, bias, bias_dtype, residual, out,
                 out_dtype, scratch, scratch_bytes, n_sms, form, extras, stream);
}
