// The persistent product on pairs of SMs: a cluster of two blocks computes a 256 x BN tile with
// one MMA of 256 rows (`tcgen05.mma.cta_group::2`).  Block r of the pair loads rows
// [128 r, 128 r + 128) of the A tile and rows [BN/2 r, BN/2 r + BN/2) of the B tile into its own
// shared memory and holds rows [128 r, 128 r + 128) of the accumulator in its own tensor memory;
// the tensor cores of both SMs read both halves of B.  Against the one-block kernel's 128 x BN
// tile every block stages a third less operand data per flop (A + B/2 instead of A + B), and
// every B tile leaves L2 once per 256 rows instead of once per 128.  Each product alone is hardly
// faster for it, but the prefill step runs at the GPU's power limit, and there the step of a
// 7B-sized model took 7 % less time (24.7 against 26.7 ms for 2,048 tokens).
//
// Included by gemm_tc5.cu after the one-block persistent kernel, whose epilogue it shares.
//
// Who signals whom (r = block's rank in its cluster; block 0 issues the MMAs):
//   full[s]      block 0's only.  Block 0's producer arms it with the bytes of both blocks'
//                loads; the TMA loads of both blocks count on it (`.cta_group::2` loads may name
//                a barrier of the other block).
//   empty[s]     one in each block, for that block's producer; block 0's MMA thread commits to
//                both at once (`tcgen05.commit ... multicast::cluster`).
//   acc_full[a]  one in each block, for that block's epilogue warps; committed to both at once.
//   acc_empty[a] block 0's only; the eight epilogue warps of both blocks arrive on it.
// Every wait is bounded; a block whose wait runs out records a code, stops issuing and goes to
// the common end, where the two blocks meet before tensor memory is given back.
//
// Few rows and a long inner dimension leave most pairs without a tile (256 rows of the 3,584 x
// 18,944 product: 14 tiles for 74 pairs).  Then K is split (p.k_splits > 1): a pair's unit of work
// is a tile's stretch of K blocks, its float32 accumulator goes to scratch [split][row][column]
// as it is, and tc5_splitk_reduce_kernel adds the splits in order and applies the epilogue.
#pragma once

namespace {

constexpr int PAIR_M = 2 * BM;
constexpr int PAIR_STAGES = 6;
// Two groups of four epilogue warps per block (a warp reaches its quarter of the tensor memory's
// lanes only): the groups take alternate 32-column chunks of the tile, which halves the time the
// last tile's epilogue, hidden behind nothing, takes.
constexpr int PAIR_EPI_GROUPS = 2;
constexpr int PAIR_THREADS = 64 + 128 * PAIR_EPI_GROUPS;
constexpr int pair_stage_bytes(int bn) { return (BM + bn / 2) * BK * 2; }
constexpr int pair_smem_bytes(int bn, int stages) {
  return stages * pair_stage_bytes(bn) + PAIR_EPI_GROUPS * PERSIST_STAGING + 1024 + 256;
}
static_assert(pair_smem_bytes(256, PAIR_STAGES) <= 232448, "the pair kernel's shared memory");
// float32 accumulator, bfloat16 A and B, both K-major, M = 256 over the pair, N = bn
__host__ __device__ constexpr uint32_t pair_instr_desc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(PAIR_M >> 4) << 24);
}

template <int BN, int STAGES, typename TO>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS)
gemm_tc5_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b, const Tc5Params p) {
  static_assert(BN % 16 == 0 && BN <= 256, "the MMA's width");
  static_assert(pair_stage_bytes(BN) % 1024 == 0, "stages keep the swizzle's 1024-byte alignment");
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t staging = tiles + STAGES * pair_stage_bytes(BN);
  const uint32_t bars = staging + PAIR_EPI_GROUPS * PERSIST_STAGING;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;
  const uint32_t acc_full0 = bars + 16 * STAGES, acc_empty0 = acc_full0 + 16;
  const uint32_t tmem_slot = acc_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(smem_raw + (tmem_slot - raw));
  constexpr uint32_t ACC_COLS = 256;                   // column offset of the second accumulator

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  sb_pdl_launch();
  const int S = p.k_splits;                            // K splits of a tile (1: none)
  const int n_tiles = p.tiles_a * p.tiles_b * S;       // units of work: (tile of 256 x BN, split), splits first
  const int n_k_all = (p.K + BK - 1) / BK, k_per = (n_k_all + S - 1) / S;
  const int first = (int)(blockIdx.x >> 1), step = (int)(gridDim.x >> 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, 8 * PAIR_EPI_GROUPS);   // one arrival per epilogue warp of both blocks
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_arrive();                                    // the other block's barriers exist from here on
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0 && lane == 0) {
    // ---- producer (both blocks): this block's half of every stage
    sb_pdl_wait();
    const uint32_t full_of_0 = map_to_block(full0, 0);
    uint32_t it = 0;
    bool ok = true;
    for (int unit = first; unit < n_tiles && ok; unit += step) {
      const int tile = unit / S, split = unit % S;
      const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
      const int a_row = tile_a * PAIR_M + (int)rank * BM, b_row = tile_b * BN + (int)rank * (BN / 2);
      const int k_end = min(n_k_all, (split + 1) * k_per);
      for (int kt = split * k_per; kt < k_end; ++kt, ++it) {
        const uint32_t s = it % STAGES;
        ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, 1);
        if (!ok) break;
        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * pair_stage_bytes(BN));
        const uint32_t a_dst = tiles + s * pair_stage_bytes(BN), b_dst = a_dst + BM * BK * 2;
        tma_load_2d_pair(a_dst, &map_a, kt * BK, a_row, full_of_0 + 8 * s);
        tma_load_2d_pair(b_dst, &map_b, kt * BK, b_row, full_of_0 + 8 * s);
      }
    }
    if (!ok && rank == 0) {
      // let copies that are still in flight land before the block's memory goes away
      for (uint32_t i = it > STAGES ? it - STAGES : 0; i < it; ++i)
        mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, 2);
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer (block 0 for the pair)
    constexpr uint32_t idesc = pair_instr_desc(BN);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int unit = first; unit < n_tiles && ok; unit += step, ++lt) {
      const uint32_t acc = lt & 1;
      ok = mbar_wait(acc_empty0 + 8 * acc, ((lt >> 1) & 1) ^ 1, 5);   // both epilogues have drained it
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
      const int k_begin = (unit % S) * k_per, k_end = min(n_k_all, k_begin + k_per);
      for (int kt = k_begin; kt < k_end; ++kt, ++it) {
        const uint32_t s = it % STAGES;
        ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, 3);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = tiles + s * pair_stage_bytes(BN), b_addr = a_addr + BM * BK * 2;
        const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(b_addr);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16_pair(d_tmem, adesc + (uint64_t)(k * UMMA_K * 2 >> 4),
                         bdesc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, (kt > k_begin || k > 0) ? 1u : 0u);
        umma_commit_pair(empty0 + 8 * s, 3);
      }
      if (ok) umma_commit_pair(acc_full0 + 8 * acc, 3);
    }
  } else if (warp >= 2) {
    // ---- epilogue (both blocks): this warp reads TMEM lanes [32 q, 32 q + 32) of this block's
    // half of the finished accumulator
    sb_pdl_wait();
    const int q = warp & 3, group = (warp - 2) >> 2;
    float* stage = reinterpret_cast<float*>(smem_raw + (staging - raw)) + (warp - 2) * 32 * 33;
    const uint32_t acc_empty_of_0 = map_to_block(acc_empty0, 0);
    uint32_t lt = 0;
    for (int unit = first; unit < n_tiles; unit += step, ++lt) {
      const int tile = unit / S, split = unit % S;
      const int tile_a = tile % p.tiles_a, tile_b = tile / p.tiles_a;
      const uint32_t acc = lt & 1;
      if (!mbar_wait(acc_full0 + 8 * acc, (lt >> 1) & 1, 4)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
      const int m_base = tile_a * PAIR_M + (int)rank * BM + q * 32;
      if (S > 1) {
        // the split's part of the sum as it is: the thread's row, 16 bytes at a time
        const int m = m_base + lane;
        float* dst = p.scratch + ((size_t)split * p.M + (m < p.M ? m : 0)) * p.N;
#pragma unroll 1
        for (int c = group; c < BN / 32; c += PAIR_EPI_GROUPS) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          const int n0 = tile_b * BN + c * 32;
          if (m < p.M)
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (n0 + j < p.N)
                *reinterpret_cast<float4*>(dst + n0 + j) = make_float4(
                    __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      } else {
#pragma unroll 1
      for (int c = group; c < BN / 32; c += PAIR_EPI_GROUPS) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        const int n0 = tile_b * BN + c * 32;
        if (n0 < p.N) store_chunk<TO>(p, stage, r, m_base, n0, lane);
      }
      if (BN % 32 && group == (BN / 32) % PAIR_EPI_GROUPS) {   // a last chunk of 16 columns
        uint32_t r[32];
        tmem_ld16(t_row + (BN / 32) * 32, r);
        const int n0 = tile_b * BN + (BN / 32) * 32;
        if (n0 < p.N) store_chunk<TO, 16>(p, stage, r, m_base, n0, lane);
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_of_0 + 8 * acc);
    }
  }

  // the blocks of a pair leave together: block 0's MMAs read the other block's shared memory,
  // and the other block's loads and arrivals land on block 0's barriers
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// Adds the splits of a product whose K was split (scratch [split][row][column], float32) in
// split order and applies the epilogue.  A thread takes 16 consecutive columns of one row (a
// group of 8 gates and their 8 up values when the epilogue is the fused gate/up one).
template <typename TO>
__global__ void __launch_bounds__(256) tc5_splitk_reduce_kernel(const Tc5Params p) {
  sb_pdl_launch();
  sb_pdl_wait();
  const long groups = (long)p.N / 16, idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)p.M * groups) return;
  const int m = (int)(idx / groups), n0 = (int)(idx % groups) * 16;
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = 0.0f;
  for (int s = 0; s < p.k_splits; ++s) {
    const float4* src = reinterpret_cast<const float4*>(p.scratch + ((size_t)s * p.M + m) * p.N + n0);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 x = src[j];
      v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
    }
  }
  if (p.epilogue == SB_EPI_SWIGLU) {
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = sb_silu_out<TO>(v[j]) * v[j + 8];
    store_row((TO*)p.out + (size_t)m * (p.N / 2) + n0 / 2, o, 8);
    return;
  }
  if (p.epilogue == SB_EPI_BIAS) {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      v[j] += p.bias_dtype == SB_F32 ? bias_at<float>(p.bias, n0 + j) : bias_at<bf16>(p.bias, n0 + j);
  } else if (p.epilogue == SB_EPI_RESIDUAL) {
    const float4* res = reinterpret_cast<const float4*>(p.residual + (size_t)m * p.N + n0);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 x = res[j];
      v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
    }
  }
  store_row((TO*)p.out + (size_t)m * p.N + n0, v, 16);
}

}  // namespace
