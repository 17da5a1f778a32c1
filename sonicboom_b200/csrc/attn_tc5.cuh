// Prefill attention on the fifth-generation tensor cores, for head sizes 64 and 128.  Included
// by attn_mma.cu (same rows, same mask, same parameters as its prefill kernel).
//
// One block takes 256 query rows as two tiles of 128 (row r = new token r / G, query head r % G
// of one key/value head) and walks the visible 64-key cache pages in ascending order; both
// tiles use every K and V page the block loads, which halves the traffic from L2 per flop:
//   warp 0      TMA: K and V pages straight from the cache into rings of a few stages (one
//               tensor map over the cache entry's pages, rows = (page, k|v, head, key),
//               128-byte swizzle);
//   warps 1,10  one warp per query tile issues that tile's tcgen05.mma (one elected lane):
//               S = Q.K^T (128 x 64, accumulator in tensor memory, two buffers, issued two
//               pages ahead of the softmax) and O += P.V (128 x HD, accumulated in tensor
//               memory over all pages).  V is used as stored, [key][head size], as an MN-major
//               operand.  An issuing thread is held up by each commit and wait, so one warp
//               for both tiles left the tensor pipe idle half of the time;
//   warps 2-9   softmax, four warps per query tile: a thread owns one row.  It reads its 64
//               scores with tcgen05.ld, keeps a reference maximum and the row sum in float32
//               registers and writes the probabilities exp2(s - reference) as bfloat16 into
//               the swizzled P tile (two buffers).  The reference follows the running maximum
//               lazily: only when a row's maximum has grown by more than 2^8 over its
//               reference does the warp rescale its rows of O in tensor memory (and the sums)
//               to the new maximum, so probabilities stay below 2^8 and most pages need no
//               pass over O at all.
// Scores, maxima, sums and the output are float32; probabilities are rounded to bfloat16 only
// as the P.V operand, and the row sum uses them before rounding.
//
// Every mbarrier wait is bounded (tc5.cuh); a wait that gives up makes its role stop, the
// others then give up as well, and the block frees its tensor memory and leaves.
#pragma once

#include "tc5.cuh"

namespace {

constexpr int T5_ROWS = 128;                                // rows of a query tile = UMMA M
constexpr int T5_QT = 2;                                    // query tiles per block
constexpr int T5_ST = 3;                                    // depth of the K ring and of the V ring
constexpr int T5_THREADS = 64 + 128 * T5_QT + 32 * (T5_QT - 1);   // + the other tiles' MMA warps
constexpr int T5_SUB = HD / 64 > 0 ? HD / 64 : 1;            // 64-wide pieces of a head
constexpr uint32_t T5_Q_BYTES = T5_SUB * T5_ROWS * 128;     // one query tile
constexpr uint32_t T5_KV_BYTES = T5_SUB * KT * 128;         // one K or one V page
constexpr uint32_t T5_P_BYTES = T5_ROWS * 128;
constexpr uint32_t T5_SMEM =
    T5_QT * T5_Q_BYTES + 2 * T5_ST * T5_KV_BYTES + 2 * T5_QT * T5_P_BYTES + 512;
constexpr uint32_t T5_TILE_COLS = 2 * KT + HD;              // tensor memory of a query tile: S0 S1 O
constexpr uint32_t T5_TMEM_COLS = T5_QT * T5_TILE_COLS <= 256 ? 256 : 512;
constexpr float T5_LAZY = 8.0f;                             // log2 of how far a maximum may run ahead
static_assert(T5_QT * T5_TILE_COLS <= 512, "tensor memory has 512 columns");

// barriers: the rings first (a stage is free when every query tile's product that read it has
// been committed: T5_QT arrivals), then one set per query tile.  PFREE of a page also says "O
// holds every page up to this one".
enum { T5_KFULL = 0, T5_KFREE = T5_ST, T5_VFULL = 2 * T5_ST, T5_VFREE = 3 * T5_ST,
       T5_PER_TILE = 4 * T5_ST,
       T5_SFULL = 0, T5_SFREE = 2, T5_PFULL = 4, T5_PFREE = 6, T5_QFULL = 8,
       T5_TILE_BARS = 9, T5_NBARS = 4 * T5_ST + T5_QT * T5_TILE_BARS };
static_assert(T5_NBARS * 8 + 8 <= 512, "barrier space");

// K-major tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t t5_desc_k(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// MN-major tile with the 128-byte swizzle: a row holds 64 consecutive values of the MN
// dimension for one k; groups of 8 k-rows are 1024 bytes apart, the next 64 MN values are a
// whole [64 keys][128 bytes] piece further on.
__device__ __forceinline__ uint64_t t5_desc_mn(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((KT * 128) >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// float32 accumulator, bfloat16 operands, A K-major, B K-major or MN-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t t5_idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(T5_ROWS >> 4) << 24);
}
__device__ __forceinline__ float t5_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void t5_st_shared16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                               uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

__device__ __forceinline__ void t5_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Multiplies the thread's row of O in tensor memory by `factor` (a whole warp calls this).
__device__ __forceinline__ void t5_rescale(uint32_t taddr, float factor) {
  tc_fence_after();
#pragma unroll
  for (int c = 0; c < HD / 32; ++c) {
    uint32_t t[32];
    tmem_ld32(taddr + c * 32, t);
#pragma unroll
    for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * factor);
    t5_tmem_st32(taddr + c * 32, t);
  }
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
  tc_fence_before();
}

__global__ void __launch_bounds__(T5_THREADS, T5_SMEM <= 115712 && T5_TMEM_COLS <= 256 ? 2 : 1)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_kv, const AttnParams p) {
  extern __shared__ __align__(1024) unsigned char t5_smem[];
  const uint32_t raw = (uint32_t)__cvta_generic_to_shared(t5_smem);
  const uint32_t q_s = raw;                                  // checked below: 1024-byte aligned
  const uint32_t k_s = q_s + T5_QT * T5_Q_BYTES, v_s = k_s + T5_ST * T5_KV_BYTES;
  const uint32_t p_s = v_s + T5_ST * T5_KV_BYTES;            // [query tile][2] P buffers
  const uint32_t bars = p_s + 2 * T5_QT * T5_P_BYTES, tmem_slot = bars + 8 * T5_NBARS;
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(t5_smem + (tmem_slot - raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  sb_pdl_launch();
  sb_pdl_wait();

  // blockIdx.x = (block of query rows, key/value head), heads fastest and the last rows first:
  // blocks are handed out in this order, so the longest ones of every head start first
  const int b = blockIdx.z, kvh = blockIdx.x % p.n_kv_heads;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int row0 = p.seq_row0[b], n_new = p.seq_row0[b + 1] - row0, pos0 = p.seq_pos0[b];
  const int R = n_new * G;
  const int r_base = (int)(gridDim.x / p.n_kv_heads - 1 - blockIdx.x / p.n_kv_heads) * (T5_QT * T5_ROWS);
  if (r_base >= R) return;
  // positions without pages in the sequence's own list: nothing is read
  if (pos0 < 0 || (pos0 + n_new - 1) / KT >= p.page_off[b + 1] - p.page_off[b]) return;
  const int r_last = min(R, r_base + T5_QT * T5_ROWS) - 1;
  const int tile_lo = (p.window > 0 ? max(0, pos0 + r_base / G - p.window + 1) : 0) / KT;
  const int tile_hi = (pos0 + r_last / G) / KT;
  const int n_tiles = tile_hi - tile_lo + 1;
  if (raw & 1023u) {                       // the swizzled tiles need this alignment
    if (threadIdx.x == 0) atomicCAS(&g_status, 0, 10);
    return;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < T5_PER_TILE; ++i) {
      const bool frees = (i >= T5_KFREE && i < T5_VFULL) || i >= T5_VFREE;
      mbar_init(bars + 8 * i, frees ? T5_QT : 1);
    }
    for (int q = 0; q < T5_QT; ++q)
      for (int i = 0; i < T5_TILE_BARS; ++i) {
        const bool by_threads = (i >= T5_SFREE && i < T5_PFREE) || i == T5_QFULL;   // else: one commit
        mbar_init(bars + 8 * (T5_PER_TILE + q * T5_TILE_BARS + i), by_threads ? 128 : 1);
      }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, T5_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;

  if (warp == 0) {
    // ---- producer.  The K ring and the V ring advance independently: whichever has a free
    // stage gets its next page requested, so a wait for one never holds up the other.  The
    // whole warp walks the loop; lanes fetch 32 page ids at a time, one elected lane issues.
    const int32_t* pages = p.page_ids + p.page_off[b] + tile_lo;
    const bool leader = elect_one();
    int ik = 0, iv = 0;                       // next K page and next V page to request
    int ids_k = 0, ids_v = 0;                 // page ids of the 32-page block ik / iv lies in
    uint32_t idle = 0;
    bool ok = true;
    while (ok && (ik < n_tiles || iv < n_tiles)) {
      bool did = false;
      if (ik < n_tiles &&
          (ik < T5_ST || mbar_test(bars + 8 * (T5_KFREE + ik % T5_ST), (ik / T5_ST - 1) & 1))) {
        if ((ik & 31) == 0) ids_k = ik + lane < n_tiles ? pages[ik + lane] : 0;
        const int page = __shfl_sync(0xffffffffu, ids_k, ik & 31);
        const int s = ik % T5_ST;
        if (leader) {
          const int krow = ((page * 2) * p.n_kv_heads + kvh) * KT;
          mbar_expect_tx(bars + 8 * (T5_KFULL + s), T5_KV_BYTES);
#pragma unroll
          for (int sub = 0; sub < T5_SUB; ++sub)
            tma_load_2d(k_s + s * T5_KV_BYTES + sub * (KT * 128), &map_kv, sub * 64, krow,
                        bars + 8 * (T5_KFULL + s));
        }
        __syncwarp();
        ++ik;
        did = true;
      }
      if (iv < n_tiles &&
          (iv < T5_ST || mbar_test(bars + 8 * (T5_VFREE + iv % T5_ST), (iv / T5_ST - 1) & 1))) {
        if ((iv & 31) == 0) ids_v = iv + lane < n_tiles ? pages[iv + lane] : 0;
        const int page = __shfl_sync(0xffffffffu, ids_v, iv & 31);
        const int s = iv % T5_ST;
        if (leader) {
          const int vrow = ((page * 2 + 1) * p.n_kv_heads + kvh) * KT;
          mbar_expect_tx(bars + 8 * (T5_VFULL + s), T5_KV_BYTES);
#pragma unroll
          for (int sub = 0; sub < T5_SUB; ++sub)
            tma_load_2d(v_s + s * T5_KV_BYTES + sub * (KT * 128), &map_kv, sub * 64, vrow,
                        bars + 8 * (T5_VFULL + s));
        }
        __syncwarp();
        ++iv;
        did = true;
      }
      if (did) {
        idle = 0;
      } else if (++idle > WAIT_LIMIT) {
        if (leader) atomicCAS(&g_status, 0, 11);
        ok = false;
      } else if (idle > 4096) {
        __nanosleep(128);
      }
    }
    if (!ok) {
      // let copies that are still in flight land before the block's memory goes away
      for (int i = max(0, ik - T5_ST); i < ik; ++i)
        mbar_wait(bars + 8 * (T5_KFULL + i % T5_ST), (i / T5_ST) & 1, 13);
      for (int i = max(0, iv - T5_ST); i < iv; ++i)
        mbar_wait(bars + 8 * (T5_VFULL + i % T5_ST), (i / T5_ST) & 1, 13);
    }
  } else if (warp == 1 || warp >= 2 + 4 * T5_QT) {
    // ---- MMA issuer of one query tile (warp 1: tile 0; the warps after the softmax warps: the
    // other tiles).  The whole warp walks the loop and the waits, so that addresses,
    // descriptors and ring positions stay warp-uniform values; one elected lane issues the
    // tcgen05 instructions.  Descriptors are built once and advanced by adding
    // (byte offset >> 4) to their address field.  S runs two pages ahead of P.V.
    const int q = warp == 1 ? 0 : warp - (2 + 4 * T5_QT) + 1;
    constexpr uint32_t idesc_s = t5_idesc(KT, false), idesc_o = t5_idesc(HD, true);
    const bool leader = elect_one();
    const uint32_t tb = bars + 8 * (T5_PER_TILE + q * T5_TILE_BARS);
    const uint32_t t_tile = tmem + q * T5_TILE_COLS;
    const uint64_t q_desc = t5_desc_k(q_s + q * T5_Q_BYTES), k_desc = t5_desc_k(k_s),
                   p_desc = t5_desc_k(p_s + q * 2 * T5_P_BYTES), v_desc = t5_desc_mn(v_s);
    int ks = 0, kphase = 0;                       // K ring position of the next S product
    auto issue_s = [&](int i) -> bool {           // S of page i
      const int sb = i & 1;
      if (!mbar_wait(bars + 8 * (T5_KFULL + ks), kphase, 22)) return false;
      if (i >= 2 && !mbar_wait(tb + 8 * (T5_SFREE + sb), ((i >> 1) - 1) & 1, 23)) return false;
      tc_fence_after();
      const uint64_t kd = k_desc + (uint64_t)(ks * (int)(T5_KV_BYTES >> 4));
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_bf16(t_tile + sb * KT,
                    q_desc + (uint64_t)(((kk >> 2) * (T5_ROWS * 128) + (kk & 3) * 32) >> 4),
                    kd + (uint64_t)(((kk >> 2) * (KT * 128) + (kk & 3) * 32) >> 4), idesc_s,
                    kk > 0 ? 1u : 0u);
        umma_commit(tb + 8 * (T5_SFULL + sb));
        umma_commit(bars + 8 * (T5_KFREE + ks));
      }
      __syncwarp();
      if (++ks == T5_ST) { ks = 0; kphase ^= 1; }
      return true;
    };
    bool ok = mbar_wait(tb + 8 * T5_QFULL, 0, 21);
    for (int i = 0; i < 2 && i < n_tiles && ok; ++i) ok = issue_s(i);
    int vs = 0, vphase = 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      ok = mbar_wait(bars + 8 * (T5_VFULL + vs), vphase, 25) &&
           mbar_wait(tb + 8 * (T5_PFULL + (j & 1)), (j >> 1) & 1, 24);
      if (!ok) break;
      tc_fence_after();
      const uint64_t pd = p_desc + (uint64_t)((j & 1) * (int)(T5_P_BYTES >> 4));
      const uint64_t vd = v_desc + (uint64_t)(vs * (int)(T5_KV_BYTES >> 4));
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk)
          umma_bf16(t_tile + 2 * KT, pd + (uint64_t)((kk * 32) >> 4),
                    vd + (uint64_t)((kk * 16 * 128) >> 4), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(tb + 8 * (T5_PFREE + (j & 1)));
        umma_commit(bars + 8 * (T5_VFREE + vs));
      }
      __syncwarp();
      if (++vs == T5_ST) { vs = 0; vphase ^= 1; }
      // the softmax has read S of this page (it wrote P from it): S two pages on
      if (j + 2 < n_tiles) ok = issue_s(j + 2);
    }
  } else {
    // ---- softmax: four warps per query tile, a thread per row; a warp reads the
    // tensor-memory lanes of its quarter
    const int qt = (warp - 2) >> 2;               // warps 2 .. 2 + 4 T5_QT - 1
    const int tid_s = (threadIdx.x - 64) & 127;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t tb = bars + 8 * (T5_PER_TILE + qt * T5_TILE_BARS);
    const uint32_t t_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + qt * T5_TILE_COLS;
    const uint32_t q_tile = q_s + qt * T5_Q_BYTES, p_tile = p_s + qt * 2 * T5_P_BYTES;
    const int rq_base = r_base + qt * T5_ROWS;
    for (int idx = tid_s; idx < T5_ROWS * (HD / 8); idx += 128) {
      const int rr = idx / (HD / 8), ch = idx % (HD / 8);
      const int r = rq_base + rr;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < R)
        v = *reinterpret_cast<const uint4*>(
            p.q + ((size_t)(row0 + r / G) * p.n_q_heads + kvh * G + r % G) * HD + ch * 8);
      t5_st_shared16(q_tile + (ch >> 3) * (T5_ROWS * 128) + rr * 128 + (((ch & 7) ^ (rr & 7)) << 4),
                     v.x, v.y, v.z, v.w);
    }
    fence_async_smem();
    mbar_arrive(tb + 8 * T5_QFULL);

    const int r = rq_base + row;
    const int pos = r < R ? pos0 + r / G : -1;
    // positions of the tile's first and last real row (no real row: every page is masked)
    const int p_lo = rq_base < R ? pos0 + rq_base / G : 0x7fffffff;
    const int p_hi = rq_base < R ? pos0 + min(R - 1, rq_base + T5_ROWS - 1) / G : 0x7fffffff;
    const uint32_t o_addr = t_base + 2 * KT;
    float m_ref = -INFINITY, l = 0.0f;      // reference maximum (log2 domain) and row sum
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1, use = j >> 1, key0 = (tile_lo + j) * KT;
      // this page's P buffer is free when the product that read it two pages ago has finished
      if (j >= 2) ok = mbar_wait(tb + 8 * (T5_PFREE + s), (use - 1) & 1, 33);
      if (ok) ok = mbar_wait(tb + 8 * (T5_SFULL + s), use & 1, 31);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[KT];
      tmem_ld32_nowait(t_base + s * KT, sv);
      tmem_ld32_nowait(t_base + s * KT + 32, sv + 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(tb + 8 * (T5_SFREE + s));

      // every key of the page visible to every row of the tile: no mask to apply
      const bool open = key0 + KT - 1 <= p_lo && (p.window == 0 || p_hi - key0 < p.window);
      if (!open) {
#pragma unroll
        for (int i = 0; i < KT; ++i) {
          const int key = key0 + i;
          const bool seen = key <= pos && (p.window == 0 || pos - key < p.window);
          if (!seen) sv[i] = __float_as_uint(-INFINITY);
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < KT; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(sv[i]));
      const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;   // scale > 0
      if (__any_sync(0xffffffffu, m_tile > m_ref + T5_LAZY || (m_ref == -INFINITY && m_tile > m_ref))) {
        // move this warp's references to the rows' current maxima
        const float m_new = fmaxf(m_ref, m_tile);
        const float factor = m_new == -INFINITY ? 1.0f : t5_ex2(m_ref - m_new);
        if (j > 0) {
          ok = mbar_wait(tb + 8 * (T5_PFREE + ((j - 1) & 1)), ((j - 1) >> 1) & 1, 32);   // O is complete
          if (!ok) break;
          t5_rescale(o_addr, factor);
        }
        l *= factor;
        m_ref = m_new;
      }
      const float base = m_ref == -INFINITY ? 0.0f : m_ref;       // nothing seen yet: exp2(-inf) = 0
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int i = 0; i < KT; i += 2) {
        const float p0 = t5_ex2(fmaf(__uint_as_float(sv[i]), p.scale_log2, -base));
        const float p1 = t5_ex2(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -base));
        sum0 += p0;
        sum1 += p1;
        sv[i >> 1] = pack_bf16(p0, p1);
      }
      l += sum0 + sum1;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        t5_st_shared16(p_tile + s * T5_P_BYTES + row * 128 + ((c ^ (row & 7)) << 4), sv[4 * c],
                       sv[4 * c + 1], sv[4 * c + 2], sv[4 * c + 3]);
      fence_async_smem();
      mbar_arrive(tb + 8 * (T5_PFULL + s));
    }
    if (ok) ok = mbar_wait(tb + 8 * (T5_PFREE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, 34);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      bf16* dst = p.out + ((size_t)(row0 + r / G) * p.n_q_heads + kvh * G + r % G) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t t[32];
        tmem_ld32(o_addr + c * 32, t);       // a whole warp reads; rows beyond R are not written
        if (r < R) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(t[i + 2]) * inv, __uint_as_float(t[i + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(t[i + 4]) * inv, __uint_as_float(t[i + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(t[i + 6]) * inv, __uint_as_float(t[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, T5_TMEM_COLS);
}

// The cache entry's pages [n_pages][k|v][kv head][KT][HD] as a [rows][HD] matrix with boxes of
// 64 rows x 64 values.
inline bool t5_make_map(CUtensorMap* map, const void* cache, long rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)KT};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
