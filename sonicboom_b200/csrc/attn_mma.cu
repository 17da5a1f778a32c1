// Causal grouped-query attention over the paged cache on tensor cores (mma.sync m16n8k16,
// bfloat16 operands, float32 scores, softmax statistics and output accumulator).
//
// This file is compiled once per head size (-DSB_HD=<multiple of 16, at most 256>) into a
// library of its own, so a model pays only for the head size it has.
//
// Rows.  For one sequence and one key/value head, the query rows are the pairs
// (new token t, query head g of the group): row r = t * G + g.  All G query heads that share a
// key/value head therefore share every key and value tile that is loaded, in prefill and in
// decode alike (the reference's tensor-core kernels pack the group the same way,
// core/src/nn/boom_fdec_device.cuh:17-30, core/src/nn/boom_fattn.cu:37-84).
//
//  * prefill kernel: 128 rows per block (8 warps x 16; 64 rows above head size 128), key tiles of one cache page (64 keys)
//    taken in ascending order with a double-buffered cp.async pipeline, online softmax.
//  * decode kernel (at most 16 rows per sequence and head): the keys are cut into splits of 256
//    (512 once the sequence is longer than 4,096) at absolute positions; a block streams one
//    split through double-buffered 64-key tiles, each of its 4 warps taking 16 keys of every tile; the warps' partial (m, l, o) are merged
//    in warp order.  When a sequence has more than one split the blocks' partials go to scratch
//    memory, and the block that finishes last for a (sequence, key/value head) merges them in
//    ascending split order (core/src/model/emit.cpp:538-560 "chunk_index_asc",
//    core/src/nn/cuda_elementwise.cu:852-1017).  Tile and split boundaries depend only on
//    key positions and the sequence's own length, so a result does not depend on the batch or
//    on where the pages lie.
//
// Mask: key j is visible to the query at position i when j <= i and (window == 0 or
// i - j < window) (core/src/nn/attention.cpp:66-70).  The scale multiplies the finished dot
// product in float32.  Probabilities are rounded to bfloat16 only as the P.V operand.
#include <math.h>

#include "common.cuh"

#ifndef SB_HD
#define SB_HD 128
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int HD = SB_HD;
constexpr int KT = 64;                 // keys per tile = cache page size
constexpr int LDS = HD + 8;            // shared-memory row stride: an odd number of 16-byte chunks
constexpr int BM = HD <= 128 ? 128 : 64;  // prefill rows per block (16 per warp); registers bound it
constexpr int PREFILL_THREADS = BM / 16 * 32;
constexpr int DEC_WARPS = 4;           // decode: warps per block, 16 keys of every tile each
// decode: pages per split.  256 keys while a sequence is at most LONG_LEN long, 512 beyond: a
// longer split spreads a block's fixed costs over more keys (32,768 keys at batch 8: 110 us
// against 130 us per layer), a shorter one gives short sequences enough blocks (3,072 keys at
// batch 8: 14.9 us against 18.2 us).  It depends on the sequence's own length only.
constexpr int SPLIT_PAGES = 4, LONG_SPLIT_PAGES = 8, LONG_LEN = 4096;
__host__ __device__ constexpr int split_pages_for(int len) { return len > LONG_LEN ? LONG_SPLIT_PAGES : SPLIT_PAGES; }
constexpr int DEC_ROWS = 16;
constexpr float LOG2E = 1.4426950408889634f;

static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size in steps of 16, at most 256");

struct AttnParams {
  const bf16* q;               // [rows, n_q_heads, HD]
  bf16* out;                   // [rows, n_q_heads * HD]
  const int32_t* seq_row0;     // [n_seqs + 1]
  const int32_t* seq_pos0;     // [n_seqs] position of a sequence's first new row
  const int32_t* page_off;     // [n_seqs + 1]
  const int32_t* page_ids;
  const bf16* cache;           // [page][k|v][kv head][KT][HD]
  float* scratch;
  int* counters;               // one per (sequence, key/value head), zero between launches
  int n_q_heads, n_kv_heads, window, n_splits;
  int n_seqs;
  float scale_log2;            // scale * log2(e)
  const char* warm;            // decode: bytes the next kernel will read, asked into L2 (or null)
  size_t warm_bytes;
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
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
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copies one cache page's K and V tiles of a key/value head into shared memory.
__device__ __forceinline__ void load_kv_tile(uint32_t ks, uint32_t vs, const bf16* cache, int page,
                                             int n_kv_heads, int kvh, int tid, int n_threads) {
  const bf16* kbase = cache + (((size_t)page * 2) * n_kv_heads + kvh) * (size_t)(KT * HD);
  const bf16* vbase = kbase + (size_t)n_kv_heads * (KT * HD);
  for (int idx = tid; idx < KT * (HD / 8); idx += n_threads) {
    const int row = idx / (HD / 8), ch = idx % (HD / 8);
    const uint32_t off = (uint32_t)(row * LDS + ch * 8) * 2;
    cp_async16(ks + off, kbase + row * HD + ch * 8, true);
    cp_async16(vs + off, vbase + row * HD + ch * 8, true);
  }
}

// One key tile for a warp's 16 rows: scores, mask, online softmax update, P.V.
// `pos_a`, `pos_b`: positions of the thread's two rows (g and g + 8), -1 for padding rows.
template <int NKEYS>
__device__ __forceinline__ void tile_step(const uint32_t (&qf)[HD / 16][4], uint32_t ks,
                                          uint32_t vs, int key0, int pos_a, int pos_b, int window,
                                          float scale_log2, float (&m)[2], float (&l)[2],
                                          float (&o)[HD / 8][4], int lane) {
  float s[NKEYS / 8][4];
#pragma unroll
  for (int j = 0; j < NKEYS / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[j][i] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
    for (int j = 0; j < NKEYS / 16; ++j) {
      const int row = j * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int col = kk * 16 + ((lane >> 3) & 1) * 8;
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(ks + (uint32_t)(row * LDS + col) * 2, b0, b1, b2, b3);
      mma_bf16(s[2 * j], qf[kk], b0, b1);
      mma_bf16(s[2 * j + 1], qf[kk], b2, b3);
    }
  }
  const int t = lane & 3;
  float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NKEYS / 8; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = key0 + j * 8 + 2 * t + (i & 1);
      const int pos = (i < 2) ? pos_a : pos_b;
      const bool seen = key <= pos && (window == 0 || pos - key < window);
      const float v = seen ? s[j][i] * scale_log2 : -INFINITY;
      s[j][i] = v;
      tmax[i >> 1] = fmaxf(tmax[i >> 1], v);
    }
  }
  float alpha[2], base[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
    tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
    const float m_new = fmaxf(m[r], tmax[r]);
    base[r] = m_new == -INFINITY ? 0.0f : m_new;          // nothing seen yet: exp2(-inf - 0) = 0
    alpha[r] = exp2f(m[r] - base[r]);
    m[r] = m_new;
    l[r] *= alpha[r];
  }
  // most tiles leave every row's maximum where it was: the factors are exactly 1 then
  if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }
  }
#pragma unroll
  for (int j = 0; j < NKEYS / 8; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p = exp2f(s[j][i] - base[i >> 1]);
      s[j][i] = p;
      l[i >> 1] += p;
    }
  }
#pragma unroll
  for (int kk = 0; kk < NKEYS / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dj = 0; dj < HD / 16; ++dj) {
      const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int col = dj * 16 + (lane >> 4) * 8;
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vs + (uint32_t)(row * LDS + col) * 2, b0, b1, b2, b3);
      mma_bf16(o[2 * dj], a, b0, b1);
      mma_bf16(o[2 * dj + 1], a, b2, b3);
    }
  }
}

__device__ __forceinline__ void load_q_frags(uint32_t qs, int warp_row0, int lane,
                                             uint32_t (&qf)[HD / 16][4]) {
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const int row = warp_row0 + (lane & 15), col = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qs + (uint32_t)(row * LDS + col) * 2, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
}

}  // namespace

#if SB_HD == 64 || SB_HD == 128
#define SB_ATTN_TC5 1
#include "attn_tc5.cuh"
#endif

namespace {

// ------------------------------------------------------------------------------- prefill
constexpr int PREFILL_SMEM = (BM + 4 * KT) * LDS * 2;

__global__ void __launch_bounds__(PREFILL_THREADS) attn_prefill_kernel(const AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t qs = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t kv0 = qs + BM * LDS * 2;                     // K0, V0, K1, V1
  sb_pdl_launch();
  sb_pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blockIdx.x = (block of query rows, key/value head), heads fastest and the last rows first:
  // blocks are handed out in this order, so the longest ones of every head start first
  const int b = blockIdx.z, kvh = blockIdx.x % p.n_kv_heads;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int row0 = p.seq_row0[b], n_new = p.seq_row0[b + 1] - row0, pos0 = p.seq_pos0[b];
  const int R = n_new * G;
  const int r_base = (int)(gridDim.x / p.n_kv_heads - 1 - blockIdx.x / p.n_kv_heads) * BM;
  if (r_base >= R) return;
  // positions without pages in the sequence's own list: nothing is read
  if (pos0 < 0 || (pos0 + n_new - 1) / KT >= p.page_off[b + 1] - p.page_off[b]) return;
  const int32_t* pages = p.page_ids + p.page_off[b];

  for (int idx = tid; idx < BM * (HD / 8); idx += PREFILL_THREADS) {
    const int row = idx / (HD / 8), ch = idx % (HD / 8);
    const int r = r_base + row;
    const bool valid = r < R;
    const int t = valid ? r / G : 0, g = valid ? r % G : 0;
    cp_async16(qs + (uint32_t)(row * LDS + ch * 8) * 2,
               p.q + ((size_t)(row0 + t) * p.n_q_heads + kvh * G + g) * HD + ch * 8, valid);
  }
  const int r_last = min(R, r_base + BM) - 1;
  const int p_lo = pos0 + r_base / G, p_hi = pos0 + r_last / G;
  const int tile_lo = (p.window > 0 ? max(0, p_lo - p.window + 1) : 0) / KT, tile_hi = p_hi / KT;
  load_kv_tile(kv0, kv0 + KT * LDS * 2, p.cache, pages[tile_lo], p.n_kv_heads, kvh, tid, PREFILL_THREADS);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  uint32_t qf[HD / 16][4];
  load_q_frags(qs, warp * 16, lane, qf);
  const int ra = r_base + warp * 16 + (lane >> 2), rb = ra + 8;
  const int pos_a = ra < R ? pos0 + ra / G : -1, pos_b = rb < R ? pos0 + rb / G : -1;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    const uint32_t ks = kv0 + stage * 2 * KT * LDS * 2, vs = ks + KT * LDS * 2;
    if (tile < tile_hi) {
      const uint32_t nk = kv0 + (stage ^ 1) * 2 * KT * LDS * 2;
      load_kv_tile(nk, nk + KT * LDS * 2, p.cache, pages[tile + 1], p.n_kv_heads, kvh, tid, PREFILL_THREADS);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    tile_step<KT>(qf, ks, vs, tile * KT, pos_a, pos_b, p.window, p.scale_log2, m, l, o, lane);
    __syncthreads();
  }

  const int t4 = lane & 3;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? rb : ra;
    if (r >= R) continue;
    const float inv = 1.0f / l[half];
    bf16* dst = p.out + ((size_t)(row0 + r / G) * p.n_q_heads + kvh * G + r % G) * HD;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t4) =
          pack_bf16(o[j][half * 2] * inv, o[j][half * 2 + 1] * inv);
  }
}

// -------------------------------------------------------------------------------- decode
// Shared memory: Q [16][LDS] bf16, then two stages of K and V tiles [64][LDS]; after the keys
// are done the tiles' space is reused for the warps' partial outputs.
// K/V tiles in flight or in use.  Two: three blocks fit an SM, and their staggered stalls cover
// each other; three or four stages (two blocks or one per SM) measured 20.6 and 22.8 us
// against 14.9 us per layer at batch 8, 3,072 keys, whatever the split length.  When the whole
// grid is at most a block per SM (one to three sequences of the benchmark model) nothing covers
// a block's stalls but its own loads in flight: then four stages (DEC_STAGES_FEW), which take a
// 256-key split's tiles all at once; with at most two blocks per SM three stages
// (DEC_STAGES_SOME: two such blocks fit an SM).  Inside the decode step of a 7B-sized model:
// batch 1 2.888 to 2.849 ms, batch 2 2.935 to 2.858, batch 4 3.000 to 2.958, batch 5 3.014 to
// 2.972; batch 3 and batch 6, whose grids all but fill the SMs at that rate, unchanged.  The
// tiles are used in the same order whatever the number of stages.
constexpr int DEC_STAGES = 2, DEC_STAGES_SOME = 3, DEC_STAGES_FEW = 4;
constexpr size_t WARM_MAX_CHUNKS = 48;   // most 16 KB prefetches a block issues for the L2 hint
constexpr int decode_smem(int stages) { return (DEC_ROWS + 2 * stages * KT) * LDS * 2; }
constexpr int DECODE_SMEM = decode_smem(DEC_STAGES);
constexpr int PART_STRIDE = HD + 4;    // floats per partial row: o[HD], m, l (rows stay 16-byte aligned)
constexpr bool DECODE_FITS = DECODE_SMEM <= 227 * 1024;
constexpr bool DECODE_FEW_FITS = decode_smem(DEC_STAGES_FEW) <= 227 * 1024;
constexpr bool DECODE_SOME_FITS = 2 * (decode_smem(DEC_STAGES_SOME) + 1024) <= 228 * 1024;   // two blocks per SM
static_assert(DEC_WARPS * 16 == KT, "each warp takes 16 keys of a tile");
static_assert((DEC_WARPS * DEC_ROWS * PART_STRIDE + (DEC_WARPS + 2) * DEC_ROWS) * 4 <= 2 * DEC_STAGES * KT * LDS * 2,
              "partials and weights fit the tiles");

template <int STAGES>
__global__ void __launch_bounds__(DEC_WARPS * 32) attn_decode_kernel(const AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_last;
  const uint32_t qs = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t kv0 = qs + DEC_ROWS * LDS * 2;               // K0, V0, K1, V1
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = p.n_q_heads / p.n_kv_heads;
  // The step's plan (rows, positions, pages) was written before the step's first kernel, and
  // cache pages that lie wholly before the new positions in earlier steps: none of that
  // needs the wait for the kernel before this one, which wrote the query rows and the new
  // positions' keys and values.
  const int row0 = p.seq_row0[b], n_new = p.seq_row0[b + 1] - row0, pos0 = p.seq_pos0[b];
  const int R = n_new * G;
  const int p_hi = pos0 + n_new - 1;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int sp = split_pages_for(p_hi + 1);
  const int split_lo = key_lo / (sp * KT), split_hi = p_hi / (sp * KT);
  // A sequence whose new positions have no pages in its own list (or more splits than the grid
  // was sized for) attends to nothing: its rows are zeros, no other sequence's pages are read,
  // and its merge counter is not touched.
  const int n_own_pages = p.page_off[b + 1] - p.page_off[b];
  if (pos0 < 0 || p_hi / KT >= n_own_pages || split_hi >= p.n_splits) {
    sb_pdl_wait();
    if (split == 0)
      for (int item = tid; item < R * (HD / 4); item += DEC_WARPS * 32) {
        const int row = item / (HD / 4), c = item % (HD / 4);
        const size_t out_row = (size_t)(row0 + row / G) * p.n_q_heads + kvh * G + row % G;
        *reinterpret_cast<uint2*>(p.out + out_row * HD + 4 * c) = make_uint2(0u, 0u);
      }
    return;
  }
  if (split < split_lo || split > split_hi) return;
  const int32_t* pages = p.page_ids + p.page_off[b];
  const int tile_lo = max(split * sp, key_lo / KT);
  const int tile_hi = min(split * sp + sp - 1, p_hi / KT);
  // the split's page ids are read together
  int page_of[LONG_SPLIT_PAGES];
#pragma unroll
  for (int i = 0; i < LONG_SPLIT_PAGES; ++i)
    page_of[i] = tile_lo + i <= tile_hi ? max(pages[tile_lo + i], 0) : 0;   // never an address before the cache
  const bool first_is_old = (tile_lo + 1) * KT <= pos0;
  if (first_is_old)
    load_kv_tile(kv0, kv0 + KT * LDS * 2, p.cache, page_of[0], p.n_kv_heads, kvh, tid, DEC_WARPS * 32);
  sb_pdl_wait();
  if (!first_is_old)
    load_kv_tile(kv0, kv0 + KT * LDS * 2, p.cache, page_of[0], p.n_kv_heads, kvh, tid, DEC_WARPS * 32);
  cp_async_commit();                                  // group: the first tile
  for (int idx = tid; idx < DEC_ROWS * (HD / 8); idx += DEC_WARPS * 32) {
    const int row = idx / (HD / 8), ch = idx % (HD / 8);
    const bool valid = row < R;
    const int t = valid ? row / G : 0, g = valid ? row % G : 0;
    cp_async16(qs + (uint32_t)(row * LDS + ch * 8) * 2,
               p.q + ((size_t)(row0 + t) * p.n_q_heads + kvh * G + g) * HD + ch * 8, valid);
  }
  cp_async_commit();                                  // group: the query rows
#pragma unroll
  for (int i = 1; i < STAGES; ++i) {              // groups: the next tiles
    if (i < LONG_SPLIT_PAGES && tile_lo + i <= tile_hi)
      load_kv_tile(kv0 + i * 2 * KT * LDS * 2, kv0 + (i * 2 + 1) * KT * LDS * 2, p.cache, page_of[i],
                   p.n_kv_heads, kvh, tid, DEC_WARPS * 32);
    cp_async_commit();
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;
  const int ra = lane >> 2, rb = ra + 8;
  const int pos_a = ra < R ? pos0 + ra / G : -1, pos_b = rb < R ? pos0 + rb / G : -1;
  uint32_t qf[HD / 16][4];

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) % STAGES;
    const uint32_t ks = kv0 + stage * 2 * KT * LDS * 2, vs = ks + KT * LDS * 2;
    cp_async_wait<STAGES - 1>();                  // this tile has landed; the next may be in flight
    __syncthreads();
    if (tile == tile_lo) load_q_frags(qs, 0, lane, qf);
    // this warp's 16 keys of the tile
    const uint32_t off = (uint32_t)(warp * 16 * LDS) * 2;
    tile_step<16>(qf, ks + off, vs + off, tile * KT + warp * 16, pos_a, pos_b, p.window, p.scale_log2,
                  m, l, o, lane);
    __syncthreads();                                  // the stage is free: request a later tile into it
    if (tile + STAGES <= tile_hi) {
      int pg = page_of[0];
#pragma unroll
      for (int i = 1; i < LONG_SPLIT_PAGES; ++i)
        if (tile + STAGES - tile_lo == i) pg = page_of[i];
      load_kv_tile(ks, vs, p.cache, pg, p.n_kv_heads, kvh, tid, DEC_WARPS * 32);
    }
    cp_async_commit();
  }
  sb_pdl_launch();                                    // the keys and values have been read
  if (p.warm_bytes && tid == 0)
    // what is left of this kernel (the merges) reads little: every block asks for its share
    // of the bytes the next kernel will stream
    sb_warm_l2(p.warm, p.warm_bytes, ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
               (size_t)gridDim.x * gridDim.y * gridDim.z);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  float* part = reinterpret_cast<float*>(smem + DEC_ROWS * LDS * 2);   // [warp][16][PART_STRIDE]
  float* fac = part + DEC_WARPS * DEC_ROWS * PART_STRIDE;              // [warp][16] weights
  float* row_m = fac + DEC_WARPS * DEC_ROWS;                           // [16] merged maximum
  float* row_l = row_m + DEC_ROWS;                                     // [16] merged sum
  const int t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float* dst = part + ((size_t)warp * DEC_ROWS + (half ? rb : ra)) * PART_STRIDE;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<float2*>(dst + j * 8 + 2 * t4) = make_float2(o[j][half * 2], o[j][half * 2 + 1]);
    if (t4 == 0) {
      dst[HD] = m[half];
      dst[HD + 1] = l[half];
    }
  }
  __syncthreads();
  // merge the warps in warp order: first each row's weights exp2(m_w - max) and its sum,
  if (tid < DEC_ROWS) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w)
      mm = fmaxf(mm, part[((size_t)w * DEC_ROWS + tid) * PART_STRIDE + HD]);
    const float base = mm == -INFINITY ? 0.0f : mm;
    float ll = 0.0f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float* src = part + ((size_t)w * DEC_ROWS + tid) * PART_STRIDE;
      const float f = exp2f(src[HD] - base);
      fac[w * DEC_ROWS + tid] = f;
      ll += src[HD + 1] * f;
    }
    row_m[tid] = mm;
    row_l[tid] = ll;
  }
  __syncthreads();
  // then the outputs, four values of a row per thread
  const bool single = split_lo == split_hi;
  for (int item = tid; item < R * (HD / 4); item += DEC_WARPS * 32) {
    const int row = item / (HD / 4), c = item % (HD / 4);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float4 v = *reinterpret_cast<const float4*>(
          part + ((size_t)w * DEC_ROWS + row) * PART_STRIDE + 4 * c);
      const float f = fac[w * DEC_ROWS + row];
      acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
    }
    const size_t out_row = (size_t)(row0 + row / G) * p.n_q_heads + kvh * G + row % G;
    if (single) {
      const float inv = 1.0f / row_l[row];
      uint2 v;
      v.x = pack_bf16(acc.x * inv, acc.y * inv);
      v.y = pack_bf16(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(p.out + out_row * HD + 4 * c) = v;
    } else {
      // scratch: [row of the batch][query head][split][PART_STRIDE]
      float* dst = p.scratch + (out_row * p.n_splits + split) * PART_STRIDE;
      *reinterpret_cast<float4*>(dst + 4 * c) = acc;
      if (c == 0) {
        dst[HD] = row_m[row];
        dst[HD + 1] = row_l[row];
      }
    }
  }
  if (single) return;

  // The block that finishes last for this (sequence, key/value head) merges its splits in
  // ascending order; the counter is left at zero for the next launch.
  // Release / acquire through the counter: the block's partial results are ordered before
  // thread 0's atomic by the barrier, the atomic releases them device-wide, and the last
  // block's atomic acquires every earlier block's; the barrier after it orders the reads below.
  __syncthreads();
  if (tid == 0) {
    int* counter = p.counters + (size_t)b * p.n_kv_heads + kvh;
    int seen;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;\n" : "=r"(seen) : "l"(counter) : "memory");
    s_last = seen == split_hi - split_lo;
    if (s_last) *counter = 0;
  }
  __syncthreads();
  if (!s_last) return;
  // Final merge.  The splits' (m, l) go to shared memory first, one thread per row turns
  // them into weights exp2(m_s - max) and the row's 1 / sum, and then four values of a row
  // are a weighted sum over the splits whose loads are independent of each other and issued
  // eight at a time (partials come from other blocks: they are read from L2).
  const int ns = split_hi - split_lo + 1;
  float* wgt = part;                               // [row][ns]
  float* den = part + DEC_ROWS * ns;               // [row][ns], then den[row * ns] = 1 / sum
  for (int i = tid; i < R * ns; i += DEC_WARPS * 32) {
    const int row = i / ns, sp = split_lo + i % ns;
    const size_t out_row = (size_t)(row0 + row / G) * p.n_q_heads + kvh * G + row % G;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(
        p.scratch + (out_row * p.n_splits + sp) * PART_STRIDE + HD));
    wgt[i] = ml.x;
    den[i] = ml.y;
  }
  __syncthreads();
  if (tid < R) {
    float mm = -INFINITY;
    for (int i = 0; i < ns; ++i) mm = fmaxf(mm, wgt[tid * ns + i]);
    const float ref = mm == -INFINITY ? 0.0f : mm;
    float sum = 0.0f;
    for (int i = 0; i < ns; ++i) {                 // ascending split order
      const float f = exp2f(wgt[tid * ns + i] - ref);
      sum += den[tid * ns + i] * f;
      wgt[tid * ns + i] = f;
    }
    den[tid * ns] = 1.0f / sum;
  }
  __syncthreads();
  // A thread takes two of the (row, four values) tasks at a time, DEC_WARPS * 32 apart, and
  // issues the loads of both before it adds either: the merge is a chain of rounds of L2
  // latency, and the block that runs it is the last one of its sequence and head.
  constexpr int MT = DEC_WARPS * 32;
  for (int item = tid; item < R * (HD / 4); item += 2 * MT) {
    const bool two = item + MT < R * (HD / 4);
    const int row_a = item / (HD / 4), c_a = item % (HD / 4);
    const int row_b = two ? (item + MT) / (HD / 4) : row_a, c_b = two ? (item + MT) % (HD / 4) : c_a;
    const size_t out_a = (size_t)(row0 + row_a / G) * p.n_q_heads + kvh * G + row_a % G;
    const size_t out_b = (size_t)(row0 + row_b / G) * p.n_q_heads + kvh * G + row_b % G;
    const float* src_a = p.scratch + (out_a * p.n_splits + split_lo) * PART_STRIDE + 4 * c_a;
    const float* src_b = p.scratch + (out_b * p.n_splits + split_lo) * PART_STRIDE + 4 * c_b;
    const float* w_a = wgt + row_a * ns;
    const float* w_b = wgt + row_b * ns;
    float4 acc_a = make_float4(0.0f, 0.0f, 0.0f, 0.0f), acc_b = acc_a;
    for (int i = 0; i < ns; i += 8) {               // ascending split order, eight of each task at a time
      float4 va[8], vb[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = i + u < ns;
        va[u] = in ? __ldcg(reinterpret_cast<const float4*>(src_a + (size_t)(i + u) * PART_STRIDE))
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        vb[u] = in && two ? __ldcg(reinterpret_cast<const float4*>(src_b + (size_t)(i + u) * PART_STRIDE))
                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (i + u >= ns) break;
        const float fa = w_a[i + u], fb = w_b[i + u];
        acc_a.x = fmaf(va[u].x, fa, acc_a.x); acc_a.y = fmaf(va[u].y, fa, acc_a.y);
        acc_a.z = fmaf(va[u].z, fa, acc_a.z); acc_a.w = fmaf(va[u].w, fa, acc_a.w);
        acc_b.x = fmaf(vb[u].x, fb, acc_b.x); acc_b.y = fmaf(vb[u].y, fb, acc_b.y);
        acc_b.z = fmaf(vb[u].z, fb, acc_b.z); acc_b.w = fmaf(vb[u].w, fb, acc_b.w);
      }
    }
    const float inv_a = den[row_a * ns], inv_b = den[row_b * ns];
    uint2 v;
    v.x = pack_bf16(acc_a.x * inv_a, acc_a.y * inv_a);
    v.y = pack_bf16(acc_a.z * inv_a, acc_a.w * inv_a);
    *reinterpret_cast<uint2*>(p.out + out_a * HD + 4 * c_a) = v;
    if (two) {
      v.x = pack_bf16(acc_b.x * inv_b, acc_b.y * inv_b);
      v.y = pack_bf16(acc_b.z * inv_b, acc_b.w * inv_b);
      *reinterpret_cast<uint2*>(p.out + out_b * HD + 4 * c_b) = v;
    }
  }
}


// The final merge stages every split's (m, l) of up to 16 rows in the tiles' shared memory.
constexpr int MAX_MERGE_SPLITS = 4 * LDS;

// Splits the grid needs when no sequence is longer than max_len: short sequences use short splits.
int n_splits_for(int max_len) {
  if (max_len <= LONG_LEN) return (max_len + SPLIT_PAGES * KT - 1) / (SPLIT_PAGES * KT);
  const int most_short = LONG_LEN / (SPLIT_PAGES * KT);
  const int longs = (max_len + LONG_SPLIT_PAGES * KT - 1) / (LONG_SPLIT_PAGES * KT);
  return longs > most_short ? longs : most_short;
}

}  // namespace

#ifdef SB_ATTN_TC5
#include "attn_decode_tma.cuh"
#endif

extern "C" int sb_attention_head_dim() { return HD; }

// Kernels the last sb_attention call of this library launched (1, or 2 when a split merge followed).
static int g_last_launches = 1;
extern "C" int sb_attention_last_launches() { return g_last_launches; }

// Kernel choice: 0 (default) the tensor-memory prefill kernel where it applies and the persistent
// TMA decode kernel where it applies and pays, 1 always the earlier mma.sync kernels, 2 the
// persistent decode kernel whatever the number of splits (tests compare them).
static int g_force_mma = 0;
extern "C" void sb_attention_force_mma(int on) { g_force_mma = on; }

// 0 when no tensor-memory kernel of this library has given up on a wait since the last call,
// else the code of that wait; -1 when this head size has no such kernel.
extern "C" int sb_attention_status() {
#ifdef SB_ATTN_TC5
  return tc5_read_status();
#else
  return -1;
#endif
}

// Bytes of scratch sb_attention needs for a step with these bounds (0 when none is used).
extern "C" size_t sb_attention_scratch_bytes(int n_rows, int n_q_heads, int n_kv_heads, int max_new,
                                             int max_len) {
  const int G = n_q_heads / (n_kv_heads > 0 ? n_kv_heads : 1);
  if (max_new * G > DEC_ROWS || !DECODE_FITS || n_splits_for(max_len) > MAX_MERGE_SPLITS) return 0;
  const int n_splits = n_splits_for(max_len);
  if (n_splits <= 1) return 0;
  return (size_t)n_rows * n_q_heads * n_splits * PART_STRIDE * sizeof(float);
}

// q [rows, heads, HD] and out [rows, heads*HD] bfloat16; cache: one schedule entry's pages,
// bfloat16; max_new / max_len: upper bounds of new rows per sequence and of any sequence's
// length after this step (they size the grid; the true values are read on the device).
// counters: n_counters ints that are zero (the kernel leaves them zero), at least sequences x
// key/value heads of them when scratch is needed.
extern "C" int sb_attention(const void* q, void* out, int n_rows, int n_seqs, int max_new,
                            const int32_t* seq_row0, const int32_t* seq_pos0,
                            const int32_t* page_off, const int32_t* page_ids, int page_size,
                            const void* cache, int n_q_heads, int n_kv_heads, int hd, int window,
                            float scale, void* scratch, size_t scratch_bytes, int* counters,
                            int n_counters, int max_len, int n_pages, int n_sms,
                            const void* warm, size_t warm_bytes, cudaStream_t stream) {
  if (hd != HD) SB_FAIL(SB_ERR_ARG, "sb_attention: built for head size %d, called with %d", HD, hd);
  if (page_size != KT)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention: cache pages of %d keys (needs %d)", page_size, KT);
  if (n_rows <= 0 || n_seqs <= 0 || max_new <= 0 || max_len <= 0 || n_q_heads <= 0 || n_kv_heads <= 0)
    SB_FAIL(SB_ERR_ARG, "sb_attention: rows=%d seqs=%d max_new=%d max_len=%d heads=%d/%d", n_rows,
            n_seqs, max_new, max_len, n_q_heads, n_kv_heads);
  if (n_q_heads % n_kv_heads)
    SB_FAIL(SB_ERR_ARG, "sb_attention: %d query heads are not a multiple of %d key/value heads",
            n_q_heads, n_kv_heads);
  if (n_kv_heads > 65535 || n_seqs > 65535)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention: %d key/value heads, %d sequences", n_kv_heads, n_seqs);
  if ((((uintptr_t)q | (uintptr_t)cache | (uintptr_t)scratch) & 15) || ((uintptr_t)out & 7))
    SB_FAIL(SB_ERR_ARG, "sb_attention: unaligned operands");
  AttnParams p;
  p.warm = (const char*)warm; p.warm_bytes = sb_warm_bytes(warm, warm_bytes);
  p.q = (const bf16*)q; p.out = (bf16*)out;
  p.seq_row0 = seq_row0; p.seq_pos0 = seq_pos0; p.page_off = page_off; p.page_ids = page_ids;
  p.cache = (const bf16*)cache; p.scratch = (float*)scratch; p.counters = counters;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.window = window; p.n_seqs = n_seqs;
  p.scale_log2 = scale * LOG2E;
  const int G = n_q_heads / n_kv_heads;
  static bool configured = false;
  if (!configured) {
    cudaError_t e1 = cudaFuncSetAttribute(attn_prefill_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, PREFILL_SMEM);
    cudaError_t e2 = !DECODE_FITS ? cudaSuccess :
        cudaFuncSetAttribute(attn_decode_kernel<DEC_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DECODE_SMEM);
    if (e2 == cudaSuccess && DECODE_FEW_FITS)
      e2 = cudaFuncSetAttribute(attn_decode_kernel<DEC_STAGES_FEW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                decode_smem(DEC_STAGES_FEW));
    if (e2 == cudaSuccess && DECODE_SOME_FITS)
      e2 = cudaFuncSetAttribute(attn_decode_kernel<DEC_STAGES_SOME>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                decode_smem(DEC_STAGES_SOME));
    if (e1 != cudaSuccess || e2 != cudaSuccess)
      SB_FAIL(SB_ERR_CUDA, "sb_attention: shared memory opt-in failed: %s",
              cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    configured = true;
  }
  if (max_new * G <= DEC_ROWS && DECODE_FITS && n_splits_for(max_len) <= MAX_MERGE_SPLITS) {
    p.n_splits = n_splits_for(max_len);
    const size_t need = sb_attention_scratch_bytes(n_rows, n_q_heads, n_kv_heads, max_new, max_len);
    if (need > scratch_bytes || (need && !scratch))
      SB_FAIL(SB_ERR_ARG, "sb_attention: %zu bytes of scratch needed, %zu given", need, scratch_bytes);
    if (need && (!counters || n_counters < n_seqs * n_kv_heads))
      SB_FAIL(SB_ERR_ARG, "sb_attention: %d zeroed counters needed, %d given", n_seqs * n_kv_heads,
              n_counters);
    // The L2 hint pays only when many SMs share it: a block's share goes through its SM's copy
    // engine, and a few blocks with megabytes each hold the kernel up (a step of one 768-key
    // sequence, 16 blocks: 2.5 us a layer slower than without the hint).
    g_last_launches = 1;
#ifdef SB_ATTN_TC5
    // Head sizes 64 and 128, many splits: persistent blocks that stream the pages with TMA, then
    // the merge of the splits as a kernel of its own.
    const long cache_rows_d = (long)n_pages * 2 * n_kv_heads * KT;
    const long n_items = (long)n_seqs * n_kv_heads * p.n_splits;
    // It pays when there are many splits.  Measured on B200 at 28/4 heads of 128, the kernels
    // alone (this one with its merge kernel): 8 sequences of 3,072 keys 15.7 us the earlier kernel
    // and 15.8 us this one, 16 sequences 27.7 and 25.0 us, 32 sequences 48.8 and 41.5 us, 64
    // sequences 87.6 and 75.2 us; 8 sequences of 32,768 keys 111 and 92 us.  Inside the decode
    // step of a 7B-sized model the earlier kernel's many short blocks overlap the kernels around
    // them better, and the merge kernel is one more launch: 16 sequences around position 6,144
    // (768 splits) 3.94 and 4.23 ms a step, 8 around 12,288 (768) 3.92 and 3.99 ms, 32 around
    // 3,072 (1,536) 4.21 and 4.18 ms, 8 around 24,576 (1,536) 5.09 and 4.93 ms, 64 around 3,072
    // (3,072) 5.93 and 5.68 ms.  So from ten blocks' worth of splits per SM on.  Launched without
    // programmatic dependent launch: its blocks fill every SM's shared memory, and starting them
    // early cost 0.02 to 0.06 ms a step at 32 and 64 sequences.
    static bool dt_misaligned = false;
    if (g_force_mma != 1 && !dt_misaligned && n_pages > 0 && n_sms > 0 && cache_rows_d < 2147483647L &&
        n_items < 2147483647L && (n_items > 10L * n_sms || g_force_mma == 2) && (size_t)(2 * p.n_splits + 3 + DT_MERGE_PARTS * HD) * sizeof(float) <= 48 * 1024 &&
        n_seqs <= 65535 && max_new * G <= 65535) {
      static bool configured_dt = false;
      if (!configured_dt) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM);
        if (e == cudaSuccess)                          // all of the SM's memory as shared memory: three blocks fit
          e = cudaFuncSetAttribute(attn_decode_tma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess)
          SB_FAIL(SB_ERR_CUDA, "sb_attention: shared memory opt-in failed: %s", cudaGetErrorString(e));
        configured_dt = true;
      }
      CUtensorMap map_kv;
      if (!t5_make_map(&map_kv, cache, cache_rows_d))
        SB_FAIL(SB_ERR_CUDA, "sb_attention: cuTensorMapEncodeTiled failed");
      const long slots = (long)n_sms * DT_BLOCKS_PER_SM;
      const int blocks = (int)(n_items < slots ? n_items : slots);
      if ((size_t)blocks * WARM_MAX_CHUNKS * SB_WARM_CHUNK < p.warm_bytes) p.warm_bytes = 0;
      sb_launch<0>(attn_decode_tma_kernel, dim3(blocks), dim3(DT_THREADS), DT_SMEM, stream, map_kv, p,
                   (int)n_items);
      SB_CHECK_LAUNCH("sb_attention (decode, TMA)");
      // Once: the kernel's tiles need shared memory that starts on a 1024-byte boundary, which it
      // checks itself (status 10, nothing computed).  Should that ever be reported, this step and
      // all later ones run on the earlier kernel.
      static bool dt_checked = false;
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      if (!dt_checked && cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) {
        if (cudaStreamSynchronize(stream) != cudaSuccess)
          SB_FAIL(SB_ERR_CUDA, "sb_attention: the persistent decode kernel failed");
        dt_checked = true;
        const int st = tc5_read_status();
        if (st == 10) dt_misaligned = true;
        else if (st != 0) SB_FAIL(SB_ERR_CUDA, "sb_attention: a wait in the decode kernel gave up (code %d)", st);
      }
      if (!dt_misaligned && p.n_splits > 1) {
        sb_launch<SB_K_ATTENTION>(attn_merge_kernel, dim3(n_kv_heads, n_seqs, max_new * G), dim3(DT_MERGE_THREADS),
                                  (size_t)(2 * p.n_splits + 3 + DT_MERGE_PARTS * HD) * sizeof(float), stream, p);
        SB_CHECK_LAUNCH("sb_attention (split merge)");
        g_last_launches = 2;
      }
      if (!dt_misaligned) return SB_OK;
    }
#endif
    if ((size_t)p.n_splits * n_kv_heads * n_seqs * WARM_MAX_CHUNKS * SB_WARM_CHUNK < p.warm_bytes)
      p.warm_bytes = 0;
    if (DECODE_FEW_FITS && n_sms > 0 && (long)p.n_splits * n_kv_heads * n_seqs <= n_sms)
      sb_launch<SB_K_ATTENTION>(attn_decode_kernel<DEC_STAGES_FEW>, dim3(p.n_splits, n_kv_heads, n_seqs),
                                dim3(DEC_WARPS * 32), decode_smem(DEC_STAGES_FEW), stream, p);
    else if (DECODE_SOME_FITS && n_sms > 0 && (long)p.n_splits * n_kv_heads * n_seqs <= 2L * n_sms)
      sb_launch<SB_K_ATTENTION>(attn_decode_kernel<DEC_STAGES_SOME>, dim3(p.n_splits, n_kv_heads, n_seqs),
                                dim3(DEC_WARPS * 32), decode_smem(DEC_STAGES_SOME), stream, p);
    else
      sb_launch<SB_K_ATTENTION>(attn_decode_kernel<DEC_STAGES>, dim3(p.n_splits, n_kv_heads, n_seqs),
                                dim3(DEC_WARPS * 32), DECODE_SMEM, stream, p);
    SB_CHECK_LAUNCH("sb_attention (decode)");
    return SB_OK;
  }
  p.n_splits = 1;
  g_last_launches = 1;
#ifdef SB_ATTN_TC5
  // tensor-memory kernel: needs the extent of the cache entry for its tensor map, row
  // coordinates that fit an int, and a positive scale (it takes the maximum before scaling)
  const long cache_rows = (long)n_pages * 2 * n_kv_heads * KT;
  static bool tc5_checked = false, tc5_misaligned = false;
  if (n_pages > 0 && cache_rows < 2147483647L && scale > 0.0f && g_force_mma != 1 && !tc5_misaligned) {
    static bool configured5 = false;
    if (!configured5) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, T5_SMEM);
      if (e != cudaSuccess)
        SB_FAIL(SB_ERR_CUDA, "sb_attention: shared memory opt-in failed: %s", cudaGetErrorString(e));
      configured5 = true;
    }
    CUtensorMap map_kv;
    if (!t5_make_map(&map_kv, cache, cache_rows))
      SB_FAIL(SB_ERR_CUDA, "sb_attention: cuTensorMapEncodeTiled failed");
    const long tiles5 = ((long)max_new * G + T5_QT * T5_ROWS - 1) / (T5_QT * T5_ROWS);
    if (tiles5 * n_kv_heads > 2147483647L) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention: too many rows");
    sb_launch<SB_K_ATTENTION>(attn_prefill_tc5_kernel, dim3((unsigned)(tiles5 * n_kv_heads), 1, n_seqs),
              dim3(T5_THREADS), T5_SMEM, stream, map_kv, p);
    SB_CHECK_LAUNCH("sb_attention (prefill, tcgen05)");
    if (tc5_checked) return SB_OK;
    // Once: the kernel's tiles need shared memory that starts on a 1024-byte boundary, which it
    // checks itself (status 10, nothing computed).  Should that ever be reported, this step and
    // all later ones run on the mma.sync kernel.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
      return SB_OK;
    if (cudaStreamSynchronize(stream) != cudaSuccess)
      SB_FAIL(SB_ERR_CUDA, "sb_attention: the tensor-memory prefill kernel failed");
    tc5_checked = true;
    const int st = tc5_read_status();
    if (st == 0) return SB_OK;
    if (st != 10) SB_FAIL(SB_ERR_CUDA, "sb_attention: a wait in the tensor-memory kernel gave up (code %d)", st);
    tc5_misaligned = true;
  }
#endif
  const long tiles = ((long)max_new * G + BM - 1) / BM;
  if (tiles * n_kv_heads > 2147483647L) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention: too many rows");
  sb_launch<SB_K_ATTENTION>(attn_prefill_kernel, dim3((unsigned)(tiles * n_kv_heads), 1, n_seqs),
                            dim3(PREFILL_THREADS), PREFILL_SMEM, stream, p);
  SB_CHECK_LAUNCH("sb_attention (prefill)");
  return SB_OK;
}

// ------------------------------------------------------------------- no-allocation variant
// See no_alloc.h: the split decode attention with its scratch in a fixed device array.
#include "no_alloc.h"

namespace {

// In host code this name is only a handle for the runtime; it is not a device address.  The
// address the kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[SB_STATIC_SCRATCH_BYTES];
// Arrival counters of the split merge, one per (sequence, key/value head); zero at load and
// left at zero by every launch.
constexpr int STATIC_COUNTERS = 16384;
static __device__ int g_static_counters[STATIC_COUNTERS];

constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {};     // per device, filled at that device's first call
int* g_static_counters_ptr[MAX_DEVICES] = {};

}  // namespace

extern "C" size_t sb_attention_static_scratch_bytes(void) { return SB_STATIC_SCRATCH_BYTES; }

extern "C" int sb_attention_decode_static(const void* q, void* out, int n_rows, int n_seqs,
                                          int max_new, const int32_t* seq_row0,
                                          const int32_t* seq_pos0, const int32_t* page_off,
                                          const int32_t* page_ids, int page_size, const void* cache,
                                          int n_q_heads, int n_kv_heads, int hd, int window,
                                          float scale, int max_len, cudaStream_t stream) {
  const char* who = "sb_attention_decode_static";
  if (hd != HD) SB_FAIL(SB_ERR_ARG, "%s: built for head size %d, called with %d", who, HD, hd);
  if (page_size != KT)
    SB_FAIL(SB_ERR_UNSUPPORTED, "%s: cache pages of %d keys (needs %d)", who, page_size, KT);
  if (n_rows <= 0 || n_seqs <= 0 || max_new <= 0 || max_len <= 0 || n_q_heads <= 0 ||
      n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    SB_FAIL(SB_ERR_ARG, "%s: rows=%d seqs=%d max_new=%d max_len=%d heads=%d/%d", who, n_rows, n_seqs,
            max_new, max_len, n_q_heads, n_kv_heads);
  if (n_kv_heads > 65535 || n_seqs > 65535 || n_q_heads > 65535)
    SB_FAIL(SB_ERR_UNSUPPORTED, "%s: %d/%d heads, %d sequences", who, n_q_heads, n_kv_heads, n_seqs);
  if ((((uintptr_t)q | (uintptr_t)cache) & 15) || ((uintptr_t)out & 7))
    SB_FAIL(SB_ERR_ARG, "%s: unaligned operands", who);
  const int G = n_q_heads / n_kv_heads;
  if (max_new * G > DEC_ROWS || !DECODE_FITS || n_splits_for(max_len) > MAX_MERGE_SPLITS)
    SB_FAIL(SB_ERR_UNSUPPORTED,
            "%s: decode steps only (%d new rows x %d heads per group is above %d rows, the head "
            "size is too large for the decode kernel, or max_len %d is above %d splits)", who,
            max_new, G, DEC_ROWS, max_len, MAX_MERGE_SPLITS);
  const int n_splits = n_splits_for(max_len);
  const size_t need = (size_t)n_rows * n_q_heads * n_splits * PART_STRIDE * sizeof(float);
  if ((long)n_seqs * n_kv_heads > STATIC_COUNTERS)
    SB_FAIL(SB_ERR_UNSUPPORTED, "%s: %d sequences x %d key/value heads is above the %d built-in "
            "merge counters", who, n_seqs, n_kv_heads, STATIC_COUNTERS);
  if (need > SB_STATIC_SCRATCH_BYTES)
    SB_FAIL(SB_ERR_UNSUPPORTED,
            "%s: this step needs %zu bytes of scratch, the built-in array holds %u "
            "(rows %d x heads %d x splits %d x %d floats)", who, need, SB_STATIC_SCRATCH_BYTES,
            n_rows, n_q_heads, n_splits, PART_STRIDE);

  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES)
    SB_FAIL(SB_ERR_CUDA, "%s: cudaGetDevice: %s (device %d)", who, cudaGetErrorString(e), device);
  if (!g_static_scratch_ptr[device]) {
    // set-up, once per device, with that device current
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr)
      SB_FAIL(SB_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
    e = cudaFuncSetAttribute(attn_decode_kernel<DEC_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DECODE_SMEM);
    if (e != cudaSuccess)
      SB_FAIL(SB_ERR_CUDA, "%s: shared memory opt-in failed: %s", who, cudaGetErrorString(e));
    void* cptr = nullptr;
    e = cudaGetSymbolAddress(&cptr, g_static_counters);
    if (e != cudaSuccess || !cptr)
      SB_FAIL(SB_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
    g_static_counters_ptr[device] = (int*)cptr;
    g_static_scratch_ptr[device] = (float*)ptr;
  }

  AttnParams p;
  p.warm = nullptr; p.warm_bytes = 0;
  p.q = (const bf16*)q; p.out = (bf16*)out;
  p.seq_row0 = seq_row0; p.seq_pos0 = seq_pos0; p.page_off = page_off; p.page_ids = page_ids;
  p.cache = (const bf16*)cache; p.scratch = g_static_scratch_ptr[device];
  p.counters = g_static_counters_ptr[device];
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.window = window; p.n_splits = n_splits;
  p.n_seqs = n_seqs;
  p.scale_log2 = scale * LOG2E;
  sb_launch<SB_K_ATTENTION>(attn_decode_kernel<DEC_STAGES>, dim3(n_splits, n_kv_heads, n_seqs), dim3(DEC_WARPS * 32), DECODE_SMEM,
            stream, p);
  SB_CHECK_LAUNCH("sb_attention_decode_static (decode)");
  return SB_OK;
}
