// Decode attention as persistent blocks, three per SM, for head sizes 64 and 128.  Included by
// attn_mma.cu after its decode kernel: the same rows, mask, splits, scratch layout and split
// merge order, so a sequence's result still depends on nothing but its own keys and length.
//
// The earlier kernel gives every (sequence, key/value head, split) a block of its own; a block
// lives for four key tiles, and its set-up (plan and page-table reads, the query rows), its
// first load's latency and its merge are hidden only by the two other blocks of the SM.  Here
// the splits are work items that the blocks walk (block i takes items i, i + grid, ...):
//   warp 4      producer, one thread.  For each of the block's items it works out what the
//               item is (sequence, head, tiles, rows), puts that record and the item's query
//               rows (cp.async.bulk) into a small queue in shared memory, and brings the
//               item's K and V pages in with TMA (cp.async.bulk.tensor boxes of 64 keys x 64
//               values from the tensor map over the cache entry's pages, 128-byte swizzle) into
//               a ring of stages.  It runs ahead across item boundaries, so neither the page
//               stream nor the consumers wait for an item's set-up.
//   warps 0-3   consumers.  The ring's tiles alternate between the warp pairs (0,1) and (2,3);
//               within a pair each warp takes 32 of the tile's 64 keys (mma.sync m16n8k16,
//               operands read with ldmatrix from the swizzled tile; the running output is
//               rescaled only when a row's maximum moved).  A warp waits for a stage's "full"
//               barrier and arrives on its "empty" barrier; the warps meet only for the merge.
// Merge of an item: the stage of the item's last tile is kept a little longer and serves as
// the merge area (the four warps' partial outputs are exactly one stage); the warps are merged
// in warp order, and the split's partial goes to scratch (or the finished rows out when the
// sequence has one split).  The splits of a sequence are merged, in ascending order as before,
// by a small kernel of its own after this one (attn_merge_kernel).  Handing the partials over
// inside this kernel, through an arrival counter as in attn_decode_kernel, takes a device-wide
// release/acquire atomic per item, and every form of it that was tried cost more than the
// merge kernel's launch (measured at 64 sequences of 3,072 keys, per launch, against 70 us for
// the walk alone plus 3 us for the merge kernel: the arrival by a thread of the first warp pair
// 140 us, by a thread of the second pair, which waits for its next tile then anyway, 118 us; by
// a second thread of the producer warp, which holds up the producer, 129 us; for all of a
// block's items at the end of its walk, which puts most merges on the blocks that finish last,
// 108 us).
//
// Every wait on an mbarrier is bounded (tc5.cuh); after the first wait that gives up the block
// stops loading and computing, keeps walking its items so that every barrier is still reached,
// writes nothing more, and the status word tells the host.
#pragma once

#include "tc5.cuh"

namespace {

constexpr int DT_SUB = HD / 64;                              // 64-value pieces of a head
constexpr uint32_t DT_TILE_BYTES = DT_SUB * KT * 128;        // one K or one V page of a head
constexpr uint32_t DT_STAGE_BYTES = 2 * DT_TILE_BYTES;       // K, then V
constexpr int DT_STAGES = HD == 128 ? 2 : 4;
constexpr int DT_BLOCKS_PER_SM = 3;
constexpr int DT_WARPS = 4;                                  // consumer warps: two pairs
constexpr int DT_CONSUMERS = DT_WARPS * 32;
constexpr int DT_THREADS = DT_CONSUMERS + 32;
constexpr int DT_QUEUE = 2;                                  // items whose records and query rows are queued
constexpr uint32_t DT_Q_ROW = HD * 2 + 16;                   // a query row and 16 bytes: rows fall into different banks
constexpr uint32_t DT_Q_BYTES = DEC_ROWS * DT_Q_ROW;         // an item's query rows
static_assert(DT_WARPS * DEC_ROWS * HD * 4 == DT_STAGE_BYTES, "the warps' partial outputs fill one stage");
// after the ring: the queue's query rows and records; per-warp (m, l) of 16 rows; barriers
constexpr uint32_t DT_REC_INTS = 12;
constexpr uint32_t DT_FLAGS = 4;                             // two flags of the kernel, padded to 16 bytes
constexpr uint32_t DT_SMALL_BYTES = 2 * DT_WARPS * DEC_ROWS * 4;
// ... and the record the consumers are on with two flags.  No statically allocated shared memory
// and no slack for aligning by hand: the ring starts the block's shared memory, which is where
// the 1024-byte boundary is (checked in the kernel), so that three blocks fit an SM's 228 KB in
// the 1 KB units it is handed out in.
constexpr uint32_t DT_SMEM = DT_STAGES * DT_STAGE_BYTES + DT_QUEUE * (DT_Q_BYTES + DT_REC_INTS * 4) +
                             DT_SMALL_BYTES + (DT_REC_INTS + DT_FLAGS) * 4 + 8 * (2 * DT_STAGES + 2 * DT_QUEUE);
static_assert(DT_BLOCKS_PER_SM * ((DT_SMEM + 1023) / 1024 + 1) <= 228, "three blocks per SM");

// Place of four consecutive values (c = 0 ... HD/4-1) of `row` of warp `w` in the merge area:
// rows are HD floats apart, so groups of eight values are exchanged by the row's low bits to
// spread the rows over the banks.
__device__ __forceinline__ int dt_part_at(int w, int row, int c) {
  return (w * DEC_ROWS + row) * HD + ((((c >> 1) ^ (row & 7)) << 3) | ((c & 1) << 2));
}

__device__ __forceinline__ void dt_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Address of 16-byte chunk `chunk` (0..HD/8-1) of row `row` in a page tile with the 128-byte
// swizzle: pieces of 64 values, rows of 128 bytes, chunk index xor (row mod 8).
__device__ __forceinline__ uint32_t dt_addr(uint32_t tile, int row, int chunk) {
  return tile + (uint32_t)(chunk >> 3) * (KT * 128) + (uint32_t)row * 128 +
         (uint32_t)(((chunk & 7) ^ (row & 7)) << 4);
}

// One warp's 32 keys (rows key_row0 ... + 31 of the tile) for its 16 query rows.
__device__ __forceinline__ void dt_tile_step(uint32_t qs, uint32_t ks, uint32_t vs,
                                             int key_row0, int key0, int pos_a, int pos_b, int window,
                                             float scale_log2, float (&m)[2], float (&l)[2],
                                             float (&o)[HD / 8][4], int lane) {
  float s[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[j][i] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    // the query rows stay in shared memory (registers are what bounds the blocks per SM)
    uint32_t qf[4];
    ldmatrix_x4(qs + (uint32_t)(lane & 15) * DT_Q_ROW + (uint32_t)(kk * 16 + (lane >> 4) * 8) * 2, qf[0], qf[1],
                qf[2], qf[3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = key_row0 + h * 16 + (lane & 7) + ((lane >> 4) << 3);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(dt_addr(ks, row, kk * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
      mma_bf16(s[2 * h], qf, b0, b1);
      mma_bf16(s[2 * h + 1], qf, b2, b3);
    }
  }
  const int t = lane & 3;
  float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
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
    base[r] = m_new == -INFINITY ? 0.0f : m_new;
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
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p = exp2f(s[j][i] - base[i >> 1]);
      s[j][i] = p;
      l[i >> 1] += p;
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * h][0], s[2 * h][1]);
    a[1] = pack_bf16(s[2 * h][2], s[2 * h][3]);
    a[2] = pack_bf16(s[2 * h + 1][0], s[2 * h + 1][1]);
    a[3] = pack_bf16(s[2 * h + 1][2], s[2 * h + 1][3]);
#pragma unroll
    for (int dj = 0; dj < HD / 16; ++dj) {
      const int row = key_row0 + h * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(dt_addr(vs, row, dj * 2 + (lane >> 4)), b0, b1, b2, b3);
      mma_bf16(o[2 * dj], a, b0, b1);
      mma_bf16(o[2 * dj + 1], a, b2, b3);
    }
  }
}

__device__ __forceinline__ void dt_bar_sync(int id, int n) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(n) : "memory");
}
__device__ __forceinline__ void dt_bar_arrive(int id, int n) {
  asm volatile("bar.arrive %0, %1;\n" ::"r"(id), "r"(n) : "memory");
}

// What every role works out for an item, the same way.
struct DtItem {
  int b, kvh, split;
  int row0, R, pos0, p_hi, split_lo, split_hi, tile_lo, n_tiles;
};
__device__ __forceinline__ bool dt_item(const AttnParams& p, int item, DtItem& it) {
  it.split = item % p.n_splits;
  const int bh = item / p.n_splits;
  it.kvh = bh % p.n_kv_heads;
  it.b = bh / p.n_kv_heads;
  const int G = p.n_q_heads / p.n_kv_heads;
  it.row0 = p.seq_row0[it.b];
  const int n_new = p.seq_row0[it.b + 1] - it.row0;
  it.pos0 = p.seq_pos0[it.b];
  it.R = n_new * G;
  it.p_hi = it.pos0 + n_new - 1;
  const int key_lo = p.window > 0 ? max(0, it.pos0 - p.window + 1) : 0;
  const int sp = split_pages_for(it.p_hi + 1);
  it.split_lo = key_lo / (sp * KT);
  it.split_hi = it.p_hi / (sp * KT);
  const int n_own_pages = p.page_off[it.b + 1] - p.page_off[it.b];
  // positions without pages in the sequence's own list: nothing is read (see attn_decode_kernel)
  if (it.pos0 < 0 || n_new <= 0 || it.p_hi / KT >= n_own_pages || it.split_hi >= p.n_splits) {
    it.n_tiles = -1;
    return false;
  }
  if (it.split < it.split_lo || it.split > it.split_hi) {
    it.n_tiles = 0;
    return false;
  }
  it.tile_lo = max(it.split * sp, key_lo / KT);
  it.n_tiles = min(it.split * sp + sp - 1, it.p_hi / KT) - it.tile_lo + 1;
  return true;
}

// Merges the splits of every (sequence, key/value head) that has more than one.  One block per
// (key/value head, sequence, query row): the first warp turns the splits' (m, l) into weights
// exp2(m_s - max) and the row's 1 / sum; then the splits are shared out over four groups of
// threads, each of which adds its stretch in ascending order (four values of the row per thread,
// loads independent of each other and issued eight at a time), and the four sums are added in
// group order.  How the splits are shared out depends on their number alone, that is on the
// sequence's own length.  With one block per (head, sequence) and one thread per four values,
// eight sequences of 32,768 keys took 18 us here (32 blocks, 64 splits one after the other).
// Dynamic shared memory: (2 * n_splits + 3 + 4 * head size) floats.
constexpr int DT_MERGE_PARTS = 4;
constexpr int DT_MERGE_THREADS = (HD / 4) * DT_MERGE_PARTS;
static_assert(DT_MERGE_THREADS >= 32 && DT_MERGE_THREADS % 32 == 0, "whole warps");
__global__ void __launch_bounds__(DT_MERGE_THREADS) attn_merge_kernel(const AttnParams p) {
  extern __shared__ __align__(16) float mg_smem[];
  __shared__ float inv_sum;
  sb_pdl_launch();
  const int tid = threadIdx.x;
  const int kvh = blockIdx.x, b = blockIdx.y, row = blockIdx.z;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int row0 = p.seq_row0[b], n_new = p.seq_row0[b + 1] - row0, pos0 = p.seq_pos0[b];
  const int R = n_new * G, p_hi = pos0 + n_new - 1;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int sp = split_pages_for(p_hi + 1);
  const int split_lo = key_lo / (sp * KT), split_hi = p_hi / (sp * KT);
  // one split, or a sequence the attention kernel gave rows of zeros: nothing to merge
  if (row >= R || pos0 < 0 || n_new <= 0 || p_hi / KT >= p.page_off[b + 1] - p.page_off[b] ||
      split_hi >= p.n_splits || split_lo == split_hi)
    return;
  sb_pdl_wait();
  const int ns = split_hi - split_lo + 1;
  float* wgt = mg_smem;                            // [ns]
  float* den = mg_smem + p.n_splits;               // [ns]
  float* part = mg_smem + ((2 * p.n_splits + 3) & ~3);   // [group][HD], 16-byte aligned
  const size_t out_row = (size_t)(row0 + row / G) * p.n_q_heads + kvh * G + row % G;
  const float* src0 = p.scratch + (out_row * p.n_splits + split_lo) * PART_STRIDE;
  if (tid < 32) {
    float mm = -INFINITY;
    for (int i = tid; i < ns; i += 32) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(src0 + (size_t)i * PART_STRIDE + HD));
      wgt[i] = ml.x;
      den[i] = ml.y;
      mm = fmaxf(mm, ml.x);
    }
    mm = sb_warp_max(mm);
    const float ref = mm == -INFINITY ? 0.0f : mm;
    float sum = 0.0f;
    for (int i = tid; i < ns; i += 32) {           // each lane its splits in ascending order
      const float f = exp2f(wgt[i] - ref);
      sum += den[i] * f;
      wgt[i] = f;
    }
    sum = sb_warp_sum(sum);                        // then a fixed tree over the lanes
    if (tid == 0) inv_sum = 1.0f / sum;
  }
  __syncthreads();
  const int c = tid % (HD / 4), group = tid / (HD / 4);
  const int per = (ns + DT_MERGE_PARTS - 1) / DT_MERGE_PARTS;
  const int k_end = min(ns, (group + 1) * per);
  const float* src = src0 + 4 * c;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  int k = group * per;
  for (; k + 8 <= k_end; k += 8) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      v[u] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(k + u) * PART_STRIDE));
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc.x = fmaf(v[u].x, wgt[k + u], acc.x); acc.y = fmaf(v[u].y, wgt[k + u], acc.y);
      acc.z = fmaf(v[u].z, wgt[k + u], acc.z); acc.w = fmaf(v[u].w, wgt[k + u], acc.w);
    }
  }
  if (k < k_end) {                                  // up to seven left: loaded together as well
    float4 v[7];
#pragma unroll
    for (int u = 0; u < 7; ++u)
      v[u] = k + u < k_end ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(k + u) * PART_STRIDE))
                           : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int u = 0; u < 7; ++u) {
      if (k + u >= k_end) break;
      acc.x = fmaf(v[u].x, wgt[k + u], acc.x); acc.y = fmaf(v[u].y, wgt[k + u], acc.y);
      acc.z = fmaf(v[u].z, wgt[k + u], acc.z); acc.w = fmaf(v[u].w, wgt[k + u], acc.w);
    }
  }
  *reinterpret_cast<float4*>(part + group * HD + 4 * c) = acc;
  __syncthreads();
  if (group == 0) {
#pragma unroll
    for (int g = 1; g < DT_MERGE_PARTS; ++g) {
      const float4 o = *reinterpret_cast<const float4*>(part + g * HD + 4 * c);
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    const float inv = inv_sum;
    uint2 v;
    v.x = pack_bf16(acc.x * inv, acc.y * inv);
    v.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.out + out_row * HD + 4 * c) = v;
  }
}

__global__ void __launch_bounds__(DT_THREADS, DT_BLOCKS_PER_SM)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const AttnParams p, int n_items) {
  extern __shared__ __align__(1024) unsigned char dt_smem[];
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dt_smem);
  unsigned char* ring_ptr = dt_smem;
  if (ring & 1023u) {                      // the swizzled tiles need this alignment
    if (threadIdx.x == 0) atomicCAS(&g_status, 0, 10);
    return;
  }
  unsigned char* q_ptr = ring_ptr + DT_STAGES * DT_STAGE_BYTES;              // [queue][16][HD] bf16
  const uint32_t q_s = ring + DT_STAGES * DT_STAGE_BYTES;
  int* recs = reinterpret_cast<int*>(q_ptr + DT_QUEUE * DT_Q_BYTES);        // [queue][DT_REC_INTS]
  float* warp_m = reinterpret_cast<float*>(recs + DT_QUEUE * DT_REC_INTS);  // [warp][16]
  float* warp_l = warp_m + DT_WARPS * DEC_ROWS;            // [warp][16]
  int* s_cur = reinterpret_cast<int*>(warp_l + DT_WARPS * DEC_ROWS);   // [DT_REC_INTS] the record of the item the consumers are on
  int* flags = s_cur + DT_REC_INTS;
  int& s_ok = flags[0];                    // one view of "nothing gave up" for every consumer thread
  int& s_abort = flags[1];                 // a bounded wait gave up: nothing more is loaded, computed or written
  const uint32_t bars = q_s + DT_QUEUE * (DT_Q_BYTES + DT_REC_INTS * 4) + DT_SMALL_BYTES + (DT_REC_INTS + DT_FLAGS) * 4;
  const uint32_t full0 = bars, empty0 = full0 + 8 * DT_STAGES;
  const uint32_t qfull0 = empty0 + 8 * DT_STAGES, qempty0 = qfull0 + 8 * DT_QUEUE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.n_q_heads / p.n_kv_heads;

  if (tid == 0) {
    for (int s = 0; s < DT_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 2);                    // the two warps that read the stage
    }
    for (int d = 0; d < DT_QUEUE; ++d) {
      mbar_init(qfull0 + 8 * d, 1);
      mbar_init(qempty0 + 8 * d, DT_WARPS);
    }
    for (int i = 0; i < (int)DT_FLAGS; ++i) flags[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();
  volatile int* abort_flag = &s_abort;

  if (warp == DT_WARPS) {
    // ------------------------------------------------------------------ producer (one thread)
    if (lane == 0) {
      bool waited = false;
      uint32_t it = 0, issued = 0, k = 0;
      for (int item = blockIdx.x;; item += gridDim.x) {
        DtItem w;
        const bool end = item >= n_items;              // after the block's last item: the terminator
        if (end) {
          w.n_tiles = -2;                              // the terminator
        } else {
          dt_item(p, item, w);
          if (w.n_tiles == 0) continue;                // the sequence has no keys in this split
        }
        if (*abort_flag) break;
        const int d = k % DT_QUEUE;
        if (k >= (uint32_t)DT_QUEUE && !mbar_wait(qempty0 + 8 * d, ((k / DT_QUEUE) - 1) & 1, 24)) {
          *abort_flag = 1;
          break;
        }
        {
          int* rec = recs + d * DT_REC_INTS;
          rec[0] = w.b; rec[1] = w.kvh; rec[2] = w.split; rec[3] = w.row0; rec[4] = w.R; rec[5] = w.pos0;
          rec[6] = w.p_hi; rec[7] = w.split_lo; rec[8] = w.split_hi; rec[9] = w.tile_lo; rec[10] = w.n_tiles;
        }
        ++k;
        if (w.n_tiles < 0) {                           // nothing to load: the record alone
          mbar_arrive(qfull0 + 8 * d);
          if (end) break;
          continue;
        }
        const int32_t* pages = p.page_ids + p.page_off[w.b] + w.tile_lo;
        int page_of[LONG_SPLIT_PAGES];                 // the item's page ids are read together
#pragma unroll
        for (int i = 0; i < LONG_SPLIT_PAGES; ++i) page_of[i] = i < w.n_tiles ? max(pages[i], 0) : 0;
        bool q_issued = false;
#pragma unroll
        for (int j = 0; j <= LONG_SPLIT_PAGES; ++j) {
          // The query rows, and pages that may hold a new key, were written by the kernel before
          // this one: they wait for it.  Pages that lie wholly before the new positions are from
          // earlier steps; up to a ring of them are requested before that wait.
          const bool fresh = j < w.n_tiles && (w.tile_lo + j + 1) * KT > w.pos0;
          if (!q_issued && (waited || fresh || j >= w.n_tiles || j == DT_STAGES - 1)) {
            if (!waited) {
              sb_pdl_wait();
              waited = true;
            }
            mbar_expect_tx(qfull0 + 8 * d, (uint32_t)w.R * HD * 2);
            for (int r = 0; r < w.R; ++r)              // row r: new token r / G, query head r % G of the group
              dt_bulk_load(q_s + d * DT_Q_BYTES + r * DT_Q_ROW,
                           p.q + ((size_t)(w.row0 + r / G) * p.n_q_heads + (size_t)w.kvh * G + r % G) * HD,
                           HD * 2, qfull0 + 8 * d);
            q_issued = true;
          }
          if (j >= w.n_tiles) break;
          const int s = it % DT_STAGES;
          if (!*abort_flag) {
            if (it >= (uint32_t)DT_STAGES && !mbar_wait(empty0 + 8 * s, ((it / DT_STAGES) - 1) & 1, 21)) {
              *abort_flag = 1;
            } else {
              const uint32_t dst = ring + s * DT_STAGE_BYTES;
              const int krow = ((page_of[j] * 2) * p.n_kv_heads + w.kvh) * KT;
              const int vrow = ((page_of[j] * 2 + 1) * p.n_kv_heads + w.kvh) * KT;
              mbar_expect_tx(full0 + 8 * s, DT_STAGE_BYTES);
#pragma unroll
              for (int sub = 0; sub < DT_SUB; ++sub) {
                tma_load_2d(dst + sub * (KT * 128), &map_kv, sub * 64, krow, full0 + 8 * s);
                tma_load_2d(dst + DT_TILE_BYTES + sub * (KT * 128), &map_kv, sub * 64, vrow, full0 + 8 * s);
              }
              issued = it + 1;
            }
          }
          ++it;
        }
      }
      if (!waited) sb_pdl_wait();
      sb_pdl_launch();                                 // every load of this block is on its way
      if (p.warm_bytes) sb_warm_l2(p.warm, p.warm_bytes, blockIdx.x, gridDim.x);
      // The block's memory must outlive its copies.  A stage whose consumers went on has landed;
      // after a wait that gave up, the copies still in flight are waited for here.
      if (*abort_flag)
        for (uint32_t i = issued > (uint32_t)DT_STAGES ? issued - DT_STAGES : 0; i < issued; ++i)
          mbar_wait(full0 + 8 * (i % DT_STAGES), (i / DT_STAGES) & 1, 22);
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int pair = warp >> 1, half = warp & 1;
    const int ra = lane >> 2, rb = ra + 8, t4 = lane & 3;
    sb_pdl_wait();                                     // nothing is written before the kernel before this one is done
    uint32_t it = 0, k = 0;
    // Thread 0 takes the next record from the queue (or ends the walk: the terminator, a wait
    // that gave up) and everybody reads it after a barrier, so the warps always agree.
    auto fetch = [&]() {
      if (tid == 0) {
        const int d = k % DT_QUEUE;
        if (*abort_flag || !mbar_wait(qfull0 + 8 * d, (k / DT_QUEUE) & 1, 25)) {
          *abort_flag = 1;
          s_cur[10] = -2;
        } else {
#pragma unroll
          for (int i = 0; i < 11; ++i) s_cur[i] = recs[d * DT_REC_INTS + i];
        }
      }
    };
    fetch();
    dt_bar_sync(1, DT_CONSUMERS);
    while (true) {
      DtItem w;
      w.b = s_cur[0]; w.kvh = s_cur[1]; w.split = s_cur[2]; w.row0 = s_cur[3]; w.R = s_cur[4]; w.pos0 = s_cur[5];
      w.p_hi = s_cur[6]; w.split_lo = s_cur[7]; w.split_hi = s_cur[8]; w.tile_lo = s_cur[9]; w.n_tiles = s_cur[10];
      if (w.n_tiles == -2) break;
      const int d = k % DT_QUEUE;
      ++k;
      if (w.n_tiles < 0) {
        // a sequence with nothing to read: its rows are zeros (the block that has its split 0 writes them)
        if (w.split == 0)
          for (int i = tid; i < w.R * (HD / 4); i += DT_CONSUMERS) {
            const int row = i / (HD / 4), c = i % (HD / 4);
            const size_t out_row = (size_t)(w.row0 + row / G) * p.n_q_heads + w.kvh * G + row % G;
            *reinterpret_cast<uint2*>(p.out + out_row * HD + 4 * c) = make_uint2(0u, 0u);
          }
        __syncwarp();
        if (lane == 0) mbar_arrive(qempty0 + 8 * d);
        dt_bar_sync(1, DT_CONSUMERS);                  // everybody has read the record
        fetch();
        dt_bar_sync(1, DT_CONSUMERS);
        continue;
      }
      // the item's query rows are in its queue slot (rows beyond R hold whatever an earlier
      // item left: their results are never written); thread 0 saw the copy complete
      mbar_wait(qfull0 + 8 * d, ((k - 1) / DT_QUEUE) & 1, 26);
      const uint32_t qs = q_s + d * DT_Q_BYTES;
      const int pos_a = ra < w.R ? w.pos0 + ra / G : -1, pos_b = rb < w.R ? w.pos0 + rb / G : -1;
      float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
      float o[HD / 8][4];
#pragma unroll
      for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.0f;
      for (int j = 0; j < w.n_tiles; ++j) {
        const uint32_t t = it + j;
        if ((int)(t & 1) != pair) continue;            // the other pair's tile
        const int s = t % DT_STAGES;
        // the whole warp goes on or nobody does (the MMAs and shuffles below need every lane)
        const int landed = !*abort_flag && mbar_wait(full0 + 8 * s, (t / DT_STAGES) & 1, 23);
        if (!__all_sync(0xffffffffu, landed)) {
          if (lane == 0) *abort_flag = 1;
          continue;
        }
        const uint32_t ks = ring + s * DT_STAGE_BYTES, vs = ks + DT_TILE_BYTES;
        dt_tile_step(qs, ks, vs, half * 32, (w.tile_lo + j) * KT + half * 32, pos_a, pos_b, p.window,
                     p.scale_log2, m, l, o, lane);
        if (j + 1 < w.n_tiles) {                       // the last tile's stage stays for the merge
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
      }
      it += w.n_tiles;
      __syncwarp();
      if (lane == 0) mbar_arrive(qempty0 + 8 * d);     // the query rows are no longer read
      const int s_merge = (it - 1) % DT_STAGES, last_pair = (it - 1) & 1;
      float* part = reinterpret_cast<float*>(ring_ptr + s_merge * DT_STAGE_BYTES);   // [warp][16][HD], see dt_part_at
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      }
      dt_bar_sync(1, DT_CONSUMERS);                    // every warp has read the last tile
      fetch();                                         // the next record, while the merge goes on
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = hf ? rb : ra;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)               // values j*8 + 2*t4, +1: chunk c = 2j + (t4 >> 1)
          *reinterpret_cast<float2*>(part + dt_part_at(warp, row, 2 * j + (t4 >> 1)) + 2 * (t4 & 1)) =
              make_float2(o[j][hf * 2], o[j][hf * 2 + 1]);
        if (t4 == 0) {
          warp_m[warp * DEC_ROWS + row] = m[hf];
          warp_l[warp * DEC_ROWS + row] = l[hf];
        }
      }
      if (tid == 0) s_ok = !*abort_flag;               // one view of "nothing gave up" for everybody
      dt_bar_sync(1, DT_CONSUMERS);
      const bool ok = s_ok != 0;
      const bool single = w.split_lo == w.split_hi;
      // The warps are merged in warp order.  Four values of a row per thread, which works out
      // the row's weights exp2(m_w - max) and its sum itself.
      for (int i = tid; i < w.R * (HD / 4) && ok; i += DT_CONSUMERS) {
        const int row = i / (HD / 4), c = i % (HD / 4);
        float mm = -INFINITY;
#pragma unroll
        for (int q = 0; q < DT_WARPS; ++q) mm = fmaxf(mm, warp_m[q * DEC_ROWS + row]);
        const float base = mm == -INFINITY ? 0.0f : mm;
        float ll = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int q = 0; q < DT_WARPS; ++q) {
          const float f = exp2f(warp_m[q * DEC_ROWS + row] - base);
          ll += warp_l[q * DEC_ROWS + row] * f;
          const float4 v = *reinterpret_cast<const float4*>(part + dt_part_at(q, row, c));
          acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        const size_t out_row = (size_t)(w.row0 + row / G) * p.n_q_heads + w.kvh * G + row % G;
        if (single) {
          const float inv = 1.0f / ll;
          uint2 v;
          v.x = pack_bf16(acc.x * inv, acc.y * inv);
          v.y = pack_bf16(acc.z * inv, acc.w * inv);
          *reinterpret_cast<uint2*>(p.out + out_row * HD + 4 * c) = v;
        } else {
          float* dst = p.scratch + (out_row * p.n_splits + w.split) * PART_STRIDE;
          *reinterpret_cast<float4*>(dst + 4 * c) = acc;
          if (c == 0) {
            dst[HD] = mm;
            dst[HD + 1] = ll;
          }
        }
      }
      // hand the stage back: the merge wrote it with ordinary stores, the next page comes by TMA
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      dt_bar_sync(1, DT_CONSUMERS);
      if (pair == last_pair && lane == 0) mbar_arrive(empty0 + 8 * s_merge);
    }
  }
}

}  // namespace
