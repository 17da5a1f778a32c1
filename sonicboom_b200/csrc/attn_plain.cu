// Plain attention over the paged cache: one block per (row, query head), float32 arithmetic.
// It is the true 32-bit path's attention and, with bfloat16 storage, the kernel the
// tensor-core attention is checked against.
//
// For the query at absolute position i: key j is visible when j <= i and (window == 0 or
// i < j + window); s_j = (q . k_j) * scale with the scale applied after the whole dot;
// out = sum(exp(s_j - m) v_j) / sum(exp(s_j - m)) (core/src/nn/attention.cpp:26-105,
// 121-183).  Keys are taken in chunks whose boundaries are absolute multiples of the chunk
// length and merged in ascending order, as the reference's split decode attention does
// (core/src/model/emit.cpp:538-544, core/src/nn/cuda_elementwise.cu:886-897), so the sum
// depends only on the positions, not on the batch or on where the pages lie.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int CHUNK = 256;
constexpr int THREADS = 128;
constexpr int MAX_HD = 256;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(THREADS)
attn_plain_kernel(const TQ* q, TQ* out, const int32_t* row_seq, const int32_t* row_pos,
                  const int32_t* page_off, const int32_t* page_ids, int page_size,
                  const TC* cache, int n_q_heads, int n_kv_heads,
                  int hd, int window, float scale) {
  __shared__ float qs[MAX_HD];
  __shared__ float scores[CHUNK];
  __shared__ float bcast[2];
  sb_pdl_launch();
  sb_pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = h / (n_q_heads / n_kv_heads);
  const int pos = row_pos[t];
  const int seq = row_seq[t];
  const int32_t* pages = page_ids + page_off[seq];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  // a position without a page in the sequence's own list: the row is zeros, nothing is read
  if (pos < 0 || pos / page_size >= page_off[seq + 1] - page_off[seq]) {
    for (int d = tid; d < hd; d += THREADS)
      out[((size_t)t * n_q_heads + h) * hd + d] = sb_from_f32<TQ>(0.0f);
    return;
  }

  for (int d = tid; d < hd; d += THREADS)
    qs[d] = sb_to_f32<TQ>(q[((size_t)t * n_q_heads + h) * hd + d]);
  __syncthreads();

  float m = -INFINITY, l = 0.0f;
  float acc[MAX_HD / THREADS] = {};

  for (int cs = (lo / CHUNK) * CHUNK; cs <= pos; cs += CHUNK) {
    const int ce = min(cs + CHUNK, pos + 1);                 // keys [cs, ce), visible from lo
    for (int j = cs + warp; j < cs + CHUNK; j += THREADS / 32) {
      float s = -INFINITY;
      if (j >= lo && j < ce) {
        const TC* krow = cache + ((((size_t)pages[j / page_size] * 2) * n_kv_heads + kvh) *
                                      page_size + j % page_size) * hd;
        float dot = 0.0f;
        for (int d = lane; d < hd; d += 32) dot = fmaf(qs[d], sb_to_f32<TC>(krow[d]), dot);
        s = sb_warp_sum(dot) * scale;
      }
      if (lane == 0) scores[j - cs] = s;
    }
    __syncthreads();
    if (warp == 0) {
      float cm = -INFINITY;
      for (int i = lane; i < CHUNK; i += 32) cm = fmaxf(cm, scores[i]);
      cm = sb_warp_max(cm);
      const float m_new = fmaxf(m, cm);
      float sum = 0.0f;
      for (int i = lane; i < CHUNK; i += 32) {
        const float p = scores[i] == -INFINITY ? 0.0f : expf(scores[i] - m_new);
        scores[i] = p;
        sum += p;
      }
      sum = sb_warp_sum(sum);
      if (lane == 0) {
        bcast[0] = m == -INFINITY ? 0.0f : expf(m - m_new);   // rescale of what came before
        bcast[1] = sum;
      }
      m = m_new;
    }
    __syncthreads();
    const float alpha = bcast[0];
    l = l * alpha + bcast[1];
#pragma unroll
    for (int i = 0; i < MAX_HD / THREADS; ++i) acc[i] *= alpha;
    const int j0 = max(cs, lo);
    for (int j = j0; j < ce; ++j) {
      const float p = scores[j - cs];
      const TC* vrow = cache + ((((size_t)pages[j / page_size] * 2 + 1) * n_kv_heads + kvh) *
                                    page_size + j % page_size) * hd;
#pragma unroll
      for (int i = 0; i < MAX_HD / THREADS; ++i) {
        const int d = tid + i * THREADS;
        if (d < hd) acc[i] = fmaf(p, sb_to_f32<TC>(vrow[d]), acc[i]);
      }
    }
    __syncthreads();
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < MAX_HD / THREADS; ++i) {
    const int d = tid + i * THREADS;
    if (d < hd) out[((size_t)t * n_q_heads + h) * hd + d] = sb_from_f32<TQ>(acc[i] * inv);
  }
}

}  // namespace

int sb_check_attention_args(const char* who, int n_rows, int n_q_heads, int n_kv_heads, int hd,
                            int window, int page_size) {
  if (n_rows <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || hd <= 0 || page_size <= 0)
    SB_FAIL(SB_ERR_ARG, "%s: n_rows=%d heads=%d/%d hd=%d page=%d", who, n_rows, n_q_heads,
            n_kv_heads, hd, page_size);
  if (n_q_heads % n_kv_heads)
    SB_FAIL(SB_ERR_ARG, "%s: %d query heads are not a multiple of %d key/value heads", who,
            n_q_heads, n_kv_heads);
  if (window < 0) SB_FAIL(SB_ERR_ARG, "%s: window %d", who, window);
  return SB_OK;
}

extern "C" int sb_attention_plain(const void* q, void* out, int act_dtype, int n_rows,
                                  const int32_t* row_seq, const int32_t* row_pos,
                                  const int32_t* page_off, const int32_t* page_ids, int page_size,
                                  const void* cache, int cache_dtype, int n_q_heads,
                                  int n_kv_heads, int hd, int window, float scale,
                                  cudaStream_t stream) {
  if (int rc = sb_check_attention_args("sb_attention_plain", n_rows, n_q_heads, n_kv_heads, hd,
                                       window, page_size))
    return rc;
  if (hd > MAX_HD)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention_plain: head dim %d is above %d", hd, MAX_HD);
  if (!sb_valid_dtype(act_dtype) || !sb_valid_dtype(cache_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_attention_plain: dtype codes %d %d", act_dtype, cache_dtype);
  if (n_q_heads > 65535) SB_FAIL(SB_ERR_UNSUPPORTED, "sb_attention_plain: %d heads", n_q_heads);
  const dim3 grid(n_rows, n_q_heads);
  SB_DISPATCH_DTYPE(act_dtype, TQ, {
    SB_DISPATCH_DTYPE(cache_dtype, TC, {
      sb_launch(attn_plain_kernel<TQ, TC>, grid, dim3(THREADS), 0, stream,
          (const TQ*)q, (TQ*)out, row_seq, row_pos, page_off, page_ids, page_size,
          (const TC*)cache, n_q_heads, n_kv_heads, hd, window, scale);
    });
  });
  SB_CHECK_LAUNCH("sb_attention_plain");
  return SB_OK;
}
