// Token selection on the device: greedy argmax and the seeded sampler, one block per row.
//
// The order of stages is the reference's (capi/include/sonicboom/capi.h:629-645,
// core/src/nn/sampling.cpp:157-203, 257-352):
//   1. repetition / presence / frequency penalties over the row's history window;
//   2. temperature <= 0: the argmax of the penalized logits, ties toward the lowest id;
//   3. otherwise z = logit / T (one float division); the 256 highest z, ties toward the lower
//      id, in (z descending, id ascending) order;
//   4. candidates more than 30 below the maximum are dropped; top_k; min_p (z < max + ln(min_p)
//      dropped); nucleus (shortest prefix whose normalized mass reaches top_p);
//   5. Gumbel-max draw: u = (bits[0] + 0.5) / 2^32 with bits = Philox4x32-10(counter =
//      {pos_lo, pos_hi, id, 0}, key = seed); the highest z - log(-log u) wins, ties toward the
//      lower id.  `position` is the absolute position of the token being produced, so a
//      sequence's draws do not depend on its row in the batch.
// Penalties are applied to the logits row in place and undone before the kernel returns.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int CANDIDATES = 256;      // core/include/sonicboom/nn/sampling.h:68
constexpr float LOGIT_WINDOW = 30.0f;  // core/include/sonicboom/nn/sampling.h:61
constexpr int MAX_HISTORY = 1024;    // the reference's device penalty window (capi.cpp:2711-2715)

__device__ __forceinline__ uint32_t order_key(float z) {
  // Monotone map float -> uint32 (larger z, larger key); NaN sorts lowest.
  if (z != z) return 0u;
  const uint32_t b = __float_as_uint(z);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint64_t key,
                              uint32_t out[4]) {
  // Random123 constants (core/src/nn/sampling.cpp:207-227).
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Block-wide argmax of (value, lowest id); every thread returns the winner.
__device__ int block_argmax(float v, int id, float* sv, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, id, o);
    if (oi >= 0 && (id < 0 || ov > v || (ov == v && oi < id))) { v = ov; id = oi; }
  }
  if (lane == 0) { sv[warp] = v; si[warp] = id; }
  __syncthreads();
  if (warp == 0) {
    v = lane < (blockDim.x >> 5) ? sv[lane] : 0.0f;
    id = lane < (blockDim.x >> 5) ? si[lane] : -1;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (oi >= 0 && (id < 0 || ov > v || (ov == v && oi < id))) { v = ov; id = oi; }
    }
    if (lane == 0) si[0] = id;
  }
  __syncthreads();
  const int r = si[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(float* logits, int vocab, const SbSampleParams* params, const int32_t* history,
              int history_stride, const int32_t* fed_pos, int32_t* out_tokens) {
  __shared__ int32_t h_tok[MAX_HISTORY];
  __shared__ float h_old[MAX_HISTORY];
  __shared__ uint32_t hist[256];
  __shared__ unsigned long long cand[CANDIDATES];   // (key << 32) | (~id): sorts z desc, id asc
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ uint32_t s_prefix, s_need, s_count, s_running;
  __shared__ int s_keep;

  sb_pdl_launch();
  sb_pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  SbSampleParams p = params[row];
  // with `fed_pos`, the token produced follows the one fed at fed_pos[row] in this step
  if (fed_pos) p.position = (uint64_t)fed_pos[row] + 1u;
  float* lg = logits + (size_t)row * vocab;

  // 1. penalties, in place (undone at the end).  h_tok[i] >= 0 marks a first occurrence.
  const bool penal = p.history_len > 0 && (p.repeat_penalty != 1.0f || p.presence_penalty != 0.0f ||
                                           p.frequency_penalty != 0.0f);
  const int win = penal ? min(p.history_len, MAX_HISTORY) : 0;
  if (penal) {
    const int32_t* hrow = history + (size_t)row * history_stride;
    for (int i = tid; i < win; i += THREADS) {
      const int32_t t = hrow[i];
      int count = 0;
      bool first = true;
      for (int j = 0; j < win; ++j) {
        if (hrow[j] == t) {
          ++count;
          if (j < i) first = false;
        }
      }
      h_tok[i] = -1;
      if (first && t >= 0 && t < vocab) {
        const float old = lg[t];
        float v = old;
        if (p.repeat_penalty != 1.0f)
          v = v > 0.0f ? __fdiv_rn(v, p.repeat_penalty) : __fmul_rn(v, p.repeat_penalty);
        const float adjust = __fmaf_rn(p.frequency_penalty, (float)count, p.presence_penalty);
        h_tok[i] = t;
        h_old[i] = old;
        lg[t] = __fsub_rn(v, adjust);
      }
    }
    __syncthreads();
  }

  int result = -1;
  if (!(p.temperature > 0.0f)) {
    // 2. greedy
    float best = 0.0f;
    int best_i = -1;
    for (int i = tid; i < vocab; i += THREADS) {
      const float v = lg[i];
      if (best_i < 0 || v > best) { best = v; best_i = i; }
    }
    result = block_argmax(best, best_i, red_v, red_i);
  } else {
    // 3. the CANDIDATES highest z: radix select of the threshold key, then collection.
    const float T = p.temperature;
    const uint32_t want = (uint32_t)min(vocab, CANDIDATES);
    if (tid == 0) { s_prefix = 0u; s_need = want; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0u;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < vocab; i += THREADS) {
        const uint32_t k = order_key(__fdiv_rn(lg[i], T));
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        uint32_t need = s_need, b = 255u;
        for (;; --b) {                       // highest digit whose suffix count reaches `need`
          if (hist[b] >= need || b == 0u) break;
          need -= hist[b];
        }
        s_need = need;                       // how many of the ties at this digit are wanted
        s_prefix = prefix | (b << shift);
      }
      __syncthreads();
    }
    const uint32_t kth = s_prefix;           // key of the last candidate
    const uint32_t n_ties = s_need;          // how many ids with exactly that key are taken
    if (tid == 0) { s_count = 0u; s_running = 0u; }
    for (int i = tid; i < CANDIDATES; i += THREADS) cand[i] = 0ull;
    __syncthreads();
    for (int i = tid; i < vocab; i += THREADS) {
      const uint32_t k = order_key(__fdiv_rn(lg[i], T));
      if (k > kth) {
        const uint32_t slot = atomicAdd(&s_count, 1u);
        cand[slot] = ((unsigned long long)k << 32) | (uint32_t)(~(uint32_t)i);
      }
    }
    __syncthreads();
    const uint32_t n_gt = s_count;
    // ties at the threshold key: the lowest ids, found by an ordered scan over the row
    for (int base = 0; base < vocab; base += THREADS) {
      if (s_running >= n_ties) break;
      const int i = base + tid;
      const bool flag = i < vocab && order_key(__fdiv_rn(lg[i], T)) == kth;
      const uint32_t ballot = __ballot_sync(0xffffffffu, flag);
      const int lane = tid & 31, warp = tid >> 5;
      if (lane == 0) hist[warp] = __popc(ballot);
      __syncthreads();
      uint32_t before = s_running;
      for (int w = 0; w < warp; ++w) before += hist[w];
      const uint32_t rank = before + __popc(ballot & ((1u << lane) - 1u));
      if (flag && rank < n_ties)
        cand[n_gt + rank] = ((unsigned long long)kth << 32) | (uint32_t)(~(uint32_t)i);
      __syncthreads();
      if (tid == 0) {
        uint32_t total = 0;
        for (int w = 0; w < THREADS / 32; ++w) total += hist[w];
        s_running += total;
      }
      __syncthreads();
    }
    const int n_cand = (int)want;
    // bitonic sort, descending (empty slots are 0 and sink to the end)
    for (int k = 2; k <= CANDIDATES; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        if (tid < CANDIDATES) {
          const int partner = tid ^ j;
          if (partner > tid) {
            const unsigned long long a = cand[tid], b = cand[partner];
            const bool desc = (tid & k) == 0;
            if (desc ? a < b : a > b) { cand[tid] = b; cand[partner] = a; }
          }
        }
        __syncthreads();
      }
    }
    // 4. filters: each keeps a prefix of the sorted list
    if (tid == 0) {
      auto z_of = [&](int c) { return __fdiv_rn(lg[~(uint32_t)(cand[c] & 0xffffffffull)], T); };
      const float zmax = z_of(0);
      int keep = 0;
      const float floor_z = zmax - LOGIT_WINDOW;
      while (keep < n_cand && z_of(keep) >= floor_z) ++keep;
      if (p.top_k > 0u && (uint32_t)keep > p.top_k) keep = (int)p.top_k;
      if (p.min_p > 0.0f) {
        const float cutoff = zmax + logf(p.min_p);
        int k2 = 0;
        while (k2 < keep && z_of(k2) >= cutoff) ++k2;
        keep = k2;
      }
      if (p.top_p > 0.0f && p.top_p < 1.0f && keep > 0) {
        double total = 0.0;
        for (int c = 0; c < keep; ++c) total += exp((double)z_of(c) - (double)zmax);
        if (total > 0.0) {
          double acc = 0.0;
          int k2 = 0;
          while (k2 < keep) {
            acc += exp((double)z_of(k2) - (double)zmax);
            ++k2;
            if (acc / total >= (double)p.top_p) break;
          }
          keep = k2 < 1 ? 1 : k2;
        }
      }
      s_keep = keep;
    }
    __syncthreads();
    // 5. Gumbel-max over the kept prefix
    const int keep = s_keep;
    double best = 0.0;
    int best_i = -1;
    if (tid < keep) {
      const int id = (int)(~(uint32_t)(cand[tid] & 0xffffffffull));
      const float z = __fdiv_rn(lg[id], T);
      uint32_t bits[4];
      philox4x32_10((uint32_t)p.position, (uint32_t)(p.position >> 32), (uint32_t)id, 0u, p.seed, bits);
      const double u = ((double)bits[0] + 0.5) / 4294967296.0;
      best = (double)z + (-log(-log(u)));
      best_i = id;
    }
    // reduce in double through shared memory (at most CANDIDATES entries)
    __shared__ double g_score[CANDIDATES];
    __shared__ int g_id[CANDIDATES];
    if (tid < CANDIDATES) { g_score[tid] = best; g_id[tid] = best_i; }
    __syncthreads();
    if (tid == 0) {
      int win_id = -1;
      double win_score = 0.0;
      for (int c = 0; c < keep; ++c) {
        if (win_id < 0 || g_score[c] > win_score || (g_score[c] == win_score && g_id[c] < win_id)) {
          win_id = g_id[c];
          win_score = g_score[c];
        }
      }
      red_i[0] = win_id;
    }
    __syncthreads();
    result = red_i[0];
  }

  __syncthreads();
  if (penal) {
    for (int i = tid; i < win; i += THREADS)
      if (h_tok[i] >= 0) lg[h_tok[i]] = h_old[i];
  }
  if (tid == 0) out_tokens[row] = result;
}

__global__ void add_kernel(int32_t* x, int n, int delta) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += delta;
}

// x[i] = min(x[i] + 1, last[i]): a row of a captured decode batch moves to its next position
// but never past the last position it holds pages for; a row that has finished stays there.
__global__ void advance_kernel(int32_t* x, const int32_t* __restrict__ last, int n) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = min(x[i] + 1, last[i]);
}

}  // namespace

extern "C" int sb_advance_rows(int32_t* x, const int32_t* last, int n, cudaStream_t stream) {
  if (n <= 0 || !x || !last) SB_FAIL(SB_ERR_ARG, "sb_advance_rows: n=%d", n);
  sb_launch(advance_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, x, last, n);
  SB_CHECK_LAUNCH("sb_advance_rows");
  return SB_OK;
}

// x[i] += delta: advances the positions of a decode loop that stays on the device.
extern "C" int sb_add_i32(int32_t* x, int n, int delta, cudaStream_t stream) {
  if (n <= 0) SB_FAIL(SB_ERR_ARG, "sb_add_i32: n=%d", n);
  sb_launch(add_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, x, n, delta);
  SB_CHECK_LAUNCH("sb_add_i32");
  return SB_OK;
}

extern "C" int sb_sample_params_size() { return (int)sizeof(SbSampleParams); }

// logits [n_rows, vocab] float32 (penalties touch it in place and restore it); params: one
// SbSampleParams per row in device memory; history [n_rows, history_stride] int32 (may be null
// when no row has history); fed_pos, when given, holds the position of the token each row was
// fed in this step and overrides the records' `position` with fed_pos + 1 (a loop that runs
// on the device advances it there); out_tokens int32 [n_rows].
extern "C" int sb_sample(float* logits, int n_rows, int vocab, const void* params,
                         const int32_t* history, int history_stride, const int32_t* fed_pos,
                         int32_t* out_tokens, cudaStream_t stream) {
  if (n_rows <= 0 || vocab <= 0) SB_FAIL(SB_ERR_ARG, "sb_sample: n_rows=%d vocab=%d", n_rows, vocab);
  if (history_stride < 0 || history_stride > MAX_HISTORY)
    SB_FAIL(SB_ERR_UNSUPPORTED, "sb_sample: a penalty window of %d tokens is above the cap of %d",
            history_stride, MAX_HISTORY);
  sb_launch(sample_kernel, dim3(n_rows), dim3(THREADS), 0, stream, logits, vocab,
            (const SbSampleParams*)params, history, history_stride, fed_pos, out_tokens);
  SB_CHECK_LAUNCH("sb_sample");
  return SB_OK;
}
