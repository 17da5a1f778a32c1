// Embedding gather, RMSNorm, dtype casts and the fused rotation + cache write.
// Each kernel is templated on its storage types; arithmetic is float32 throughout.
#include "common.cuh"

extern "C" int sb_abi_version() { return 1; }

// ------------------------------------------------------------------------------- embedding
// x[t, :] = E[tokens[t], :] * scale as float32.  The scale is the model's (1 for this
// architecture; the reference multiplies by sqrt(width) for the architectures whose trait says
// so: core/src/model/emit.cpp:237-247, core/src/nn/embedding.cpp:23-28); 1 multiplies nothing.
// Inputs that an earlier kernel of the step wrote are plain pointers, not `const __restrict__`:
// with programmatic dependent launch a kernel may start before its predecessor has finished, and
// the non-coherent load path that `const __restrict__` selects could then return stale lines.
// An id outside the table (the sampler's -1 for a row of logits that are not finite, when ids are
// fed back on the device) reads nothing and gives a row of NaN, which stays visible downstream.
template <typename TW>
__global__ void embed_kernel(const int32_t* tokens, const TW* __restrict__ table, int vocab,
                             int width, float scale, float* __restrict__ out) {
  sb_pdl_launch();
  sb_pdl_wait();
  const int t = blockIdx.x;
  const int id = tokens[t];
  float* o = out + (size_t)t * width;
  if ((unsigned)id >= (unsigned)vocab) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
    return;
  }
  const TW* row = table + (size_t)id * width;
  if (scale == 1.0f)
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = sb_to_f32<TW>(row[i]);
  else
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = sb_to_f32<TW>(row[i]) * scale;
}

extern "C" int sb_embed(const int32_t* tokens, int n_rows, const void* table, int table_dtype,
                        int vocab, int width, float scale, float* out, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0 || vocab <= 0)
    SB_FAIL(SB_ERR_ARG, "sb_embed: n_rows=%d vocab=%d width=%d", n_rows, vocab, width);
  if (!sb_valid_dtype(table_dtype)) SB_FAIL(SB_ERR_ARG, "sb_embed: table dtype %d", table_dtype);
  SB_DISPATCH_DTYPE(table_dtype, TW, {
    sb_launch<SB_K_ELEMENTWISE>(embed_kernel<TW>, dim3(n_rows), dim3(256), 0, stream, tokens, (const TW*)table, vocab, width, scale, out);
  });
  SB_CHECK_LAUNCH("sb_embed");
  return SB_OK;
}

// --------------------------------------------------------------------------------- RMSNorm
// inv = 1/sqrt(mean(x^2) + eps); y = (x * inv) * w, plain weight
// (core/src/nn/norm.cpp:25-42, core/src/nn/cuda_elementwise.cu:684-711).  One block per row;
// the sum is a fixed tree (thread-strided partial sums, warp shuffles, then the warps in
// order), so a row's result does not depend on which other rows are in the launch.
// `rows`, when given, gathers: output row r is the norm of input row rows[r].
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* x, const int32_t* rows,
                               const TW* __restrict__ w, int width, float eps,
                               TO* __restrict__ out) {
  __shared__ float warp_sums[32];
  __shared__ float inv_shared;
  sb_pdl_launch();
  sb_pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
  float s = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = xr[i];
    s = fmaf(v, v, s);
  }
  s = sb_warp_sum(s);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  if (lane == 0) warp_sums[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int i = 0; i < n_warps; ++i) total += warp_sums[i];
    inv_shared = 1.0f / sqrtf(total / (float)width + eps);
  }
  __syncthreads();
  const float inv = inv_shared;
  TO* o = out + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = sb_from_f32<TO>((xr[i] * inv) * sb_to_f32<TW>(w[i]));
}

// The same for widths that are multiples of 4 and at most 4096: every thread keeps its part of the
// row in registers (one read of x), with 16-byte loads and stores.
template <typename T>
__device__ __forceinline__ void sb_load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void sb_load4<float>(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
template <>
__device__ __forceinline__ void sb_load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <typename T>
__device__ __forceinline__ void sb_store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void sb_store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void sb_store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

constexpr int NORM_THREADS = 256, NORM_VEC = 4;      // 256 threads x 4 vectors of 4 = 4096 values

template <typename TW, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec_kernel(const float* x, const int32_t* rows, const TW* __restrict__ w, int width,
                   float eps, TO* __restrict__ out) {
  __shared__ float warp_sums[NORM_THREADS / 32];
  __shared__ float inv_shared;
  sb_pdl_launch();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * width;     // `rows` is part of the step's plan
  sb_pdl_wait();
  float v[NORM_VEC][4];
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NORM_VEC; ++i) {
    const int e = (threadIdx.x + i * NORM_THREADS) * 4;
    if (e < width) {
      sb_load4<float>(xr + e, v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) s = fmaf(v[i][j], v[i][j], s);
    }
  }
  s = sb_warp_sum(s);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_sums[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int i = 0; i < NORM_THREADS / 32; ++i) total += warp_sums[i];
    inv_shared = 1.0f / sqrtf(total / (float)width + eps);
  }
  __syncthreads();
  const float inv = inv_shared;
  TO* o = out + (size_t)r * width;
#pragma unroll
  for (int i = 0; i < NORM_VEC; ++i) {
    const int e = (threadIdx.x + i * NORM_THREADS) * 4;
    if (e < width) {
      float wv[4], y[4];
      sb_load4<TW>(w + e, wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = (v[i][j] * inv) * wv[j];
      sb_store4<TO>(o + e, y);
    }
  }
}

extern "C" int sb_rmsnorm(const float* x, const int32_t* rows, int n_rows, int width,
                          const void* weight, int weight_dtype, float eps, void* out,
                          int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) SB_FAIL(SB_ERR_ARG, "sb_rmsnorm: n_rows=%d width=%d", n_rows, width);
  if (!sb_valid_dtype(weight_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_rmsnorm: dtype codes %d %d", weight_dtype, out_dtype);
  if (!(eps >= 0.0f)) SB_FAIL(SB_ERR_ARG, "sb_rmsnorm: eps %g", eps);
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const bool vec = width % 4 == 0 && width <= NORM_THREADS * NORM_VEC * 4 &&
                   (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  SB_DISPATCH_DTYPE(weight_dtype, TW, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      if (vec)
        sb_launch<SB_K_ELEMENTWISE>(rmsnorm_vec_kernel<TW, TO>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, x, rows,
                  (const TW*)weight, width, eps, (TO*)out);
      else
        sb_launch<SB_K_ELEMENTWISE>(rmsnorm_kernel<TW, TO>, dim3(n_rows), dim3(threads), 0, stream, x, rows,
                  (const TW*)weight, width, eps, (TO*)out);
    });
  });
  SB_CHECK_LAUNCH("sb_rmsnorm");
  return SB_OK;
}

// --------------------------------------------------------------------------------- logit cap
// x = cap * tanh(x / cap) in place (core/src/model/emit.cpp:520-522, the reference's Softcap op
// on the logits; core/src/nn/sampling.cpp:229).  Not used by this architecture: a model whose
// spec names a cap gets it here.
__global__ void softcap_kernel(float* x, size_t n, float cap) {
  sb_pdl_launch();
  sb_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int sb_softcap(float* x, size_t n, float cap, cudaStream_t stream) {
  if (!(cap > 0.0f)) SB_FAIL(SB_ERR_ARG, "sb_softcap: cap %g must be positive", cap);
  if (n == 0) return SB_OK;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  sb_launch<SB_K_ELEMENTWISE>(softcap_kernel, dim3(blocks), dim3(256), 0, stream, x, n, cap);
  SB_CHECK_LAUNCH("sb_softcap");
  return SB_OK;
}

// -------------------------------------------------------------------------------- row bias
// x[m, n] += bias[n] in place on float32 rows: the bias of a projection whose product epilogue is
// taken by the residual add (an output projection with a bias; the reference keeps such a bias
// as its own AddBias node, core/src/model/emit.cpp:203-210).
template <typename TB>
__global__ void add_bias_kernel(float* x, const TB* __restrict__ bias, size_t rows, int width) {
  sb_pdl_launch();
  sb_pdl_wait();
  const size_t n = rows * (size_t)width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] += sb_to_f32<TB>(bias[i % width]);
}

extern "C" int sb_add_bias(float* x, const void* bias, int bias_dtype, int rows, int width,
                           cudaStream_t stream) {
  if (rows <= 0 || width <= 0 || !x || !bias) SB_FAIL(SB_ERR_ARG, "sb_add_bias: rows=%d width=%d", rows, width);
  if (!sb_valid_dtype(bias_dtype)) SB_FAIL(SB_ERR_ARG, "sb_add_bias: dtype code %d", bias_dtype);
  const size_t n = (size_t)rows * width;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  SB_DISPATCH_DTYPE(bias_dtype, TB, {
    sb_launch<SB_K_ELEMENTWISE>(add_bias_kernel<TB>, dim3(blocks), dim3(256), 0, stream, x, (const TB*)bias,
                                (size_t)rows, width);
  });
  SB_CHECK_LAUNCH("sb_add_bias");
  return SB_OK;
}

// ------------------------------------------------------------------------------------ cast
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* in, TO* out, size_t n) {
  sb_pdl_launch();
  sb_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = sb_from_f32<TO>(sb_to_f32<TI>(in[i]));
}

extern "C" int sb_cast(const void* in, int in_dtype, void* out, int out_dtype, size_t n,
                       cudaStream_t stream) {
  if (!sb_valid_dtype(in_dtype) || !sb_valid_dtype(out_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_cast: dtype codes %d %d", in_dtype, out_dtype);
  if (n == 0) return SB_OK;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  SB_DISPATCH_DTYPE(in_dtype, TI, {
    SB_DISPATCH_DTYPE(out_dtype, TO, {
      sb_launch<SB_K_ELEMENTWISE>(cast_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)in, (TO*)out, n);
    });
  });
  SB_CHECK_LAUNCH("sb_cast");
  return SB_OK;
}

// ------------------------------------------------------------- rotation + cache write
// Input: the fused projection row [q heads | k heads | v heads] in float32 (bias already added).
// Half-split rotation of the first `rot` dims of each q and k head: for i < rot/2,
// theta = float(pos) * inv_freq[i]; x'_i = x_i c - x_{i+rot/2} s; x'_{i+rot/2} = x_i s +
// x_{i+rot/2} c, in float32 with the accurate sinf/cosf (core/src/nn/rope.cpp:26-82,
// core/src/nn/cuda_elementwise.cu:326-347).  Rotated q goes to q_out [row, head, hd]; rotated k
// and v go to the sequence's cache page of that position (core/src/model/emit.cpp:291-293,
// core/src/nn/cuda_elementwise.cu:2639), rounded only to the cache's own dtype.
//
// Cache of one schedule entry: [page][k|v][kv head][slot in page][hd].  The page of position p
// of sequence b is page_ids[page_off[b] + p / page_size].
// A row whose position has no page in its own sequence's list (a position before 0 or beyond
// what the sequence has reserved, or a page that was given back) writes no key and no value:
// another sequence's pages are never touched, whatever the plan says.
__device__ __forceinline__ int sb_page_of(const int32_t* page_off, const int32_t* page_ids, int seq,
                                          int pos, int page_size) {
  const int first = page_off[seq], n = page_off[seq + 1] - first;
  const int i = pos / page_size;
  return (pos >= 0 && i < n) ? page_ids[first + i] : -1;
}

// Few rows (decode): one block per (row, head), so that even one row spreads over many SMs.
template <typename TQ, typename TC>
__global__ void rope_store_head_kernel(const float* qkv, int n_q_heads, int n_kv_heads, int hd,
                                       int rot, const float* __restrict__ inv_freq,
                                       const int32_t* row_seq, const int32_t* row_pos,
                                       const int32_t* page_off, const int32_t* page_ids,
                                       int page_size, TC* cache, TQ* q_out, int has_kv) {
  sb_pdl_launch();
  const int t = blockIdx.x;
  const int head = blockIdx.y;                       // q heads, then k heads, then v heads
  const int width_in = (n_q_heads + (has_kv ? 2 * n_kv_heads : 0)) * hd;
  const float* src = qkv + (size_t)t * width_in + (size_t)head * hd;
  const int half = rot >> 1;
  const bool is_v = head >= n_q_heads + n_kv_heads;
  // The position, the page and the angles come from the step's plan, which was complete
  // before the step's first kernel: they are worked out before the wait for the kernel that
  // writes q|k|v.
  const int pos = row_pos[t];
  size_t dst_row = 0;
  if (head >= n_q_heads) {
    const int page = sb_page_of(page_off, page_ids, row_seq[t], pos, page_size);
    if (page < 0) return;                            // no page of its own there: nothing is written
    const int kvh = is_v ? head - n_q_heads - n_kv_heads : head - n_q_heads;
    dst_row = (((size_t)page * 2 + (is_v ? 1 : 0)) * n_kv_heads + kvh) * page_size + pos % page_size;
  }
  float c0 = 1.0f, sn0 = 0.0f;                       // of this thread's first element
  if (!is_v && (int)threadIdx.x < rot) {
    const int i = (int)threadIdx.x < half ? threadIdx.x : threadIdx.x - half;
    const float theta = (float)pos * inv_freq[i];
    c0 = cosf(theta);
    sn0 = sinf(theta);
  }
  sb_pdl_wait();
  for (int e = threadIdx.x; e < hd; e += blockDim.x) {
    float v = src[e];
    if (!is_v && e < rot) {
      float c = c0, sn = sn0;
      if (e != (int)threadIdx.x) {
        const int i = e < half ? e : e - half;
        const float theta = (float)pos * inv_freq[i];
        c = cosf(theta);
        sn = sinf(theta);
      }
      v = e < half ? sb_rot_lo(src[e], src[e + half], c, sn) : sb_rot_hi(src[e - half], src[e], c, sn);
    }
    if (head < n_q_heads)
      q_out[((size_t)t * n_q_heads + head) * hd + e] = sb_from_f32<TQ>(v);
    else
      cache[dst_row * hd + e] = sb_from_f32<TC>(v);
  }
}

// Many rows (prefill):
template <typename TQ, typename TC>
__global__ void rope_store_kernel(const float* qkv, int n_q_heads, int n_kv_heads,
                                  int hd, int rot, const float* __restrict__ inv_freq,
                                  const int32_t* row_seq, const int32_t* row_pos,
                                  const int32_t* page_off, const int32_t* page_ids,
                                  int page_size, TC* cache, TQ* q_out, int has_kv) {
  // One block per row: the angles depend on the position and the pair only, so cos and sin
  // are computed once per row and reused by every head.
  extern __shared__ float cs[];                      // cos[rot/2], then sin[rot/2]
  sb_pdl_launch();
  sb_pdl_wait();
  const int t = blockIdx.x;
  const int pos = row_pos[t];
  const int half = rot >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float theta = (float)pos * inv_freq[i];
    cs[i] = cosf(theta);
    cs[half + i] = sinf(theta);
  }
  __syncthreads();
  const int n_heads = n_q_heads + (has_kv ? 2 * n_kv_heads : 0);
  const float* src_row = qkv + (size_t)t * n_heads * hd;
  size_t k_base = 0, v_base = 0;
  bool stores = has_kv;
  if (has_kv) {
    const int page = sb_page_of(page_off, page_ids, row_seq[t], pos, page_size);
    stores = page >= 0;                              // no page of its own there: queries only
    k_base = (((size_t)(stores ? page : 0) * 2) * n_kv_heads * page_size + pos % page_size) * hd;
    v_base = (((size_t)(stores ? page : 0) * 2 + 1) * n_kv_heads * page_size + pos % page_size) * hd;
  }
  for (int idx = threadIdx.x; idx < n_heads * hd; idx += blockDim.x) {
    const int head = idx / hd, e = idx % hd;       // q heads, then k heads, then v heads
    const float* src = src_row + (size_t)head * hd;
    const bool is_v = head >= n_q_heads + n_kv_heads;
    float v = src[e];
    if (!is_v && e < rot) {
      const int i = e < half ? e : e - half;
      const float c = cs[i], sn = cs[half + i];
      v = e < half ? sb_rot_lo(src[e], src[e + half], c, sn) : sb_rot_hi(src[e - half], src[e], c, sn);
    }
    if (head < n_q_heads) {
      q_out[((size_t)t * n_q_heads + head) * hd + e] = sb_from_f32<TQ>(v);
    } else if (!stores) {
      continue;
    } else if (is_v) {
      cache[v_base + (size_t)(head - n_q_heads - n_kv_heads) * page_size * hd + e] = sb_from_f32<TC>(v);
    } else {
      cache[k_base + (size_t)(head - n_q_heads) * page_size * hd + e] = sb_from_f32<TC>(v);
    }
  }
}

// The same work four values at a time, for bfloat16 outputs: a task is four pairs (e, e + half)
// of one head, or four of the values beyond the rotated part.  float4 loads and 8-byte stores;
// needs half and (hd - rot) to be multiples of 4.
__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}

__global__ void rope_store_vec_kernel(const float* qkv, int n_q_heads, int n_kv_heads, int hd,
                                      int rot, const float* __restrict__ inv_freq,
                                      const int32_t* row_seq, const int32_t* row_pos,
                                      const int32_t* page_off, const int32_t* page_ids,
                                      int page_size, __nv_bfloat16* cache, __nv_bfloat16* q_out,
                                      int has_kv) {
  extern __shared__ float cs[];                      // cos[rot/2], then sin[rot/2]
  sb_pdl_launch();
  sb_pdl_wait();
  const int t = blockIdx.x;
  const int pos = row_pos[t];
  const int half = rot >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float theta = (float)pos * inv_freq[i];
    cs[i] = cosf(theta);
    cs[half + i] = sinf(theta);
  }
  __syncthreads();
  const int n_heads = n_q_heads + (has_kv ? 2 * n_kv_heads : 0);
  const float* src_row = qkv + (size_t)t * n_heads * hd;
  size_t k_base = 0, v_base = 0;
  bool stores = has_kv;
  if (has_kv) {
    const int page = sb_page_of(page_off, page_ids, row_seq[t], pos, page_size);
    stores = page >= 0;                              // no page of its own there: queries only
    k_base = (((size_t)(stores ? page : 0) * 2) * n_kv_heads * page_size + pos % page_size) * hd;
    v_base = (((size_t)(stores ? page : 0) * 2 + 1) * n_kv_heads * page_size + pos % page_size) * hd;
  }
  const int pair_tasks = half >> 2, per_head = pair_tasks + ((hd - rot) >> 2);
  for (int task = threadIdx.x; task < n_heads * per_head; task += blockDim.x) {
    const int head = task / per_head, k = task % per_head;
    const float* src = src_row + (size_t)head * hd;
    const bool is_v = head >= n_q_heads + n_kv_heads;
    if (head >= n_q_heads && !stores) continue;
    __nv_bfloat16* dst =
        head < n_q_heads ? q_out + ((size_t)t * n_q_heads + head) * hd
        : is_v ? cache + v_base + (size_t)(head - n_q_heads - n_kv_heads) * page_size * hd
               : cache + k_base + (size_t)(head - n_q_heads) * page_size * hd;
    if (k >= pair_tasks) {                           // beyond the rotated part: a copy
      const int e = rot + 4 * (k - pair_tasks);
      const float4 a = *reinterpret_cast<const float4*>(src + e);
      store_bf16x4(dst + e, a.x, a.y, a.z, a.w);
      continue;
    }
    const int e = 4 * k;
    const float4 a = *reinterpret_cast<const float4*>(src + e);
    const float4 b = *reinterpret_cast<const float4*>(src + e + half);
    if (is_v) {
      store_bf16x4(dst + e, a.x, a.y, a.z, a.w);
      store_bf16x4(dst + e + half, b.x, b.y, b.z, b.w);
    } else {
      const float4 c = *reinterpret_cast<const float4*>(cs + e);
      const float4 sn = *reinterpret_cast<const float4*>(cs + half + e);
      store_bf16x4(dst + e, sb_rot_lo(a.x, b.x, c.x, sn.x), sb_rot_lo(a.y, b.y, c.y, sn.y),
                   sb_rot_lo(a.z, b.z, c.z, sn.z), sb_rot_lo(a.w, b.w, c.w, sn.w));
      store_bf16x4(dst + e + half, sb_rot_hi(a.x, b.x, c.x, sn.x), sb_rot_hi(a.y, b.y, c.y, sn.y),
                   sb_rot_hi(a.z, b.z, c.z, sn.z), sb_rot_hi(a.w, b.w, c.w, sn.w));
    }
  }
}

extern "C" int sb_rope_store(const float* qkv, int n_rows, int n_q_heads, int n_kv_heads, int hd,
                             int rot, const float* inv_freq, const int32_t* row_seq,
                             const int32_t* row_pos, const int32_t* page_off,
                             const int32_t* page_ids, int page_size, void* cache, int cache_dtype,
                             void* q_out, int q_dtype, int has_kv, cudaStream_t stream) {
  if (n_rows <= 0 || n_q_heads <= 0 || hd <= 0 || (has_kv && n_kv_heads <= 0))
    SB_FAIL(SB_ERR_ARG, "sb_rope_store: n_rows=%d heads=%d/%d hd=%d", n_rows, n_q_heads,
            n_kv_heads, hd);
  if (rot < 0 || rot > hd || (rot & 1))
    SB_FAIL(SB_ERR_ARG, "sb_rope_store: rotary dims %d of head dim %d (must be even, <= hd)", rot, hd);
  if (!sb_valid_dtype(cache_dtype) || !sb_valid_dtype(q_dtype))
    SB_FAIL(SB_ERR_ARG, "sb_rope_store: dtype codes %d %d", cache_dtype, q_dtype);
  if (has_kv && (page_size <= 0 || !cache || !page_off || !page_ids))
    SB_FAIL(SB_ERR_ARG, "sb_rope_store: cache arguments missing");
  const dim3 grid(n_rows);
  const int width = (n_q_heads + (has_kv ? 2 * n_kv_heads : 0)) * hd;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
  if (n_rows < 64 && n_q_heads + 2 * n_kv_heads <= 65535) {
    const dim3 hgrid(n_rows, n_q_heads + (has_kv ? 2 * n_kv_heads : 0));
    const int hthreads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    SB_DISPATCH_DTYPE(q_dtype, TQ, {
      SB_DISPATCH_DTYPE(cache_dtype, TC, {
        sb_launch<SB_K_ELEMENTWISE>(rope_store_head_kernel<TQ, TC>, hgrid, dim3(hthreads), 0, stream, qkv, n_q_heads,
                  n_kv_heads, hd, rot, inv_freq, row_seq, row_pos, page_off, page_ids, page_size,
                  (TC*)cache, (TQ*)q_out, has_kv);
      });
    });
    SB_CHECK_LAUNCH("sb_rope_store");
    return SB_OK;
  }
  if (q_dtype == SB_BF16 && cache_dtype == SB_BF16 && (rot & 7) == 0 && ((hd - rot) & 3) == 0 &&
      (((uintptr_t)qkv | (uintptr_t)inv_freq) & 15) == 0 &&
      (((uintptr_t)q_out | (uintptr_t)cache) & 7) == 0) {
    sb_launch<SB_K_ELEMENTWISE>(rope_store_vec_kernel, grid, dim3(threads), smem, stream, qkv, n_q_heads, n_kv_heads,
              hd, rot, inv_freq, row_seq, row_pos, page_off, page_ids, page_size,
              (__nv_bfloat16*)cache, (__nv_bfloat16*)q_out, has_kv);
    SB_CHECK_LAUNCH("sb_rope_store");
    return SB_OK;
  }
  SB_DISPATCH_DTYPE(q_dtype, TQ, {
    SB_DISPATCH_DTYPE(cache_dtype, TC, {
      sb_launch<SB_K_ELEMENTWISE>(rope_store_kernel<TQ, TC>, grid, dim3(threads), smem, stream,
          qkv, n_q_heads, n_kv_heads, hd, rot, inv_freq, row_seq, row_pos, page_off, page_ids,
          page_size, (TC*)cache, (TQ*)q_out, has_kv);
    });
  });
  SB_CHECK_LAUNCH("sb_rope_store");
  return SB_OK;
}
