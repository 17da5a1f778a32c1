/* Public C interface of the sonicboom_b200 kernel libraries (sm_100a).
 *
 * Two kinds of shared library are built from this folder:
 *   libsonicboom_b200.so              the core library: everything under "core library" below;
 *   libsonicboom_b200_attn_hd<N>.so   one per head size N (16 ... 256 in steps of 16): the
 *                                     tensor-core attention kernels, under "attention library".
 * Every library also exports sb_last_error, sb_pdl_enabled and sb_set_pdl (its own copies).
 *
 * Conventions.  Every entry point takes raw device pointers and a CUDA stream, checks its
 * arguments on the host before anything is launched and returns an SbStatus; on a non-zero
 * status sb_last_error() of the same library describes what was refused.  Nothing here
 * allocates device memory: scratch is passed in by the caller (or, for
 * sb_attention_decode_static, lives in the library: see no_alloc.h).  Tensors are contiguous and
 * row-major; dtype arguments are SbDtype codes.  The header compiles as C and as C++.
 */
#ifndef SONICBOOM_B200_H
#define SONICBOOM_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__) || defined(__CUDA_RUNTIME_API_H__) || defined(__DRIVER_TYPES_H__)
#include <cuda_runtime_api.h>
typedef cudaStream_t sb_stream_t;
#else
typedef struct CUstream_st* sb_stream_t;       /* the type cuda_runtime_api.h calls cudaStream_t */
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum SbDtype { SB_F32 = 0, SB_BF16 = 1 };
enum SbStatus { SB_OK = 0, SB_ERR_ARG = 1, SB_ERR_UNSUPPORTED = 2, SB_ERR_CUDA = 3 };
/* What a product does with its finished rows.  SB_EPI_SWIGLU: the weight's rows alternate in
 * blocks of 8 (8 gate rows, the 8 up rows of the same outputs); out[m, o] = silu(gate) * up and
 * has N / 2 columns. */
enum SbEpilogue { SB_EPI_NONE = 0, SB_EPI_BIAS = 1, SB_EPI_RESIDUAL = 2, SB_EPI_SWIGLU = 3 };
/* Kernel classes: bits of the mask that says which kernels are launched with programmatic
 * dependent launch (sb_set_pdl). */
enum SbKernelClass {
  SB_K_TC5 = 1,          /* tcgen05 products */
  SB_K_SKINNY = 2,       /* weight-streaming and tiled mma.sync products */
  SB_K_ATTENTION = 4,
  SB_K_ELEMENTWISE = 8,  /* embedding, norms, rotation, casts, small adds */
  SB_K_REDUCE = 16,      /* the split-K reduce of the tcgen05 product */
  SB_K_OTHER = 32        /* sampler, plain kernels */
};

/* The rotation and cache write that may finish a fused q|k|v product (the arguments of
 * sb_rope_store without the input row, which the product supplies). */
typedef struct SbRopeStore {
  int n_q_heads, n_kv_heads, hd, rot;
  const float* inv_freq;
  const int32_t* row_seq;
  const int32_t* row_pos;
  const int32_t* page_off;
  const int32_t* page_ids;
  int page_size;
  void* cache;                 /* bfloat16 pages of the schedule entry; null: queries only */
  void* q_out;                 /* bfloat16 [rows, n_q_heads, hd] */
} SbRopeStore;

/* What may accompany a product (all optional): the RMSNorm of its finished rows, memory to ask
 * into L2 for a later kernel, and the rotation + cache write of a q|k|v product's rows (then the
 * product's own output is not written: `out` may be null). */
typedef struct SbLinearExtras {
  const void* norm_weight;     /* null: no norm */
  int norm_weight_dtype;
  float norm_eps;
  void* norm_out;
  int norm_out_dtype;
  const void* warm;            /* null: nothing; else bytes a later kernel will stream */
  size_t warm_bytes;
  const SbRopeStore* rope;     /* null: none; only where sb_gemm_tc5_fuses_rope says so */
} SbLinearExtras;

/* One row's sampling record (sb_sample reads an array of them from device memory). */
typedef struct SbSampleParams {
  float temperature, top_p, min_p, repeat_penalty, presence_penalty, frequency_penalty;
  uint32_t top_k;
  int32_t history_len;         /* tokens of this row in `history` (already cut to the window) */
  uint64_t seed;
  uint64_t position;           /* absolute position of the token being produced */
} SbSampleParams;

/* ------------------------------------------------------------------ every library */
const char* sb_last_error(void);
int sb_pdl_enabled(void);                 /* the mask of SbKernelClass bits in force */
void sb_set_pdl(int mask);

/* ------------------------------------------------------------------ core library */
int sb_abi_version(void);

/* out[t, :] = table[tokens[t], :] * scale as float32; an id outside the table gives NaN. */
int sb_embed(const int32_t* tokens, int n_rows, const void* table, int table_dtype, int vocab,
             int width, float scale, float* out, sb_stream_t stream);
/* out[r] = x[rows ? rows[r] : r] / sqrt(mean(x^2) + eps) * weight */
int sb_rmsnorm(const float* x, const int32_t* rows, int n_rows, int width, const void* weight,
               int weight_dtype, float eps, void* out, int out_dtype, sb_stream_t stream);
int sb_softcap(float* x, size_t n, float cap, sb_stream_t stream);     /* x = cap tanh(x / cap) */
int sb_add_bias(float* x, const void* bias, int bias_dtype, int rows, int width, sb_stream_t stream);   /* x[m, n] += bias[n] */
int sb_cast(const void* in, int in_dtype, void* out, int out_dtype, size_t n, sb_stream_t stream);
/* Rotates q and k of the fused row [q | k | v], writes q to q_out and k, v into the pages of
 * each row's sequence; a position without a page in its own sequence's list writes nothing. */
int sb_rope_store(const float* qkv, int n_rows, int n_q_heads, int n_kv_heads, int hd, int rot,
                  const float* inv_freq, const int32_t* row_seq, const int32_t* row_pos,
                  const int32_t* page_off, const int32_t* page_ids, int page_size, void* cache,
                  int cache_dtype, void* q_out, int q_dtype, int has_kv, sb_stream_t stream);

/* out[M, N] = A[M, K] . W[N, K]^T with an SbEpilogue; float32 accumulation. */
int sb_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                  int epilogue, const void* bias, int bias_dtype, const float* residual,
                  void* out, int out_dtype, sb_stream_t stream);
int sb_gemm_skinny(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                   int epilogue, const void* bias, int bias_dtype, const float* residual,
                   void* out, int out_dtype, sb_stream_t stream);
int sb_gemm_tiled(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                  int epilogue, const void* bias, int bias_dtype, const float* residual,
                  void* out, int out_dtype, sb_stream_t stream);
/* TMA + tcgen05.  form: 0 by the number of rows, 1 the normal form, 2 the swapped (decode) form. */
int sb_gemm_tc5(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                int epilogue, const void* bias, int bias_dtype, const float* residual, void* out,
                int out_dtype, void* scratch, size_t scratch_bytes, int n_sms, int form,
                sb_stream_t stream);
int sb_gemm_tc5_ex(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                   int epilogue, const void* bias, int bias_dtype, const float* residual,
                   void* out, int out_dtype, void* scratch, size_t scratch_bytes, int n_sms,
                   int form, const SbLinearExtras* extras, sb_stream_t stream);
size_t sb_gemm_tc5_scratch_bytes(int M, int N, int K, int n_sms);
int sb_gemm_tc5_fuses_norm(int M, int N, int K, int n_sms, int epilogue, int out_dtype, int form);
/* Whether sb_gemm_tc5_ex can finish a q|k|v product of these sizes with the rotation and the
 * cache write (the split-K decode form, bfloat16 queries and cache, head sizes in steps of 8). */
int sb_gemm_tc5_fuses_rope(int M, int N, int K, int n_sms, int n_q_heads, int n_kv_heads, int hd,
                           int rot, int has_kv);
int sb_tc5_status(void);      /* 0, or the code of a bounded wait that gave up; clears it */
void sb_gemm_tc5_pairs(int mode);   /* products of more than 128 rows on pairs of SMs: 1 yes, 0 no, -1 by SB_TC5_PAIR */
void sb_gemm_tc5_force_width(int bn);   /* 256, 240, 224, 208 or 192 for every many-rows product; else by the sizes */
int sb_gemm_tc5_tile_width(int M, int N, int n_sms);   /* tile width of the many-rows form; 0: that form does not run */

/* Plain attention over the paged cache (float32 arithmetic, any head size up to 256). */
int sb_attention_plain(const void* q, void* out, int act_dtype, int n_rows, const int32_t* row_seq,
                       const int32_t* row_pos, const int32_t* page_off, const int32_t* page_ids,
                       int page_size, const void* cache, int cache_dtype, int n_q_heads,
                       int n_kv_heads, int hd, int window, float scale, sb_stream_t stream);

int sb_sample_params_size(void);
int sb_sample(float* logits, int n_rows, int vocab, const void* params, const int32_t* history,
              int history_stride, const int32_t* fed_pos, int32_t* out_tokens, sb_stream_t stream);
int sb_add_i32(int32_t* x, int n, int delta, sb_stream_t stream);
/* x[i] = min(x[i] + 1, last[i]) */
int sb_advance_rows(int32_t* x, const int32_t* last, int n, sb_stream_t stream);
/* out[e] = mean + std * z_e, z standard normal, a function of (key0, key1, e) only. */
int sb_random_normal(void* out, int out_dtype, size_t n, uint32_t key0, uint32_t key1, float mean,
                     float std, sb_stream_t stream);

/* ------------------------------------------------------------------ attention library */
int sb_attention_head_dim(void);
void sb_attention_force_mma(int mode);    /* 0 by size; 1 the mma.sync kernels; 2 the TMA decode kernel always */
int sb_attention_status(void);            /* as sb_tc5_status; -1: no tensor-memory kernel */
int sb_attention_last_launches(void);     /* kernels the last sb_attention call launched */
size_t sb_attention_scratch_bytes(int n_rows, int n_q_heads, int n_kv_heads, int max_new,
                                  int max_len);
/* Causal grouped-query attention of a step's rows over one cache entry's pages (bfloat16). */
int sb_attention(const void* q, void* out, int n_rows, int n_seqs, int max_new,
                 const int32_t* seq_row0, const int32_t* seq_pos0, const int32_t* page_off,
                 const int32_t* page_ids, int page_size, const void* cache, int n_q_heads,
                 int n_kv_heads, int hd, int window, float scale, void* scratch,
                 size_t scratch_bytes, int* counters, int n_counters, int max_len, int n_pages,
                 int n_sms, const void* warm, size_t warm_bytes, sb_stream_t stream);

#ifdef __cplusplus
}
#endif

#include "no_alloc.h"        /* sb_attention_decode_static (attention library) */

#endif /* SONICBOOM_B200_H */
