// Attention whose keys and values are made from one low-rank latent per token.
//
// Per token the cache keeps one row of `rank + rot` elements: the latent c (RMS-normed) and a rotated key part
// r that all heads share.  Head j's key is [W_uk_j c ; r] and its value W_uv_j c, so with the query folded
// through W_uk_j (a_j = W_uk_j^T q_j, done by a batched product before this kernel)
//     score_j(t, s) = (a_j(t) . c(s) + qr_j(t) . r(s)) * scale,      out_j(t) = W_uv_j sum_s p_j(t, s) c(s)
// which is attention with ONE key head of width rank + rot whose value is the first `rank` elements of
// the key.  This file has the two kernels in between the products:
//
//   latent_append     per token: c = rmsnorm(dkv[:rank]) * w, r = rotate(dkv[rank:]), both stored in the token's
//                     page; qr_j = rotate(q_j[dim:]) written behind a_j in the folded query rows.  Rotary pairs
//                     are (2i, 2i+1), angle = position * inv_freq[i] in fp32, on the first 2 * n_freq elements.
//   latent_attention  causal softmax attention of the folded queries [tokens, heads, rank + rot] (fp32) over
//                     the paged latent rows; out [tokens, heads, rank] (fp32).  CUDA cores, fp32 throughout:
//                     one warp owns one (token, head) row and walks the keys in blocks of 32 aligned to absolute
//                     positions, so a row's arithmetic does not depend on how the batch was cut.
#include "common.cuh"
#include <math_constants.h>

namespace tib {

struct LatentAppendArgs {
  const int* positions;    // [tokens]
  const int* token_slot;   // [tokens]
  const int* block_table;
  int table_stride;
  const float* norm_weight;   // [rank]
  const float* inv_freq;      // [n_freq]
  int n_freq;
  int rank, rot, heads, dim;  // dim: unrotated query elements per head
  int64_t ld_dkv, ld_q;
  int page_size, num_pages;
  int64_t page_stride;
  float eps;
  int* error_word;
};

template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ dkv, const T* __restrict__ q, T* __restrict__ pool,
                                     float* __restrict__ folded, LatentAppendArgs a) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  const int pos = a.positions[t];
  const int width = a.rank + a.rot;
  const T* src = dkv + t * a.ld_dkv;
  T* dst = nullptr;
  if (pool) {
    const int page = a.block_table[(size_t)a.token_slot[t] * a.table_stride + pos / a.page_size];
    if (page >= 0 && page < a.num_pages) {
      dst = pool + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * width;
    } else if (a.error_word && threadIdx.x == 0) {
      atomicExch(a.error_word, 0x20000 + (int)(t & 0xffff));
    }
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < a.rank; c += blockDim.x) {
    const float v = to_f32(src[c]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)a.rank + a.eps);
  if (dst)
    for (int c = threadIdx.x; c < a.rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32(src[c]) * inv * a.norm_weight[c]);
  // the shared key part (job 0) and every head's rotated query part (jobs 1 .. heads): pairs (2i, 2i + 1)
  const int half = a.rot / 2;      // an odd last element, if any, passes unchanged below
  for (int e = threadIdx.x; e < (a.heads + 1) * half; e += blockDim.x) {
    const int job = e / half, i = e - job * half;
    const T* from = job == 0 ? src + a.rank : q + t * a.ld_q + (size_t)(job - 1) * (a.dim + a.rot) + a.dim;
    float lo = to_f32(from[2 * i]), hi = to_f32(from[2 * i + 1]);
    if (i < a.n_freq) {
      const float angle = (float)pos * a.inv_freq[i];
      const float c = cosf(angle), s = sinf(angle);
      const float l2 = rope_lo(lo, hi, c, s), h2 = rope_hi(lo, hi, c, s);
      lo = l2; hi = h2;
    }
    if (job == 0) {
      if (dst) { dst[a.rank + 2 * i] = from_f32<T>(lo); dst[a.rank + 2 * i + 1] = from_f32<T>(hi); }
    } else {
      float* f = folded + (t * a.heads + (job - 1)) * (size_t)width + a.rank;
      f[2 * i] = lo; f[2 * i + 1] = hi;
    }
  }
  if ((a.rot & 1) && threadIdx.x == 0) {
    if (dst) dst[width - 1] = src[width - 1];
    for (int h = 0; h < a.heads; ++h)
      folded[(t * a.heads + h) * (size_t)width + width - 1] = to_f32(q[t * a.ld_q + (size_t)h * (a.dim + a.rot) + a.dim + a.rot - 1]);
  }
}

// ---------------------------------------------------------------- attention
constexpr int kLatWarps = 4;
constexpr int kLatRowsPerWarp = 4;
constexpr int kLatRows = kLatWarps * kLatRowsPerWarp;
constexpr int kLatKeys = 32;

struct LatentAttnArgs {
  const int* q_start;
  const int* kv_start;
  const int* slots;
  const int* block_table;
  int table_stride;
  int heads, rank, width;     // width = rank + rot
  int page_size, num_pages;
  int64_t page_stride;
  float scale;
  int head_chunk, q_tile;
  int* error_word;
};

template <typename T, int DPL>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const float* __restrict__ folded, const T* __restrict__ pool, float* __restrict__ out,
                        LatentAttnArgs a) {
  extern __shared__ float smem[];
  const int w = a.width, wp = w + 1;
  float* q_s = smem;                       // [kLatRows][w]
  float* k_s = q_s + kLatRows * w;         // [32][w + 1]
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.y;
  const int h0 = blockIdx.z * a.head_chunk;
  const int hc = min(a.head_chunk, a.heads - h0);
  const int row0 = a.q_start[entry];
  const int q_len = a.q_start[entry + 1] - row0;
  const int t0 = blockIdx.x * a.q_tile;
  if (t0 >= q_len) return;
  const int nt = min(a.q_tile, q_len - t0);
  const int nrows = nt * hc;
  const int pos0 = a.kv_start[entry] + t0;
  const int last_pos = pos0 + nt - 1;
  const int* table = a.block_table + (size_t)a.slots[entry] * a.table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int e = threadIdx.x; e < nrows * w; e += blockDim.x) {
    const int r = e / w, dd = e - r * w;
    const int t = r / hc, g = r - t * hc;
    q_s[r * w + dd] = folded[((size_t)(row0 + t0 + t) * a.heads + h0 + g) * w + dd];
  }
  float m[kLatRowsPerWarp], l[kLatRowsPerWarp], acc[kLatRowsPerWarp][DPL];
#pragma unroll
  for (int i = 0; i < kLatRowsPerWarp; ++i) {
    m[i] = -CUDART_INF_F;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[i][j] = 0.f;
  }
  const int b_hi = last_pos / kLatKeys;
  for (int b = 0; b <= b_hi; ++b) {
    __syncthreads();
    // Latent rows of block b; rows past last_pos are not written yet (or are nobody's): zeros, always masked.
    for (int e = threadIdx.x; e < kLatKeys * w; e += blockDim.x) {
      const int j = e / w, dd = e - j * w;
      const int kp = b * kLatKeys + j;
      float kval = 0.f;
      if (kp <= last_pos) {
        const int page = table[kp / a.page_size];
        if (page >= 0 && page < a.num_pages) {
          kval = to_f32(pool[(size_t)page * a.page_stride + (size_t)(kp % a.page_size) * w + dd]);
        } else if (a.error_word) {
          atomicExch(a.error_word, 0x30000 + entry);
        }
      }
      k_s[j * wp + dd] = kval;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kLatRowsPerWarp; ++i) {
      const int r = warp * kLatRowsPerWarp + i;
      if (r >= nrows) continue;                       // uniform in the warp
      const int qpos = pos0 + r / hc;
      if (b * kLatKeys > qpos) continue;
      const int kp = b * kLatKeys + lane;
      const bool allowed = kp <= qpos;
      float s = 0.f;
      const float* qr = q_s + r * w;
      const float* kr = k_s + lane * wp;
      for (int dd = 0; dd < w; ++dd) s = fmaf(qr[dd], kr[dd], s);
      s = allowed ? s * a.scale : -CUDART_INF_F;
      const float m_new = fmaxf(m[i], warp_max(s));
      const float alpha = m[i] == -CUDART_INF_F ? 0.f : expf(m[i] - m_new);
      const float p = allowed ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[i][j] *= alpha;
      for (int kk = 0; kk < kLatKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
          const int dd = lane + 32 * j;
          if (dd < a.rank) acc[i][j] = fmaf(pk, k_s[kk * wp + dd], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kLatRowsPerWarp; ++i) {
    const int r = warp * kLatRowsPerWarp + i;
    if (r >= nrows) continue;
    const int t = r / hc, g = r - t * hc;
    float* dst = out + ((size_t)(row0 + t0 + t) * a.heads + h0 + g) * a.rank;
    const float inv = 1.f / l[i];
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int dd = lane + 32 * j;
      if (dd < a.rank) dst[dd] = acc[i][j] * inv;
    }
  }
}

template <typename T, int DPL>
static int launch_latent_attention(const float* folded, const void* pool, float* out, const LatentAttnArgs& a, int n_entries,
                                   int max_q_len, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)kLatRows * a.width + (size_t)kLatKeys * (a.width + 1));
  if (smem > 227 * 1024) return TIB_E_SMEM;
  auto kern = latent_attention_kernel<T, DPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(ceil_div(max_q_len, a.q_tile), n_entries, ceil_div(a.heads, a.head_chunk));
  TIB_LAUNCH_DEPENDENT(kern, grid, kLatWarps * 32, smem, stream, folded, (const T*)pool, out, a);
  return TIB_OK;
}

}  // namespace tib

using namespace tib;

// dkv: [tokens, rank + rot] (row stride ld_dkv); q: [tokens, heads * (dim + rot)] (row stride ld_q); pool: this layer's
// pages, each [page_size][rank + rot] (null: nothing is stored); folded: [tokens, heads, rank + rot] fp32, of which
// this call writes the last `rot` elements of every head.
TIB_API int tib_latent_append(const void* dkv, int64_t ld_dkv, const void* q, int64_t ld_q, void* pool, float* folded,
                              const int* positions, const int* token_slot, const int* block_table, int table_stride,
                              const float* norm_weight, float eps, const float* inv_freq, int n_freq, int n_tokens, int heads,
                              int dim, int rank, int rot, int page_size, int64_t page_stride, int num_pages,
                              int* error_word, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return TIB_OK;
  if (!dkv || !q || !folded || !positions || !norm_weight || (n_freq > 0 && !inv_freq)) return TIB_E_ARG;
  if (pool && (!token_slot || !block_table || page_size < 1)) return TIB_E_ARG;
  if (heads < 1 || dim < 0 || rank < 1 || rot < 0 || 2 * n_freq > rot) return TIB_E_SIZE;
  LatentAppendArgs a;
  a.positions = positions; a.token_slot = token_slot; a.block_table = block_table; a.table_stride = table_stride;
  a.norm_weight = norm_weight; a.inv_freq = inv_freq; a.n_freq = n_freq; a.rank = rank; a.rot = rot; a.heads = heads;
  a.dim = dim; a.ld_dkv = ld_dkv; a.ld_q = ld_q; a.page_size = page_size; a.num_pages = num_pages;
  a.page_stride = page_stride; a.eps = eps; a.error_word = error_word;
  if (dtype == TIB_F32)
    TIB_LAUNCH_DEPENDENT(latent_append_kernel<float>, n_tokens, 128, 0, stream, (const float*)dkv, (const float*)q,
                         (float*)pool, folded, a);
  else if (dtype == TIB_BF16)
    TIB_LAUNCH_DEPENDENT(latent_append_kernel<__nv_bfloat16>, n_tokens, 128, 0, stream, (const __nv_bfloat16*)dkv,
                         (const __nv_bfloat16*)q, (__nv_bfloat16*)pool, folded, a);
  else
    return TIB_E_DTYPE;
  return TIB_OK;
}

// folded: [tokens, heads, rank + rot] fp32; pool: pages of [page_size][rank + rot] in `dtype`; out: [tokens, heads, rank] fp32.
TIB_API int tib_latent_attention(const float* folded, const void* pool, float* out, const int* q_start, const int* kv_start,
                                 const int* slots, const int* block_table, int table_stride, int n_entries, int max_q_len,
                                 int heads, int rank, int rot, int page_size, int64_t page_stride, int num_pages, float scale,
                                 int* error_word, int dtype, cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!folded || !pool || !out || !q_start || !kv_start || !slots || !block_table) return TIB_E_ARG;
  if (heads < 1 || rank < 1 || rot < 0 || page_size < 1 || rank > 512 || n_entries > 65535) return TIB_E_SIZE;
  LatentAttnArgs a;
  a.q_start = q_start; a.kv_start = kv_start; a.slots = slots; a.block_table = block_table; a.table_stride = table_stride;
  a.heads = heads; a.rank = rank; a.width = rank + rot; a.page_size = page_size; a.num_pages = num_pages;
  a.page_stride = page_stride; a.scale = scale; a.error_word = error_word;
  a.head_chunk = heads < kLatRows ? heads : kLatRows;
  a.q_tile = kLatRows / a.head_chunk;
  if (ceil_div(heads, a.head_chunk) > 65535) return TIB_E_SIZE;
  const int dpl = (rank + 31) / 32;
#define TIB_LAT_DISPATCH(T)                                                                             \
  (dpl <= 1 ? launch_latent_attention<T, 1>(folded, pool, out, a, n_entries, max_q_len, stream)        \
   : dpl <= 2 ? launch_latent_attention<T, 2>(folded, pool, out, a, n_entries, max_q_len, stream)      \
   : dpl <= 4 ? launch_latent_attention<T, 4>(folded, pool, out, a, n_entries, max_q_len, stream)      \
   : dpl <= 8 ? launch_latent_attention<T, 8>(folded, pool, out, a, n_entries, max_q_len, stream)      \
              : launch_latent_attention<T, 16>(folded, pool, out, a, n_entries, max_q_len, stream))
  if (dtype == TIB_F32) return TIB_LAT_DISPATCH(float);
  if (dtype == TIB_BF16) return TIB_LAT_DISPATCH(__nv_bfloat16);
#undef TIB_LAT_DISPATCH
  return TIB_E_DTYPE;
}
