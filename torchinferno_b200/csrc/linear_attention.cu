// Linear attention with a fixed decay per head over per-request state:
//     S_t = lambda * S_(t-1) + k_t v_t^T        (S: [key_dim, value_dim], fp32, one per request, layer call and head)
//     o_t = S_t^T q_t
// for the tokens of a ragged batch: portions of prompts and single decoded tokens alike.  An optional
// activation (silu) is applied to q, k and v as they are read, in fp32.
//
// One block owns one (request entry, head, run of value columns): the columns of S do not depend on one another, so
// a head is cut into runs of columns that go to blocks of their own until the grid fills the GPU (each recomputes the
// chunk's scores, which are cheap beside the state).  A block keeps its columns of S in shared memory and walks the
// entry's tokens in chunks of up to C: within a chunk of n tokens
//     A[i][j] = (q_i . k_j) lambda^(i-j)                                    j <= i
//     o_i     = lambda^(i+1) S^T q_i + sum_(j<=i) A[i][j] v_j
//     S      <- lambda^n S + sum_j lambda^(n-1-j) k_j v_j^T
// which is the recurrence written out.  Scores, decay powers, state and sums are fp32; the powers
// lambda^0 .. lambda^C come from the host as a table (made in double precision).  A single token is a chunk
// of one.  State is read from and written back to the request's slot; a new request's slot is zero.
#include "common.cuh"

namespace tib {

struct LinAttnArgs {
  const int* q_start;     // [n_entries + 1]
  const int* slots;       // [n_entries]
  const float* powers;    // [heads, chunk + 1]
  float* state;           // [slots, heads, key_dim, value_dim]
  float* out;             // [tokens, heads * value_dim]
  int64_t ldq, ldk, ldv;  // row strides of q, k, v (elements)
  int heads, key_dim, value_dim, chunk, activation;
  int cols;               // value columns per block
};

__device__ __forceinline__ float lin_act(float z, int activation) { return activation ? z / (1.f + expf(-z)) : z; }

template <typename T>
__global__ void __launch_bounds__(256)
linear_attention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, LinAttnArgs a) {
  extern __shared__ float smem[];
  const int D = a.key_dim, C = a.chunk, DP = D + 1;
  const int col0 = blockIdx.z * a.cols;
  const int V = min(a.cols, a.value_dim - col0);       // this block's columns: col0 .. col0 + V - 1 of the head's value_dim
  float* S = smem;                 // [D][V]
  float* qs = S + D * a.cols;      // [C][DP]
  float* ks = qs + C * DP;         // [C][DP]
  float* vs = ks + C * DP;         // [C][V], on a 16-byte boundary (rows of four columns are read as one)
  vs += (4 - (int)((vs - smem) & 3)) & 3;
  float* A = vs + C * a.cols;      // [C][C]
  float* pw = A + C * C;           // [C + 1]
  const int head = blockIdx.x, entry = blockIdx.y;
  pdl_wait();
  pdl_trigger();
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  if (len <= 0) return;
  float* state = a.state + ((size_t)a.slots[entry] * a.heads + head) * D * a.value_dim + col0;      // row stride value_dim
  for (int e = threadIdx.x; e < D * V; e += blockDim.x) S[e] = state[(size_t)(e / V) * a.value_dim + e % V];
  for (int e = threadIdx.x; e <= C; e += blockDim.x) pw[e] = a.powers[head * (C + 1) + e];

  // bf16 rows on 16-byte boundaries are fetched eight elements a load, and the next chunk's rows are asked for before
  // the current chunk is worked on (they wait in registers): fetched element by element where they were needed, the
  // rows cost a chain of memory latencies per chunk, more than the arithmetic.
  constexpr int kPieces = 4;       // 16-byte pieces a thread holds per tensor
  const int dp = D / 8, vp = V / 8;
  bool wide = false;
  if constexpr (sizeof(T) == 2) {
    wide = D % 8 == 0 && V % 8 == 0 && col0 % 8 == 0 && a.value_dim % 8 == 0 && a.ldq % 8 == 0 && a.ldk % 8 == 0 && a.ldv % 8 == 0 &&
           ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0 &&
           C * dp <= kPieces * (int)blockDim.x && C * vp <= kPieces * (int)blockDim.x;
  }
  uint4 rq[kPieces], rk[kPieces], rv[kPieces];
  auto ask = [&](int t0) {
    const int n = min(C, len - t0);
#pragma unroll
    for (int it = 0; it < kPieces; ++it) {
      const int p = threadIdx.x + it * blockDim.x;
      if (p < n * dp) {
        const int i = p / dp, c = (p - i * dp) * 8;
        const size_t row = row0 + t0 + i;
        rq[it] = *reinterpret_cast<const uint4*>(q + row * a.ldq + head * D + c);
        rk[it] = *reinterpret_cast<const uint4*>(k + row * a.ldk + head * D + c);
      }
      if (p < n * vp) {
        const int i = p / vp, c = (p - i * vp) * 8;
        rv[it] = *reinterpret_cast<const uint4*>(v + (size_t)(row0 + t0 + i) * a.ldv + head * a.value_dim + col0 + c);
      }
    }
  };
  auto unpack = [&](const uint4& raw, float* dst) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float2 f = bf16x2_floats(h2[x]);
      dst[2 * x] = lin_act(f.x, a.activation);
      dst[2 * x + 1] = lin_act(f.y, a.activation);
    }
  };
  if (wide) ask(0);

  for (int t0 = 0; t0 < len; t0 += C) {
    const int n = min(C, len - t0);
    __syncthreads();               // the chunk before is done with qs, ks, vs, A (and S, pw are loaded)
    if (wide) {
#pragma unroll
      for (int it = 0; it < kPieces; ++it) {
        const int p = threadIdx.x + it * blockDim.x;
        if (p < n * dp) {
          const int i = p / dp, c = (p - i * dp) * 8;
          unpack(rq[it], qs + i * DP + c);
          unpack(rk[it], ks + i * DP + c);
        }
        if (p < n * vp) {
          const int i = p / vp, c = (p - i * vp) * 8;
          unpack(rv[it], vs + i * V + c);
        }
      }
      if (t0 + C < len) ask(t0 + C);
    } else {
      for (int e = threadIdx.x; e < n * D; e += blockDim.x) {
        const int i = e / D, d = e - i * D;
        const size_t row = row0 + t0 + i;
        qs[i * DP + d] = lin_act(to_f32(q[row * a.ldq + head * D + d]), a.activation);
        ks[i * DP + d] = lin_act(to_f32(k[row * a.ldk + head * D + d]), a.activation);
      }
      for (int e = threadIdx.x; e < n * V; e += blockDim.x) {
        const int i = e / V, c = e - i * V;
        vs[i * V + c] = lin_act(to_f32(v[(size_t)(row0 + t0 + i) * a.ldv + head * a.value_dim + col0 + c]), a.activation);
      }
    }
    __syncthreads();
    // scores: a thread takes a 2 x 2 block (rows i, i + 1; keys j, j + 1), so four products share four loads
    {
      const int half = (n + 1) / 2;
      for (int e = threadIdx.x; e < half * half; e += blockDim.x) {
        const int bi = e / half, bj = e - bi * half;
        const int i = 2 * bi, j = 2 * bj;
        if (j > i + 1) continue;                       // the block lies above the diagonal
        const int i1 = min(i + 1, n - 1), j1 = min(j + 1, n - 1);
        float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;
        for (int d = 0; d < D; ++d) {
          const float q0 = qs[i * DP + d], q1 = qs[i1 * DP + d], k0 = ks[j * DP + d], k1 = ks[j1 * DP + d];
          s00 = fmaf(q0, k0, s00); s01 = fmaf(q0, k1, s01); s10 = fmaf(q1, k0, s10); s11 = fmaf(q1, k1, s11);
        }
        A[i * C + j] = j <= i ? s00 * pw[i - j] : 0.f;
        if (j + 1 < n) A[i * C + j + 1] = j + 1 <= i ? s01 * pw[i - j - 1] : 0.f;
        if (i + 1 < n) {
          A[(i + 1) * C + j] = s10 * pw[i + 1 - j];
          if (j + 1 < n) A[(i + 1) * C + j + 1] = j + 1 <= i + 1 ? s11 * pw[i - j] : 0.f;
        }
      }
    }
    __syncthreads();
    if ((V & 3) == 0) {
      // outputs and state: a thread takes four neighbouring columns (one 16-byte load of S or v per step)
      const int V4 = V >> 2;
      for (int e = threadIdx.x; e < n * V4; e += blockDim.x) {
        const int i = e / V4, c = (e - i * V4) * 4;
        float4 carried = make_float4(0.f, 0.f, 0.f, 0.f), inside = carried;
        for (int d = 0; d < D; ++d) {
          const float qv = qs[i * DP + d];
          const float4 sv = *reinterpret_cast<const float4*>(S + d * V + c);
          carried.x = fmaf(qv, sv.x, carried.x); carried.y = fmaf(qv, sv.y, carried.y);
          carried.z = fmaf(qv, sv.z, carried.z); carried.w = fmaf(qv, sv.w, carried.w);
        }
        for (int j = 0; j <= i; ++j) {
          const float av = A[i * C + j];
          const float4 vv = *reinterpret_cast<const float4*>(vs + j * V + c);
          inside.x = fmaf(av, vv.x, inside.x); inside.y = fmaf(av, vv.y, inside.y);
          inside.z = fmaf(av, vv.z, inside.z); inside.w = fmaf(av, vv.w, inside.w);
        }
        float* dst = a.out + (size_t)(row0 + t0 + i) * a.heads * a.value_dim + head * a.value_dim + col0 + c;
        const float pi = pw[i + 1];
        dst[0] = fmaf(pi, carried.x, inside.x); dst[1] = fmaf(pi, carried.y, inside.y);
        dst[2] = fmaf(pi, carried.z, inside.z); dst[3] = fmaf(pi, carried.w, inside.w);
      }
      __syncthreads();               // every o of the chunk has read the old S
      for (int e = threadIdx.x; e < D * V4; e += blockDim.x) {
        const int d = e / V4, c = (e - d * V4) * 4;
        float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < n; ++j) {
          const float kv = pw[n - 1 - j] * ks[j * DP + d];
          const float4 vv = *reinterpret_cast<const float4*>(vs + j * V + c);
          add.x = fmaf(kv, vv.x, add.x); add.y = fmaf(kv, vv.y, add.y); add.z = fmaf(kv, vv.z, add.z); add.w = fmaf(kv, vv.w, add.w);
        }
        float4* sp = reinterpret_cast<float4*>(S + d * V + c);
        float4 sv = *sp;
        const float pn = pw[n];
        sv.x = fmaf(pn, sv.x, add.x); sv.y = fmaf(pn, sv.y, add.y); sv.z = fmaf(pn, sv.z, add.z); sv.w = fmaf(pn, sv.w, add.w);
        *sp = sv;
      }
    } else {
      for (int e = threadIdx.x; e < n * V; e += blockDim.x) {
        const int i = e / V, c = e - i * V;
        float carried = 0.f, inside = 0.f;
        for (int d = 0; d < D; ++d) carried = fmaf(qs[i * DP + d], S[d * V + c], carried);
        for (int j = 0; j <= i; ++j) inside = fmaf(A[i * C + j], vs[j * V + c], inside);
        a.out[(size_t)(row0 + t0 + i) * a.heads * a.value_dim + head * a.value_dim + col0 + c] = fmaf(pw[i + 1], carried, inside);
      }
      __syncthreads();               // every o of the chunk has read the old S
      for (int e = threadIdx.x; e < D * V; e += blockDim.x) {
        const int d = e / V, c = e - d * V;
        float add = 0.f;
        for (int j = 0; j < n; ++j) add = fmaf(pw[n - 1 - j] * ks[j * DP + d], vs[j * V + c], add);
        S[e] = fmaf(pw[n], S[e], add);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < D * V; e += blockDim.x) state[(size_t)(e / V) * a.value_dim + e % V] = S[e];
}

static inline size_t lin_attn_smem(int D, int V, int C) {
  return sizeof(float) * ((size_t)D * V + 2 * (size_t)C * (D + 1) + 3 + (size_t)C * V + (size_t)C * C + C + 1);
}

}  // namespace tib

using namespace tib;

// The largest chunk (32, 16, 8, 4, 2 or 1 tokens) whose working set fits an SM's shared memory; 0 if none does.
TIB_API int tib_linear_attention_chunk(int key_dim, int value_dim) {
  for (int c = 32; c >= 1; c >>= 1)
    if (lin_attn_smem(key_dim, value_dim, c) <= 227 * 1024) return c;
  return 0;
}

// q, k: [tokens, >= heads * key_dim] and v: [tokens, >= heads * value_dim] with row strides ldq, ldk, ldv (they may be
// slices of one wider row); out: [tokens, heads * value_dim] fp32; state: [slots, heads, key_dim, value_dim] fp32;
// powers: [heads, chunk + 1] fp32, powers[h][m] = lambda_h^m; activation: 0 none, 1 silu on q, k and v.
TIB_API int tib_linear_attention(const void* q, const void* k, const void* v, int64_t ldq, int64_t ldk, int64_t ldv,
                                 float* out, float* state, const float* powers, const int* q_start, const int* slots,
                                 int n_entries, int heads, int key_dim, int value_dim, int chunk, int activation, int dtype,
                                 cudaStream_t stream) {
  if (n_entries == 0) return TIB_OK;
  if (!q || !k || !v || !out || !state || !powers || !q_start || !slots) return TIB_E_ARG;
  if (heads < 1 || key_dim < 1 || value_dim < 1 || chunk < 1 || chunk > 32 || n_entries > 65535) return TIB_E_SIZE;
  LinAttnArgs a;
  a.q_start = q_start; a.slots = slots; a.powers = powers; a.state = state; a.out = out;
  a.ldq = ldq; a.ldk = ldk; a.ldv = ldv;
  a.heads = heads; a.key_dim = key_dim; a.value_dim = value_dim; a.chunk = chunk; a.activation = activation;
  // runs of value columns: halve them (down to 8) while the grid has fewer than two blocks per SM
  int cols = value_dim;
  while (cols >= 16 && cols % 2 == 0 && (int64_t)heads * n_entries * (value_dim / cols) < 2 * 148) cols /= 2;
  a.cols = cols;
  const size_t smem = lin_attn_smem(key_dim, cols, chunk);
  if (smem > 227 * 1024) return TIB_E_SMEM;
  dim3 grid(heads, n_entries, ceil_div(value_dim, cols));
  if (dtype == TIB_F32) {
    auto kern = linear_attention_kernel<float>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    TIB_LAUNCH_DEPENDENT(kern, grid, 256, smem, stream, (const float*)q, (const float*)k, (const float*)v, a);
  } else if (dtype == TIB_BF16) {
    auto kern = linear_attention_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    TIB_LAUNCH_DEPENDENT(kern, grid, 256, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                         (const __nv_bfloat16*)v, a);
  } else {
    return TIB_E_DTYPE;
  }
  return TIB_OK;
}
