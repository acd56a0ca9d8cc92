// Layer norm with weight and bias, in the places a block with norms before and after each sublayer needs it, and
// the weighted sum over the outputs of all earlier layers (a depth average) that such a block may end with.
//
//   y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b
//
// Mean, squared deviations, the scaling and every sum into the residual are fp32: a row is read once into shared
// memory as floats, the mean is taken, then the deviations from it (two passes over the staged row, not the
// one-pass E[x^2] - E[x]^2 form, which loses digits when the mean is large).
//
//   layernorm          out[i] = LN(x[rows ? rows[i] : i])                   x: fp32 residual or activation rows
//   layernorm_add      residual[i] += LN_a(y[i]);  optionally out[i] = LN_b(residual[i])
//   depth_average      next[i] = sum_{j < count} coef[j] * history[j][i], written to history[count][i];
//                      optionally out[i] = LN_b(next[i]).  With y given it first does residual += LN_a(y) on
//                      history[count - 1] (the running layer's stream), so the tail of a layer is one launch.
//
// One block per row.  Rows wider than the staged limit are refused.
#include "common.cuh"

namespace tib {

constexpr int kLnMaxWidth = 16384;      // floats of one staged row (64 KB)

__device__ __forceinline__ float ln_load(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void ln_store(void* p, int dtype, size_t i, float v) {
  if (dtype == TIB_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// mean and 1 / sqrt(variance + eps) of the staged row
__device__ __forceinline__ void ln_stats(const float* row, int width, float eps, float* scratch, float& mean, float& inv) {
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) s += row[c];
  mean = block_sum(s, scratch) / (float)width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row[c] - mean;
    ss = fmaf(d, d, ss);
  }
  inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
}

struct LnTail {
  // residual[i] += LN(y[i]; wa, ba)      (y null: skipped)
  const void* y; int y_dtype; int64_t ldy; const float* wa; const float* ba;
  float* residual;                       // [n, width] fp32 (for the depth average: history[count - 1])
  // next = sum_j coef[j] history[j]     (history null: skipped, next = residual)
  float* history; int64_t slice; const float* coef; int count;
  // out[i] = LN(next[i]; wb, bb)        (out null: skipped)
  const float* wb; const float* bb; void* out; int out_dtype;
  int width; float eps;
};

__global__ void __launch_bounds__(256) layernorm_tail_kernel(LnTail a) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const size_t i = blockIdx.x;
  const int width = a.width;
  float mean, inv;
  if (a.y) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = ln_load(a.y, a.y_dtype, i * a.ldy + c);
    __syncthreads();
    ln_stats(row, width, a.eps, scratch, mean, inv);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float v = a.residual[i * width + c] + ((row[c] - mean) * inv * a.wa[c] + a.ba[c]);
      a.residual[i * width + c] = v;
      row[c] = v;
    }
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = a.residual[i * width + c];
  }
  if (a.history) {
    // (the newest output, history[count - 1], is the row at hand)
    float* next = a.history + (size_t)a.count * a.slice + i * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float v = 0.f;
      for (int j = 0; j + 1 < a.count; ++j) v = fmaf(a.coef[j], a.history[(size_t)j * a.slice + i * width + c], v);
      v = fmaf(a.coef[a.count - 1], row[c], v);
      next[c] = v;
      row[c] = v;
    }
  }
  if (!a.out) return;
  __syncthreads();
  ln_stats(row, width, a.eps, scratch, mean, inv);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    ln_store(a.out, a.out_dtype, i * width + c, (row[c] - mean) * inv * a.wb[c] + a.bb[c]);
}

__global__ void __launch_bounds__(256)
layernorm_kernel(const void* __restrict__ x, int x_dtype, int64_t ldx, const int* __restrict__ rows, const float* __restrict__ w,
                 const float* __restrict__ b, float eps, void* __restrict__ out, int out_dtype, int width) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const size_t i = blockIdx.x;
  const size_t src = rows ? (size_t)rows[i] : i;
  for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = ln_load(x, x_dtype, src * ldx + c);
  __syncthreads();
  float mean, inv;
  ln_stats(row, width, eps, scratch, mean, inv);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    ln_store(out, out_dtype, i * width + c, (row[c] - mean) * inv * w[c] + b[c]);
}

static inline int ln_threads(int width) { return width >= 2048 ? 256 : width >= 512 ? 128 : 64; }

}  // namespace tib

using namespace tib;

// x: [*, width] rows (row stride ldx) in x_dtype; rows: [n] int32 or null; out: [n, width] in out_dtype.
TIB_API int tib_layernorm(const void* x, int x_dtype, int64_t ldx, const int* rows, const float* w, const float* b, float eps,
                          void* out, int out_dtype, int n, int width, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!x || !w || !b || !out || n < 0 || width < 1) return TIB_E_ARG;
  if (width > kLnMaxWidth) return TIB_E_SIZE;
  if ((x_dtype != TIB_F32 && x_dtype != TIB_BF16) || (out_dtype != TIB_F32 && out_dtype != TIB_BF16)) return TIB_E_DTYPE;
  const size_t smem = sizeof(float) * (size_t)width;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  TIB_LAUNCH_DEPENDENT(layernorm_kernel, n, ln_threads(width), smem, stream, x, x_dtype, ldx, rows, w, b, eps, out, out_dtype, width);
  return TIB_OK;
}

// The tail of a sublayer or of a layer (see the head of this file).  y: [n, width] rows (row stride ldy) or null;
// residual: [n, width] fp32; history: [depth, n, width] fp32 or null, with residual == history[count - 1] and
// count + 1 <= depth; coef: [count] fp32; out: [n, width] or null.
TIB_API int tib_layernorm_tail(const void* y, int y_dtype, int64_t ldy, const float* wa, const float* ba, float* residual,
                               float* history, int64_t slice, const float* coef, int count, const float* wb, const float* bb,
                               void* out, int out_dtype, int n, int width, float eps, cudaStream_t stream) {
  if (n == 0) return TIB_OK;
  if (!residual || n < 0 || width < 1) return TIB_E_ARG;
  if (y && (!wa || !ba)) return TIB_E_ARG;
  if (out && (!wb || !bb)) return TIB_E_ARG;
  if (history && (!coef || count < 1 || residual != history + (size_t)(count - 1) * slice)) return TIB_E_ARG;
  if (width > kLnMaxWidth) return TIB_E_SIZE;
  if (y && y_dtype != TIB_F32 && y_dtype != TIB_BF16) return TIB_E_DTYPE;
  if (out && out_dtype != TIB_F32 && out_dtype != TIB_BF16) return TIB_E_DTYPE;
  LnTail a;
  a.y = y; a.y_dtype = y_dtype; a.ldy = ldy; a.wa = wa; a.ba = ba; a.residual = residual;
  a.history = history; a.slice = slice; a.coef = coef; a.count = count;
  a.wb = wb; a.bb = bb; a.out = out; a.out_dtype = out_dtype; a.width = width; a.eps = eps;
  const size_t smem = sizeof(float) * (size_t)width;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(layernorm_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  TIB_LAUNCH_DEPENDENT(layernorm_tail_kernel, n, ln_threads(width), smem, stream, a);
  return TIB_OK;
}
