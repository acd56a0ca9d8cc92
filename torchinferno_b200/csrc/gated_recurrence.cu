// An element-wise gated recurrence whose gates read only the current token (the minimal GRU form):
//
//   z_t = sigmoid(a_t + bias_z)                      a, u: two projections of the token
//   c_t = u_t + bias_u + 1/2 where that is >= 0, else sigmoid(u_t + bias_u)
//   S_t = (1 - z_t) * S_(t-1) + z_t * c_t            per channel, S in 32-bit, carried per request
//   out_t = S_t * silu(g_t)                          g: a third projection (null: out_t = S_t)
//
// Everything after the projections is fp32.  The state lives in the cache manager's slots (zero for a new
// request).  The step is affine in S, so a run of tokens composes to S_out = A * S_in + B with A = prod(1 - z),
// and a long portion is cut into runs that are scanned side by side:
//
//   pass 1  every (run, channel) folds its tokens into (A, B)
//   pass 2  every (run, channel) folds the (A, B) of the runs before it onto the request's state, scans its
//           tokens again from there and writes the outputs; the last run leaves the new state
//
// A portion of up to one run (a decoded token above all) takes pass 2 alone.
//
// A thread owns a channel and walks its run token by token; what it reads is two bytes a token, 12 KB apart.  For
// bf16 rows the block therefore first has its whole tile (64 tokens x 128 channels of each projection) copied
// into shared memory by cp.async in 16-byte pieces, all in flight at once, and walks it from there.
#include "mma.cuh"

namespace tib {

struct GruArgs {
  const void* proj; int dtype; int64_t ld;      // rows of the fused projection
  int z_off, u_off, g_off;                      // columns of a, u, g in a row (g_off < 0: no output gate)
  const float* bias_z; const float* bias_u;     // [width] or null
  float* state;                                 // [slots, width]
  const int* q_start; const int* slots;
  void* out; int out_dtype;                     // [tokens, width]
  float* run_a; float* run_b;                   // [entries, runs, width] scratch (null when runs == 1)
  int width, run_len, max_runs;
  int staged;                                   // bf16 tiles through shared memory (blocks of kGruChannels threads)
};

constexpr int kGruChannels = 128, kGruRun = 64;   // the staged tile: channels a block, tokens a run at most

// Copies rows first .. first + n - 1, channels c0 .. c0 + 127 of NSRC projections into tile[token][projection][channel].
template <int NSRC>
__device__ __forceinline__ void gru_stage(const GruArgs& a, __nv_bfloat16* tile, size_t first, int n, int c0) {
  constexpr int PIECES = kGruChannels / 8;
  const __nv_bfloat16* proj = reinterpret_cast<const __nv_bfloat16*>(a.proj);
  for (int e = threadIdx.x; e < n * NSRC * PIECES; e += blockDim.x) {
    const int t = e / (NSRC * PIECES), rem = e - t * (NSRC * PIECES);
    const int src = rem / PIECES, c = (rem - src * PIECES) * 8;
    const int off = src == 0 ? a.z_off : src == 1 ? a.u_off : a.g_off;
    const bool ok = c0 + c < a.width;
    cp_async16(tile + ((size_t)t * NSRC + src) * kGruChannels + c, proj + (first + t) * a.ld + off + (ok ? c0 + c : 0), ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
}
__device__ __forceinline__ void gru_gates_staged(const __nv_bfloat16* tile, int nsrc, int t, float bz, float bu, float& z, float& cand) {
  z = 1.f / (1.f + expf(-(__bfloat162float(tile[((size_t)t * nsrc) * kGruChannels + threadIdx.x]) + bz)));
  const float u = __bfloat162float(tile[((size_t)t * nsrc + 1) * kGruChannels + threadIdx.x]) + bu;
  cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
}

constexpr int kGruAhead = 8;      // tokens whose gates are computed ahead of the serial chain

__device__ __forceinline__ float gru_load(const void* p, int dtype, size_t i) {
  return dtype == TIB_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float gru_sigmoid(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ void gru_gates(const GruArgs& a, size_t row, int c, float bz, float bu, float& z, float& cand) {
  z = gru_sigmoid(gru_load(a.proj, a.dtype, row * a.ld + a.z_off + c) + bz);
  const float u = gru_load(a.proj, a.dtype, row * a.ld + a.u_off + c) + bu;
  cand = u >= 0.f ? u + 0.5f : gru_sigmoid(u);
}

__global__ void __launch_bounds__(128) gated_recurrence_fold_kernel(GruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.z, run = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  const int t0 = run * a.run_len;
  extern __shared__ __align__(16) __nv_bfloat16 gru_tile[];
  if (a.staged) {      // (whole blocks leave together, ahead of the barrier in gru_stage)
    if (t0 >= len || run == (len - 1) / a.run_len) return;
    gru_stage<2>(a, gru_tile, (size_t)(row0 + t0), a.run_len, blockIdx.x * kGruChannels);
  }
  if (c >= a.width || t0 >= len) return;
  const int last_run = (len - 1) / a.run_len;
  if (run == last_run) return;      // (the last run's sum is never read; its place holds the state the step began with)
  if (run == 0)                     // (the last run writes the slot while others may not have read it yet: they read this copy)
    a.run_b[((size_t)entry * a.max_runs + last_run) * a.width + c] = a.state[(size_t)a.slots[entry] * a.width + c];
  const float bz = a.bias_z ? a.bias_z[c] : 0.f, bu = a.bias_u ? a.bias_u[c] : 0.f;
  float A = 1.f, B = 0.f;
  for (int t = t0; t < t0 + a.run_len; t += kGruAhead) {
    // (the gates of several tokens are made side by side; only the two products a token are a chain)
    float z[kGruAhead], cand[kGruAhead];
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      if (t + i >= t0 + a.run_len) continue;
      if (a.staged) gru_gates_staged(gru_tile, 2, t + i - t0, bz, bu, z[i], cand[i]);
      else gru_gates(a, (size_t)(row0 + t + i), c, bz, bu, z[i], cand[i]);
    }
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      if (t + i >= t0 + a.run_len) break;
      A *= (1.f - z[i]);
      B = fmaf(1.f - z[i], B, z[i] * cand[i]);
    }
  }
  const size_t at = ((size_t)entry * a.max_runs + run) * a.width + c;
  a.run_a[at] = A;
  a.run_b[at] = B;
}

__global__ void __launch_bounds__(128) gated_recurrence_scan_kernel(GruArgs a) {
  pdl_wait();
  pdl_trigger();
  const int entry = blockIdx.z, run = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int row0 = a.q_start[entry], len = a.q_start[entry + 1] - row0;
  const int t0 = run * a.run_len;
  extern __shared__ __align__(16) __nv_bfloat16 gru_tile[];
  const int nsrc = a.g_off >= 0 ? 3 : 2;
  if (a.staged) {
    if (t0 >= len) return;
    if (nsrc == 3) gru_stage<3>(a, gru_tile, (size_t)(row0 + t0), min(len - t0, a.run_len), blockIdx.x * kGruChannels);
    else gru_stage<2>(a, gru_tile, (size_t)(row0 + t0), min(len - t0, a.run_len), blockIdx.x * kGruChannels);
  }
  if (c >= a.width || t0 >= len) return;
  const int t1 = min(len, t0 + a.run_len);
  const float bz = a.bias_z ? a.bias_z[c] : 0.f, bu = a.bias_u ? a.bias_u[c] : 0.f;
  float* slot = a.state + (size_t)a.slots[entry] * a.width;
  const int last_run = (len - 1) / a.run_len;
  float S = last_run == 0 ? slot[c] : a.run_b[((size_t)entry * a.max_runs + last_run) * a.width + c];
  for (int r = 0; r < run; ++r) {
    const size_t at = ((size_t)entry * a.max_runs + r) * a.width + c;
    S = fmaf(a.run_a[at], S, a.run_b[at]);
  }
  for (int t = t0; t < t1; t += kGruAhead) {
    float z[kGruAhead], cand[kGruAhead], gate[kGruAhead];
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      if (t + i >= t1) continue;
      const size_t row = (size_t)(row0 + t + i);
      if (a.staged) gru_gates_staged(gru_tile, nsrc, t + i - t0, bz, bu, z[i], cand[i]);
      else gru_gates(a, row, c, bz, bu, z[i], cand[i]);
      gate[i] = 1.f;
      if (a.g_off >= 0) {
        const float g = a.staged ? __bfloat162float(gru_tile[((size_t)(t + i - t0) * nsrc + 2) * kGruChannels + threadIdx.x])
                                 : gru_load(a.proj, a.dtype, row * a.ld + a.g_off + c);
        gate[i] = g / (1.f + expf(-g));
      }
    }
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      if (t + i >= t1) break;
      const size_t row = (size_t)(row0 + t + i);
      S = fmaf(1.f - z[i], S, z[i] * cand[i]);
      const float o = S * gate[i];
      if (a.out_dtype == TIB_F32) reinterpret_cast<float*>(a.out)[row * a.width + c] = o;
      else reinterpret_cast<__nv_bfloat16*>(a.out)[row * a.width + c] = __float2bfloat16_rn(o);
    }
  }
  if (t1 == len) slot[c] = S;
}

}  // namespace tib

using namespace tib;

// proj: [tokens, ld] rows in `dtype`; out: [tokens, width] in out_dtype; state: [slots, width] fp32;
// run_a / run_b: [n_entries, runs, width] fp32 each (may be null when every entry fits one run).
TIB_API int tib_gated_recurrence(const void* proj, int dtype, int64_t ld, int z_off, int u_off, int g_off, const float* bias_z,
                                 const float* bias_u, float* state, const int* q_start, const int* slots, void* out,
                                 int out_dtype, float* run_a, float* run_b, int n_entries, int max_q_len, int width, int run_len,
                                 cudaStream_t stream) {
  if (n_entries == 0 || max_q_len == 0) return TIB_OK;
  if (!proj || !state || !q_start || !slots || !out || width < 1 || run_len < 1 || n_entries < 0) return TIB_E_ARG;
  if ((dtype != TIB_F32 && dtype != TIB_BF16) || (out_dtype != TIB_F32 && out_dtype != TIB_BF16)) return TIB_E_DTYPE;
  const int runs = ceil_div(max_q_len, run_len);
  if (runs > 1 && (!run_a || !run_b)) return TIB_E_ARG;
  if (runs > 65535 || n_entries > 65535) return TIB_E_SIZE;
  GruArgs a;
  a.proj = proj; a.dtype = dtype; a.ld = ld; a.z_off = z_off; a.u_off = u_off; a.g_off = g_off; a.bias_z = bias_z;
  a.bias_u = bias_u; a.state = state; a.q_start = q_start; a.slots = slots; a.out = out; a.out_dtype = out_dtype;
  a.run_a = run_a; a.run_b = run_b; a.width = width; a.run_len = run_len; a.max_runs = runs;
  a.staged = dtype == TIB_BF16 && max_q_len > 4 && run_len <= kGruRun && width % 8 == 0 && ld % 8 == 0 && z_off % 8 == 0 &&
             u_off % 8 == 0 && (g_off < 0 || g_off % 8 == 0) && ((uintptr_t)proj & 15) == 0;
  const int threads = a.staged || width >= 128 ? 128 : 32 * ceil_div(width, 32);
  dim3 grid(ceil_div(width, threads), runs, n_entries);
  const size_t tile = sizeof(__nv_bfloat16) * (size_t)run_len * kGruChannels;      // of one projection
  if (runs > 1) TIB_LAUNCH_DEPENDENT(gated_recurrence_fold_kernel, grid, threads, a.staged ? 2 * tile : 0, stream, a);
  TIB_LAUNCH_DEPENDENT(gated_recurrence_scan_kernel, grid, threads, a.staged ? (g_off >= 0 ? 3 : 2) * tile : 0, stream, a);
  return TIB_OK;
}
