// A residual kept as several copies ("streams", hyper-connections) with scaled branch outputs, fused
// with the RMS norm that feeds the next branch.
//
// The hidden state of a row is X[s][h], s < S copies of width H, float32.  A branch reads a weighted
// sum of the copies and its output y[h] goes back into every copy while the copies are mixed:
//     X'[t][h] = sum_s mix[s][t] X[s][h] + write[t] * (scale[h] * y[h])        (mix is [from][to])
// and the next branch reads
//     u[h] = sum_t read[t] X'[t][h],   out[h] = u[h] / sqrt(mean_h(u^2) + eps) * weight[h].
// One kernel does both steps for a row: the update of the branch before (pending until now) and the
// read and norm of the branch to come.  Absent pieces fall away: no y (first norm of the model), no mix
// (identity), no write weights (ones), no per-channel scale (the scalar `mult` alone), no read weights
// (ones: the sum of the copies, which is also what the model's last norm reads).  With S = 1 this is the
// plain scaled residual x' = x + mult * scale[h] * y.
//
// y may be a stack of float32 partial sums of a split-k product; they are added in index order from zero.
// Everything is float32; the result is rounded once when `out` is bfloat16.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_residual_streams)

namespace {
constexpr int RS_MAX_STREAMS = 8;
constexpr int RS_THREADS = 256;

template <typename TD, typename TO>
__global__ void __launch_bounds__(RS_THREADS)
streams_update_rmsnorm_kernel(float* __restrict__ X, const TD* __restrict__ delta, int n_partials,
                              long long partial_stride, const float* __restrict__ scale, float mult,
                              const float* __restrict__ mix, const float* __restrict__ write_w,
                              const float* __restrict__ read_w, const float* __restrict__ weight,
                              TO* __restrict__ out, const int* __restrict__ rows, int S, int H, float eps,
                              int write_back, int source_rows) {
  extern __shared__ float u_s[];   // [H] what the next branch reads, before the norm
  __shared__ float scratch[32];
  __shared__ float mix_s[RS_MAX_STREAMS * RS_MAX_STREAMS], write_s[RS_MAX_STREAMS], read_s[RS_MAX_STREAMS];
  pdl_launch_dependents();
  // the small tables do not depend on earlier kernels
  if (threadIdx.x < S * S) mix_s[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
  if (threadIdx.x < S) {
    write_s[threadIdx.x] = write_w ? write_w[threadIdx.x] : 1.f;
    read_s[threadIdx.x] = read_w ? read_w[threadIdx.x] : 1.f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const int s_row = rows ? LSE_CHECKED(rows[r], -1, source_rows, -1, LSE_CHECK_ROW) : r;
  if (s_row < 0) return;
  float* x_row = X + (size_t)s_row * S * H;
  const TD* del = delta ? delta + (size_t)s_row * H : nullptr;
  float sq = 0.f;
  for (int h = threadIdx.x; h < H; h += RS_THREADS) {
    float x[RS_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < RS_MAX_STREAMS; ++s) x[s] = s < S ? x_row[(size_t)s * H + h] : 0.f;
    float u = 0.f;
    if (del) {
      float y = 0.f;
      for (int p = 0; p < n_partials; ++p) y += to_f32<TD>(del[(size_t)p * partial_stride + h]);
      y *= scale ? mult * scale[h] : mult;
#pragma unroll
      for (int t = 0; t < RS_MAX_STREAMS; ++t) {
        if (t < S) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < RS_MAX_STREAMS; ++s)
            if (s < S) v = fmaf(mix_s[s * S + t], x[s], v);
          v = fmaf(write_s[t], y, v);
          if (write_back) x_row[(size_t)t * H + h] = v;
          u = fmaf(read_s[t], v, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < RS_MAX_STREAMS; ++t)
        if (t < S) u = fmaf(read_s[t], x[t], u);
    }
    u_s[h] = u;
    sq = fmaf(u, u, sq);
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TO* dst = out + (size_t)r * H;
  for (int h = threadIdx.x; h < H; h += RS_THREADS) dst[h] = from_f32<TO>((u_s[h] * inv) * weight[h]);
}
}  // namespace

// X float32 [source_rows][S][H] (updated in place when write_back); delta [source_rows][H] of delta_dtype, or
// n_partials float32 stacks partial_stride apart, or null; out [n_rows][H]; rows: int32 row numbers or null.
extern "C" int lse_streams_update_rmsnorm(float* X, const void* delta, int delta_dtype, int n_partials,
                                          long long partial_stride, const float* scale, float mult, const float* mix,
                                          const float* write_w, const float* read_w, const float* weight, void* out,
                                          int out_dtype, const int* rows, int n_rows, int S, int H, float eps,
                                          int write_back, int source_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S <= 0 || S > RS_MAX_STREAMS || H <= 0) return LSE_ERR_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * (size_t)H;
  if (smem > 160 * 1024) return LSE_ERR_TOO_LARGE;
#define LSE_RS_CASE(TD, TO)                                                                                      \
  {                                                                                                              \
    if (smem > 48 * 1024) {                                                                                      \
      static bool configured = false;                                                                            \
      if (!configured) {                                                                                         \
        cudaError_t err = cudaFuncSetAttribute(streams_update_rmsnorm_kernel<TD, TO>,                            \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);        \
        if (err != cudaSuccess) return (int)err;                                                                 \
        configured = true;                                                                                       \
      }                                                                                                          \
    }                                                                                                            \
    lse_launch(streams_update_rmsnorm_kernel<TD, TO>, n_rows, RS_THREADS, smem, stream, X, (const TD*)delta,     \
               n_partials, partial_stride, scale, mult, mix, write_w, read_w, weight, (TO*)out, rows, S, H, eps, \
               write_back, source_rows);                                                                         \
  }
  const bool d32 = delta_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_RS_CASE(float, float)
  else if (d32 && !o32) LSE_RS_CASE(float, __nv_bfloat16)
  else if (!d32 && o32) LSE_RS_CASE(__nv_bfloat16, float)
  else LSE_RS_CASE(__nv_bfloat16, __nv_bfloat16)
#undef LSE_RS_CASE
  LSE_LAUNCH_CHECK();
}
