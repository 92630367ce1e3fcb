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

template <typename TD> __device__ __forceinline__ void rs_load(const TD* p, float (&v)[4], int vec);
template <> __device__ __forceinline__ void rs_load<float>(const float* p, float (&v)[4], int vec) {
  if (vec == 4) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  else v[0] = p[0];
}
template <> __device__ __forceinline__ void rs_load<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4], int vec) {
  if (vec == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  } else v[0] = __bfloat162float(p[0]);
}
template <typename TO> __device__ __forceinline__ void rs_store(TO* p, const float (&v)[4], int vec);
template <> __device__ __forceinline__ void rs_store<float>(float* p, const float (&v)[4], int vec) {
  if (vec == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}
template <> __device__ __forceinline__ void rs_store<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4], int vec) {
  if (vec == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  } else p[0] = __float2bfloat16_rn(v[0]);
}

// VEC: channels a thread handles at a time (4: sixteen-byte loads and stores; H and the strides are multiples of 4).
template <typename TD, typename TO, int VEC>
__global__ void __launch_bounds__(RS_THREADS)
streams_update_rmsnorm_kernel(float* __restrict__ X, const TD* __restrict__ delta, int n_partials,
                              long long partial_stride, const float* __restrict__ scale, float mult,
                              const float* __restrict__ mix, const float* __restrict__ write_w,
                              const float* __restrict__ read_w, const float* __restrict__ weight,
                              TO* __restrict__ out, const int* __restrict__ rows, int S, int H, float eps,
                              int write_back, int source_rows) {
  extern __shared__ __align__(16) float u_s[];   // [H] what the next branch reads, before the norm
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
  for (int h = threadIdx.x * VEC; h < H; h += RS_THREADS * VEC) {
    float x[RS_MAX_STREAMS][4];
#pragma unroll
    for (int s = 0; s < RS_MAX_STREAMS; ++s)
      if (s < S) rs_load<float>(x_row + (size_t)s * H + h, x[s], VEC);
    float u[4] = {0.f, 0.f, 0.f, 0.f};
    if (del) {
      float y[4] = {0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < n_partials; ++p) {
        float part[4];
        rs_load<TD>(del + (size_t)p * partial_stride + h, part, VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) y[e] += part[e];
      }
      float sc[4] = {1.f, 1.f, 1.f, 1.f};
      if (scale) rs_load<float>(scale + h, sc, VEC);
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] *= scale ? mult * sc[e] : mult;
#pragma unroll
      for (int t = 0; t < RS_MAX_STREAMS; ++t) {
        if (t < S) {
          float v[4];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < RS_MAX_STREAMS; ++s)
              if (s < S) acc = fmaf(mix_s[s * S + t], x[s][e], acc);
            v[e] = fmaf(write_s[t], y[e], acc);
            u[e] = fmaf(read_s[t], v[e], u[e]);
          }
          if (write_back) rs_store<float>(x_row + (size_t)t * H + h, v, VEC);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < RS_MAX_STREAMS; ++t)
        if (t < S) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = fmaf(read_s[t], x[t][e], u[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) { u_s[h + e] = u[e]; sq = fmaf(u[e], u[e], sq); }
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TO* dst = out + (size_t)r * H;
  for (int h = threadIdx.x * VEC; h < H; h += RS_THREADS * VEC) {
    float w[4], y[4];
    rs_load<float>(weight + h, w, VEC);
#pragma unroll
    for (int e = 0; e < VEC; ++e) y[e] = (u_s[h + e] * inv) * w[e];
    rs_store<TO>(dst + h, y, VEC);
  }
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
  const bool vec = H % 4 == 0 && partial_stride % 4 == 0 &&
                   (((uintptr_t)X | (uintptr_t)delta | (uintptr_t)scale | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
#define LSE_RS_ONE(TD, TO, VEC)                                                                                  \
  {                                                                                                              \
    if (smem > 48 * 1024) {                                                                                      \
      static bool configured = false;                                                                            \
      if (!configured) {                                                                                         \
        cudaError_t err = cudaFuncSetAttribute(streams_update_rmsnorm_kernel<TD, TO, VEC>,                       \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);        \
        if (err != cudaSuccess) return (int)err;                                                                 \
        configured = true;                                                                                       \
      }                                                                                                          \
    }                                                                                                            \
    lse_launch(streams_update_rmsnorm_kernel<TD, TO, VEC>, n_rows, RS_THREADS, smem, stream, X, (const TD*)delta, \
               n_partials, partial_stride, scale, mult, mix, write_w, read_w, weight, (TO*)out, rows, S, H, eps, \
               write_back, source_rows);                                                                         \
  }
#define LSE_RS_CASE(TD, TO) { if (vec) LSE_RS_ONE(TD, TO, 4) else LSE_RS_ONE(TD, TO, 1) }
  const bool d32 = delta_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_RS_CASE(float, float)
  else if (d32 && !o32) LSE_RS_CASE(float, __nv_bfloat16)
  else if (!d32 && o32) LSE_RS_CASE(__nv_bfloat16, float)
  else LSE_RS_CASE(__nv_bfloat16, __nv_bfloat16)
#undef LSE_RS_CASE
#undef LSE_RS_ONE
  LSE_LAUNCH_CHECK();
}
