// Linear attention with a decay per head, carried from token to token in a float32 state per request:
//     S_t = decay_h * S_(t-1) + k_t v_t^T      (S is [dim][vdim] per head)
//     o_t = S_t^T q_t
// with q, k, v = act(projection) (act: SiLU, or none), and the gated norm that follows it:
//     y = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g)      over the concatenated heads.
//
// The scan kernel walks the rows of one request in order, from the state that earlier steps left in the
// request's slot, and leaves the new state there.  A block owns (request, head, a tile of state columns); a
// thread owns 32 rows of one column of S in registers, so a token costs it 32 updates and a 32-term dot
// product, and the threads that share a column (dim > 32) add their parts by shuffles.  Columns of S are
// independent of one another, which is what lets them be spread over blocks.  Tokens are staged in shared
// memory TT at a time.  Everything is float32: the projections arrive in float32, in bfloat16 or as a
// stack of float32 partial sums, and are activated in float32.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_linear_attention)

namespace {
constexpr int LA_THREADS = 128;
constexpr int LA_TT = 16;        // tokens staged at a time
constexpr int LA_DPT = 32;       // rows of the state that a thread keeps

template <typename TD>
__device__ __forceinline__ float la_load(const TD* p, int n_partials, long long partial_stride) {
  float v = 0.f;
  for (int i = 0; i < n_partials; ++i) v += to_f32<TD>(p[(size_t)i * partial_stride]);
  return v;
}
__device__ __forceinline__ float la_act(float z, int act) { return act == 1 ? z / (1.f + expf(-z)) : z; }

// proj: rows of `ld` values; q of head h at q_off + h * dim, k at k_off + h * dim, v at v_off + h * vdim.
// PARTS threads share a column (PARTS * 32 >= dim), CW = 32 / PARTS columns a warp, 4 * CW a block.
template <typename TD, int PARTS>
__global__ void __launch_bounds__(LA_THREADS)
linear_attention_scan_kernel(const TD* __restrict__ proj, int n_partials, long long partial_stride, long long ld,
                             int q_off, int k_off, int v_off, const float* __restrict__ decay,
                             float* __restrict__ state, const int* __restrict__ segment_start,
                             const int* __restrict__ segment_slot, float* __restrict__ out, int heads, int dim,
                             int vdim, int act, int num_slots) {
  constexpr int CW = 32 / PARTS;
  constexpr int CB = 4 * CW;
  constexpr int QS = PARTS * (LA_DPT + 1);          // a token's q (or k) in shared memory: parts padded apart
  __shared__ float q_s[LA_TT * QS], k_s[LA_TT * QS], v_s[LA_TT * CB];
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * CB;
  const int row0 = segment_start[seg], row1 = segment_start[seg + 1];
  if (row1 <= row0) return;
  const int slot = LSE_CHECKED(segment_slot[seg], 0, num_slots, 0, LSE_CHECK_ROW);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane / CW, cb = warp * CW + lane % CW, col = col0 + cb;
  const float dk = decay[h];
  float* st = state + ((size_t)slot * heads + h) * dim * vdim;
  float s[LA_DPT];
#pragma unroll
  for (int i = 0; i < LA_DPT; ++i) {
    const int d = part * LA_DPT + i;
    s[i] = (d < dim && col < vdim) ? st[(size_t)d * vdim + col] : 0.f;
  }
  for (int base = row0; base < row1; base += LA_TT) {
    const int n = min(LA_TT, row1 - base);
    __syncthreads();
    for (int e = threadIdx.x; e < n * PARTS * LA_DPT; e += LA_THREADS) {
      const int t = e / (PARTS * LA_DPT), d = e % (PARTS * LA_DPT);
      float qv = 0.f, kv = 0.f;
      if (d < dim) {
        const TD* row = proj + (size_t)(base + t) * ld;
        qv = la_act(la_load(row + q_off + h * dim + d, n_partials, partial_stride), act);
        kv = la_act(la_load(row + k_off + h * dim + d, n_partials, partial_stride), act);
      }
      const int at = t * QS + (d / LA_DPT) * (LA_DPT + 1) + d % LA_DPT;
      q_s[at] = qv;
      k_s[at] = kv;
    }
    for (int e = threadIdx.x; e < n * CB; e += LA_THREADS) {
      const int t = e / CB, c = e % CB;
      float vv = 0.f;
      if (col0 + c < vdim)
        vv = la_act(la_load(proj + (size_t)(base + t) * ld + v_off + h * vdim + col0 + c, n_partials, partial_stride), act);
      v_s[t * CB + c] = vv;
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float* qr = q_s + t * QS + part * (LA_DPT + 1);
      const float* kr = k_s + t * QS + part * (LA_DPT + 1);
      const float vv = v_s[t * CB + cb];
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < LA_DPT; ++i) {
        s[i] = fmaf(dk, s[i], kr[i] * vv);
        o = fmaf(s[i], qr[i], o);
      }
#pragma unroll
      for (int off = CW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (part == 0 && col < vdim) out[(size_t)(base + t) * heads * vdim + h * vdim + col] = o;
    }
  }
#pragma unroll
  for (int i = 0; i < LA_DPT; ++i) {
    const int d = part * LA_DPT + i;
    if (d < dim && col < vdim) st[(size_t)d * vdim + col] = s[i];
  }
}

// out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * weight * sigmoid(g[t]); g: columns g_off .. g_off + n of proj.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, const TD* __restrict__ proj, int n_partials, long long partial_stride,
                     long long ld, int g_off, const float* __restrict__ weight, TO* __restrict__ out, int n, float eps,
                     const int* __restrict__ segment_of_token) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (segment_of_token && segment_of_token[t] < 0) return;
  const float* row = o + (size_t)t * n;
  float sq = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)n + eps);
  const TD* g = proj + (size_t)t * ld + g_off;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gate = 1.f / (1.f + expf(-la_load(g + i, n_partials, partial_stride)));
    out[(size_t)t * n + i] = from_f32<TO>(((row[i] * inv) * weight[i]) * gate);
  }
}
}  // namespace

// grid: one block row per request of the step (max_segments), empty requests leave at once.
extern "C" int lse_linear_attention_scan(const void* proj, int proj_dtype, int n_partials, long long partial_stride,
                                         long long ld, int q_off, int k_off, int v_off, const float* decay,
                                         float* state, const int* segment_start, const int* segment_slot, float* out,
                                         int max_segments, int heads, int dim, int vdim, int act, int num_slots,
                                         cudaStream_t stream) {
  if (max_segments <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > 8 * LA_DPT || heads > 65535) return LSE_ERR_BAD_ARGUMENT;
  int parts = 1;
  while (parts * LA_DPT < dim) parts <<= 1;
#define LSE_LA_CASE(TD, P)                                                                                       \
  {                                                                                                              \
    const int cb = 4 * (32 / P);                                                                                 \
    dim3 grid(max_segments, heads, (vdim + cb - 1) / cb);                                                        \
    lse_launch(linear_attention_scan_kernel<TD, P>, grid, LA_THREADS, 0, stream, (const TD*)proj, n_partials,    \
               partial_stride, ld, q_off, k_off, v_off, decay, state, segment_start, segment_slot, out, heads,   \
               dim, vdim, act, num_slots);                                                                       \
  }
#define LSE_LA_PARTS(TD)                                  \
  switch (parts) {                                        \
    case 1: LSE_LA_CASE(TD, 1) break;                     \
    case 2: LSE_LA_CASE(TD, 2) break;                     \
    case 4: LSE_LA_CASE(TD, 4) break;                     \
    default: LSE_LA_CASE(TD, 8) break;                    \
  }
  if (proj_dtype == LSE_DTYPE_F32) { LSE_LA_PARTS(float) }
  else if (proj_dtype == LSE_DTYPE_BF16) { LSE_LA_PARTS(__nv_bfloat16) }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_LA_PARTS
#undef LSE_LA_CASE
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_gated_rmsnorm(const float* o, const void* proj, int proj_dtype, int n_partials,
                                 long long partial_stride, long long ld, int g_off, const float* weight, void* out,
                                 int out_dtype, int tokens, int n, float eps, const int* segment_of_token,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0) return LSE_ERR_BAD_ARGUMENT;
#define LSE_GN_CASE(TD, TO)                                                                                   \
  lse_launch(gated_rmsnorm_kernel<TD, TO>, tokens, 256, 0, stream, o, (const TD*)proj, n_partials,            \
             partial_stride, ld, g_off, weight, (TO*)out, n, eps, segment_of_token);
  const bool d32 = proj_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (d32 && o32) LSE_GN_CASE(float, float)
  else if (d32 && !o32) LSE_GN_CASE(float, __nv_bfloat16)
  else if (!d32 && o32) LSE_GN_CASE(__nv_bfloat16, float)
  else LSE_GN_CASE(__nv_bfloat16, __nv_bfloat16)
#undef LSE_GN_CASE
  LSE_LAUNCH_CHECK();
}
