// A product per head: out[t][h][n] = gate[t][h] * sum_k a[t][h][k] * w[h](k, n), the heads' matrices
// side by side in one tensor.  It is what folds a per-head up-projection into the queries of an attention
// over a shared latent (w[h] read as [k][n]) and what expands the attended latent into a head's values
// afterwards (w[h] stored [n][k]): the strides of w say which.  float32 accumulation in k order (one chain
// per output, so a row's result does not depend on which other rows are in the launch); operands float32
// or bfloat16, rounded once at the store.  Tiles of 64 x 64 outputs, 16 k at a time, 4 x 4 outputs a thread.
#include "common.cuh"

namespace {
constexpr int HG_TILE = 64, HG_K = 16, HG_THREADS = 256;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(HG_THREADS)
head_gemm_kernel(const TA* __restrict__ a, long long a_t, long long a_h, const TW* __restrict__ w, long long w_h,
                 long long w_k, long long w_n, TO* __restrict__ out, long long o_t, long long o_h,
                 const float* __restrict__ gate, int T, int N, int K) {
  __shared__ float a_s[HG_K][HG_TILE + 4], w_s[HG_K][HG_TILE + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.z, t0 = blockIdx.y * HG_TILE, n0 = blockIdx.x * HG_TILE;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const TA* ah = a + (size_t)h * a_h;
  const TW* wh = w + (size_t)h * w_h;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HG_K) {
    __syncthreads();
    for (int e = threadIdx.x; e < HG_K * HG_TILE; e += HG_THREADS) {
      const int kk = e % HG_K, tt = e / HG_K;     // k fastest: a's rows are contiguous in k
      const int t = t0 + tt, k = k0 + kk;
      a_s[kk][tt] = (t < T && k < K) ? to_f32<TA>(ah[(size_t)t * a_t + k]) : 0.f;
    }
    for (int e = threadIdx.x; e < HG_K * HG_TILE; e += HG_THREADS) {
      int kk, nn;
      if (w_n == 1) { nn = e % HG_TILE; kk = e / HG_TILE; } else { kk = e % HG_K; nn = e / HG_K; }
      const int n = n0 + nn, k = k0 + kk;
      w_s[kk][nn] = (n < N && k < K) ? to_f32<TW>(wh[(size_t)k * w_k + (size_t)n * w_n]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HG_K; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = a_s[kk][ty * 4 + i]; wv[i] = w_s[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
    const float g = gate ? gate[(size_t)t * gridDim.z + h] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)t * o_t + (size_t)h * o_h + n] = from_f32<TO>(acc[i][j] * g);
    }
  }
}
// Few rows (decoding): the matrices are read once, by many warps, with all of a lane's loads in flight together.
// Up to eight rows at a time wait in shared memory as float32.  Two layouts of w:
//   * a column's k values lie side by side (w_k == 1): a warp owns four columns, its lanes split k in pieces of
//     eight (sixteen bytes of bfloat16 a load, a warp reads a column's 512 bytes in one go) and add their parts by
//     shuffles;
//   * a k's columns lie side by side (w_n == 1): a lane owns a column, the block's four warps split k, and the
//     warps' parts are added in warp order through shared memory.
// The order of the sums differs from the tiled kernel's by rounding only.
constexpr int HF_THREADS = 128, HF_ROWS = 8, HF_COLS = 4;

template <typename TW> __device__ __forceinline__ void load_w8(const TW* p, float (&v)[8]);
template <> __device__ __forceinline__ void load_w8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load_w8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 two = *reinterpret_cast<const __nv_bfloat162*>(&words[i]);
    v[2 * i] = __low2float(two);
    v[2 * i + 1] = __high2float(two);
  }
}

// KSIDE: w_k == 1 and aligned for vector loads (grid.x = N / 16 columns a block); else grid.x = N / 32.
template <typename TA, typename TW, typename TO, bool KSIDE>
__global__ void __launch_bounds__(HF_THREADS)
head_gemm_few_kernel(const TA* __restrict__ a, long long a_t, long long a_h, const TW* __restrict__ w, long long w_h,
                     long long w_k, long long w_n, TO* __restrict__ out, long long o_t, long long o_h,
                     const float* __restrict__ gate, int T, int N, int K) {
  extern __shared__ __align__(16) float a_sh[];   // [HF_ROWS][K], then (columns side by side) [4][HF_ROWS][32] parts
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TW* wh = w + (size_t)h * w_h;
  for (int t0 = 0; t0 < T; t0 += HF_ROWS) {
    const int rows = min(HF_ROWS, T - t0);
    __syncthreads();
    // unrolled so that several loads are in flight before the first store waits for its value
#pragma unroll 8
    for (int e = threadIdx.x; e < HF_ROWS * K; e += HF_THREADS) {
      const int r = e / K, k = e % K;
      a_sh[e] = r < rows ? to_f32<TA>(a[(size_t)(t0 + r) * a_t + (size_t)h * a_h + k]) : 0.f;
    }
    __syncthreads();
    if (KSIDE) {
      const int n0 = (blockIdx.x * 4 + warp) * HF_COLS;
      float acc[HF_COLS][HF_ROWS];
#pragma unroll
      for (int c = 0; c < HF_COLS; ++c)
#pragma unroll
        for (int r = 0; r < HF_ROWS; ++r) acc[c][r] = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        float wv[HF_COLS][8];
#pragma unroll
        for (int c = 0; c < HF_COLS; ++c) {
          if (n0 + c < N) load_w8<TW>(wh + (size_t)(n0 + c) * w_n + k, wv[c]);
          else {
#pragma unroll
            for (int i = 0; i < 8; ++i) wv[c][i] = 0.f;
          }
        }
#pragma unroll
        for (int r = 0; r < HF_ROWS; ++r) {
          const float4 lo = *reinterpret_cast<const float4*>(a_sh + r * K + k), hi = *reinterpret_cast<const float4*>(a_sh + r * K + k + 4);
          const float av[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
          for (int c = 0; c < HF_COLS; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[c][r] = fmaf(av[i], wv[c][i], acc[c][r]);
        }
      }
#pragma unroll
      for (int c = 0; c < HF_COLS; ++c)
#pragma unroll
        for (int r = 0; r < HF_ROWS; ++r) {
          float v = acc[c][r];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0 && r < rows && n0 + c < N) {
            const float g = gate ? gate[(size_t)(t0 + r) * gridDim.y + h] : 1.f;
            out[(size_t)(t0 + r) * o_t + (size_t)h * o_h + n0 + c] = from_f32<TO>(v * g);
          }
        }
    } else {
      float* part_s = a_sh + HF_ROWS * K;
      const int n = blockIdx.x * 32 + lane;
      const int per_warp = (K + 3) / 4, k_lo = warp * per_warp, k_hi = min(K, k_lo + per_warp);
      float acc[HF_ROWS];
#pragma unroll
      for (int r = 0; r < HF_ROWS; ++r) acc[r] = 0.f;
      if (n < N) {
        const TW* wp = wh + (size_t)n * w_n;
#pragma unroll 8
        for (int k = k_lo; k < k_hi; ++k) {
          const float wv = to_f32<TW>(wp[(size_t)k * w_k]);
#pragma unroll
          for (int r = 0; r < HF_ROWS; ++r) acc[r] = fmaf(a_sh[r * K + k], wv, acc[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < HF_ROWS; ++r) part_s[(warp * HF_ROWS + r) * 32 + lane] = acc[r];
      __syncthreads();
      for (int e = threadIdx.x; e < HF_ROWS * 32; e += HF_THREADS) {
        const int r = e / 32, c = e % 32;
        if (r < rows && blockIdx.x * 32 + c < N) {
          float v = 0.f;
#pragma unroll
          for (int p = 0; p < 4; ++p) v += part_s[(p * HF_ROWS + r) * 32 + c];
          const float g = gate ? gate[(size_t)(t0 + r) * gridDim.y + h] : 1.f;
          out[(size_t)(t0 + r) * o_t + (size_t)h * o_h + blockIdx.x * 32 + c] = from_f32<TO>(v * g);
        }
      }
    }
  }
}
}  // namespace

// a: element (t, h, k) at t * a_t + h * a_h + k; w: element (h, k, n) at h * w_h + k * w_k + n * w_n;
// out: element (t, h, n) at t * o_t + h * o_h + n; gate: float32 [T][heads] or null.
extern "C" int lse_head_gemm(const void* a, int a_dtype, long long a_t, long long a_h, const void* w, int w_dtype,
                             long long w_h, long long w_k, long long w_n, void* out, int out_dtype, long long o_t,
                             long long o_h, const float* gate, int T, int heads, int N, int K, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || heads > 65535 || N <= 0 || K <= 0) return LSE_ERR_BAD_ARGUMENT;
  dim3 grid((N + HG_TILE - 1) / HG_TILE, (T + HG_TILE - 1) / HG_TILE, heads);
  if (grid.y > 65535) return LSE_ERR_TOO_LARGE;
  const size_t few_smem = (size_t)HF_ROWS * (K + 4 * 32) * sizeof(float);
  const bool few = T <= 32 && few_smem <= 48 * 1024;
  const size_t w_bytes = w_dtype == LSE_DTYPE_BF16 ? 2 : 4;
  const bool k_side = w_k == 1 && K % 8 == 0 && (w_h * w_bytes) % 16 == 0 && (w_n * w_bytes) % 16 == 0 &&
                      ((uintptr_t)w & 15) == 0;
  const dim3 few_grid(k_side ? (N + 4 * HF_COLS - 1) / (4 * HF_COLS) : (N + 31) / 32, heads);
#define LSE_HG_CASE(TA, TW, TO)                                                                                 \
  if (few && k_side)                                                                                            \
    lse_launch(head_gemm_few_kernel<TA, TW, TO, true>, few_grid, HF_THREADS, few_smem, stream, (const TA*)a,    \
               a_t, a_h, (const TW*)w, w_h, w_k, w_n, (TO*)out, o_t, o_h, gate, T, N, K);                        \
  else if (few)                                                                                                 \
    lse_launch(head_gemm_few_kernel<TA, TW, TO, false>, few_grid, HF_THREADS, few_smem, stream, (const TA*)a,   \
               a_t, a_h, (const TW*)w, w_h, w_k, w_n, (TO*)out, o_t, o_h, gate, T, N, K);                        \
  else                                                                                                          \
    lse_launch(head_gemm_kernel<TA, TW, TO>, grid, HG_THREADS, 0, stream, (const TA*)a, a_t, a_h, (const TW*)w,  \
               w_h, w_k, w_n, (TO*)out, o_t, o_h, gate, T, N, K);
  typedef __nv_bfloat16 bf;
  const int code = (a_dtype == LSE_DTYPE_BF16 ? 4 : 0) | (w_dtype == LSE_DTYPE_BF16 ? 2 : 0) | (out_dtype == LSE_DTYPE_BF16 ? 1 : 0);
  switch (code) {
    case 0: LSE_HG_CASE(float, float, float) break;
    case 1: LSE_HG_CASE(float, float, bf) break;
    case 2: LSE_HG_CASE(float, bf, float) break;
    case 3: LSE_HG_CASE(float, bf, bf) break;
    case 4: LSE_HG_CASE(bf, float, float) break;
    case 5: LSE_HG_CASE(bf, float, bf) break;
    case 6: LSE_HG_CASE(bf, bf, float) break;
    default: LSE_HG_CASE(bf, bf, bf) break;
  }
#undef LSE_HG_CASE
  LSE_LAUNCH_CHECK();
}
