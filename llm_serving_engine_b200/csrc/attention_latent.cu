// Attention over a cached low-rank latent (keys and values of all heads are linear maps of one latent row per
// token, plus one rotated key part that the heads share).
//
// What is cached per token is one row of DK = rank + rot values: the normed latent c (rank values) and the rotated
// shared key part (rot values).  With the per-head key map folded into the query (q'_h = W_uk,h^T q_h, see
// gemm_heads.cu) the score of head h against token j is
//     s = scale * ( q'_h . c_j  +  q_rot,h . k_rot,j )  =  scale * ( [q'_h | q_rot,h] . row_j ),
// and the attended latent sum_j p_j c_j (the first DV = rank values of the rows) is expanded into the head's values
// afterwards.  So the attention itself is a multi-query attention with one shared "head" of keys of width DK whose
// first DV columns are also the values.
//
// Three kernels:
//   * latent_prepare: per row of the step, from the fused down-projection: RMS norm of the query latent (if any),
//     RMS norm of the key/value latent and rotation of the shared key part, both written into the cache row of the
//     token; the per-head output gates sigmoid(g) (if any).
//   * latent_query: sums the query projection's partial sums, copies the unrotated part of every head out and writes
//     the rotated part behind the place where the folded part will go.
//   * latent_attention: the attention proper, any sizes, float32 arithmetic, storage float32 or bfloat16, keys in
//     tiles of 32 and chunks of 256 counted from key 0 (a chunk per block with few rows, merged in order by a second
//     kernel: the same bits either way), with an optional sink per head: a term exp(sink_h) in the softmax's
//     denominator that has no key and no value.
//
// Rotation: the pair (2i, 2i+1), i < rot_dims / 2, by the angle position * freq[i]; cos and sin times `rot_factor`
// (frequency scaling schemes are folded into freq and rot_factor by the host).  The angle is formed and brought into [-pi, pi] in
// double precision, its sine and cosine taken in float32: a float32 product of a position in the thousands and a frequency near one is already off by 1e-4.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_attention_latent)

namespace {
template <typename TD>
__device__ __forceinline__ float lat_load(const TD* p, int n_partials, long long partial_stride) {
  float v = 0.f;
  for (int i = 0; i < n_partials; ++i) v += to_f32<TD>(p[(size_t)i * partial_stride]);
  return v;
}

__device__ __forceinline__ void lat_sincos(int position, double freq, float factor, float& sn, float& cs) {
  double angle = (double)position * freq;
  angle -= 6.283185307179586 * rint(angle * 0.15915494309189535);    // into [-pi, pi], still in double
  float s, c;
  sincosf((float)angle, &s, &c);
  sn = s * factor;
  cs = c * factor;
}

constexpr int PREP_THREADS = 128;

// `width` columns of the row are used (all that the stacked projection has).  staged: the row's partial sums are added
// once, sixteen bytes and eight partial sums a round trip, into shared memory (width floats), and every later pass
// reads it there; else (a row too wide for that) every pass adds them up again from global memory.
template <typename TI, typename TO>
__global__ void __launch_bounds__(PREP_THREADS)
latent_prepare_kernel(const TI* __restrict__ proj, int n_partials, long long partial_stride, long long ld,
                      int q_off, int q_rank, const float* __restrict__ q_norm, TO* __restrict__ q_latent,
                      int kv_off, int rank, const float* __restrict__ kv_norm, int rot, int rot_dims,
                      const double* __restrict__ freq, float rot_factor, const int* __restrict__ positions,
                      const int* __restrict__ slot_mapping, TO* __restrict__ cache, int g_off, int heads,
                      float* __restrict__ gate, float eps, int num_slots, int width, int staged) {
  extern __shared__ float row_s[];
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const TI* row = proj + (size_t)t * ld;
  const int slot = LSE_CHECKED(slot_mapping[t], -1, num_slots, -1, LSE_CHECK_CACHE_SLOT);
  if (staged) {
    for (int c = threadIdx.x; c < width; c += PREP_THREADS) {
      float total = 0.f;
      for (int p0 = 0; p0 < n_partials; p0 += 8) {
        float part[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) part[p] = p0 + p < n_partials ? to_f32<TI>(row[(size_t)(p0 + p) * partial_stride + c]) : 0.f;
#pragma unroll
        for (int p = 0; p < 8; ++p) total += part[p];
      }
      row_s[c] = total;
    }
    __syncthreads();
  }
  auto value = [&](int c) { return staged ? row_s[c] : lat_load(row + c, n_partials, partial_stride); };
  if (q_rank > 0) {
    float sq = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += PREP_THREADS) {
      const float v = value(q_off + i);
      sq = fmaf(v, v, sq);
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += PREP_THREADS)
      q_latent[(size_t)t * q_rank + i] = from_f32<TO>((value(q_off + i) * inv) * q_norm[i]);
  }
  if (gate) {
    for (int h = threadIdx.x; h < heads; h += PREP_THREADS)
      gate[(size_t)t * heads + h] = 1.f / (1.f + expf(-value(g_off + h)));
  }
  if (kv_off >= 0) {
    float sq = 0.f;
    for (int i = threadIdx.x; i < rank; i += PREP_THREADS) {
      const float v = value(kv_off + i);
      sq = fmaf(v, v, sq);
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)rank + eps);
    if (slot < 0) return;    // a padding row: nothing is cached
    TO* dst = cache + (size_t)slot * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += PREP_THREADS)
      dst[i] = from_f32<TO>((value(kv_off + i) * inv) * kv_norm[i]);
    const int position = positions[t];
    const int src = kv_off + rank;
    for (int i = threadIdx.x; i < rot / 2 + (rot & 1); i += PREP_THREADS) {
      const float a = value(src + 2 * i);
      if (2 * i + 1 >= rot) { dst[rank + 2 * i] = from_f32<TO>(a); continue; }
      const float b = value(src + 2 * i + 1);
      if (2 * i + 1 < rot_dims) {
        float sn, cs;
        lat_sincos(position, freq[i], rot_factor, sn, cs);
        dst[rank + 2 * i] = from_f32<TO>(a * cs - b * sn);
        dst[rank + 2 * i + 1] = from_f32<TO>(b * cs + a * sn);
      } else {
        dst[rank + 2 * i] = from_f32<TO>(a);
        dst[rank + 2 * i + 1] = from_f32<TO>(b);
      }
    }
  }
}

// q of head h: columns q_off + h * (dim + rot) .. of the projection: [dim unrotated | rot rotated].
// q_plain [T][heads][dim] gets the unrotated part, q_wide [T][heads][wide] gets the rotated part at column `at`.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
latent_query_kernel(const TI* __restrict__ proj, int n_partials, long long partial_stride, long long ld, int q_off,
                    int heads, int dim, int rot, int rot_dims, const double* __restrict__ freq, float rot_factor,
                    const int* __restrict__ positions, const int* __restrict__ segment_of_token,
                    TO* __restrict__ q_plain, TO* __restrict__ q_wide, int wide, int at) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  if (segment_of_token[t] < 0) return;
  const TI* src = proj + (size_t)t * ld + q_off + (size_t)h * (dim + rot);
  for (int i = threadIdx.x; i < dim; i += blockDim.x)
    q_plain[((size_t)t * heads + h) * dim + i] = from_f32<TO>(lat_load(src + i, n_partials, partial_stride));
  const int position = positions[t];
  TO* dst = q_wide + ((size_t)t * heads + h) * wide + at;
  src += dim;
  for (int i = threadIdx.x; i < rot / 2 + (rot & 1); i += blockDim.x) {
    const float a = lat_load(src + 2 * i, n_partials, partial_stride);
    if (2 * i + 1 >= rot) { dst[2 * i] = from_f32<TO>(a); continue; }
    const float b = lat_load(src + 2 * i + 1, n_partials, partial_stride);
    if (2 * i + 1 < rot_dims) {
      float sn, cs;
      lat_sincos(position, freq[i], rot_factor, sn, cs);
      dst[2 * i] = from_f32<TO>(a * cs - b * sn);
      dst[2 * i + 1] = from_f32<TO>(b * cs + a * sn);
    } else {
      dst[2 * i] = from_f32<TO>(a);
      dst[2 * i + 1] = from_f32<TO>(b);
    }
  }
}

// ------------------------------------------------------------------ the attention
constexpr int KT = 32;        // keys per tile (one warp lane per key)
constexpr int CHUNK = 256;    // keys per chunk (a multiple of KT)
constexpr int GC = 8;         // query heads per block
constexpr int THREADS = 128;  // 4 warps

__device__ __forceinline__ void merge_chunk(float& M, float& L, float m, float l, float& wa, float& wb) {
  const float m_new = fmaxf(M, m);
  wa = expf(M - m_new);    // exp(-inf) = 0 before the first chunk; every chunk of a row has a visible key
  wb = expf(m - m_new);
  L = fmaf(l, wb, L * wa);
  M = m_new;
}
// The sink joins the denominator once, after all keys: returns the factor on the accumulated outputs.
__device__ __forceinline__ float merge_sink(float& M, float& L, float sink) {
  const float m_new = fmaxf(M, sink);
  const float wa = expf(M - m_new);
  L = L * wa + expf(sink - m_new);
  M = m_new;
  return wa;
}

// q [T][n_q][DK]; cache [pages][page_size][DK]; out [T][n_q][DV]; DPT * THREADS >= DV.
// SPLIT: blockIdx.z also numbers the chunk; the block leaves acc [DV], m, l of its chunk and heads in `partials`
// [t][head][chunk][DV + 2].
template <typename T, int DPT, bool SPLIT>
__global__ void __launch_bounds__(THREADS)
latent_attention_kernel(const T* __restrict__ q, const T* __restrict__ cache, T* __restrict__ out,
                        const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ segment_of_token,
                        const int* __restrict__ positions, const float* __restrict__ sink, int n_q, int DK, int DV,
                        int page_size, float scale, int window, int num_pages, int num_segments,
                        float* __restrict__ partials, int max_chunks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int gchunks = (n_q + GC - 1) / GC;
  const int g0 = (SPLIT ? blockIdx.z % gchunks : blockIdx.z) * GC;
  const int gcount = min(GC, n_q - g0);
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0) return;
  const int pos = positions[t];
  const int ctx = pos + 1;
  const int kv_begin = window > 0 ? max(0, ctx - window) : 0;
  int chunk_lo = kv_begin / CHUNK, chunk_hi = pos / CHUNK;
  if (SPLIT) {
    const int mine = blockIdx.z / gchunks;
    if (mine < chunk_lo || mine > chunk_hi) return;
    chunk_lo = chunk_hi = mine;
  }
  const int* bt = block_tables + (size_t)seg * bt_stride;

  long long* base_s = (long long*)smem_raw;   // [KT] element offset of key j's row in the cache, -1 = masked
  float* q_s = (float*)(base_s + KT);      // [GC][DK]
  float* k_s = q_s + GC * DK;              // [KT][DK + 1]
  float* p_s = k_s + KT * (DK + 1);        // [GC][KT]
  float* corr_s = p_s + GC * KT;           // [GC]
  float* l_s = corr_s + GC;                // [GC]
  float* m_s = l_s + GC;                   // [GC]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < gcount * DK; e += THREADS) {
    const int g = e / DK, d = e % DK;
    q_s[g * DK + d] = to_f32<T>(q[((size_t)t * n_q + g0 + g) * DK + d]);
  }

  float total[GC][DPT], M[GC], L[GC];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    M[g] = -INFINITY;
    L[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) total[g][i] = 0.f;
  }

  for (int chunk = chunk_lo; chunk <= chunk_hi; ++chunk) {
    float acc[GC][DPT];
#pragma unroll
    for (int g = 0; g < GC; ++g)
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[g][i] = 0.f;
    float m_run[GC / 4], l_run[GC / 4];
#pragma unroll
    for (int i = 0; i < GC / 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

    const int tile_begin = max(chunk * CHUNK, (kv_begin / KT) * KT);
    const int tile_end = min(ctx, (chunk + 1) * CHUNK);
    for (int base = tile_begin; base < tile_end; base += KT) {
      __syncthreads();  // previous tile fully consumed (also orders the q_s fill)
      if (tid < KT) {
        const int j = base + tid;
        long long off = -1;
        if (j < ctx && j >= kv_begin) {
          const int page = LSE_CHECKED(bt[j / page_size], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
          off = ((long long)page * page_size + (j % page_size)) * DK;
        }
        base_s[tid] = off;
      }
      __syncthreads();
      for (int e = tid; e < KT * DK; e += THREADS) {
        const int j = e / DK, d = e % DK;
        const long long off = base_s[j];
        k_s[j * (DK + 1) + d] = off >= 0 ? to_f32<T>(cache[off + d]) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < GC / 4; ++i) {
        const int g = warp + 4 * i;
        if (g < gcount) {
          const bool valid = base_s[lane] >= 0;
          float s = 0.f;
          const float* qr = q_s + g * DK;
          const float* kr = k_s + lane * (DK + 1);
          for (int d = 0; d < DK; ++d) s = fmaf(qr[d], kr[d], s);
          s = valid ? s * scale : -INFINITY;
          const float m_new = fmaxf(m_run[i], warp_max(s));
          const float c = expf(m_run[i] - m_new);
          const float p = valid ? expf(s - m_new) : 0.f;
          p_s[g * KT + lane] = p;
          float tile_sum = 0.f;  // keys in order, the same in every lane
          for (int j = 0; j < KT; ++j) tile_sum += __shfl_sync(0xffffffffu, p, j);
          l_run[i] = l_run[i] * c + tile_sum;
          m_run[i] = m_new;
          if (lane == 0) { corr_s[g] = c; l_s[g] = l_run[i]; m_s[g] = m_new; }
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = tid + i * THREADS;
        if (d < DV) {
#pragma unroll
          for (int g = 0; g < GC; ++g) {
            if (g < gcount) {
              float a = acc[g][i] * corr_s[g];
              const float* pr = p_s + g * KT;
              for (int j = 0; j < KT; ++j) a = fmaf(pr[j], k_s[j * (DK + 1) + d], a);
              acc[g][i] = a;
            }
          }
        }
      }
    }
    __syncthreads();   // m_s and l_s of the chunk's last tile
    if (SPLIT) {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        if (g < gcount) {
          float* dst = partials + (((size_t)t * n_q + g0 + g) * max_chunks + chunk) * (DV + 2);
#pragma unroll
          for (int i = 0; i < DPT; ++i) {
            const int d = tid + i * THREADS;
            if (d < DV) dst[d] = acc[g][i];
          }
          if (tid == 0) { dst[DV] = m_s[g]; dst[DV + 1] = l_s[g]; }
        }
      }
      return;
    }
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      if (g < gcount) {
        float wa, wb;
        merge_chunk(M[g], L[g], m_s[g], l_s[g], wa, wb);
#pragma unroll
        for (int i = 0; i < DPT; ++i) total[g][i] = fmaf(acc[g][i], wb, total[g][i] * wa);
      }
    }
  }
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    if (g < gcount) {
      const float wa = sink ? merge_sink(M[g], L[g], sink[g0 + g]) : 1.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = tid + i * THREADS;
        if (d < DV) out[((size_t)t * n_q + g0 + g) * DV + d] = from_f32<T>(total[g][i] * wa / L[g]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
latent_attention_merge_kernel(const float* __restrict__ partials, T* __restrict__ out,
                              const int* __restrict__ segment_of_token, const int* __restrict__ positions,
                              const float* __restrict__ sink, int n_q, int DV, int window, int max_chunks,
                              int num_segments) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0) return;
  const int pos = positions[t];
  const int kv_begin = window > 0 ? max(0, pos + 1 - window) : 0;
  const float* src = partials + ((size_t)t * n_q + head) * max_chunks * (DV + 2);
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float total = 0.f, M = -INFINITY, L = 0.f;
    for (int chunk = kv_begin / CHUNK; chunk <= pos / CHUNK; ++chunk) {
      const float* part = src + (size_t)chunk * (DV + 2);
      float wa, wb;
      merge_chunk(M, L, part[DV], part[DV + 1], wa, wb);
      total = fmaf(part[d], wb, total * wa);
    }
    if (sink) total *= merge_sink(M, L, sink[head]);
    out[((size_t)t * n_q + head) * DV + d] = from_f32<T>(total / L);
  }
}

size_t latent_smem_bytes(int DK) {
  return sizeof(float) * ((size_t)GC * DK + (size_t)KT * (DK + 1) + GC * KT + 3 * GC + 1) + sizeof(long long) * KT + 16;
}
constexpr int LATENT_MAX_SMEM = 200 * 1024;
}  // namespace

extern "C" int lse_latent_prepare(const void* proj, int in_dtype, int n_partials, long long partial_stride, long long ld,
                                  int q_off, int q_rank, const float* q_norm, void* q_latent, int kv_off, int rank,
                                  const float* kv_norm, int rot, int rot_dims, const double* freq, float rot_factor,
                                  const int* positions, const int* slot_mapping, void* cache, int out_dtype, int g_off,
                                  int heads, float* gate, float eps, int tokens, int num_slots, int width,
                                  cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims > rot || (rot_dims & 1) || rank < 0 || width <= 0) return LSE_ERR_BAD_ARGUMENT;
  // one set of sums (many rows: a prompt's portion) is read where it lies; a stack of partial sums is added up once
  const int staged = (n_partials > 1 && (size_t)width * sizeof(float) <= 40 * 1024) ? 1 : 0;
  const size_t smem = staged ? (size_t)width * sizeof(float) : 0;
#define LSE_PREP_CASE(TI, TO)                                                                                      \
  lse_launch(latent_prepare_kernel<TI, TO>, tokens, PREP_THREADS, smem, stream, (const TI*)proj, n_partials,      \
             partial_stride, ld, q_off, q_rank, q_norm, (TO*)q_latent, kv_off, rank, kv_norm, rot, rot_dims, freq, \
             rot_factor, positions, slot_mapping, (TO*)cache, g_off, heads, gate, eps, num_slots, width, staged);
  const bool i32 = in_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (i32 && o32) LSE_PREP_CASE(float, float)
  else if (i32 && !o32) LSE_PREP_CASE(float, __nv_bfloat16)
  else if (!i32 && !o32) LSE_PREP_CASE(__nv_bfloat16, __nv_bfloat16)
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_PREP_CASE
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_latent_query(const void* proj, int in_dtype, int n_partials, long long partial_stride, long long ld,
                                int q_off, int heads, int dim, int rot, int rot_dims, const double* freq,
                                float rot_factor, const int* positions, const int* segment_of_token, void* q_plain,
                                void* q_wide, int out_dtype, int wide, int at, int tokens, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims > rot || (rot_dims & 1) || heads <= 0 || heads > 65535) return LSE_ERR_BAD_ARGUMENT;
  dim3 grid(tokens, heads);
#define LSE_LQ_CASE(TI, TO)                                                                                       \
  lse_launch(latent_query_kernel<TI, TO>, grid, 128, 0, stream, (const TI*)proj, n_partials, partial_stride, ld,  \
             q_off, heads, dim, rot, rot_dims, freq, rot_factor, positions, segment_of_token, (TO*)q_plain,       \
             (TO*)q_wide, wide, at);
  const bool i32 = in_dtype == LSE_DTYPE_F32, o32 = out_dtype == LSE_DTYPE_F32;
  if (i32 && o32) LSE_LQ_CASE(float, float)
  else if (i32 && !o32) LSE_LQ_CASE(float, __nv_bfloat16)
  else if (!i32 && !o32) LSE_LQ_CASE(__nv_bfloat16, __nv_bfloat16)
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_LQ_CASE
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_latent_attention_chunk(void) { return CHUNK; }

// The merge alone: adds up the chunks that a split kernel (this file's, or the tensor-core one) left in `partials`.
extern "C" int lse_latent_attention_merge(const float* partials, void* out, int dtype, const int* segment_of_token,
                                          const int* positions, const float* sink, int tokens, int n_q, int DV,
                                          int window, int max_chunks, int num_segments, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n_q <= 0 || n_q > 65535 || DV <= 0 || max_chunks <= 0) return LSE_ERR_BAD_ARGUMENT;
  const dim3 grid(tokens, n_q);
  const int threads = min(256, ((DV + 31) / 32) * 32);
  if (dtype == LSE_DTYPE_F32)
    lse_launch(latent_attention_merge_kernel<float>, grid, threads, 0, stream, partials, (float*)out, segment_of_token,
               positions, sink, n_q, DV, window, max_chunks, num_segments);
  else if (dtype == LSE_DTYPE_BF16)
    lse_launch(latent_attention_merge_kernel<__nv_bfloat16>, grid, threads, 0, stream, partials, (__nv_bfloat16*)out,
               segment_of_token, positions, sink, n_q, DV, window, max_chunks, num_segments);
  else return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// partials != null: a block per chunk of a row, merged by a second kernel (few rows); partials holds
// tokens * n_q * max_chunks * (DV + 2) floats.
extern "C" int lse_latent_attention(const void* q, const void* cache, void* out, int dtype, const int* block_tables,
                                    int bt_stride, const int* segment_of_token, const int* positions,
                                    const float* sink, int tokens, int n_q, int DK, int DV, int page_size, float scale,
                                    int window, int num_pages, int num_segments, float* partials, int max_chunks,
                                    cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (DK <= 0 || DV <= 0 || DV > DK || n_q <= 0 || page_size <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (DV > 4 * THREADS) return LSE_ERR_TOO_LARGE;   // a thread keeps at most four output columns of eight heads
  const size_t smem = latent_smem_bytes(DK);
  if (smem > LATENT_MAX_SMEM) return LSE_ERR_TOO_LARGE;
  const int gchunks = (n_q + GC - 1) / GC;
  const bool split = partials != nullptr;
  if (split && (max_chunks <= 0 || (long long)gchunks * max_chunks > 65535 ||
                (long long)max_chunks * CHUNK < (long long)bt_stride * page_size))
    return LSE_ERR_BAD_ARGUMENT;
  dim3 grid(tokens, 1, split ? gchunks * max_chunks : gchunks);
  const dim3 merge_grid(tokens, n_q);
  const int merge_threads = min(256, ((DV + 31) / 32) * 32);
#define LSE_LAT_ONE(T, DPT, SPLIT)                                                                                 \
  {                                                                                                                \
    static bool configured = false;                                                                                \
    if (!configured) {                                                                                             \
      cudaError_t err = cudaFuncSetAttribute(latent_attention_kernel<T, DPT, SPLIT>,                               \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, LATENT_MAX_SMEM);        \
      if (err != cudaSuccess) return (int)err;                                                                     \
      configured = true;                                                                                           \
    }                                                                                                              \
    lse_launch(latent_attention_kernel<T, DPT, SPLIT>, grid, THREADS, smem, stream, (const T*)q, (const T*)cache,  \
               (T*)out, block_tables, bt_stride, segment_of_token, positions, sink, n_q, DK, DV, page_size, scale, \
               window, num_pages, num_segments, partials, max_chunks);                                             \
  }
#define LSE_LAT_CASE(T, DPT)                                                                                       \
  if (split) {                                                                                                     \
    LSE_LAT_ONE(T, DPT, true)                                                                                      \
    lse_launch(latent_attention_merge_kernel<T>, merge_grid, merge_threads, 0, stream, (const float*)partials,     \
               (T*)out, segment_of_token, positions, sink, n_q, DV, window, max_chunks, num_segments);             \
  } else LSE_LAT_ONE(T, DPT, false)
#define LSE_LAT_DPT(T)                                    \
  if (DV <= THREADS) { LSE_LAT_CASE(T, 1) }               \
  else if (DV <= 2 * THREADS) { LSE_LAT_CASE(T, 2) }      \
  else { LSE_LAT_CASE(T, 4) }
  if (dtype == LSE_DTYPE_F32) { LSE_LAT_DPT(float) }
  else if (dtype == LSE_DTYPE_BF16) { LSE_LAT_DPT(__nv_bfloat16) }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_LAT_DPT
#undef LSE_LAT_CASE
#undef LSE_LAT_ONE
  LSE_LAUNCH_CHECK();
}
