// Attention over a cached latent on the tensor cores (bfloat16 storage, float32 scores, softmax and sums):
// the serving-precision form of attention_latent.cu's kernel, same arguments, same result up to rounding.
//
// All heads of a token read the same cached rows, so the rows of a block's score tile are (token, head) pairs of
// one request: 32 rows = as many consecutive tokens of a portion as 32 / heads allows, times the heads (a single
// decoded token fills `heads` rows; more than 32 heads are spread over blockIdx.y).  A block walks the request's
// keys in tiles of 64 rows of the cache, brought in page by page with cp.async into two buffers in turn:
//   scores   S[32][64] = Q[32][DK] K^T        mma.sync m16n8k16, warp w owns keys 8w .. 8w+7
//   softmax  per row over the tile, float32: running maximum m and sum l, the factor exp(m_old - m_new)
//   output   O[32][DV] = O * factor + P[32][64] V[64][DV]     warp w owns DV / 8 columns; P rounded to bfloat16 for
//            the product, V the first DV columns of the very rows that were the keys
// With few rows (decoding) every chunk of 256 keys has a block of its own (blockIdx.z) that leaves O, m and l of
// its chunk in the layout of attention_latent.cu's split kernel, whose merge kernel adds the chunks up and lets
// the sink join the denominator.  With many rows a block walks all its keys and finishes the row itself.
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_attention_latent_mma)

namespace {
constexpr int ROWS = 32, KEYS = 64, THREADS = 256, CHUNK = 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;   // 0: the sixteen bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared memory, in bytes from the start: two key buffers [KEYS][DK + 8] bf16, the queries [ROWS][DK + 8] bf16,
// the probabilities [ROWS][KEYS + 8] bf16, the scores [ROWS][KEYS + 4] float, per row m, l, factor (float) and
// position (int), per key of a tile the element offset of its cache row (long long).
struct Layout {
  int dks;
  size_t k_bytes, q_at, p_at, s_at, stat_at, off_at, total;
  __host__ __device__ explicit Layout(int DK) {
    dks = DK + 8;
    k_bytes = (size_t)KEYS * dks * 2;
    q_at = 2 * k_bytes;
    p_at = q_at + (size_t)ROWS * dks * 2;
    s_at = p_at + (size_t)ROWS * (KEYS + 8) * 2;
    stat_at = s_at + (size_t)ROWS * (KEYS + 4) * 4;
    off_at = (stat_at + (size_t)ROWS * 4 * 4 + 15) / 16 * 16;
    total = off_at + (size_t)KEYS * 8;
  }
};

// NT: tiles of 8 output columns a warp owns (8 warps * NT * 8 >= DV).
template <int NT>
__global__ void __launch_bounds__(THREADS, 1)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ block_tables, int bt_stride,
                            const int* __restrict__ segment_start, const int* __restrict__ segment_first_position,
                            const float* __restrict__ sink, int num_segments, int n_q, int DK, int DV, int page_size,
                            float scale, int num_pages, float* __restrict__ partials, int max_chunks,
                            int tokens_per_tile, int heads_per_block) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int tile_slot[3];
  pdl_launch_dependents();
  pdl_wait();
  const Layout lay(DK);
  const int dks = lay.dks;
  __nv_bfloat16* q_s = (__nv_bfloat16*)(smem + lay.q_at);
  __nv_bfloat16* p_s = (__nv_bfloat16*)(smem + lay.p_at);
  float* s_s = (float*)(smem + lay.s_at);
  float* m_s = (float*)(smem + lay.stat_at);
  float* l_s = m_s + ROWS;
  float* f_s = l_s + ROWS;
  int* pos_s = (int*)(f_s + ROWS);
  long long* off_s = (long long*)(smem + lay.off_at);
  constexpr int PS = KEYS + 8, SS = KEYS + 4;

  int seg, r0, cnt;
  lse_find_tile(segment_start, num_segments, tokens_per_tile, 0, (int)blockIdx.x, tile_slot, seg, r0, cnt);
  if (seg < 0) return;
  const bool split = partials != nullptr;
  const int tile_tokens = min(tokens_per_tile, cnt - r0);
  const int first_row = segment_start[seg] + r0;                  // the tile's first token among the step's rows
  const int first_pos = segment_first_position[seg] + r0;
  const int ctx = first_pos + tile_tokens;                        // keys that the tile's last token sees
  const int h0 = blockIdx.y * heads_per_block;
  const int heads_here = min(heads_per_block, n_q - h0);
  int key_lo = 0, key_hi = ctx;
  if (split) {
    key_lo = blockIdx.z * CHUNK;
    key_hi = min(ctx, key_lo + CHUNK);
    if (key_lo >= ctx) return;
  }
  const int* bt = block_tables + (size_t)seg * bt_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunks_per_row = DK >> 3;                             // 16-byte pieces of a row

  if (tid < ROWS) {
    const int tok = tid / heads_per_block, hh = tid % heads_per_block;
    pos_s[tid] = (tok < tile_tokens && hh < heads_here) ? first_pos + tok : -1;
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  for (int e = tid; e < ROWS * chunks_per_row; e += THREADS) {
    const int r = e / chunks_per_row, c = e % chunks_per_row;
    const int tok = r / heads_per_block, hh = r % heads_per_block;
    const bool valid = tok < tile_tokens && hh < heads_here;
    const __nv_bfloat16* src = valid ? q + ((size_t)(first_row + tok) * n_q + h0 + hh) * DK + c * 8 : q;
    cp_async16(smem_u32(q_s + (size_t)r * dks + c * 8), src, valid);
  }
  auto load_keys = [&](int base, int buffer) {    // keys base .. base + KEYS - 1 (zeros beyond key_hi)
    __syncthreads();                              // off_s of the tile before has been used
    if (tid < KEYS) {
      const int j = base + tid;
      long long off = -1;
      if (j < key_hi) {
        const int page = LSE_CHECKED(bt[j / page_size], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
        off = ((long long)page * page_size + (j % page_size)) * DK;
      }
      off_s[tid] = off;
    }
    __syncthreads();
    __nv_bfloat16* dst = (__nv_bfloat16*)(smem + (size_t)buffer * lay.k_bytes);
    for (int e = tid; e < KEYS * chunks_per_row; e += THREADS) {
      const int j = e / chunks_per_row, c = e % chunks_per_row;
      const long long off = off_s[j];
      cp_async16(smem_u32(dst + (size_t)j * dks + c * 8), off >= 0 ? cache + off + c * 8 : cache, off >= 0);
    }
    cp_async_commit();
  };

  float acc[2][NT][4];
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mi][nt][i] = 0.f;

  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
  const int col_base = warp * NT * 8;
  const int first_tile = key_lo / KEYS, last_tile = (key_hi - 1) / KEYS;
  load_keys(first_tile * KEYS, 0);
  for (int tile = first_tile; tile <= last_tile; ++tile) {
    const int buffer = (tile - first_tile) & 1;
    cp_async_wait_all();
    __syncthreads();             // the tile (and, the first time, the queries) has landed; the tile before is used up
    if (tile < last_tile) load_keys((tile + 1) * KEYS, buffer ^ 1);
    const uint32_t k_addr = smem_u32(smem + (size_t)buffer * lay.k_bytes);
    const int base = tile * KEYS;
    // ---- scores of keys 8 * warp .. + 7 against all 32 rows
    {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t b_lane = k_addr + (uint32_t)(((warp * 8 + (lane & 7)) * dks + ((lane >> 3) & 1) * 8) * 2);
      const uint32_t a_lane = q_addr + (uint32_t)((a_row * dks + a_col) * 2);
      for (int ks = 0; ks < DK; ks += 16) {
        uint32_t a0[4], a1[4], b[2];
        ldmatrix_x4(a0, a_lane + ks * 2);
        ldmatrix_x4(a1, a_lane + (16 * dks + ks) * 2);
        ldmatrix_x2(b, b_lane + ks * 2);
        mma_bf16(s[0], a0, b[0], b[1]);
        mma_bf16(s[1], a1, b[0], b[1]);
      }
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = mi * 16 + (lane >> 2) + (i >> 1) * 8, c = warp * 8 + (lane & 3) * 2 + (i & 1);
          const int j = base + c;
          s_s[r * SS + c] = (j <= pos_s[r] && j >= key_lo && j < key_hi) ? s[mi][i] * scale : -INFINITY;
        }
    }
    __syncthreads();
    // ---- softmax of the tile: eight threads a row, eight keys each
    {
      const int r = tid >> 3, c0 = (tid & 7) * 8;
      float v[8], top = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[i] = s_s[r * SS + c0 + i]; top = fmaxf(top, v[i]); }
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
      top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 4));
      const float m_old = m_s[r], l_old = l_s[r];
      const float m_new = fmaxf(m_old, top);
      float factor = 1.f, sum = 0.f;
      if (m_new == -INFINITY) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      } else {
        factor = __expf(m_old - m_new);
#pragma unroll
        for (int i = 0; i < 8; ++i) { v[i] = __expf(v[i] - m_new); sum += v[i]; }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      uint32_t packed[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        packed[i] = *reinterpret_cast<uint32_t*>(&two);
      }
      *reinterpret_cast<uint4*>(p_s + r * PS + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      __syncwarp();
      if ((tid & 7) == 0) { m_s[r] = m_new; l_s[r] = l_old * factor + sum; f_s[r] = factor; }
    }
    __syncthreads();
    // ---- O = O * factor + P V for this warp's columns
    {
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        const float f_lo = f_s[mi * 16 + (lane >> 2)], f_hi = f_s[mi * 16 + (lane >> 2) + 8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          acc[mi][nt][0] *= f_lo; acc[mi][nt][1] *= f_lo;
          acc[mi][nt][2] *= f_hi; acc[mi][nt][3] *= f_hi;
        }
      }
      const uint32_t pa_lane = p_addr + (uint32_t)((a_row * PS + a_col) * 2);
#pragma unroll
      for (int kk = 0; kk < KEYS; kk += 16) {
        uint32_t p0[4], p1[4];
        ldmatrix_x4(p0, pa_lane + kk * 2);
        ldmatrix_x4(p1, pa_lane + (16 * PS + kk) * 2);
        const uint32_t v_lane = k_addr + (uint32_t)(((kk + (lane & 15)) * dks + col_base) * 2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (col_base + nt * 8 < DV) {       // the same for the whole warp
            uint32_t vb[2];
            ldmatrix_x2_trans(vb, v_lane + nt * 16);
            mma_bf16(acc[0][nt], p0, vb[0], vb[1]);
            mma_bf16(acc[1][nt], p1, vb[0], vb[1]);
          }
        }
      }
    }
  }
  __syncthreads();
  // ---- the rows' results
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mi * 16 + (lane >> 2) + half * 8;
      if (pos_s[r] < 0) continue;
      const int tok = r / heads_per_block, head = h0 + r % heads_per_block;
      const size_t row = (size_t)(first_row + tok) * n_q + head;
      if (split) {
        if (pos_s[r] < key_lo) continue;     // the row sees no key of this chunk; the merge does not read it
        float* dst = partials + (row * max_chunks + blockIdx.z) * (DV + 2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int c = col_base + nt * 8 + (lane & 3) * 2;
          if (c < DV) { dst[c] = acc[mi][nt][half * 2]; dst[c + 1] = acc[mi][nt][half * 2 + 1]; }
        }
        if (warp == 0 && (lane & 3) == 0) { dst[DV] = m_s[r]; dst[DV + 1] = l_s[r]; }
      } else {
        float m = m_s[r], l = l_s[r], wa = 1.f;
        if (sink) {
          const float m_new = fmaxf(m, sink[head]);
          wa = __expf(m - m_new);
          l = l * wa + __expf(sink[head] - m_new);
        }
        const float inv = wa / l;
        __nv_bfloat16* dst = out + row * DV;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int c = col_base + nt * 8 + (lane & 3) * 2;
          if (c < DV)
            *reinterpret_cast<__nv_bfloat162*>(dst + c) =
                __floats2bfloat162_rn(acc[mi][nt][half * 2] * inv, acc[mi][nt][half * 2 + 1] * inv);
        }
      }
    }
}

constexpr size_t MMA_MAX_SMEM = 220 * 1024;
}  // namespace

// bfloat16, DK a multiple of 16, DV a multiple of 8 up to 512, the buffers within an SM's shared memory.
extern "C" int lse_latent_attention_mma_supported(int DK, int DV) {
  return (DK > 0 && DK % 16 == 0 && DV > 0 && DV % 8 == 0 && DV <= 512 && DV <= DK && Layout(DK).total <= MMA_MAX_SMEM) ? 1 : 0;
}

// The arguments of lse_latent_attention, with the step's segments instead of its rows' segment numbers.  partials
// (tokens * n_q * max_chunks * (DV + 2) floats): a block per chunk of 256 keys; the caller then runs the merge of
// lse_latent_attention_merge.
extern "C" int lse_latent_attention_mma(const void* q, const void* cache, void* out, const int* block_tables,
                                        int bt_stride, const int* segment_start, const int* segment_first_position,
                                        const float* sink, int tokens, int num_segments, int n_q, int DK, int DV,
                                        int page_size, float scale, int num_pages, float* partials, int max_chunks,
                                        cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (!lse_latent_attention_mma_supported(DK, DV) || n_q <= 0 || page_size <= 0 || num_segments <= 0) return LSE_ERR_BAD_ARGUMENT;
  const int heads_per_block = min(n_q, ROWS);
  const int tokens_per_tile = max(1, ROWS / heads_per_block);
  const int tiles = min(tokens, tokens / tokens_per_tile + num_segments);       // an upper bound
  const bool split = partials != nullptr;
  if (split && (max_chunks <= 0 || max_chunks > 65535 || (long long)max_chunks * CHUNK < (long long)bt_stride * page_size))
    return LSE_ERR_BAD_ARGUMENT;
  dim3 grid(tiles, (n_q + heads_per_block - 1) / heads_per_block, split ? max_chunks : 1);
  const size_t smem = Layout(DK).total;
  const int per_warp = (DV + 63) / 64;
#define LSE_LMMA_CASE(NT)                                                                                          \
  {                                                                                                                \
    static bool configured = false;                                                                                \
    if (!configured) {                                                                                             \
      cudaError_t err = cudaFuncSetAttribute(latent_attention_mma_kernel<NT>,                                      \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_MAX_SMEM);      \
      if (err != cudaSuccess) return (int)err;                                                                     \
      configured = true;                                                                                           \
    }                                                                                                              \
    lse_launch(latent_attention_mma_kernel<NT>, grid, THREADS, smem, stream, (const __nv_bfloat16*)q,              \
               (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, block_tables, bt_stride, segment_start,           \
               segment_first_position, sink, num_segments, n_q, DK, DV, page_size, scale, num_pages, partials,     \
               max_chunks, tokens_per_tile, heads_per_block);                                                      \
  }
  if (per_warp <= 1) LSE_LMMA_CASE(1)
  else if (per_warp <= 2) LSE_LMMA_CASE(2)
  else if (per_warp <= 4) LSE_LMMA_CASE(4)
  else LSE_LMMA_CASE(8)
#undef LSE_LMMA_CASE
  LSE_LAUNCH_CHECK();
}
