// Attention over a cached latent: per token the cache holds one vector [c | r], c the normed latent
// of `rank` entries from which every head's keys and values are linear maps (k_h = Uk_h c,
// v_h = Uv_h c), r a rotated key part of `rot` entries shared by all heads.  Nothing is expanded per
// cached token: the key map moves to the query side and the value map behind the weighted sum,
//
//   score_h(i, j) = ((Uk_h^T q_h) . c_j + qr_h . r_j) * scale,    o_h = Uv_h (sum_j p_h(i, j) c_j),
//
// so all heads read the same cached vectors (one key/value head of size rank + rot whose first
// `rank` entries are also the value).  The softmax may have a sink: exp(sink_h) joins the
// denominator, with no key and no value.  Scores, weights and sums are float32.
//
// Kernels: latent_prepare (norm of the latent, rotation of r and of the queries' rotated parts,
// cache write), per_head_linear (one small matrix per head applied to every token: the two maps),
// latent_attention (the softmax over the cached vectors).

#include "common.cuh"

#include <math.h>

#define LAT_THREADS 256
#define LAT_WARPS 8
#define LAT_MAX_CH 16      // value entries per lane: rank <= 512

// ------------------------------------------------------------------------------ prepare

// One block per token.  u holds the token's projections: the queries at q_col (per head `dim` plain
// entries, then `rot`), the compressed row at c_col (`rank` entries to norm, then `rot`).
template <typename T, typename TW>
__global__ void __launch_bounds__(LAT_THREADS)
latent_prepare_kernel(const T* __restrict__ u, long long u_stride, int q_col, int c_col, int heads, int dim, int rot,
                      int rank, const TW* __restrict__ norm_w, float eps, const float* __restrict__ inv_freq,
                      int rot_dims, float mag, T* __restrict__ q_full, PagedCache cache,
                      const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = positions[t], seq = row_seq[t];
  const T* row = u + (long long)t * u_stride;
  const int D = rank + rot;
  // the queries' rotated parts, behind the place of the mapped plain parts
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    float sn, cs;
    sincosf((float)pos * inv_freq[p], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const T* x = row + q_col + (long long)h * (dim + rot) + dim;
    const float a = to_float(x[2 * p]), b = to_float(x[2 * p + 1]);
    T* dst = q_full + ((long long)t * heads + h) * D + rank;
    dst[2 * p] = from_float<T>(a * cs - b * sn);
    dst[2 * p + 1] = from_float<T>(b * cs + a * sn);
  }
  for (int i = threadIdx.x; i < heads * (rot - rot_dims); i += blockDim.x) {
    const int h = i / (rot - rot_dims), c = rot_dims + i - h * (rot - rot_dims);
    q_full[((long long)t * heads + h) * D + rank + c] = row[q_col + (long long)h * (dim + rot) + dim + c];
  }
  // the latent and the shared rotated key part
  const T* x = row + c_col;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(x[i]);
    sq += v * v;
  }
  const float scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)rank + eps);
  if (!write_cache) return;
  const long long off = cache_offset(cache, seq, pos, 0);
  if (off < 0) return;
  T* dst = (T*)cache.k + off;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(to_float(x[i]) * scale * to_float(norm_w[i]));
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[p], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const float a = to_float(x[rank + 2 * p]), b = to_float(x[rank + 2 * p + 1]);
    dst[rank + 2 * p] = from_float<T>(a * cs - b * sn);
    dst[rank + 2 * p + 1] = from_float<T>(b * cs + a * sn);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = x[rank + c];
}

extern "C" int llm_latent_prepare(const void* u, int dtype, long long u_stride, int q_col, int c_col, int heads, int dim,
                                  int rot, int rank, const void* norm_w, float eps, const float* inv_freq, int rot_dims,
                                  float mag, void* q_full, void* k_base, const int32_t* block_table, long long page_stride,
                                  int table_stride, int page_tokens, const int32_t* positions, const int32_t* row_seq,
                                  int write_cache, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot && (rot_dims == 0 || inv_freq), ERR_BAD_SIZE);
  PagedCache c{k_base, k_base, block_table, page_stride, table_stride, page_tokens, 1, rank + rot};
  if (dtype == DT_F32)
    launch_kernel(latent_prepare_kernel<float, float>, n_tokens, LAT_THREADS, 0, stream, (const float*)u, u_stride,
                  q_col, c_col, heads, dim, rot, rank, (const float*)norm_w, eps, inv_freq, rot_dims, mag,
                  (float*)q_full, c, positions, row_seq, write_cache);
  else if (dtype == DT_BF16)
    launch_kernel(latent_prepare_kernel<__nv_bfloat16, __nv_bfloat16>, n_tokens, LAT_THREADS, 0, stream,
                  (const __nv_bfloat16*)u, u_stride, q_col, c_col, heads, dim, rot, rank, (const __nv_bfloat16*)norm_w,
                  eps, inv_freq, rot_dims, mag, (__nv_bfloat16*)q_full, c, positions, row_seq, write_cache);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------------ one matrix per head

// out[t, h, o] = sum_i x[t, h, i] * W_h[i, o] for every token t and head h, where head h's matrix is
// rows h * n_in .. of w [heads * n_in, n_out] (W_IN_ROWS: out = x W) or rows h * n_out .. of
// w [heads * n_out, n_in] (out = x W^T).  With `gate`: out *= sigmoid(gate[t, h * n_out + o]).
// A block takes 64 tokens x 64 outputs of one head, a thread 4 x 4 of them; float32 sums in the
// order of i.
#define PH_TILE 64
#define PH_K 16

template <typename T, bool W_IN_ROWS>
__global__ void __launch_bounds__(256)
per_head_linear_kernel(const T* __restrict__ x, long long x_row, long long x_head, const T* __restrict__ w,
                       T* __restrict__ out, long long o_row, long long o_head, const T* __restrict__ gate,
                       long long gate_row, int n_tokens, int n_in, int n_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[PH_K][PH_TILE + 4];
  __shared__ float ws[PH_K][PH_TILE + 4];
  const int h = blockIdx.z, t0 = blockIdx.x * PH_TILE, o0 = blockIdx.y * PH_TILE;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // tx: outputs, ty: tokens
  const T* wh = w + (long long)h * n_in * n_out;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < n_in; k0 += PH_K) {
    for (int e = threadIdx.x; e < PH_K * PH_TILE; e += 256) {
      {  // x tile: neighbouring threads read neighbouring inputs of one token
        const int kk = e % PH_K, tt = e / PH_K;
        const int t = t0 + tt, k = k0 + kk;
        xs[kk][tt] = (t < n_tokens && k < n_in) ? to_float(x[(long long)t * x_row + (long long)h * x_head + k]) : 0.0f;
      }
      if (W_IN_ROWS) {
        const int oo = e % PH_TILE, kk = e / PH_TILE;
        const int o = o0 + oo, k = k0 + kk;
        ws[kk][oo] = (o < n_out && k < n_in) ? to_float(wh[(long long)k * n_out + o]) : 0.0f;
      } else {
        const int kk = e % PH_K, oo = e / PH_K;
        const int o = o0 + oo, k = k0 + kk;
        ws[kk][oo] = (o < n_out && k < n_in) ? to_float(wh[(long long)o * n_in + k]) : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < PH_K; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int o = o0 + tx * 4 + j;
      if (o >= n_out) continue;
      float v = acc[i][j];
      if (gate) v = v / (1.0f + expf(-to_float(gate[(long long)t * gate_row + (long long)h * n_out + o])));
      out[(long long)t * o_row + (long long)h * o_head + o] = from_float<T>(v);
    }
  }
}

extern "C" int llm_per_head_linear(const void* x, long long x_row, long long x_head, const void* w, int w_in_rows,
                                   void* out, long long o_row, long long o_head, const void* gate, long long gate_row,
                                   int dtype, int n_tokens, int heads, int n_in, int n_out, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  dim3 grid((n_tokens + PH_TILE - 1) / PH_TILE, (n_out + PH_TILE - 1) / PH_TILE, heads);
  LLM_HOST_CHECK(grid.y <= 65535 && grid.z <= 65535, ERR_BAD_SIZE);
#define GO(T, IN_ROWS)                                                                                             \
  launch_kernel(per_head_linear_kernel<T, IN_ROWS>, grid, 256, 0, stream, (const T*)x, x_row, x_head, (const T*)w, \
                (T*)out, o_row, o_head, (const T*)gate, gate_row, n_tokens, n_in, n_out)
  if (dtype == DT_F32) { if (w_in_rows) GO(float, true); else GO(float, false); }
  else if (dtype == DT_BF16) { if (w_in_rows) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
  else return ERR_BAD_DTYPE;
#undef GO
  return launch_status();
}

// ------------------------------------------------------------------------------ attention

// Grid (token, group of LAT_WARPS heads).  The block brings 32 cached vectors at a time into shared
// memory (as float32, a warp four of them), and each warp, one head, scores them (a lane one key),
// keeps a running maximum and sum, and adds the weighted first `rank` entries (a lane the entries
// lane, lane + 32, ...).  Key blocks start at multiples of 32 positions, so the order of a row's
// sums depends on positions only.
template <typename T, typename TW>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_kernel(const T* __restrict__ q, T* __restrict__ out, PagedCache cache, int rank,
                        const TW* __restrict__ sink, const int32_t* __restrict__ positions,
                        const int32_t* __restrict__ row_seq, int heads, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float lat_smem[];     // keys [32][D + 1], then q [LAT_WARPS][D]
  const int D = cache.head_dim, ld = D + 1;
  float* keys = lat_smem;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = lat_smem + 32 * ld + warp * D;
  const int t = blockIdx.x, h = blockIdx.y * LAT_WARPS + warp;
  const bool active = h < heads;
  if (active)
    for (int c = lane; c < D; c += 32) qs[c] = to_float(q[((long long)t * heads + h) * D + c]);
  const int pos = positions[t], seq = row_seq[t];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const T* kc = (const T*)cache.k;
  float m = -INFINITY, l = 0.0f;
  float acc[LAT_MAX_CH];
#pragma unroll
  for (int i = 0; i < LAT_MAX_CH; ++i) acc[i] = 0.0f;
  for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
    __syncthreads();      // the last block's keys have been read
    for (int kk = warp; kk < 32; kk += LAT_WARPS) {
      const int j = j0 + kk;
      long long off = -1;
      if (j >= first && j <= pos) off = cache_offset(cache, seq, j, 0);
      float* dst = keys + kk * ld;
      if (off >= 0)
        for (int c = lane; c < D; c += 32) dst[c] = to_float(kc[off + c]);
      if (lane == 0) dst[D] = off >= 0 ? 1.0f : 0.0f;      // the spare entry says whether the key is there
    }
    __syncthreads();
    if (!active) continue;
    const float* mine = keys + lane * ld;
    float s = -INFINITY;
    if (mine[D] != 0.0f) {
      float dot = 0.0f;
      for (int c = 0; c < D; ++c) dot = fmaf(qs[c], mine[c], dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LAT_MAX_CH; ++i) acc[i] *= corr;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      if (pj == 0.0f) continue;
      const float* vj = keys + jj * ld;
#pragma unroll
      for (int i = 0; i < LAT_MAX_CH; ++i) {
        const int c = lane + 32 * i;
        if (c < rank) acc[i] = fmaf(pj, vj[c], acc[i]);
      }
    }
    m = m_new;
  }
  if (!active) return;
  if (sink) {
    const float sk = to_float(sink[h]);
    const float m_new = fmaxf(m, sk);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < LAT_MAX_CH; ++i) acc[i] *= corr;
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
  for (int i = 0; i < LAT_MAX_CH; ++i) {
    const int c = lane + 32 * i;
    if (c < rank) out[((long long)t * heads + h) * rank + c] = from_float<T>(acc[i] * inv);
  }
}

// dtype: element type of q, out, the cache and the sinks.  q [tokens, heads, D = rank + rot], out
// [tokens, heads, rank].
extern "C" int llm_latent_attention(const void* q, void* out, int dtype, void* k_base, const int32_t* block_table,
                                    long long page_stride, int table_stride, int page_tokens, int D, int rank,
                                    const void* sink, const int32_t* positions, const int32_t* row_seq, int heads,
                                    int n_tokens, float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(rank >= 1 && rank <= D && rank <= 32 * LAT_MAX_CH, ERR_BAD_SIZE);
  PagedCache c{k_base, k_base, block_table, page_stride, table_stride, page_tokens, 1, D};
  const size_t smem = ((size_t)32 * (D + 1) + (size_t)LAT_WARPS * D) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  dim3 grid(n_tokens, (heads + LAT_WARPS - 1) / LAT_WARPS);
  LLM_HOST_CHECK(grid.y <= 65535, ERR_BAD_SIZE);
  if (dtype == DT_F32) {
    auto kernel = latent_attention_kernel<float, float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, LAT_THREADS, smem, stream, (const float*)q, (float*)out, c, rank, (const float*)sink,
                  positions, row_seq, heads, scale, window);
  } else if (dtype == DT_BF16) {
    auto kernel = latent_attention_kernel<__nv_bfloat16, __nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, LAT_THREADS, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, c, rank,
                  (const __nv_bfloat16*)sink, positions, row_seq, heads, scale, window);
  } else {
    return ERR_BAD_DTYPE;
  }
  return launch_status();
}
