// The matrix memory of xLSTM (mLSTM) around the engine's state scan.  Per head, with log gates
// i_t = cap tanh(zi / cap) and f_t = logsigmoid(cap tanh(zf / cap)) and a running maximum m
// (m_0 = 0):
//
//   m_t = max(f_t + m_(t-1), i_t),   a_t = exp(f_t + m_(t-1) - m_t),   b_t = exp(i_t - m_t),
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,   n_t = a_t n_(t-1) + b_t k_t,
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).
//
// n rides in the state as one more value column (the values get a column of ones), so the scan of
// csrc/linear_attention.cu - S = diag(a) S + k v^T, o = S^T q - does both sums: it is given the
// decay a_t for every key channel, b_t k_t as the key, and float32 copies of q and v.  Here are the
// kernels before it (gates and the walk of m; the float32 operands) and after it (the quotient, the
// unit norm of every head, the norm weight and the sigmoid gate).  Everything is float32.

#include "common.cuh"

#include <math.h>

#define GATE_THREADS 256
#define GATE_CHUNK 1024

// Grid (sequence, head).  coef[row][head] = (a, b, exp(-m), m) for every new token of the sequence;
// m_state[slot][head] is read at the start and written at the end.  The gates of a chunk of tokens
// are computed side by side, m is walked through the chunk as a scan, then a and b side by side.
template <typename TW>
__global__ void __launch_bounds__(GATE_THREADS)
mlstm_gates_kernel(const float* __restrict__ z, long long z_stride, int i_col, int f_col, const TW* __restrict__ i_bias,
                   const TW* __restrict__ f_bias, float cap, float* __restrict__ m_state, float4* __restrict__ coef,
                   const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_start,
                   const int32_t* __restrict__ seq_q_len, int heads) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float gi[GATE_CHUNK], gf[GATE_CHUNK], mm[GATE_CHUNK + 1], wF[GATE_THREADS / 32], wI[GATE_THREADS / 32];
  const int s = blockIdx.x, h = blockIdx.y;
  const int len = seq_q_len[s];
  if (len <= 0) return;
  const int slot = seq_slot[s];
  const long long start = seq_q_start[s];
  const float bi = to_float(i_bias[h]), bf = to_float(f_bias[h]);
  float m_prev = m_state[(long long)slot * heads + h];
  for (int c0 = 0; c0 < len; c0 += GATE_CHUNK) {
    const int n = min(GATE_CHUNK, len - c0);
    for (int t = threadIdx.x; t < n; t += blockDim.x) {
      const float* row = z + (start + c0 + t) * z_stride;
      gi[t] = cap * tanhf((row[i_col + h] + bi) / cap);
      const float u = cap * tanhf((row[f_col + h] + bf) / cap);
      gf[t] = fminf(u, 0.0f) - log1pf(expf(-fabsf(u)));      // logsigmoid(u)
    }
    __syncthreads();
    // A token maps m to max(m + f, i); two tokens in a row map it to max(m + (f1 + f2), max(i1 + f2, i2)).
    // So a thread folds the maps of its four tokens, the threads' maps are scanned (shuffles inside a
    // warp, the warps' totals through shared memory), and every thread walks its four tokens from the
    // m that comes in.
    {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t0 = threadIdx.x * 4;
      float F = 0.0f, I = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (t0 + j < n) {
          F += gf[t0 + j];
          I = fmaxf(I + gf[t0 + j], gi[t0 + j]);
        }
      for (int o = 1; o < 32; o <<= 1) {
        const float pF = __shfl_up_sync(0xffffffffu, F, o), pI = __shfl_up_sync(0xffffffffu, I, o);
        if (lane >= o) {
          I = fmaxf(pI + F, I);      // the earlier map first, then this one
          F = pF + F;
        }
      }
      if (lane == 31) {
        wF[warp] = F;
        wI[warp] = I;
      }
      float eF = __shfl_up_sync(0xffffffffu, F, 1), eI = __shfl_up_sync(0xffffffffu, I, 1);
      if (lane == 0) {
        eF = 0.0f;
        eI = -INFINITY;
      }
      __syncthreads();
      float pF = 0.0f, pI = -INFINITY;
      for (int v = 0; v < warp; ++v) {
        pI = fmaxf(pI + wF[v], wI[v]);
        pF += wF[v];
      }
      float m = fmaxf(m_prev + (pF + eF), fmaxf(pI + eF, eI));
      if (threadIdx.x == 0) mm[0] = m_prev;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (t0 + j < n) {
          m = fmaxf(gf[t0 + j] + m, gi[t0 + j]);
          mm[t0 + j + 1] = m;
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n; t += blockDim.x) {
      const float m = mm[t + 1];
      coef[(start + c0 + t) * heads + h] = make_float4(expf(gf[t] + mm[t] - m), expf(gi[t] - m), expf(-m), m);
    }
    m_prev = mm[n];
    __syncthreads();
  }
  if (threadIdx.x == 0) m_state[(long long)slot * heads + h] = m_prev;
}

extern "C" int llm_mlstm_gates(const float* z, long long z_stride, int i_col, int f_col, const void* i_bias,
                               const void* f_bias, int bias_dtype, float cap, float* m_state, float* coef,
                               const int32_t* seq_slot, const int32_t* seq_q_start, const int32_t* seq_q_len, int n_seqs,
                               int heads, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  LLM_HOST_CHECK(heads >= 1 && heads <= 65535 && cap > 0.0f, ERR_BAD_SIZE);
  dim3 grid(n_seqs, heads);
  if (bias_dtype == DT_F32)
    launch_kernel(mlstm_gates_kernel<float>, grid, GATE_THREADS, 0, stream, z, z_stride, i_col, f_col,
                  (const float*)i_bias, (const float*)f_bias, cap, m_state, (float4*)coef, seq_slot, seq_q_start,
                  seq_q_len, heads);
  else if (bias_dtype == DT_BF16)
    launch_kernel(mlstm_gates_kernel<__nv_bfloat16>, grid, GATE_THREADS, 0, stream, z, z_stride, i_col, f_col,
                  (const __nv_bfloat16*)i_bias, (const __nv_bfloat16*)f_bias, cap, m_state, (float4*)coef, seq_slot,
                  seq_q_start, seq_q_len, heads);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// Grid (token, head): the scan's float32 operands.  qf = q, kf = b k, decay[token][head] = a,
// vf = [v | 1 | 0 ...] (dvp columns per head).
template <typename T>
__global__ void mlstm_operands_kernel(const T* __restrict__ u, long long u_stride, int q_col, int k_col, int v_col,
                                      const float4* __restrict__ coef, float* __restrict__ qf, float* __restrict__ kf,
                                      float* __restrict__ decay, float* __restrict__ vf, int heads, int dk, int dv,
                                      int dvp) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  const int h = blockIdx.y;
  const float4 c = coef[t * heads + h];
  const T* row = u + t * u_stride;
  const long long kbase = (t * heads + h) * dk, vbase = (t * heads + h) * dvp;
  if (threadIdx.x == 0) decay[t * heads + h] = c.x;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) {
    qf[kbase + i] = to_float(row[q_col + h * dk + i]);
    kf[kbase + i] = c.y * to_float(row[k_col + h * dk + i]);
  }
  for (int i = threadIdx.x; i < dvp; i += blockDim.x)
    vf[vbase + i] = i < dv ? to_float(row[v_col + h * dv + i]) : (i == dv ? 1.0f : 0.0f);
}

extern "C" int llm_mlstm_operands(const void* u, int dtype, long long u_stride, int q_col, int k_col, int v_col,
                                  const float* coef, float* qf, float* kf, float* decay, float* vf, int n_tokens,
                                  int heads, int dk, int dv, int dvp, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(dvp > dv && heads <= 65535, ERR_BAD_SIZE);
  dim3 grid(n_tokens, heads);
  const int threads = dk > 64 || dvp > 64 ? 128 : 64;
  if (dtype == DT_F32)
    launch_kernel(mlstm_operands_kernel<float>, grid, threads, 0, stream, (const float*)u, u_stride, q_col, k_col, v_col,
                  (const float4*)coef, qf, kf, decay, vf, heads, dk, dv, dvp);
  else if (dtype == DT_BF16)
    launch_kernel(mlstm_operands_kernel<__nv_bfloat16>, grid, threads, 0, stream, (const __nv_bfloat16*)u, u_stride,
                  q_col, k_col, v_col, (const float4*)coef, qf, kf, decay, vf, heads, dk, dv, dvp);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// A warp per (token, head): the scan's row [S^T q | n . q | ...] -> the quotient, divided by its root
// mean square over the head, times the norm weight, times sigmoid(gate).
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
mlstm_finish_kernel(const float* __restrict__ scanned, const float4* __restrict__ coef, const TW* __restrict__ norm_w,
                    const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, long long out_stride,
                    long long items, int heads, int dv, int dvp, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const long long t = item / heads;
  const int h = (int)(item - t * heads);
  const float* row = scanned + item * dvp;
  const float den = fmaxf(fabsf(row[dv]), coef[item].z) + 1e-6f;
  float sq = 0.0f;
  for (int c = lane; c < dv; c += 32) {
    const float v = row[c] / den;
    sq += v * v;
  }
  const float scale = 1.0f / sqrtf(warp_sum(sq) / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const int col = h * dv + c;
    const float g = to_float(gate[t * gate_stride + col]);
    out[t * out_stride + col] = from_float<T>(row[c] / den * scale * to_float(norm_w[col]) / (1.0f + expf(-g)));
  }
}

extern "C" int llm_mlstm_finish(const float* scanned, const float* coef, const void* norm_w, const void* gate,
                                long long gate_stride, void* out, long long out_stride, int dtype, int n_tokens,
                                int heads, int dv, int dvp, float eps, cudaStream_t stream) {
  const long long items = (long long)n_tokens * heads;
  if (items <= 0) return 0;
  const int blocks = (int)((items + 3) / 4);
  if (dtype == DT_F32)
    launch_kernel(mlstm_finish_kernel<float, float>, blocks, 128, 0, stream, scanned, (const float4*)coef,
                  (const float*)norm_w, (const float*)gate, gate_stride, (float*)out, out_stride, items, heads, dv, dvp,
                  eps);
  else if (dtype == DT_BF16)
    launch_kernel(mlstm_finish_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 128, 0, stream, scanned,
                  (const float4*)coef, (const __nv_bfloat16*)norm_w, (const __nv_bfloat16*)gate, gate_stride,
                  (__nv_bfloat16*)out, out_stride, items, heads, dv, dvp, eps);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------------ one token per request

// A step that brings one token per request (decoding) does all of the above in one kernel: grid
// (sequence, head), the head's [S | n] read, updated and written once.  A warp takes the key rows
// w, w + 8, ..., a lane the value columns lane, lane + 32, ...; the warps' shares of S^T q meet in shared
// memory.  u holds q, k, v and the output gate's projection as projected, z the gates' (float32).
#define STEP_THREADS 256
#define STEP_MAX_COLS 9      // value columns per lane: vdim + pad <= 288

template <typename T, typename TW>
__global__ void __launch_bounds__(STEP_THREADS)
mlstm_step_kernel(const T* __restrict__ u, long long u_stride, int q_col, int k_col, int v_col, int g_col,
                  const float* __restrict__ z, long long z_stride, int i_col, int f_col, const TW* __restrict__ i_bias,
                  const TW* __restrict__ f_bias, float cap, float* __restrict__ state, float* __restrict__ m_state,
                  const TW* __restrict__ norm_w, T* __restrict__ out, long long out_stride,
                  const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_start,
                  const int32_t* __restrict__ seq_q_len, int heads, int dk, int dv, int dvp, float q_scale, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float step_smem[];      // q [dk], k [dk], v [dvp], parts [8][dvp], then 8 spare
  float* qs = step_smem;
  float* kk = qs + dk;
  float* vs = kk + dk;
  float* parts = vs + dvp;
  float* spare = parts + 8 * dvp;
  __shared__ float scratch[32];
  const int s = blockIdx.x, h = blockIdx.y;
  if (seq_q_len[s] <= 0) return;
  const int slot = seq_slot[s];
  const long long t = seq_q_start[s];
  const T* row = u + t * u_stride;
  if (threadIdx.x == 0) {
    const float* zr = z + t * z_stride;
    const float gi = cap * tanhf((zr[i_col + h] + to_float(i_bias[h])) / cap);
    const float x = cap * tanhf((zr[f_col + h] + to_float(f_bias[h])) / cap);
    const float gf = fminf(x, 0.0f) - log1pf(expf(-fabsf(x)));
    const float m_prev = m_state[(long long)slot * heads + h];
    const float m = fmaxf(gf + m_prev, gi);
    m_state[(long long)slot * heads + h] = m;
    spare[0] = expf(gf + m_prev - m);
    spare[1] = expf(gi - m);
    spare[2] = expf(-m);
  }
  __syncthreads();
  const float a = spare[0], b = spare[1], floor_ = spare[2];
  for (int i = threadIdx.x; i < dk; i += STEP_THREADS) {
    qs[i] = to_float(row[q_col + h * dk + i]) * q_scale;
    kk[i] = b * to_float(row[k_col + h * dk + i]);
  }
  for (int i = threadIdx.x; i < dvp; i += STEP_THREADS)
    vs[i] = i < dv ? to_float(row[v_col + h * dv + i]) : (i == dv ? 1.0f : 0.0f);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* S = state + (((long long)slot * heads + h) * dk) * dvp;
  float acc[STEP_MAX_COLS];
#pragma unroll
  for (int j = 0; j < STEP_MAX_COLS; ++j) acc[j] = 0.0f;
  // four rows at a time: their loads are under way together
  for (int r = warp; r < dk; r += 32) {
    float sv[4][STEP_MAX_COLS];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < STEP_MAX_COLS; ++j) {
        const int c = lane + 32 * j, rr = r + 8 * i;
        if (c < dvp && rr < dk) sv[i][j] = S[(long long)rr * dvp + c];
      }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = r + 8 * i;
      if (rr >= dk) break;
      const float kr = kk[rr], qr = qs[rr];
#pragma unroll
      for (int j = 0; j < STEP_MAX_COLS; ++j) {
        const int c = lane + 32 * j;
        if (c < dvp) {
          const float v = a * sv[i][j] + kr * vs[c];
          S[(long long)rr * dvp + c] = v;
          acc[j] = fmaf(v, qr, acc[j]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < STEP_MAX_COLS; ++j) {
    const int c = lane + 32 * j;
    if (c < dvp) parts[warp * dvp + c] = acc[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c <= dv; c += STEP_THREADS) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) v += parts[w * dvp + c];
    vs[c] = v;      // the head's S^T q, and n . q behind it
  }
  __syncthreads();
  const float den = fmaxf(fabsf(vs[dv]), floor_) + 1e-6f;
  float sq = 0.0f;
  for (int c = threadIdx.x; c < dv; c += STEP_THREADS) {
    const float v = vs[c] / den;
    sq += v * v;
  }
  const float scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)dv + eps);
  for (int c = threadIdx.x; c < dv; c += STEP_THREADS) {
    const int col = h * dv + c;
    const float g = to_float(row[g_col + col]);
    out[t * out_stride + col] = from_float<T>(vs[c] / den * scale * to_float(norm_w[col]) / (1.0f + expf(-g)));
  }
}

// dtype: element type of u, out, the biases and the norm weight.
extern "C" int llm_mlstm_step(const void* u, int dtype, long long u_stride, int q_col, int k_col, int v_col, int g_col,
                              const float* z, long long z_stride, int i_col, int f_col, const void* i_bias,
                              const void* f_bias, float cap, float* state, float* m_state, const void* norm_w, void* out,
                              long long out_stride, const int32_t* seq_slot, const int32_t* seq_q_start,
                              const int32_t* seq_q_len, int n_seqs, int heads, int dk, int dv, int dvp, float q_scale,
                              float eps, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  LLM_HOST_CHECK(dvp > dv && dvp <= 32 * STEP_MAX_COLS && heads <= 65535 && cap > 0.0f, ERR_BAD_SIZE);
  const size_t smem = (size_t)(2 * dk + 9 * dvp + 8) * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  dim3 grid(n_seqs, heads);
  if (dtype == DT_F32)
    launch_kernel(mlstm_step_kernel<float, float>, grid, STEP_THREADS, smem, stream, (const float*)u, u_stride, q_col,
                  k_col, v_col, g_col, z, z_stride, i_col, f_col, (const float*)i_bias, (const float*)f_bias, cap, state,
                  m_state, (const float*)norm_w, (float*)out, out_stride, seq_slot, seq_q_start, seq_q_len, heads, dk, dv,
                  dvp, q_scale, eps);
  else if (dtype == DT_BF16)
    launch_kernel(mlstm_step_kernel<__nv_bfloat16, __nv_bfloat16>, grid, STEP_THREADS, smem, stream,
                  (const __nv_bfloat16*)u, u_stride, q_col, k_col, v_col, g_col, z, z_stride, i_col, f_col,
                  (const __nv_bfloat16*)i_bias, (const __nv_bfloat16*)f_bias, cap, state, m_state,
                  (const __nv_bfloat16*)norm_w, (__nv_bfloat16*)out, out_stride, seq_slot, seq_q_start, seq_q_len, heads,
                  dk, dv, dvp, q_scale, eps);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}
