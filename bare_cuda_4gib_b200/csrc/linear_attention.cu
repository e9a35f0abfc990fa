// Linear attention with a decaying matrix state per (request, head):
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,        S [key dim][value dim], float32,
//
// where the decay a_t is one fixed number per head, or one number per key channel computed from
// the token.  The state lives in the cache manager's state slots and is carried from step to
// step; a step brings any number of new tokens per request (a prompt's portion or one decoded
// token), which one kernel walks in order.  q, k and v are read as the projection left them
// (float32 or bfloat16, rows may be strided); scores, decays, the state and the output are float32.
//
// Also here: the decay gate (sigmoid(z)^(1/tau) from a low-rank projection) and the gated group
// norm that follows the scan.

#include "common.cuh"

#include <math.h>

#define SCAN_WARPS 4
#define SCAN_THREADS (SCAN_WARPS * 32)
#define SCAN_ROWS 8        // state rows a thread keeps in registers
#define SCAN_STAGE 32      // elements of the next chunk a thread holds while it works on this one

#define DECAY_PER_HEAD 0
#define DECAY_PER_CHANNEL 1

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// Grid (sequence, head, slice of value columns).  A warp's 32 lanes are KS row groups times
// 32 / KS value columns; a thread owns the state elements (r * KS + kr, column) for r < SCAN_ROWS.
// Tokens are staged through shared memory a chunk at a time: while the block walks one chunk,
// every thread already holds its share of the next chunk's q, k, v (and decays) in registers.
template <typename T, int ACT, int DECAY>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_attention_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                             long long q_stride, long long k_stride, long long v_stride,
                             const float* __restrict__ decay,          // [heads] or [tokens][heads * dk]
                             float* __restrict__ state,                // [slots][heads][dk][dv]
                             float* __restrict__ out,                  // [tokens][heads * dv]
                             const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_start,
                             const int32_t* __restrict__ seq_q_len, int heads, int dk, int dv, int ks, int chunk,
                             float q_scale) {
  pdl_launch_dependents();
  extern __shared__ float work[];   // [chunk][q dk | k dk | (a dk) | v cols]
  const int seq = blockIdx.x, head = blockIdx.y;
  const int cols_per_warp = 32 / ks;
  const int cols_per_block = cols_per_warp * SCAN_WARPS;
  const int col0 = blockIdx.z * cols_per_block;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kr = lane % ks;
  const int col = col0 + warp * cols_per_warp + lane / ks;
  const bool live = col < dv;
  const int n_cols = min(cols_per_block, dv - col0);
  const int per_token = (DECAY == DECAY_PER_CHANNEL ? 3 : 2) * dk + cols_per_block;
  const int a_off = 2 * dk, v_off = (DECAY == DECAY_PER_CHANNEL ? 3 : 2) * dk;
  pdl_wait();
  const int n = seq_q_len[seq];
  if (n <= 0) return;
  const int row0 = seq_q_start[seq];
  const int slot = seq_slot[seq];
  float* S_g = state + (((long long)slot * heads + head) * dk) * dv;
  float S[SCAN_ROWS];
#pragma unroll
  for (int r = 0; r < SCAN_ROWS; ++r) {
    const int i = r * ks + kr;
    S[r] = (live && i < dk) ? S_g[(long long)i * dv + col] : 0.0f;
  }
  const float head_decay = DECAY == DECAY_PER_HEAD ? decay[head] : 0.0f;

  float stage[SCAN_STAGE];
  // element e of a chunk: token e / per_token, field e % per_token
  auto fetch = [&](int first, int count) {
    const int total = count * per_token;
#pragma unroll
    for (int j = 0; j < SCAN_STAGE; ++j) {
      const int e = threadIdx.x + j * SCAN_THREADS;
      float val = 0.0f;
      if (e < total) {
        const int t = e / per_token, f = e - t * per_token;
        const long long row = row0 + first + t;
        if (f < dk) {
          val = to_float(q[row * q_stride + head * dk + f]);
          val = (ACT ? silu_f(val) : val) * q_scale;
        } else if (f < 2 * dk) {
          val = to_float(k[row * k_stride + head * dk + (f - dk)]);
          if (ACT) val = silu_f(val);
        } else if (DECAY == DECAY_PER_CHANNEL && f < 3 * dk) {
          val = decay[row * ((long long)heads * dk) + head * dk + (f - 2 * dk)];
        } else {
          const int c = f - v_off;
          if (c < n_cols) {
            val = to_float(v[row * v_stride + head * dv + col0 + c]);
            if (ACT) val = silu_f(val);
          }
        }
      }
      stage[j] = val;
    }
  };
  fetch(0, min(chunk, n));
  for (int first = 0; first < n; first += chunk) {
    const int count = min(chunk, n - first);
    __syncthreads();   // the chunk before this one has been walked
#pragma unroll
    for (int j = 0; j < SCAN_STAGE; ++j) {
      const int e = threadIdx.x + j * SCAN_THREADS;
      if (e < count * per_token) work[e] = stage[j];
    }
    __syncthreads();
    if (first + chunk < n) fetch(first + chunk, min(chunk, n - first - chunk));
    for (int t = 0; t < count; ++t) {
      const float* w = work + t * per_token;
      const float vv = w[v_off + warp * cols_per_warp + lane / ks];
      float acc = 0.0f;
#pragma unroll
      for (int r = 0; r < SCAN_ROWS; ++r) {
        const int i = r * ks + kr;
        if (i < dk) {
          const float a = DECAY == DECAY_PER_CHANNEL ? w[a_off + i] : head_decay;
          S[r] = a * S[r] + w[dk + i] * vv;
          acc += S[r] * w[i];
        }
      }
      for (int o = ks >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && kr == 0) out[(long long)(row0 + first + t) * ((long long)heads * dv) + head * dv + col] = acc;
    }
  }
#pragma unroll
  for (int r = 0; r < SCAN_ROWS; ++r) {
    const int i = r * ks + kr;
    if (live && i < dk) S_g[(long long)i * dv + col] = S[r];
  }
}

extern "C" int llm_linear_attention_scan(const void* q, const void* k, const void* v, int dtype, long long q_stride,
                                         long long k_stride, long long v_stride, const float* decay, int per_channel,
                                         int act_silu, float* state, float* out, const int32_t* seq_slot,
                                         const int32_t* seq_q_start, const int32_t* seq_q_len, int n_seqs, int heads,
                                         int dk, int dv, float q_scale, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  LLM_HOST_CHECK(dk >= 1 && dk <= 32 * SCAN_ROWS && dv >= 1 && heads >= 1, ERR_BAD_SIZE);
  int ks = 1;
  while (ks * SCAN_ROWS < dk) ks <<= 1;          // row groups: a power of two, at most 32
  const int cols_per_block = (32 / ks) * SCAN_WARPS;
  const int slices = (dv + cols_per_block - 1) / cols_per_block;
  const int per_token = (per_channel ? 3 : 2) * dk + cols_per_block;
  int chunk = SCAN_STAGE * SCAN_THREADS / per_token;
  if (chunk > 16) chunk = 16;
  LLM_HOST_CHECK(chunk >= 1, ERR_BAD_SIZE);
  const size_t smem = (size_t)chunk * per_token * sizeof(float);
  dim3 grid(n_seqs, heads, slices);
#define LAUNCH(T, ACT, DEC)                                                                                     \
  launch_kernel(linear_attention_scan_kernel<T, ACT, DEC>, grid, SCAN_THREADS, smem, stream, (const T*)q,       \
                (const T*)k, (const T*)v, q_stride, k_stride, v_stride, decay, state, out, seq_slot, seq_q_start, \
                seq_q_len, heads, dk, dv, ks, chunk, q_scale)
  if (dtype == DT_F32) {
    if (per_channel) { if (act_silu) LAUNCH(float, 1, 1); else LAUNCH(float, 0, 1); }
    else { if (act_silu) LAUNCH(float, 1, 0); else LAUNCH(float, 0, 0); }
  } else if (dtype == DT_BF16) {
    if (per_channel) { if (act_silu) LAUNCH(__nv_bfloat16, 1, 1); else LAUNCH(__nv_bfloat16, 0, 1); }
    else { if (act_silu) LAUNCH(__nv_bfloat16, 1, 0); else LAUNCH(__nv_bfloat16, 0, 0); }
  } else {
    return ERR_BAD_DTYPE;
  }
#undef LAUNCH
  return launch_status();
}

// ----------------------------------------------------------------------------- decay gate

// a[t][c] = sigmoid(z)^(1/tau), z = sum_r up[c][r] low[t][r] + bias[c], as exp(-softplus(-z) / tau).
template <typename T>
__global__ void decay_gate_kernel(const T* __restrict__ low, long long low_stride, const float* __restrict__ up,
                                  const float* __restrict__ bias, float* __restrict__ out, int channels, int rank,
                                  float inv_tau) {
  pdl_launch_dependents();
  extern __shared__ float low_row[];
  pdl_wait();
  const long long t = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) low_row[r] = to_float(low[t * low_stride + r]);
  __syncthreads();
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float z = 0.0f;
    const float* urow = up + (long long)c * rank;
    for (int r = 0; r < rank; ++r) z += urow[r] * low_row[r];
    if (bias) z += bias[c];
    const float sp = fmaxf(-z, 0.0f) + log1pf(expf(-fabsf(z)));   // softplus(-z)
    out[t * channels + c] = expf(-sp * inv_tau);
  }
}

extern "C" int llm_decay_gate(const void* low, int dtype, long long low_stride, const float* up, const float* bias,
                              float* out, int rows, int channels, int rank, float inv_tau, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)rank * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  const int threads = channels >= 1024 ? 256 : 128;
  if (dtype == DT_F32)
    launch_kernel(decay_gate_kernel<float>, rows, threads, smem, stream, (const float*)low, low_stride, up, bias, out,
                  channels, rank, inv_tau);
  else if (dtype == DT_BF16)
    launch_kernel(decay_gate_kernel<__nv_bfloat16>, rows, threads, smem, stream, (const __nv_bfloat16*)low, low_stride,
                  up, bias, out, channels, rank, inv_tau);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------ gated group norm

#define GATE_SIGMOID 0
#define GATE_SILU 1

// One warp per (row, group): out = x / sqrt(mean_group(x^2) + eps) * weight[c % weight_len] *
// gate_act(gate) * out_scale.  A group is `group` neighbouring channels of the row.
template <typename TG, typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ x, const TG* __restrict__ gate, long long gate_stride,
                                        const float* __restrict__ weight, int weight_len, TO* __restrict__ out,
                                        long long out_stride, int rows, int channels, int group, int gate_kind,
                                        float eps, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int groups = channels / group;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * groups) return;
  const long long r = item / groups;
  const int g = (int)(item - r * groups);
  const int lane = threadIdx.x & 31;
  const float* xr = x + r * channels + (long long)g * group;
  float sq = 0.0f;
  for (int i = lane; i < group; i += 32) sq += xr[i] * xr[i];
  sq = warp_sum(sq);
  const float scale = 1.0f / sqrtf(sq / (float)group + eps);
  for (int i = lane; i < group; i += 32) {
    const int c = g * group + i;
    const float z = to_float(gate[r * gate_stride + c]);
    const float gz = gate_kind == GATE_SILU ? z / (1.0f + expf(-z)) : 1.0f / (1.0f + expf(-z));
    out[r * out_stride + c] = from_float<TO>(xr[i] * scale * weight[c % weight_len] * gz * out_scale);
  }
}

extern "C" int llm_gated_group_norm(const float* x, const void* gate, int gate_dtype, long long gate_stride,
                                    const float* weight, int weight_len, void* out, int out_dtype, long long out_stride,
                                    int rows, int channels, int group, int gate_kind, float eps, float out_scale,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  LLM_HOST_CHECK(group >= 1 && channels % group == 0 && weight_len >= 1, ERR_BAD_SIZE);
  const long long items = (long long)rows * (channels / group);
  const int warps = 4;
  const int blocks = (int)((items + warps - 1) / warps);
#define LAUNCH(TG, TO)                                                                                      \
  launch_kernel(gated_group_norm_kernel<TG, TO>, blocks, warps * 32, 0, stream, x, (const TG*)gate, gate_stride, \
                weight, weight_len, (TO*)out, out_stride, rows, channels, group, gate_kind, eps, out_scale)
  if (gate_dtype == DT_F32 && out_dtype == DT_F32) LAUNCH(float, float);
  else if (gate_dtype == DT_BF16 && out_dtype == DT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (gate_dtype == DT_F32 && out_dtype == DT_BF16) LAUNCH(float, __nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}
