// Kernels around a residual that is kept as several parallel streams (hyper-connections), the
// embedding that fills them, and element-wise activations of a plain (ungated) feed-forward.
// All arithmetic is float32; the streams are float32 [tokens][streams][width].
//
// The order in which any sum is formed depends on the operation's own sizes only (width, number
// of streams, number of partial results), never on how many rows a launch carries.

#include "common.cuh"

#include <math.h>

#define MAX_STREAMS 16

// ------------------------------------------------- embedding * scale + learned position vector

template <typename TW>
__global__ void embed_positions_kernel(const TW* __restrict__ table, const TW* __restrict__ pos_table,
                                       const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                                       float* __restrict__ out, int width, int streams, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const TW* row = table + (long long)ids[t] * width;
  const TW* prow = pos_table ? pos_table + (long long)positions[t] * width : nullptr;
  float* dst = out + (long long)t * streams * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_float(row[i]) * scale;
    if (prow) v += to_float(prow[i]);
    for (int s = 0; s < streams; ++s) dst[(long long)s * width + i] = v;
  }
}

extern "C" int llm_embed_positions(const void* table, const void* pos_table, int dtype, const int32_t* ids,
                                   const int32_t* positions, float* out, int n_tokens, int width, int streams,
                                   float scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(streams >= 1 && streams <= MAX_STREAMS, ERR_BAD_SIZE);
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == DT_F32) {
    launch_kernel(embed_positions_kernel<float>, n_tokens, threads, 0, stream, (const float*)table,
                  (const float*)pos_table, ids, positions, out, width, streams, scale);
  } else if (dtype == DT_BF16) {
    launch_kernel(embed_positions_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table,
                  (const __nv_bfloat16*)pos_table, ids, positions, out, width, streams, scale);
  } else {
    return ERR_BAD_DTYPE;
  }
  return launch_status();
}

// ------------------------------------------ stream update + stream read + RMSNorm in one kernel

// One block per output row.  With `delta` (the sublayer result that has not been written into the
// streams yet, possibly as partial sums that are added in index order):
//   y = sum(delta partials) * delta_scale;  x_t <- sum_s mix[s][t] x_s + write[t] * y   for every t,
// all from the old streams, written back.  Then u = sum_t read[t] x_t (read == nullptr: plain sum)
// and out = u / sqrt(mean(u^2) + eps) * weight.
// SMAX bounds the number of streams at compile time (the loops over streams are unrolled to it).
template <typename TD, typename TO, int SMAX>
__global__ void __launch_bounds__(256) stream_step_kernel(float* __restrict__ streams_buf, int n_streams, const TD* __restrict__ delta,
                                   int n_partials, long long partial_stride, long long delta_row_stride,
                                   const float* __restrict__ delta_scale, const float* __restrict__ write_vec,
                                   const float* __restrict__ mix, const float* __restrict__ read_vec,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int32_t* __restrict__ row_index, int width, float eps) {
  pdl_launch_dependents();
  extern __shared__ float smem[];  // width floats (u) + 32 scratch + S*S mix + 2 S vectors
  float* u_row = smem;
  float* scratch = smem + width;
  float* s_mix = scratch + 32;
  float* s_write = s_mix + MAX_STREAMS * MAX_STREAMS;
  float* s_read = s_write + MAX_STREAMS;
  const int S = n_streams;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.0f : 0.0f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    s_write[i] = write_vec ? write_vec[i] : 1.0f;
    s_read[i] = read_vec ? read_vec[i] : 1.0f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const long long src = row_index ? row_index[r] : r;
  float* x = streams_buf + src * S * width;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float xs[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s)
      if (s < S) xs[s] = x[(long long)s * width + i];
    float u = 0.0f;
    if (delta) {
      float y = 0.0f;
      for (int p = 0; p < n_partials; ++p) y += to_float(delta[p * partial_stride + src * delta_row_stride + i]);
      if (delta_scale) y *= delta_scale[i];
#pragma unroll
      for (int t = 0; t < SMAX; ++t) {
        if (t < S) {
          float v = 0.0f;
#pragma unroll
          for (int s = 0; s < SMAX; ++s)
            if (s < S) v += s_mix[s * S + t] * xs[s];
          v += s_write[t] * y;
          x[(long long)t * width + i] = v;
          u += s_read[t] * v;
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < SMAX; ++t)
        if (t < S) u += s_read[t] * xs[t];
    }
    u_row[i] = u;
    sq += u * u;
  }
  if (!out) return;
  const float total = block_sum(sq, scratch);
  const float scale = 1.0f / sqrtf(total / (float)width + eps);
  TO* dst = out + (long long)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<TO>(u_row[i] * scale * weight[i]);
}

// The same with four neighbouring channels per thread and 16-byte accesses: width a multiple of 4,
// float32 partial results, every row 16-byte aligned.
__device__ __forceinline__ float4 f4_scale_add(float4 acc, float s, float4 x) {
  acc.x += s * x.x; acc.y += s * x.y; acc.z += s * x.z; acc.w += s * x.w;
  return acc;
}

template <typename TO, int SMAX>
__global__ void __launch_bounds__(256) stream_step_vec_kernel(float* __restrict__ streams_buf, int n_streams,
                                   const float* __restrict__ delta, int n_partials, long long partial_stride,
                                   long long delta_row_stride, const float* __restrict__ delta_scale,
                                   const float* __restrict__ write_vec, const float* __restrict__ mix,
                                   const float* __restrict__ read_vec, const float* __restrict__ weight,
                                   TO* __restrict__ out, const int32_t* __restrict__ row_index, int width, float eps) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float smem[];
  float4* u_row = reinterpret_cast<float4*>(smem);
  float* scratch = smem + width;
  float* s_mix = scratch + 32;
  float* s_write = s_mix + MAX_STREAMS * MAX_STREAMS;
  float* s_read = s_write + MAX_STREAMS;
  const int S = n_streams;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.0f : 0.0f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    s_write[i] = write_vec ? write_vec[i] : 1.0f;
    s_read[i] = read_vec ? read_vec[i] : 1.0f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const long long src = row_index ? row_index[r] : r;
  const int w4 = width / 4;
  float4* x = reinterpret_cast<float4*>(streams_buf + src * S * width);
  float sq = 0.0f;
  for (int i = threadIdx.x; i < w4; i += blockDim.x) {
    float4 xs[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s)
      if (s < S) xs[s] = x[(long long)s * w4 + i];
    float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (delta) {
      float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int p = 0; p < n_partials; ++p)
        y = f4_scale_add(y, 1.0f, reinterpret_cast<const float4*>(delta + p * partial_stride + src * delta_row_stride)[i]);
      if (delta_scale) {
        const float4 g = reinterpret_cast<const float4*>(delta_scale)[i];
        y.x *= g.x; y.y *= g.y; y.z *= g.z; y.w *= g.w;
      }
#pragma unroll
      for (int t = 0; t < SMAX; ++t) {
        if (t < S) {
          float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int s = 0; s < SMAX; ++s)
            if (s < S) v = f4_scale_add(v, s_mix[s * S + t], xs[s]);
          v = f4_scale_add(v, s_write[t], y);
          x[(long long)t * w4 + i] = v;
          u = f4_scale_add(u, s_read[t], v);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < SMAX; ++t)
        if (t < S) u = f4_scale_add(u, s_read[t], xs[t]);
    }
    u_row[i] = u;
    sq += u.x * u.x;
    sq += u.y * u.y;
    sq += u.z * u.z;
    sq += u.w * u.w;
  }
  if (!out) return;
  const float total = block_sum(sq, scratch);
  const float scale = 1.0f / sqrtf(total / (float)width + eps);
  TO* dst = out + (long long)r * width;
  for (int i = threadIdx.x; i < w4; i += blockDim.x) {
    const float4 u = u_row[i];
    const float4 g = reinterpret_cast<const float4*>(weight)[i];
    dst[4 * i] = from_float<TO>(u.x * scale * g.x);
    dst[4 * i + 1] = from_float<TO>(u.y * scale * g.y);
    dst[4 * i + 2] = from_float<TO>(u.z * scale * g.z);
    dst[4 * i + 3] = from_float<TO>(u.w * scale * g.w);
  }
}

extern "C" int llm_stream_step(float* streams_buf, int n_streams, const void* delta, int delta_dtype, int n_partials,
                               long long partial_stride, long long delta_row_stride, const float* delta_scale,
                               const float* write_vec, const float* mix, const float* read_vec, const float* weight,
                               void* out, int out_dtype, const int32_t* row_index, int rows, int width, float eps,
                               cudaStream_t stream) {
  if (rows <= 0) return 0;
  LLM_HOST_CHECK(n_streams >= 1 && n_streams <= MAX_STREAMS, ERR_BAD_SIZE);
  const int threads = width >= 512 ? 256 : 128;   // (__launch_bounds__ of the kernel)
  const size_t smem = (size_t)(width + 32 + MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
#define LAUNCH_S(TD, TO, SMAX)                                                                                 \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(stream_step_kernel<TD, TO, SMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                           (int)smem);                                                                         \
    launch_kernel(stream_step_kernel<TD, TO, SMAX>, rows, threads, smem, stream, streams_buf, n_streams,       \
                  (const TD*)delta, n_partials, partial_stride, delta_row_stride, delta_scale, write_vec, mix,  \
                  read_vec, weight, (TO*)out, row_index, width, eps);                                          \
  } while (0)
  // four channels per thread where everything is 16-byte aligned and the partial results are float32
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = width % 4 == 0 && n_streams <= 4 && (!delta || (delta_dtype == DT_F32 && al(delta) &&
                   partial_stride % 4 == 0 && delta_row_stride % 4 == 0)) && al(streams_buf) && al(delta_scale) &&
                   al(weight) && al(out);
#define LAUNCH_V(TO, SMAX)                                                                                     \
  launch_kernel(stream_step_vec_kernel<TO, SMAX>, rows, width >= 2048 ? 256 : 128, smem, stream, streams_buf,  \
                n_streams, (const float*)delta, n_partials, partial_stride, delta_row_stride, delta_scale,     \
                write_vec, mix, read_vec, weight, (TO*)out, row_index, width, eps)
  if (vec && smem <= 48 * 1024 && (out_dtype == DT_F32 || out_dtype == DT_BF16)) {
    if (out_dtype == DT_F32) {
      if (n_streams == 1) LAUNCH_V(float, 1); else if (n_streams == 2) LAUNCH_V(float, 2); else LAUNCH_V(float, 4);
    } else {
      if (n_streams == 1) LAUNCH_V(__nv_bfloat16, 1); else if (n_streams == 2) LAUNCH_V(__nv_bfloat16, 2);
      else LAUNCH_V(__nv_bfloat16, 4);
    }
    return launch_status();
  }
#undef LAUNCH_V
#define LAUNCH(TD, TO)                                     \
  do {                                                     \
    if (n_streams == 1) LAUNCH_S(TD, TO, 1);               \
    else if (n_streams <= 2) LAUNCH_S(TD, TO, 2);          \
    else if (n_streams <= 4) LAUNCH_S(TD, TO, 4);          \
    else if (n_streams <= 8) LAUNCH_S(TD, TO, 8);          \
    else LAUNCH_S(TD, TO, MAX_STREAMS);                    \
  } while (0)
  if (delta_dtype == DT_F32 && out_dtype == DT_F32) LAUNCH(float, float);
  else if (delta_dtype == DT_F32 && out_dtype == DT_BF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == DT_BF16 && out_dtype == DT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == DT_BF16 && out_dtype == DT_F32) LAUNCH(__nv_bfloat16, float);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
#undef LAUNCH_S
  return launch_status();
}

// ------------------------------------------------------------------- element-wise activations

#define ACT_RELU2 0
#define ACT_GELU_TANH 1
#define ACT_SILU 2
#define ACT_RELU 3

__device__ __forceinline__ float activate(float z, int kind) {
  switch (kind) {
    case ACT_RELU2: { const float r = fmaxf(z, 0.0f); return r * r; }
    case ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    case ACT_SILU: return z / (1.0f + expf(-z));
    default: return fmaxf(z, 0.0f);
  }
}

// out[r][c] = act(sum of partials in[p][r][c]); rows of `in` and `out` may be strided, and `out`
// may be `in` itself (one partial, equal types and strides).
template <typename TI, typename TO>
__global__ void activation_kernel(const TI* in, int n_partials, long long partial_stride,
                                  long long in_stride, TO* out, long long out_stride, int rows,
                                  int width, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)rows * width;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / width;
    const int c = (int)(e - r * width);
    float z = 0.0f;
    for (int p = 0; p < n_partials; ++p) z += to_float(in[p * partial_stride + r * in_stride + c]);
    out[r * out_stride + c] = from_float<TO>(activate(z, kind));
  }
}

// The same for one bfloat16 matrix in and out (possibly the same one), eight elements at a time:
// width, both strides and both addresses multiples of eight elements.
__global__ void activation_bf16x8_kernel(const __nv_bfloat16* in, long long in_stride, __nv_bfloat16* out,
                                         long long out_stride, int rows, int width8, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c8 >= width8) return;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    uint4 raw = *reinterpret_cast<const uint4*>(in + (long long)r * in_stride + c8 * 8);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      h[j] = __floats2bfloat162_rn(activate(__low2float(h[j]), kind), activate(__high2float(h[j]), kind));
    *reinterpret_cast<uint4*>(out + (long long)r * out_stride + c8 * 8) = raw;
  }
}

extern "C" int llm_activation(const void* in, int in_dtype, int n_partials, long long partial_stride,
                              long long in_stride, void* out, int out_dtype, long long out_stride, int rows, int width,
                              int kind, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  LLM_HOST_CHECK(kind >= 0 && kind <= 3, ERR_BAD_SIZE);
  if (in_dtype == DT_BF16 && out_dtype == DT_BF16 && n_partials == 1 && width % 8 == 0 && in_stride % 8 == 0 &&
      out_stride % 8 == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const int width8 = width / 8;
    dim3 grid((width8 + 127) / 128, rows < 2048 ? rows : 2048);
    launch_kernel(activation_bf16x8_kernel, grid, 128, 0, stream, (const __nv_bfloat16*)in, in_stride,
                  (__nv_bfloat16*)out, out_stride, rows, width8, kind);
    return launch_status();
  }
  const long long total = (long long)rows * width;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
#define LAUNCH(TI, TO)                                                                                         \
  launch_kernel(activation_kernel<TI, TO>, blocks, threads, 0, stream, (const TI*)in, n_partials, partial_stride, \
                in_stride, (TO*)out, out_stride, rows, width, kind)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) LAUNCH(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}
