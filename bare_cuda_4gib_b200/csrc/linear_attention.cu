// Linear attention with a decaying matrix state per (request, head):
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,        S [key dim][value dim], float32,
//
// where the decay a_t is one fixed number per head, or one number per key channel computed from
// the token.  The state lives in the cache manager's state slots and is carried from step to
// step; a step brings any number of new tokens per request (a prompt's portion or one decoded
// token), which one kernel walks in order.  q, k and v are read as they were stored (float32 or
// bfloat16, rows may be strided; an activation on them is applied before, in place); scores,
// decays, the state and the output are float32.
//
// Also here: the decay gate (sigmoid(z)^(1/tau) from a low-rank projection) and the gated group
// norm that follows the scan.

#include "common.cuh"

#include <math.h>

#define SCAN_WARPS 8
#define SCAN_THREADS (SCAN_WARPS * 32)
#define SCAN_BUFFERS 4     // chunks in shared memory: one being walked, the others on their way

#define DECAY_PER_HEAD 0
#define DECAY_PER_CHANNEL 1
#define DECAY_PER_TOKEN 2      // one number per (token, head), the same for every key channel: decay [tokens][heads]

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}

// ROWS numbers as floats.  VEC: 16-byte pieces (8 bfloat16 or 4 float32 numbers each, 16-byte aligned),
// piece j starting at p + j * stride; else the ROWS numbers starting at p.
template <typename T, int ROWS, bool VEC>
__device__ __forceinline__ void load_rows(const T* p, int valid, float (&dst)[ROWS], int stride) {
  if constexpr (VEC && sizeof(T) == 2) {
#pragma unroll
    for (int j = 0; j < ROWS / 8; ++j) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + j * stride);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dst[j * 8 + 2 * e] = __uint_as_float(w[e] << 16);
        dst[j * 8 + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
      }
    }
  } else if constexpr (VEC) {
#pragma unroll
    for (int j = 0; j < ROWS / 4; ++j) {
      const float4 raw = *reinterpret_cast<const float4*>(p + j * stride);
      dst[j * 4] = raw.x; dst[j * 4 + 1] = raw.y; dst[j * 4 + 2] = raw.z; dst[j * 4 + 3] = raw.w;
    }
  } else {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) dst[r] = r < valid ? to_float(p[r]) : 0.0f;
  }
}

// Grid (sequence, head, slice of value columns).  A warp's 32 lanes are `ks` row groups times
// 32 / ks value columns; a thread owns ROWS state rows of one column, so a token costs it ROWS
// multiply-adds for the state, ROWS for the output, log2(ks) shuffles, and (VEC: rows and buffers
// 16-byte aligned, the threads' rows cover the key size exactly) a few 16-byte loads of q and k from
// shared memory.  Which rows: the neighbouring rows kr * ROWS ..; or, with DEAL (VEC launches of steps
// that bring some request more than four tokens), 16-byte pieces dealt round-robin to the row groups
// (piece j of group kr covers rows (j * ks + kr) * PIECE ..), so that the row groups of a warp read
// neighbouring pieces of a token's q and k and no two of them meet in a shared-memory bank.  (A step
// of single tokens is bound by reading and writing the state and measured 2 % faster with neighbouring rows.)
// Tokens come through shared memory a chunk at a time, SCAN_BUFFERS chunks deep: while the block walks
// one chunk, the next ones' q, k, v (and decays) are on their way as 16-byte asynchronous copies, as
// the projection left them (rows and head slices that are not 16-byte aligned are copied element
// by element instead).  q_scale multiplies the output.
template <typename T, int DECAY, int ROWS, bool VEC, bool DEAL>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_attention_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                             long long q_stride, long long k_stride, long long v_stride,
                             const float* __restrict__ decay,          // [heads], [tokens][heads * dk] or [tokens][heads]
                             float* __restrict__ state,                // [slots][heads][dk][dv]
                             float* __restrict__ out,                  // [tokens][heads * dv]
                             const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_start,
                             const int32_t* __restrict__ seq_q_len, int heads, int dk, int dv, int ks, int chunk,
                             int aligned, float q_scale, int seg_len, int n_segs, int slices,
                             float* __restrict__ seg_state,      // [sequences][n_segs][heads][dk][dv]
                             float* __restrict__ seg_decay,      // [sequences][n_segs][heads][dk]
                             float* __restrict__ cum) {          // [tokens][heads * dk]
  pdl_launch_dependents();
  extern __shared__ __align__(16) uint8_t scan_smem[];
  const int seq = blockIdx.x, head = blockIdx.y;
  const int seg = blockIdx.z / slices;      // with n_segs > 1: which stretch of seg_len tokens (see scan_carry_kernel)
  const int cols_per_warp = 32 / ks;
  const int cols_per_block = cols_per_warp * SCAN_WARPS;
  const int col0 = (blockIdx.z % slices) * cols_per_block;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kr = lane % ks;
  const int my_col = warp * cols_per_warp + lane / ks;
  const int col = col0 + my_col;
  const bool live = col < dv;
  const int n_cols = min(cols_per_block, dv - col0);
  const int tok = 2 * dk + cols_per_block;                 // elements of T per token in a buffer
  const int t_bytes = (chunk * tok * (int)sizeof(T) + 15) & ~15;
  const int buf_bytes = t_bytes + (DECAY == DECAY_PER_CHANNEL ? chunk * dk * 4 : DECAY == DECAY_PER_TOKEN ? ((chunk * 4 + 15) & ~15) : 0);
  pdl_wait();
  const int n_all = seq_q_len[seq];
  const int seg_first = n_segs > 1 ? seg * seg_len : 0;
  if (n_all <= seg_first) return;
  const int n = n_segs > 1 ? min(seg_len, n_all - seg_first) : n_all;
  const int row0 = seq_q_start[seq] + seg_first;
  const int slot = seq_slot[seq];
  float* S_g = state + (((long long)slot * heads + head) * dk) * dv;
  constexpr int PIECE = 16 / (int)sizeof(T);      // rows in a 16-byte piece of q or k
  auto row_of = [&](int r) { return DEAL ? ((r / PIECE) * ks + kr) * PIECE + (r % PIECE) : kr * ROWS + r; };
  float S[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = row_of(r);
    S[r] = (live && i < dk && seg == 0) ? S_g[(long long)i * dv + col] : 0.0f;   // later stretches start from nothing
  }
  // a later stretch also leaves, per token, the product of the decays from its start (one thread group
  // per head does: the first value column's)
  const bool keeps_cum = DECAY != DECAY_PER_HEAD && n_segs > 1 && seg > 0 && col == 0;
  float cp[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) cp[r] = 1.0f;
  const int valid = min(ROWS, dk - kr * ROWS);     // rows of this thread inside the key size (may be <= 0)
  const float head_decay = DECAY == DECAY_PER_HEAD ? decay[head] : 0.0f;

  auto issue = [&](int first, int b) {
    const int count = min(chunk, n - first);
    T* raw = reinterpret_cast<T*>(scan_smem + (size_t)b * buf_bytes);
    float* dec = reinterpret_cast<float*>(scan_smem + (size_t)b * buf_bytes + t_bytes);
    if (aligned) {
      constexpr int PER = 16 / (int)sizeof(T);               // elements per 16-byte copy
      const int nq = dk / PER, nv = n_cols / PER, na = DECAY == DECAY_PER_CHANNEL ? dk / 4 : 0;
      const int per_token = 2 * nq + nv + na;
      for (int e = threadIdx.x; e < count * per_token; e += SCAN_THREADS) {
        const int t = e / per_token, f = e - t * per_token;
        const long long row = row0 + first + t;
        if (f < nq) cp_async_16(raw + t * tok + f * PER, q + row * q_stride + head * dk + f * PER);
        else if (f < 2 * nq) cp_async_16(raw + t * tok + dk + (f - nq) * PER, k + row * k_stride + head * dk + (f - nq) * PER);
        else if (f < 2 * nq + nv)
          cp_async_16(raw + t * tok + 2 * dk + (f - 2 * nq) * PER, v + row * v_stride + head * dv + col0 + (f - 2 * nq) * PER);
        else
          cp_async_16(dec + t * dk + (f - 2 * nq - nv) * 4, decay + row * ((long long)heads * dk) + head * dk + (f - 2 * nq - nv) * 4);
      }
    } else {
      const int per_token = 2 * dk + n_cols + (DECAY == DECAY_PER_CHANNEL ? dk : 0);
      for (int t = 0; t < count; ++t) {
        const long long row = row0 + first + t;
        for (int f = threadIdx.x; f < per_token; f += SCAN_THREADS) {
          if (f < dk) raw[t * tok + f] = q[row * q_stride + head * dk + f];
          else if (f < 2 * dk) raw[t * tok + f] = k[row * k_stride + head * dk + (f - dk)];
          else if (f < 2 * dk + n_cols) raw[t * tok + f] = v[row * v_stride + head * dv + col0 + (f - 2 * dk)];
          else dec[t * dk + (f - 2 * dk - n_cols)] = decay[row * ((long long)heads * dk) + head * dk + (f - 2 * dk - n_cols)];
        }
      }
    }
    if (DECAY == DECAY_PER_TOKEN && threadIdx.x < count)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dec + threadIdx.x)),
                   "l"(decay + (row0 + first + threadIdx.x) * (long long)heads + head) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // one group of copies per chunk, empty past the end, so that "all but the newest SCAN_BUFFERS - 2
  // groups have landed" always means "this chunk has landed"
#pragma unroll
  for (int j = 0; j < SCAN_BUFFERS - 1; ++j) {
    if (j * chunk < n) issue(j * chunk, j);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  int b = 0;
  for (int first = 0; first < n; first += chunk, b = (b + 1) % SCAN_BUFFERS) {
    const int count = min(chunk, n - first);
    asm volatile("cp.async.wait_group %0;" ::"n"(SCAN_BUFFERS - 2) : "memory");
    __syncthreads();   // this chunk has landed, and the chunk before it has been walked by every warp
    if (first + (SCAN_BUFFERS - 1) * chunk < n) issue(first + (SCAN_BUFFERS - 1) * chunk, (b + SCAN_BUFFERS - 1) % SCAN_BUFFERS);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const T* raw = reinterpret_cast<const T*>(scan_smem + (size_t)b * buf_bytes);
    const float* dec = reinterpret_cast<const float*>(scan_smem + (size_t)b * buf_bytes + t_bytes);
    float* o_row = out + (long long)(row0 + first) * ((long long)heads * dv) + head * dv + col;
    // tokens in groups: a group's loads and products are independent of one another but for the one
    // multiply-add per state element that carries the state on, and its reductions run side by side
    constexpr int GROUP = DECAY == DECAY_PER_CHANNEL ? 2 : 4;
    const int token_decay = DECAY == DECAY_PER_TOKEN;
    const int at = DEAL ? kr * PIECE : (valid > 0 ? kr * ROWS : 0);
    const int piece_stride = DEAL ? ks * PIECE : PIECE;
    auto token = [&](int t) -> float {
      const T* w = raw + t * tok;
      const float vv = to_float(w[2 * dk + my_col]);
      float qq[ROWS], kk[ROWS], aa[ROWS];
      load_rows<T, ROWS, VEC>(w + at, valid, qq, piece_stride);
      load_rows<T, ROWS, VEC>(w + dk + at, valid, kk, piece_stride);
      if (DECAY != DECAY_PER_HEAD) {
        if (token_decay) {
          const float a = dec[t];
#pragma unroll
          for (int r = 0; r < ROWS; ++r) aa[r] = a;
        } else if (VEC) {
#pragma unroll
          for (int r = 0; r < ROWS; r += 4) {      // a thread's rows come in runs of at least four
            const float4 x = *reinterpret_cast<const float4*>(dec + t * dk + row_of(r));
            aa[r] = x.x; aa[r + 1] = x.y; aa[r + 2] = x.z; aa[r + 3] = x.w;
          }
        } else {
          load_rows<float, ROWS, false>(dec + t * dk + at, valid, aa, 0);
        }
        if (keeps_cum) {
          float* c_row = cum + (long long)(row0 + first + t) * ((long long)heads * dk) + head * dk;
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            cp[r] *= aa[r];
            if (r < valid) c_row[row_of(r)] = cp[r];
          }
        }
      }
      float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const float a = DECAY != DECAY_PER_HEAD ? aa[r] : head_decay;
        S[r] = a * S[r] + kk[r] * vv;
        part[r & 3] += S[r] * qq[r];
      }
      return (part[0] + part[1]) + (part[2] + part[3]);
    };
    int t0 = 0;
    for (; t0 + GROUP <= count; t0 += GROUP) {      // whole groups: straight-line code
      float accs[GROUP];
#pragma unroll
      for (int g = 0; g < GROUP; ++g) accs[g] = token(t0 + g);
      for (int o = ks >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int g = 0; g < GROUP; ++g) accs[g] += __shfl_xor_sync(0xffffffffu, accs[g], o);
      }
      if (live && kr == 0) {
#pragma unroll
        for (int g = 0; g < GROUP; ++g) o_row[(long long)(t0 + g) * ((long long)heads * dv)] = accs[g] * q_scale;
      }
    }
    for (; t0 < count; ++t0) {                       // the chunk's last tokens
      float acc = token(t0);
      for (int o = ks >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && kr == 0) o_row[(long long)t0 * ((long long)heads * dv)] = acc * q_scale;
    }
  }
  if (n_segs > 1) {
    S_g = seg_state + ((((long long)seq * n_segs + seg) * heads + head) * dk) * dv;
    if (keeps_cum) {
      float* d_row = seg_decay + (((long long)seq * n_segs + seg) * heads + head) * dk;
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
        if (r < valid) d_row[row_of(r)] = cp[r];
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = row_of(r);
    if (live && i < dk) S_g[(long long)i * dv + col] = S[r];
  }
}

// A long portion is walked as n_segs stretches of seg_len tokens side by side: stretch 0 from the
// request's state, the others from nothing.  With D_p the product of the decays over stretch p and
// E_p the state stretch p ends with, the state the request really has at the start of stretch p is
//   C_0 = state,   C_(p+1) = D_p C_p + E_p   (E_0 already contains C_0),
// and token t of stretch p >= 1 misses (c_t q_t)^T C_p in its output, c_t the product of the decays
// from the stretch's start to t.  This kernel walks p in order per (request, head): it leaves C_p in
// place of E_(p-1) and the final state in the request's slot.
template <int DECAY>
__global__ void scan_carry_kernel(float* __restrict__ state, float* __restrict__ seg_state,
                                  const float* __restrict__ seg_decay, const float* __restrict__ decay,
                                  const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_len,
                                  int heads, int dk, int dv, int seg_len, int n_segs) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y;
  const int n = seq_q_len[seq];
  if (n <= 0) return;
  const int used = (n + seg_len - 1) / seg_len;
  float* S_g = state + (((long long)seq_slot[seq] * heads + head) * dk) * dv;
  const long long per = (long long)dk * dv;
  float* E = seg_state + (((long long)seq * n_segs) * heads + head) * per;      // stretch p at E + p * heads * per
  const float lam = DECAY == DECAY_PER_HEAD ? decay[head] : 0.0f;
  // every state element walks the stretches by itself: one per thread, blockIdx.z times blockDim.x apart
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < dk * dv; e += gridDim.z * blockDim.x) {
    const int i = e / dv;
    float S = E[e];
#pragma unroll 4
    for (int p = 1; p < used; ++p) {
      float* Ep = E + (long long)p * heads * per;
      const int len = min(seg_len, n - p * seg_len);
      const float d = DECAY == DECAY_PER_HEAD
                          ? powf(lam, (float)len)
                          : seg_decay[(((long long)seq * n_segs + p) * heads + head) * dk + i];
      const float mine = Ep[e];
      Ep[e - (long long)heads * per] = S;      // C_p, where E_(p-1) was
      S = d * S + mine;
    }
    S_g[e] = S;
  }
}

#define CORRECT_TOKENS 32
#define CORRECT_THREADS 128

// out[t] += ((c_t q_t)^T C_p) * q_scale for the tokens of stretches p >= 1.  A block takes
// CORRECT_TOKENS tokens of one stretch and one head: C_p and the scaled queries in shared memory.
template <typename T, int DECAY>
__global__ void __launch_bounds__(CORRECT_THREADS)
scan_correct_kernel(const T* __restrict__ q, long long q_stride, const float* __restrict__ decay,
                    const float* __restrict__ cum, const float* __restrict__ seg_state, float* __restrict__ out,
                    const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_q_len, int heads, int dk,
                    int dv, int seg_len, int n_segs, float q_scale) {
  pdl_launch_dependents();
  extern __shared__ float cs[];        // [dk][dv] then [CORRECT_TOKENS][dk]
  float* qs = cs + dk * dv;
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int first = blockIdx.x * CORRECT_TOKENS;      // seg_len is a multiple of CORRECT_TOKENS
  const int n = seq_q_len[seq];
  const int p = first / seg_len;
  if (p == 0 || first >= n) return;
  const int count = min(CORRECT_TOKENS, n - first);
  const long long row0 = seq_q_start[seq] + first;
  const float* C = seg_state + ((((long long)seq * n_segs + (p - 1)) * heads + head) * dk) * dv;
  for (int e = threadIdx.x; e < dk * dv; e += CORRECT_THREADS) cs[e] = C[e];
  const float lam = DECAY == DECAY_PER_HEAD ? decay[head] : 0.0f;
  for (int e = count * dk + threadIdx.x; e < CORRECT_TOKENS * dk; e += CORRECT_THREADS) qs[e] = 0.0f;
  for (int e = threadIdx.x; e < count * dk; e += CORRECT_THREADS) {
    const int t = e / dk, i = e - t * dk;
    const float c = DECAY == DECAY_PER_HEAD ? powf(lam, (float)(first + t - p * seg_len + 1))
                                            : cum[(row0 + t) * ((long long)heads * dk) + head * dk + i];
    qs[e] = to_float(q[(row0 + t) * q_stride + head * dk + i]) * c;
  }
  __syncthreads();
  // a thread takes 4 tokens x 4 neighbouring value columns: per key channel four numbers of the
  // scaled queries and one 16-byte piece of C_p feed sixteen multiply-adds
  const int col_groups = (dv + 3) / 4;
  const bool vec = (dv & 3) == 0;
  for (int tile = threadIdx.x; tile < (CORRECT_TOKENS / 4) * col_groups; tile += CORRECT_THREADS) {
    const int cg = tile % col_groups, tg = tile / col_groups;
    if (tg * 4 >= count) continue;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][c] = 0.0f;
    const float* q0 = qs + (tg * 4) * dk;
    for (int i = 0; i < dk; ++i) {
      float cv[4];
      if (vec) {
        const float4 x = *reinterpret_cast<const float4*>(cs + i * dv + cg * 4);
        cv[0] = x.x; cv[1] = x.y; cv[2] = x.z; cv[3] = x.w;
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) cv[c] = cg * 4 + c < dv ? cs[i * dv + cg * 4 + c] : 0.0f;
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float qv = q0[a * dk + i];      // rows past `count` are zero and never stored
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][c] += qv * cv[c];
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int t = tg * 4 + a;
      if (t >= count) continue;
      float* o = out + (row0 + t) * ((long long)heads * dv) + head * dv + cg * 4;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (cg * 4 + c < dv) o[c] += acc[a][c] * q_scale;
    }
  }
}

template <typename T, int DECAY, int ROWS, bool VEC, bool DEAL>
static int scan_launch(dim3 grid, size_t smem, cudaStream_t stream, const void* q, const void* k, const void* v,
                       long long q_stride, long long k_stride, long long v_stride, const float* decay, float* state,
                       float* out, const int32_t* seq_slot, const int32_t* seq_q_start, const int32_t* seq_q_len,
                       int heads, int dk, int dv, int ks, int chunk, int aligned, float q_scale, int seg_len, int n_segs,
                       int slices, float* seg_state, float* seg_decay, float* cum) {
  auto kern = linear_attention_scan_kernel<T, DECAY, ROWS, VEC, DEAL>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return launch_status();
  launch_kernel(kern, grid, SCAN_THREADS, smem, stream, (const T*)q, (const T*)k, (const T*)v, q_stride, k_stride,
                v_stride, decay, state, out, seq_slot, seq_q_start, seq_q_len, heads, dk, dv, ks, chunk, aligned, q_scale,
                seg_len, n_segs, slices, seg_state, seg_decay, cum);
  return launch_status();
}

extern "C" int llm_linear_attention_scan(const void* q, const void* k, const void* v, int dtype, long long q_stride,
                                         long long k_stride, long long v_stride, const float* decay, int per_channel,
                                         float* state, float* out, const int32_t* seq_slot,
                                         const int32_t* seq_q_start, const int32_t* seq_q_len, int n_seqs, int heads,
                                         int dk, int dv, float q_scale, int seg_len, int n_segs, float* seg_state,
                                         float* seg_decay, float* cum, int max_q_len, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  LLM_HOST_CHECK(per_channel >= 0 && per_channel <= 2, ERR_BAD_SIZE);
  LLM_HOST_CHECK(n_segs >= 1 && (n_segs == 1 || (seg_len > 0 && seg_len % CORRECT_TOKENS == 0 && seg_state &&
                                                 (!per_channel || (seg_decay && cum)))), ERR_BAD_SIZE);
  LLM_HOST_CHECK(dk >= 1 && dk <= 256 && dv >= 1 && heads >= 1 && heads <= 65535, ERR_BAD_SIZE);
  LLM_HOST_CHECK(dtype == DT_F32 || dtype == DT_BF16, ERR_BAD_DTYPE);
  const int rows = dk <= 32 ? 8 : 16;
  int ks = 1;
  while (ks * rows < dk) ks <<= 1;          // row groups: a power of two, at most 16
  const int cols_per_block = (32 / ks) * SCAN_WARPS;
  const int slices = (dv + cols_per_block - 1) / cols_per_block;
  const int esize = dtype == DT_F32 ? 4 : 2;
  const int token_bytes = (2 * dk + cols_per_block) * esize + (per_channel == 1 ? dk * 4 : per_channel == 2 ? 4 : 0);
  int chunk = 16;
  while (chunk > 2 && chunk * token_bytes > 16 * 1024) chunk >>= 1;
  const size_t smem = SCAN_BUFFERS * (size_t)(((chunk * (2 * dk + cols_per_block) * esize + 15) & ~15) +
                                              (per_channel == 1 ? chunk * dk * 4 : per_channel == 2 ? ((chunk * 4 + 15) & ~15) : 0));
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  // 16-byte copies need every head slice of every row to start and end on a 16-byte boundary
  const int per = 16 / esize;
  auto ok = [&](const void* p, long long stride) { return ((uintptr_t)p % 16) == 0 && stride % per == 0; };
  int aligned = ok(q, q_stride) && ok(k, k_stride) && ok(v, v_stride) && dk % per == 0 && dv % per == 0 &&
                cols_per_block % per == 0 && (per_channel != 1 || (dk % 4 == 0 && ((uintptr_t)decay % 16) == 0));
  dim3 grid(n_seqs, heads, slices * n_segs);
  LLM_HOST_CHECK(grid.z <= 65535, ERR_BAD_SIZE);
  // 16-byte loads of a thread's rows from shared memory: the threads' rows cover the key size exactly, and
  // the buffers' token stride a multiple of 16 bytes (the aligned copies give the rest)
  const bool vec = aligned && dk == ks * rows && ((2 * dk + cols_per_block) * esize) % 16 == 0;
#define GO(T, DEC, ROWS)                                                                                        \
  do {                                                                                                          \
    if (vec && max_q_len > 4)                                                                                   \
      return scan_launch<T, DEC, ROWS, true, true>(grid, smem, stream, q, k, v, q_stride, k_stride, v_stride, decay, \
                                             state, out, seq_slot, seq_q_start, seq_q_len, heads, dk, dv, ks,   \
                                             chunk, aligned, q_scale, seg_len, n_segs, slices, seg_state, seg_decay, cum); \
    if (vec)                                                                                                    \
      return scan_launch<T, DEC, ROWS, true, false>(grid, smem, stream, q, k, v, q_stride, k_stride, v_stride, decay, \
                                             state, out, seq_slot, seq_q_start, seq_q_len, heads, dk, dv, ks,   \
                                             chunk, aligned, q_scale, seg_len, n_segs, slices, seg_state, seg_decay, cum); \
    return scan_launch<T, DEC, ROWS, false, false>(grid, smem, stream, q, k, v, q_stride, k_stride, v_stride, decay, \
                                            state, out, seq_slot, seq_q_start, seq_q_len, heads, dk, dv, ks,    \
                                            chunk, aligned, q_scale, seg_len, n_segs, slices, seg_state, seg_decay, cum); \
  } while (0)
  if (dtype == DT_F32) {
    if (per_channel == 2) { if (rows == 8) GO(float, 2, 8); else GO(float, 2, 16); }
    else if (per_channel) { if (rows == 8) GO(float, 1, 8); else GO(float, 1, 16); }
    else { if (rows == 8) GO(float, 0, 8); else GO(float, 0, 16); }
  } else {
    if (per_channel == 2) { if (rows == 8) GO(__nv_bfloat16, 2, 8); else GO(__nv_bfloat16, 2, 16); }
    else if (per_channel) { if (rows == 8) GO(__nv_bfloat16, 1, 8); else GO(__nv_bfloat16, 1, 16); }
    else { if (rows == 8) GO(__nv_bfloat16, 0, 8); else GO(__nv_bfloat16, 0, 16); }
  }
#undef GO
  return ERR_BAD_SIZE;
}

// After a scan in n_segs > 1 stretches: the states the stretches really start from, the request's
// final state, and what the later stretches' outputs miss.  `max_q_len`: the longest portion.
extern "C" int llm_linear_attention_join(const void* q, int dtype, long long q_stride, const float* decay,
                                         int per_channel, float* state, float* out, const int32_t* seq_slot,
                                         const int32_t* seq_q_start, const int32_t* seq_q_len, int n_seqs, int heads,
                                         int dk, int dv, float q_scale, int seg_len, int n_segs, int max_q_len,
                                         float* seg_state, const float* seg_decay, const float* cum,
                                         cudaStream_t stream) {
  if (n_seqs <= 0 || n_segs <= 1) return 0;
  LLM_HOST_CHECK(seg_len > 0 && seg_len % CORRECT_TOKENS == 0 && n_seqs <= 65535 && heads <= 65535, ERR_BAD_SIZE);
  dim3 carry_grid(n_seqs, heads, (dk * dv + 1023) / 1024);
  if (per_channel)
    launch_kernel(scan_carry_kernel<1>, carry_grid, 256, 0, stream, state, seg_state, seg_decay, decay, seq_slot,
                  seq_q_len, heads, dk, dv, seg_len, n_segs);
  else
    launch_kernel(scan_carry_kernel<0>, carry_grid, 256, 0, stream, state, seg_state, seg_decay, decay, seq_slot,
                  seq_q_len, heads, dk, dv, seg_len, n_segs);
  int status = launch_status();
  if (status) return status;
  const size_t smem = ((size_t)dk * dv + (size_t)CORRECT_TOKENS * dk) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  dim3 grid((max_q_len + CORRECT_TOKENS - 1) / CORRECT_TOKENS, heads, n_seqs);
#define GO(T, DEC)                                                                                                  \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(scan_correct_kernel<T, DEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    launch_kernel(scan_correct_kernel<T, DEC>, grid, CORRECT_THREADS, smem, stream, (const T*)q, q_stride, decay, cum, \
                  seg_state, out, seq_q_start, seq_q_len, heads, dk, dv, seg_len, n_segs, q_scale);                  \
  } while (0)
  if (dtype == DT_F32) { if (per_channel) GO(float, 1); else GO(float, 0); }
  else if (dtype == DT_BF16) { if (per_channel) GO(__nv_bfloat16, 1); else GO(__nv_bfloat16, 0); }
  else return ERR_BAD_DTYPE;
#undef GO
  return launch_status();
}

// ----------------------------------------------------------------------------- decay gate

#define GATE_ROWS 16      // token rows a block takes
#define GATE_THREADS 128  // channels a block takes

// a[t][c] = sigmoid(z)^(1/tau), z = sum_r up[c][r] low[t][r] + bias[c], as exp(-softplus(-z) / tau).
// A block takes GATE_ROWS tokens and GATE_THREADS channels; a thread owns one channel, reads its
// row of `up` once, eight numbers at a time, and uses it for every token of the block.
template <typename T>
__global__ void __launch_bounds__(GATE_THREADS)
decay_gate_kernel(const T* __restrict__ low, long long low_stride, const float* __restrict__ up,
                  const float* __restrict__ bias, float* __restrict__ out, int rows, int channels, int rank,
                  float inv_tau) {
  pdl_launch_dependents();
  extern __shared__ float low_rows[];    // [GATE_ROWS][rank]
  pdl_wait();
  const int t0 = blockIdx.y * GATE_ROWS;
  const int n = min(GATE_ROWS, rows - t0);
  for (int e = threadIdx.x; e < n * rank; e += GATE_THREADS)
    low_rows[e] = to_float(low[(long long)(t0 + e / rank) * low_stride + e % rank]);
  __syncthreads();
  const int c = blockIdx.x * GATE_THREADS + threadIdx.x;
  if (c >= channels) return;
  float z[GATE_ROWS];
#pragma unroll
  for (int t = 0; t < GATE_ROWS; ++t) z[t] = 0.0f;
  const float* urow = up + (long long)c * rank;
  for (int r0 = 0; r0 < rank; r0 += 8) {
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = r0 + j < rank ? urow[r0 + j] : 0.0f;
#pragma unroll
    for (int t = 0; t < GATE_ROWS; ++t) {
      if (t < n) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (r0 + j < rank) z[t] += w[j] * low_rows[t * rank + r0 + j];
      }
    }
  }
  const float b = bias ? bias[c] : 0.0f;
#pragma unroll
  for (int t = 0; t < GATE_ROWS; ++t) {
    if (t < n) {
      const float zz = z[t] + b;
      const float sp = fmaxf(-zz, 0.0f) + log1pf(expf(-fabsf(zz)));   // softplus(-z)
      out[(long long)(t0 + t) * channels + c] = expf(-sp * inv_tau);
    }
  }
}

extern "C" int llm_decay_gate(const void* low, int dtype, long long low_stride, const float* up, const float* bias,
                              float* out, int rows, int channels, int rank, float inv_tau, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)GATE_ROWS * rank * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  dim3 grid((channels + GATE_THREADS - 1) / GATE_THREADS, (rows + GATE_ROWS - 1) / GATE_ROWS);
  LLM_HOST_CHECK(grid.y <= 65535, ERR_BAD_SIZE);
  if (dtype == DT_F32)
    launch_kernel(decay_gate_kernel<float>, grid, GATE_THREADS, smem, stream, (const float*)low, low_stride, up, bias,
                  out, rows, channels, rank, inv_tau);
  else if (dtype == DT_BF16)
    launch_kernel(decay_gate_kernel<__nv_bfloat16>, grid, GATE_THREADS, smem, stream, (const __nv_bfloat16*)low,
                  low_stride, up, bias, out, rows, channels, rank, inv_tau);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------ gated group norm

#define GATE_SIGMOID 0
#define GATE_SILU 1

// One warp (WIDE: one block of 256 threads) per (row, group): out = x / sqrt(mean_group(x^2) + eps) *
// weight[c % weight_len] * gate_act(gate) * out_scale.  A group is `group` neighbouring channels
// of the row.  Which form runs depends on the group's size only.
template <typename TG, typename TO, bool WIDE>
__global__ void gated_group_norm_kernel(const float* __restrict__ x, const TG* __restrict__ gate, long long gate_stride,
                                        const float* __restrict__ weight, int weight_len, TO* __restrict__ out,
                                        long long out_stride, int rows, int channels, int group, int gate_kind,
                                        float eps, float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int groups = channels / group;
  const long long item = WIDE ? (long long)blockIdx.x : (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * groups) return;
  const long long r = item / groups;
  const int g = (int)(item - r * groups);
  const int lane = WIDE ? threadIdx.x : threadIdx.x & 31;
  const int step = WIDE ? blockDim.x : 32;
  const float* xr = x + r * channels + (long long)g * group;
  float sq = 0.0f;
  for (int i = lane; i < group; i += step) sq += xr[i] * xr[i];
  sq = WIDE ? block_sum(sq, scratch) : warp_sum(sq);
  const float scale = 1.0f / sqrtf(sq / (float)group + eps);
  for (int i = lane; i < group; i += step) {
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
  const bool wide = group >= 512;
  const int blocks = wide ? (int)items : (int)((items + warps - 1) / warps);
#define LAUNCH(TG, TO)                                                                                            \
  do {                                                                                                            \
    if (wide)                                                                                                     \
      launch_kernel(gated_group_norm_kernel<TG, TO, true>, blocks, 256, 0, stream, x, (const TG*)gate, gate_stride, \
                    weight, weight_len, (TO*)out, out_stride, rows, channels, group, gate_kind, eps, out_scale);  \
    else                                                                                                          \
      launch_kernel(gated_group_norm_kernel<TG, TO, false>, blocks, warps * 32, 0, stream, x, (const TG*)gate,    \
                    gate_stride, weight, weight_len, (TO*)out, out_stride, rows, channels, group, gate_kind, eps, \
                    out_scale);                                                                                   \
  } while (0)
  if (gate_dtype == DT_F32 && out_dtype == DT_F32) LAUNCH(float, float);
  else if (gate_dtype == DT_BF16 && out_dtype == DT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (gate_dtype == DT_F32 && out_dtype == DT_BF16) LAUNCH(float, __nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}
