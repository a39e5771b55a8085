// Row-wise kernels of the decoder: embedding gather, (residual add +) RMSNorm, per-head
// QK-norm + rotary embedding + KV page write, SwiGLU. Each is templated on the storage type
// (float for the true 32-bit path, bf16 for serving); all arithmetic is in 32-bit floats and
// the bf16 instantiation rounds where the reference's bf16 tensors round.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[t, :] = table[id, :]   (layover/model.py:219,247: no scaling). The id is ids[t], or, where
// token_src[t] >= 0, the last token in record token_src[t] of the per-request records: a step may
// be launched before the host has read the token that the step before it sampled.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ token_src,
                             const int* __restrict__ records, const T* __restrict__ table, T* __restrict__ x,
                             int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  int id = ids[blockIdx.x];
  if (token_src && records) {
    const int slot = token_src[blockIdx.x];
    if (slot >= 0) id = records[(size_t)slot * LB_RECORD_WORDS + LB_RECORD_LAST_TOKEN];
  }
  id = min(max(id, 0), vocab - 1);    // a record that was never sampled into cannot index outside the table
  const T* src = table + (size_t)id * hidden;
  T* dst = x + (size_t)blockIdx.x * hidden;
  if (sizeof(T) * hidden % 16 == 0 && ((uintptr_t)table % 16 == 0) && ((uintptr_t)x % 16 == 0)) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const int n = (int)(sizeof(T) * hidden / 16);
    for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

// The same gather into a 32-bit residual stream: x[t, :] = float(table[id, :]).
template <typename T>
__global__ void embed_wide_kernel(const int* __restrict__ ids, const int* __restrict__ token_src,
                                  const int* __restrict__ records, const T* __restrict__ table, float* __restrict__ x,
                                  int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  int id = ids[blockIdx.x];
  if (token_src && records) {
    const int slot = token_src[blockIdx.x];
    if (slot >= 0) id = records[(size_t)slot * LB_RECORD_WORDS + LB_RECORD_LAST_TOKEN];
  }
  id = min(max(id, 0), vocab - 1);
  const T* src = table + (size_t)id * hidden;
  float* dst = x + (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Elem<T>::load(src + i);
}

LB_EXPORT int lb_embed_wide(int dtype, const int* ids, const int* token_src, const int* records, const void* table,
                            float* x, int tokens, int hidden, int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (vocab <= 0) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    lb_launch(embed_wide_kernel<float>, tokens, 256, 0, stream, ids, token_src, records, (const float*)table, x, hidden, vocab);
  else if (dtype == LB_BF16)
    lb_launch(embed_wide_kernel<bf16>, tokens, 256, 0, stream, ids, token_src, records, (const bf16*)table, x, hidden, vocab);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

LB_EXPORT int lb_embed(int dtype, const int* ids, const int* token_src, const int* records, const void* table, void* x,
                       int tokens, int hidden, int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (vocab <= 0) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    lb_launch(embed_kernel<float>, tokens, 256, 0, stream, ids, token_src, records, (const float*)table, (float*)x, hidden,
              vocab);
  else if (dtype == LB_BF16)
    lb_launch(embed_kernel<bf16>, tokens, 256, 0, stream, ids, token_src, records, (const bf16*)table, (bf16*)x, hidden,
              vocab);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- add + RMSNorm
// v = x[row] + delta[row] (sum in 32-bit, rounded to T once; written back to x unless rows are
// picked), out = weight * round_T(v * rsqrt(mean(v^2) + eps))   (layover/model.py:31-36,165-166)
// With `rows`, output row r reads source row rows[r] and x is not written (final norm of the
// wanted rows only). The norm weight is always 32-bit.
// eight (bf16) or four (float) elements per 16-byte access
template <typename T> struct Pack;
template <> struct Pack<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Pack<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      v[2 * i] = __low2float(pair);
      v[2 * i + 1] = __high2float(pair);
    }
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T, bool VEC>
__global__ void add_rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ weight,
                                   T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  extern __shared__ float row_vals[];  // hidden floats + 33 for the reduction
  pdl_launch_dependents();
  pdl_wait();
  float* scratch = row_vals + hidden;
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  T* xr = x + src * hidden;
  const T* dr = delta ? delta + src * hidden : nullptr;
  float ss = 0.f;
  if (VEC) {
    constexpr int N = Pack<T>::N;
    for (int i = threadIdx.x * N; i < hidden; i += blockDim.x * N) {
      float v[N];
      Pack<T>::load(xr + i, v);
      if (dr) {
        float d[N];
        Pack<T>::load(dr + i, d);
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = Elem<T>::round(v[j] + d[j]);
        if (!rows) Pack<T>::store(xr + i, v);
      }
#pragma unroll
      for (int j = 0; j < N; ++j) { row_vals[i + j] = v[j]; ss += v[j] * v[j]; }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = Elem<T>::load(xr + i);
      if (dr) {
        v = Elem<T>::round(v + Elem<T>::load(dr + i));
        if (!rows) Elem<T>::store(xr + i, v);
      }
      row_vals[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)blockIdx.x * hidden;
  if (VEC) {
    constexpr int N = Pack<T>::N;
    for (int i = threadIdx.x * N; i < hidden; i += blockDim.x * N) {
      float v[N];
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = weight[i + j] * Elem<T>::round(row_vals[i + j] * inv);
      Pack<T>::store(o + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      Elem<T>::store(o + i, weight[i] * Elem<T>::round(row_vals[i] * inv));
  }
}

// The same for many rows whose width is exactly one 16-byte piece per thread: a block takes RPB rows
// at once, issues the loads of all of them before any arithmetic and keeps the values in registers.
// Every row's sums are taken in the order of the kernel above, so the results are the same bits.
template <typename T, int RPB>
__global__ void add_rmsnorm_rows_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ weight,
                                        T* __restrict__ out, int n_rows, int hidden, float eps) {
  constexpr int N = Pack<T>::N;
  __shared__ float scratch[RPB][33];
  pdl_launch_dependents();
  const int i = threadIdx.x * N, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float w[N];
#pragma unroll
  for (int j = 0; j < N; j += 4) Pack<float>::load(weight + i + j, *reinterpret_cast<float(*)[4]>(&w[j]));   // weights: no kernel writes them
  pdl_wait();
  float v[RPB][N], d[RPB][N], ss[RPB];
#pragma unroll
  for (int r = 0; r < RPB; ++r) {
    const size_t row = (size_t)blockIdx.x * RPB + r;
#pragma unroll
    for (int j = 0; j < N; ++j) v[r][j] = d[r][j] = 0.f;
    if (row < (size_t)n_rows) {
      Pack<T>::load(x + row * hidden + i, v[r]);
      if (delta) Pack<T>::load(delta + row * hidden + i, d[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < RPB; ++r) {
    const size_t row = (size_t)blockIdx.x * RPB + r;
    if (delta) {
#pragma unroll
      for (int j = 0; j < N; ++j) v[r][j] = Elem<T>::round(v[r][j] + d[r][j]);
      if (row < (size_t)n_rows) Pack<T>::store(x + row * hidden + i, v[r]);
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) sum += v[r][j] * v[r][j];
    sum = warp_sum(sum);
    if (lane == 0) scratch[r][warp] = sum;
  }
  __syncthreads();
  if (threadIdx.x < RPB) {
    float total = 0.f;
    for (int k = 0; k < nwarps; ++k) total += scratch[threadIdx.x][k];
    scratch[threadIdx.x][32] = total;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < RPB; ++r) {
    const size_t row = (size_t)blockIdx.x * RPB + r;
    ss[r] = scratch[r][32];
    const float inv = 1.0f / sqrtf(ss[r] / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < N; ++j) v[r][j] = w[j] * Elem<T>::round(v[r][j] * inv);
    if (row < (size_t)n_rows) Pack<T>::store(out + row * hidden + i, v[r]);
  }
}

template <typename T>
static int launch_add_rmsnorm(void* x, const void* delta, const float* weight, void* out, const int* rows, int n_rows,
                              int hidden, float eps, size_t smem, cudaStream_t stream) {
  constexpr int N = Pack<T>::N;
  const bool vec = hidden % N == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                   (!delta || (uintptr_t)delta % 16 == 0);
  // the sum's order depends on the block size only, and that depends on the width only
  int threads = vec ? ((hidden / N + 31) / 32) * 32 : (hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128));
  if (threads > 512) threads = 512;
  if (threads < 32) threads = 32;
  if (vec && !rows && n_rows >= 256 && hidden == threads * N && (uintptr_t)weight % 16 == 0) {
    constexpr int RPB = 2;
    lb_launch(add_rmsnorm_rows_kernel<T, RPB>, (n_rows + RPB - 1) / RPB, threads, 0, stream, (T*)x, (const T*)delta, weight,
              (T*)out, n_rows, hidden, eps);
    return lb_last_error();
  }
  if (vec) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lb_launch(add_rmsnorm_kernel<T, true>, n_rows, threads, smem, stream, (T*)x, (const T*)delta, weight, (T*)out, rows,
              hidden, eps);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lb_launch(add_rmsnorm_kernel<T, false>, n_rows, threads, smem, stream, (T*)x, (const T*)delta, weight, (T*)out, rows,
              hidden, eps);
  }
  return lb_last_error();
}

LB_EXPORT int lb_add_rmsnorm(int dtype, void* x, const void* delta, const float* weight, void* out,
                             const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  if (smem > 200 * 1024) return LB_ERR_SIZE;
  if (dtype == LB_F32) return launch_add_rmsnorm<float>(x, delta, weight, out, rows, n_rows, hidden, eps, smem, stream);
  if (dtype == LB_BF16) return launch_add_rmsnorm<bf16>(x, delta, weight, out, rows, n_rows, hidden, eps, smem, stream);
  return LB_ERR_DTYPE;
}

// ---------------------------------------------------------------- rotary tables
// table[t][0][i] = cos(pos_t * inv_freq[i]), table[t][1][i] = sin(...), 32-bit (layover/model.py:193-197).
// Made once per step and read by every layer, as the reference makes its tables once per call.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ table, int tokens, int n_freq) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * n_freq) return;
  const int t = idx / n_freq, i = idx - t * n_freq;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  table[((size_t)t * 2) * n_freq + i] = cs;
  table[((size_t)t * 2 + 1) * n_freq + i] = sn;
}

LB_EXPORT int lb_rope_table(const int* positions, const float* inv_freq, float* table, int tokens, int n_freq,
                            cudaStream_t stream) {
  const int total = tokens * n_freq;
  if (total <= 0) return 0;
  lb_launch(rope_table_kernel, (total + 255) / 256, 256, 0, stream, positions, inv_freq, table, tokens, n_freq);
  return lb_last_error();
}

// ---------------------------------------------------------------- QK-norm + rotary + KV write
// Over the (token, head) items of the fused projection row [q heads | k heads | v heads] x dim
// (dim a multiple of 16; rows, outputs and pages 16-byte aligned).
//   q, k: per-head RMSNorm over dim (weight shared by the heads, layover/model.py:124-125), then
//         x*cos + rotate_half(x)*sin with cos/sin from the step's table, rounded to T
//         (layover/model.py:100-102,127-128,193-197); dims >= 2*n_freq pass through unrotated.
//   q is written to q_out [tokens, q_heads, dim]; k and v go to their page:
//         pool[(page * kv_heads + head) * page_tokens + slot][dim], page*page_tokens+slot = slot_map[t]
//         (layover/model.py:133,139-140).
// Null norm weights skip the norm, a null table skips the rotation, null pools skip the write
// (then k is written back in place into the projection row, for a position encoding that runs
// as a separate step), a null q_out skips the q heads (the pass that only writes pages).
// A group of `lanes` lanes (a power of two) serves ROUNDS (1 or 2) consecutive heads of ONE token
// (ROUNDS divides the number of heads), each lane one 16-byte piece of each half of a head; a warp serves
// 32 / lanes such groups. The token's cos/sin pieces are read once for all the group's heads, and
// the loads of all rounds are issued before any arithmetic, so that enough bytes are in flight.
template <typename T, int ROUNDS>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, const float* __restrict__ rope_table,
                                       const int* __restrict__ slot_map,
                                       int tokens, int q_heads, int kv_heads, int dim, int n_freq, int page_tokens,
                                       float eps, int lanes) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int N = Pack<T>::N;
  const int heads = q_heads + 2 * kv_heads, half = dim >> 1;
  const int per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31, sub = lane / lanes, i0 = (lane % lanes) * N;
  const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long total = (long)tokens * heads;
  const long first = (warp * per_warp + sub) * ROUNDS;      // this group's heads: first .. first + ROUNDS - 1
  const bool mine = i0 < half, live = first < total;        // heads % ROUNDS == 0: a group is all live or all not
  const int t = live ? (int)(first / heads) : 0, h0 = live ? (int)(first % heads) : 0;

  float lo[ROUNDS][N], hi[ROUNDS][N], cs[N], sn[N];
  const bool rotate = rope_table && i0 + N <= n_freq;    // n_freq = half whenever a table is given
#pragma unroll
  for (int j = 0; j < N; ++j) { cs[j] = 1.f; sn[j] = 0.f; }
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
#pragma unroll
    for (int j = 0; j < N; ++j) lo[r][j] = hi[r][j] = 0.f;
    if (live && mine) {
      const T* src = qkv + (size_t)(first + r) * dim;
      Pack<T>::load(src + i0, lo[r]);
      Pack<T>::load(src + i0 + half, hi[r]);
    }
  }
  if (live && mine && rotate && h0 < q_heads + kv_heads) {     // the table's values travel with the data
    const float* cos_row = rope_table + ((size_t)t * 2) * n_freq + i0;
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      float c4[4], s4[4];
      Pack<float>::load(cos_row + j, c4);
      Pack<float>::load(cos_row + n_freq + j, s4);
#pragma unroll
      for (int e = 0; e < 4; ++e) { cs[j + e] = Elem<T>::round(c4[e]); sn[j + e] = Elem<T>::round(s4[e]); }
    }
  }
  int slot = 0;
  if (live && h0 + ROUNDS > q_heads && (k_pool || v_pool)) slot = slot_map[t];
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const int h = h0 + r;
    const bool is_q = h < q_heads, is_k = !is_q && h < q_heads + kv_heads;
    T* dst = nullptr;
    if (live) {
      if (is_q) {
        dst = q_out ? q_out + ((size_t)t * q_heads + h) * dim : nullptr;   // null: a pass that only writes pages
      } else {
        T* pool = is_k ? k_pool : v_pool;
        if (pool) {
          const int kvh = is_k ? h - q_heads : h - q_heads - kv_heads;
          const size_t page = slot / page_tokens, within = slot % page_tokens;
          dst = pool + ((page * kv_heads + kvh) * page_tokens + within) * dim;
        } else {
          dst = is_k ? qkv + (size_t)(first + r) * dim : nullptr;          // k goes back in place, v stays
        }
      }
    }
    const float* w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) ss += lb_square_pair(lo[r][j], hi[r][j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      if (o < lanes) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // whole groups agree, every lane joins
    if (!dst || !mine) continue;
    if (w) {
      const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        lo[r][j] = Elem<T>::round(w[i0 + j] * Elem<T>::round(lo[r][j] * inv));
        hi[r][j] = Elem<T>::round(w[i0 + j + half] * Elem<T>::round(hi[r][j] * inv));
      }
    }
    if (rotate && (is_q || is_k)) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        // rotate_half(x) = (-hi, lo): each product and the sum round to T
        const float a = Elem<T>::round(Elem<T>::round(lo[r][j] * cs[j]) + Elem<T>::round(-hi[r][j] * sn[j]));
        const float b = Elem<T>::round(Elem<T>::round(hi[r][j] * cs[j]) + Elem<T>::round(lo[r][j] * sn[j]));
        lo[r][j] = a;
        hi[r][j] = b;
      }
    }
    Pack<T>::store(dst + i0, lo[r]);
    Pack<T>::store(dst + i0 + half, hi[r]);
  }
}

template <typename T, int ROUNDS>
static void launch_qk_norm_rope_kv(void* qkv, void* q_out, void* k_pool, void* v_pool, const float* q_norm_w,
                                   const float* k_norm_w, const float* rope_table, const int* slot_map, int tokens,
                                   int q_heads, int kv_heads, int dim, int n_freq, int page_tokens, float eps, int lanes,
                                   cudaStream_t stream) {
  const long groups = (long)tokens * (q_heads + 2 * kv_heads) / ROUNDS;
  const int per_warp = 32 / lanes, threads = 128;
  const long warps = (groups + per_warp - 1) / per_warp;
  const long blocks = (warps * 32 + threads - 1) / threads;
  lb_launch(qk_norm_rope_kv_kernel<T, ROUNDS>, (unsigned)blocks, threads, 0, stream, (T*)qkv, (T*)q_out, (T*)k_pool,
            (T*)v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads, kv_heads, dim, n_freq, page_tokens, eps,
            lanes);
}

template <typename T>
static void dispatch_qk_norm_rope_kv(void* qkv, void* q_out, void* k_pool, void* v_pool, const float* q_norm_w,
                                     const float* k_norm_w, const float* rope_table, const int* slot_map, int tokens,
                                     int q_heads, int kv_heads, int dim, int n_freq, int page_tokens, float eps, int lanes,
                                     cudaStream_t stream) {
  const int heads = q_heads + 2 * kv_heads;
  // two heads share the read of the token's cos/sin row; four measured slower (29 against 23 us for
  // 2,048 tokens of 48 heads: 114 registers a thread leave too few warps in flight)
  if (heads % 2 == 0)
    launch_qk_norm_rope_kv<T, 2>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                 kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
  else
    launch_qk_norm_rope_kv<T, 1>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                 kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
}

LB_EXPORT int lb_qk_norm_rope_kv(int dtype, void* qkv, void* q_out, void* k_pool, void* v_pool,
                                 const float* q_norm_w, const float* k_norm_w, const float* rope_table,
                                 const int* slot_map, int tokens, int q_heads, int kv_heads, int dim, int n_freq,
                                 int page_tokens, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim % 16 || dim > 512 || 2 * n_freq > dim) return LB_ERR_SIZE;   // one 16-byte piece of each half per lane
  // a rotation pairs i with i + dim/2 only when the rotary part spans the whole head
  if (rope_table && 2 * n_freq != dim) return LB_ERR_SIZE;
  const int piece = dtype == LB_BF16 ? 8 : 4;               // elements in 16 bytes
  int lanes = 1;
  while (lanes * piece * 2 < dim) lanes *= 2;
  if (dtype == LB_F32)
    dispatch_qk_norm_rope_kv<float>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                    kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
  else if (dtype == LB_BF16)
    dispatch_qk_norm_rope_kv<bf16>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                   kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- SwiGLU
// out[t, j] = silu(gu[t, j]) * gu[t, inter + j], silu(z) = z / (1 + exp(-z)); silu and the
// product each round to T (layover/model.py:152-153).
// `block` 0: the row is [all gates | all ups]. `block` b > 0: gates and ups alternate in blocks of b
// features ([b gates | b ups | b gates | ...]), the layout of the products' fused epilogue.
// ACT 0: silu (above); ACT 1: relu (max(z, 0), exact in T, so only the product rounds);
// ACT 2: the tanh form of gelu, 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
template <int ACT> __device__ __forceinline__ float gate_activation(float g) {
  if (ACT == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return ACT == 1 ? fmaxf(g, 0.f) : g / (1.0f + expf(-g));
}

template <typename T, bool VEC, int ACT = 0>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long total, int inter, int block) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int N = VEC ? Pack<T>::N : 1;
  const long idx = ((long)blockIdx.x * blockDim.x + threadIdx.x) * N;
  if (idx >= total) return;
  const long t = idx / inter;
  const int j = (int)(idx - t * inter);
  const T* gp = gate_up + t * 2 * inter + (block > 0 ? (j / block) * 2 * block + j % block : j);
  const int up_at = block > 0 ? block : inter;
  if (VEC) {
    float g[Pack<T>::N], u[Pack<T>::N];
    Pack<T>::load(gp, g);
    Pack<T>::load(gp + up_at, u);
#pragma unroll
    for (int i = 0; i < Pack<T>::N; ++i) g[i] = Elem<T>::round(gate_activation<ACT>(g[i])) * u[i];
    Pack<T>::store(out + idx, g);
  } else {
    const float g = Elem<T>::load(gp), u = Elem<T>::load(gp + up_at);
    Elem<T>::store(out + idx, Elem<T>::round(gate_activation<ACT>(g)) * u);
  }
}

template <typename T, int ACT = 0>
static int launch_swiglu(const void* gate_up, void* out, long total, int inter, int block, cudaStream_t stream) {
  constexpr int N = Pack<T>::N;
  const bool vec = inter % N == 0 && (block == 0 || block % N == 0) && (uintptr_t)gate_up % 16 == 0 &&
                   (uintptr_t)out % 16 == 0;
  const int threads = 256;
  const long work = vec ? total / N : total;
  const unsigned blocks = (unsigned)((work + threads - 1) / threads);
  if (vec) lb_launch(swiglu_kernel<T, true, ACT>, blocks, threads, 0, stream, (const T*)gate_up, (T*)out, total, inter, block);
  else lb_launch(swiglu_kernel<T, false, ACT>, blocks, threads, 0, stream, (const T*)gate_up, (T*)out, total, inter, block);
  return lb_last_error();
}

LB_EXPORT int lb_swiglu(int dtype, const void* gate_up, void* out, int tokens, int inter, int block,
                        cudaStream_t stream) {
  const long total = (long)tokens * inter;
  if (total <= 0) return 0;
  if (block < 0 || (block > 0 && inter % block)) return LB_ERR_SIZE;
  if (dtype == LB_F32) return launch_swiglu<float>(gate_up, out, total, inter, block, stream);
  if (dtype == LB_BF16) return launch_swiglu<bf16>(gate_up, out, total, inter, block, stream);
  return LB_ERR_DTYPE;
}

// The same gated product with the activation named by the caller: act 0 silu, 1 relu, 2 gelu (tanh form).
template <typename T>
static int launch_gated_act(const void* gate_up, void* out, long total, int inter, int block, int act, cudaStream_t stream) {
  if (act == 2) return launch_swiglu<T, 2>(gate_up, out, total, inter, block, stream);
  return act ? launch_swiglu<T, 1>(gate_up, out, total, inter, block, stream)
             : launch_swiglu<T, 0>(gate_up, out, total, inter, block, stream);
}

LB_EXPORT int lb_gated_act(int dtype, const void* gate_up, void* out, int tokens, int inter, int block, int act,
                           cudaStream_t stream) {
  const long total = (long)tokens * inter;
  if (total <= 0) return 0;
  if (block < 0 || (block > 0 && inter % block) || act < 0 || act > 2) return LB_ERR_SIZE;
  if (dtype == LB_F32) return launch_gated_act<float>(gate_up, out, total, inter, block, act, stream);
  if (dtype == LB_BF16) return launch_gated_act<bf16>(gate_up, out, total, inter, block, act, stream);
  return LB_ERR_DTYPE;
}

// ---------------------------------------------------------------- 32-bit residual stream: (normed) add + RMSNorm
// For models whose residual stream stays in 32-bit floats whatever the run's type T, and whose
// sub-layers' outputs are RMS-normed before they are added (a norm before and after each sub-layer):
//   v      = x[row] + delta[row] * s + extra[row]
//            s = delta_w * rsqrt(mean(delta[row]^2) + delta_eps) per channel (delta_w null: s = 1);
//            delta and extra may each be null
//   x[row] = v                                         (not with `rows`: then x is only read)
//   out[r] = T(weight * v * rsqrt(mean(v^2) + eps))    (weight null: no output, only the sum)
// Everything is computed in 32-bit and rounded once, at the store of out. One block per row; the
// block size depends on the width only, so a row's sums do not depend on the batch.
// four neighbouring elements with one access (8 bytes of bf16, 16 of float)
template <typename T> struct Four;
template <> struct Four<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Four<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const uint32_t*>(&a);
    r.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

// VEC: the width is a multiple of 4 and every row starts on a 16-byte (8-byte for bf16) boundary.
template <typename T, bool VEC>
__global__ void residual_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                        const float* __restrict__ delta_w, float delta_eps,
                                        const float* __restrict__ extra, const float* __restrict__ weight,
                                        T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps,
                                        float delta_scale) {
  extern __shared__ float row_vals[];  // hidden floats + 33 for the reductions
  pdl_launch_dependents();
  pdl_wait();
  float* scratch = row_vals + hidden;
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* xr = x + src * hidden;
  const T* dr = delta ? delta + src * hidden : nullptr;
  const float* er = extra ? extra + src * hidden : nullptr;
  float dinv = 1.f;
  if (dr && delta_w) {
    float ds = 0.f;
    if (VEC) {
      for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
        const float4 d = Four<T>::load(dr + i);
        ds += d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w;
      }
    } else {
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = Elem<T>::load(dr + i);
        ds += d * d;
      }
    }
    ds = block_sum(ds, scratch);
    dinv = 1.0f / sqrtf(ds / (float)hidden + delta_eps);
  }
  const bool scaled = delta_scale != 1.f;    // the normed output times one more factor: x += scale * (w * d * inv)
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = Four<float>::load(xr + i);
      if (dr) {
        const float4 d = Four<T>::load(dr + i);
        if (delta_w) {
          const float4 w = Four<float>::load(delta_w + i);
          if (scaled) {
            v.x += delta_scale * (d.x * dinv * w.x); v.y += delta_scale * (d.y * dinv * w.y);
            v.z += delta_scale * (d.z * dinv * w.z); v.w += delta_scale * (d.w * dinv * w.w);
          } else {
            v.x += d.x * dinv * w.x; v.y += d.y * dinv * w.y; v.z += d.z * dinv * w.z; v.w += d.w * dinv * w.w;
          }
        } else {
          v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
      }
      if (er) {
        const float4 e = Four<float>::load(er + i);
        v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
      }
      if (!rows && (dr || er)) Four<float>::store(xr + i, v);
      Four<float>::store(row_vals + i, v);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = xr[i];
      if (dr) v += delta_w ? (scaled ? delta_scale * (Elem<T>::load(dr + i) * dinv * delta_w[i]) : Elem<T>::load(dr + i) * dinv * delta_w[i])
                           : Elem<T>::load(dr + i);
      if (er) v += er[i];
      if (!rows && (dr || er)) xr[i] = v;
      row_vals[i] = v;
      ss += v * v;
    }
  }
  if (!weight) {
    if (out) {      // no norm of the sum: the stream itself in the run's type, as the next matrix product reads it
      T* o = out + (size_t)blockIdx.x * hidden;
      __syncthreads();
      if (VEC) for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) Four<T>::store(o + i, Four<float>::load(row_vals + i));
      else for (int i = threadIdx.x; i < hidden; i += blockDim.x) Elem<T>::store(o + i, row_vals[i]);
    }
    return;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)blockIdx.x * hidden;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = Four<float>::load(row_vals + i), w = Four<float>::load(weight + i);
      Four<T>::store(o + i, make_float4(w.x * (v.x * inv), w.y * (v.y * inv), w.z * (v.z * inv), w.w * (v.w * inv)));
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) Elem<T>::store(o + i, weight[i] * (row_vals[i] * inv));
  }
}

template <typename T>
static int launch_residual_rmsnorm(float* x, const void* delta, const float* delta_w, float delta_eps, const float* extra,
                                   const float* weight, void* out, const int* rows, int n_rows, int hidden, float eps,
                                   float delta_scale, cudaStream_t stream) {
  static LbPerDeviceOnce once;
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  if (smem > 200 * 1024) return LB_ERR_SIZE;
  if (smem > 48 * 1024 && once.first()) {
    cudaFuncSetAttribute(residual_rmsnorm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(residual_rmsnorm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  }
  // the form, like the block size, depends on the width and the buffers' alignment only, never on the batch
  const bool vec = hidden % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)extra % 16 == 0 &&
                   (uintptr_t)out % 16 == 0 && (uintptr_t)delta_w % 16 == 0 && (uintptr_t)weight % 16 == 0;
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  if (vec)
    lb_launch(residual_rmsnorm_kernel<T, true>, n_rows, threads, smem, stream, x, (const T*)delta, delta_w, delta_eps, extra,
              weight, (T*)out, rows, hidden, eps, delta_scale);
  else
    lb_launch(residual_rmsnorm_kernel<T, false>, n_rows, threads, smem, stream, x, (const T*)delta, delta_w, delta_eps, extra,
              weight, (T*)out, rows, hidden, eps, delta_scale);
  return lb_last_error();
}

LB_EXPORT int lb_residual_rmsnorm(int dtype, float* x, const void* delta, const float* delta_w, float delta_eps,
                                  const float* extra, const float* weight, void* out, const int* rows, int n_rows,
                                  int hidden, float eps, float delta_scale, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || (weight && !out)) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    return launch_residual_rmsnorm<float>(x, delta, delta_w, delta_eps, extra, weight, out, rows, n_rows, hidden, eps, delta_scale, stream);
  if (dtype == LB_BF16)
    return launch_residual_rmsnorm<bf16>(x, delta, delta_w, delta_eps, extra, weight, out, rows, n_rows, hidden, eps, delta_scale, stream);
  return LB_ERR_DTYPE;
}

// ---------------------------------------------------------------- whole-row QK-norm + KV write + head gates
// For attention whose q and k are RMS-normed over the whole projection (all heads at once, one
// weight per channel) and are not rotated. A token's row of the stacked projection is
//   [ q: q_heads * dim | k: kv_heads * dim | v: kv_heads * vdim | gate logits: q_heads (optional) ].
//   q_out[t]  = T(q * rsqrt(mean(q^2) + eps) * q_w)          (q_w null: q is copied)
//   k page    = T(k * rsqrt(mean(k^2) + eps) * k_w),  v page = v
//               k_pool[((page * kv_heads + g) * page_tokens + slot) * k_room + c], v_pool likewise with v_room,
//               page * page_tokens + slot = slot_map[t]
//   gates[t, h] = 1 / (1 + exp(-logit_h))  in 32-bit          (gates null: the row has no logits)
// A head may have more room where it is written than it has channels (q_room >= dim per head of q_out,
// k_room >= dim and v_room >= vdim per page row: kernels that want keys and values of one size); the
// rest of the room is filled with zeros, which change no score and no weighted sum.
// One block per token; statistics in 32-bit.
template <typename T>
__global__ void qk_rownorm_kv_kernel(const T* __restrict__ proj, long row_stride, T* __restrict__ q_out,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, const float* __restrict__ q_w,
                                     const float* __restrict__ k_w, const int* __restrict__ slot_map,
                                     float* __restrict__ gates, int q_heads, int kv_heads, int dim, int vdim,
                                     int page_tokens, float eps, int q_room, int k_room, int v_room) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, nq = q_heads * dim, nk = kv_heads * dim, nv = kv_heads * vdim;
  const T* row = proj + (size_t)t * row_stride;
  float qinv = 1.f, kinv = 1.f;
  if (q_w) {
    float s = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = Elem<T>::load(row + i); s += v * v; }
    qinv = 1.0f / sqrtf(block_sum(s, scratch) / (float)nq + eps);
  }
  if (k_w) {
    float s = 0.f;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = Elem<T>::load(row + nq + i); s += v * v; }
    kinv = 1.0f / sqrtf(block_sum(s, scratch) / (float)nk + eps);
  }
  T* qo = q_out + (size_t)t * q_heads * q_room;
  for (int i = threadIdx.x; i < q_heads * q_room; i += blockDim.x) {
    const int h = i / q_room, c = i - h * q_room;
    float v = 0.f;
    if (c < dim) {
      v = Elem<T>::load(row + h * dim + c);
      if (q_w) v = v * qinv * q_w[h * dim + c];
    }
    Elem<T>::store(qo + i, v);
  }
  const int slot = slot_map[t];
  const size_t page = (size_t)(slot / page_tokens), in_page = (size_t)(slot % page_tokens);
  for (int i = threadIdx.x; i < kv_heads * k_room; i += blockDim.x) {
    const int g = i / k_room, c = i - g * k_room;
    float v = 0.f;
    if (c < dim) {
      v = Elem<T>::load(row + nq + g * dim + c);
      if (k_w) v = v * kinv * k_w[g * dim + c];
    }
    Elem<T>::store(k_pool + ((page * kv_heads + g) * page_tokens + in_page) * k_room + c, v);
  }
  for (int i = threadIdx.x; i < kv_heads * v_room; i += blockDim.x) {
    const int g = i / v_room, c = i - g * v_room;
    Elem<T>::store(v_pool + ((page * kv_heads + g) * page_tokens + in_page) * v_room + c,
                   c < vdim ? Elem<T>::load(row + nq + nk + g * vdim + c) : 0.f);
  }
  if (gates)
    for (int h = threadIdx.x; h < q_heads; h += blockDim.x)
      gates[(size_t)t * q_heads + h] = 1.0f / (1.0f + expf(-Elem<T>::load(row + nq + nk + nv + h)));
}

LB_EXPORT int lb_qk_rownorm_kv(int dtype, const void* proj, long row_stride, void* q_out, void* k_pool, void* v_pool,
                               const float* q_w, const float* k_w, const int* slot_map, float* gates, int tokens,
                               int q_heads, int kv_heads, int dim, int vdim, int page_tokens, float eps, int q_room,
                               int k_room, int v_room, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || page_tokens <= 0 || q_room < dim || k_room < dim ||
      v_room < vdim)
    return LB_ERR_SIZE;
  const int threads = q_heads * dim >= 1024 ? 256 : 128;
  if (dtype == LB_F32)
    lb_launch(qk_rownorm_kv_kernel<float>, tokens, threads, 0, stream, (const float*)proj, row_stride, (float*)q_out,
              (float*)k_pool, (float*)v_pool, q_w, k_w, slot_map, gates, q_heads, kv_heads, dim, vdim, page_tokens, eps,
              q_room, k_room, v_room);
  else if (dtype == LB_BF16)
    lb_launch(qk_rownorm_kv_kernel<bf16>, tokens, threads, 0, stream, (const bf16*)proj, row_stride, (bf16*)q_out,
              (bf16*)k_pool, (bf16*)v_pool, q_w, k_w, slot_map, gates, q_heads, kv_heads, dim, vdim, page_tokens, eps,
              q_room, k_room, v_room);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- 32-bit residual stream: add + LayerNorm
// For blocks whose sub-layers all read ONE norm of the stream and whose outputs are added together
// (a parallel block): the stream takes up to two not-yet-added outputs at once,
//   v      = x[row] + delta_a[row] + delta_b[row]          (either may be null)
//   x[row] = v                                             (not with `rows`: then x is only read)
//   out[r] = T((v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * weight + bias)   (weight null: only the sum)
// in 32-bit, rounded once at the store of out. The variance is the mean of the squared deviations
// from the mean (two passes over the row, which sits in shared memory). One block per row; the
// block size depends on the width only, so a row's sums do not depend on the batch.
// VEC: the width is a multiple of 4 and every row starts on a 16-byte (8-byte for bf16) boundary: four elements an
// access. Which form runs depends on the width and the buffers' alignment only, never on the batch.
template <typename T, bool VEC>
__global__ void residual_layernorm_kernel(float* __restrict__ x, const T* __restrict__ delta_a,
                                          const T* __restrict__ delta_b, const float* __restrict__ weight,
                                          const float* __restrict__ bias, T* __restrict__ out,
                                          const int* __restrict__ rows, int hidden, float eps) {
  extern __shared__ __align__(16) float row_vals[];  // hidden floats + 33 for the reductions
  pdl_launch_dependents();
  pdl_wait();
  float* scratch = row_vals + hidden;
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* xr = x + src * hidden;
  const T* ar = delta_a ? delta_a + src * hidden : nullptr;
  const T* br = delta_b ? delta_b + src * hidden : nullptr;
  float sum = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = Four<float>::load(xr + i);
      if (ar && br) {                                  // the sub-layers' sum joins the stream
        const float4 a = Four<T>::load(ar + i), b = Four<T>::load(br + i);
        v.x += a.x + b.x; v.y += a.y + b.y; v.z += a.z + b.z; v.w += a.w + b.w;
      } else if (ar || br) {
        const float4 a = Four<T>::load((ar ? ar : br) + i);
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
      }
      if (!rows && (ar || br)) Four<float>::store(xr + i, v);
      Four<float>::store(row_vals + i, v);
      sum += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = xr[i];
      if (ar && br) v += Elem<T>::load(ar + i) + Elem<T>::load(br + i);
      else if (ar) v += Elem<T>::load(ar + i);
      else if (br) v += Elem<T>::load(br + i);
      if (!rows && (ar || br)) xr[i] = v;
      row_vals[i] = v;
      sum += v;
    }
  }
  if (!weight) return;
  const float mean = block_sum(sum, scratch) / (float)hidden;
  float sq = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = Four<float>::load(row_vals + i);
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      sq += (a * a + b * b) + (c * c + d * d);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = row_vals[i] - mean;
      sq += d * d;
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps);
  T* o = out + (size_t)blockIdx.x * hidden;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = Four<float>::load(row_vals + i), w = Four<float>::load(weight + i);
      const float4 b = bias ? Four<float>::load(bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      Four<T>::store(o + i, make_float4((v.x - mean) * inv * w.x + b.x, (v.y - mean) * inv * w.y + b.y,
                                        (v.z - mean) * inv * w.z + b.z, (v.w - mean) * inv * w.w + b.w));
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      Elem<T>::store(o + i, (row_vals[i] - mean) * inv * weight[i] + (bias ? bias[i] : 0.f));
  }
}

template <typename T>
static int launch_residual_layernorm(float* x, const void* delta_a, const void* delta_b, const float* weight, const float* bias,
                                     void* out, const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
  static LbPerDeviceOnce once;
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  if (smem > 200 * 1024) return LB_ERR_SIZE;
  if (smem > 48 * 1024 && once.first()) {
    cudaFuncSetAttribute(residual_layernorm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(residual_layernorm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  }
  const bool vec = hidden % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)delta_a % 16 == 0 && (uintptr_t)delta_b % 16 == 0 &&
                   (uintptr_t)out % 16 == 0 && (uintptr_t)weight % 16 == 0 && (uintptr_t)bias % 16 == 0;
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  if (vec)
    lb_launch(residual_layernorm_kernel<T, true>, n_rows, threads, smem, stream, x, (const T*)delta_a, (const T*)delta_b, weight,
              bias, (T*)out, rows, hidden, eps);
  else
    lb_launch(residual_layernorm_kernel<T, false>, n_rows, threads, smem, stream, x, (const T*)delta_a, (const T*)delta_b, weight,
              bias, (T*)out, rows, hidden, eps);
  return lb_last_error();
}

LB_EXPORT int lb_residual_layernorm(int dtype, float* x, const void* delta_a, const void* delta_b, const float* weight,
                                    const float* bias, void* out, const int* rows, int n_rows, int hidden, float eps,
                                    cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || (weight && !out)) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    return launch_residual_layernorm<float>(x, delta_a, delta_b, weight, bias, out, rows, n_rows, hidden, eps, stream);
  if (dtype == LB_BF16)
    return launch_residual_layernorm<bf16>(x, delta_a, delta_b, weight, bias, out, rows, n_rows, hidden, eps, stream);
  return LB_ERR_DTYPE;
}

// ---------------------------------------------------------------- biases + partial rotation + value blend + KV write
// For attention whose projections have biases, whose rotation covers only the first `2 n_freq`
// channels of a head, and whose values may be blended with the values that an earlier layer made
// for the same token. A token's row of the stacked projection, in 32-bit whatever the run's type, is
//   [ q: q_heads * dim | k: kv_heads * dim | v: kv_heads * vdim | ... ].
//   q, k, v += their biases                                              (each null: none)
//   every q head *= q_norm_w * rsqrt(mean(head^2) + norm_eps), every k head likewise with k_norm_w (weights of
//   `dim` entries shared by the heads; each null: no norm), before the rotation
//   channels i and i + n_freq of every q and k head (i < n_freq) turn by the token's angle i:
//       (u, w) -> (u cos - w sin, w cos + u sin), cos/sin from table[t] ([T, 2, n_freq]; null: no rotation)
//       (flags & 1: neighbouring channels 2i and 2i + 1 turn together instead, by angle i)
//   values: blend 1 stores v (with its bias) to first_v[t] ([T, kv_heads * vdim] floats) and uses it as it is;
//           blend 2 uses (1 - lambda) v + lambda first_v[t]; blend 0 uses v
//           (flags & 2: the row holds no v; a value head is its key head as projected, with the key's bias, before
//           norm and rotation; vdim = dim)
//   q_out[t] = T(q), k page = T(k), v page = T(v), laid out and zero-filled up to each tensor's room per
//   head as in the whole-row kernel above.
// One block per token; all arithmetic 32-bit, rounded once at the stores.
template <typename T>
__global__ void heads_bias_rope_kv_kernel(const float* __restrict__ proj, long row_stride, T* __restrict__ q_out,
                                          T* __restrict__ k_pool, T* __restrict__ v_pool,
                                          const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                          const float* __restrict__ v_bias, const float* __restrict__ table, int n_freq,
                                          const int* __restrict__ slot_map, float* __restrict__ first_v, int blend,
                                          const float* __restrict__ lambda, int q_heads, int kv_heads, int dim, int vdim,
                                          int page_tokens, int q_room, int k_room, int v_room,
                                          const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                                          float norm_eps, int flags) {
  extern __shared__ float head_inv[];     // q_heads + kv_heads: 1 / root mean square of every normed head
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, nq = q_heads * dim, nk = kv_heads * dim;
  const float* row = proj + (size_t)t * row_stride;
  if (q_norm_w || k_norm_w) {             // a warp per head, lanes over its channels: the same sum for every batch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int h = warp; h < q_heads + kv_heads; h += warps) {
      const bool is_q = h < q_heads;
      const float* src = is_q ? row + h * dim : row + nq + (h - q_heads) * dim;
      const float* b = is_q ? q_bias : k_bias;
      if (b) b += (is_q ? h : h - q_heads) * dim;
      float ss = 0.f;
      for (int c = lane; c < dim; c += 32) {
        const float v = src[c] + (b ? b[c] : 0.f);
        ss += v * v;
      }
      ss = warp_sum(ss);
      if (lane == 0) head_inv[h] = (is_q ? q_norm_w : k_norm_w) ? 1.0f / sqrtf(ss / (float)dim + norm_eps) : 1.f;
    }
    __syncthreads();
  }
  const float* cs = table ? table + (size_t)t * 2 * n_freq : nullptr;
  const float* sn = cs ? cs + n_freq : nullptr;
  const int rotated = cs ? 2 * n_freq : 0;
  const int slot = slot_map[t];
  const size_t page = (size_t)(slot / page_tokens), in_page = (size_t)(slot % page_tokens);
  // q and k heads share one loop: head index h over q_heads + kv_heads
  const int qk_items = q_heads * q_room + kv_heads * k_room;
  for (int i = threadIdx.x; i < qk_items; i += blockDim.x) {
    const bool is_q = i < q_heads * q_room;
    const int j = is_q ? i : i - q_heads * q_room;
    const int room = is_q ? q_room : k_room;
    const int h = j / room, c = j - h * room;
    const float* src = row + (is_q ? 0 : nq) + h * dim;
    const float* b = is_q ? q_bias : k_bias;
    if (b) b += h * dim;
    const float* nw = is_q ? q_norm_w : k_norm_w;
    const float inv = nw ? head_inv[is_q ? h : q_heads + h] : 1.f;
    float v = 0.f;
    if (c < dim) {
      v = src[c] + (b ? b[c] : 0.f);
      if (nw) v = v * inv * nw[c];
      if (c < rotated) {
        const bool neighbours = flags & 1;
        const bool first = neighbours ? !(c & 1) : c < n_freq;     // the pair's first member takes the minus sign
        const int f = neighbours ? c >> 1 : (c < n_freq ? c : c - n_freq);
        const int other = neighbours ? c ^ 1 : (c < n_freq ? c + n_freq : c - n_freq);
        float w = src[other] + (b ? b[other] : 0.f);
        if (nw) w = w * inv * nw[other];
        v = first ? v * cs[f] - w * sn[f] : v * cs[f] + w * sn[f];
      }
    }
    if (is_q) Elem<T>::store(q_out + (size_t)t * q_heads * q_room + j, v);
    else Elem<T>::store(k_pool + ((page * kv_heads + h) * page_tokens + in_page) * k_room + c, v);
  }
  const float lam = blend == 2 ? *lambda : 0.f;
  for (int i = threadIdx.x; i < kv_heads * v_room; i += blockDim.x) {
    const int g = i / v_room, c = i - g * v_room;
    float v = 0.f;
    if (c < vdim) {
      const int at = g * vdim + c;
      if (flags & 2) v = row[nq + at] + (k_bias ? k_bias[at] : 0.f);
      else v = row[nq + nk + at] + (v_bias ? v_bias[at] : 0.f);
      if (blend == 1) first_v[(size_t)t * kv_heads * vdim + at] = v;
      else if (blend == 2) v = (1.f - lam) * v + lam * first_v[(size_t)t * kv_heads * vdim + at];
    }
    Elem<T>::store(v_pool + ((page * kv_heads + g) * page_tokens + in_page) * v_room + c, v);
  }
}

LB_EXPORT int lb_heads_bias_rope_kv(int dtype, const float* proj, long row_stride, void* q_out, void* k_pool, void* v_pool,
                                    const float* q_bias, const float* k_bias, const float* v_bias, const float* table,
                                    int n_freq, const int* slot_map, float* first_v, int blend, const float* lambda,
                                    int tokens, int q_heads, int kv_heads, int dim, int vdim, int page_tokens, int q_room,
                                    int k_room, int v_room, const float* q_norm_w, const float* k_norm_w, float norm_eps,
                                    int flags, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || page_tokens <= 0 || q_room < dim || k_room < dim ||
      v_room < vdim || n_freq < 0 || 2 * n_freq > dim || blend < 0 || blend > 2 || (blend && !first_v) ||
      (blend == 2 && !lambda) || ((flags & 2) && vdim != dim))
    return LB_ERR_SIZE;
  const int threads = q_heads * dim >= 1024 ? 256 : 128;
  const size_t smem = (size_t)(q_heads + kv_heads) * sizeof(float);
  if (smem > 32 * 1024) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    lb_launch(heads_bias_rope_kv_kernel<float>, tokens, threads, smem, stream, proj, row_stride, (float*)q_out, (float*)k_pool,
              (float*)v_pool, q_bias, k_bias, v_bias, table, n_freq, slot_map, first_v, blend, lambda, q_heads, kv_heads, dim,
              vdim, page_tokens, q_room, k_room, v_room, q_norm_w, k_norm_w, norm_eps, flags);
  else if (dtype == LB_BF16)
    lb_launch(heads_bias_rope_kv_kernel<bf16>, tokens, threads, smem, stream, proj, row_stride, (bf16*)q_out, (bf16*)k_pool,
              (bf16*)v_pool, q_bias, k_bias, v_bias, table, n_freq, slot_map, first_v, blend, lambda, q_heads, kv_heads, dim,
              vdim, page_tokens, q_room, k_room, v_room, q_norm_w, k_norm_w, norm_eps, flags);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- a sigmoid gate per channel of the heads' outputs
// out[t, h * vdim + c] = T(heads[t, h * room + c] * sigmoid(logits[t, h * vdim + c])): the gate of every
// channel of the concatenated heads, from 32-bit logits that sit in a wider row (`logit_stride` floats
// a token); the heads may come padded to `room` channels each, the output is dense.
// VEC: four channels a thread (sizes, strides and addresses allow 16-byte accesses of the logits).
template <typename T, bool VEC>
__global__ void channel_gate_kernel(const T* __restrict__ heads, const float* __restrict__ logits, long logit_stride,
                                    T* __restrict__ out, long total, int q_heads, int vdim, int room) {
  pdl_launch_dependents();
  pdl_wait();
  const int width = q_heads * vdim;
  if (VEC) {
    for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += (long)gridDim.x * blockDim.x * 4) {
      const long t = i / width;
      const int j = (int)(i - t * width), h = j / vdim, c = j - h * vdim;
      const float4 z = *reinterpret_cast<const float4*>(logits + t * logit_stride + j);
      float4 v = Four<T>::load(heads + (t * q_heads + h) * room + c);
      v.x *= 1.0f / (1.0f + expf(-z.x)); v.y *= 1.0f / (1.0f + expf(-z.y));
      v.z *= 1.0f / (1.0f + expf(-z.z)); v.w *= 1.0f / (1.0f + expf(-z.w));
      Four<T>::store(out + i, v);
    }
    return;
  }
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / width;
    const int j = (int)(i - t * width), h = j / vdim, c = j - h * vdim;
    const float gate = 1.0f / (1.0f + expf(-logits[t * logit_stride + j]));
    Elem<T>::store(out + i, Elem<T>::load(heads + (t * q_heads + h) * room + c) * gate);
  }
}

LB_EXPORT int lb_channel_gate(int dtype, const void* heads, const float* logits, long logit_stride, void* out, int tokens,
                              int q_heads, int vdim, int room, cudaStream_t stream) {
  const long total = (long)tokens * q_heads * vdim;
  if (total <= 0) return 0;
  if (room < vdim) return LB_ERR_SIZE;
  const int threads = 256;
  const bool vec = vdim % 4 == 0 && room % 4 == 0 && logit_stride % 4 == 0 && (uintptr_t)heads % 16 == 0 &&
                   (uintptr_t)logits % 16 == 0 && (uintptr_t)out % 16 == 0;
  const long items = vec ? total / 4 : total;
  const int blocks = (int)((items + threads - 1) / threads < 148 * 16 ? (items + threads - 1) / threads : 148 * 16);
#define LB_GATE_ARGS(T) (const T*)heads, logits, logit_stride, (T*)out, total, q_heads, vdim, room
  if (dtype == LB_F32) {
    if (vec) lb_launch(channel_gate_kernel<float, true>, blocks, threads, 0, stream, LB_GATE_ARGS(float));
    else lb_launch(channel_gate_kernel<float, false>, blocks, threads, 0, stream, LB_GATE_ARGS(float));
  } else if (dtype == LB_BF16) {
    if (vec) lb_launch(channel_gate_kernel<bf16, true>, blocks, threads, 0, stream, LB_GATE_ARGS(bf16));
    else lb_launch(channel_gate_kernel<bf16, false>, blocks, threads, 0, stream, LB_GATE_ARGS(bf16));
  } else
    return LB_ERR_DTYPE;
#undef LB_GATE_ARGS
  return lb_last_error();
}

// ---------------------------------------------------------------- plain activations and the logits' soft cap
// out = act(in) element by element: 0 relu(z)^2, 1 gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))),
// 2 silu(z). 32-bit arithmetic, rounded once.
template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, long total, int act) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const float z = Elem<T>::load(in + i);
    float y;
    if (act == 0) { const float r = fmaxf(z, 0.f); y = r * r; }
    else if (act == 1) y = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    else y = z / (1.f + expf(-z));
    Elem<T>::store(out + i, y);
  }
}

LB_EXPORT int lb_activation(int dtype, const void* in, void* out, long total, int act, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (act < 0 || act > 2) return LB_ERR_SIZE;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == LB_F32) lb_launch(activation_kernel<float>, blocks, threads, 0, stream, (const float*)in, (float*)out, total, act);
  else if (dtype == LB_BF16) lb_launch(activation_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)in, (bf16*)out, total, act);
  else return LB_ERR_DTYPE;
  return lb_last_error();
}

// logits <- cap * tanh(logits / cap), in place, 32-bit.
__global__ void softcap_kernel(float* __restrict__ logits, long total, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x)
    logits[i] = cap * tanhf(logits[i] / cap);
}

LB_EXPORT int lb_softcap(float* logits, long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return LB_ERR_SIZE;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  lb_launch(softcap_kernel, blocks, threads, 0, stream, logits, total, cap);
  return lb_last_error();
}

// ---------------------------------------------------------------- learned positions
// x[t, :] += table[min(positions[t], rows - 1), :] over a 32-bit residual stream (the table in the run's
// type T), and, where `lowered` is given, lowered[t, :] = T(x[t, :]): the stream as the first layer's
// matrix products read it.
template <typename T>
__global__ void add_position_rows_kernel(float* __restrict__ x, const int* __restrict__ positions,
                                         const T* __restrict__ table, int rows, int hidden, T* __restrict__ lowered) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = min(max(positions[blockIdx.x], 0), rows - 1);
  const T* src = table + (size_t)p * hidden;
  float* dst = x + (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = dst[i] + Elem<T>::load(src + i);
    dst[i] = v;
    if (lowered) Elem<T>::store(lowered + (size_t)blockIdx.x * hidden + i, v);
  }
}

LB_EXPORT int lb_add_position_rows(int dtype, float* x, const int* positions, const void* table, int rows, void* lowered,
                                   int tokens, int hidden, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rows <= 0 || hidden <= 0) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    lb_launch(add_position_rows_kernel<float>, tokens, 256, 0, stream, x, positions, (const float*)table, rows, hidden,
              (float*)lowered);
  else if (dtype == LB_BF16)
    lb_launch(add_position_rows_kernel<bf16>, tokens, 256, 0, stream, x, positions, (const bf16*)table, rows, hidden,
              (bf16*)lowered);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- 32-bit residual stream: norm AFTER the sum
// For models that norm the stream after every sub-layer has been added (the normed sum IS the stream):
//   d      = factor * (a[row] * sa + b[row] * sb)
//            sa = a_w * rsqrt(mean(a[row]^2) + part_eps) per channel (a_w null: sa = 1); the same for b; b may be null
//   v      = alpha * x[row] + d
//   x[row] = weight * v * rsqrt(mean(v^2) + eps)
//   out[row] = T(x[row])                               (out null: no copy in the run's type)
// a and b are sub-layer outputs in the run's type T; everything is computed in 32-bit and x is never
// rounded. One block per row; the block size depends on the width only, so a row's sums do not depend
// on the batch.
template <typename T>
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ a, const float* __restrict__ a_w,
                                          const T* __restrict__ b, const float* __restrict__ b_w, float part_eps,
                                          float factor, float alpha, const float* __restrict__ weight, float eps,
                                          T* __restrict__ out, int hidden) {
  extern __shared__ float row_vals[];  // hidden floats + 33 for the reductions
  pdl_launch_dependents();
  pdl_wait();
  float* scratch = row_vals + hidden;
  const size_t at = (size_t)blockIdx.x * hidden;
  float ainv = 1.f, binv = 1.f;
  if (a && a_w) {
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = Elem<T>::load(a + at + i);
      s += d * d;
    }
    ainv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + part_eps);
  }
  if (b && b_w) {
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = Elem<T>::load(b + at + i);
      s += d * d;
    }
    binv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + part_eps);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float d = 0.f;
    if (a) d = a_w ? Elem<T>::load(a + at + i) * ainv * a_w[i] : Elem<T>::load(a + at + i);
    if (b) d += b_w ? Elem<T>::load(b + at + i) * binv * b_w[i] : Elem<T>::load(b + at + i);
    const float v = alpha * x[at + i] + factor * d;
    row_vals[i] = v;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = weight[i] * (row_vals[i] * inv);
    x[at + i] = v;
    if (out) Elem<T>::store(out + at + i, v);
  }
}

template <typename T>
static int launch_scaled_add_rmsnorm(float* x, const void* a, const float* a_w, const void* b, const float* b_w,
                                     float part_eps, float factor, float alpha, const float* weight, float eps, void* out,
                                     int n_rows, int hidden, cudaStream_t stream) {
  static LbPerDeviceOnce once;
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  if (smem > 200 * 1024) return LB_ERR_SIZE;
  if (smem > 48 * 1024 && once.first())
    cudaFuncSetAttribute(scaled_add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  lb_launch(scaled_add_rmsnorm_kernel<T>, n_rows, threads, smem, stream, x, (const T*)a, a_w, (const T*)b, b_w, part_eps, factor,
            alpha, weight, eps, (T*)out, hidden);
  return lb_last_error();
}

LB_EXPORT int lb_scaled_add_rmsnorm(int dtype, float* x, const void* a, const float* a_w, const void* b, const float* b_w,
                                    float part_eps, float factor, float alpha, const float* weight, float eps, void* out,
                                    int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || !weight || (b && !a)) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    return launch_scaled_add_rmsnorm<float>(x, a, a_w, b, b_w, part_eps, factor, alpha, weight, eps, out, n_rows, hidden, stream);
  if (dtype == LB_BF16)
    return launch_scaled_add_rmsnorm<bf16>(x, a, a_w, b, b_w, part_eps, factor, alpha, weight, eps, out, n_rows, hidden, stream);
  return LB_ERR_DTYPE;
}

// ---------------------------------------------------------------- a 32-bit stream as the matrix products read it
// out[i] = T(x[i]).
template <typename T>
__global__ void lower_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x)
    Elem<T>::store(out + i, x[i]);
}

LB_EXPORT int lb_lower_rows(int dtype, const float* x, void* out, long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == LB_F32) lb_launch(lower_rows_kernel<float>, blocks, threads, 0, stream, x, (float*)out, total);
  else if (dtype == LB_BF16) lb_launch(lower_rows_kernel<bf16>, blocks, threads, 0, stream, x, (bf16*)out, total);
  else return LB_ERR_DTYPE;
  return lb_last_error();
}
