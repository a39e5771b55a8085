// Attention over a latent: every token leaves one small vector c (RMS-normed) and one rotated key part
// in the cache, and every head's keys and values are linear maps of c. The maps are folded into the
// query and the output instead of being applied to every cached token:
//
//   score_h(i, j) = (W_uk_h^T q_h(i)) . c(j) + q_rot_h(i) . k_rot(j)         out_h(i) = W_uv_h sum_j p_h(i, j) c(j)
//
// so a step is attention with ONE key/value head whose key is [c | k_rot] and whose value is the key's
// leading channels. Here: the kernel that makes a token's cache row and the rotated query parts, and the
// per-head matrix products on both sides of the attention.
#include <math.h>

#include "common.cuh"

namespace {
// One block per token over its 32-bit projection row. With `dkv_off` >= 0 the row holds [latent: rank |
// rotated key part: rot] there: c = latent * rsqrt(mean(latent^2) + eps) * norm_w goes to channels [0, rank) of
// the token's cache row, the rotated key part to [rank, rank + rot), zeros up to `room`. q at `q_off` is
// q_heads x [dim | rot]: the rotated part of every head goes to channels [rank, rank + rot) of q_out's head (zeros
// up to room); channels [0, rank) are left to the product that folds the key map into the query.
// Rotation: channels 2i and 2i + 1 turn by the token's angle i, (u, v) -> (u cos - v sin, v cos + u sin), cos/sin
// from table[t] ([T, 2, rot / 2]).
template <typename T>
__global__ void latent_rows_kernel(const float* __restrict__ proj, long row_stride, int q_off, int dkv_off,
                                   const float* __restrict__ norm_w, float eps, const float* __restrict__ table,
                                   const int* __restrict__ slot_map, T* __restrict__ k_pool, T* __restrict__ q_out,
                                   int q_heads, int dim, int rot, int rank, int room, int page_tokens) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, half = rot >> 1;
  const float* row = proj + (size_t)t * row_stride;
  const float* cs = table + (size_t)t * 2 * half;
  const float* sn = cs + half;
  auto turned = [&](const float* part, int c) {      // channel c of a rotated part
    const int i = c >> 1;
    const float u = part[2 * i], v = part[2 * i + 1];
    return (c & 1) ? v * cs[i] + u * sn[i] : u * cs[i] - v * sn[i];
  };
  if (dkv_off >= 0) {
    const float* latent = row + dkv_off;
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) ss += latent[c] * latent[c];
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    const int slot = slot_map[t];
    T* dst = k_pool + ((size_t)(slot / page_tokens) * page_tokens + slot % page_tokens) * room;
    for (int c = threadIdx.x; c < room; c += blockDim.x) {
      float v = 0.f;
      if (c < rank) v = latent[c] * inv * norm_w[c];
      else if (c < rank + rot) v = turned(latent + rank, c - rank);
      Elem<T>::store(dst + c, v);
    }
  }
  const int tail = room - rank;
  for (int i = threadIdx.x; i < q_heads * tail; i += blockDim.x) {
    const int h = i / tail, c = i - h * tail;
    const float v = c < rot ? turned(row + q_off + h * (dim + rot) + dim, c) : 0.f;
    Elem<T>::store(q_out + ((size_t)t * q_heads + h) * room + rank + c, v);
  }
}

// out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]  (* sigmoid(gate[t, h * N + n])), one product per head:
// a rows `a_row` elements apart with heads `a_head` apart, out likewise, w [heads, N, K] dense. 32-bit sums in
// the order of k, so a row's result does not depend on the batch or on the tile. A block: 8 TPT tokens x 64 outputs of
// one head, TPT tokens x 4 outputs a thread (2 for a few tokens, 8 for many: 32 products for 12 reads of shared memory).
constexpr int HL_OUT = 64, HL_K = 32;

template <typename TA, typename T, int TPT>
__global__ void __launch_bounds__(128)
heads_linear_kernel(const TA* __restrict__ a, long a_row, long a_head, const T* __restrict__ w, T* __restrict__ out,
                    long out_row, long out_head, const float* __restrict__ gate, long gate_row, int tokens, int n_out,
                    int k_dim) {
  constexpr int HL_TOKENS = 8 * TPT;
  __shared__ float a_s[HL_TOKENS][HL_K + 1];
  __shared__ float w_s[HL_OUT][HL_K + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * HL_TOKENS, n0 = blockIdx.y * HL_OUT, h = blockIdx.z;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // outputs tx + 16 j, tokens TPT ty .. TPT ty + TPT - 1
  float acc[TPT][4] = {};
  for (int k0 = 0; k0 < k_dim; k0 += HL_K) {
    __syncthreads();
    for (int i = threadIdx.x; i < HL_TOKENS * HL_K; i += 128) {
      const int r = i / HL_K, c = i - r * HL_K;
      const bool in = t0 + r < tokens && k0 + c < k_dim;
      a_s[r][c] = in ? Elem<TA>::load(a + (size_t)(t0 + r) * a_row + (size_t)h * a_head + k0 + c) : 0.f;
    }
    for (int i = threadIdx.x; i < HL_OUT * HL_K; i += 128) {
      const int r = i / HL_K, c = i - r * HL_K;
      const bool in = n0 + r < n_out && k0 + c < k_dim;
      w_s[r][c] = in ? Elem<T>::load(w + ((size_t)h * n_out + n0 + r) * k_dim + k0 + c) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < HL_K; ++c) {
      float wv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_s[tx + 16 * j][c];
#pragma unroll
      for (int r = 0; r < TPT; ++r) {
        const float av = a_s[TPT * ty + r][c];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[r][j] = fmaf(av, wv[j], acc[r][j]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < TPT; ++r) {
    const int t = t0 + TPT * ty + r;
    if (t >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= n_out) continue;
      float v = acc[r][j];
      if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_row + (size_t)h * n_out + n]));
      Elem<T>::store(out + (size_t)t * out_row + (size_t)h * out_head + n, v);
    }
  }
}
}  // namespace

LB_EXPORT int lb_latent_rows(int dtype, const float* proj, long row_stride, int q_off, int dkv_off, const float* norm_w,
                             float eps, const float* table, const int* slot_map, void* k_pool, void* q_out, int tokens,
                             int q_heads, int dim, int rot, int rank, int room, int page_tokens, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_heads <= 0 || dim <= 0 || rot < 0 || rot % 2 || rank <= 0 || room < rank + rot || page_tokens <= 0 || !table ||
      (dkv_off >= 0 && (!norm_w || !slot_map || !k_pool)))
    return LB_ERR_SIZE;
  if (dtype == LB_F32)
    lb_launch(latent_rows_kernel<float>, tokens, 128, 0, stream, proj, row_stride, q_off, dkv_off, norm_w, eps, table, slot_map,
              (float*)k_pool, (float*)q_out, q_heads, dim, rot, rank, room, page_tokens);
  else if (dtype == LB_BF16)
    lb_launch(latent_rows_kernel<bf16>, tokens, 128, 0, stream, proj, row_stride, q_off, dkv_off, norm_w, eps, table, slot_map,
              (bf16*)k_pool, (bf16*)q_out, q_heads, dim, rot, rank, room, page_tokens);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// a_float: a is 32-bit whatever `dtype` (the projection's unrounded rows); w and out are of `dtype`.
LB_EXPORT int lb_heads_linear(int dtype, int a_float, const void* a, long a_row, long a_head, const void* w, void* out,
                              long out_row, long out_head, const float* gate, long gate_row, int tokens, int heads, int n_out,
                              int k_dim, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || heads > 65535 || n_out <= 0 || k_dim <= 0 || (n_out + HL_OUT - 1) / HL_OUT > 65535) return LB_ERR_SIZE;
  const int tpt = tokens >= 256 ? 8 : 2;
  dim3 grid((tokens + 8 * tpt - 1) / (8 * tpt), (n_out + HL_OUT - 1) / HL_OUT, heads);
#define LB_HL_T(TA, T, TPT)                                                                                                    \
  lb_launch(heads_linear_kernel<TA, T, TPT>, grid, 128, 0, stream, (const TA*)a, a_row, a_head, (const T*)w, (T*)out, out_row, \
            out_head, gate, gate_row, tokens, n_out, k_dim)
#define LB_HL(TA, T)             \
  do {                           \
    if (tpt == 8) LB_HL_T(TA, T, 8); \
    else LB_HL_T(TA, T, 2);      \
  } while (0)
  if (dtype == LB_F32) LB_HL(float, float);
  else if (dtype == LB_BF16) {
    if (a_float) LB_HL(float, bf16);
    else LB_HL(bf16, bf16);
  } else
    return LB_ERR_DTYPE;
#undef LB_HL
#undef LB_HL_T
  return lb_last_error();
}
