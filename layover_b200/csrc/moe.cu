// Routed experts: a router that sends every token to its `top` best experts, the grouping of the
// (token, expert) pairs by expert, the experts' two matrix products over those groups, and the sum
// of a token's expert outputs. Nothing here returns to the host between the steps: the group sizes
// stay on the device and the products are launched for the largest number of tiles the pairs can make.
//
//   route     z = W_router h in 32-bit, one warp per token; score = sigmoid(z); the `top` largest z
//             (ties: the lower index) with their scores; optionally one more 32-bit dot product per
//             token, sigmoid(w_shared . h), the factor of a shared expert
//   group     offsets[e] .. offsets[e + 1] = the places of expert e's pairs in `order`, order[place] =
//             pair = token * top + k
//   products  for every expert e and every pair in its group
//               up    act[place]  = T(act_fn(s * (Wg_e h)) * (s * (Wu_e h)))   s = the pair's score
//               down  y[pair]     = Wd_e act[place]                             (32-bit)
//             The score multiplies the expert's INPUT; W (s h) = s (W h), and the factor is applied to
//             the 32-bit sums rather than to a rounded s h. Every output element is one dot product
//             summed in the order of k, so it does not depend on where its row sits in a tile or on
//             what else is in the batch. (For designs that weight the expert's output the same
//             kernels serve: up with s = 1, the weight in `combine`.)
//   combine   out[t] = T(sum_k y[t * top + k] * (c_k) + f_t * shared[t]), c_k = 1 or the pair's score
//
// Three forms of the products: `moe_expert_rows_kernel` for a few rows per expert (decode steps: a stream of the chosen
// experts' weight rows, 16 bytes a load), `moe_expert_product_kernel` in tiles on the FFMA pipes (32-bit runs with many
// pairs, and sizes that cannot be read 16 bytes at a time), and for many pairs in a bfloat16 run the tensor-core product
// of gemm_tcgen05.cu in its grouped form, for which `moe_group_tiles_kernel` pads every expert's group to whole tiles of
// 128 rows and `moe_scatter_rows_kernel` lays the scaled rows out (the score then multiplies the rounded input itself).
// In a bfloat16 run with many tokens the router's logits may also come from that product (`moe_select_kernel`).
#include <math.h>

#include "common.cuh"

namespace {


// Sixteen bytes of a row at once: 8 bfloat16 or 4 floats, as floats.
template <typename T> struct Piece;
template <> struct Piece<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ uint4 raw(const float* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const uint4& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { unpack(raw(p), v); }
};
template <> struct Piece<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ uint4 raw(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) { unpack(raw(p), v); }
  static __device__ __forceinline__ void unpack(const uint4& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      v[2 * i] = __low2float(pair);
      v[2 * i + 1] = __high2float(pair);
    }
  }
};

// How a token's experts are chosen beyond "the `top` largest logits", for routers that need it:
//   correction  float [experts] or null: the choice is made on sigmoid(z) + correction, the weights are sigmoid(z)
//   groups      > 1: the experts are `groups` equal groups of neighbours; a group's score is the sum of its two largest
//               choice scores (its only one, if a group has one expert); only experts of the `keep` best groups can be
//               chosen (ties: the lower index)
//   renorm      the chosen weights are divided by their sum (+ 1e-20)
//   scale       then multiplied by this
// All of it is one warp's work per token on 32-bit numbers in shared memory.
struct RouteOptions {
  const float* correction;
  int groups, keep, renorm;
  float scale;
  __host__ __device__ bool general() const { return correction || groups > 1 || renorm || scale != 1.f; }
};

// z [experts]: the token's logits (overwritten); s [experts] and g [groups]: room for the scores. One warp.
__device__ __forceinline__ void choose_general(float* z, float* s, float* g, int experts, int top, const RouteOptions& opt,
                                               int lane, int* ids, float* scores) {
  for (int e = lane; e < experts; e += 32) {
    const float score = 1.0f / (1.0f + expf(-z[e]));
    s[e] = score;
    z[e] = score + (opt.correction ? opt.correction[e] : 0.f);
  }
  __syncwarp();
  if (opt.groups > 1) {
    const int size = experts / opt.groups;
    for (int i = lane; i < opt.groups; i += 32) {
      float m1 = -INFINITY, m2 = -INFINITY;
      for (int e = i * size; e < (i + 1) * size; ++e) {
        const float v = z[e];
        if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
      }
      g[i] = size >= 2 ? m1 + m2 : m1;
    }
    __syncwarp();
    for (int k = 0; k < opt.keep; ++k) {          // a kept group is marked with a NaN, which no comparison picks again
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int i = lane; i < opt.groups; i += 32) {
        const float v = g[i];
        if (v > best || (v == best && i < at)) { best = v; at = i; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at >= opt.groups) break;                // nothing comparable is left
      if (lane == 0) g[at] = NAN;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (!isnan(g[e / size])) z[e] = -INFINITY;
    __syncwarp();
  }
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= experts) at = k;                    // only when every score left is NaN or -inf
    if (lane == 0) {
      ids[k] = at;
      scores[k] = s[at];
      sum += s[at];
      z[at] = -INFINITY;                          // taken
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float factor = (opt.renorm ? 1.0f / (sum + 1e-20f) : 1.f) * opt.scale;
    for (int k = 0; k < top; ++k) scores[k] *= factor;
  }
}

// A block takes TT tokens; its warps share the experts (warp w takes experts w, w + WARPS, ...) and one more row for the
// shared expert's factor. A logit is one warp's dot product: lane l holds the channels N (l + 32 i) .. + N - 1 (N = 16
// bytes of h), multiplies them in order, and the lanes' sums meet in a butterfly, the same order whatever TT is and
// whatever else the batch holds. Then warp t picks token t's `top` experts. VEC: rows start on 16-byte boundaries and
// the width is a multiple of N.
template <typename T, int TT, int WARPS, bool VEC>
__global__ void __launch_bounds__(WARPS * 32)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ shared_w,
                 int* __restrict__ ids, float* __restrict__ scores, float* __restrict__ shared_factor, int tokens,
                 int hidden, int experts, int top, RouteOptions opt) {
  constexpr int N = Piece<T>::N, ROUTE_WARPS = WARPS;
  extern __shared__ float logits[];                 // [TT][experts] (+ [TT][experts + groups] for a general choice)
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TT, n_t = min(TT, tokens - t0);
  for (int e = warp; e <= experts; e += ROUTE_WARPS) {
    if (e == experts && !shared_w) break;
    const float* w = e < experts ? router + (size_t)e * hidden : shared_w;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[t] = 0.f;
    if (VEC) {
      for (int i = lane * N; i < hidden; i += 32 * N) {
        float wv[N];
#pragma unroll
        for (int c = 0; c < N; c += 4) {
          const float4 r = *reinterpret_cast<const float4*>(w + i + c);
          wv[c] = r.x; wv[c + 1] = r.y; wv[c + 2] = r.z; wv[c + 3] = r.w;
        }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          if (t < n_t) {
            float x[N];
            Piece<T>::load(h + (size_t)(t0 + t) * hidden + i, x);
#pragma unroll
            for (int c = 0; c < N; ++c) acc[t] = fmaf(x[c], wv[c], acc[t]);
          }
        }
      }
    } else {
      for (int i0 = lane * N; i0 < hidden; i0 += 32 * N) {
        for (int i = i0; i < min(i0 + N, hidden); ++i) {
          const float wv = w[i];
#pragma unroll
          for (int t = 0; t < TT; ++t)
            if (t < n_t) acc[t] = fmaf(Elem<T>::load(h + (size_t)(t0 + t) * hidden + i), wv, acc[t]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      const float s = warp_sum(acc[t]);
      if (lane == 0 && t < n_t) {
        if (e < experts) logits[t * experts + e] = s;
        else shared_factor[t0 + t] = 1.0f / (1.0f + expf(-s));
      }
    }
  }
  __syncthreads();
  for (int t = warp; t < n_t; t += ROUTE_WARPS) {
    float* z = logits + t * experts;
    if (opt.general()) {
      float* room = logits + TT * experts + t * (experts + opt.groups);
      choose_general(z, room, room + experts, experts, top, opt, lane, ids + (size_t)(t0 + t) * top, scores + (size_t)(t0 + t) * top);
      continue;
    }
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int e = lane; e < experts; e += 32) {
        const float v = z[e];
        if (v > best || (v == best && e < at)) { best = v; at = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at >= experts) at = k;                    // only when every logit left is NaN or -inf
      if (lane == 0) {
        ids[(size_t)(t0 + t) * top + k] = at;
        scores[(size_t)(t0 + t) * top + k] = 1.0f / (1.0f + expf(-best));
        z[at] = -INFINITY;                          // taken
      }
      __syncwarp();
    }
  }
}

// The same choice from logits that a matrix product left in memory (a bfloat16 run: products of bfloat16 numbers are
// exact in 32-bit and the tensor cores add them up in 32-bit, so these are 32-bit logits): row t of `logits` holds the
// experts' logits and, behind them, the shared expert's. A warp per token.
constexpr int SELECT_WARPS = 4;
__global__ void __launch_bounds__(SELECT_WARPS * 32)
moe_select_kernel(const float* __restrict__ logits, long stride, int* __restrict__ ids, float* __restrict__ scores,
                  float* __restrict__ shared_factor, int tokens, int experts, int top, RouteOptions opt) {
  extern __shared__ float picked[];                 // [SELECT_WARPS][experts] (+ [SELECT_WARPS][experts + groups])
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * SELECT_WARPS + warp;
  if (t >= tokens) return;
  float* z = picked + warp * experts;
  const float* row = logits + (size_t)t * stride;
  for (int e = lane; e < experts; e += 32) z[e] = row[e];
  if (shared_factor && lane == 0) shared_factor[t] = 1.0f / (1.0f + expf(-row[experts]));
  __syncwarp();
  if (opt.general()) {
    float* room = picked + SELECT_WARPS * experts + warp * (experts + opt.groups);
    choose_general(z, room, room + experts, experts, top, opt, lane, ids + (size_t)t * top, scores + (size_t)t * top);
    return;
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= experts) at = k;                      // only when every logit left is NaN or -inf
    if (lane == 0) {
      ids[(size_t)t * top + k] = at;
      scores[(size_t)t * top + k] = 1.0f / (1.0f + expf(-best));
      z[at] = -INFINITY;                            // taken
    }
    __syncwarp();
  }
}

// One block: count, scan, place. The order inside a group is the order of arrival; no result depends on it.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ offsets, int* __restrict__ order) {
  extern __shared__ int counts[];                   // [experts] counts, then [experts] cursors
  pdl_launch_dependents();
  pdl_wait();
  int* cursor = counts + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      run += counts[e];
    }
    offsets[experts] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) order[atomicAdd(&cursor[ids[i]], 1)] = i;
}

// The same grouping for the tensor-core products, whose tiles of 128 rows must each belong to one expert: expert
// e's pairs take the places padded[e] .. padded[e] + count_e of buffers with room for pairs + 127 * experts rows
// rounded up to 128, every padded[e] a multiple of 128. place_of[pair] is the pair's row there; tile_up[i] /
// tile_down[i] = expert * rows_up / expert * rows_down for tile i of 128 rows (where that expert's weights start
// in the stacked matrices), -1 for a tile without pairs; one more entry behind the tiles' holds the number of tiles in use.
__global__ void __launch_bounds__(1024)
moe_group_tiles_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ place_of,
                       int* __restrict__ tile_up, int* __restrict__ tile_down, int n_tiles, int rows_up, int rows_down) {
  extern __shared__ int counts[];                   // [experts] counts, then [experts] cursors
  pdl_launch_dependents();
  pdl_wait();
  int* cursor = counts + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) { tile_up[i] = -1; tile_down[i] = -1; }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = run;
      const int tiles = (counts[e] + 127) >> 7;
      for (int i = 0; i < tiles; ++i) { tile_up[(run >> 7) + i] = e * rows_up; tile_down[(run >> 7) + i] = e * rows_down; }
      run += tiles << 7;
    }
    tile_up[n_tiles] = run >> 7;      // the tiles in use, all at the front
    tile_down[n_tiles] = run >> 7;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) place_of[i] = atomicAdd(&cursor[ids[i]], 1);
}

// rows[place_of[pair]] = T(scale[pair] * h[pair / top]): every pair's copy of its token's row, scaled by the pair's
// score (scale null: copied), in the layout of the grouped products.
template <typename T>
__global__ void moe_scatter_rows_kernel(const T* __restrict__ h, long h_stride, const int* __restrict__ place_of,
                                        const float* __restrict__ scale, T* __restrict__ rows, int hidden, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  const T* src = h + (size_t)(pair / top) * h_stride;
  T* dst = rows + (size_t)place_of[pair] * hidden;
  const float s = scale ? scale[pair] : 1.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) Elem<T>::store(dst + i, s * Elem<T>::load(src + i));
}

// Which expert's rows block `tile` of a products' launch owns, when every expert's group is cut into tiles of `rows_per_tile`
// places: all threads read the group sizes at once (one round trip to memory), thread 0 walks the tiles' counts in shared
// memory. found[0] = expert (-1: no such tile), found[1] = first place, found[2] = places. `counts`: `experts` ints.
__device__ __forceinline__ void find_tile(const int* __restrict__ offsets, int experts, int rows_per_tile, int tile,
                                          int* counts, int* found) {
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = offsets[e + 1] - offsets[e];
  __syncthreads();
  if (threadIdx.x == 0) {
    int left = tile, expert = -1, first = 0, rows = 0, begin = 0;
    for (int e = 0; e < experts && expert < 0; ++e) {
      const int count = counts[e], tiles = (count + rows_per_tile - 1) / rows_per_tile;
      if (left < tiles) {
        expert = e;
        first = begin + left * rows_per_tile;
        rows = min(rows_per_tile, count - left * rows_per_tile);
      }
      left -= tiles;
      begin += count;
    }
    found[0] = expert; found[1] = first; found[2] = rows;
  }
  __syncthreads();
}

template <int ACT> __device__ __forceinline__ float expert_activation(float g) {
  if (ACT == 1) return fmaxf(g, 0.f);
  if (ACT == 2) { const float r = fmaxf(g, 0.f); return r * r; }
  return g / (1.0f + expf(-g));      // silu
}

// The experts' products on the FFMA pipes (both precisions; 32-bit sums). A block owns BM places of one
// expert's group and BN output columns; a thread TM x TN of them. The k loop runs in steps of BK through
// shared memory, every element's sum in the order of k.
//   GATED: two weight tiles (gate rows w, up rows w + n_out * k_dim); out = T(act(s g) * (s u)), s = pair_scale[pair]
//   else:  out = the plain product, or (ACT 2) the square of its relu: an expert without a gate
// `a_rows`: the row of `a` for a place is a_rows[place] / a_div (null: the place itself);
// `out_rows`: the row of out is out_rows[place] (null: the place itself).
template <typename T, typename OutT, int BM, int BN, int TM, int TN, bool GATED, int ACT>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
moe_expert_product_kernel(const T* __restrict__ a, long a_stride, const int* __restrict__ a_rows, int a_div,
                          const int* __restrict__ offsets, int experts, const T* __restrict__ w, long expert_stride,
                          int n_out, int k_dim, OutT* __restrict__ out, long out_stride,
                          const int* __restrict__ out_rows, const float* __restrict__ pair_scale,
                          const int* __restrict__ order, int interleaved) {
  constexpr int BK = 32, THREADS = (BM / TM) * (BN / TN);
  __shared__ float a_s[BK][BM + 1];
  __shared__ float w_s[GATED ? 2 : 1][BK][BN + 1];
  __shared__ int found[3];
  extern __shared__ int group_counts[];          // [experts]
  pdl_launch_dependents();
  pdl_wait();
  find_tile(offsets, experts, BM, blockIdx.x, group_counts, found);
  const int expert = found[0], first = found[1], rows = found[2];
  if (expert < 0) return;
  const int n0 = blockIdx.y * BN;
  const T* wg = w + (size_t)expert * expert_stride;
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  float acc[GATED ? 2 : 1][TM][TN];
#pragma unroll
  for (int z = 0; z < (GATED ? 2 : 1); ++z)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[z][i][j] = 0.f;

  for (int k0 = 0; k0 < k_dim; k0 += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += THREADS) {
      const int r = i / BK, c = i - r * BK;
      float v = 0.f;
      if (r < rows && k0 + c < k_dim) {
        const int place = first + r;
        const long src = a_rows ? a_rows[place] / a_div : place;
        v = Elem<T>::load(a + src * a_stride + k0 + c);
      }
      a_s[c][r] = v;
    }
    for (int i = threadIdx.x; i < BN * BK; i += THREADS) {
      const int r = i / BK, c = i - r * BK;
      const bool live = n0 + r < n_out && k0 + c < k_dim;
      // gate row n and up row n: the two halves of the matrix, or (interleaved) blocks of 64 gate rows followed by
      // the 64 up rows of the same features, the layout of the tensor-core product's fused activation
      const int n = n0 + r;
      const size_t gate_row = (GATED && interleaved) ? (size_t)(n >> 6) * 128 + (n & 63) : (size_t)n;
      const size_t up_row = (GATED && interleaved) ? gate_row + 64 : (size_t)n_out + n;
      w_s[0][c][r] = live ? Elem<T>::load(wg + gate_row * k_dim + k0 + c) : 0.f;
      if (GATED) w_s[1][c][r] = live ? Elem<T>::load(wg + up_row * k_dim + k0 + c) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < BK; ++k) {
      float av[TM], bv[GATED ? 2 : 1][TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = a_s[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        bv[0][j] = w_s[0][k][tx + j * (BN / TN)];
        if (GATED) bv[1][j] = w_s[1][k][tx + j * (BN / TN)];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[0][i][j] = fmaf(av[i], bv[0][j], acc[0][i][j]);
          if (GATED) acc[1][i][j] = fmaf(av[i], bv[1][j], acc[1][i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (r >= rows) continue;
    const int place = first + r;
    const long dst = out_rows ? out_rows[place] : place;
    const float s = (GATED && pair_scale) ? pair_scale[order[place]] : 1.f;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx + j * (BN / TN);
      if (n >= n_out) continue;
      if (GATED) Elem<OutT>::store(out + dst * out_stride + n, expert_activation<ACT>(s * acc[0][i][j]) * (s * acc[GATED ? 1 : 0][i][j]));
      else Elem<OutT>::store(out + dst * out_stride + n, ACT == 2 ? expert_activation<2>(acc[0][i][j]) : acc[0][i][j]);
    }
  }
}

// The experts' products for a handful of rows per expert (decode steps): a stream of the chosen experts' weights.
// A block owns up to ROWS places of one expert's group and FEATURES output features per warp; a lane reads 16 bytes of
// a weight row at a time (and the same channels of every row of the group, which the L1 holds), multiplies in the
// order of k and the lanes' sums meet in a butterfly. GATED / interleaved / a_rows / out_rows / pair_scale as in the
// tiled kernel above. Needs rows of `a` and `w` that start on 16-byte boundaries and k_dim a multiple of Piece<T>::N.
constexpr int FEW_ROWS = 4, FEW_WARPS = 8, FEW_FEATURES = 2;

template <typename T, typename OutT, bool GATED, int ACT>
__global__ void __launch_bounds__(FEW_WARPS * 32)
moe_expert_rows_kernel(const T* __restrict__ a, long a_stride, const int* __restrict__ a_rows, int a_div,
                       const int* __restrict__ offsets, int experts, const T* __restrict__ w, long expert_stride,
                       int n_out, int k_dim, OutT* __restrict__ out, long out_stride,
                       const int* __restrict__ out_rows, const float* __restrict__ pair_scale,
                       const int* __restrict__ order, int interleaved, int features_per_warp) {
  constexpr int N = Piece<T>::N, Z = GATED ? 2 : 1, F = FEW_FEATURES;
  __shared__ int found[3];
  __shared__ long row_of[FEW_ROWS];
  extern __shared__ int group_counts[];          // [experts]
  pdl_launch_dependents();
  pdl_wait();
  find_tile(offsets, experts, FEW_ROWS, blockIdx.x, group_counts, found);
  const int expert = found[0], first = found[1], rows = found[2];
  if (expert < 0) return;
  if (threadIdx.x < rows) row_of[threadIdx.x] = a_rows ? a_rows[first + threadIdx.x] / a_div : first + threadIdx.x;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* wg = w + (size_t)expert * expert_stride;
  const int f0 = (blockIdx.y * FEW_WARPS + warp) * features_per_warp;
  for (int n0 = f0; n0 < min(f0 + features_per_warp, n_out); n0 += F) {
    // F features at once, so that a lane has 2 F (gated) rows of weights on their way at any time
    const T* wr[Z][F];
#pragma unroll
    for (int f = 0; f < F; ++f) {
      const int n = min(n0 + f, n_out - 1);           // a feature past the end repeats the last one and is not stored
      const size_t gate_row = (GATED && interleaved) ? (size_t)(n >> 6) * 128 + (n & 63) : (size_t)n;
      wr[0][f] = wg + gate_row * k_dim;
      if (GATED) wr[Z - 1][f] = wg + ((GATED && interleaved) ? gate_row + 64 : (size_t)n_out + n) * k_dim;
    }
    float acc[Z][F][FEW_ROWS];
#pragma unroll
    for (int z = 0; z < Z; ++z)
#pragma unroll
      for (int f = 0; f < F; ++f)
#pragma unroll
        for (int r = 0; r < FEW_ROWS; ++r) acc[z][f][r] = 0.f;
    // the next 16 bytes of every weight row are asked for (and kept as they come) before this step's are used
    uint4 ahead[Z][F];
    if (lane * N < k_dim) {
#pragma unroll
      for (int z = 0; z < Z; ++z)
#pragma unroll
        for (int f = 0; f < F; ++f) ahead[z][f] = Piece<T>::raw(wr[z][f] + lane * N);
    }
    for (int k = lane * N; k < k_dim; k += 32 * N) {
      float wv[Z][F][N];
#pragma unroll
      for (int z = 0; z < Z; ++z)
#pragma unroll
        for (int f = 0; f < F; ++f) Piece<T>::unpack(ahead[z][f], wv[z][f]);
      if (k + 32 * N < k_dim) {
#pragma unroll
        for (int z = 0; z < Z; ++z)
#pragma unroll
          for (int f = 0; f < F; ++f) ahead[z][f] = Piece<T>::raw(wr[z][f] + k + 32 * N);
      }
#pragma unroll
      for (int r = 0; r < FEW_ROWS; ++r) {
        if (r < rows) {
          float x[N];
          Piece<T>::load(a + row_of[r] * a_stride + k, x);
#pragma unroll
          for (int z = 0; z < Z; ++z)
#pragma unroll
            for (int f = 0; f < F; ++f)
#pragma unroll
              for (int i = 0; i < N; ++i) acc[z][f][r] = fmaf(x[i], wv[z][f][i], acc[z][f][r]);
        }
      }
    }
#pragma unroll
    for (int f = 0; f < F; ++f) {
#pragma unroll
      for (int r = 0; r < FEW_ROWS; ++r) {
        if (r < rows) {            // uniform over the block
          const float g = warp_sum(acc[0][f][r]);
          const float u = GATED ? warp_sum(acc[Z - 1][f][r]) : 0.f;
          if (lane == 0 && n0 + f < n_out) {
            const int place = first + r;
            const long dst = out_rows ? out_rows[place] : place;
            if (GATED) {
              const float sc = pair_scale ? pair_scale[order[place]] : 1.f;
              Elem<OutT>::store(out + dst * out_stride + n0 + f, expert_activation<ACT>(sc * g) * (sc * u));
            } else {
              Elem<OutT>::store(out + dst * out_stride + n0 + f, ACT == 2 ? expert_activation<2>(g) : g);
            }
          }
        }
      }
    }
  }
}

template <typename T, typename YT>
__global__ void moe_combine_kernel(const YT* __restrict__ y, const float* __restrict__ pair_scale,
                                   const T* __restrict__ shared_out, const float* __restrict__ shared_factor,
                                   T* __restrict__ out, long total, int hidden, int top, const int* __restrict__ rows) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / hidden;
    const int c = (int)(i - t * hidden);
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const float part = Elem<YT>::load(y + (rows ? (long)rows[t * top + k] : t * top + k) * hidden + c);
      v += pair_scale ? pair_scale[t * top + k] * part : part;
    }
    if (shared_out) v += (shared_factor ? shared_factor[t] : 1.f) * Elem<T>::load(shared_out + i);
    Elem<T>::store(out + i, v);
  }
}

template <typename T, bool GATED, typename OutT>
int launch_product(bool few, int act, const void* a, long a_stride, const int* a_rows, int a_div, const int* offsets,
                   int experts, const void* w, long expert_stride, int n_out, int k_dim, void* out, long out_stride,
                   const int* out_rows, const float* pair_scale, const int* order, int n_pairs, cudaStream_t stream,
                   int interleaved = 0) {
#define LB_MOE_ARGS (const T*)a, a_stride, a_rows, a_div, offsets, experts, (const T*)w, expert_stride, n_out, k_dim, \
                    (OutT*)out, out_stride, out_rows, pair_scale, order, interleaved
  const bool aligned = (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0 && k_dim % Piece<T>::N == 0 &&
                       (a_stride * sizeof(T)) % 16 == 0;
  if (few && aligned) {     // a handful of rows per expert: a stream of the chosen experts' weight rows
    // enough blocks to fill the GPU: the tiles are about the experts in use, the features are dealt over grid y
    int tiles = (n_pairs + FEW_ROWS - 1) / FEW_ROWS + experts;
    if (tiles > n_pairs) tiles = n_pairs;
    int per_warp = 8;
    while (per_warp > FEW_FEATURES && (long)tiles * ((n_out + FEW_WARPS * per_warp - 1) / (FEW_WARPS * per_warp)) < 4 * 148) per_warp >>= 1;
    dim3 grid(tiles, (n_out + FEW_WARPS * per_warp - 1) / (FEW_WARPS * per_warp));
    if (act == 1) lb_launch(moe_expert_rows_kernel<T, OutT, GATED, 1>, grid, FEW_WARPS * 32, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS, per_warp);
    else if (act == 2) lb_launch(moe_expert_rows_kernel<T, OutT, GATED, 2>, grid, FEW_WARPS * 32, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS, per_warp);
    else lb_launch(moe_expert_rows_kernel<T, OutT, GATED, 0>, grid, FEW_WARPS * 32, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS, per_warp);
  } else if (few) {      // the same through tiles of 8 places, for sizes and addresses that cannot be read 16 bytes at a time
    constexpr int BM = 8, BN = 128;
    dim3 grid((n_pairs + BM - 1) / BM + experts, (n_out + BN - 1) / BN);
    if (grid.x > (unsigned)n_pairs) grid.x = n_pairs;   // every tile holds a pair
    if (act == 1) lb_launch(moe_expert_product_kernel<T, OutT, BM, BN, 1, 4, GATED, 1>, grid, 256, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS);
    else if (act == 2) lb_launch(moe_expert_product_kernel<T, OutT, BM, BN, 1, 4, GATED, 2>, grid, 256, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS);
    else lb_launch(moe_expert_product_kernel<T, OutT, BM, BN, 1, 4, GATED, 0>, grid, 256, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS);
  } else {
    constexpr int BM = 64, BN = 64;
    dim3 grid((n_pairs + BM - 1) / BM + experts, (n_out + BN - 1) / BN);
    if (grid.x > (unsigned)n_pairs) grid.x = n_pairs;
    if (act == 1) lb_launch(moe_expert_product_kernel<T, OutT, BM, BN, 4, 4, GATED, 1>, grid, 256, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS);
    else if (act == 2) lb_launch(moe_expert_product_kernel<T, OutT, BM, BN, 4, 4, GATED, 2>, grid, 256, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS);
    else lb_launch(moe_expert_product_kernel<T, OutT, BM, BN, 4, 4, GATED, 0>, grid, 256, (size_t)experts * sizeof(int), stream, LB_MOE_ARGS);
  }
#undef LB_MOE_ARGS
  return lb_last_error();
}

}  // namespace

template <typename T>
static void launch_route(const void* h, const float* router, const float* shared_w, int* ids, float* scores,
                         float* shared_factor, int tokens, int hidden, int experts, int top, RouteOptions opt,
                         cudaStream_t stream) {
  const bool vec = hidden % Piece<T>::N == 0 && (uintptr_t)router % 16 == 0 && (uintptr_t)shared_w % 16 == 0 &&
                   (uintptr_t)h % 16 == 0;
#define LB_ROUTE_ARGS (const T*)h, router, shared_w, ids, scores, shared_factor, tokens, hidden, experts, top, opt
  const size_t per_token = (size_t)(experts + (opt.general() ? experts + opt.groups : 0)) * sizeof(float);
  // few tokens: a block of 32 warps each (a warp an expert or two), so that the step's latency is about one dot product's;
  // many: eight a block share every weight they read
  if (tokens <= 64) {
    const size_t smem = per_token;
    if (vec) lb_launch(moe_route_kernel<T, 1, 32, true>, tokens, 1024, smem, stream, LB_ROUTE_ARGS);
    else lb_launch(moe_route_kernel<T, 1, 32, false>, tokens, 1024, smem, stream, LB_ROUTE_ARGS);
  } else {
    const size_t smem = 8 * per_token;
    const int blocks = (tokens + 7) / 8;
    if (vec) lb_launch(moe_route_kernel<T, 8, 8, true>, blocks, 256, smem, stream, LB_ROUTE_ARGS);
    else lb_launch(moe_route_kernel<T, 8, 8, false>, blocks, 256, smem, stream, LB_ROUTE_ARGS);
  }
#undef LB_ROUTE_ARGS
}

static bool route_options(RouteOptions& opt, const float* correction, int groups, int keep, int renorm, float scale, int experts) {
  opt = RouteOptions{correction, groups > 1 ? groups : 0, keep, renorm, scale};
  return !(groups > 1 && (experts % groups || keep <= 0 || keep > groups)) && scale > 0.f;
}

// correction, groups, keep, renorm, scale: see RouteOptions (null, 0, 0, 0, 1: the `top` largest logits and their sigmoids).
LB_EXPORT int lb_moe_route(int dtype, const void* h, const float* router, const float* shared_w, int* ids, float* scores,
                           float* shared_factor, int tokens, int hidden, int experts, int top, const float* correction,
                           int groups, int keep, int renorm, float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  RouteOptions opt;
  if (hidden <= 0 || experts <= 0 || top <= 0 || top > experts || experts > 1024 || (shared_w && !shared_factor) ||
      !route_options(opt, correction, groups, keep, renorm, scale, experts))
    return LB_ERR_SIZE;
  if (dtype == LB_F32) launch_route<float>(h, router, shared_w, ids, scores, shared_factor, tokens, hidden, experts, top, opt, stream);
  else if (dtype == LB_BF16) launch_route<bf16>(h, router, shared_w, ids, scores, shared_factor, tokens, hidden, experts, top, opt, stream);
  else return LB_ERR_DTYPE;
  return lb_last_error();
}

// ids, scores (and shared_factor, from column `experts`, when not null) from logits [tokens, >= experts (+ 1)] with row
// stride `stride` floats.
LB_EXPORT int lb_moe_select(const float* logits, long stride, int* ids, float* scores, float* shared_factor, int tokens,
                            int experts, int top, const float* correction, int groups, int keep, int renorm, float scale,
                            cudaStream_t stream) {
  if (tokens <= 0) return 0;
  RouteOptions opt;
  if (experts <= 0 || top <= 0 || top > experts || experts > 1024 || stride < experts + (shared_factor ? 1 : 0) ||
      !route_options(opt, correction, groups, keep, renorm, scale, experts))
    return LB_ERR_SIZE;
  lb_launch(moe_select_kernel, (tokens + SELECT_WARPS - 1) / SELECT_WARPS, SELECT_WARPS * 32,
            (size_t)SELECT_WARPS * (experts + (opt.general() ? experts + opt.groups : 0)) * sizeof(float), stream, logits, stride, ids,
            scores, shared_factor, tokens, experts, top, opt);
  return lb_last_error();
}

LB_EXPORT int lb_moe_group(const int* ids, int n_pairs, int experts, int* offsets, int* order, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (experts <= 0 || experts > 4096) return LB_ERR_SIZE;
  lb_launch(moe_group_kernel, 1, 1024, (size_t)2 * experts * sizeof(int), stream, ids, n_pairs, experts, offsets, order);
  return lb_last_error();
}

// act[place, :] = T(act_fn(s g) * (s u)) for every place of `order`: h [tokens, hidden] (row stride h_stride), gate_up
// [experts, 2 * inter, hidden] (gate rows, then up rows; `interleaved`: blocks of 64 gate rows + the 64 up rows of the same
// features), scores by pair (null: s = 1). activation 0 silu, 1 relu, 2 the square of relu. gated 0: the experts have no
// gate; gate_up is [experts, inter, hidden] and act[place, :] = T(relu(up_e h)^2) (activation 2 only, no scores).
LB_EXPORT int lb_moe_expert_up(int dtype, const void* h, long h_stride, const int* order, const int* offsets,
                               const float* scores, const void* gate_up, void* act, int n_pairs, int top, int experts,
                               int hidden, int inter, int activation, int interleaved, int gated, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (experts <= 0 || experts > 1024 || hidden <= 0 || inter <= 0 || top <= 0 || activation < 0 || activation > 2) return LB_ERR_SIZE;
  if (interleaved && inter % 64) return LB_ERR_SIZE;
  const bool few = n_pairs <= 4 * experts;
  if (!gated) {
    if (activation != 2 || interleaved || scores) return LB_ERR_SIZE;
    if (dtype == LB_F32)
      return launch_product<float, false, float>(few, 2, h, h_stride, order, top, offsets, experts, gate_up, (long)inter * hidden,
                                                 inter, hidden, act, inter, nullptr, nullptr, order, n_pairs, stream);
    if (dtype == LB_BF16)
      return launch_product<bf16, false, bf16>(few, 2, h, h_stride, order, top, offsets, experts, gate_up, (long)inter * hidden,
                                               inter, hidden, act, inter, nullptr, nullptr, order, n_pairs, stream);
    return LB_ERR_DTYPE;
  }
  const long expert_stride = 2L * inter * hidden;
  if (dtype == LB_F32)
    return launch_product<float, true, float>(few, activation, h, h_stride, order, top, offsets, experts, gate_up, expert_stride,
                                              inter, hidden, act, inter, nullptr, scores, order, n_pairs, stream, interleaved);
  if (dtype == LB_BF16)
    return launch_product<bf16, true, bf16>(few, activation, h, h_stride, order, top, offsets, experts, gate_up, expert_stride,
                                            inter, hidden, act, inter, nullptr, scores, order, n_pairs, stream, interleaved);
  return LB_ERR_DTYPE;
}

// y[pair, :] = down_e act[place, :] in 32-bit: act [n_pairs, inter] by place, down [experts, hidden, inter], y [n_pairs, hidden].
LB_EXPORT int lb_moe_expert_down(int dtype, const void* act, const int* order, const int* offsets, const void* down, float* y,
                                 int n_pairs, int experts, int hidden, int inter, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (experts <= 0 || experts > 1024 || hidden <= 0 || inter <= 0) return LB_ERR_SIZE;
  const bool few = n_pairs <= 4 * experts;
  const long expert_stride = (long)hidden * inter;
  if (dtype == LB_F32)
    return launch_product<float, false, float>(few, 0, act, inter, nullptr, 1, offsets, experts, down, expert_stride, hidden,
                                               inter, y, hidden, order, nullptr, order, n_pairs, stream);
  if (dtype == LB_BF16)
    return launch_product<bf16, false, float>(few, 0, act, inter, nullptr, 1, offsets, experts, down, expert_stride, hidden,
                                              inter, y, hidden, order, nullptr, order, n_pairs, stream);
  return LB_ERR_DTYPE;
}

// out[t] = T(sum_k c_k y[row(t * top + k)] + f_t shared_out[t]); c_k = pair_scale[t * top + k] or 1; f_t = shared_factor[t]
// or 1; row(pair) = rows[pair], or the pair itself when rows is null. y is 32-bit, or (y_dtype) in the run's type; the sum is 32-bit.
LB_EXPORT int lb_moe_combine(int dtype, const void* y, int y_dtype, const float* pair_scale, const void* shared_out,
                             const float* shared_factor, void* out, int tokens, int hidden, int top, const int* rows,
                             cudaStream_t stream) {
  const long total = (long)tokens * hidden;
  if (total <= 0) return 0;
  if (top <= 0) return LB_ERR_SIZE;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == LB_F32 && y_dtype == LB_F32)
    lb_launch(moe_combine_kernel<float, float>, blocks, threads, 0, stream, (const float*)y, pair_scale, (const float*)shared_out,
              shared_factor, (float*)out, total, hidden, top, rows);
  else if (dtype == LB_BF16 && y_dtype == LB_F32)
    lb_launch(moe_combine_kernel<bf16, float>, blocks, threads, 0, stream, (const float*)y, pair_scale, (const bf16*)shared_out,
              shared_factor, (bf16*)out, total, hidden, top, rows);
  else if (dtype == LB_BF16 && y_dtype == LB_BF16)
    lb_launch(moe_combine_kernel<bf16, bf16>, blocks, threads, 0, stream, (const bf16*)y, pair_scale, (const bf16*)shared_out,
              shared_factor, (bf16*)out, total, hidden, top, rows);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// The grouping for the tensor-core products (see moe_group_tiles_kernel): n_tiles = the tiles of 128 rows the buffers have.
LB_EXPORT int lb_moe_group_tiles(const int* ids, int n_pairs, int experts, int* place_of, int* tile_up, int* tile_down,
                                 int n_tiles, int rows_up, int rows_down, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (experts <= 0 || experts > 4096 || (long)n_tiles * 128 < (long)n_pairs + 127L * experts) return LB_ERR_SIZE;
  lb_launch(moe_group_tiles_kernel, 1, 1024, (size_t)2 * experts * sizeof(int), stream, ids, n_pairs, experts, place_of,
            tile_up, tile_down, n_tiles, rows_up, rows_down);
  return lb_last_error();
}

LB_EXPORT int lb_moe_scatter_rows(int dtype, const void* h, long h_stride, const int* place_of, const float* scale,
                                  void* rows, int n_pairs, int hidden, int top, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (hidden <= 0 || top <= 0) return LB_ERR_SIZE;
  const int threads = hidden >= 2048 ? 256 : 128;
  if (dtype == LB_F32)
    lb_launch(moe_scatter_rows_kernel<float>, n_pairs, threads, 0, stream, (const float*)h, h_stride, place_of, scale,
              (float*)rows, hidden, top);
  else if (dtype == LB_BF16)
    lb_launch(moe_scatter_rows_kernel<bf16>, n_pairs, threads, 0, stream, (const bf16*)h, h_stride, place_of, scale,
              (bf16*)rows, hidden, top);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}
