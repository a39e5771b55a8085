// Time mixing with a decay per key channel that depends on the token (the WKV recurrence), as kernels over
// the requests' state rows.
//
// A request's state row (32-bit floats): S of every head [heads, dim, dim] (key channel, value channel), then
// the previous token's input h [width].
//
//   shift + mix   m_s[t] = T(h[t] + (h[t-1] - h[t]) * mu_s)        for every mix s (r, k, v, g, w read one each), a block a token;
//                 h[-1] of a step's first token is the state row's tail (zeros at the start of a sequence);
//                 a second launch then leaves the step's last h there
//   decay         w[t, c] = exp(-exp(w0[c] + sum_j W2[c, j] tanh(a[t, j])))      a = W1 m_w, 32-bit throughout
//   scan          per head:  o_t = (S + diag(u) k_t v_t^T)^T r_t,   S <- diag(w_t) S + k_t v_t^T
//                 o_t[e] = sum_d r_t[d] (S[d, e] + u[d] k_t[d] v_t[e])
//
// One scan kernel serves a whole prompt, a portion of one and a single decoded token: a sequence's tokens of the
// step are walked in order from the state the step before left. Every state element takes the same operations
// whatever the cut, and the sums over d run in an order that depends on the head size alone, so results do not
// depend on how the tokens were cut into steps or on what else is in the batch, bit for bit.
//
// Scan grid (ceil(dim / 16), heads, sequences), 8 warps (heads of up to 32 channels: 32 columns a block): a block owns
// 16 columns of one head's S, a thread DPT rows of one column (16 groups of rows a block, two a warp), so a lone
// prompt of 16 heads of 128 is 128 blocks. Tokens come CHUNK at a time through two shared-memory buffers filled by
// cp.async while the chunk before is worked on; r, k, w are read as 16-byte broadcasts; each group of rows leaves its
// partial sums of o per token and they are added in group order at the end of the chunk.
#include <math.h>

#include "common.cuh"

namespace {
constexpr int MIX_TOKENS = 16;     // tokens of one sequence that a block of the mix kernel takes
constexpr int CHUNK = 8, RANGES = 8, SCAN_THREADS = RANGES * 32;
constexpr int DECAY_TOKENS = 16;

// Four neighbouring channels at once: 16 bytes of floats, 8 bytes of bfloat16.
template <typename T> struct Quad;
template <> struct Quad<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

// A block per token: grid (tiles, MIX_TOKENS), the tile lists name the sequence and the first token of a tile.
// VEC: the width is a multiple of 4 and every row starts where four channels can be read at once.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
wkv_shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ mu, const float* __restrict__ state, long state_stride,
                     int shift_off, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                     const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, T* __restrict__ mixes, int tokens,
                     int width, int n_mix) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = tile_seq[blockIdx.x], at = tile_q0[blockIdx.x] + blockIdx.y;
  const int row0 = cu_q[seq];
  if (at >= cu_q[seq + 1] - row0) return;
  const size_t row = (size_t)(row0 + at);
  const T* cur_row = h + row * width;
  const T* prev_row = at > 0 ? cur_row - width : nullptr;
  const float* before = state + (size_t)state_slots[seq] * state_stride + shift_off;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
      const float4 cur = Quad<T>::load(cur_row + c);
      const float4 prev = prev_row ? Quad<T>::load(prev_row + c) : *reinterpret_cast<const float4*>(before + c);
      const float4 d = make_float4(prev.x - cur.x, prev.y - cur.y, prev.z - cur.z, prev.w - cur.w);
      for (int s = 0; s < n_mix; ++s) {
        const float4 m = *reinterpret_cast<const float4*>(mu + (size_t)s * width + c);
        Quad<T>::store(mixes + ((size_t)s * tokens + row) * width + c,
                       make_float4(fmaf(d.x, m.x, cur.x), fmaf(d.y, m.y, cur.y), fmaf(d.z, m.z, cur.z), fmaf(d.w, m.w, cur.w)));
      }
    }
    return;
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float cur = Elem<T>::load(cur_row + c);
    const float prev = prev_row ? Elem<T>::load(prev_row + c) : before[c];
    for (int s = 0; s < n_mix; ++s)
      Elem<T>::store(mixes + ((size_t)s * tokens + row) * width + c, fmaf(prev - cur, mu[(size_t)s * width + c], cur));
  }
}

// The request's newest input, for the next step's first token.
template <typename T>
__global__ void wkv_shift_tail_kernel(const T* __restrict__ h, float* __restrict__ state, long state_stride, int shift_off,
                                      const int* __restrict__ cu_q, const int* __restrict__ state_slots, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, last = cu_q[seq + 1] - 1;
  if (last < cu_q[seq]) return;
  float* tail = state + (size_t)state_slots[seq] * state_stride + shift_off;
  for (int c = threadIdx.x; c < width; c += blockDim.x) tail[c] = Elem<T>::load(h + (size_t)last * width + c);
}

// DECAY_TOKENS tokens a block share every weight they read; a thread owns channels, its sum runs in the order of j. The
// tokens' tanh(a) sit in shared memory, rows padded with zeros to whole 16-byte pieces that every thread reads at once.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
wkv_decay_kernel(const float* __restrict__ a, long a_stride, const T* __restrict__ w2, const float* __restrict__ w0,
                 float* __restrict__ decay, int tokens, int channels, int rank) {
  extern __shared__ __align__(16) float z_s[];     // [DECAY_TOKENS][padded rank]
  pdl_launch_dependents();
  pdl_wait();
  const int padded = (rank + 3) & ~3;
  const int t0 = blockIdx.x * DECAY_TOKENS, n = min(DECAY_TOKENS, tokens - t0);
  for (int i = threadIdx.x; i < DECAY_TOKENS * padded; i += blockDim.x) {
    const int t = i / padded, j = i - t * padded;
    z_s[i] = (t < n && j < rank) ? tanhf(a[(size_t)(t0 + t) * a_stride + j]) : 0.f;
  }
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float acc[DECAY_TOKENS];
#pragma unroll
    for (int t = 0; t < DECAY_TOKENS; ++t) acc[t] = 0.f;
    const T* row = w2 + (size_t)c * rank;
#pragma unroll 4
    for (int j = 0; j < padded; j += 4) {
      float w[4];
      if (VEC) {        // the rank is a multiple of 4 and a row starts where four of its weights can be read at once
        const float4 q = Quad<T>::load(row + j);
        w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
      } else {
#pragma unroll
        for (int x = 0; x < 4; ++x) w[x] = j + x < rank ? Elem<T>::load(row + j + x) : 0.f;
      }
#pragma unroll
      for (int t = 0; t < DECAY_TOKENS; ++t) {
        const float4 z = *reinterpret_cast<const float4*>(z_s + t * padded + j);
        acc[t] = fmaf(w[0], z.x, acc[t]);
        acc[t] = fmaf(w[1], z.y, acc[t]);
        acc[t] = fmaf(w[2], z.z, acc[t]);
        acc[t] = fmaf(w[3], z.w, acc[t]);
      }
    }
    const float bias = w0[c];
#pragma unroll
    for (int t = 0; t < DECAY_TOKENS; ++t)
      if (t < n) decay[(size_t)(t0 + t) * channels + c] = expf(-expf(acc[t] + bias));
  }
}

__device__ __forceinline__ void copy_async_4(float* dst_shared, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_16(float* dst_shared, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// r, k, v float [T, *] with row strides; w float [T, heads * dim]; u float [heads, dim]; out float [T, heads * dim].
// COLS value columns a block (16, or 32 for small heads); a warp holds 32 / COLS groups of rows of them, a block
// GROUPS = 8 * 32 / COLS groups of DPT rows each. VEC: dim is a multiple of 4 and every row of r, k, w starts on a
// 16-byte boundary.
template <int DPT, int COLS, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS, DPT <= 8 ? 3 : 1)      // single tokens are bound by the state's traffic: three blocks an SM keep it in flight
wkv_scan_kernel(const float* __restrict__ r, long r_stride, const float* __restrict__ k, long k_stride,
                const float* __restrict__ v, long v_stride, const float* __restrict__ w, const float* __restrict__ u,
                float* __restrict__ out, float* __restrict__ state, long state_stride, const int* __restrict__ cu_q,
                const int* __restrict__ state_slots, int heads, int dim) {
  static_assert(DPT % 4 == 0, "16-byte broadcasts");
  constexpr int GROUPS = RANGES * (32 / COLS), DPAD = GROUPS * DPT;
  extern __shared__ __align__(16) float wkv_smem[];
  float (*rkw_s)[3][CHUNK][DPAD] = reinterpret_cast<float (*)[3][CHUNK][DPAD]>(wkv_smem);                          // [2][3][CHUNK][DPAD]
  float (*v_s)[CHUNK][COLS] = reinterpret_cast<float (*)[CHUNK][COLS]>(wkv_smem + 2 * 3 * CHUNK * DPAD);            // [2][CHUNK][COLS]
  float (*part_s)[GROUPS][COLS] = reinterpret_cast<float (*)[GROUPS][COLS]>(wkv_smem + 2 * 3 * CHUNK * DPAD + 2 * CHUNK * COLS);
  pdl_launch_dependents();
  const int head = blockIdx.y, e0 = blockIdx.x * COLS, seq = blockIdx.z;
  const int lane = threadIdx.x & 31, j = lane % COLS, group = (threadIdx.x >> 5) * (32 / COLS) + lane / COLS, e = e0 + j;
  const int d0 = group * DPT;
  for (int i = threadIdx.x; i < 2 * 3 * CHUNK * DPAD + 2 * CHUNK * COLS; i += SCAN_THREADS) wkv_smem[i] = 0.f;   // rows past dim stay zero
  __syncthreads();
  pdl_wait();
  const int first = cu_q[seq], count = cu_q[seq + 1] - first;
  if (count <= 0) return;
  float* mine = state + (size_t)state_slots[seq] * state_stride + (size_t)head * dim * dim;
  float s[DPT], bonus[DPT];
#pragma unroll
  for (int x = 0; x < DPT; ++x) {
    const int d = d0 + x;
    s[x] = (d < dim && e < dim) ? mine[(size_t)d * dim + e] : 0.f;
    bonus[x] = d < dim ? u[(size_t)head * dim + d] : 0.f;
  }
  const size_t col0 = (size_t)head * dim;
  // which 16-byte pieces of a chunk's r, k and w rows this thread copies: the same for every chunk, worked out once
  constexpr int PIECES_EACH = (CHUNK * DPAD / 4 + SCAN_THREADS - 1) / SCAN_THREADS;
  int piece_t[PIECES_EACH], piece_d[PIECES_EACH];
#pragma unroll
  for (int x = 0; x < PIECES_EACH; ++x) {
    const int i = threadIdx.x + x * SCAN_THREADS, pieces = max(dim >> 2, 1);
    piece_t[x] = i / pieces;                           // CHUNK and beyond: nothing to copy
    piece_d[x] = 4 * (i - piece_t[x] * pieces);
  }
  auto issue = [&](int buf, int t0) {
    const int n = min(CHUNK, count - t0);
    if (VEC) {
#pragma unroll
      for (int x = 0; x < PIECES_EACH; ++x) {
        if (piece_t[x] < n) {
          const size_t row = (size_t)(first + t0 + piece_t[x]);
          copy_async_16(&rkw_s[buf][0][piece_t[x]][piece_d[x]], r + row * r_stride + col0 + piece_d[x]);
          copy_async_16(&rkw_s[buf][1][piece_t[x]][piece_d[x]], k + row * k_stride + col0 + piece_d[x]);
          copy_async_16(&rkw_s[buf][2][piece_t[x]][piece_d[x]], w + row * heads * dim + col0 + piece_d[x]);
        }
      }
    } else {
      for (int i = threadIdx.x; i < 3 * n * dim; i += SCAN_THREADS) {
        const int which = i / (n * dim), rest = i - which * n * dim, t = rest / dim, d = rest - t * dim;
        const size_t row = (size_t)(first + t0 + t);
        const float* src = which == 0 ? r + row * r_stride : (which == 1 ? k + row * k_stride : w + row * heads * dim);
        copy_async_4(&rkw_s[buf][which][t][d], src + col0 + d);
      }
    }
    for (int i = threadIdx.x; i < n * COLS; i += SCAN_THREADS) {
      const int t = i / COLS, c = i - t * COLS;
      if (e0 + c < dim) copy_async_4(&v_s[buf][t][c], v + (size_t)(first + t0 + t) * v_stride + col0 + e0 + c);
    }
    copy_async_commit();
  };
  issue(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < count; t0 += CHUNK, buf ^= 1) {
    const int n = min(CHUNK, count - t0);
    if (t0 + CHUNK < count) {
      issue(buf ^ 1, t0 + CHUNK);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    auto token = [&](int t) {
      const float vt = v_s[buf][t][j];
      float p0 = 0.f, p1 = 0.f;
#pragma unroll
      for (int x = 0; x < DPT; x += 4) {
        const float4 rr = *reinterpret_cast<const float4*>(&rkw_s[buf][0][t][d0 + x]);
        const float4 kk = *reinterpret_cast<const float4*>(&rkw_s[buf][1][t][d0 + x]);
        const float4 ww = *reinterpret_cast<const float4*>(&rkw_s[buf][2][t][d0 + x]);
        float kv;
        kv = kk.x * vt; p0 = fmaf(rr.x, fmaf(bonus[x], kv, s[x]), p0); s[x] = fmaf(ww.x, s[x], kv);
        kv = kk.y * vt; p1 = fmaf(rr.y, fmaf(bonus[x + 1], kv, s[x + 1]), p1); s[x + 1] = fmaf(ww.y, s[x + 1], kv);
        kv = kk.z * vt; p0 = fmaf(rr.z, fmaf(bonus[x + 2], kv, s[x + 2]), p0); s[x + 2] = fmaf(ww.z, s[x + 2], kv);
        kv = kk.w * vt; p1 = fmaf(rr.w, fmaf(bonus[x + 3], kv, s[x + 3]), p1); s[x + 3] = fmaf(ww.w, s[x + 3], kv);
      }
      part_s[t][group][j] = p0 + p1;
    };
    if (n == CHUNK) {           // a whole chunk: its tokens' loads and sums interleave (the same operations per token either way)
#pragma unroll
      for (int t = 0; t < CHUNK; ++t) token(t);
    } else {
      for (int t = 0; t < n; ++t) token(t);
    }
    __syncthreads();
    if (threadIdx.x < n * COLS) {
      const int t = threadIdx.x / COLS, c = threadIdx.x - t * COLS;
      if (e0 + c < dim) {
        float sum = 0.f;
#pragma unroll
        for (int x = 0; x < GROUPS; ++x) sum += part_s[t][x][c];
        out[(size_t)(first + t0 + t) * heads * dim + col0 + e0 + c] = sum;
      }
    }
  }
#pragma unroll
  for (int x = 0; x < DPT; ++x) {
    const int d = d0 + x;
    if (d < dim && e < dim) mine[(size_t)d * dim + e] = s[x];
  }
}

template <int DPT, int COLS>
int launch_scan(const float* r, long r_stride, const float* k, long k_stride, const float* v, long v_stride, const float* w,
                const float* u, float* out, float* state, long state_stride, const int* cu_q, const int* state_slots, int n_seqs,
                int heads, int dim, cudaStream_t stream) {
  dim3 grid((dim + COLS - 1) / COLS, heads, n_seqs);
  constexpr int GROUPS = RANGES * (32 / COLS);
  constexpr size_t smem = (size_t)(2 * 3 * CHUNK * GROUPS * DPT + 2 * CHUNK * COLS + CHUNK * GROUPS * COLS) * sizeof(float);
  static LbPerDeviceOnce once;
  if (smem > 48 * 1024 && once.first()) {
    cudaFuncSetAttribute(wkv_scan_kernel<DPT, COLS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(wkv_scan_kernel<DPT, COLS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const bool vec = dim % 4 == 0 && r_stride % 4 == 0 && k_stride % 4 == 0 && (uintptr_t)r % 16 == 0 && (uintptr_t)k % 16 == 0 &&
                   (uintptr_t)w % 16 == 0;
  if (vec) lb_launch(wkv_scan_kernel<DPT, COLS, true>, grid, SCAN_THREADS, smem, stream, r, r_stride, k, k_stride, v, v_stride, w, u, out, state,
                     state_stride, cu_q, state_slots, heads, dim);
  else lb_launch(wkv_scan_kernel<DPT, COLS, false>, grid, SCAN_THREADS, smem, stream, r, r_stride, k, k_stride, v, v_stride, w, u, out, state,
                 state_stride, cu_q, state_slots, heads, dim);
  return lb_last_error();
}
}  // namespace

LB_EXPORT int lb_wkv_mix_tokens() { return MIX_TOKENS; }

// h [T, width] in the run's type; mu float [n_mix, width]; mixes [n_mix, T, width] in the run's type; state float
// [slots, state_stride] with the previous input at shift_off. Also leaves every request's newest input there (a second launch).
LB_EXPORT int lb_wkv_shift_mix(int dtype, const void* h, const float* mu, float* state, long state_stride, int shift_off,
                               const int* cu_q, const int* state_slots, const int* tile_seq, const int* tile_q0, int n_tiles,
                               int n_seqs, void* mixes, int tokens, int width, int n_mix, cudaStream_t stream) {
  if (n_tiles <= 0 || n_seqs <= 0 || tokens <= 0) return 0;
  if (width <= 0 || n_mix <= 0) return LB_ERR_SIZE;
  if (n_tiles > 0x7fffffff / MIX_TOKENS) return LB_ERR_SIZE;
  const dim3 grid(n_tiles, MIX_TOKENS);
  // the form depends on the width and the buffers' alignment only, never on the batch
  const bool vec = width % 4 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)mixes % 16 == 0 && (uintptr_t)mu % 16 == 0 &&
                   (uintptr_t)state % 16 == 0 && state_stride % 4 == 0 && shift_off % 4 == 0;
  const int threads = width >= 1024 ? 256 : 128;
#define LB_MIX_ARGS(T) (const T*)h, mu, (const float*)state, state_stride, shift_off, cu_q, state_slots, tile_seq, tile_q0, (T*)mixes, tokens, width, n_mix
  if (dtype == LB_F32) {
    if (vec) lb_launch(wkv_shift_mix_kernel<float, true>, grid, threads, 0, stream, LB_MIX_ARGS(float));
    else lb_launch(wkv_shift_mix_kernel<float, false>, grid, threads, 0, stream, LB_MIX_ARGS(float));
    lb_launch(wkv_shift_tail_kernel<float>, n_seqs, 256, 0, stream, (const float*)h, state, state_stride, shift_off, cu_q, state_slots, width);
  } else if (dtype == LB_BF16) {
    if (vec) lb_launch(wkv_shift_mix_kernel<bf16, true>, grid, threads, 0, stream, LB_MIX_ARGS(bf16));
    else lb_launch(wkv_shift_mix_kernel<bf16, false>, grid, threads, 0, stream, LB_MIX_ARGS(bf16));
    lb_launch(wkv_shift_tail_kernel<bf16>, n_seqs, 256, 0, stream, (const bf16*)h, state, state_stride, shift_off, cu_q, state_slots, width);
  } else {
    return LB_ERR_DTYPE;
  }
#undef LB_MIX_ARGS
  return lb_last_error();
}

// a float [T, a_stride] (the first `rank` columns); w2 [channels, rank] in the run's type; w0 float [channels]; decay float [T, channels].
LB_EXPORT int lb_wkv_decay(int dtype, const float* a, long a_stride, const void* w2, const float* w0, float* decay, int tokens,
                           int channels, int rank, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const size_t smem = (size_t)DECAY_TOKENS * ((rank + 3) & ~3) * sizeof(float);
  if (channels <= 0 || rank <= 0 || smem > 48 * 1024) return LB_ERR_SIZE;
  dim3 grid((tokens + DECAY_TOKENS - 1) / DECAY_TOKENS, (channels + 255) / 256);
  const bool vec = rank % 4 == 0 && (uintptr_t)w2 % 16 == 0;
  if (dtype == LB_F32) {
    if (vec) lb_launch(wkv_decay_kernel<float, true>, grid, 256, smem, stream, a, a_stride, (const float*)w2, w0, decay, tokens, channels, rank);
    else lb_launch(wkv_decay_kernel<float, false>, grid, 256, smem, stream, a, a_stride, (const float*)w2, w0, decay, tokens, channels, rank);
  } else if (dtype == LB_BF16) {
    if (vec) lb_launch(wkv_decay_kernel<bf16, true>, grid, 256, smem, stream, a, a_stride, (const bf16*)w2, w0, decay, tokens, channels, rank);
    else lb_launch(wkv_decay_kernel<bf16, false>, grid, 256, smem, stream, a, a_stride, (const bf16*)w2, w0, decay, tokens, channels, rank);
  } else {
    return LB_ERR_DTYPE;
  }
  return lb_last_error();
}

// S of head h of a request at state[slot * state_stride + h * dim * dim].
LB_EXPORT int lb_wkv_scan(const float* r, long r_stride, const float* k, long k_stride, const float* v, long v_stride,
                          const float* w, const float* u, float* out, float* state, long state_stride, const int* cu_q,
                          const int* state_slots, int n_seqs, int heads, int dim, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || heads > 65535 || n_seqs > 65535 || dim <= 0 || dim > 256) return LB_ERR_SIZE;
#define LB_WKV(DPT, COLS) launch_scan<DPT, COLS>(r, r_stride, k, k_stride, v, v_stride, w, u, out, state, state_stride, cu_q, state_slots, n_seqs, heads, dim, stream)
  // the split of S over lanes and warps is a function of the head size alone
  if (dim <= 32) return LB_WKV(4, 32);
  if (dim <= 64) return LB_WKV(4, 16);
  if (dim <= 128) return LB_WKV(8, 16);
  if (dim <= 192) return LB_WKV(12, 16);
  return LB_WKV(16, 16);
#undef LB_WKV
}
