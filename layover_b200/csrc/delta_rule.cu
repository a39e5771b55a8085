// The gated delta rule: linear attention whose state is corrected towards each new value before it
// is read, with a decay per head and token, behind short causal convolutions of q, k and v.
//
// A token's row of the stacked projection (32-bit, `row_stride` floats) starts with the convolved
// channels [ q: kv_heads * dim | k: kv_heads * dim | v: heads * vdim ]; further on it holds, per head,
// the logits of the write strength (`b_off`) and of the decay's step size (`a_off`).
//
//   prepare   y_c(t) = silu(sum_j taps[c, j] x_c(t - (n_taps - 1) + j))       x before the step's first token comes
//             from the request's state (the last n_taps - 1 inputs, zeros at the start of a sequence)
//             q, k heads -> y / sqrt(sum(y^2) + unit_eps), q also times dim^(-1/2)
//             beta = sigmoid(b), decay = exp(-exp(A_log) * softplus(a + dt_bias))
//   scan      S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q            per head, S [dim, vdim]
//   finish    out = T(o * rsqrt(mean(o^2) + eps) * weight * silu(gate))                    per head over vdim
//
// Everything is 32-bit arithmetic in a fixed order per token, so a request's results do not depend on
// how its tokens are cut into steps or on what else shares the batch. The state of a request is one
// row of `state`: S of every head, then the last n_taps - 1 inputs of every convolved channel.
#include <math.h>

#include "common.cuh"

namespace {
constexpr int PREP_TOKENS = 16;    // tokens of one sequence that a block of the prepare kernel takes
constexpr int PREP_THREADS = 256;
constexpr int PREP_UNITS = 4;      // heads (of q, k or v) that a block takes for its tokens

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// prepared [T, 2 kv_heads dim + heads vdim + 2 heads]: q (unit, scaled) | k (unit) | v | beta | decay
// A warp takes one (token, unit): a unit is a head of q, of k or of v, and one more unit is the heads' beta and
// decay. A q or k head's sum of squares is the lanes' sums over channels lane, lane + 32, ... and then the warp's
// tree: the same order whatever the batch or the cut. blockIdx.x: a tile of tokens of one sequence; blockIdx.y: units.
__global__ void __launch_bounds__(PREP_THREADS)
delta_prepare_kernel(const float* __restrict__ proj, long row_stride, int b_off, int a_off,
                     const float* __restrict__ taps, int n_taps, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, const float* __restrict__ state, long state_stride, int conv_off,
                     const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                     const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, float* __restrict__ prepared,
                     int heads, int kv_heads, int dim, int vdim, float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int row0 = cu_q[seq], q_len = cu_q[seq + 1] - row0;
  const int n_q = min(PREP_TOKENS, q_len - q0);
  const int qk = kv_heads * dim, channels = 2 * qk + heads * vdim, width = channels + 2 * heads;
  const int units = 2 * kv_heads + heads + 1, unit0 = blockIdx.y * PREP_UNITS;
  const int n_units = min(PREP_UNITS, units - unit0);
  const float* tail = state + (size_t)state_slots[seq] * state_stride + conv_off;    // [n_taps - 1][channels]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = PREP_THREADS >> 5;
  const float q_scale = rsqrtf((float)dim);
  for (int item = warp; item < n_q * n_units; item += warps) {
    const int local = q0 + item / n_units, unit = unit0 + item % n_units;
    const float* row = proj + (size_t)(row0 + local) * row_stride;
    float* dst = prepared + (size_t)(row0 + local) * width;
    if (unit == units - 1) {
      for (int h = lane; h < heads; h += 32) {
        dst[channels + h] = 1.0f / (1.0f + expf(-row[b_off + h]));
        dst[channels + heads + h] = expf(-expf(a_log[h]) * softplus_f(row[a_off + h] + dt_bias[h]));
      }
      continue;
    }
    const bool unit_norm = unit < 2 * kv_heads;
    const int c0 = unit_norm ? unit * dim : 2 * qk + (unit - 2 * kv_heads) * vdim, n_c = unit_norm ? dim : vdim;
    float ss = 0.f;
    for (int c = c0 + lane; c < c0 + n_c; c += 32) {
      float acc = 0.f;
      for (int j = 0; j < n_taps; ++j) {
        const int at = local - (n_taps - 1) + j;       // the input's place in this step; negative: before it
        const float x = at >= 0 ? proj[(size_t)(row0 + at) * row_stride + c] : tail[(size_t)(n_taps - 1 + at) * channels + c];
        acc = fmaf(taps[(size_t)c * n_taps + j], x, acc);
      }
      const float y = silu_f(acc);
      dst[c] = y;
      ss += y * y;
    }
    if (!unit_norm) continue;
    ss = warp_sum(ss);
    const float inv = (1.0f / sqrtf(ss + unit_eps)) * (unit < kv_heads ? q_scale : 1.f);
    for (int c = c0 + lane; c < c0 + n_c; c += 32) dst[c] *= inv;      // the lane's own writes
  }
}

// The request's last n_taps - 1 inputs of every convolved channel, after this step's tokens.
__global__ void conv_tail_kernel(const float* __restrict__ proj, long row_stride, float* __restrict__ state, long state_stride,
                                 int conv_off, const int* __restrict__ cu_q, const int* __restrict__ state_slots, int n_taps,
                                 int channels) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, row0 = cu_q[seq], n = cu_q[seq + 1] - row0;
  float* tail = state + (size_t)state_slots[seq] * state_stride + conv_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    // slot s takes the input at place n - (n_taps - 1) + s of this step, or, before the step, the tail's
    // slot s + n: read from slots above the one written, so ascending order moves the tail in place
    for (int s = 0; s < n_taps - 1; ++s) {
      const int at = n - (n_taps - 1) + s;
      tail[(size_t)s * channels + c] = at >= 0 ? proj[(size_t)(row0 + at) * row_stride + c] : tail[(size_t)(s + n) * channels + c];
    }
  }
}

// A warp owns 32 / SL columns of one head's state in registers; a column's rows are split over SL lanes (RPL rows
// each, rows past `dim` are zeros). A block is SCAN_WARPS warps on neighbouring columns of one (sequence, head). A
// token is a chain of dependent steps, and a lone warp issues one instruction in about three cycles, so a lane's share
// is kept small (a head of 128 rows: 8 rows a lane, 16 lanes a column, 1,024 warps for 16 heads of 128 columns) and
// the chain short: both sums over rows are taken from the state BEFORE the token's write, side by side,
//     a = S^T k,  b = S^T q            (one round of shuffles for the two)
//     u = beta (v - g a),   o = g b + u (k . q),   S <- g S + k u^T
// which is the recurrence S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with the read-out written through
// the update. The tokens' operands come through shared memory, SCAN_TOKENS tokens at a time, the next tokens' copies
// in flight while these are worked on: k and q of a token are stored so that lane slice s reads 16-byte piece
// j * SL + s for its j-th four rows (its rows are 4 (j SL + s) .. + 3), which a warp reads without a bank conflict.
// Each sum over rows runs in four partial sums and the lanes' tree, k . q in a warp's strided sums and its tree: orders
// that depend on the head size alone.
constexpr int SCAN_TOKENS = 8, SCAN_WARPS = 8, SCAN_THREADS = 32 * SCAN_WARPS;

__device__ __forceinline__ void copy_async_4(float* dst_shared, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_16(float* dst_shared, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int RPL, int SL>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ prepared, float* __restrict__ out, float* __restrict__ state, long state_stride,
                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads, int kv_heads, int dim,
                  int vdim) {
  constexpr int ROWS = RPL * SL, COLS = SCAN_WARPS * (32 / SL), J = RPL / 4;
  static_assert(RPL % 4 == 0, "a lane's rows come in fours");
  __shared__ __align__(16) float kq_s[2][SCAN_TOKENS][2 * ROWS];      // k rows, then q rows
  __shared__ float v_s[2][SCAN_TOKENS][COLS];
  __shared__ float bd_s[2][SCAN_TOKENS][2];                            // beta, decay
  __shared__ float dot_s[SCAN_TOKENS];                                 // k . q
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, slice = lane & (SL - 1);
  const int col_local = warp * (32 / SL) + lane / SL, col0 = blockIdx.x * COLS, col = col0 + col_local;
  const bool live = col < vdim;
  const int row0 = cu_q[seq], n = cu_q[seq + 1] - row0;
  const int qk = kv_heads * dim, channels = 2 * qk + heads * vdim, width = channels + 2 * heads;
  const int kv_head = head / (heads / kv_heads);
  auto row_of = [&](int i) { return ((i >> 2) * SL + slice) * 4 + (i & 3); };      // the lane's i-th row
  float* s_g = state + (size_t)state_slots[seq] * state_stride + (size_t)head * dim * vdim;
  float s[RPL];
  // With many lanes a column a warp's direct reads of S would touch 8 bytes of every 32-byte sector: the block's
  // columns of S go through shared memory instead (whole runs of COLS floats a row), both ways.
  constexpr bool VIA_SHARED = SL >= 8;
  constexpr int TILE_STRIDE = COLS + 1 <= 2 * SCAN_TOKENS * 2 ? COLS + 1 : COLS;      // ROWS x TILE_STRIDE floats fit kq_s
  static_assert(!VIA_SHARED || COLS <= 2 * SCAN_TOKENS * 2, "the state tile borrows the operand buffers");
  float* tile = &kq_s[0][0][0];
  if constexpr (VIA_SHARED) {
    for (int i = threadIdx.x; i < dim * COLS; i += SCAN_THREADS) {
      const int r = i / COLS, c = i - r * COLS;
      tile[r * TILE_STRIDE + c] = col0 + c < vdim ? s_g[(size_t)r * vdim + col0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RPL; ++i) s[i] = row_of(i) < dim ? tile[row_of(i) * TILE_STRIDE + col_local] : 0.f;
    __syncthreads();
  } else {
#pragma unroll
    for (int i = 0; i < RPL; ++i) s[i] = (live && row_of(i) < dim) ? s_g[(size_t)row_of(i) * vdim + col] : 0.f;
  }
  for (int i = threadIdx.x; i < 2 * SCAN_TOKENS * 2 * ROWS; i += SCAN_THREADS) (&kq_s[0][0][0])[i] = 0.f;     // rows past dim stay zeros
  for (int i = threadIdx.x; i < 2 * SCAN_TOKENS * COLS; i += SCAN_THREADS) (&v_s[0][0][0])[i] = 0.f;
  __syncthreads();

  const float* p = prepared + (size_t)row0 * width;
  const int q_at = kv_head * dim, k_at = qk + kv_head * dim, v_at = 2 * qk + head * vdim + col0;
  const int n_cols = min(COLS, vdim - col0);
  // 16-byte copies where every piece of k and q starts on a 16-byte boundary (head sizes and row widths in fours)
  const bool wide = ((dim | width | qk) & 3) == 0 && (reinterpret_cast<size_t>(prepared) & 15) == 0;
  auto stage = [&](int buffer, int t0) {       // tokens t0 .. of the sequence's step into a buffer
    const int count = min(SCAN_TOKENS, n - t0);
    const float* src0 = p + (size_t)t0 * width;
    if (wide) {
      const int per = dim >> 2;                // 16-byte pieces of a token's k, and of its q
      for (int i = threadIdx.x; i < count * 2 * per; i += SCAN_THREADS) {
        const int t = i / (2 * per), rest = i - t * 2 * per, is_q = rest >= per ? 1 : 0, piece = rest - is_q * per;
        copy_async_16(&kq_s[buffer][t][is_q * ROWS + 4 * piece], src0 + (size_t)t * width + (is_q ? q_at : k_at) + 4 * piece);
      }
    } else {
      for (int i = threadIdx.x; i < count * 2 * dim; i += SCAN_THREADS) {
        const int t = i / (2 * dim), rest = i - t * 2 * dim, is_q = rest >= dim ? 1 : 0, r = rest - is_q * dim;
        copy_async_4(&kq_s[buffer][t][is_q * ROWS + r], src0 + (size_t)t * width + (is_q ? q_at : k_at) + r);
      }
    }
    for (int i = threadIdx.x; i < count * COLS; i += SCAN_THREADS) {
      const int t = i / COLS, c = i - t * COLS;
      if (c < n_cols) copy_async_4(&v_s[buffer][t][c], src0 + (size_t)t * width + v_at + c);
    }
    if (threadIdx.x < 2 * count)
      copy_async_4(&bd_s[buffer][threadIdx.x >> 1][threadIdx.x & 1],
                   src0 + (size_t)(threadIdx.x >> 1) * width + channels + (threadIdx.x & 1) * heads + head);
    copy_async_commit();
  };
  if (n > 0) stage(0, 0);
  for (int t0 = 0, buffer = 0; t0 < n; t0 += SCAN_TOKENS, buffer ^= 1) {
    const int count = min(SCAN_TOKENS, n - t0);
    copy_async_wait_all();
    __syncthreads();           // this buffer is whole; every warp is done with the other one and with dot_s
    if (t0 + SCAN_TOKENS < n) stage(buffer ^ 1, t0 + SCAN_TOKENS);
    for (int t = warp; t < count; t += SCAN_WARPS) {
      float part = 0.f;
      for (int r = lane; r < ROWS; r += 32) part = fmaf(kq_s[buffer][t][r], kq_s[buffer][t][ROWS + r], part);
      part = warp_sum(part);
      if (lane == 0) dot_s[t] = part;
    }
    __syncthreads();
    for (int t = 0; t < count; ++t) {
      const float4* k4 = reinterpret_cast<const float4*>(&kq_s[buffer][t][0]) + slice;
      const float4* q4 = reinterpret_cast<const float4*>(&kq_s[buffer][t][ROWS]) + slice;
      const float v = v_s[buffer][t][col_local], beta = bd_s[buffer][t][0], decay = bd_s[buffer][t][1], k_dot_q = dot_s[t];
      float4 k[J];
      float pa[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < J; ++j) {
        k[j] = k4[j * SL];
        const float4 q = q4[j * SL];
        pa[0] = fmaf(s[4 * j], k[j].x, pa[0]);
        pa[1] = fmaf(s[4 * j + 1], k[j].y, pa[1]);
        pa[2] = fmaf(s[4 * j + 2], k[j].z, pa[2]);
        pa[3] = fmaf(s[4 * j + 3], k[j].w, pa[3]);
        pb[0] = fmaf(s[4 * j], q.x, pb[0]);
        pb[1] = fmaf(s[4 * j + 1], q.y, pb[1]);
        pb[2] = fmaf(s[4 * j + 2], q.z, pb[2]);
        pb[3] = fmaf(s[4 * j + 3], q.w, pb[3]);
      }
      float a = (pa[0] + pa[1]) + (pa[2] + pa[3]), b = (pb[0] + pb[1]) + (pb[2] + pb[3]);
#pragma unroll
      for (int m = 1; m < SL; m <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, m);
        b += __shfl_xor_sync(0xffffffffu, b, m);
      }
      const float u = beta * (v - decay * a);
#pragma unroll
      for (int j = 0; j < J; ++j) {
        s[4 * j] = fmaf(k[j].x, u, decay * s[4 * j]);
        s[4 * j + 1] = fmaf(k[j].y, u, decay * s[4 * j + 1]);
        s[4 * j + 2] = fmaf(k[j].z, u, decay * s[4 * j + 2]);
        s[4 * j + 3] = fmaf(k[j].w, u, decay * s[4 * j + 3]);
      }
      if (slice == 0 && live) out[(size_t)(row0 + t0 + t) * heads * vdim + head * vdim + col] = fmaf(u, k_dot_q, decay * b);
    }
  }
  // The next kernel's blocks are let in only now: let in at the start they would sit beside this block's few warps
  // for the whole walk over the tokens, waiting.
  pdl_launch_dependents();
  if constexpr (VIA_SHARED) {
    __syncthreads();           // every warp is done with the operand buffers
#pragma unroll
    for (int i = 0; i < RPL; ++i)
      if (row_of(i) < dim) tile[row_of(i) * TILE_STRIDE + col_local] = s[i];
    __syncthreads();
    for (int i = threadIdx.x; i < dim * COLS; i += SCAN_THREADS) {
      const int r = i / COLS, c = i - r * COLS;
      if (col0 + c < vdim) s_g[(size_t)r * vdim + col0 + c] = tile[r * TILE_STRIDE + c];
    }
  } else {
#pragma unroll
    for (int i = 0; i < RPL; ++i)
      if (live && row_of(i) < dim) s_g[(size_t)row_of(i) * vdim + col] = s[i];
  }
}

template <int RPL, int SL>
static int launch_scan(const float* prepared, float* out, float* state, long state_stride, const int* cu_q,
                       const int* state_slots, int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  constexpr int COLS = SCAN_WARPS * (32 / SL);       // columns of a block
  dim3 grid((vdim + COLS - 1) / COLS, heads, n_seqs);
  lb_launch(delta_scan_kernel<RPL, SL>, grid, SCAN_THREADS, 0, stream, prepared, out, state, state_stride, cu_q, state_slots,
            heads, kv_heads, dim, vdim);
  return lb_last_error();
}

// out[t, h, c] = T(o * rsqrt(mean_c o^2 + eps) * weight[h * weight_stride + c] * silu(gate[t, h, c])): a warp per (token,
// head). weight_stride 0: one weight of vdim entries shared by the heads; vdim: a weight per channel of all heads.
template <typename T>
__global__ void head_gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, long gate_stride,
                                          const float* __restrict__ weight, T* __restrict__ out, int heads, int vdim,
                                          float eps, int weight_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const size_t t = blockIdx.x;
  for (int h = warp; h < heads; h += warps) {
    const float* src = o + (t * heads + h) * vdim;
    const float* g = gate + t * gate_stride + (size_t)h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss += src[c] * src[c];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    const float* wh = weight + (size_t)h * weight_stride;
    for (int c = lane; c < vdim; c += 32) Elem<T>::store(out + (t * heads + h) * vdim + c, src[c] * inv * wh[c] * silu_f(g[c]));
  }
}
}  // namespace

LB_EXPORT int lb_delta_prepare_tokens() { return PREP_TOKENS; }

// proj float [T, row_stride]; taps float [2 kv_heads dim + heads vdim, n_taps] (the last column is the current
// token's); state float [slots, state_stride] with the convolutions' tail at conv_off; prepared float
// [T, 2 kv_heads dim + heads vdim + 2 heads]. Also moves every request's tail past this step's tokens (a second launch).
LB_EXPORT int lb_delta_prepare(const float* proj, long row_stride, int b_off, int a_off, const float* taps, int n_taps,
                               const float* a_log, const float* dt_bias, float* state, long state_stride, int conv_off,
                               const int* cu_q, const int* state_slots, const int* tile_seq, const int* tile_q0, int n_tiles,
                               int n_seqs, float* prepared, int heads, int kv_heads, int dim, int vdim, float unit_eps,
                               cudaStream_t stream) {
  if (n_tiles <= 0 || n_seqs <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || n_taps <= 0 || n_seqs > 65535) return LB_ERR_SIZE;
  const int channels = 2 * kv_heads * dim + heads * vdim, units = 2 * kv_heads + heads + 1;
  dim3 grid(n_tiles, (units + PREP_UNITS - 1) / PREP_UNITS);
  if (grid.y > 65535) return LB_ERR_SIZE;
  lb_launch(delta_prepare_kernel, grid, PREP_THREADS, 0, stream, proj, row_stride, b_off, a_off, taps, n_taps, a_log, dt_bias,
            (const float*)state, state_stride, conv_off, cu_q, state_slots, tile_seq, tile_q0, prepared, heads, kv_heads, dim, vdim,
            unit_eps);
  int code = lb_last_error();
  if (code || n_taps == 1) return code;
  lb_launch(conv_tail_kernel, dim3(n_seqs, min((channels + 255) / 256, 64)), 256, 0, stream, proj, row_stride, state, state_stride, conv_off, cu_q, state_slots, n_taps,
            channels);
  return lb_last_error();
}

// prepared as above; out float [T, heads * vdim]; S of head h of a request at state[slot * state_stride + h * dim * vdim].
LB_EXPORT int lb_delta_scan(const float* prepared, float* out, float* state, long state_stride, const int* cu_q,
                            const int* state_slots, int n_seqs, int heads, int kv_heads, int dim, int vdim,
                            cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || heads > 65535 || n_seqs > 65535 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > 256 || vdim <= 0)
    return LB_ERR_SIZE;
  // the split of S over lanes is a function of the head size alone
#define LB_DELTA(R, S) launch_scan<R, S>(prepared, out, state, state_stride, cu_q, state_slots, n_seqs, heads, kv_heads, dim, vdim, stream)
  if (dim <= 16) return LB_DELTA(4, 4);
  if (dim <= 32) return LB_DELTA(4, 8);
  if (dim <= 64) return LB_DELTA(4, 16);
  if (dim <= 128) return LB_DELTA(8, 16);
  if (dim <= 192) return LB_DELTA(12, 16);
  return LB_DELTA(16, 16);
#undef LB_DELTA
}

LB_EXPORT int lb_head_gated_rmsnorm(int dtype, const float* o, const float* gate, long gate_stride, const float* weight,
                                    void* out, int tokens, int heads, int vdim, float eps, int weight_stride,
                                    cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || vdim <= 0 || (weight_stride != 0 && weight_stride != vdim)) return LB_ERR_SIZE;
  const int threads = 32 * (heads < 8 ? heads : 8);
  if (dtype == LB_F32)
    lb_launch(head_gated_rmsnorm_kernel<float>, tokens, threads, 0, stream, o, gate, gate_stride, weight, (float*)out, heads, vdim, eps, weight_stride);
  else if (dtype == LB_BF16)
    lb_launch(head_gated_rmsnorm_kernel<bf16>, tokens, threads, 0, stream, o, gate, gate_stride, weight, (bf16*)out, heads, vdim, eps, weight_stride);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}
