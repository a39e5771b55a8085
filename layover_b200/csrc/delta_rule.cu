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

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// prepared [T, 2 kv_heads dim + heads vdim + 2 heads]: q (unit, scaled) | k (unit) | v | beta | decay
__global__ void __launch_bounds__(PREP_THREADS)
delta_prepare_kernel(const float* __restrict__ proj, long row_stride, int b_off, int a_off,
                     const float* __restrict__ taps, int n_taps, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, const float* __restrict__ state, long state_stride, int conv_off,
                     const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                     const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, float* __restrict__ prepared,
                     int heads, int kv_heads, int dim, int vdim, float unit_eps) {
  extern __shared__ float convolved[];     // the token's convolved channels
  pdl_launch_dependents();
  pdl_wait();
  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int row0 = cu_q[seq], q_len = cu_q[seq + 1] - row0;
  const int n_q = min(PREP_TOKENS, q_len - q0);
  const int qk = kv_heads * dim, channels = 2 * qk + heads * vdim, width = channels + 2 * heads;
  const float* tail = state + (size_t)state_slots[seq] * state_stride + conv_off;    // [n_taps - 1][channels]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = PREP_THREADS >> 5;
  const float q_scale = rsqrtf((float)dim);
  for (int i = 0; i < n_q; ++i) {
    const int local = q0 + i;
    const float* row = proj + (size_t)(row0 + local) * row_stride;
    float* dst = prepared + (size_t)(row0 + local) * width;
    for (int c = threadIdx.x; c < channels; c += PREP_THREADS) {
      float acc = 0.f;
      for (int j = 0; j < n_taps; ++j) {
        const int at = local - (n_taps - 1) + j;       // the input's place in this step; negative: before it
        const float x = at >= 0 ? proj[(size_t)(row0 + at) * row_stride + c] : tail[(size_t)(n_taps - 1 + at) * channels + c];
        acc = fmaf(taps[(size_t)c * n_taps + j], x, acc);
      }
      const float y = silu_f(acc);
      convolved[c] = y;
      if (c >= 2 * qk) dst[c] = y;
    }
    for (int h = threadIdx.x; h < heads; h += PREP_THREADS) {
      dst[channels + h] = 1.0f / (1.0f + expf(-row[b_off + h]));
      dst[channels + heads + h] = expf(-expf(a_log[h]) * softplus_f(row[a_off + h] + dt_bias[h]));
    }
    __syncthreads();
    for (int h = warp; h < 2 * kv_heads; h += warps) {     // a warp per q or k head: the same sum whatever the batch
      const float* src = convolved + h * dim;
      float ss = 0.f;
      for (int c = lane; c < dim; c += 32) ss += src[c] * src[c];
      ss = warp_sum(ss);
      const float inv = (1.0f / sqrtf(ss + unit_eps)) * (h < kv_heads ? q_scale : 1.f);
      for (int c = lane; c < dim; c += 32) dst[h * dim + c] = src[c] * inv;
    }
    __syncthreads();
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
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    // slot s takes the input at place n - (n_taps - 1) + s of this step, or, before the step, the tail's
    // slot s + n: read from slots above the one written, so ascending order moves the tail in place
    for (int s = 0; s < n_taps - 1; ++s) {
      const int at = n - (n_taps - 1) + s;
      tail[(size_t)s * channels + c] = at >= 0 ? proj[(size_t)(row0 + at) * row_stride + c] : tail[(size_t)(s + n) * channels + c];
    }
  }
}

// A warp owns 32 / SL columns of one head's state; a column's rows are split over SL lanes (RPL rows each, rows
// past `dim` are zeros), so the two sums over rows are a few shuffles each and no warp waits for another.
// A block is 4 warps on neighbouring columns of one (sequence, head).
template <int RPL, int SL, bool PREFETCH>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ prepared, float* __restrict__ out, float* __restrict__ state, long state_stride,
                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads, int kv_heads, int dim,
                  int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, slice = lane & (SL - 1);
  const int col = (blockIdx.x * 4 + warp) * (32 / SL) + lane / SL;
  const bool live = col < vdim;
  const int row0 = cu_q[seq], n = cu_q[seq + 1] - row0;
  const int qk = kv_heads * dim, channels = 2 * qk + heads * vdim, width = channels + 2 * heads;
  const int kv_head = head / (heads / kv_heads), r0 = slice * RPL;
  float* s_g = state + (size_t)state_slots[seq] * state_stride + (size_t)head * dim * vdim;
  float s[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) s[i] = (live && r0 + i < dim) ? s_g[(size_t)(r0 + i) * vdim + col] : 0.f;

  const float* p = prepared + (size_t)row0 * width;
  const int q_at = kv_head * dim + r0, k_at = qk + kv_head * dim + r0, v_at = 2 * qk + head * vdim + col;
  float k[RPL], q[RPL], v, beta, decay;
  auto fetch = [&](const float* src, float (&kk)[RPL], float (&qq)[RPL], float& vv, float& bb, float& dd) {
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const bool in = r0 + i < dim;
      kk[i] = in ? src[k_at + i] : 0.f;
      qq[i] = in ? src[q_at + i] : 0.f;
    }
    vv = live ? src[v_at] : 0.f;
    bb = src[channels + head];
    dd = src[channels + heads + head];
  };
  if (n > 0) fetch(p, k, q, v, beta, decay);
  for (int t = 0; t < n; ++t) {
    float kn[RPL], qn[RPL], vn = 0.f, bn = 0.f, dn = 0.f;      // the next token's operands, asked for before this token's sums
    if constexpr (PREFETCH) {
      if (t + 1 < n) fetch(p + (size_t)(t + 1) * width, kn, qn, vn, bn, dn);
    }
    float kv = 0.f;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      s[i] *= decay;
      kv = fmaf(s[i], k[i], kv);
    }
#pragma unroll
    for (int m = 1; m < SL; m <<= 1) kv += __shfl_xor_sync(0xffffffffu, kv, m);
    const float u = beta * (v - kv);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      s[i] = fmaf(k[i], u, s[i]);
      o = fmaf(s[i], q[i], o);
    }
#pragma unroll
    for (int m = 1; m < SL; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
    if (slice == 0 && live) out[(size_t)(row0 + t) * heads * vdim + head * vdim + col] = o;
    if constexpr (PREFETCH) {
#pragma unroll
      for (int i = 0; i < RPL; ++i) { k[i] = kn[i]; q[i] = qn[i]; }
      v = vn; beta = bn; decay = dn;
    } else {
      if (t + 1 < n) fetch(p + (size_t)(t + 1) * width, k, q, v, beta, decay);
    }
  }
#pragma unroll
  for (int i = 0; i < RPL; ++i)
    if (live && r0 + i < dim) s_g[(size_t)(r0 + i) * vdim + col] = s[i];
}

template <int RPL, int SL>
static int launch_scan(const float* prepared, float* out, float* state, long state_stride, const int* cu_q,
                       const int* state_slots, int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  constexpr int COLS = 4 * (32 / SL);       // columns of a block
  dim3 grid((vdim + COLS - 1) / COLS, heads, n_seqs);
  lb_launch(delta_scan_kernel<RPL, SL, true>, grid, 128, 0, stream, prepared, out, state, state_stride, cu_q, state_slots,
            heads, kv_heads, dim, vdim);
  return lb_last_error();
}

// out[t, h, c] = T(o * rsqrt(mean_c o^2 + eps) * weight[c] * silu(gate[t, h, c])): a warp per (token, head).
template <typename T>
__global__ void head_gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, long gate_stride,
                                          const float* __restrict__ weight, T* __restrict__ out, int heads, int vdim,
                                          float eps) {
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
    for (int c = lane; c < vdim; c += 32) Elem<T>::store(out + (t * heads + h) * vdim + c, src[c] * inv * weight[c] * silu_f(g[c]));
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
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const size_t smem = (size_t)channels * sizeof(float);
  if (smem > 200 * 1024) return LB_ERR_SIZE;
  static LbPerDeviceOnce once;
  if (smem > 48 * 1024 && once.first())
    cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  lb_launch(delta_prepare_kernel, n_tiles, PREP_THREADS, smem, stream, proj, row_stride, b_off, a_off, taps, n_taps, a_log,
            dt_bias, (const float*)state, state_stride, conv_off, cu_q, state_slots, tile_seq, tile_q0, prepared, heads, kv_heads,
            dim, vdim, unit_eps);
  int code = lb_last_error();
  if (code || n_taps == 1) return code;
  lb_launch(conv_tail_kernel, n_seqs, 256, 0, stream, proj, row_stride, state, state_stride, conv_off, cu_q, state_slots, n_taps,
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
  if (dim <= 32) return LB_DELTA(8, 4);
  if (dim <= 64) return LB_DELTA(16, 4);
  if (dim <= 96) return LB_DELTA(24, 4);
  if (dim <= 128) return LB_DELTA(32, 4);
  if (dim <= 192) return LB_DELTA(24, 8);
  return LB_DELTA(32, 8);
#undef LB_DELTA
}

LB_EXPORT int lb_head_gated_rmsnorm(int dtype, const float* o, const float* gate, long gate_stride, const float* weight,
                                    void* out, int tokens, int heads, int vdim, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads <= 0 || vdim <= 0) return LB_ERR_SIZE;
  const int threads = 32 * (heads < 8 ? heads : 8);
  if (dtype == LB_F32)
    lb_launch(head_gated_rmsnorm_kernel<float>, tokens, threads, 0, stream, o, gate, gate_stride, weight, (float*)out, heads, vdim, eps);
  else if (dtype == LB_BF16)
    lb_launch(head_gated_rmsnorm_kernel<bf16>, tokens, threads, 0, stream, o, gate, gate_stride, weight, (bf16*)out, heads, vdim, eps);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}
