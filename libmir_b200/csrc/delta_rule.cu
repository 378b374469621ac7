// The gated delta rule: a recurrent mixer whose state per head is a matrix S [key channels, value channels].
//
// Per token, with q and k already unit vectors (q also times key_dim^-1/2), v the value row, beta in (0, 1) and a
// decay g in (0, 1) per head or per key channel:
//     S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
// so the read-out sees the write of its own token.  The state is 32-bit, lives in the request's state slot and is
// carried from step to step; everything that enters the recurrence is computed in 32-bit here: the unit norms, the
// sigmoid of beta, softplus, both exponentials of the decay.
//
// Kernels of this file:
//   short_conv_silu   y[t, c] = silu(sum_j w[c, j] x[t - (taps-1) + j, c]) over a request's own tokens, with the
//                     taps-1 inputs before the portion taken from the request's state; then the state's update.
//   delta_rule_scan   the recurrence, one warp per (request, head, value channel): the warp holds one column of S in
//                     registers (key channel i in lane i % 32), walks over the request's tokens of this step, and
//                     writes the column back.  No shared memory, no block barrier: the two dot products per token
//                     are warp reductions.  The state is stored [head][value channel][key channel], so a column is
//                     one contiguous run and every access of it is coalesced.
//   gated_head_norm   out = o / rms(o) * weight * act(gate) per (token, head), act = silu or sigmoid.
// A row of a captured decode batch whose position is negative is padding: nothing of it is read or written.
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kMaxTaps = 8;
constexpr int kMaxPerLane = 8;          // key channels per lane: key_dim <= 256

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// grid (tokens, ceil(channels / 256)).  x: the packed projection rows, channel c of token t at x[t * ldx + c].
template <typename T>
__global__ void short_conv_silu_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w,
                                       const float* __restrict__ tail, const int* __restrict__ row_of_token,
                                       const int* __restrict__ query_starts, const int* __restrict__ state_slots,
                                       const int* __restrict__ positions, float* __restrict__ out, int channels,
                                       int taps) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels || positions[token] < 0) return;
  const int row = row_of_token[token];
  const int start = query_starts[row];
  const int local = token - start;
  const float* old = tail + (size_t)state_slots[row] * (taps - 1) * channels;
  float acc = 0.0f;
  for (int j = 0; j < taps; ++j) {
    const int src = local - (taps - 1) + j;
    const float value = src >= 0 ? to_float(x[(size_t)(start + src) * ldx + c]) : old[(size_t)(taps - 1 + src) * channels + c];
    acc = fmaf(to_float(w[(size_t)c * taps + j]), value, acc);
  }
  out[(size_t)token * channels + c] = silu(acc);
}

// grid (rows, ceil(channels / 256)): the last taps-1 inputs of the request, old ones where the portion is shorter.
template <typename T>
__global__ void short_conv_tail_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ tail,
                                       const int* __restrict__ query_starts, const int* __restrict__ state_slots,
                                       const int* __restrict__ positions, int channels, int taps) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int start = query_starts[row], count = query_starts[row + 1] - start;
  if (c >= channels || count <= 0 || positions[start] < 0) return;
  float* mine = tail + (size_t)state_slots[row] * (taps - 1) * channels;
  float keep[kMaxTaps];
  for (int j = 0; j < taps - 1; ++j) {
    const int src = count - (taps - 1) + j;
    keep[j] = src >= 0 ? to_float(x[(size_t)(start + src) * ldx + c]) : mine[(size_t)(taps - 1 + src) * channels + c];
  }
  for (int j = 0; j < taps - 1; ++j) mine[(size_t)j * channels + c] = keep[j];
}

// One warp per (request row, head, value channel); blockDim (32, warps), grid (rows, heads, ceil(vdim / warps)).
//   qkv       [tokens, 2 G D + H V] 32-bit: q | k | v after the short convolution and silu
//   beta_raw  element (t, h) at beta_raw[t * ld_beta + h], before the sigmoid
//   decay_raw PER_CHANNEL: element (t, h, i) at decay_raw[t * ld_decay + h * D + i], else (t, h) at [t * ld_decay + h]
//   dt_bias   [H D] or [H], a_log [H]
//   state     [slots, H, V, D] 32-bit
//   out       [tokens, H V] 32-bit: o before the head norm
template <typename TB, typename TD, int PER, bool PER_CHANNEL>
__global__ void delta_rule_scan_kernel(const float* __restrict__ qkv, const TB* __restrict__ beta_raw, long long ld_beta,
                                       const TD* __restrict__ decay_raw, long long ld_decay,
                                       const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                       float* __restrict__ state, const int* __restrict__ query_starts,
                                       const int* __restrict__ state_slots, const int* __restrict__ positions,
                                       float* __restrict__ out, int heads, int kv_heads, int key_dim, int value_dim) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x;
  const int row = blockIdx.x, head = blockIdx.y;
  const int column = blockIdx.z * blockDim.y + threadIdx.y;
  const int start = query_starts[row], end = query_starts[row + 1];
  if (column >= value_dim || end <= start || positions[start] < 0) return;
  const int kv_head = head / (heads / kv_heads);
  const int width = 2 * kv_heads * key_dim + heads * value_dim;
  const size_t q_offset = (size_t)kv_head * key_dim, k_offset = (size_t)(kv_heads + kv_head) * key_dim;
  const size_t v_offset = (size_t)2 * kv_heads * key_dim + (size_t)head * value_dim + column;
  float* column_state = state + (((size_t)state_slots[row] * heads + head) * value_dim + column) * key_dim;
  const float rate = expf(a_log[head]);
  const float q_scale = rsqrtf((float)key_dim);

  float s[PER], bias[PER];
#pragma unroll
  for (int m = 0; m < PER; ++m) {
    const int i = lane + 32 * m;
    s[m] = i < key_dim ? column_state[i] : 0.0f;
    bias[m] = (PER_CHANNEL && i < key_dim) ? dt_bias[(size_t)head * key_dim + i] : 0.0f;
  }
  const float head_bias = PER_CHANNEL ? 0.0f : dt_bias[head];

  for (int token = start; token < end; ++token) {
    const float* row_values = qkv + (size_t)token * width;
    float q[PER], k[PER], g[PER];
    float q_square = 0.0f, k_square = 0.0f;
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      const int i = lane + 32 * m;
      q[m] = i < key_dim ? row_values[q_offset + i] : 0.0f;
      k[m] = i < key_dim ? row_values[k_offset + i] : 0.0f;
      q_square = fmaf(q[m], q[m], q_square);
      k_square = fmaf(k[m], k[m], k_square);
      if (PER_CHANNEL)
        g[m] = i < key_dim ? expf(-rate * softplus(to_float(decay_raw[(size_t)token * ld_decay + (size_t)head * key_dim + i]) + bias[m]))
                           : 1.0f;
    }
    if (!PER_CHANNEL) {
      const float one = expf(-rate * softplus(to_float(decay_raw[(size_t)token * ld_decay + head]) + head_bias));
#pragma unroll
      for (int m = 0; m < PER; ++m) g[m] = one;
    }
    const float beta = sigmoid(to_float(beta_raw[(size_t)token * ld_beta + head]));
    const float value = row_values[v_offset];
    const float q_unit = rsqrtf(warp_sum(q_square) + 1e-6f) * q_scale;
    const float k_unit = rsqrtf(warp_sum(k_square) + 1e-6f);
    float seen = 0.0f;
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      k[m] *= k_unit;
      q[m] *= q_unit;
      s[m] *= g[m];
      seen = fmaf(s[m], k[m], seen);
    }
    const float update = beta * (value - warp_sum(seen));
    float read = 0.0f;
#pragma unroll
    for (int m = 0; m < PER; ++m) {
      s[m] = fmaf(k[m], update, s[m]);
      read = fmaf(s[m], q[m], read);
    }
    read = warp_sum(read);
    if (lane == 0) out[((size_t)token * heads + head) * value_dim + column] = read;
  }
#pragma unroll
  for (int m = 0; m < PER; ++m) {
    const int i = lane + 32 * m;
    if (i < key_dim) column_state[i] = s[m];
  }
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * weight * act(gate).
template <typename T>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long ld_gate,
                                       const float* __restrict__ weight, T* __restrict__ out, int units,
                                       int heads, int value_dim, float eps, int sigmoid_gate) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int unit = blockIdx.x * blockDim.y + threadIdx.y;       // token * heads + head
  if (unit >= units) return;
  const int lane = threadIdx.x;
  const float* src = o + (size_t)unit * value_dim;
  float sum = 0.0f;
  for (int d = lane; d < value_dim; d += 32) sum = fmaf(src[d], src[d], sum);
  const float inverse = rsqrtf(warp_sum(sum) / (float)value_dim + eps);
  const T* gate_row = gate + (size_t)(unit / heads) * ld_gate + (size_t)(unit % heads) * value_dim;
  for (int d = lane; d < value_dim; d += 32) {
    const float z = to_float(gate_row[d]);
    const float act = sigmoid_gate ? sigmoid(z) : silu(z);
    out[(size_t)unit * value_dim + d] = from_float<T>(src[d] * inverse * weight[d] * act);
  }
}

template <typename TB, typename TD, bool PER_CHANNEL>
int launch_scan(int per, dim3 grid, dim3 block, cudaStream_t stream, const float* qkv, const TB* beta, long long ld_beta,
                const TD* decay, long long ld_decay, const float* dt_bias, const float* a_log, float* state,
                const int* query_starts, const int* state_slots, const int* positions, float* out, int heads,
                int kv_heads, int key_dim, int value_dim) {
#define MIR_SCAN(P)                                                                                                  \
  case P:                                                                                                            \
    return mir_launch("delta_rule_scan", delta_rule_scan_kernel<TB, TD, P, PER_CHANNEL>, grid, block, 0, stream, 0, \
                      qkv, beta, ld_beta, decay, ld_decay, dt_bias, a_log, state, query_starts, state_slots,        \
                      positions, out, heads, kv_heads, key_dim, value_dim);
  switch (per) {
    MIR_SCAN(1) MIR_SCAN(2) MIR_SCAN(3) MIR_SCAN(4) MIR_SCAN(5) MIR_SCAN(6) MIR_SCAN(7) MIR_SCAN(8)
    default: break;
  }
#undef MIR_SCAN
  mir_set_error("delta_rule_scan: key_dim %d is larger than %d", key_dim, 32 * kMaxPerLane);
  return MIR_BAD_ARGUMENT;
}

}  // namespace

// x: first convolved channel of token 0 (q | k | v lie side by side in the packed projection); w [channels, taps]
// in the activations' type; tail [slots, taps - 1, channels] 32-bit; out [tokens, channels] 32-bit.
MIR_EXPORT int mir_short_conv_silu(int bf16, const void* x, long long ldx, const void* w, float* tail,
                                   const int* row_of_token, const int* query_starts, const int* state_slots,
                                   const int* positions, float* out, int tokens, int rows, int channels, int taps,
                                   cudaStream_t stream) {
  if (tokens == 0 || rows == 0) return MIR_OK;
  if (tokens < 0 || rows < 0 || channels <= 0 || taps < 1 || taps > kMaxTaps) {
    mir_set_error("short_conv_silu: bad sizes (tokens %d, rows %d, channels %d, taps %d; at most %d taps)", tokens, rows,
                  channels, taps, kMaxTaps);
    return MIR_BAD_ARGUMENT;
  }
  const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
  const dim3 grid(tokens, (channels + threads - 1) / threads), tail_grid(rows, (channels + threads - 1) / threads);
  int status;
  if (bf16)
    status = mir_launch("short_conv_silu", short_conv_silu_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, 0,
                        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const float*)tail, row_of_token,
                        query_starts, state_slots, positions, out, channels, taps);
  else
    status = mir_launch("short_conv_silu", short_conv_silu_kernel<float>, grid, dim3(threads), 0, stream, 0,
                        (const float*)x, ldx, (const float*)w, (const float*)tail, row_of_token, query_starts,
                        state_slots, positions, out, channels, taps);
  if (status != MIR_OK || taps == 1) return status;
  if (bf16)
    return mir_launch("short_conv_tail", short_conv_tail_kernel<__nv_bfloat16>, tail_grid, dim3(threads), 0, stream, 0,
                      (const __nv_bfloat16*)x, ldx, tail, query_starts, state_slots, positions, channels, taps);
  return mir_launch("short_conv_tail", short_conv_tail_kernel<float>, tail_grid, dim3(threads), 0, stream, 0,
                    (const float*)x, ldx, tail, query_starts, state_slots, positions, channels, taps);
}

// bf16: the type of beta_raw (and of decay_raw unless decay_f32).  per_channel: one decay per head and key channel.
MIR_EXPORT int mir_delta_rule_scan(int bf16, int decay_f32, int per_channel, const float* qkv, const void* beta_raw,
                                   long long ld_beta, const void* decay_raw, long long ld_decay, const float* dt_bias,
                                   const float* a_log, float* state, const int* query_starts, const int* state_slots,
                                   const int* positions, float* out, int rows, int heads, int kv_heads, int key_dim,
                                   int value_dim, cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || key_dim <= 0 || value_dim <= 0) {
    mir_set_error("delta_rule_scan: bad sizes (rows %d, heads %d, kv heads %d, key_dim %d, value_dim %d)", rows, heads,
                  kv_heads, key_dim, value_dim);
    return MIR_BAD_ARGUMENT;
  }
  const int per = (key_dim + 31) / 32;
  const int warps = value_dim >= 8 ? 8 : value_dim;
  const dim3 grid(rows, heads, (value_dim + warps - 1) / warps), block(32, warps);
#define MIR_ARGS dt_bias, a_log, state, query_starts, state_slots, positions, out, heads, kv_heads, key_dim, value_dim
  if (bf16) {
    const __nv_bfloat16* beta = (const __nv_bfloat16*)beta_raw;
    if (per_channel) {
      if (decay_f32) return launch_scan<__nv_bfloat16, float, true>(per, grid, block, stream, qkv, beta, ld_beta, (const float*)decay_raw, ld_decay, MIR_ARGS);
      return launch_scan<__nv_bfloat16, __nv_bfloat16, true>(per, grid, block, stream, qkv, beta, ld_beta, (const __nv_bfloat16*)decay_raw, ld_decay, MIR_ARGS);
    }
    if (decay_f32) return launch_scan<__nv_bfloat16, float, false>(per, grid, block, stream, qkv, beta, ld_beta, (const float*)decay_raw, ld_decay, MIR_ARGS);
    return launch_scan<__nv_bfloat16, __nv_bfloat16, false>(per, grid, block, stream, qkv, beta, ld_beta, (const __nv_bfloat16*)decay_raw, ld_decay, MIR_ARGS);
  }
  const float* beta = (const float*)beta_raw;
  if (per_channel) return launch_scan<float, float, true>(per, grid, block, stream, qkv, beta, ld_beta, (const float*)decay_raw, ld_decay, MIR_ARGS);
  return launch_scan<float, float, false>(per, grid, block, stream, qkv, beta, ld_beta, (const float*)decay_raw, ld_decay, MIR_ARGS);
#undef MIR_ARGS
}

// o [tokens, heads, value_dim] 32-bit; gate element (t, h, d) at gate[t * ld_gate + h * value_dim + d] and out
// [tokens, heads * value_dim] contiguous, both in the activations' type.
MIR_EXPORT int mir_gated_head_norm(int bf16, const float* o, const void* gate, long long ld_gate, const float* weight, void* out,
                                   int tokens, int heads, int value_dim, float eps, int sigmoid_gate,
                                   cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || value_dim <= 0) { mir_set_error("gated_head_norm: bad sizes"); return MIR_BAD_ARGUMENT; }
  const int units = tokens * heads;
  const dim3 grid((units + 3) / 4), block(32, 4);
  if (bf16)
    return mir_launch("gated_head_norm", gated_head_norm_kernel<__nv_bfloat16>, grid, block, 0, stream, 0, o,
                      (const __nv_bfloat16*)gate, ld_gate, weight, (__nv_bfloat16*)out, units, heads, value_dim, eps,
                      sigmoid_gate);
  return mir_launch("gated_head_norm", gated_head_norm_kernel<float>, grid, block, 0, stream, 0, o, (const float*)gate,
                    ld_gate, weight, (float*)out, units, heads, value_dim, eps, sigmoid_gate);
}
