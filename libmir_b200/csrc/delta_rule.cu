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
//   delta_rule_prepare the same convolution, then what else the recurrence needs of a token: q and k as unit vectors,
//                     sigmoid(beta), the decay; all tokens in parallel.
//   delta_rule_scan   the recurrence: a few lanes per (request, head, value channel) hold one column of S in
//                     registers, walk over the request's tokens of this step, and write the column back.  No shared
//                     memory, no block barrier: the two dot products per token are a few shuffles.  The state is
//                     stored [head][value channel][key channel], so a column is one contiguous run.
//   gated_head_norm   out = o / rms(o) * weight * act(gate) per (token, head), act = silu or sigmoid.
// A row of a captured decode batch whose position is negative is padding: nothing of it is read or written.
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kMaxTaps = 16;
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
                                       const int* __restrict__ positions, int channels, int taps, int skip_single) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int start = query_starts[row], count = query_starts[row + 1] - start;
  if (c >= channels || count <= 0 || positions[start] < 0 || (skip_single && count == 1)) return;
  float* mine = tail + (size_t)state_slots[row] * (taps - 1) * channels;
  float keep[kMaxTaps];
  for (int j = 0; j < taps - 1; ++j) {
    const int src = count - (taps - 1) + j;
    keep[j] = src >= 0 ? to_float(x[(size_t)(start + src) * ldx + c]) : mine[(size_t)(taps - 1 + src) * channels + c];
  }
  for (int j = 0; j < taps - 1; ++j) mine[(size_t)j * channels + c] = keep[j];
}

// Everything the recurrence needs of a token, in 32-bit, one CTA per token: the short convolution and silu of
// q | k | v (as short_conv_silu), q and k made unit vectors per key head (q also times key_dim^-1/2),
// beta = sigmoid(beta_raw), decay = exp(-exp(a_log) * softplus(decay_raw + dt_bias)).  A warp takes a key head at a
// time and keeps its channels in registers between the convolution and the norm; the rest is elementwise.
//   x          packed projection rows, convolved channel c of token t at x[t * ldx + c]; w [channels, taps]
//   beta_raw   (t, h) at beta_raw[t * ld_beta + h];  decay_raw (t, j) at decay_raw[t * ld_decay + j], j < decay_width
//   qkv        out [tokens, channels]; beta out [tokens, heads]; decay out [tokens, decay_width]
__device__ __forceinline__ float2 pair_of(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 pair_of(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// PAIRED: every thread works on two neighbouring channels (4- or 8-byte loads of the inputs); needs an even head
// width, an even number of value channels, an even row stride and a pointer aligned to two elements.
template <typename T, typename TD, bool PAIRED>
__global__ void delta_rule_prepare_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w,
                                          float* __restrict__ tail, const T* __restrict__ beta_raw,
                                          long long ld_beta, const TD* __restrict__ decay_raw, long long ld_decay,
                                          const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                          const int* __restrict__ row_of_token, const int* __restrict__ query_starts,
                                          const int* __restrict__ state_slots, const int* __restrict__ positions,
                                          float* __restrict__ qkv, float* __restrict__ beta, float* __restrict__ decay,
                                          int heads, int kv_heads, int key_dim, int value_dim, int decay_width,
                                          int taps) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  if (positions[token] < 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int row = row_of_token[token];
  const int start = query_starts[row];
  const int local = token - start;
  const int channels = 2 * kv_heads * key_dim + heads * value_dim;
  float* old = tail + (size_t)state_slots[row] * (taps - 1) * channels;
  float* out = qkv + (size_t)token * channels;
  // A request that brings one token moves its tail on right here: a channel's tail is read by the one thread that
  // convolves the channel, which then shifts it and appends the token's input (short_conv_tail skips such rows).
  const bool alone = query_starts[row + 1] - start == 1;
  auto convolved = [&](int c) {
    float acc = 0.0f;
    for (int j = 0; j < taps; ++j) {
      const int src = local - (taps - 1) + j;
      const float value = src >= 0 ? to_float(x[(size_t)(start + src) * ldx + c])
                                   : old[(size_t)(taps - 1 + src) * channels + c];
      acc = fmaf(to_float(w[(size_t)c * taps + j]), value, acc);
    }
    if (alone) {
      for (int j = 0; j + 2 < taps; ++j) old[(size_t)j * channels + c] = old[(size_t)(j + 1) * channels + c];
      if (taps > 1) old[(size_t)(taps - 2) * channels + c] = to_float(x[(size_t)token * ldx + c]);
    }
    return silu(acc);
  };
  // q heads, then k heads: unit vectors
  const float q_scale = rsqrtf((float)key_dim);
  // the CTAs of a token (gridDim.y of them, more where a step has few tokens) share its heads and channels out
  const int part = blockIdx.y, parts = gridDim.y;
  const int index = part * blockDim.x + threadIdx.x, stride = parts * blockDim.x;
  auto convolved_pair = [&](int c) {                           // channels c and c + 1, c even
    float first = 0.0f, second = 0.0f;
    for (int j = 0; j < taps; ++j) {
      const int src = local - (taps - 1) + j;
      const float2 value = src >= 0 ? pair_of(x + (size_t)(start + src) * ldx + c)
                                    : pair_of(old + (size_t)(taps - 1 + src) * channels + c);
      first = fmaf(to_float(w[(size_t)c * taps + j]), value.x, first);
      second = fmaf(to_float(w[(size_t)(c + 1) * taps + j]), value.y, second);
    }
    if (alone) {
      for (int j = 0; j + 2 < taps; ++j)
        *reinterpret_cast<float2*>(old + (size_t)j * channels + c) = pair_of(old + (size_t)(j + 1) * channels + c);
      if (taps > 1) *reinterpret_cast<float2*>(old + (size_t)(taps - 2) * channels + c) = pair_of(x + (size_t)token * ldx + c);
    }
    return make_float2(silu(first), silu(second));
  };
  for (int unit = part * warps + warp; unit < 2 * kv_heads; unit += parts * warps) {
    float values[kMaxPerLane];
    float square = 0.0f;
    if (PAIRED) {
#pragma unroll
      for (int m = 0; m < kMaxPerLane; m += 2) {
        const int i = 2 * lane + 32 * m;
        const float2 both = i < key_dim ? convolved_pair(unit * key_dim + i) : make_float2(0.0f, 0.0f);
        values[m] = both.x;
        values[m + 1] = both.y;
        square = fmaf(both.x, both.x, fmaf(both.y, both.y, square));
      }
    } else {
#pragma unroll
      for (int m = 0; m < kMaxPerLane; ++m) {
        const int i = lane + 32 * m;
        values[m] = i < key_dim ? convolved(unit * key_dim + i) : 0.0f;
        square = fmaf(values[m], values[m], square);
      }
    }
    const float unit_scale = rsqrtf(warp_sum(square) + 1e-6f) * (unit < kv_heads ? q_scale : 1.0f);
    if (PAIRED) {
#pragma unroll
      for (int m = 0; m < kMaxPerLane; m += 2) {
        const int i = 2 * lane + 32 * m;
        if (i < key_dim)
          *reinterpret_cast<float2*>(out + unit * key_dim + i) = make_float2(values[m] * unit_scale, values[m + 1] * unit_scale);
      }
    } else {
#pragma unroll
      for (int m = 0; m < kMaxPerLane; ++m) {
        const int i = lane + 32 * m;
        if (i < key_dim) out[unit * key_dim + i] = values[m] * unit_scale;
      }
    }
  }
  if (PAIRED) {
    for (int c = 2 * kv_heads * key_dim + 2 * index; c < channels; c += 2 * stride)
      *reinterpret_cast<float2*>(out + c) = convolved_pair(c);
  } else {
    for (int c = 2 * kv_heads * key_dim + index; c < channels; c += stride) out[c] = convolved(c);
  }
  for (int h = index; h < heads; h += stride)
    beta[(size_t)token * heads + h] = sigmoid(to_float(beta_raw[(size_t)token * ld_beta + h]));
  const int per_head = decay_width / heads;
  for (int j = index; j < decay_width; j += stride)
    decay[(size_t)token * decay_width + j] =
        expf(-expf(a_log[j / per_head]) * softplus(to_float(decay_raw[(size_t)token * ld_decay + j]) + dt_bias[j]));
}

__device__ __forceinline__ void copy_async(float* dst, const float* src, bool wide) {
  const unsigned target = (unsigned)__cvta_generic_to_shared(dst);
  if (wide) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(target), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(target), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kScanWarps = 4;
constexpr int kScanChunk = 16;          // tokens whose inputs one stage of shared memory holds

// The recurrence.  LANES lanes share one column of S (one value channel of one head): lane l holds the key channels
// 4 (m LANES + l) .. + 3 for m < PER / 4 in registers, so a warp works on 32 / LANES columns at once, the two dot
// products per token are log2(LANES) shuffle steps, and the state of a column (stored [head][value channel][key
// channel]) is read and written in 16-byte pieces that lie side by side across the lanes.  The inputs of a token are
// the same for every column of its head: the CTA (all its warps work on columns of one head) copies them for 16
// tokens at a time into shared memory with cp.async, two stages, so that the walk over the tokens never waits for
// global memory.  blockDim (32, kScanWarps), grid (rows, heads, ceil(value_dim / (kScanWarps * 32 / LANES))).
//   qkv    [tokens, 2 G D + H V] 32-bit: unit q | unit k | v (delta_rule_prepare)
//   beta   [tokens, H]; decay [tokens, H D] (PER_CHANNEL) or [tokens, H]
//   state  [slots, H, V, D] 32-bit;  out [tokens, H V] 32-bit: o before the head norm
template <int LANES, int PER, bool PER_CHANNEL>
__global__ void __launch_bounds__(kScanWarps * 32)
delta_rule_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                       float* __restrict__ state, const int* __restrict__ query_starts,
                       const int* __restrict__ state_slots, const int* __restrict__ positions,
                       float* __restrict__ out, int heads, int kv_heads, int key_dim, int value_dim) {
  static_assert(PER % 4 == 0, "a lane holds whole 16-byte pieces");
  extern __shared__ __align__(16) float staged[];              // [2 stages][kScanChunk tokens][row]
  grid_launch_dependents();
  grid_dependency_wait();
  constexpr int COLUMNS = 32 / LANES;                           // per warp
  constexpr int BLOCK_COLUMNS = COLUMNS * kScanWarps;
  constexpr int PADDED = LANES * PER;                           // key channels with padding
  constexpr int DECAYS = PER_CHANNEL ? PADDED : 4;
  constexpr int ROW = 2 * PADDED + DECAYS + 4 + BLOCK_COLUMNS;  // q | k | decay | beta | v of this CTA's columns
  const int thread = threadIdx.y * 32 + threadIdx.x;
  const int l = threadIdx.x % LANES;
  const int row = blockIdx.x, head = blockIdx.y;
  const int first_column = blockIdx.z * BLOCK_COLUMNS;
  const int local_column = threadIdx.y * COLUMNS + threadIdx.x / LANES;
  const int column = first_column + local_column;
  const int start = query_starts[row], end = query_starts[row + 1];
  if (end <= start || positions[start] < 0) return;             // the whole CTA: an empty or padding row
  const bool active = column < value_dim;                        // idle lanes still take part in the shuffles
  const int kv_head = head / (heads / kv_heads);
  const int width = 2 * kv_heads * key_dim + heads * value_dim;
  const int g_width = PER_CHANNEL ? heads * key_dim : heads;
  // 16-byte accesses: every piece lies wholly inside or outside the head, and every row starts on a 16-byte boundary
  const bool wide = (key_dim % 4 == 0) && (width % 4 == 0);
  float* column_state = state + (((size_t)state_slots[row] * heads + head) * value_dim + (active ? column : 0)) * key_dim;

  // one stage: the inputs of tokens [from, from + kScanChunk) of this request, zero where a head is narrower than PADDED
  auto stage_in = [&](int from, float* dst) {
    const int count = min(kScanChunk, end - from);
    const int pieces = wide ? 4 : 1;
    const int per_row = (2 * key_dim + (PER_CHANNEL ? key_dim : 0)) / pieces;
    for (int index = thread; index < count * per_row; index += kScanWarps * 32) {
      const int t = index / per_row, e = (index - t * per_row) * pieces;
      const int which = e / key_dim, i = e - which * key_dim;    // 0 q, 1 k, 2 decay
      const float* src = which == 2 ? decay + (size_t)(from + t) * g_width + (size_t)head * key_dim + i
                                    : qkv + (size_t)(from + t) * width + (size_t)(which * kv_heads + kv_head) * key_dim + i;
      copy_async(dst + t * ROW + which * PADDED + i, src, wide);
    }
    for (int index = thread; index < count * (BLOCK_COLUMNS + 2); index += kScanWarps * 32) {
      const int t = index / (BLOCK_COLUMNS + 2), e = index - t * (BLOCK_COLUMNS + 2);
      float* target = dst + t * ROW + 2 * PADDED + DECAYS;
      if (e == 0) copy_async(target, beta + (size_t)(from + t) * heads + head, false);
      else if (e == 1) { if (!PER_CHANNEL) copy_async(target - DECAYS, decay + (size_t)(from + t) * g_width + head, false); }
      else if (first_column + e - 2 < value_dim)
        copy_async(target + 4 + e - 2, qkv + (size_t)(from + t) * width + (size_t)2 * kv_heads * key_dim +
                                           (size_t)head * value_dim + first_column + e - 2, false);
    }
  };
  // padding channels (key_dim < PADDED) are read as q = k = 0: zero them once in both stages
  if (key_dim < PADDED)
    for (int index = thread; index < 2 * kScanChunk * ROW; index += kScanWarps * 32) staged[index] = 0.0f;
  __syncthreads();

  float s[PER];
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * LANES + l) * 4;
    if (wide) {
      const float4 piece = (active && i < key_dim) ? *reinterpret_cast<const float4*>(column_state + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s[m] = piece.x; s[m + 1] = piece.y; s[m + 2] = piece.z; s[m + 3] = piece.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[m + e] = (active && i + e < key_dim) ? column_state[i + e] : 0.0f;
    }
  }

  stage_in(start, staged);
  copy_commit();
  int stage = 0;
  float pending = 0.0f;                                          // the last token's read-out, not yet summed over the lanes
  bool has_pending = false;
  __shared__ __align__(16) float exchange[kScanWarps][2][64];   // [warp][token parity][S^T k parts | read-out parts]
  int parity = 0;
  auto sum_over_lanes = [&](float& first, float& second) {       // both sums in one fixed order, whichever token it is
    float* parts = exchange[threadIdx.y][parity];
    parts[threadIdx.x] = first;
    parts[32 + threadIdx.x] = second;
    __syncwarp();
    const float* mine = parts + (threadIdx.x / LANES) * LANES;
    float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
    for (int piece = 0; piece < LANES; piece += 4) {
      const float4 a = *reinterpret_cast<const float4*>(mine + piece);
      const float4 b = *reinterpret_cast<const float4*>(mine + 32 + piece);
      sum_a += (a.x + a.y) + (a.z + a.w);
      sum_b += (b.x + b.y) + (b.z + b.w);
    }
    first = sum_a;
    second = sum_b;
    parity ^= 1;
  };
  const bool writer = l == 0 && active;
  const size_t out_step = (size_t)heads * value_dim;
  float* out_at = out + ((size_t)start * heads + head) * value_dim + (active ? column : 0) - out_step;   // the pending token's place
  for (int from = start; from < end; from += kScanChunk, stage ^= 1) {
    if (from + kScanChunk < end) stage_in(from + kScanChunk, staged + (stage ^ 1) * kScanChunk * ROW);
    copy_commit();
    copy_wait<1>();
    __syncthreads();
    const int count = min(kScanChunk, end - from);
    const float* in = staged + stage * kScanChunk * ROW - ROW;
#pragma unroll 2
    for (int t = 0; t < count; ++t) {
      in += ROW;
      const float b = in[2 * PADDED + DECAYS];
      const float v = in[2 * PADDED + DECAYS + 4 + local_column];
      const float head_decay = in[2 * PADDED];
      float k[PER];
      float seen[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int m = 0; m < PER; m += 4) {
        const int i = (m / 4 * LANES + l) * 4;
        const float4 key = *reinterpret_cast<const float4*>(in + PADDED + i);
        float4 g = make_float4(head_decay, head_decay, head_decay, head_decay);
        if (PER_CHANNEL) g = *reinterpret_cast<const float4*>(in + 2 * PADDED + i);
        k[m] = key.x; k[m + 1] = key.y; k[m + 2] = key.z; k[m + 3] = key.w;
        s[m] *= g.x; s[m + 1] *= g.y; s[m + 2] *= g.z; s[m + 3] *= g.w;
        seen[0] = fmaf(s[m], key.x, seen[0]);
        seen[1] = fmaf(s[m + 1], key.y, seen[1]);
        seen[2] = fmaf(s[m + 2], key.z, seen[2]);
        seen[3] = fmaf(s[m + 3], key.w, seen[3]);
      }
      float total = (seen[0] + seen[1]) + (seen[2] + seen[3]);
      // Two sums over the lanes of a column at once: this token's S^T k and the token before's read-out, which is not
      // on the path to the next state.  The lanes exchange their parts through shared memory (a store, a warp barrier
      // and 16-byte loads that every lane of the column adds up in the same order) rather than by shuffles: a chain
      // of log2(LANES) dependent shuffles costs this lone warp more than the round trip.  Two buffers by the
      // token's parity: a lane may still read one while the next token's parts are written.
      sum_over_lanes(total, pending);
      if (has_pending && writer) *out_at = pending;
      out_at += out_step;
      const float update = b * (v - total);
      float read[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int m = 0; m < PER; m += 4) {
        const int i = (m / 4 * LANES + l) * 4;
        const float4 query = *reinterpret_cast<const float4*>(in + i);
        s[m] = fmaf(k[m], update, s[m]);
        s[m + 1] = fmaf(k[m + 1], update, s[m + 1]);
        s[m + 2] = fmaf(k[m + 2], update, s[m + 2]);
        s[m + 3] = fmaf(k[m + 3], update, s[m + 3]);
        read[0] = fmaf(s[m], query.x, read[0]);
        read[1] = fmaf(s[m + 1], query.y, read[1]);
        read[2] = fmaf(s[m + 2], query.z, read[2]);
        read[3] = fmaf(s[m + 3], query.w, read[3]);
      }
      pending = (read[0] + read[1]) + (read[2] + read[3]);
      has_pending = true;
    }
    __syncthreads();                                              // the stage is free for the chunk after next
  }
  copy_wait<0>();
  {
    float unused = 0.0f;
    sum_over_lanes(unused, pending);                             // the last token's read-out
  }
  if (!active) return;
  if (l == 0) *out_at = pending;
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * LANES + l) * 4;
    if (wide) {
      if (i < key_dim) *reinterpret_cast<float4*>(column_state + i) = make_float4(s[m], s[m + 1], s[m + 2], s[m + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i + e < key_dim) column_state[i + e] = s[m + e];
    }
  }
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) * weight * act(gate); the weight is [value_dim], the
// same for every head, or (weight_per_head) [heads, value_dim].
template <typename T, typename TG>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const TG* __restrict__ gate, long long ld_gate,
                                       const float* __restrict__ weight, T* __restrict__ out, int units,
                                       int heads, int value_dim, float eps, int sigmoid_gate, int weight_per_head) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int unit = blockIdx.x * blockDim.y + threadIdx.y;       // token * heads + head
  if (unit >= units) return;
  const int lane = threadIdx.x;
  const float* src = o + (size_t)unit * value_dim;
  float sum = 0.0f;
  for (int d = lane; d < value_dim; d += 32) sum = fmaf(src[d], src[d], sum);
  const float inverse = rsqrtf(warp_sum(sum) / (float)value_dim + eps);
  const TG* gate_row = gate + (size_t)(unit / heads) * ld_gate + (size_t)(unit % heads) * value_dim;
  const float* scale = weight + (weight_per_head ? (size_t)(unit % heads) * value_dim : 0);
  for (int d = lane; d < value_dim; d += 32) {
    const float z = to_float(gate_row[d]);
    const float act = sigmoid_gate ? sigmoid(z) : silu(z);
    out[(size_t)unit * value_dim + d] = from_float<T>(src[d] * inverse * scale[d] * act);
  }
}

// How many lanes share a column of the state: 0 lets the launcher choose, 8 / 16 / 32 fix it (for measurements).
int g_scan_lanes = 0;

template <int LANES, int PER, bool PER_CHANNEL>
int launch_scan_as(cudaStream_t stream, const float* qkv, const float* beta, const float* decay, float* state,
                   const int* query_starts, const int* state_slots, const int* positions, float* out, int rows,
                   int heads, int kv_heads, int key_dim, int value_dim) {
  constexpr int columns = kScanWarps * (32 / LANES);
  constexpr int padded = LANES * PER;
  constexpr int row = 2 * padded + (PER_CHANNEL ? padded : 4) + 4 + columns;
  constexpr size_t smem = (size_t)2 * kScanChunk * row * sizeof(float);
  static bool raised = false;                                    // more than 48 KB of shared memory needs the opt-in
  if (smem > 48 * 1024 && !raised) {
    const cudaError_t err = cudaFuncSetAttribute(delta_rule_scan_kernel<LANES, PER, PER_CHANNEL>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mir_set_error("delta_rule_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    raised = true;
  }
  return mir_launch("delta_rule_scan", delta_rule_scan_kernel<LANES, PER, PER_CHANNEL>,
                    dim3(rows, heads, (value_dim + columns - 1) / columns), dim3(32, kScanWarps), smem, stream, 0, qkv,
                    beta, decay, state, query_starts, state_slots, positions, out, heads, kv_heads, key_dim, value_dim);
}

template <bool PER_CHANNEL>
int launch_scan(cudaStream_t stream, const float* qkv, const float* beta, const float* decay, float* state,
                const int* query_starts, const int* state_slots, const int* positions, float* out, int rows, int heads,
                int kv_heads, int key_dim, int value_dim, bool single_tokens) {
#define MIR_SCAN(L, P)                                                                                              \
  return launch_scan_as<L, P, PER_CHANNEL>(stream, qkv, beta, decay, state, query_starts, state_slots, positions, \
                                           out, rows, heads, kv_heads, key_dim, value_dim);
  // 0: chosen here.  Measured at 16 heads of 128 x 128: a prompt of 2,048 tokens takes 766 / 796 / 935 us with 8 / 16 /
  // 32 lanes a column; a step of eight single tokens inside a captured graph 8.1 us with 8 lanes, 10.5 with 16.  One
  // choice for every shape of step, so that a request's 32-bit results do not depend on how it was cut.
  (void)single_tokens;
  const int lanes = g_scan_lanes ? g_scan_lanes : 8;
  if (lanes == 8) {
    if (key_dim <= 32) { MIR_SCAN(8, 4) }
    if (key_dim <= 64) { MIR_SCAN(8, 8) }
    if (key_dim <= 96) { MIR_SCAN(8, 12) }
    if (key_dim <= 128) { MIR_SCAN(8, 16) }
  }
  if (lanes == 16) {
    if (key_dim <= 64) { MIR_SCAN(16, 4) }
    if (key_dim <= 128) { MIR_SCAN(16, 8) }
  }
  if (key_dim <= 128) { MIR_SCAN(32, 4) }
  if (key_dim <= 256) { MIR_SCAN(32, 8) }
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
                      (const __nv_bfloat16*)x, ldx, tail, query_starts, state_slots, positions, channels, taps, 0);
  return mir_launch("short_conv_tail", short_conv_tail_kernel<float>, tail_grid, dim3(threads), 0, stream, 0,
                    (const float*)x, ldx, tail, query_starts, state_slots, positions, channels, taps, 0);
}

// bf16: the type of x, w and beta_raw (and of decay_raw unless decay_f32).  decay_width: heads, or heads * key_dim for
// one decay per key channel.  Writes qkv [tokens, channels], beta [tokens, heads], decay [tokens, decay_width] (32-bit)
// and moves the convolution's tail [slots, taps - 1, channels] on.
MIR_EXPORT int mir_delta_rule_prepare(int bf16, int decay_f32, const void* x, long long ldx, const void* w, float* tail,
                                      const void* beta_raw, long long ld_beta, const void* decay_raw, long long ld_decay,
                                      const float* dt_bias, const float* a_log, const int* row_of_token,
                                      const int* query_starts, const int* state_slots, const int* positions, float* qkv,
                                      float* beta, float* decay, int tokens, int rows, int heads, int kv_heads,
                                      int key_dim, int value_dim, int decay_width, int taps, cudaStream_t stream) {
  if (tokens == 0 || rows == 0) return MIR_OK;
  if (tokens < 0 || rows < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || key_dim <= 0 ||
      key_dim > 32 * kMaxPerLane || value_dim <= 0 || taps < 1 || taps > kMaxTaps ||
      (decay_width != heads && decay_width != heads * key_dim)) {
    mir_set_error("delta_rule_prepare: bad sizes (heads %d, kv heads %d, key_dim %d up to %d, value_dim %d, taps %d up "
                  "to %d, decay width %d)", heads, kv_heads, key_dim, 32 * kMaxPerLane, value_dim, taps, kMaxTaps,
                  decay_width);
    return MIR_BAD_ARGUMENT;
  }
  const int channels = 2 * kv_heads * key_dim + heads * value_dim;
  // one CTA per token where the step has many; with few tokens each token's work is shared out over several CTAs
  const int most = (2 * kv_heads + 7) / 8 > (channels + 255) / 256 ? (2 * kv_heads + 7) / 8 : (channels + 255) / 256;
  int parts = (2 * mir_sm_count() + tokens - 1) / tokens;
  parts = parts < 1 ? 1 : (parts > most ? most : parts);
  int status;
  const size_t element = bf16 ? 2 : 4;
  const bool paired = key_dim % 2 == 0 && (heads * value_dim) % 2 == 0 && ldx % 2 == 0 &&
                      (uintptr_t)x % (2 * element) == 0 && (uintptr_t)qkv % 8 == 0 && (uintptr_t)tail % 8 == 0;
#define MIR_PREPARE_AS(T, TD, P)                                                                                       \
  status = mir_launch("delta_rule_prepare", delta_rule_prepare_kernel<T, TD, P>, dim3(tokens, parts), dim3(256), 0,    \
                      stream, 0, (const T*)x, ldx, (const T*)w, tail, (const T*)beta_raw, ld_beta,       \
                      (const TD*)decay_raw, ld_decay, dt_bias, a_log, row_of_token, query_starts, state_slots,         \
                      positions, qkv, beta, decay, heads, kv_heads, key_dim, value_dim, decay_width, taps)
#define MIR_PREPARE(T, TD)                                                                                             \
  do {                                                                                                                 \
    if (paired) MIR_PREPARE_AS(T, TD, true);                                                                           \
    else MIR_PREPARE_AS(T, TD, false);                                                                                 \
  } while (0)
  if (bf16 && decay_f32) MIR_PREPARE(__nv_bfloat16, float);
  else if (bf16) MIR_PREPARE(__nv_bfloat16, __nv_bfloat16);
  else MIR_PREPARE(float, float);
#undef MIR_PREPARE
#undef MIR_PREPARE_AS
  // rows of one token have moved their tails on themselves; a step of single tokens needs nothing more
  if (status != MIR_OK || taps == 1 || tokens == rows) return status;
  const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
  const dim3 tail_grid(rows, (channels + threads - 1) / threads);
  if (bf16)
    return mir_launch("short_conv_tail", short_conv_tail_kernel<__nv_bfloat16>, tail_grid, dim3(threads), 0, stream, 0,
                      (const __nv_bfloat16*)x, ldx, tail, query_starts, state_slots, positions, channels, taps, 1);
  return mir_launch("short_conv_tail", short_conv_tail_kernel<float>, tail_grid, dim3(threads), 0, stream, 0,
                    (const float*)x, ldx, tail, query_starts, state_slots, positions, channels, taps, 1);
}

MIR_EXPORT int mir_delta_rule_set_lanes(int lanes) {
  if (lanes != 0 && lanes != 8 && lanes != 16 && lanes != 32) { mir_set_error("delta_rule: lanes are 0, 8, 16 or 32"); return MIR_BAD_ARGUMENT; }
  g_scan_lanes = lanes;
  return MIR_OK;
}

// qkv, beta, decay as delta_rule_prepare leaves them; per_channel: decay is [tokens, heads * key_dim].
MIR_EXPORT int mir_delta_rule_scan(int per_channel, const float* qkv, const float* beta, const float* decay, float* state,
                                   const int* query_starts, const int* state_slots, const int* positions, float* out,
                                   int tokens, int rows, int heads, int kv_heads, int key_dim, int value_dim,
                                   cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || key_dim <= 0 || value_dim <= 0) {
    mir_set_error("delta_rule_scan: bad sizes (rows %d, heads %d, kv heads %d, key_dim %d, value_dim %d)", rows, heads,
                  kv_heads, key_dim, value_dim);
    return MIR_BAD_ARGUMENT;
  }
  if (per_channel)
    return launch_scan<true>(stream, qkv, beta, decay, state, query_starts, state_slots, positions, out, rows, heads,
                             kv_heads, key_dim, value_dim, tokens == rows);
  return launch_scan<false>(stream, qkv, beta, decay, state, query_starts, state_slots, positions, out, rows, heads,
                            kv_heads, key_dim, value_dim, tokens == rows);
}

// o [tokens, heads, value_dim] 32-bit; gate element (t, h, d) at gate[t * ld_gate + h * value_dim + d], in the
// activations' type or (gate_f32) in 32-bit; out [tokens, heads * value_dim] contiguous in the activations' type.
MIR_EXPORT int mir_gated_head_norm(int bf16, int gate_f32, const float* o, const void* gate, long long ld_gate,
                                   const float* weight, void* out, int tokens, int heads, int value_dim, float eps,
                                   int sigmoid_gate, int weight_per_head, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || value_dim <= 0) { mir_set_error("gated_head_norm: bad sizes"); return MIR_BAD_ARGUMENT; }
  const int units = tokens * heads;
  const dim3 grid((units + 3) / 4), block(32, 4);
  if (bf16 && gate_f32)
    return mir_launch("gated_head_norm", gated_head_norm_kernel<__nv_bfloat16, float>, grid, block, 0, stream, 0, o,
                      (const float*)gate, ld_gate, weight, (__nv_bfloat16*)out, units, heads, value_dim, eps, sigmoid_gate,
                      weight_per_head);
  if (bf16)
    return mir_launch("gated_head_norm", gated_head_norm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, 0, o,
                      (const __nv_bfloat16*)gate, ld_gate, weight, (__nv_bfloat16*)out, units, heads, value_dim, eps,
                      sigmoid_gate, weight_per_head);
  return mir_launch("gated_head_norm", gated_head_norm_kernel<float, float>, grid, block, 0, stream, 0, o, (const float*)gate,
                    ld_gate, weight, (float*)out, units, heads, value_dim, eps, sigmoid_gate, weight_per_head);
}
