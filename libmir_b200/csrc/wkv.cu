// Kernels of the wkv mixer: time mixing with a matrix state per head, a decay per head and key channel, and a bonus for
// the current token.
//
//   wkv_mix    the five inputs of the projections: mix_s[t] = h[t] + (h[t - 1] - h[t]) * mu_s, with h[t - 1] of a
//              portion's first token taken from the request's state (zeros at its start); a request that brings one
//              token moves its state on in the same kernel, the others in wkv_tail
//   wkv_scan   per head, with S [key channel, value channel] (stored per value channel, a column contiguous):
//                o_t = S^T r_t + (sum_i r_i u_i k_i) v_t;   S <- diag(w_t) S + k_t v_t^T;   w_t = exp(-exp(z_t + w0))
// The decays, the state and every sum are 32-bit; T is the storage type of the projections' results.
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kMixes = 5;

template <typename T>
__global__ void wkv_mix_kernel(const T* __restrict__ h, long long ld, float* __restrict__ tail,
                               const float* __restrict__ mu, const int* __restrict__ row_of_token,
                               const int* __restrict__ query_starts, const int* __restrict__ state_slots,
                               const int* __restrict__ positions, T* __restrict__ out, int tokens, int width) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  if (positions[token] < 0) return;                              // a padding row of a captured batch
  const int row = row_of_token[token];
  const int start = query_starts[row], end = query_starts[row + 1];
  const T* mine = h + (size_t)token * ld;
  const T* before = token > start ? h + (size_t)(token - 1) * ld : nullptr;
  float* kept = tail + (size_t)state_slots[row] * width;
  const bool alone = end - start == 1;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_float(mine[c]);
    const float previous = before != nullptr ? to_float(before[c]) : kept[c];
    const float step = previous - x;
#pragma unroll
    for (int s = 0; s < kMixes; ++s)
      out[((size_t)s * tokens + token) * width + c] = from_float<T>(fmaf(step, mu[(size_t)s * width + c], x));
    if (alone) kept[c] = x;
  }
}

// The state's last input of every request that brought more than one token.
template <typename T>
__global__ void wkv_tail_kernel(const T* __restrict__ h, long long ld, float* __restrict__ tail,
                                const int* __restrict__ query_starts, const int* __restrict__ state_slots,
                                const int* __restrict__ positions, int width) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int start = query_starts[row], end = query_starts[row + 1];
  if (end - start < 2 || positions[start] < 0) return;
  const T* last = h + (size_t)(end - 1) * ld;
  float* kept = tail + (size_t)state_slots[row] * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) kept[c] = to_float(last[c]);
}

constexpr int kScanWarps = 4;
constexpr int kScanChunkNarrow = 32;                              // tokens staged at a time: heads up to 64 wide,
constexpr int kScanChunkWide = 16;                                // up to 128 wide,
constexpr int kScanChunkWidest = 8;                               // and wider ones (the stage stays under 48 KB)
constexpr int kLanes = 8;                                        // lanes that share one column of the state

// blockDim (32, kScanWarps), grid (rows, heads, ceil(dim / (kScanWarps * 4))).  Lane l of a column holds the key
// channels 4 (m kLanes + l) .. + 3, m < PER / 4.  The inputs of kScanChunk tokens at a time are staged in shared
// memory (every column of a head reads the same r, k and decay); the read-out's sum over the lanes is no part of the
// chain from state to state.  One lane count and one order of sums for every shape of step.
template <typename T, int PER, bool SHORT>
__global__ void __launch_bounds__(kScanWarps * 32)
wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                const float* __restrict__ decay_raw, const float* __restrict__ decay_bias, const float* __restrict__ bonus,
                float* __restrict__ state, const int* __restrict__ query_starts, const int* __restrict__ state_slots,
                const int* __restrict__ positions, float* __restrict__ out, int heads, int dim) {
  constexpr int COLUMNS = 32 / kLanes;
  constexpr int BLOCK_COLUMNS = COLUMNS * kScanWarps;
  constexpr int PADDED = kLanes * PER;
  constexpr int ROW = 3 * PADDED + 4 + BLOCK_COLUMNS;            // r | k | decay | bonus term | v of this CTA's columns
  // SHORT: a step of single tokens stages one token a warp: few registers, so that all its CTAs are resident at once
  constexpr int kScanChunk = SHORT ? kScanWarps : (PER <= 8 ? kScanChunkNarrow : (PER <= 16 ? kScanChunkWide : kScanChunkWidest));
  __shared__ __align__(16) float staged[kScanChunk * ROW];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x, warp = threadIdx.y;
  const int thread = warp * 32 + lane;
  const int l = lane % kLanes;
  const int row = blockIdx.x, head = blockIdx.y;
  const int first_column = blockIdx.z * BLOCK_COLUMNS;
  const int local_column = warp * COLUMNS + lane / kLanes;
  const int column = first_column + local_column;
  const int start = query_starts[row], end = query_starts[row + 1];
  if (end <= start || positions[start] < 0) return;             // the whole CTA: an empty or padding row
  const bool active = column < dim;
  const int width = heads * dim;
  const bool wide = dim % 4 == 0;
  float* column_state = state + (((size_t)state_slots[row] * heads + head) * dim + (active ? column : 0)) * dim;

  float s[PER];
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * kLanes + l) * 4;
    if (wide) {
      const float4 piece = (active && i < dim) ? *reinterpret_cast<const float4*>(column_state + i)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
      s[m] = piece.x; s[m + 1] = piece.y; s[m + 2] = piece.z; s[m + 3] = piece.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[m + e] = (active && i + e < dim) ? column_state[i + e] : 0.0f;
    }
  }
  const size_t head_at = (size_t)head * dim;
  // What the next chunk needs is fetched into registers before the walk over the current chunk starts and goes to
  // shared memory after it, so that the walk never waits for global memory.  A warp stages whole tokens: r, k and
  // the decay exp(-exp(z + w0)) of every channel, and the token's bonus term sum_i r_i u_i k_i, which is the same for
  // every column of the head.
  constexpr int TOKENS_PER_WARP = kScanChunk / kScanWarps;
  constexpr int PER_LANE = PADDED / 32;
  constexpr int VALUES_PER_THREAD = (kScanChunk * BLOCK_COLUMNS + kScanWarps * 32 - 1) / (kScanWarps * 32);
  float next_r[TOKENS_PER_WARP][PER_LANE], next_k[TOKENS_PER_WARP][PER_LANE], next_w[TOKENS_PER_WARP][PER_LANE];
  float next_v[VALUES_PER_THREAD];
  auto fetch = [&](int from) {
    const int count = min(kScanChunk, end - from);
#pragma unroll
    for (int tt = 0; tt < TOKENS_PER_WARP; ++tt) {
      const int t = warp + tt * kScanWarps;
#pragma unroll
      for (int e = 0; e < PER_LANE; ++e) {
        const int i = lane + 32 * e;
        next_r[tt][e] = 0.0f; next_k[tt][e] = 0.0f; next_w[tt][e] = 0.0f;
        if (t < count && i < dim) {
          const size_t source = (size_t)(from + t) * ld + head_at + i;
          next_r[tt][e] = to_float(r[source]);
          next_k[tt][e] = to_float(k[source]);
          next_w[tt][e] = decay_raw[(size_t)(from + t) * width + head_at + i];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VALUES_PER_THREAD; ++j) {
      const int index = thread + j * kScanWarps * 32;
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      next_v[j] = (t < count && first_column + c < dim) ? to_float(v[(size_t)(from + t) * ld + head_at + first_column + c]) : 0.0f;
      // (t may lie beyond the chunk where the chunk has fewer values than the CTA has threads: commit skips those)
    }
  };
  auto commit = [&](int from) {
    const int count = min(kScanChunk, end - from);
#pragma unroll
    for (int tt = 0; tt < TOKENS_PER_WARP; ++tt) {
      const int t = warp + tt * kScanWarps;
      if (t >= count) continue;                                  // (the same for the whole warp)
      float* at = staged + t * ROW;
      float sum = 0.0f;
#pragma unroll
      for (int e = 0; e < PER_LANE; ++e) {
        const int i = lane + 32 * e;
        float ww = 0.0f;
        if (i < dim) {
          ww = expf(-expf(next_w[tt][e] + decay_bias[head_at + i]));
          sum = fmaf(next_r[tt][e] * bonus[head_at + i], next_k[tt][e], sum);
        }
        at[i] = next_r[tt][e]; at[PADDED + i] = next_k[tt][e]; at[2 * PADDED + i] = ww;
      }
      sum = warp_sum(sum);
      if (lane == 0) at[3 * PADDED] = sum;
    }
#pragma unroll
    for (int j = 0; j < VALUES_PER_THREAD; ++j) {
      const int index = thread + j * kScanWarps * 32;
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      if (t < kScanChunk) staged[t * ROW + 3 * PADDED + 4 + c] = next_v[j];
    }
  };
  fetch(start);
  for (int from = start; from < end; from += kScanChunk) {
    const int count = min(kScanChunk, end - from);
    __syncthreads();                                             // the chunk before has been read
    commit(from);
    __syncthreads();
    if (from + kScanChunk < end) fetch(from + kScanChunk);
    const float* in = staged - ROW;
#pragma unroll 2
    for (int t = 0; t < count; ++t) {
      in += ROW;
      const float value = in[3 * PADDED + 4 + local_column];
      float read[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int m = 0; m < PER; m += 4) {
        const int i = (m / 4 * kLanes + l) * 4;
        const float4 query = *reinterpret_cast<const float4*>(in + i);
        const float4 key = *reinterpret_cast<const float4*>(in + PADDED + i);
        const float4 g = *reinterpret_cast<const float4*>(in + 2 * PADDED + i);
        read[0] = fmaf(s[m], query.x, read[0]);
        read[1] = fmaf(s[m + 1], query.y, read[1]);
        read[2] = fmaf(s[m + 2], query.z, read[2]);
        read[3] = fmaf(s[m + 3], query.w, read[3]);
        s[m] = fmaf(s[m], g.x, key.x * value);
        s[m + 1] = fmaf(s[m + 1], g.y, key.y * value);
        s[m + 2] = fmaf(s[m + 2], g.z, key.z * value);
        s[m + 3] = fmaf(s[m + 3], g.w, key.w * value);
      }
      float total = (read[0] + read[1]) + (read[2] + read[3]);
      total += __shfl_xor_sync(0xffffffffu, total, 1);
      total += __shfl_xor_sync(0xffffffffu, total, 2);
      total += __shfl_xor_sync(0xffffffffu, total, 4);
      if (l == 0 && active) out[(size_t)(from + t) * width + head_at + column] = fmaf(in[3 * PADDED], value, total);
    }
  }
  if (!active) return;
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * kLanes + l) * 4;
    if (wide) {
      if (i < dim) *reinterpret_cast<float4*>(column_state + i) = make_float4(s[m], s[m + 1], s[m + 2], s[m + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i + e < dim) column_state[i + e] = s[m + e];
    }
  }
}

template <typename T, int PER, bool SHORT>
int launch_scan(cudaStream_t stream, const void* r, const void* k, const void* v, long long ld, const float* decay_raw,
                const float* decay_bias, const float* bonus, float* state, const int* query_starts,
                const int* state_slots, const int* positions, float* out, int rows, int heads, int dim) {
  constexpr int columns = kScanWarps * (32 / kLanes);
  return mir_launch("wkv_scan", wkv_scan_kernel<T, PER, SHORT>, dim3(rows, heads, (dim + columns - 1) / columns),
                    dim3(32, kScanWarps), 0, stream, 0, (const T*)r, (const T*)k, (const T*)v, ld, decay_raw, decay_bias,
                    bonus, state, query_starts, state_slots, positions, out, heads, dim);
}

template <typename T>
int launch_scan_for(cudaStream_t stream, const void* r, const void* k, const void* v, long long ld,
                    const float* decay_raw, const float* decay_bias, const float* bonus, float* state,
                    const int* query_starts, const int* state_slots, const int* positions, float* out, int rows,
                    int heads, int dim, bool single_tokens) {
#define MIR_WKV(P)                                                                                                  \
  if (single_tokens)                                                                                                \
    return launch_scan<T, P, true>(stream, r, k, v, ld, decay_raw, decay_bias, bonus, state, query_starts,         \
                                   state_slots, positions, out, rows, heads, dim);                                 \
  return launch_scan<T, P, false>(stream, r, k, v, ld, decay_raw, decay_bias, bonus, state, query_starts,          \
                                  state_slots, positions, out, rows, heads, dim);
  if (dim <= 32) { MIR_WKV(4) }
  if (dim <= 64) { MIR_WKV(8) }
  if (dim <= 96) { MIR_WKV(12) }
  if (dim <= 128) { MIR_WKV(16) }
  if (dim <= 192) { MIR_WKV(24) }
  if (dim <= 256) { MIR_WKV(32) }
#undef MIR_WKV
  mir_set_error("wkv_scan: heads of %d channels are wider than 256", dim);
  return MIR_BAD_ARGUMENT;
}

}  // namespace

// h [tokens, width] with row stride ld; tail [slots, width] 32-bit; mu [5, width] 32-bit; out [5, tokens, width].
MIR_EXPORT int mir_wkv_mix(int bf16, const void* h, long long ld, float* tail, const float* mu, const int* row_of_token,
                           const int* query_starts, const int* state_slots, const int* positions, void* out, int tokens,
                           int rows, int width, int single_tokens_only, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || rows <= 0 || width <= 0) {
    mir_set_error("wkv_mix: bad sizes (tokens %d, rows %d, width %d)", tokens, rows, width);
    return MIR_BAD_ARGUMENT;
  }
  const int threads = width >= 1024 ? 256 : 128;
  int status;
  if (bf16)
    status = mir_launch("wkv_mix", wkv_mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, 0,
                        (const __nv_bfloat16*)h, ld, tail, mu, row_of_token, query_starts, state_slots, positions,
                        (__nv_bfloat16*)out, tokens, width);
  else
    status = mir_launch("wkv_mix", wkv_mix_kernel<float>, dim3(tokens), dim3(threads), 0, stream, 0, (const float*)h, ld,
                        tail, mu, row_of_token, query_starts, state_slots, positions, (float*)out, tokens, width);
  if (status != MIR_OK || single_tokens_only) return status;
  if (bf16)
    return mir_launch("wkv_tail", wkv_tail_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, 0,
                      (const __nv_bfloat16*)h, ld, tail, query_starts, state_slots, positions, width);
  return mir_launch("wkv_tail", wkv_tail_kernel<float>, dim3(rows), dim3(threads), 0, stream, 0, (const float*)h, ld, tail,
                    query_starts, state_slots, positions, width);
}

// r, k, v [tokens, heads * dim] with row stride ld in the activations' type; decay_raw [tokens, heads * dim] 32-bit
// (the low-rank pair's result), decay_bias and bonus [heads * dim] 32-bit; state [slots, heads, dim (value channel),
// dim (key channel)] 32-bit; out [tokens, heads * dim] 32-bit: o before the head norm.
MIR_EXPORT int mir_wkv_scan(int bf16, const void* r, const void* k, const void* v, long long ld, const float* decay_raw,
                            const float* decay_bias, const float* bonus, float* state, const int* query_starts,
                            const int* state_slots, const int* positions, float* out, int tokens, int rows, int heads,
                            int dim, cudaStream_t stream) {
  if (tokens == 0 || rows == 0) return MIR_OK;
  if (tokens < 0 || rows < 0 || heads <= 0 || dim <= 0 || heads > 65535) {
    mir_set_error("wkv_scan: bad sizes (tokens %d, rows %d, heads %d, dim %d)", tokens, rows, heads, dim);
    return MIR_BAD_ARGUMENT;
  }
  const bool single_tokens = tokens == rows;                     // a step of decoded tokens: every row brings one
  if (bf16)
    return launch_scan_for<__nv_bfloat16>(stream, r, k, v, ld, decay_raw, decay_bias, bonus, state, query_starts,
                                          state_slots, positions, out, rows, heads, dim, single_tokens);
  return launch_scan_for<float>(stream, r, k, v, ld, decay_raw, decay_bias, bonus, state, query_starts, state_slots,
                                positions, out, rows, heads, dim, single_tokens);
}
