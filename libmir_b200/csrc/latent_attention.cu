// Kernels of latent attention: queries, keys and values come through low-rank latents, and what is cached per token
// is one normed latent (read as key and as value by every head) beside one rotated key part shared by all heads.
//
//   latent_prepare   per token: RMS norm of the query latent (out: the normed latent for the query up-projection),
//                    RMS norm of the key/value latent and rotation of the shared key part, both written to the
//                    token's cache row [kv_rank | rotary dims]
//   rope_rows        rotation of [tokens, heads, dims] views by position, half-split or interleaved pairs, cos and sin
//                    times a magnitude; in place or into another buffer
//   head_linear      out[t, h, :] = W_h x[t, h, :], a product per head on strided views, optionally times the
//                    sigmoid of a gate: the key up-projection folded into the queries, and the value up-projection
//                    of the attended latents
// Norms, angles and accumulation are 32-bit; T is the storage type of activations, weights and cache.
#include "common.cuh"

using namespace mir;

namespace {

__device__ __forceinline__ float sigmoid_of(float z) { return 1.0f / (1.0f + expf(-z)); }

// (u, v) at `position` for the pair with inverse frequency f: (u cos a - v sin a, v cos a + u sin a), a = position * f
// as a 32-bit product, cos and sin times `magnitude`.
__device__ __forceinline__ void rotate_pair(float& u, float& v, int position, float frequency, float magnitude) {
  float sine, cosine;
  sincosf((float)position * frequency, &sine, &cosine);
  sine *= magnitude;
  cosine *= magnitude;
  const float a = u * cosine - v * sine;
  const float b = v * cosine + u * sine;
  u = a;
  v = b;
}

// One CTA per token.  packed: the token's row of the mixer's first product; the query latent starts at q_offset
// (q_rank wide), the key/value latent at kv_offset (kv_rank wide) with the shared key part (rotary wide) behind it.
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ packed, long long ld, int q_offset, int q_rank, int kv_offset,
                                      int kv_rank, int rotary, const float* __restrict__ q_norm,
                                      const float* __restrict__ kv_norm, float eps, const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                      float magnitude, int interleaved, T* __restrict__ latent_q, T* __restrict__ pages) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  const int position = positions[token];
  if (position < 0) return;                                      // a padding row of a captured batch
  const T* row = packed + (size_t)token * ld;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float x = to_float(row[q_offset + i]);
    sum = fmaf(x, x, sum);
  }
  sum = block_sum(sum, scratch);
  const float q_inverse = rsqrtf(sum / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    latent_q[(size_t)token * q_rank + i] = from_float<T>(to_float(row[q_offset + i]) * q_inverse * q_norm[i]);
  const int slot = slot_mapping != nullptr ? slot_mapping[token] : -1;
  if (slot < 0) return;                                          // (uniform over the CTA)
  sum = 0.0f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float x = to_float(row[kv_offset + i]);
    sum = fmaf(x, x, sum);
  }
  sum = block_sum(sum, scratch);
  const float kv_inverse = rsqrtf(sum / (float)kv_rank + eps);
  T* cached = pages + (size_t)slot * (kv_rank + rotary);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    cached[i] = from_float<T>(to_float(row[kv_offset + i]) * kv_inverse * kv_norm[i]);
  const int half = rotary / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int first = interleaved ? 2 * i : i, second = interleaved ? 2 * i + 1 : i + half;
    float u = to_float(row[kv_offset + kv_rank + first]), v = to_float(row[kv_offset + kv_rank + second]);
    rotate_pair(u, v, position, inv_freq[i], magnitude);
    cached[kv_rank + first] = from_float<T>(u);
    cached[kv_rank + second] = from_float<T>(v);
  }
}

// One thread per (token, head, pair).  src and dst may be the same buffer.
template <typename T>
__global__ void rope_rows_kernel(const T* __restrict__ src, long long src_token, long long src_head, T* dst,
                                 long long dst_token, long long dst_head, const int* __restrict__ positions,
                                 const float* __restrict__ inv_freq, float magnitude, int interleaved, int tokens,
                                 int heads, int rotary) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int half = rotary / 2;
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= (long long)tokens * heads * half) return;
  const int i = (int)(index % half);
  const int head = (int)((index / half) % heads);
  const int token = (int)(index / ((long long)half * heads));
  const int position = positions[token];
  if (position < 0) return;
  const int first = interleaved ? 2 * i : i, second = interleaved ? 2 * i + 1 : i + half;
  const T* from = src + (size_t)token * src_token + (size_t)head * src_head;
  T* to = dst + (size_t)token * dst_token + (size_t)head * dst_head;
  float u = to_float(from[first]), v = to_float(from[second]);
  rotate_pair(u, v, position, inv_freq[i], magnitude);
  to[first] = from_float<T>(u);
  to[second] = from_float<T>(v);
}

constexpr int kHeadLinearTokens = 8;
constexpr int kHeadLinearChunk = 256;

// out[t, h, o] = sum_i x[t, h, i] * w[h, i, o] (times sigmoid(gate[t, h, o])): blockDim (32, 8), a CTA takes 32
// outputs of one head for 8 tokens; every output is one ascending chain over i, whatever else is in the batch.
template <typename T>
__global__ void head_linear_kernel(const T* __restrict__ x, long long x_token, long long x_head,
                                   const T* __restrict__ w, T* __restrict__ out, long long out_token, long long out_head,
                                   const T* __restrict__ gate, long long gate_token, int tokens, int in_dim, int out_dim) {
  __shared__ float rows[kHeadLinearTokens][kHeadLinearChunk];
  grid_launch_dependents();
  grid_dependency_wait();
  const int head = blockIdx.y;
  const int o = blockIdx.x * 32 + threadIdx.x;
  const int token = blockIdx.z * kHeadLinearTokens + threadIdx.y;
  const T* weights = w + (size_t)head * in_dim * out_dim;
  float acc = 0.0f;
  for (int from = 0; from < in_dim; from += kHeadLinearChunk) {
    const int count = min(kHeadLinearChunk, in_dim - from);
    __syncthreads();
    if (token < tokens)
      for (int i = threadIdx.x; i < count; i += 32)
        rows[threadIdx.y][i] = to_float(x[(size_t)token * x_token + (size_t)head * x_head + from + i]);
    __syncthreads();
    if (o < out_dim && token < tokens)
      for (int i = 0; i < count; ++i) acc = fmaf(rows[threadIdx.y][i], to_float(weights[(size_t)(from + i) * out_dim + o]), acc);
  }
  if (o >= out_dim || token >= tokens) return;
  if (gate != nullptr) {
    // the product is rounded to the activations' type as a projection is, then gated
    acc = to_float(from_float<T>(acc)) * sigmoid_of(to_float(gate[(size_t)token * gate_token + (size_t)head * out_dim + o]));
  }
  out[(size_t)token * out_token + (size_t)head * out_head + o] = from_float<T>(acc);
}

// x[t, c] *= sigmoid(gate[t, c]) on rows with strides, in place; the product was rounded to the activations' type
// before, as a projection is.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                    int columns, size_t total) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t row = index / columns;
  const int c = (int)(index - row * columns);
  T* at = x + row * x_stride + c;
  *at = from_float<T>(to_float(*at) * sigmoid_of(to_float(gate[row * gate_stride + c])));
}

}  // namespace

MIR_EXPORT int mir_sigmoid_gate(int bf16, void* x, long long x_stride, const void* gate, long long gate_stride, int rows,
                                int columns, cudaStream_t stream) {
  if (rows == 0 || columns == 0) return MIR_OK;
  if (rows < 0 || columns < 0) { mir_set_error("sigmoid_gate: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)rows * columns;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (bf16)
    return mir_launch("sigmoid_gate", sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 0, (__nv_bfloat16*)x,
                      x_stride, (const __nv_bfloat16*)gate, gate_stride, columns, total);
  return mir_launch("sigmoid_gate", sigmoid_gate_kernel<float>, grid, dim3(256), 0, stream, 0, (float*)x, x_stride,
                    (const float*)gate, gate_stride, columns, total);
}

MIR_EXPORT int mir_latent_prepare(int bf16, const void* packed, long long ld, int q_offset, int q_rank, int kv_offset,
                                  int kv_rank, int rotary, const float* q_norm, const float* kv_norm, float eps,
                                  const int* positions, const int* slot_mapping, const float* inv_freq, float magnitude,
                                  int interleaved, void* latent_q, void* pages, int tokens, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || q_rank <= 0 || kv_rank <= 0 || rotary < 0 || rotary % 2) {
    mir_set_error("latent_prepare: bad sizes (tokens %d, ranks %d and %d, rotary %d)", tokens, q_rank, kv_rank, rotary);
    return MIR_BAD_ARGUMENT;
  }
  if (bf16)
    return mir_launch("latent_prepare", latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, 0,
                      (const __nv_bfloat16*)packed, ld, q_offset, q_rank, kv_offset, kv_rank, rotary, q_norm, kv_norm, eps,
                      positions, slot_mapping, inv_freq, magnitude, interleaved, (__nv_bfloat16*)latent_q,
                      (__nv_bfloat16*)pages);
  return mir_launch("latent_prepare", latent_prepare_kernel<float>, dim3(tokens), dim3(256), 0, stream, 0,
                    (const float*)packed, ld, q_offset, q_rank, kv_offset, kv_rank, rotary, q_norm, kv_norm, eps, positions,
                    slot_mapping, inv_freq, magnitude, interleaved, (float*)latent_q, (float*)pages);
}

MIR_EXPORT int mir_rope_rows(int bf16, const void* src, long long src_token, long long src_head, void* dst,
                             long long dst_token, long long dst_head, const int* positions, const float* inv_freq,
                             float magnitude, int interleaved, int tokens, int heads, int rotary, cudaStream_t stream) {
  if (tokens == 0 || heads == 0 || rotary == 0) return MIR_OK;
  if (tokens < 0 || heads < 0 || rotary < 0 || rotary % 2) {
    mir_set_error("rope_rows: bad sizes (tokens %d, heads %d, rotary %d)", tokens, heads, rotary);
    return MIR_BAD_ARGUMENT;
  }
  const long long total = (long long)tokens * heads * (rotary / 2);
  const dim3 grid((unsigned)((total + 255) / 256));
  if (bf16)
    return mir_launch("rope_rows", rope_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 0,
                      (const __nv_bfloat16*)src, src_token, src_head, (__nv_bfloat16*)dst, dst_token, dst_head, positions,
                      inv_freq, magnitude, interleaved, tokens, heads, rotary);
  return mir_launch("rope_rows", rope_rows_kernel<float>, grid, dim3(256), 0, stream, 0, (const float*)src, src_token,
                    src_head, (float*)dst, dst_token, dst_head, positions, inv_freq, magnitude, interleaved, tokens, heads,
                    rotary);
}

MIR_EXPORT int mir_head_linear(int bf16, const void* x, long long x_token, long long x_head, const void* w, void* out,
                               long long out_token, long long out_head, const void* gate, long long gate_token,
                               int tokens, int heads, int in_dim, int out_dim, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || in_dim <= 0 || out_dim <= 0 || heads > 65535) {
    mir_set_error("head_linear: bad sizes (tokens %d, heads %d, in %d, out %d)", tokens, heads, in_dim, out_dim);
    return MIR_BAD_ARGUMENT;
  }
  const int token_tiles = (tokens + kHeadLinearTokens - 1) / kHeadLinearTokens;
  if (token_tiles > 65535) {
    mir_set_error("head_linear: %d tokens are more than a launch takes", tokens);
    return MIR_BAD_ARGUMENT;
  }
  const dim3 grid((out_dim + 31) / 32, heads, token_tiles), block(32, kHeadLinearTokens);
  if (bf16)
    return mir_launch("head_linear", head_linear_kernel<__nv_bfloat16>, grid, block, 0, stream, 0,
                      (const __nv_bfloat16*)x, x_token, x_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_token,
                      out_head, (const __nv_bfloat16*)gate, gate_token, tokens, in_dim, out_dim);
  return mir_launch("head_linear", head_linear_kernel<float>, grid, block, 0, stream, 0, (const float*)x, x_token, x_head,
                    (const float*)w, (float*)out, out_token, out_head, (const float*)gate, gate_token, tokens, in_dim,
                    out_dim);
}
