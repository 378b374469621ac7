// Attention over cached latents on tensor cores (bf16, mma.sync m16n8k16), for prompt portions and decoded tokens.
//
// Every query head of a token is a vector of W = kv_rank + rotary numbers (the key up-projection folded into the
// query), every cached row is one key of W numbers whose first R = kv_rank numbers are also its value, and all heads
// read the same rows.  So the (token, head) pairs of a request are the rows of one tall query matrix: a CTA takes 64
// consecutive pairs (token-major) and walks over the request's keys 64 at a time:
//   S = Q K^T       the 8 warps take 8 keys each (all 64 query rows), scores go to shared memory
//   softmax         4 threads per query row: causal mask by the row's own position, running maximum and sum, P in bf16
//   O += P V        the 8 warps take NT * 8 value columns each (all 64 query rows); V is the key tile itself, read
//                   transposed by ldmatrix
// The key tile is read from the pages once per 64 query rows, which for decoded tokens means once for all heads.
// With more than one partition a CTA walks over its share of the keys only and leaves an unnormalised partial result
// (sum, maximum, weights' sum per row); a second kernel merges them.  Scores, softmax and sums are 32-bit.
#include <algorithm>
#include <cfloat>
#include "common.cuh"
#include "launchers.h"

using namespace mir;

namespace {

constexpr int kRows = 64;            // (token, head) pairs per CTA
constexpr int kKeys = 64;            // keys per tile
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void copy16(void* dst, const void* src) {
  const unsigned target = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// grid (row blocks, request rows, partitions), kThreads threads.
//   q [tokens, heads * width] (row stride q_stride): the folded queries; out [tokens, heads * rank]
//   pages [cache rows, width]; block_table [request rows, table_width]; query_starts [rows + 1]; context_lens [rows]
//   partial_o [tokens * heads, partitions, rank], partial_ml [tokens * heads, partitions, 2]: only with partitions > 1
template <int NT>
__global__ void __launch_bounds__(kThreads)
latent_attention_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ out,
                        const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ query_starts, const int* __restrict__ context_lens, int page_size,
                        int heads, int width, int rank, float scale, int partition_keys, int partitions,
                        float* __restrict__ partial_o, float* __restrict__ partial_ml, int query_rows, int key_buffers) {
  extern __shared__ __align__(16) unsigned char shared[];
  const int padded = (width + 15) / 16 * 16;                    // the reduction runs in steps of 16
  const int ld = padded + 8;                                     // row stride of the query and key tiles (elements)
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(shared);
  __nv_bfloat16* k_s = q_s + (size_t)query_rows * ld;            // query_rows: what the launch keeps of the 64 (a multiple of 16)
  float* s_s = reinterpret_cast<float*>(k_s + (size_t)key_buffers * kKeys * ld);   // key_buffers: 1, or 2 where they fit
  constexpr int lds = kKeys + 4;
  __nv_bfloat16* p_s = reinterpret_cast<__nv_bfloat16*>(s_s + kRows * lds);
  constexpr int ldp = kKeys + 8;
  float* correction_s = reinterpret_cast<float*>(p_s + kRows * ldp);
  float* sum_s = correction_s + kRows;
  float* max_s = sum_s + kRows;

  const int thread = threadIdx.x, lane = thread & 31, warp = thread >> 5;
  const int row = blockIdx.y;
  const int start = query_starts[row];
  const int count = query_starts[row + 1] - start;               // tokens of this request in the step
  const int pairs = count * heads;
  const int first_pair = blockIdx.x * kRows;
  if (first_pair >= pairs) return;
  const int context = context_lens[row];
  const int first_position = context - count;                    // of the request's first token in the step
  const int last_pair = min(first_pair + kRows, pairs) - 1;
  const int last_position = first_position + last_pair / heads;  // the furthest key any row of this block sees
  const int key_begin = blockIdx.z * partition_keys;
  const int key_end = min(min((blockIdx.z + 1) * partition_keys, last_position + 1), context);
  const int* table = block_table + (size_t)row * table_width;

  // the query rows of this block: four threads copy a row, 16 bytes at a time (no division in the loop)
  {
    const int r = thread >> 2;
    const int pair = first_pair + r;
    const bool there = pair < pairs;
    const __nv_bfloat16* from = there ? q + (size_t)(start + pair / heads) * q_stride + (size_t)(pair % heads) * width : q;
    __nv_bfloat16* to = q_s + (size_t)r * ld;
    for (int c = (thread & 3) * 8; c < padded && r < query_rows; c += 32) {
      uint4 value = make_uint4(0u, 0u, 0u, 0u);
      if (there && c < width) value = *reinterpret_cast<const uint4*>(from + c);
      *reinterpret_cast<uint4*>(to + c) = value;
    }
  }

  // softmax owners: 4 threads per query row
  const int my_row = thread >> 2, quarter = thread & 3;
  const int my_pair = first_pair + my_row;
  const int my_position = my_pair < pairs ? first_position + my_pair / heads : -1;
  float running_max = -INFINITY, running_sum = 0.0f;
  const float scale2 = scale * kLog2e;

  float o[4][NT][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[mt][nt][e] = 0.0f;
  const int first_column = warp * NT * 8;
  const int row_tiles = (min(kRows, pairs - first_pair) + 15) / 16;   // tiles of 16 query rows that hold any row

  // four threads copy a key's row: one look at the block table per thread and tile, then 16-byte copies
  auto fetch_keys = [&](int k0, __nv_bfloat16* tile) {
    const int r = thread >> 2;
    const int key = k0 + r;
    const int page = key < key_end ? table[key / page_size] : -1;
    const __nv_bfloat16* from = page >= 0 ? pages + ((size_t)page * page_size + key % page_size) * width : pages;
    __nv_bfloat16* to = tile + (size_t)r * ld;
    for (int c = (thread & 3) * 8; c < padded; c += 32) {
      if (page >= 0 && c < width) copy16(to + c, from + c);
      else *reinterpret_cast<uint4*>(to + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  __nv_bfloat16* const first_tile = k_s;
  int buffer = 0;
  for (int k0 = key_begin; k0 < key_end; k0 += kKeys) {
    // One buffer: the tile is fetched here, after everybody is done with the tile before.  Two buffers: this tile was
    // asked for while the tile before was multiplied, and the next one is asked for as soon as this one has landed.
    if (key_buffers == 1 || k0 == key_begin) {
      __syncthreads();                                           // (also: q_s is written)
      fetch_keys(k0, first_tile + (size_t)buffer * kKeys * ld);
    }
    copy_wait_all();
    __syncthreads();
    k_s = first_tile + (size_t)buffer * kKeys * ld;
    if (key_buffers == 2) {
      if (k0 + kKeys < key_end) fetch_keys(k0 + kKeys, first_tile + (size_t)(buffer ^ 1) * kKeys * ld);
      buffer ^= 1;
    }
    // S = Q K^T: this warp's 8 keys against all 64 query rows
    {
      float s[4][4];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[mt][e] = 0.0f;
      const __nv_bfloat16* b_at = k_s + (size_t)(warp * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8;
      const __nv_bfloat16* a_at = q_s + (size_t)(lane & 15) * ld + (lane >> 4) * 8;
#pragma unroll 4
      for (int k = 0; k < padded; k += 16) {                      // (unrolled: the loads of later steps start early)
        unsigned b[2];
        ldmatrix_x2(b, b_at + k);
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          if (mt < row_tiles) {                                   // (decoded tokens: heads / 16 of the four)
            unsigned a[4];
            ldmatrix_x4(a, a_at + (size_t)mt * 16 * ld + k);
            mma_bf16(s[mt], a, b);
          }
        }
      }
      const int g = lane >> 2, c = warp * 8 + (lane & 3) * 2;
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        s_s[(mt * 16 + g) * lds + c] = s[mt][0];
        s_s[(mt * 16 + g) * lds + c + 1] = s[mt][1];
        s_s[(mt * 16 + g + 8) * lds + c] = s[mt][2];
        s_s[(mt * 16 + g + 8) * lds + c + 1] = s[mt][3];
      }
    }
    __syncthreads();
    // softmax of the tile: every row against its own position
    {
      float values[16];
      float tile_max = -INFINITY;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int key = k0 + quarter * 16 + j;
        const bool seen = key <= my_position && key < key_end;
        values[j] = seen ? s_s[my_row * lds + quarter * 16 + j] * scale2 : -INFINITY;
        tile_max = fmaxf(tile_max, values[j]);
      }
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      const float next_max = fmaxf(running_max, tile_max);
      const float correction = next_max == -INFINITY ? 1.0f : exp2f(running_max - next_max);
      float tile_sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const float a = next_max == -INFINITY ? 0.0f : exp2f(values[j] - next_max);
        const float b = next_max == -INFINITY ? 0.0f : exp2f(values[j + 1] - next_max);
        const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
        // the sum is of the weights as the product will see them
        tile_sum += __low2float(pair) + __high2float(pair);
        *reinterpret_cast<__nv_bfloat162*>(p_s + my_row * ldp + quarter * 16 + j) = pair;
      }
      tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, 1);
      tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, 2);
      running_sum = running_sum * correction + tile_sum;
      running_max = next_max;
      if (quarter == 0) correction_s[my_row] = correction;
    }
    __syncthreads();
    // O = O * correction + P V: this warp's value columns for all 64 query rows
    if (first_column < rank) {
      const int g = lane >> 2;
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        const float low = correction_s[mt * 16 + g], high = correction_s[mt * 16 + g + 8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          o[mt][nt][0] *= low; o[mt][nt][1] *= low; o[mt][nt][2] *= high; o[mt][nt][3] *= high;
        }
      }
      const __nv_bfloat16* a_at = p_s + (lane & 15) * ldp + (lane >> 4) * 8;
      const __nv_bfloat16* b_at = k_s + (size_t)(lane & 15) * ld + first_column;
#pragma unroll
      for (int k = 0; k < kKeys; k += 16) {
        unsigned a[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt)
          if (mt < row_tiles) ldmatrix_x4(a[mt], a_at + mt * 16 * ldp + k);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (first_column + nt * 8 < rank) {
            unsigned b[2];
            ldmatrix_x2_trans(b, b_at + (size_t)k * ld + nt * 8);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
              if (mt < row_tiles) mma_bf16(o[mt][nt], a[mt], b);
          }
        }
      }
    }
  }
  __syncthreads();
  if (quarter == 0) {
    sum_s[my_row] = running_sum;
    max_s[my_row] = running_max;
  }
  __syncthreads();
  const int g = lane >> 2, c2 = (lane & 3) * 2;
  if (partitions == 1) {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = mt * 16 + g + half * 8;
        const int pair = first_pair + r;
        if (pair >= pairs) continue;
        const float inverse = sum_s[r] > 0.0f ? 1.0f / sum_s[r] : 0.0f;
        __nv_bfloat16* to = out + ((size_t)(start + pair / heads) * heads + pair % heads) * rank;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int column = first_column + nt * 8 + c2;
          if (column < rank)          // (rank is a multiple of 8: both columns are inside)
            *reinterpret_cast<__nv_bfloat162*>(to + column) =
                __floats2bfloat162_rn(o[mt][nt][half * 2] * inverse, o[mt][nt][half * 2 + 1] * inverse);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mt * 16 + g + half * 8;
      const int pair = first_pair + r;
      if (pair >= pairs) continue;
      const size_t unit = ((size_t)(start + pair / heads) * heads + pair % heads) * partitions + blockIdx.z;
      if (warp == 0 && (lane & 3) == 0) {
        partial_ml[unit * 2] = max_s[r];
        partial_ml[unit * 2 + 1] = sum_s[r];
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int column = first_column + nt * 8 + c2;
        if (column < rank)
          *reinterpret_cast<float2*>(partial_o + unit * rank + column) = make_float2(o[mt][nt][half * 2], o[mt][nt][half * 2 + 1]);
      }
    }
  }
}

// One CTA per (token, head): the partitions' partial results into the normalised output.
__global__ void latent_attention_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                              __nv_bfloat16* __restrict__ out, int rank, int partitions) {
  const size_t unit = blockIdx.x;
  float top = -INFINITY;
  for (int p = 0; p < partitions; ++p) top = fmaxf(top, partial_ml[(unit * partitions + p) * 2]);
  float total = 0.0f;
  for (int p = 0; p < partitions; ++p) {
    const float m = partial_ml[(unit * partitions + p) * 2];
    if (m != -INFINITY) total += partial_ml[(unit * partitions + p) * 2 + 1] * exp2f(m - top);
  }
  const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float sum = 0.0f;
    for (int p = 0; p < partitions; ++p) {
      const float m = partial_ml[(unit * partitions + p) * 2];
      if (m != -INFINITY) sum = fmaf(partial_o[(unit * partitions + p) * rank + c], exp2f(m - top), sum);
    }
    out[unit * rank + c] = __float2bfloat16_rn(sum * inverse);
  }
}

size_t shared_bytes(int width, int query_rows = kRows, int key_buffers = 1) {
  const int padded = (width + 15) / 16 * 16;
  const size_t ld = padded + 8;
  return (size_t)(query_rows + key_buffers * kKeys) * ld * 2 + (size_t)kRows * (kKeys + 4) * 4 +
         (size_t)kRows * (kKeys + 8) * 2 + 3 * kRows * 4;
}

template <int NT>
int launch(cudaStream_t stream, dim3 grid, size_t smem, const void* q, long long q_stride, void* out, const void* pages,
           const int* block_table, int table_width, const int* query_starts, const int* context_lens, int page_size,
           int heads, int width, int rank, float scale, int partition_keys, int partitions, float* partial_o,
           float* partial_ml, int query_rows, int key_buffers) {
  static size_t raised = 0;
  if (smem > raised) {
    const cudaError_t err = cudaFuncSetAttribute(latent_attention_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
    if (err != cudaSuccess) {
      mir_set_error("latent_attention: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    raised = smem;
  }
  latent_attention_kernel<NT><<<grid, kThreads, smem, stream>>>(
      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)pages, block_table, table_width,
      query_starts, context_lens, page_size, heads, width, rank, scale, partition_keys, partitions, partial_o, partial_ml,
      query_rows, key_buffers);
  return mir_check_launch("latent_attention");
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes: rows of 16-byte pieces, at most 512 value columns, a tile that fits
// into shared memory.
MIR_EXPORT int mir_latent_attention_takes(int width, int rank) {
  return width > 0 && rank > 0 && width % 8 == 0 && rank % 8 == 0 && rank <= width && rank <= 512 &&
         shared_bytes(width) <= 227 * 1024;
}

// max_pairs: the most (token, head) pairs any request row brings; partitions > 1 needs partial_o [tokens * heads *
// partitions * rank] and partial_ml [tokens * heads * partitions * 2] floats.
MIR_EXPORT int mir_latent_attention_bf16(const void* q, long long q_stride, void* out, const void* pages,
                                         const int* block_table, int table_width, const int* query_starts,
                                         const int* context_lens, int num_rows, int tokens, int max_pairs, int page_size,
                                         int heads, int width, int rank, float scale, int partition_keys, int partitions,
                                         float* partial_o, float* partial_ml, cudaStream_t stream) {
  if (num_rows == 0 || tokens == 0) return MIR_OK;
  if (!mir_latent_attention_takes(width, rank) || heads <= 0 || page_size <= 0 || partitions < 1 ||
      partition_keys <= 0 || partition_keys % kKeys || num_rows > 65535 || partitions > 65535 || max_pairs <= 0 ||
      (partitions > 1 && (partial_o == nullptr || partial_ml == nullptr))) {
    mir_set_error("latent_attention: sizes the kernel does not take (width %d, rank %d, heads %d, partitions %d of %d keys)",
                  width, rank, heads, partitions, partition_keys);
    return MIR_BAD_ARGUMENT;
  }
  const dim3 grid((max_pairs + kRows - 1) / kRows, num_rows, partitions);
  // decoded tokens bring few query rows: the shared memory they leave holds a second key tile, fetched during the products
  const int query_rows = std::min(kRows, (max_pairs + 15) / 16 * 16);
  const int key_buffers = shared_bytes(width, query_rows, 2) <= 227 * 1024 ? 2 : 1;
  const size_t smem = shared_bytes(width, query_rows, key_buffers);
  int status;
#define MIR_LATENT(N)                                                                                              \
  status = launch<N>(stream, grid, smem, q, q_stride, out, pages, block_table, table_width, query_starts,         \
                     context_lens, page_size, heads, width, rank, scale, partition_keys, partitions, partial_o, \
                     partial_ml, query_rows, key_buffers)
  if (rank <= 64) MIR_LATENT(1);
  else if (rank <= 128) MIR_LATENT(2);
  else if (rank <= 256) MIR_LATENT(4);
  else MIR_LATENT(8);
#undef MIR_LATENT
  if (status != MIR_OK || partitions == 1) return status;
  latent_attention_merge_kernel<<<dim3(tokens * heads), dim3(128), 0, stream>>>(partial_o, partial_ml,
                                                                               (__nv_bfloat16*)out, rank, partitions);
  return mir_check_launch("latent_attention_merge");
}
