// Paged causal attention for any batch: prompt portions and single decoded
// tokens alike, float or bfloat16, any head size that is a multiple of 8 up to
// 256, any number of heads and groups, with an optional sliding window.
//
// This is the 32-bit path's attention and the fallback of the bfloat16 path for
// sizes its tensor-core kernels do not cover.  One warp owns one (token, query
// head) row and walks the keys of its request 32 at a time straight from the
// pages named by the block table:
//   scores: lane j computes q . K[j] in 32-bit (q is pre-multiplied by scale)
//   online softmax in 32-bit across the warp (max, exp, sum)
//   output: lane d accumulates sum_j p_j V[j][d] in 32-bit
// (reference for the maths: src/einf/executors/torch/ops/csrc/paged_attention_cuda.cu:74-147
// and flash_attention_cuda.cu:126-195; lower-right causal mask model_runner.py:145.)
// A token at position p of request r sees keys lo..p of r, lo = max(0, p - window + 1).
#include "common.cuh"

namespace einf {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadSize = 256;

template <typename T>
struct Vec;  // 16-byte vector of T
template <>
struct Vec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(&raw);
    return __bfloat162float(p[i]);
  }
};

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ block_table,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               T* __restrict__ out, int num_rows, int num_heads, int num_kv_heads,
                               int head_size, int page_size, int num_pages, int table_width,
                               float scale, int window, int* status) {
  __shared__ float q_smem[kWarpsPerBlock][kMaxHeadSize];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  if (row >= num_rows) return;
  const int t = row / num_heads;
  const int h = row - t * num_heads;
  const int kv_head = h / (num_heads / num_kv_heads);
  const int r = seq_of_token[t];
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (size_t)r * table_width;

  const T* q_row = q + (size_t)row * head_size;
  for (int d = lane; d < head_size; d += 32) q_smem[warp][d] = to_float(q_row[d]) * scale;
  __syncwarp();
  const float* qs = q_smem[warp];

  constexpr int kDimsPerLane = kMaxHeadSize / 32;
  float acc[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  bool bad_page = false;

  for (int base = lo; base <= pos; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    long long key_offset = -1;  // element offset of (page, kv_head, slot) row, or -1
    if (j <= pos) {
      const int logical = j / page_size;
      const int page = table[logical];
      if (page < 0 || page >= num_pages) {
        bad_page = true;
      } else {
        key_offset = (((long long)page * num_kv_heads + kv_head) * page_size + (j - logical * page_size)) * head_size;
        const T* k_row = k_cache + key_offset;
        float dot = 0.f;
        for (int d = 0; d < head_size; d += Vec<T>::N) {
          Vec<T> kv;
          kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(k_row + d);
#pragma unroll
          for (int e = 0; e < Vec<T>::N; ++e) dot = fmaf(qs[d + e], kv.get(e), dot);
        }
        s = dot;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    // m_new is finite: key `pos` itself is always visible unless its page is bad.
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float correction = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * correction + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) acc[i] *= correction;
    m = m_new;
    const int count = min(32, pos - base + 1);
    for (int kk = 0; kk < count; ++kk) {
      const float pj = __shfl_sync(0xffffffffu, p, kk);
      const long long off = __shfl_sync(0xffffffffu, key_offset, kk);
      if (off < 0) continue;
      const T* v_row = v_cache + off;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < head_size) acc[i] = fmaf(pj, to_float(v_row[d]), acc[i]);
      }
    }
  }
  if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(status, kStatusBadPage);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* o_row = out + (size_t)row * head_size;
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < head_size) o_row[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace einf

using namespace einf;

extern "C" int einf_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                            int dtype, const int* block_table, const int* seq_of_token,
                                            const int* positions, void* out, int num_tokens,
                                            int num_heads, int num_kv_heads, int head_size,
                                            int page_size, int num_pages, int table_width, float scale,
                                            int window, int* status, cudaStream_t stream) {
  const int rows = num_tokens * num_heads;
  if (rows == 0) return 0;
  if (head_size > kMaxHeadSize || head_size % 8 != 0) return (int)cudaErrorInvalidValue;
  const int blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  EINF_DISPATCH_2(dtype, T, {
    paged_attention_generic_kernel<T><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, seq_of_token, positions, (T*)out,
        rows, num_heads, num_kv_heads, head_size, page_size, num_pages, table_width, scale, window, status);
  })
  return (int)cudaGetLastError();
}
