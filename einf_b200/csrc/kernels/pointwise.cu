// Memory-bound kernels between the matrix products: embedding gather,
// residual-add + RMSNorm, rotary encoding fused with the QKV bias and the paged
// key/value write, SiLU-and-multiply.
//
// Arithmetic is 32-bit throughout; a value is rounded once, when it is stored in
// the activation type.  The residual stream is a float tensor in both modes.
#include <cuda.h>

#include "common.cuh"

namespace einf {

// ---------------------------------------------------------------------------
// Embedding: residual[t, :] = table[token[t], :]   (reference: nn.Embedding,
// src/einf/executors/torch/qwen.py:744)
// ---------------------------------------------------------------------------
template <typename TTable>
__global__ void embed_kernel(const int* __restrict__ tokens, const TTable* __restrict__ table,
                             float* __restrict__ residual, int hidden, int vocab, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int token = tokens[t];
  float* out = residual + (size_t)t * hidden;
  if (token < 0 || token >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadToken);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const TTable* row = table + (size_t)token * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_float(row[i]);
}

// The input of a consumer may be the partial sums of a split-K product, [splits, T, width].
template <typename TIn>
__device__ __forceinline__ float sum_splits(const TIn* __restrict__ p, int splits, size_t split_stride) {
  // Sixteen loads in flight at a time: the partial sums sit in L2, and a chain of dependent
  // loads would cost a round trip each.
  constexpr int kBatch = 16;
  float v = 0.f;
  int s = 0;
  for (; s + kBatch <= splits; s += kBatch) {
    float t[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) t[u] = to_float(p[(size_t)(s + u) * split_stride]);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) v += t[u];
  }
  if (s < splits) {
    float t[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) t[u] = s + u < splits ? to_float(p[(size_t)(s + u) * split_stride]) : 0.f;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) v += t[u];
  }
  return v;
}

// ---------------------------------------------------------------------------
// residual += sum_s x[s]; out = weight * (residual * rsqrt(mean(residual^2) + eps))
// (reference: fused_add_rmsnorm / rmsnorm, src/einf/executors/torch/fused_ops.py:41-68).
// x may be absent (first norm of the model), or hold `splits` partial sums of a
// split-K matrix product, stacked [splits, T, hidden].  With `rows`, output row r
// is computed from input row rows[r] and the residual is left untouched (used to
// normalise only the rows whose logits are wanted).
// ---------------------------------------------------------------------------
template <typename TX, typename TOut>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, int splits, size_t split_stride,
                                   float* __restrict__ residual, const float* __restrict__ weight,
                                   float eps, TOut* __restrict__ out, const int* __restrict__ rows,
                                   int hidden, int write_residual, int vectorised) {
  extern __shared__ float smem[];
  float* row_buf = smem;                          // [hidden]
  float* scratch = smem + (hidden + 3) / 4 * 4;   // [33]
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  float ss = 0.f;
  if (vectorised) {
    // hidden is a multiple of 4 and there are no partial sums: 16-byte loads of the residual
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(res + i);
      if (x) {
        const TX* xp = x + (size_t)src * hidden + i;
        v.x += to_float(xp[0]);
        v.y += to_float(xp[1]);
        v.z += to_float(xp[2]);
        v.w += to_float(xp[3]);
      }
      *reinterpret_cast<float4*>(row_buf + i) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = res[i];
      if (x) v += sum_splits(x + (size_t)src * hidden + i, splits, split_stride);
      row_buf[i] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (vectorised) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row_buf + i);
      if (write_residual && x) *reinterpret_cast<float4*>(res + i) = v;
      const float4 w = *reinterpret_cast<const float4*>(weight + i);
      TOut* o = out + (size_t)r * hidden + i;
      o[0] = from_float<TOut>(w.x * (v.x * rstd));
      o[1] = from_float<TOut>(w.y * (v.y * rstd));
      o[2] = from_float<TOut>(w.z * (v.z * rstd));
      o[3] = from_float<TOut>(w.w * (v.w * rstd));
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = row_buf[i];
    if (write_residual && x) res[i] = v;
    out[(size_t)r * hidden + i] = from_float<TOut>(weight[i] * (v * rstd));
  }
}

// The same for few rows (decode), where one CTA per row would leave all but a few SMs idle while
// it adds up dozens of partial sums: the CTAs of a cluster split a row's columns and exchange
// their sums of squares through distributed shared memory.  Up to four elements per thread.
template <typename TX, typename TOut>
__global__ void add_rmsnorm_cluster_kernel(const TX* __restrict__ x, int splits, size_t split_stride,
                                           float* __restrict__ residual, const float* __restrict__ weight,
                                           float eps, TOut* __restrict__ out, const int* __restrict__ rows,
                                           int hidden, int write_residual) {
  __shared__ float sums[8 * 32];   // slot c * warps + w: the sum of squares of warp w of CTA c (clusters of up to 8)
  pdl_launch_dependents();
  const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
  const int r = blockIdx.y;
  const int src = rows ? rows[r] : r;                 // rows: an input of the step
  const int slice = (hidden + (int)csize - 1) / (int)csize;
  const int begin = (int)rank * slice, end = min(hidden, begin + slice);
  float w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = begin + (int)threadIdx.x + k * (int)blockDim.x;
    w[k] = i < end ? weight[i] : 0.f;
  }
  pdl_wait();
  float* res = residual + (size_t)src * hidden;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = begin + (int)threadIdx.x + k * (int)blockDim.x;
    v[k] = 0.f;
    if (i < end) {
      v[k] = res[i];
      if (x) v[k] += sum_splits(x + (size_t)src * hidden + i, splits, split_stride);
      ss += v[k] * v[k];
    }
  }
  // Every warp pushes its sum into every CTA of the cluster before the one barrier, so nothing is
  // read remotely after it and no CTA has to be held back from leaving; each warp then adds the
  // same values in the same order.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  ss = warp_sum(ss);
  if (lane < (int)csize) st_cluster_peer(&sums[(int)rank * warps + warp], (uint32_t)lane, ss);
  cluster_barrier();
  float mine = 0.f;
  for (int s = lane; s < (int)csize * warps; s += 32) mine += sums[s];
  const float total = warp_sum(mine);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = begin + (int)threadIdx.x + k * (int)blockDim.x;
    if (i < end) {
      if (write_residual && x) res[i] = v[k];
      out[(size_t)r * hidden + i] = from_float<TOut>(w[k] * (v[k] * rstd));
    }
  }
}

// The same for many rows without partial sums: one warp per row, the row in registers
// (kVec float4 per lane, hidden <= 128 * kVec), no shared memory and no block barrier.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TX, typename TOut, int kVec>
__global__ void add_rmsnorm_warp_kernel(const TX* __restrict__ x, float* __restrict__ residual,
                                        const float* __restrict__ weight, float eps, TOut* __restrict__ out,
                                        const int* __restrict__ rows, int hidden, int num_rows, int write_residual) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= num_rows) return;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  // Loads first, without a branch between them (an index past the row is clamped, its value
  // unused), so that a whole row is in flight at once; a branch per vector would wait for each.
  float4 v[kVec];
#pragma unroll
  for (int j = 0; j < kVec; ++j) v[j] = load4(res + min((j * 32 + lane) * 4, hidden - 4));
  if (x) {
    const TX* xr = x + (size_t)src * hidden;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      const float4 a = load4(xr + min((j * 32 + lane) * 4, hidden - 4));
      v[j].x += a.x;
      v[j].y += a.y;
      v[j].z += a.z;
      v[j].w += a.w;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kVec; ++j)
    if ((j * 32 + lane) * 4 < hidden) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  const float rstd = rsqrtf(warp_sum(ss) / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    const int i = (j * 32 + lane) * 4;
    if (i < hidden) {
      if (write_residual && x) store4(res + i, v[j]);
      const float4 w = load4(weight + i);
      store4(out + (size_t)r * hidden + i,
             make_float4(w.x * (v[j].x * rstd), w.y * (v[j].y * rstd), w.z * (v[j].z * rstd), w.w * (v[j].w * rstd)));
    }
  }
}

// The same for few rows with partial sums when a row fits one CTA at one float4 per thread
// (hidden <= 4096, a multiple of 4): every load of a thread is issued before the first is used
// (the partial sums of up to sixteen K ranges at a time: each batch is a round trip to L2), and
// one block barrier is all the synchronisation there is.
constexpr int kRowBatch = 16;
template <typename TX, typename TOut>
__global__ void add_rmsnorm_row_kernel(const TX* __restrict__ x, int splits, size_t split_stride,
                                       float* __restrict__ residual, const float* __restrict__ weight,
                                       float eps, TOut* __restrict__ out, const int* __restrict__ rows,
                                       int hidden, int write_residual) {
  __shared__ float warp_ss[32];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int i = (int)threadIdx.x * 4;
  const bool live = i < hidden;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  const float4 w = live ? load4(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  const int src = rows ? rows[r] : r;                 // rows: an input of the step
  pdl_wait();
  float* res = residual + (size_t)src * hidden;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    v = load4(res + i);
    if (x) {
      const TX* xp = x + (size_t)src * hidden + i;
      for (int s = 0; s < splits; s += kRowBatch) {
        float4 t[kRowBatch];
#pragma unroll
        for (int u = 0; u < kRowBatch; ++u) t[u] = load4(xp + (size_t)min(s + u, splits - 1) * split_stride);
#pragma unroll
        for (int u = 0; u < kRowBatch; ++u) {
          if (s + u < splits) {
            v.x += t[u].x;
            v.y += t[u].y;
            v.z += t[u].z;
            v.w += t[u].w;
          }
        }
      }
    }
  }
  const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
  if (lane == 0) warp_ss[warp] = ss;
  __syncthreads();
  const float total = warp_sum(lane < warps ? warp_ss[lane] : 0.f);   // the same order in every warp
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (live) {
    if (write_residual && x) store4(res + i, v);
    store4(out + (size_t)r * hidden + i,
           make_float4(w.x * (v.x * rstd), w.y * (v.y * rstd), w.z * (v.z * rstd), w.w * (v.w * rstd)));
  }
}

// The same with the partial sums fetched by TMA: a row's partial sums (up to sixteen K ranges of
// up to 1,536 columns: 98 KB) come into shared memory as a few boxes of one three-dimensional
// tensor map [split, row, column], and the threads add them up from there.  Through the load
// pipe of the one SM that owns a row the same bytes take several times as long (an SM keeps too
// few of its own loads in flight), and the norm of a decode step is 49 such kernels.
constexpr int kRowTmaCols = 256;        // columns per box (a box dimension is at most 256)
constexpr int kRowTmaPolls = 1 << 22;
__device__ __forceinline__ uint32_t pw_smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
template <typename TOut>
__global__ void add_rmsnorm_row_tma_kernel(const __grid_constant__ CUtensorMap map_x, int splits,
                                           float* __restrict__ residual, const float* __restrict__ weight, float eps,
                                           TOut* __restrict__ out, const int* __restrict__ rows, int hidden,
                                           int write_residual, int* status) {
  extern __shared__ __align__(128) unsigned char row_smem[];      // [box][split][256 columns] float, then the barrier
  __shared__ float warp_ss[32];
  __shared__ __align__(8) unsigned long long row_bar;
  const uint32_t bar = pw_smem_addr(&row_bar);
  const int boxes = (hidden + kRowTmaCols - 1) / kRowTmaCols;
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int i = (int)threadIdx.x * 4;
  const bool live = i < hidden;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  const float4 w = live ? load4(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  const int src = rows ? rows[r] : r;                 // rows: an input of the step
  __syncthreads();                                    // the barrier is initialised
  pdl_wait();
  if (threadIdx.x == 0) {
    const uint32_t bytes = (uint32_t)boxes * (uint32_t)splits * kRowTmaCols * 4u;   // a box is counted whole, also past the row's end
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    for (int b = 0; b < boxes; ++b) {
      const uint32_t dst = pw_smem_addr(row_smem) + (uint32_t)b * (uint32_t)splits * kRowTmaCols * 4u;
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
          ::"r"(dst), "l"(&map_x), "r"(b * kRowTmaCols), "r"(src), "r"(0), "r"(bar)
          : "memory");
    }
  }
  float* res = residual + (size_t)src * hidden;
  float4 v = live ? load4(res + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  bool arrived = false;
  for (int poll = 0; poll < kRowTmaPolls && !arrived; ++poll) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(0)
        : "memory");
    arrived = done != 0;
  }
  if (!arrived && threadIdx.x == 0) atomicOr(status, kStatusWaitExpired);
  if (live && arrived) {
    const float* box = reinterpret_cast<const float*>(row_smem) + (size_t)(i / kRowTmaCols) * splits * kRowTmaCols +
                       (i % kRowTmaCols);
    for (int s = 0; s < splits; ++s) {
      const float4 t = *reinterpret_cast<const float4*>(box + (size_t)s * kRowTmaCols);
      v.x += t.x;
      v.y += t.y;
      v.z += t.z;
      v.w += t.w;
    }
  }
  const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
  if (lane == 0) warp_ss[warp] = ss;
  __syncthreads();
  const float total = warp_sum(lane < warps ? warp_ss[lane] : 0.f);   // the same order in every warp
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (live) {
    if (write_residual) store4(res + i, v);
    store4(out + (size_t)r * hidden + i,
           make_float4(w.x * (v.x * rstd), w.y * (v.y * rstd), w.z * (v.z * rstd), w.w * (v.w * rstd)));
  }
}

// ---------------------------------------------------------------------------
// Rotary encoding (rotate-half layout) of Q and K after the bias, and the paged
// write of K and V.  qkv is [T, (Hq + 2 Hkv) * D]: Q heads, then K heads, then V.
//   x'[i]        = x[i] cos(a_i) - x[i + R/2] sin(a_i)
//   x'[i + R/2]  = x[i + R/2] cos(a_i) + x[i] sin(a_i),   a_i = position * inv_freq[i]
// for i < R/2 (R = rotary_dim <= D); dims >= R pass through.  (reference:
// src/einf/executors/torch/model_runner.py:42-78; cache write
// src/einf/executors/torch/ops/csrc/kv_cache_cuda.cu:14-58.)  inv_freq is a
// float table made on the host so that angles match a host computation exactly.
// Cache layout: [page, kv_head, slot_in_page, D]; slots[t] = page * page_size + offset,
// negative = do not write.
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void rope_kv_write_kernel(const TIn* __restrict__ qkv, int splits, size_t split_stride,
                                     const float* __restrict__ bias,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                     T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int num_heads, int num_kv_heads,
                                     int head_size, int rotary_dim, int page_size, int num_pages,
                                     int* status) {
  extern __shared__ float smem[];
  const int half = rotary_dim >> 1;
  float* cos_t = smem;          // [half]
  float* sin_t = smem + half;   // [half]
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];   // an input of the step, like inv_freq: no need to wait
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    cos_t[i] = c;
    sin_t[i] = s;
  }
  pdl_wait();
  __syncthreads();
  const int width = (num_heads + 2 * num_kv_heads) * head_size;
  const TIn* row = qkv + (size_t)t * width;
  const int slot = slots ? slots[t] : -1;
  int page = -1, offset = 0;
  if (slot >= 0) {
    page = slot / page_size;
    offset = slot - page * page_size;
    if (page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
      page = -1;
    }
  }
  // Work items: one per (head, dim pair) for rotated dims, one per dim beyond them.
  const int rot_heads = num_heads + num_kv_heads;
  const int per_head = half + (head_size - rotary_dim);
  const int rot_items = rot_heads * per_head;
  for (int item = threadIdx.x; item < rot_items; item += blockDim.x) {
    const int head = item / per_head;
    const int j = item - head * per_head;
    const int base = head * head_size;
    T* dst;
    if (head < num_heads) {
      dst = q_out + ((size_t)t * num_heads + head) * head_size;
    } else {
      if (page < 0) continue;
      dst = k_cache + (((size_t)page * num_kv_heads + (head - num_heads)) * page_size + offset) * head_size;
    }
    if (j < half) {
      float a = sum_splits(row + base + j, splits, split_stride);
      float b = sum_splits(row + base + j + half, splits, split_stride);
      if (bias) {
        a += bias[base + j];
        b += bias[base + j + half];
      }
      const float c = cos_t[j], s = sin_t[j];
      dst[j] = from_float<T>(a * c - b * s);
      dst[j + half] = from_float<T>(b * c + a * s);
    } else {
      const int d = rotary_dim + (j - half);
      float a = sum_splits(row + base + d, splits, split_stride);
      if (bias) a += bias[base + d];
      dst[d] = from_float<T>(a);
    }
  }
  if (page >= 0) {
    const int v_items = num_kv_heads * head_size;
    const int v_base = rot_heads * head_size;
    for (int item = threadIdx.x; item < v_items; item += blockDim.x) {
      const int head = item / head_size;
      const int d = item - head * head_size;
      float a = sum_splits(row + v_base + item, splits, split_stride);
      if (bias) a += bias[v_base + item];
      v_cache[(((size_t)page * num_kv_heads + head) * page_size + offset) * head_size + d] = from_float<T>(a);
    }
  }
}

// The same with one CTA per (token, head), for few tokens (decode): a CTA per token would
// leave the reading of the partial sums to a handful of SMs.  Each thread computes the angle of
// its own pair, before the wait for the kernel that produced qkv.
template <typename TIn, typename T>
__global__ void rope_kv_write_heads_kernel(const TIn* __restrict__ qkv, int splits, size_t split_stride,
                                           const float* __restrict__ bias, const int* __restrict__ positions,
                                           const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                           T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                           int num_heads, int num_kv_heads, int head_size, int rotary_dim,
                                           int page_size, int num_pages, int* status) {
  pdl_launch_dependents();
  const int heads_total = num_heads + 2 * num_kv_heads;
  const int t = blockIdx.x / heads_total;
  const int head = blockIdx.x - t * heads_total;
  const int half = rotary_dim >> 1;
  const int j = threadIdx.x;
  const bool is_v = head >= num_heads + num_kv_heads;
  float c = 1.f, s = 0.f;
  if (!is_v && j < half) sincosf((float)positions[t] * inv_freq[j], &s, &c);
  const int slot = slots ? slots[t] : -1;
  int page = -1, offset = 0;
  if (slot >= 0) {
    page = slot / page_size;
    offset = slot - page * page_size;
    if (page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
      page = -1;
    }
  }
  // The bias is a weight: read before the wait as well, so that after it only the partial sums
  // are a round trip away.
  const float* head_bias = bias ? bias + (size_t)head * head_size : nullptr;
  const int extra = rotary_dim + (j - half);                  // the dim of a thread past the pairs
  float bias_a = 0.f, bias_b = 0.f;
  if (head_bias) {
    if (is_v) {
      if (j < head_size) bias_a = head_bias[j];
    } else if (j < half) {
      bias_a = head_bias[j];
      bias_b = head_bias[j + half];
    } else if (j < half + (head_size - rotary_dim)) {
      bias_a = head_bias[extra];
    }
  }
  pdl_wait();
  const int width = heads_total * head_size;
  const TIn* row = qkv + (size_t)t * width + (size_t)head * head_size;
  T* dst;
  if (head < num_heads) {
    dst = q_out + ((size_t)t * num_heads + head) * head_size;
  } else {
    if (page < 0) return;
    const int kv_head = is_v ? head - num_heads - num_kv_heads : head - num_heads;
    dst = (is_v ? v_cache : k_cache) + (((size_t)page * num_kv_heads + kv_head) * page_size + offset) * head_size;
  }
  if (is_v) {
    if (j < head_size) dst[j] = from_float<T>(sum_splits(row + j, splits, split_stride) + bias_a);
    return;
  }
  if (j < half) {
    const float a = sum_splits(row + j, splits, split_stride) + bias_a;
    const float b = sum_splits(row + j + half, splits, split_stride) + bias_b;
    dst[j] = from_float<T>(a * c - b * s);
    dst[j + half] = from_float<T>(b * c + a * s);
  } else if (j < half + (head_size - rotary_dim)) {
    dst[extra] = from_float<T>(sum_splits(row + extra, splits, split_stride) + bias_a);
  }
}

// The same for dense bfloat16 rows with the whole head rotated and a head size that is a
// multiple of 16: eight pairs per thread, 16-byte loads and stores.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, const float* bias, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
  if (bias) {   // 16-byte aligned like the row (the launcher checks)
    const float4 b0 = *reinterpret_cast<const float4*>(bias), b1 = *reinterpret_cast<const float4*>(bias + 4);
    v[0] += b0.x;
    v[1] += b0.y;
    v[2] += b0.z;
    v[3] += b0.w;
    v[4] += b1.x;
    v[5] += b1.y;
    v[6] += b1.z;
    v[7] += b1.w;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Several tokens per CTA: their angles are computed side by side before the one barrier, and the
// 16-byte items of all of them are spread over the threads.
constexpr int kRopeTokens = 4;

__global__ void rope_kv_write_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ bias,
                                            const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                            const int* __restrict__ slots, __nv_bfloat16* __restrict__ q_out,
                                            __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                            int num_tokens, int num_heads, int num_kv_heads, int head_size,
                                            int page_size, int num_pages, int* status) {
  extern __shared__ float smem[];
  const int half = head_size >> 1;
  float* cos_t = smem;                          // [kRopeTokens][half]
  float* sin_t = smem + kRopeTokens * half;
  __shared__ int pages[kRopeTokens], offsets[kRopeTokens];
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kRopeTokens;
  const int here = min(kRopeTokens, num_tokens - t0);
  for (int i = threadIdx.x; i < here * half; i += blockDim.x) {
    const int tok = i / half, j = i - tok * half;
    float s, c;
    sincosf((float)positions[t0 + tok] * inv_freq[j], &s, &c);   // inputs of the step: no need to wait
    cos_t[i] = c;
    sin_t[i] = s;
  }
  if (threadIdx.x < here) {
    const int slot = slots ? slots[t0 + threadIdx.x] : -1;
    int page = -1, offset = 0;
    if (slot >= 0) {
      page = slot / page_size;
      offset = slot - page * page_size;
      if (page >= num_pages) {
        atomicOr(status, kStatusBadPage);
        page = -1;
      }
    }
    pages[threadIdx.x] = page;
    offsets[threadIdx.x] = offset;
  }
  pdl_wait();
  __syncthreads();
  const int width = (num_heads + 2 * num_kv_heads) * head_size;
  const int groups = half >> 3;                       // groups of eight pairs per head
  const int rot_items = (num_heads + num_kv_heads) * groups;
  const int v_items = num_kv_heads * (head_size >> 3);
  const int per_token = rot_items + v_items;
  for (int index = threadIdx.x; index < here * per_token; index += blockDim.x) {
    const int tok = index / per_token, item = index - tok * per_token;
    const int t = t0 + tok;
    const __nv_bfloat16* row = qkv + (size_t)t * width;
    const int page = pages[tok], offset = offsets[tok];
    if (item < rot_items) {
      const int head = item / groups;
      const int j = (item - head * groups) << 3;
      const int base = head * head_size;
      __nv_bfloat16* dst;
      if (head < num_heads) {
        dst = q_out + ((size_t)t * num_heads + head) * head_size;
      } else {
        if (page < 0) continue;
        dst = k_cache + (((size_t)page * num_kv_heads + (head - num_heads)) * page_size + offset) * head_size;
      }
      float a[8], b[8], ra[8], rb[8];
      load8(row + base + j, bias ? bias + base + j : nullptr, a);
      load8(row + base + half + j, bias ? bias + base + half + j : nullptr, b);
      const float* cs = cos_t + tok * half + j;
      const float* sn = sin_t + tok * half + j;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        ra[e] = a[e] * cs[e] - b[e] * sn[e];
        rb[e] = b[e] * cs[e] + a[e] * sn[e];
      }
      store8(dst + j, ra);
      store8(dst + half + j, rb);
    } else {
      if (page < 0) continue;
      const int v_item = item - rot_items;
      const int per_head = head_size >> 3;
      const int head = v_item / per_head;
      const int d = (v_item - head * per_head) << 3;
      const int source = (num_heads + num_kv_heads) * head_size + head * head_size + d;
      float a[8];
      load8(row + source, bias ? bias + source : nullptr, a);
      store8(v_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * head_size + d, a);
    }
  }
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i],  silu(z) = z / (1 + exp(-z))
// (reference: src/einf/executors/torch/fused_ops.py:71-77)
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void silu_mul_kernel(const TIn* __restrict__ gate_up, int splits, size_t split_stride,
                                T* __restrict__ out, int intermediate, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const size_t t = idx / intermediate;
    const int i = (int)(idx - t * intermediate);
    const float g = sum_splits(gate_up + t * 2 * intermediate + i, splits, split_stride);
    const float u = sum_splits(gate_up + t * 2 * intermediate + intermediate + i, splits, split_stride);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// The same for dense bfloat16 rows whose width is a multiple of 8: 16-byte loads and stores, one
// vector per thread, block = (token, chunk of the row).  At thousands of tokens this kernel is
// bound by arithmetic, not by memory, if it divides and calls expf exactly; the result is
// rounded to bfloat16, so the hardware exponential and reciprocal (relative error about 1e-6)
// are enough here.  The generic kernel above, which the 32-bit path uses, stays exact.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                       int intermediate, int chunks_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned t = blockIdx.x / (unsigned)chunks_per_row;
  const unsigned chunk = blockIdx.x - t * (unsigned)chunks_per_row;
  const int i = (int)(chunk * blockDim.x + threadIdx.x) << 3;
  if (i < intermediate) {
    const __nv_bfloat16* row = gate_up + (size_t)t * 2 * intermediate;
    const uint4 g = *reinterpret_cast<const uint4*>(row + i);
    const uint4 u = *reinterpret_cast<const uint4*>(row + intermediate + i);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 result;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gf = __bfloat1622float2(gp[e]);
      const float2 uf = __bfloat1622float2(up[e]);
      rp[e] = __floats2bfloat162_rn(__fdividef(gf.x, 1.f + __expf(-gf.x)) * uf.x,
                                    __fdividef(gf.y, 1.f + __expf(-gf.y)) * uf.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * intermediate + i) = result;
  }
}

// One decode step on, in place, for a step of single tokens (one thread per request): the sampled
// token becomes the input, position and context length grow by one, and the cache slot of every
// group follows the request's block table.  A request that writes nothing (slot < 0: padding of a
// graph bucket) keeps its slot.  Lets several decode steps run before the host looks.
struct AdvanceGroups {
  int* slots[4];
  const int* tables[4];
};

__global__ void advance_decode_kernel(int* __restrict__ token_ids, int* __restrict__ positions,
                                      int* __restrict__ context_lens, const int* __restrict__ sampled,
                                      int num_requests, AdvanceGroups groups, int num_groups, int table_width,
                                      int page_size) {
  // No early launch of the dependents here: this kernel writes what the kernels of the next step
  // read before their own dependency wait (positions, slots), so none of them may start before it
  // has ended; without the call the next kernel starts when this one is complete.
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_requests) return;
  token_ids[i] = sampled[i];
  const int position = positions[i] + 1;
  positions[i] = position;
  context_lens[i] += 1;
  for (int g = 0; g < num_groups; ++g) {
    if (groups.slots[g][i] < 0) continue;
    const int page = groups.tables[g][(size_t)i * table_width + position / page_size];
    groups.slots[g][i] = page * page_size + position % page_size;   // a missing page (-1) gives a negative slot: no write
  }
}

// Per-request state of fixed size is read before it is written, so the rows of requests that
// start at position 0 in this step are cleared first; on the device, from the step's own inputs,
// so that the clearing can sit inside a captured step.  Requests without a slot (-1: the padding
// requests of a graph bucket) and requests that go on from an earlier step are left alone.
template <typename Word>
__global__ void zero_fresh_state_kernel(Word* __restrict__ state, long long row_words, int num_slots,
                                        const int* __restrict__ state_slots, const int* __restrict__ q_start,
                                        const int* __restrict__ positions) {
  pdl_launch_dependents();
  pdl_wait();
  const int request = blockIdx.y;
  const int slot = state_slots[request];
  if (slot < 0 || slot >= num_slots || positions[q_start[request]] != 0) return;
  Word* row = state + (size_t)slot * row_words;
  Word zero;
  memset(&zero, 0, sizeof(Word));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < row_words; i += (long long)gridDim.x * blockDim.x)
    row[i] = zero;
}

// out[m, n] += bias[n]: the bias of a matrix product that a library computed.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, int n, size_t total) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    out[idx] = from_float<T>(to_float(out[idx]) + bias[idx % n]);
  }
}

}  // namespace einf

using namespace einf;

static inline int pick_threads(int work) {
  int threads = 32;
  while (threads < work && threads < 256) threads <<= 1;
  return threads;
}

extern "C" int einf_embed(const int* tokens, const void* table, int table_dtype, float* residual,
                          int num_tokens, int hidden, int vocab, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int threads = pick_threads(hidden);
  EINF_DISPATCH_2(table_dtype, T, {
    return (int)launch_pdl(embed_kernel<T>, num_tokens, threads, 0, stream, tokens, (const T*)table, residual, hidden,
                           vocab, status);
  })
}

typedef CUresult (*PwEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PwEncodeTiledFn pw_encode_tiled() {
  static PwEncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return (PwEncodeTiledFn) nullptr;
    return (PwEncodeTiledFn)ptr;
  }();
  return fn;
}

// status: the step's status word (may be null: the TMA-fed kernel, whose wait is bounded, is then not used).
extern "C" int einf_add_rmsnorm(const void* x, int x_dtype, int splits, long long split_stride,
                                float* residual, const float* weight, float eps, void* out,
                                int out_dtype, const int* rows, int num_rows, int hidden,
                                int write_residual, int* status, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  // With partial sums to add up, one element per thread keeps the loads of a row in flight together.
  int threads = pick_threads(hidden);
  if (splits > 1 || num_rows <= 128)
    while (threads < hidden && threads < 1024) threads <<= 1;
  const size_t smem = (size_t)(hidden + 33 + 3) / 4 * 4 * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const int vectorised = (splits == 1 && hidden % 4 == 0 && ((uintptr_t)residual & 15) == 0 &&
                          ((uintptr_t)weight & 15) == 0) ? 1 : 0;
  if (vectorised && num_rows > 128) {
    threads = 32;
    while (threads * 4 < hidden && threads < 256) threads <<= 1;
  }
  const bool few_rows = num_rows <= 16 || (splits > 1 && num_rows <= 64);
  const bool x_vector = !x || (((uintptr_t)x & 15) == 0 && split_stride % 4 == 0);
  // Partial sums of a split-K product for up to 64 rows: one CTA per row with the partial sums
  // brought in by TMA (see the kernel).  Measured, 0.5B sizes, decode steps of 1 / 8 / 16 / 32
  // requests: 0.732 -> 0.725, 0.803 -> 0.787, 0.917 -> 0.881, 1.175 -> 1.115 ms.
  if (status && x && x_dtype == kFloat32 && splits >= 2 && splits <= 16 && num_rows >= 1 && num_rows <= 64 &&
      hidden % 4 == 0 && hidden >= 128 && hidden <= 4096 &&
      (size_t)((hidden + kRowTmaCols - 1) / kRowTmaCols) * splits * kRowTmaCols * 4 <= 160 * 1024 && x_vector &&
      split_stride % hidden == 0 && split_stride / hidden >= num_rows &&
      ((uintptr_t)residual & 15) == 0 && ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0 && pw_encode_tiled()) {
    const long long x_rows = split_stride / hidden;
    CUtensorMap map_x;
    cuuint64_t dims[3] = {(cuuint64_t)hidden, (cuuint64_t)x_rows, (cuuint64_t)splits};
    cuuint64_t strides[2] = {(cuuint64_t)hidden * 4, (cuuint64_t)split_stride * 4};
    cuuint32_t box[3] = {(cuuint32_t)kRowTmaCols, 1, (cuuint32_t)splits};
    cuuint32_t element_strides[3] = {1, 1, 1};
    if (pw_encode_tiled()(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(x), dims, strides, box,
                          element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
      const int row_threads = (hidden / 4 + 31) / 32 * 32;
      const int boxes = (hidden + kRowTmaCols - 1) / kRowTmaCols;
      const size_t row_bytes = (size_t)boxes * splits * kRowTmaCols * 4;
      EINF_DISPATCH_2(out_dtype, TOut, {
        auto kernel = add_rmsnorm_row_tma_kernel<TOut>;
        if (row_bytes > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes);
          if (e != cudaSuccess) return (int)e;
        }
        return (int)launch_pdl(kernel, num_rows, row_threads, row_bytes, stream, map_x, splits, residual, weight, eps,
                               (TOut*)out, rows, hidden, write_residual, status);
      })
    }
  }
  // From five rows on one CTA per row; below that the cluster kernel, whose four CTAs per row pull
  // a row's partial sums through four SMs (0.5B sizes, decode step: 4 rows 0.803 against 0.826 ms,
  // 6 rows 0.857 against 0.843 ms).
  if (few_rows && num_rows >= 5 && hidden % 4 == 0 && hidden >= 128 && hidden <= 4096 && x_vector && ((uintptr_t)residual & 15) == 0 &&
      ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int row_threads = (hidden / 4 + 31) / 32 * 32;
    EINF_DISPATCH_2(x_dtype, TX, {
      EINF_DISPATCH_2(out_dtype, TOut, {
        return (int)launch_pdl(add_rmsnorm_row_kernel<TX, TOut>, num_rows, row_threads, 0, stream, (const TX*)x, splits,
                               (size_t)split_stride, residual, weight, eps, (TOut*)out, rows, hidden, write_residual);
      })
    })
  }
  if (few_rows && hidden >= 256 && hidden <= 4 * 4 * 1024) {
    // few rows, or partial sums to add up: a cluster of four CTAs per row
    const int cluster = 4;
    const int slice = (hidden + cluster - 1) / cluster;
    int cluster_threads = 32;
    while (cluster_threads * 4 < slice) cluster_threads <<= 1;   // at most four elements per thread ...
    while (cluster_threads < slice && cluster_threads < 256) cluster_threads <<= 1;   // ... and one where it fits
    EINF_DISPATCH_2(x_dtype, TX, {
      EINF_DISPATCH_2(out_dtype, TOut, {
        return (int)launch_pdl_cluster(add_rmsnorm_cluster_kernel<TX, TOut>, dim3(cluster, num_rows), dim3(cluster_threads),
                                       0, cluster, stream, (const TX*)x, splits, (size_t)split_stride, residual, weight,
                                       eps, (TOut*)out, rows, hidden, write_residual);
      })
    })
  }
  const bool x_aligned = !x || ((uintptr_t)x & 15) == 0;
  if (vectorised && num_rows > 128 && hidden <= 4096 && x_aligned && ((uintptr_t)out & 15) == 0) {
    const int warps_per_block = 4;   // small blocks: rows spread evenly over the SMs even at a few hundred rows
    const int blocks = (num_rows + warps_per_block - 1) / warps_per_block;
    EINF_DISPATCH_2(x_dtype, TX, {
      EINF_DISPATCH_2(out_dtype, TOut, {
        if (hidden <= 1024)
          return (int)launch_pdl(add_rmsnorm_warp_kernel<TX, TOut, 8>, blocks, warps_per_block * 32, 0, stream,
                                 (const TX*)x, residual, weight, eps, (TOut*)out, rows, hidden, num_rows, write_residual);
        if (hidden <= 2048)
          return (int)launch_pdl(add_rmsnorm_warp_kernel<TX, TOut, 16>, blocks, warps_per_block * 32, 0, stream,
                                 (const TX*)x, residual, weight, eps, (TOut*)out, rows, hidden, num_rows, write_residual);
        return (int)launch_pdl(add_rmsnorm_warp_kernel<TX, TOut, 32>, blocks, warps_per_block * 32, 0, stream,
                               (const TX*)x, residual, weight, eps, (TOut*)out, rows, hidden, num_rows, write_residual);
      })
    })
  }
  EINF_DISPATCH_2(x_dtype, TX, {
    EINF_DISPATCH_2(out_dtype, TOut, {
      auto kernel = add_rmsnorm_kernel<TX, TOut>;
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
      }
      return (int)launch_pdl(kernel, num_rows, threads, smem, stream, (const TX*)x, splits, (size_t)split_stride,
                             residual, weight, eps, (TOut*)out, rows, hidden, write_residual, vectorised);
    })
  })
}

// in_dtype / splits / split_stride: qkv is [T, width] of the activation type (splits = 1), or
// the float partial sums [splits, T, width] of a split-K product.
extern "C" int einf_rope_kv_write(const void* qkv, int in_dtype, int splits, long long split_stride, int dtype,
                                  const float* bias, const int* positions, const float* inv_freq,
                                  const int* slots, void* q_out, void* k_cache, void* v_cache, int num_tokens,
                                  int num_heads, int num_kv_heads, int head_size, int rotary_dim, int page_size,
                                  int num_pages, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int work = (num_heads + num_kv_heads) * head_size / 2;
  int threads = pick_threads(work);
  if (splits > 1 || num_tokens <= 128)
    while (threads < work && threads < 1024) threads <<= 1;
  const size_t smem = (size_t)rotary_dim * sizeof(float);
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (splits == 1 && in_dtype == kBFloat16 && dtype == kBFloat16 && rotary_dim == head_size && head_size % 16 == 0 &&
      aligned(qkv) && aligned(q_out) && aligned(k_cache) && aligned(v_cache) && (!bias || aligned(bias))) {
    const int items = (num_heads + num_kv_heads) * (head_size / 16) + num_kv_heads * (head_size / 8);
    const int tokens_here = num_tokens < kRopeTokens ? num_tokens : kRopeTokens;
    return (int)launch_pdl(rope_kv_write_bf16x8_kernel, (num_tokens + kRopeTokens - 1) / kRopeTokens,
                           pick_threads(items * tokens_here), (size_t)kRopeTokens * head_size * sizeof(float), stream,
                           (const __nv_bfloat16*)qkv, bias, positions, inv_freq, slots, (__nv_bfloat16*)q_out,
                           (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_tokens, num_heads, num_kv_heads,
                           head_size, page_size, num_pages, status);
  }
  if (num_tokens <= 64 && head_size <= 1024) {
    // few tokens: one CTA per (token, head), a thread per pair (or per value of V)
    int head_threads = 32;
    while (head_threads < head_size) head_threads <<= 1;
    const long long blocks = (long long)num_tokens * (num_heads + 2 * num_kv_heads);
    EINF_DISPATCH_2(in_dtype, TIn, {
      EINF_DISPATCH_2(dtype, T, {
        return (int)launch_pdl(rope_kv_write_heads_kernel<TIn, T>, (int)blocks, head_threads, 0, stream,
                               (const TIn*)qkv, splits, (size_t)split_stride, bias, positions, inv_freq, slots,
                               (T*)q_out, (T*)k_cache, (T*)v_cache, num_heads, num_kv_heads, head_size, rotary_dim,
                               page_size, num_pages, status);
      })
    })
  }
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(rope_kv_write_kernel<TIn, T>, num_tokens, threads, smem, stream, (const TIn*)qkv, splits,
                             (size_t)split_stride, bias, positions, inv_freq, slots, (T*)q_out, (T*)k_cache,
                             (T*)v_cache, num_heads, num_kv_heads, head_size, rotary_dim, page_size, num_pages,
                             status);
    })
  })
}

extern "C" int einf_silu_mul(const void* gate_up, int in_dtype, int splits, long long split_stride, void* out,
                             int dtype, long long num_tokens, int intermediate, cudaStream_t stream) {
  const size_t total = (size_t)num_tokens * intermediate;
  if (total == 0) return 0;
  const int threads = 256;
  if (splits == 1 && in_dtype == kBFloat16 && dtype == kBFloat16 && intermediate % 8 == 0 &&
      ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int vectors_per_row = intermediate >> 3;
    const int chunks = (vectors_per_row + threads - 1) / threads;
    if ((long long)chunks * num_tokens < (1ll << 31))
      return (int)launch_pdl(silu_mul_bf16x8_kernel, (int)(chunks * num_tokens), threads, 0, stream,
                             (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, intermediate, chunks);
  }
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(silu_mul_kernel<TIn, T>, (int)blocks, threads, 0, stream, (const TIn*)gate_up, splits,
                             (size_t)split_stride, (T*)out, intermediate, total);
    })
  })
}

extern "C" int einf_advance_decode(int* token_ids, int* positions, int* context_lens, const int* sampled,
                                   int num_requests, int* slots0, const int* table0, int* slots1, const int* table1,
                                   int* slots2, const int* table2, int* slots3, const int* table3, int num_groups,
                                   int table_width, int page_size, cudaStream_t stream) {
  if (num_requests == 0) return 0;
  if (num_groups < 0 || num_groups > 4 || page_size <= 0) return (int)cudaErrorInvalidValue;
  AdvanceGroups groups = {{slots0, slots1, slots2, slots3}, {table0, table1, table2, table3}};
  return (int)launch_pdl(advance_decode_kernel, (num_requests + 127) / 128, 128, 0, stream, token_ids, positions,
                         context_lens, sampled, num_requests, groups, num_groups, table_width, page_size);
}

extern "C" int einf_zero_fresh_state(void* state, long long row_bytes, int num_slots, const int* state_slots,
                                     const int* q_start, const int* positions, int num_requests,
                                     cudaStream_t stream) {
  if (num_requests == 0 || row_bytes == 0 || num_slots == 0) return 0;
  if (row_bytes < 0 || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const bool wide = row_bytes % 16 == 0 && (uintptr_t)state % 16 == 0;
  const bool words = row_bytes % 4 == 0 && (uintptr_t)state % 4 == 0;
  const long long row_words = wide ? row_bytes / 16 : words ? row_bytes / 4 : row_bytes;
  const int threads = 256;
  long long blocks = (row_words + threads - 1) / threads;
  if (blocks > 64) blocks = 64;
  const dim3 grid((unsigned)blocks, (unsigned)num_requests);
  if (wide)
    return (int)launch_pdl(zero_fresh_state_kernel<uint4>, grid, threads, 0, stream, (uint4*)state, row_words, num_slots,
                           state_slots, q_start, positions);
  if (words)
    return (int)launch_pdl(zero_fresh_state_kernel<uint32_t>, grid, threads, 0, stream, (uint32_t*)state, row_words,
                           num_slots, state_slots, q_start, positions);
  return (int)launch_pdl(zero_fresh_state_kernel<uint8_t>, grid, threads, 0, stream, (uint8_t*)state, row_words,
                         num_slots, state_slots, q_start, positions);
}

extern "C" int einf_add_bias(void* out, int dtype, const float* bias, long long rows, int n,
                             cudaStream_t stream) {
  const size_t total = (size_t)rows * n;
  if (total == 0) return 0;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  EINF_DISPATCH_2(dtype, T, {
    add_bias_kernel<T><<<(int)blocks, threads, 0, stream>>>((T*)out, bias, n, total);
  })
  return (int)cudaGetLastError();
}
