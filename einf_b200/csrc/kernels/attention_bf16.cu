// bfloat16 paged attention on the tensor cores, compiled for one head size
// (-DHEAD_SIZE=n, a multiple of 16 up to 128):
//
//   decode:  one CTA per (token, key/value head, split of its keys).  The query
//            heads that share the key/value head are the 16 rows of the MMA tile,
//            so every key and value is read from HBM once per key/value head (the
//            reference reads them once per query head, docs/ROADMAP.md:193-207 of
//            mon3stera/einf).  Four warps take 16 keys each of a 64-key tile; the
//            splits of one token are merged by the CTA that finishes last.
//   prefill: one CTA per (64 query rows of one request, query head: half a 128-row tile); four warps
//            take 16 rows each and walk the request's keys in 64-key tiles.
//
// Both stream K and V tiles from the pages named by the block table into shared
// memory with cp.async (two to four stages) and use mma.sync m16n8k16 with 32-bit
// accumulation; scores, the running maximum, exponentials and row sums are
// 32-bit; probabilities are rounded to bfloat16 for the second product.  The
// roofline of decode attention is the HBM read of K and V, which this instruction
// saturates; tcgen05's 128-row tiles would be 7/128 full here.
// (maths as in src/einf/executors/torch/ops/csrc/paged_attention_split_kv_cuda.cu:47-337
// and flash_attention_cuda.cu:11-219 of the reference.)
#include "common.cuh"

#ifndef HEAD_SIZE
#define HEAD_SIZE 64
#endif

namespace einf {

constexpr int D = HEAD_SIZE;
static_assert(D % 16 == 0 && D >= 16 && D <= 128, "HEAD_SIZE must be a multiple of 16 up to 128");
constexpr int kChunks = D / 8;          // 16-byte chunks in a row
constexpr int kRowStride = D + 8;       // elements; the pad keeps ldmatrix free of bank conflicts
constexpr int kTileKeys = 64;
constexpr int kThreads = 128;
constexpr int kTileElems = kTileKeys * kRowStride;
// Stages of the cp.async pipeline.  Decode is a pure stream: a CTA that owns up to
// kDecodeStages - 1 tiles has all of them in flight at once and pays HBM latency once.
constexpr int kDecodeStages = D <= 64 ? 4 : 3;
constexpr int kPrefillStages = D <= 64 ? 3 : 2;
constexpr int kMaxSplits = 64;   // most splits of one token's keys

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Bring keys [tile_begin, tile_begin + 64) of one request and key/value head into
// shared memory; rows at or beyond k_end (and rows of a bad page) are zero.
__device__ __forceinline__ bool load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs,
                                             const __nv_bfloat16* __restrict__ k_cache,
                                             const __nv_bfloat16* __restrict__ v_cache,
                                             const int* __restrict__ table, int kv_head, int num_kv_heads,
                                             int page_size, int num_pages, int tile_begin, int k_end) {
  // Consecutive threads take consecutive 16-byte chunks of a row, so one warp instruction
  // copies whole 128-byte lines; each thread makes kChunks / 2 copies per matrix.
  bool bad = false;
#pragma unroll
  for (int it = 0; it < kChunks / 2; ++it) {
    const int idx = it * kThreads + threadIdx.x;
    const int row = idx / kChunks;
    const int chunk = idx - row * kChunks;
    const int j = tile_begin + row;
    __nv_bfloat16* kd = ks + row * kRowStride + chunk * 8;
    __nv_bfloat16* vd = vs + row * kRowStride + chunk * 8;
    bool valid = j < k_end;
    long long off = 0;
    if (valid) {
      const int logical = j / page_size;
      const int page = table[logical];
      if (page < 0 || page >= num_pages) {
        bad = true;
        valid = false;
      } else {
        off = (((long long)page * num_kv_heads + kv_head) * page_size + (j - logical * page_size)) * D + chunk * 8;
      }
    }
    if (valid) {
      cp_async16(kd, k_cache + off);
      cp_async16(vd, v_cache + off);
    } else {
      *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
    }
  }
  return bad;
}

// One row block of 16 x D queries as MMA A fragments, read from global memory.
// rows g and g + 8 of the block come from q_rows[0] and q_rows[1] (null: zeros).
__device__ __forceinline__ void load_q_fragments(uint32_t (&qf)[D / 16][4], const __nv_bfloat16* row_lo,
                                                 const __nv_bfloat16* row_hi, int lane) {
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    qf[kk][0] = row_lo ? *reinterpret_cast<const uint32_t*>(row_lo + kk * 16 + c) : 0u;
    qf[kk][1] = row_hi ? *reinterpret_cast<const uint32_t*>(row_hi + kk * 16 + c) : 0u;
    qf[kk][2] = row_lo ? *reinterpret_cast<const uint32_t*>(row_lo + kk * 16 + 8 + c) : 0u;
    qf[kk][3] = row_hi ? *reinterpret_cast<const uint32_t*>(row_hi + kk * 16 + 8 + c) : 0u;
  }
}

// ---------------------------------------------------------------------------
// Decode
// ---------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* q;        // [tokens, heads, D]
  const __nv_bfloat16* k_cache;  // [pages, kv_heads, page_size, D]
  const __nv_bfloat16* v_cache;
  const int* block_table;        // [requests, table_width]
  const int* seq_of_token;       // [tokens]
  const int* positions;          // [tokens]
  __nv_bfloat16* out;            // [tokens, heads, D]
  float* ws_acc;                 // [tokens, heads, splits, D]   unnormalised partial outputs
  float* ws_ml;                  // [tokens, heads, splits, 2]   running maximum (log2 domain) and row sum
  int* counters;                 // [tokens, kv_heads * head_blocks], zero before the launch, zero after it
  int* status;
  int num_heads, num_kv_heads, page_size, num_pages, table_width, window;
  float scale_log2;              // scale * log2(e)
};

__global__ void __launch_bounds__(kThreads) paged_decode_attention_kernel(DecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ int is_last;

  const int split = blockIdx.x, num_splits = gridDim.x;
  const int group = p.num_heads / p.num_kv_heads;
  const int head_blocks = (group + 15) / 16;
  const int kv_head = blockIdx.y / head_blocks;
  const int head_block = blockIdx.y - kv_head * head_blocks;
  const int t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c2 = (lane & 3) * 2;

  pdl_launch_dependents();
  pdl_wait();
  const int pos = p.positions[t];
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int len = pos - lo + 1;
  int per = (len + num_splits - 1) / num_splits;
  per = (per + kTileKeys - 1) / kTileKeys * kTileKeys;
  const int active = (len + per - 1) / per;
  if (split >= active) return;
  const int k_begin = lo + split * per;
  const int k_end = min(pos + 1, k_begin + per);
  const int* table = p.block_table + (size_t)p.seq_of_token[t] * p.table_width;

  // Query heads of this block: rows g and g + 8.
  const int first_head = kv_head * group + head_block * 16;
  const int rows_valid = min(16, group - head_block * 16);
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* base = p.q + ((size_t)t * p.num_heads + first_head) * D;
    load_q_fragments(qf, g < rows_valid ? base + g * D : nullptr, g + 8 < rows_valid ? base + (g + 8) * D : nullptr, lane);
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int tiles = (k_end - k_begin + kTileKeys - 1) / kTileKeys;
  bool bad = false;
#pragma unroll
  for (int stage = 0; stage < kDecodeStages - 1; ++stage) {
    if (stage < tiles) {
      __nv_bfloat16* kn = smem + stage * 2 * kTileElems;
      bad |= load_kv_tile(kn, kn + kTileElems, p.k_cache, p.v_cache, table, kv_head, p.num_kv_heads, p.page_size,
                          p.num_pages, k_begin + stage * kTileKeys, k_end);
    }
    cp_async_commit();
  }
  for (int tile = 0; tile < tiles; ++tile) {
    cp_async_wait<kDecodeStages - 2>();
    __syncthreads();   // tile `tile` has landed, and every warp is done with the stage refilled below
    {
      const int next = tile + kDecodeStages - 1;
      if (next < tiles) {
        __nv_bfloat16* kn = smem + (next % kDecodeStages) * 2 * kTileElems;
        bad |= load_kv_tile(kn, kn + kTileElems, p.k_cache, p.v_cache, table, kv_head, p.num_kv_heads, p.page_size,
                            p.num_pages, k_begin + next * kTileKeys, k_end);
      }
      cp_async_commit();
    }
    __nv_bfloat16* ks = smem + (tile % kDecodeStages) * 2 * kTileElems;
    __nv_bfloat16* vs = ks + kTileElems;
    const int warp_key0 = k_begin + tile * kTileKeys + warp * 16;
    if (warp_key0 < k_end) {
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t b[4];
        const int key_row = warp * 16 + (lane >> 4) * 8 + (lane & 7);
        const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b, ks + key_row * kRowStride + dim);
        mma_bf16(s[0], qf[kk], b[0], b[1]);
        mma_bf16(s[1], qf[kk], b[2], b[3]);
      }
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = warp_key0 + nt * 8 + c2 + (e & 1);
          const float v = j < k_end ? s[nt][e] * p.scale_log2 : -INFINITY;
          s[nt][e] = v;
          tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(m_run[r], tile_max[r]);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
      uint32_t pa[4];
      {
        float pv[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pv[nt][e] = exp2f(s[nt][e] - m_use[e >> 1]);
            l_run[e >> 1] += pv[nt][e];
          }
        pa[0] = pack_bf16(pv[0][0], pv[0][1]);
        pa[1] = pack_bf16(pv[0][2], pv[0][3]);
        pa[2] = pack_bf16(pv[1][0], pv[1][1]);
        pa[3] = pack_bf16(pv[1][2], pv[1][3]);
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int dt = 0; dt < D / 16; ++dt) {
        uint32_t vb[4];
        const int key_row = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int dim = dt * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vs + key_row * kRowStride + dim);
        mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(p.status, kStatusBadPage);

  // Merge the four warps through shared memory (the K/V buffers are free now).
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float* sm_o = reinterpret_cast<float*>(smem_raw);   // [4][16][D]
  float* sm_m = sm_o + 4 * 16 * D;                      // [4][16]
  float* sm_l = sm_m + 4 * 16;                          // [4][16]
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    float* base = sm_o + (warp * 16) * D + i * 8 + c2;
    base[g * D] = o[i][0];
    base[g * D + 1] = o[i][1];
    base[(g + 8) * D] = o[i][2];
    base[(g + 8) * D + 1] = o[i][3];
  }
  if ((lane & 3) == 0) {
    sm_m[warp * 16 + g] = m_run[0];
    sm_m[warp * 16 + g + 8] = m_run[1];
    sm_l[warp * 16 + g] = l_run[0];
    sm_l[warp * 16 + g + 8] = l_run[1];
  }
  __syncthreads();
  const size_t token_heads = (size_t)t * p.num_heads;
  for (int e = threadIdx.x; e < rows_valid * D; e += kThreads) {
    const int row = e / D, d = e - row * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sm_m[w * 16 + row]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_m[w * 16 + row];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
      l += sm_l[w * 16 + row] * f;
      acc += sm_o[(w * 16 + row) * D + d] * f;
    }
    const int head = first_head + row;
    if (num_splits == 1) {
      p.out[(token_heads + head) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t slot = (token_heads + head) * num_splits + split;
      p.ws_acc[slot * D + d] = acc;
      if (d == 0) {
        p.ws_ml[slot * 2] = m;
        p.ws_ml[slot * 2 + 1] = l;
      }
    }
  }
  if (num_splits == 1) return;

  // The CTA that finishes last among this token's splits merges them.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = p.counters + (size_t)t * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1);
    is_last = done == active - 1;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // All (maximum, sum) pairs of this block's heads in one round of loads, then the weights of
  // the splits per head, then the weighted sum with eight loads in flight per thread.
  float* sm_f = reinterpret_cast<float*>(smem_raw);      // [16][kMaxSplits] weight of each split
  float* sm_inv = sm_f + 16 * kMaxSplits;                // [16] 1 / total sum
  float* sm_lsum = sm_inv + 16;                          // [16][kMaxSplits] sums, before weighting
  for (int e = threadIdx.x; e < rows_valid * active; e += kThreads) {
    const int row = e / active, sp = e - row * active;
    const size_t slot = (token_heads + first_head + row) * num_splits + sp;
    sm_f[row * kMaxSplits + sp] = __ldcg(p.ws_ml + slot * 2);
    sm_lsum[row * kMaxSplits + sp] = __ldcg(p.ws_ml + slot * 2 + 1);
  }
  __syncthreads();
  if (threadIdx.x < rows_valid) {
    const int row = threadIdx.x;
    float m = -INFINITY;
    for (int sp = 0; sp < active; ++sp) m = fmaxf(m, sm_f[row * kMaxSplits + sp]);
    float l = 0.f;
    for (int sp = 0; sp < active; ++sp) {
      const float ms = sm_f[row * kMaxSplits + sp];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
      sm_f[row * kMaxSplits + sp] = f;
      l += sm_lsum[row * kMaxSplits + sp] * f;
    }
    sm_inv[row] = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < rows_valid * D; e += kThreads) {
    const int row = e / D, d = e - row * D;
    const int head = first_head + row;
    const float* acc_base = p.ws_acc + (token_heads + head) * num_splits * D + d;
    float acc = 0.f;
    for (int s0 = 0; s0 < active; s0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = s0 + u < active ? __ldcg(acc_base + (size_t)(s0 + u) * D) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < active) acc += v[u] * sm_f[row * kMaxSplits + s0 + u];
    }
    p.out[(token_heads + head) * D + d] = __float2bfloat16_rn(acc * sm_inv[row]);
  }
}

// ---------------------------------------------------------------------------
// Decode, cluster version: the splits of one (token, key/value head) are the CTAs of a
// thread-block cluster and merge through distributed shared memory, and inside a
// CTA every warp owns whole key tiles with an online softmax of its own.  Nothing on
// the way goes through global memory, no fence, no atomic: the dependent round trips
// are position -> block-table entry -> K/V tile, then two cluster barriers.
// ---------------------------------------------------------------------------
constexpr int kClusterWarps = 8;
constexpr int kClusterThreads = kClusterWarps * 32;
constexpr int kWarpTileKeys = D <= 64 ? 64 : 32;          // keys per warp tile
constexpr int kWarpTileElems = kWarpTileKeys * kRowStride;
constexpr int kMaxCluster = 8;

struct ClusterDecodeParams {
  const int* token_list;   // packed indices of the tokens to process, or null for 0 .. n-1
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;
  const int* seq_of_token;
  const int* positions;
  __nv_bfloat16* out;
  int* status;
  int num_heads, num_kv_heads, page_size, num_pages, table_width, window;
  float scale_log2;
};

// One warp copies keys [tile_begin, tile_begin + kWarpTileKeys) into its own buffers.
__device__ __forceinline__ bool warp_load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs,
                                                  const __nv_bfloat16* __restrict__ k_cache,
                                                  const __nv_bfloat16* __restrict__ v_cache,
                                                  const int* __restrict__ table, int kv_head, int num_kv_heads,
                                                  int page_size, int num_pages, int tile_begin, int k_end, int lane) {
  // The pages of the tile in one coalesced load (one round trip), handed out by shuffles;
  // a tile that spans more than 32 pages (pages of one or two tokens) looks each one up.
  const int first_logical = tile_begin / page_size;
  const int last_key = min(k_end, tile_begin + kWarpTileKeys) - 1;
  const int span = last_key >= tile_begin ? last_key / page_size - first_logical + 1 : 0;
  const bool by_shuffle = span <= 32;
  const int my_page = (by_shuffle && lane < span) ? table[first_logical + lane] : -1;
  bool bad = false;
#pragma unroll 4
  for (int idx = lane; idx < kWarpTileKeys * kChunks; idx += 32) {
    const int row = idx / kChunks;
    const int chunk = idx - row * kChunks;
    const int j = tile_begin + row;
    __nv_bfloat16* kd = ks + row * kRowStride + chunk * 8;
    __nv_bfloat16* vd = vs + row * kRowStride + chunk * 8;
    bool valid = j < k_end;
    const int logical = j / page_size;
    int page = __shfl_sync(0xffffffffu, my_page, valid ? (logical - first_logical) & 31 : 0);
    if (valid && !by_shuffle) page = table[logical];
    long long off = 0;
    if (valid) {
      if (page < 0 || page >= num_pages) {
        bad = true;
        valid = false;
      } else {
        off = (((long long)page * num_kv_heads + kv_head) * page_size + (j - logical * page_size)) * D + chunk * 8;
      }
    }
    if (valid) {
      cp_async16(kd, k_cache + off);
      cp_async16(vd, v_cache + off);
    } else {
      *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
    }
  }
  return bad;
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The barrier before a CTA leaves only keeps its shared memory alive until its peers have read
// it; nothing is handed over, so its arrival need not wait for the output stores before it.
__device__ __forceinline__ void cluster_leave() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// Read a float at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ float ld_peer(const float* local, uint32_t rank) {
  uint32_t addr = smem_u32(local), peer;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
  float v;
  asm("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer));   // ordered by the cluster barriers around it
  return v;
}

__global__ void __launch_bounds__(kClusterThreads) paged_decode_attention_cluster_kernel(ClusterDecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // Per warp one K and one V tile; after the key loop the same memory holds the warps'
  // partial results.  The CTA's merged result lives beside it, where peers read it.
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* cta_o = reinterpret_cast<float*>(smem_raw + (size_t)kClusterWarps * 2 * kWarpTileElems * 2);   // [16][D]
  float* cta_m = cta_o + 16 * D;   // [16]
  float* cta_l = cta_m + 16;       // [16]

  const int group = p.num_heads / p.num_kv_heads;
  const int head_blocks = (group + 15) / 16;
  const int kv_head = blockIdx.y / head_blocks;
  const int head_block = blockIdx.y - kv_head * head_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c2 = (lane & 3) * 2;
  const uint32_t rank = cluster_rank(), csize = cluster_size();

  pdl_launch_dependents();
  pdl_wait();
  const int t = p.token_list ? p.token_list[blockIdx.z] : blockIdx.z;
  const int pos = p.positions[t];
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int len = pos - lo + 1;
  int per = (len + (int)csize - 1) / (int)csize;
  per = (per + kWarpTileKeys - 1) / kWarpTileKeys * kWarpTileKeys;
  const int k_begin = min(pos + 1, lo + (int)rank * per);
  const int k_end = min(pos + 1, k_begin + per);
  const int* table = p.block_table + (size_t)p.seq_of_token[t] * p.table_width;

  const int first_head = kv_head * group + head_block * 16;
  const int rows_valid = min(16, group - head_block * 16);
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* base = p.q + ((size_t)t * p.num_heads + first_head) * D;
    load_q_fragments(qf, g < rows_valid ? base + g * D : nullptr, g + 8 < rows_valid ? base + (g + 8) * D : nullptr, lane);
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  __nv_bfloat16* ks = tiles + warp * 2 * kWarpTileElems;
  __nv_bfloat16* vs = ks + kWarpTileElems;
  const int tiles_total = (k_end - k_begin + kWarpTileKeys - 1) / kWarpTileKeys;
  bool bad = false;
  for (int tile = warp; tile < tiles_total; tile += kClusterWarps) {
    const int tile_key0 = k_begin + tile * kWarpTileKeys;
    __syncwarp();   // the previous round's reads of this warp's buffers are done
    bad |= warp_load_kv_tile(ks, vs, p.k_cache, p.v_cache, table, kv_head, p.num_kv_heads, p.page_size, p.num_pages,
                             tile_key0, k_end, lane);
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    constexpr int kNT = kWarpTileKeys / 8;   // score tiles of 8 keys
    float s[kNT][4];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < kNT / 2; ++np) {
        uint32_t b[4];
        const int key_row = np * 16 + (lane >> 4) * 8 + (lane & 7);
        const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b, ks + key_row * kRowStride + dim);
        mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
      }
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = tile_key0 + nt * 8 + c2 + (e & 1);
        const float v = j < k_end ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][e] = v;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m_run[r], tile_max[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int ks16 = 0; ks16 < kNT / 2; ++ks16) {
      uint32_t pa[4];
      float pv[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pv[h][e] = exp2f(s[2 * ks16 + h][e] - m_use[e >> 1]);
          l_run[e >> 1] += pv[h][e];
        }
      pa[0] = pack_bf16(pv[0][0], pv[0][1]);
      pa[1] = pack_bf16(pv[0][2], pv[0][3]);
      pa[2] = pack_bf16(pv[1][0], pv[1][1]);
      pa[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
      for (int dt = 0; dt < D / 16; ++dt) {
        uint32_t vb[4];
        const int key_row = ks16 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int dim = dt * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vs + key_row * kRowStride + dim);
        mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
      }
    }
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(p.status, kStatusBadPage);

  // Merge the warps of this CTA (the tile buffers are free after the barrier above).
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float* sm_o = reinterpret_cast<float*>(smem_raw);     // [warps][16][D]
  float* sm_m = sm_o + kClusterWarps * 16 * D;          // [warps][16]
  float* sm_l = sm_m + kClusterWarps * 16;              // [warps][16]
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    float* base = sm_o + (warp * 16) * D + i * 8 + c2;
    base[g * D] = o[i][0];
    base[g * D + 1] = o[i][1];
    base[(g + 8) * D] = o[i][2];
    base[(g + 8) * D + 1] = o[i][3];
  }
  if ((lane & 3) == 0) {
    sm_m[warp * 16 + g] = m_run[0];
    sm_m[warp * 16 + g + 8] = m_run[1];
    sm_l[warp * 16 + g] = l_run[0];
    sm_l[warp * 16 + g + 8] = l_run[1];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * D; e += kClusterThreads) {
    const int row = e / D, d = e - row * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kClusterWarps; ++w) m = fmaxf(m, sm_m[w * 16 + row]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kClusterWarps; ++w) {
      const float mw = sm_m[w * 16 + row];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
      l += sm_l[w * 16 + row] * f;
      acc += sm_o[(w * 16 + row) * D + d] * f;
    }
    cta_o[e] = acc;
    if (d == 0) {
      cta_m[row] = m;
      cta_l[row] = l;
    }
  }
  // Merge the CTAs of the cluster: each takes a slice of the (head, dim) elements.
  cluster_sync_all();
  const int total = rows_valid * D;
  const int slice = (total + (int)csize - 1) / (int)csize;
  const int e_begin = (int)rank * slice, e_end = min(total, e_begin + slice);
  const size_t token_heads = (size_t)t * p.num_heads;
  for (int e = e_begin + threadIdx.x; e < e_end; e += kClusterThreads) {
    const int row = e / D, d = e - row * D;
    // All remote loads first, so that they are in flight together; then the arithmetic.
    float mc[kMaxCluster], lc[kMaxCluster], oc[kMaxCluster];
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) {
      const bool live = c < (int)csize;
      mc[c] = live ? ld_peer(cta_m + row, c) : -INFINITY;
      lc[c] = live ? ld_peer(cta_l + row, c) : 0.f;
      oc[c] = live ? ld_peer(cta_o + e, c) : 0.f;
    }
    float m = -INFINITY;
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) m = fmaxf(m, mc[c]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) {
      const float f = mc[c] == -INFINITY ? 0.f : exp2f(mc[c] - m);
      l += lc[c] * f;
      acc += oc[c] * f;
    }
    p.out[(token_heads + first_head + row) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
  }
  cluster_leave();   // no CTA leaves while a peer may still read its shared memory
}

constexpr size_t kClusterTileSmem = (size_t)kClusterWarps * 2 * kWarpTileElems * sizeof(__nv_bfloat16);
constexpr size_t kClusterWarpMergeSmem = ((size_t)kClusterWarps * 16 * D + 2 * kClusterWarps * 16) * sizeof(float);
constexpr size_t kClusterSmem =
    (kClusterTileSmem > kClusterWarpMergeSmem ? kClusterTileSmem : kClusterWarpMergeSmem) + (16 * D + 32) * sizeof(float);
static_assert(kClusterTileSmem >= kClusterWarpMergeSmem, "the warps' partial results must fit into the tile buffers");

// ---------------------------------------------------------------------------
// Prefill (and any mixed batch): 64 query rows of one request per CTA
// ---------------------------------------------------------------------------
struct PrefillParams {
  const __nv_bfloat16* q;        // [tokens, heads, D]
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;        // [requests, table_width]
  const int4* tiles;             // per 128-row tile: request, first token (packed index), rows, position of the first row
  __nv_bfloat16* out;
  int* status;
  int num_heads, num_kv_heads, page_size, num_pages, table_width, window;
  float scale_log2;
};

__global__ void __launch_bounds__(kThreads) paged_prefill_attention_kernel(PrefillParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c2 = (lane & 3) * 2;
  // Heads vary fastest and tiles run from the last (most keys) to the first: the longest CTAs
  // start first, and the heads that share K and V run at the same time.
  const int head = blockIdx.x;
  const int kv_head = head / (p.num_heads / p.num_kv_heads);

  pdl_launch_dependents();
  pdl_wait();
  // The tile list holds 128-row tiles; a CTA takes one half of 64 rows.
  const int reversed = gridDim.y - 1 - blockIdx.y;
  const int4 tile_info = p.tiles[reversed >> 1];
  const int half_offset = (reversed & 1) * 64;
  const int request = tile_info.x, token0 = tile_info.y + half_offset, pos0 = tile_info.w + half_offset;
  const int rows = min(64, tile_info.z - half_offset);
  if (rows <= 0) return;
  const int* table = p.block_table + (size_t)request * p.table_width;
  const int last_pos = pos0 + rows - 1;
  const int k_begin = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int k_end = last_pos + 1;

  // This thread's two rows: positions, or -1 for rows beyond the tile.
  const int row_lo = warp * 16 + g, row_hi = row_lo + 8;
  const int pos_lo = row_lo < rows ? pos0 + row_lo : -1;
  const int pos_hi = row_hi < rows ? pos0 + row_hi : -1;
  const int warp_last_pos = min(last_pos, pos0 + warp * 16 + 15);
  const bool warp_has_rows = warp * 16 < rows;
  const int warp_first_key =
      (p.window > 0) ? max(0, pos0 + warp * 16 - p.window + 1) : 0;

  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* base = p.q + ((size_t)token0 * p.num_heads + head) * D;
    const size_t row_stride = (size_t)p.num_heads * D;
    load_q_fragments(qf, pos_lo >= 0 ? base + row_lo * row_stride : nullptr,
                     pos_hi >= 0 ? base + row_hi * row_stride : nullptr, lane);
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int tiles = (k_end - k_begin + kTileKeys - 1) / kTileKeys;
  bool bad = false;
#pragma unroll
  for (int stage = 0; stage < kPrefillStages - 1; ++stage) {
    if (stage < tiles) {
      __nv_bfloat16* kn = smem + stage * 2 * kTileElems;
      bad |= load_kv_tile(kn, kn + kTileElems, p.k_cache, p.v_cache, table, kv_head, p.num_kv_heads, p.page_size,
                          p.num_pages, k_begin + stage * kTileKeys, k_end);
    }
    cp_async_commit();
  }
  for (int tile = 0; tile < tiles; ++tile) {
    cp_async_wait<kPrefillStages - 2>();
    __syncthreads();   // tile `tile` has landed, and every warp is done with the stage refilled below
    {
      const int next = tile + kPrefillStages - 1;
      if (next < tiles) {
        __nv_bfloat16* kn = smem + (next % kPrefillStages) * 2 * kTileElems;
        bad |= load_kv_tile(kn, kn + kTileElems, p.k_cache, p.v_cache, table, kv_head, p.num_kv_heads, p.page_size,
                            p.num_pages, k_begin + next * kTileKeys, k_end);
      }
      cp_async_commit();
    }
    __nv_bfloat16* ks = smem + (tile % kPrefillStages) * 2 * kTileElems;
    __nv_bfloat16* vs = ks + kTileElems;
    const int tile_key0 = k_begin + tile * kTileKeys;
    // Skip tiles that no row of this warp can see (after its last row, or before its window).
    if (warp_has_rows && tile_key0 <= warp_last_pos && tile_key0 + kTileKeys > warp_first_key) {
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b[4];
          const int key_row = np * 16 + (lane >> 4) * 8 + (lane & 7);
          const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(b, ks + key_row * kRowStride + dim);
          mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
        }
      }
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = tile_key0 + nt * 8 + c2 + (e & 1);
          const int pos = (e >> 1) ? pos_hi : pos_lo;
          const bool visible = j <= pos && (p.window <= 0 || j > pos - p.window);
          const float v = visible ? s[nt][e] * p.scale_log2 : -INFINITY;
          s[nt][e] = v;
          tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(m_run[r], tile_max[r]);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int ks16 = 0; ks16 < 4; ++ks16) {
        uint32_t pa[4];
        float pv[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pv[h][e] = exp2f(s[2 * ks16 + h][e] - m_use[e >> 1]);
            l_run[e >> 1] += pv[h][e];
          }
        pa[0] = pack_bf16(pv[0][0], pv[0][1]);
        pa[1] = pack_bf16(pv[0][2], pv[0][3]);
        pa[2] = pack_bf16(pv[1][0], pv[1][1]);
        pa[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
        for (int dt = 0; dt < D / 16; ++dt) {
          uint32_t vb[4];
          const int key_row = ks16 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int dim = dt * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(vb, vs + key_row * kRowStride + dim);
          mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
          mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(p.status, kStatusBadPage);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv_lo = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv_hi = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  __nv_bfloat16* out_base = p.out + ((size_t)token0 * p.num_heads + head) * D;
  const size_t row_stride = (size_t)p.num_heads * D;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    if (pos_lo >= 0)
      *reinterpret_cast<uint32_t*>(out_base + row_lo * row_stride + i * 8 + c2) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
    if (pos_hi >= 0)
      *reinterpret_cast<uint32_t*>(out_base + row_hi * row_stride + i * 8 + c2) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

constexpr size_t kAttentionSmem = kPrefillStages * 2 * kTileElems * sizeof(__nv_bfloat16);   // stages of K and V
constexpr size_t kDecodeStageSmem = kDecodeStages * 2 * kTileElems * sizeof(__nv_bfloat16);
constexpr size_t kWarpMergeSmem = (4 * 16 * D + 2 * 4 * 16) * sizeof(float);
constexpr size_t kSplitMergeSmem = (2 * 16 * kMaxSplits + 16) * sizeof(float);
constexpr size_t kMergeSmem = kWarpMergeSmem > kSplitMergeSmem ? kWarpMergeSmem : kSplitMergeSmem;
constexpr size_t kDecodeSmem = kDecodeStageSmem > kMergeSmem ? kDecodeStageSmem : kMergeSmem;

}  // namespace einf

using namespace einf;

extern "C" int einf_attention_bf16_head_size() { return D; }

// Scratch a decode launch needs, in bytes, for `tokens` tokens and `splits` splits:
// partial outputs, (maximum, sum) pairs, and the arrival counters.
extern "C" long long einf_decode_workspace_bytes(int tokens, int num_heads, int num_kv_heads, int splits) {
  const long long slots = (long long)tokens * num_heads * splits;
  const int head_blocks = (num_heads / num_kv_heads + 15) / 16;
  return slots * D * 4 + slots * 2 * 4 + (long long)tokens * num_kv_heads * head_blocks * 4;
}

extern "C" int einf_paged_decode_attention(const void* q, const void* k_cache, const void* v_cache,
                                           const int* block_table, const int* seq_of_token, const int* positions,
                                           void* out, float* ws_acc, float* ws_ml, int* counters, int num_tokens,
                                           int num_heads, int num_kv_heads, int page_size, int num_pages,
                                           int table_width, float scale, int window, int num_splits, int* status,
                                           cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (num_splits < 1 || num_splits > kMaxSplits) return (int)cudaErrorInvalidValue;
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q;
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table;
  p.seq_of_token = seq_of_token;
  p.positions = positions;
  p.out = (__nv_bfloat16*)out;
  p.ws_acc = ws_acc;
  p.ws_ml = ws_ml;
  p.counters = counters;
  p.status = status;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.table_width = table_width;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int head_blocks = (num_heads / num_kv_heads + 15) / 16;
  if (kDecodeSmem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kDecodeSmem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(num_splits, num_kv_heads * head_blocks, num_tokens);
  return (int)launch_pdl(paged_decode_attention_kernel, grid, kThreads, kDecodeSmem, stream, p);
}

// cluster: CTAs that share one (token, key/value head): 1, 2, 4 or 8.
// token_list: packed indices of the num_tokens tokens to process (null: tokens 0 .. num_tokens-1).
extern "C" int einf_paged_decode_attention_cluster(const void* q, const void* k_cache, const void* v_cache,
                                                   const int* block_table, const int* seq_of_token,
                                                   const int* positions, const int* token_list, void* out,
                                                   int num_tokens, int num_heads,
                                                   int num_kv_heads, int page_size, int num_pages, int table_width,
                                                   float scale, int window, int cluster, int* status,
                                                   cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return (int)cudaErrorInvalidValue;
  ClusterDecodeParams p;
  p.token_list = token_list;
  p.q = (const __nv_bfloat16*)q;
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table;
  p.seq_of_token = seq_of_token;
  p.positions = positions;
  p.out = (__nv_bfloat16*)out;
  p.status = status;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.table_width = table_width;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int head_blocks = (num_heads / num_kv_heads + 15) / 16;
  cudaError_t e = cudaFuncSetAttribute(paged_decode_attention_cluster_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kClusterSmem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(cluster, num_kv_heads * head_blocks, num_tokens);
  config.blockDim = dim3(kClusterThreads);
  config.dynamicSmemBytes = kClusterSmem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = cluster;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&config, paged_decode_attention_cluster_kernel, p);
}

extern "C" int einf_paged_prefill_attention(const void* q, const void* k_cache, const void* v_cache,
                                            const int* block_table, const int* tiles, int num_tiles, void* out,
                                            int num_heads, int num_kv_heads, int page_size, int num_pages,
                                            int table_width, float scale, int window, int* status,
                                            cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  PrefillParams p;
  p.q = (const __nv_bfloat16*)q;
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table;
  p.tiles = (const int4*)tiles;
  p.out = (__nv_bfloat16*)out;
  p.status = status;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.table_width = table_width;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (kAttentionSmem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kAttentionSmem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(num_heads, 2 * num_tiles);
  return (int)launch_pdl(paged_prefill_attention_kernel, grid, kThreads, kAttentionSmem, stream, p);
}
