// out[T, N] = X[T, K] . W[N, K]^T (+ bias) in bfloat16 on the fifth-generation tensor
// cores: TMA loads, tcgen05.mma with the accumulator in tensor memory, split-K.
//
// The weight matrix is the 128-row operand of the MMA and the tokens are its N
// dimension (16 to 256 wide), so a decode step with a handful of tokens still
// issues full-rate instructions and the kernel is what it should be there: a
// stream of W through shared memory at HBM speed.  One CTA owns one
// (128 weight rows) x (token tile) x (K range) block:
//
//   warp 0   producer: one lane issues the TMA loads of the W and X tiles of each
//            64-wide K block into a ring of shared-memory stages (128-byte swizzle);
//            the W tiles of the first stages are requested before the wait on the
//            previous kernel (weights do not depend on it), the X tiles after it
//   warp 1   allocates tensor memory; one lane issues four tcgen05.mma (K = 16 each)
//            per stage and commits the stage back to the producer
//   warps 2-5 epilogue: tcgen05.ld the accumulator (lane = weight row, column =
//            token), add the bias, store transposed into out[token, row]
//
// With split-K the CTAs of one output block each take a K range and write 32-bit
// partial sums [split, T, N]; the consumer (the norm, rotary or activation kernel
// that follows) adds them up, so no atomics and no extra pass are needed and the
// result does not depend on timing.  Every wait on a barrier is bounded; a wait
// that gives up sets a bit in the status word and the CTA drains and leaves.
//
// No multicast anywhere: every CTA fetches its own tiles.
// (replaces the library products of the reference: F.linear at
// src/einf/executors/torch/packed_qkv.py:148 and qwen.py:207-208,489,773.)
#include <cuda.h>

#include "common.cuh"

namespace einf {

constexpr int kBlockW = 128;    // weight rows per CTA (UMMA M)
constexpr int kBlockK = 64;     // K per stage: 64 bf16 = 128 bytes = one swizzle span
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kWTileBytes = kBlockW * kBlockK * 2;   // 16 KB
constexpr int kMaxPolls = 1 << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false (and a status bit) if the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
  for (int poll = 0; poll < kMaxPolls; ++poll) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  atomicOr(status, kStatusWaitExpired);
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128
// bytes, eight rows per 1024-byte group (stride byte offset 1024), descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
  uint64_t desc = (addr >> 4) & 0x3FFFu;
  desc |= (uint64_t)1 << 16;              // leading byte offset: unused for swizzled K-major, 1 by convention
  desc |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset
  desc |= (uint64_t)1 << 46;              // version
  desc |= (uint64_t)2 << 61;              // 128-byte swizzle
  return desc;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

struct GemmParams {
  void* out;            // [T, N] (out_dtype), or 32-bit partial sums [splits, T, N] when splits > 1
  const float* bias;    // [N] or null (with split-K it is added by split 0)
  int* status;
  int tokens, n, k;
  int token_tile;       // BN: 16 .. 256, a multiple of 16
  int stages;
  int kblocks_per_split;
  int out_dtype;        // kFloat32 | kBFloat16 (ignored with split-K)
  long long ldo;        // row stride of out in elements
};

__global__ void __launch_bounds__(kGemmThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // Stage ring first (1024-byte aligned tiles), barriers after it.
  const uint32_t smem_base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  const int x_tile_bytes = p.token_tile * kBlockK * 2;
  const int stage_bytes = kWTileBytes + x_tile_bytes;
  const uint32_t bar_base = smem_base + p.stages * stage_bytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  const uint32_t accum_bar = bar_base + 8u * (2 * kMaxStages);
  const uint32_t tmem_holder = bar_base + 8u * (2 * kMaxStages + 1);
  unsigned char* generic_base = smem_raw + (smem_base - smem_addr(smem_raw));
  volatile uint32_t* tmem_holder_ptr =
      reinterpret_cast<volatile uint32_t*>(generic_base + p.stages * stage_bytes + 8 * (2 * kMaxStages + 1));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kBlockW;
  const int t0 = blockIdx.y * p.token_tile;
  const int split = blockIdx.z, splits = gridDim.z;
  const int total_kblocks = (p.k + kBlockK - 1) / kBlockK;
  const int kb_begin = split * p.kblocks_per_split;
  const int kb_end = min(total_kblocks, kb_begin + p.kblocks_per_split);
  const int num_kblocks = kb_end - kb_begin;   // >= 1 by construction of the grid

  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)p.token_tile) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_holder), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder_ptr;
  // The next kernel may start its own prologue now (it waits for this grid's completion before it
  // touches anything this grid writes).  Not earlier: a kernel that is resident holds its tensor
  // memory, and this one must have its own before a later one can take columns on this SM.
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      const int first = min(p.stages, num_kblocks);
      for (int i = 0; i < first; ++i) {   // weights do not depend on the kernel before this one
        mbar_expect_tx(full_bar(i), stage_bytes);
        tma_load_2d(smem_base + i * stage_bytes, &map_w, (kb_begin + i) * kBlockK, n0, full_bar(i));
      }
      pdl_wait();
      for (int i = 0; i < first; ++i)
        tma_load_2d(smem_base + i * stage_bytes + kWTileBytes, &map_x, (kb_begin + i) * kBlockK, t0, full_bar(i));
      bool ok = true;
      for (int i = first; i < num_kblocks && ok; ++i) {
        const int s = i % p.stages;
        ok = mbar_wait(empty_bar(s), ((i / p.stages) & 1) ^ 1, p.status);
        if (!ok) break;
        mbar_expect_tx(full_bar(s), stage_bytes);
        tma_load_2d(smem_base + s * stage_bytes, &map_w, (kb_begin + i) * kBlockK, n0, full_bar(s));
        tma_load_2d(smem_base + s * stage_bytes + kWTileBytes, &map_x, (kb_begin + i) * kBlockK, t0, full_bar(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      // Instruction descriptor: D = F32, A = B = BF16, both K-major, N = token tile, M = 128.
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.token_tile >> 3) << 17) |
                             ((uint32_t)(kBlockW >> 4) << 24);
      bool ok = true;
      pdl_wait();   // bounded waits start once only this kernel's own progress is waited for
      for (int i = 0; i < num_kblocks && ok; ++i) {
        const int s = i % p.stages;
        ok = mbar_wait(full_bar(s), (i / p.stages) & 1, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // descriptors once per stage, then one add on the low word per MMA (the address field is
        // in units of 16 bytes and cannot overflow: shared memory ends below 256 KB)
        const uint64_t w_desc = umma_desc(smem_base + s * stage_bytes);
        const uint64_t x_desc = umma_desc(smem_base + s * stage_bytes + kWTileBytes);
#pragma unroll
        for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
          const uint32_t step = (uint32_t)(kk * kUmmaK * 2) >> 4;
          umma_bf16(tmem_base, (w_desc & 0xFFFFFFFF00000000ull) | (uint32_t)((uint32_t)w_desc + step),
                    (x_desc & 0xFFFFFFFF00000000ull) | (uint32_t)((uint32_t)x_desc + step), idesc,
                    (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
      }
      umma_commit(accum_bar);        // the accumulator is complete once every MMA is
    }
  } else {
    // ---- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) .. + 31 ----
    pdl_wait();   // as above
    const bool ok = mbar_wait(accum_bar, 0, p.status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const int lane_base = (warp & 3) * 32;
      const int row = n0 + lane_base + lane;         // weight row = output column
      const bool row_ok = row < p.n;
      const bool partial = splits > 1;
      const float bias = (p.bias && row_ok && split == 0) ? p.bias[row] : 0.f;
      float* out_f = partial ? reinterpret_cast<float*>(p.out) + (size_t)split * p.tokens * p.ldo
                             : reinterpret_cast<float*>(p.out);
      __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(p.out);
      const bool as_float = partial || p.out_dtype == kFloat32;
      // One store per (token, weight row), 128 bytes per warp.  Kept to a pointer bump and a store
      // per column: with an index computation and a bounds test per element this loop, which
      // one warp per 32 rows runs alone, took longer than the product itself at 64 tokens.
      for (int col0 = 0; col0 < p.token_tile; col0 += 16) {
        const int t_first = t0 + col0;
        if (t_first >= p.tokens) break;              // uniform across the warp
        uint32_t v[16];
        tmem_load16(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)col0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row_ok) {
          const int valid = min(16, p.tokens - t_first);
          if (as_float) {
            float* dst = out_f + (size_t)t_first * p.ldo + row;
            if (valid == 16) {
#pragma unroll
              for (int c = 0; c < 16; ++c, dst += p.ldo) *dst = __uint_as_float(v[c]) + bias;
            } else {
#pragma unroll
              for (int c = 0; c < 16; ++c, dst += p.ldo)
                if (c < valid) *dst = __uint_as_float(v[c]) + bias;
            }
          } else {
            __nv_bfloat16* dst = out_h + (size_t)t_first * p.ldo + row;
#pragma unroll
            for (int c = 0; c < 16; ++c, dst += p.ldo)
              if (c < valid) *dst = __float2bfloat16_rn(__uint_as_float(v[c]) + bias);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

}  // namespace einf

using namespace einf;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return (EncodeTiledFn) nullptr;
    return (EncodeTiledFn)ptr;
  }();
  return fn;
}

// A [rows, k] bfloat16 matrix with unit stride along k, as a TMA map with a (64 x box_rows) box.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long k, long long row_stride_elems,
                    int box_rows) {
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
  cuuint32_t element_strides[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                      element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Shared memory the kernel needs for a token tile and a number of stages.
static size_t smem_bytes(int token_tile, int stages) {
  return 1024 + (size_t)stages * (kWTileBytes + token_tile * kBlockK * 2) + 8 * (2 * kMaxStages + 2);
}

// The token tile the launcher picks for `tokens` rows: the smallest multiple of 16 that holds
// them, 256 at most.
extern "C" int einf_gemm_tcgen05_token_tile(int tokens) {
  int tile = (tokens + 15) / 16 * 16;
  return tile < 16 ? 16 : (tile > 256 ? 256 : tile);
}

// x: [tokens, k] bfloat16, row stride ldx; w: [n, k] bfloat16 contiguous; out as GemmParams says.
// k must be a multiple of 8 and both base pointers 16-byte aligned (TMA rules).
// splits > 1: out holds 32-bit partial sums [splits, tokens, n] (ldo = n).
extern "C" int einf_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int out_dtype,
                                 int tokens, int n, int k, long long ldx, long long ldo, int splits, int* status,
                                 cudaStream_t stream) {
  if (tokens == 0 || n == 0) return 0;
  if (k % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
  const int total_kblocks = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > total_kblocks) splits = total_kblocks;
  int per_split = (total_kblocks + splits - 1) / splits;
  splits = (total_kblocks + per_split - 1) / per_split;   // no empty split
  const int token_tile = einf_gemm_tcgen05_token_tile(tokens);
  // Two CTAs per SM when the stages allow it (about 110 KB each): one streams while the
  // other runs its epilogue.  Never fewer than three stages for a long K range.
  int stages = per_split < kMaxStages ? per_split : kMaxStages;
  while (stages > 3 && smem_bytes(token_tile, stages) > 110 * 1024) --stages;
  while (stages > 1 && smem_bytes(token_tile, stages) > 200 * 1024) --stages;
  CUtensorMap map_w, map_x;
  int rc = make_map(&map_w, w, n, k, k, kBlockW);
  if (rc) return rc;
  rc = make_map(&map_x, x, tokens, k, ldx, token_tile);
  if (rc) return rc;
  GemmParams p;
  p.out = out;
  p.bias = bias;
  p.status = status;
  p.tokens = tokens;
  p.n = n;
  p.k = k;
  p.token_tile = token_tile;
  p.stages = stages;
  p.kblocks_per_split = per_split;
  p.out_dtype = out_dtype;
  p.ldo = ldo;
  const size_t smem = smem_bytes(token_tile, stages);
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((n + kBlockW - 1) / kBlockW, (tokens + token_tile - 1) / token_tile, splits);
  return (int)launch_pdl(gemm_tcgen05_kernel, grid, dim3(kGemmThreads), smem, stream, map_w, map_x, p);
}

// Number of splits the launcher will really use for a request of `splits`.
extern "C" int einf_gemm_tcgen05_splits(int k, int splits) {
  const int total_kblocks = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > total_kblocks) splits = total_kblocks;
  const int per_split = (total_kblocks + splits - 1) / splits;
  return (total_kblocks + per_split - 1) / per_split;
}
