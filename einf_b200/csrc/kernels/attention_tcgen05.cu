// Causal paged attention for prompt portions on the fifth-generation tensor cores,
// compiled for one head size (-DHEAD_SIZE=64 or 128).
//
// On sm_100a the warp-level mma.sync path tops out near 90 TFLOP/s for the whole GPU
// (measured: its HMMA sub-pipe is 95 % busy at that rate), so attention over a long
// prompt needs tcgen05.  One CTA owns 128 query rows of one (request, query head) and
// walks the request's keys 128 at a time:
//
//   warp 0    K producer: TMA-loads the Q tile once and, per key tile, the pages the block
//             table names (one TMA box per page and 64-wide slice of the head, or one box
//             per slice where the pages follow one another) into a ring of K tiles
//             (128-byte swizzle)
//   warp 10   V producer: the same for the ring of V tiles
//   warp 1    allocates tensor memory; one lane issues S = Q K^T (both operands K-major
//             from shared memory)
//   warp 11   one lane issues O += P V (P K-major from shared memory, V as the MN-major
//             operand straight from its [key, dim] tile), O accumulating in tensor memory
//   warps 2-9 softmax: two warpgroups that take the key tiles in turn (even tiles, odd
//             tiles), each with its own S, P, O accumulator, reference and sum, like two
//             splits of the keys inside one CTA.  Query row r = tensor-memory lane r belongs
//             to one thread of each: it reads its row of S with tcgen05.ld, masks (causal,
//             window), keeps the sum in 32-bit and writes P as bfloat16 where the second
//             product reads it (shared memory in the swizzled layout, or tensor memory).
//
// A tile's softmax is a chain of steps that each wait for something (S from the tensor
// core, tensor-memory loads, the exponentials' unit), so one group of threads that does
// all of them in order leaves every unit idle most of the time; two warpgroups in
// different phases fill each other's gaps.  (Measured with both warpgroups on the same
// tile, half a row per thread: 2,780 cycles a tile at head size 64, of which the
// exponentials, at 16 a cycle, need 1,024; as it stands about 1,650, of which the two
// warpgroups' exponentials, which share the one unit, take 900.)  The same holds for
// the threads that feed them: a wait on a barrier that is long complete, a commit or a TMA
// request each cost a thread one to three hundred cycles, so one producer and one MMA
// issuer for both operands were chains of 2,500 and 1,900 cycles a tile; with the work
// split by operand (K and the first product, V and the second) each chain is half as long.
// For the same reason S is handed back as soon as its last columns are in registers.  At
// head size 64, where tensor memory has columns to spare, P goes to the second product
// through tensor memory (tcgen05.st, then the MMA form that takes A from there) and not
// through shared memory.
//
// The accumulator stays in tensor memory across tiles, scaled, like the probabilities and
// their sum, by a reference m: the maximum of the row's first tile, and after that whatever
// it was, for as long as it serves.  A tile is one walk over S that looks at no maximum:
// exponent against the reference, sum, round, store, two columns to an instruction where
// there is one that takes two.  Only when a row's sum over a tile comes out above 2^40
// (scores far above the reference; an overflow is such a sum too) does the warp walk the
// tile for its maximum, rescale its rows of O and their sums to it and do the tile again.
// bfloat16 and 32-bit keep their relative precision over that range, so the result does
// not depend on where the reference stands.  The two warpgroups' results, and then those
// of the CTAs of a cluster that share a row tile, are merged once at the end.
// Every barrier wait is bounded and reports through the status word.
// Page sizes must be 8, 16, 32, 64 or 128 (a page is a TMA box and a whole number of
// swizzle groups); other sizes use the mma.sync kernel of attention_bf16.cu.
// (maths: src/einf/executors/torch/ops/csrc/flash_attention_cuda.cu:11-219 of the reference.)
#include <cuda.h>

#include <type_traits>

#include "common.cuh"

#ifndef HEAD_SIZE
#define HEAD_SIZE 64
#endif

namespace einf {

constexpr int D = HEAD_SIZE;
static_assert(D == 64 || D == 128, "the tcgen05 attention kernel is built for head sizes 64 and 128");
constexpr int kDBlocks = D / 64;               // 64-wide slices of the head (one swizzle span each)
constexpr int kBlockQ = 128;                   // query rows per CTA = tensor-memory lanes
constexpr int kBlockKV = 128;                  // keys per tile
constexpr int kSliceBytes = 128 * 64 * 2;      // a [128 rows x 64] bf16 slice: 16 KB
constexpr int kStages = D == 64 ? 4 : 2;       // K tiles in flight, and V tiles in flight (a ring each)
// At head size 64 tensor memory has 128 columns to spare, and P goes to the second product through
// them (one 64-column tile of packed bfloat16 per warpgroup) instead of through shared memory, whose
// bandwidth is what this kernel runs out of: per key tile the tensor core reads Q, K, P and V from
// it, the softmax warps write P and TMA writes K and V (144 KB at head size 64; 80 KB without P).
constexpr bool kPInTmem = D == 64;
constexpr int kPBuffers = 1;                   // P tiles per warpgroup (two, in shared memory at head size 64, changed nothing: 253 against 254 us at 8,192 tokens)
constexpr int kAttnThreads = 384;              // K producer, first-product issuer, two softmax warpgroups of four warps, V producer, second-product issuer
constexpr int kPolls = 1 << 22;
constexpr float kSumLimit = 1099511627776.f;   // 2^40: a row's sum of probabilities over a tile above which the row's reference moves
constexpr float kLastLimit = 40.f;             // the same as an exponent, for a tile's last 32 scores
// At head size 128 the first product is eight MMAs and a warpgroup waits for its next S even when
// it hands S back after the last exponentials; there it hands it back before them (8,192 tokens at
// 28 heads: 529 -> 507 us).  At head size 64 S comes in time either way and the extra look at the
// last scores costs more than it gains (221 -> 225 us).
constexpr bool kReleaseBeforeLastExps = D == 128;

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr int kQOff = 0;
constexpr int kKOff = kQOff + kDBlocks * kSliceBytes;
constexpr int kVOff = kKOff + kStages * kDBlocks * kSliceBytes;
constexpr int kPOff = kVOff + kStages * kDBlocks * kSliceBytes;
constexpr int kPBytes = 2 * kSliceBytes;                  // one P tile: two 64-key slices
constexpr int kBarOff = kPOff + (kPInTmem ? 0 : 2 * kPBuffers * kPBytes);
constexpr int kNumBars = 1 + 4 * kStages + 6 + 2 * kPBuffers;   // q_full, k_full[], k_empty[], v_full[], v_empty[], s_full[2], p_full[2], s_free[2], o_done[2][kPBuffers]
constexpr int kXchgOff = kBarOff + 8 * kNumBars + 16;    // maximum and sum of every row, per warpgroup
constexpr int kSmemBytes = kXchgOff + 2 * 2 * 128 * 4;   // D = 64: 146 KB; D = 128: 224 KB; one CTA per SM (more than half of its shared memory, and all 512 tensor-memory columns)
static_assert(2 * kSmemBytes > 228 * 1024, "two CTAs on an SM would wait for each other's tensor memory");
static_assert(kSmemBytes <= 227 * 1024, "shared memory of the tcgen05 attention kernel exceeds an SM");
constexpr int kTmemCols = 512;                            // S: 2 x 128 columns, O: 2 x D columns, at head size 64 P: 2 x 64 columns
// what the two warpgroups exchange at the end (half a row of O each way, padded) fits the K and V rings
static_assert(2 * 128 * (D / 2 + 1) * 4 <= kPOff - kKOff, "the final exchange needs the K and V rings");
constexpr int kShareOff = kKOff + 2 * 128 * (D / 2 + 1) * 4;   // a CTA's share for the cluster merge, after the exchange area
static_assert(kShareOff % 16 == 0 && kShareOff + (128 * (D + 1) + 2 * 128) * 4 <= kBarOff, "the share for the cluster merge needs the K, V and P tiles");

__device__ __forceinline__ uint32_t saddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, int* status) {
  for (int poll = 0; poll < kPolls; ++poll) {
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
// bar_wait for a phase that has most likely completed already: asked first without suspending
// (a try_wait that finds its phase complete still took some 200 cycles).
__device__ __forceinline__ bool bar_wait_likely_done(uint32_t bar, uint32_t parity, int* status);
// True if the phase with this parity has completed; never suspends the thread.
__device__ __forceinline__ bool bar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool bar_wait_likely_done(uint32_t bar, uint32_t parity, int* status) {
  return bar_test(bar, parity) || bar_wait(bar, parity, status);
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, eight-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  uint64_t desc = (addr >> 4) & 0x3FFFu;
  desc |= (uint64_t)1 << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// MN-major operand (V as [key, dim]: the dims of a key are contiguous), 128-byte swizzle:
// 64 dims per 128-byte row, eight keys per 1024-byte group (stride byte offset), 64-dim
// slices one 16 KB slice apart (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  uint64_t desc = (addr >> 4) & 0x3FFFu;
  desc |= (uint64_t)(kSliceBytes >> 4) << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// The descriptor of the same kind of tile `bytes` further on in shared memory (a multiple of 16;
// the 14-bit address field cannot overflow: shared memory ends below 256 KB): one add on the low
// word.  The one thread that issues the MMAs ran about 70 cycles per MMA while it built both
// descriptors from an address each time.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
  return (desc & 0xFFFFFFFF00000000ull) | (uint32_t)((uint32_t)desc + (bytes >> 4));
}
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory (lane = row, two 16-bit elements of K per column).
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The registers of earlier tmem_ld32 calls are valid after this.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 columns of this thread's lane; valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
        "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
      : "r"(taddr)
      : "memory");
}
// The registers of earlier tensor-memory loads are valid after this, and the compiler is told
// that v changes here: with a later load in flight during the arithmetic on an earlier one,
// nothing else keeps a use of v from moving above the wait.
__device__ __forceinline__ void tmem_ld_wait32(float* v) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]),
        "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]), "+f"(v[16]),
        "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]), "+f"(v[22]), "+f"(v[23]), "+f"(v[24]),
        "+f"(v[25]), "+f"(v[26]), "+f"(v[27]), "+f"(v[28]), "+f"(v[29]), "+f"(v[30]), "+f"(v[31])
      :
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
// The tensor-memory stores of this thread are complete after this.
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The 256 softmax threads meet (the producer and MMA warps do not take part).
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
// The barrier before a CTA leaves, which only keeps its shared memory alive until its peers have
// read it: nothing is handed over, so the arrival need not wait for this CTA's stores to global
// memory to become visible (a releasing arrival after the output stores cost over a microsecond).
__device__ __forceinline__ void cluster_leave() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// Read a float at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ float ld_peer(const float* local, uint32_t rank) {
  uint32_t addr = saddr(local), peer;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
  float v;
  asm("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer));   // ordered by the cluster barriers around it
  return v;
}

// Reduce 16 values per lane over the 32 lanes of a warp in 16 shuffles instead of 80: each
// butterfly step exchanges half of the values a lane still holds, so a lane ends up with
// one value, the reduction for index lane / 2.  v is clobbered.
template <bool kMax>
__device__ __forceinline__ float warp_reduce16(float* v, int lane) {
  auto op = [](float a, float b) { return kMax ? fmaxf(a, b) : a + b; };
#pragma unroll
  for (int width = 8; width >= 1; width >>= 1) {
    const bool upper = (lane & (2 * width)) != 0;
#pragma unroll
    for (int k = 0; k < width; ++k) {
      const float send = upper ? v[k] : v[k + width];
      const float keep = upper ? v[k + width] : v[k];
      v[k] = op(keep, __shfl_xor_sync(0xffffffffu, send, 2 * width));
    }
  }
  return op(v[0], __shfl_xor_sync(0xffffffffu, v[0], 1));
}

struct TcAttentionParams {
  const int* block_table;   // [requests, table_width]
  const int4* tiles;        // per 128-row query tile: request, first token (packed), rows, position of the first row
  __nv_bfloat16* out;       // [tokens, heads, D]
  int* status;
  int num_heads, num_kv_heads, page_size, num_pages, table_width, window;
  float scale_log2;
};

__global__ void __launch_bounds__(kAttnThreads, 1)
paged_prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap run_k,
                                       const __grid_constant__ CUtensorMap run_v, TcAttentionParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // The tiles need 1024-byte alignment (one swizzle group); the declaration above asks for it.
  const uint32_t base = saddr(smem_raw);
  unsigned char* gbase = smem_raw;
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicOr(p.status, kStatusWaitExpired);
    return;
  }
  const uint32_t bars = base + kBarOff;
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (1 + kStages + s); };
  auto v_full = [&](int s) { return bars + 8u * (1 + 2 * kStages + s); };
  auto v_empty = [&](int s) { return bars + 8u * (1 + 3 * kStages + s); };
  auto s_full = [&](int g) { return bars + 8u * (1 + 4 * kStages + g); };
  auto p_full = [&](int g) { return bars + 8u * (1 + 4 * kStages + 2 + g); };
  auto s_free = [&](int g) { return bars + 8u * (1 + 4 * kStages + 4 + g); };
  // the second product of a warpgroup's tile number j (its own count) reports to o_done(g, j % kPBuffers)
  auto o_done = [&](int g, int b) { return bars + 8u * (1 + 4 * kStages + 6 + g * kPBuffers + b); };
  const uint32_t tmem_holder = bars + 8 * kNumBars;
  volatile uint32_t* tmem_holder_ptr = reinterpret_cast<volatile uint32_t*>(gbase + kBarOff + 8 * kNumBars);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heads vary fastest and tiles run from the last (most keys) to the first: the longest CTAs
  // start first, and the heads that share K and V run at the same time.
  const int head = blockIdx.x;
  const int kv_head = head / (p.num_heads / p.num_kv_heads);
  const int4 tile_info = p.tiles[gridDim.y - 1 - blockIdx.y];
  const int request = tile_info.x, token0 = tile_info.y, rows = tile_info.z, pos0 = tile_info.w;
  const int* table = p.block_table + (size_t)request * p.table_width;
  const int last_pos = pos0 + rows - 1;
  int k_begin = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  k_begin = k_begin / p.page_size * p.page_size;          // tiles start on a page edge
  int k_end = last_pos + 1;
  // A prompt portion of a few row tiles does not fill the GPU (four tiles of twelve heads are 48
  // CTAs with a dozen key tiles each): the CTAs of a cluster (grid z) then share a row tile, each
  // with a contiguous run of its key tiles, and merge their partial results at the end through
  // distributed shared memory, like the splits of a decode step.
  const uint32_t rank = cluster_rank(), csize = cluster_size();
  if (csize > 1) {
    const int tiles_total = (k_end - k_begin + kBlockKV - 1) / kBlockKV;
    const int per = (tiles_total + (int)csize - 1) / (int)csize * kBlockKV;
    k_begin = min(k_end, k_begin + (int)rank * per);
    k_end = min(k_end, k_begin + per);
  }
  const int num_tiles = (k_end - k_begin + kBlockKV - 1) / kBlockKV;
  const int pages_per_tile = kBlockKV / p.page_size;
  const uint32_t page_bytes = (uint32_t)p.page_size * 128u;   // one page of one 64-wide slice

  if (threadIdx.x == 0) {
    bar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      bar_init(k_full(s), 1);
      bar_init(k_empty(s), 1);
      bar_init(v_full(s), 1);
      bar_init(v_empty(s), 1);
    }
    for (int g = 0; g < 2; ++g) {
      bar_init(s_full(g), 1);
      bar_init(p_full(g), 128);
      for (int b = 0; b < kPBuffers; ++b) bar_init(o_done(g, b), 1);
      bar_init(s_free(g), 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_holder), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder_ptr;
  auto tmem_s = [&](int g) { return tmem_base + 128u * g; };          // S of warpgroup g's current tile
  auto tmem_o = [&](int g) { return tmem_base + 256u + (uint32_t)D * g; };   // its accumulator
  auto tmem_p = [&](int g) { return tmem_base + 384u + 64u * g; };           // its P, where that is in tensor memory

  pdl_launch_dependents();   // after the tensor-memory allocation, see gemm_tcgen05.cu
  pdl_wait();
  if (warp == 0 || warp == 10) {
    // ---- producers: warp 0 the K tiles (and Q), warp 10 the V tiles; lane g fetches page g of a tile ----
    const int which = warp == 0 ? 0 : 1;
    if (which == 0 && lane == 0) {
      bar_expect_tx(q_full, kDBlocks * kSliceBytes);
      for (int db = 0; db < kDBlocks; ++db)
        tma_2d(base + kQOff + db * kSliceBytes, &map_q, head * D + db * 64, token0, q_full);
    }
    const CUtensorMap* map = which ? &map_v : &map_k;
    const CUtensorMap* run_map = which ? &run_v : &run_k;
    const int page_shift = __ffs(p.page_size) - 1;            // a page is a power of two tokens
    const int first_entry = k_begin >> page_shift;
    const int tail_pages = num_tiles > 0 ? (k_end - (k_begin + (num_tiles - 1) * kBlockKV) + p.page_size - 1) >> page_shift : 0;
    auto pages_of = [&](int i) { return i + 1 < num_tiles ? pages_per_tile : tail_pages; };
    // Lane g's page of tile i, read two tiles before its use: the block table's latency would
    // otherwise stand between a freed stage and its next load.
    auto read_page = [&](int i) {
      if (i >= num_tiles || lane >= pages_of(i)) return 0;
      return table[first_entry + i * pages_per_tile + lane];   // one coalesced read per tile
    };
    bool bad = false;
    int page = read_page(0), page_next = read_page(1);
    for (int i = 0; i < num_tiles; ++i) {
      const int page_after = read_page(i + 2);
      const int s = i % kStages;
      const uint32_t full = which ? v_full(s) : k_full(s);
      const int pages = pages_of(i);
      if (page < 0 || page >= p.num_pages) {
        bad = true;
        page = 0;   // keep the byte count right; the status word fails the step
      }
      // Pages that follow one another in the pool: one box of the four-dimensional view of the cache
      // per 64-dim slice instead of one box a page (with 16-token pages at head size 128 the TMA
      // unit's time per box was a quarter of the kernel's).
      const int page0 = __shfl_sync(0xffffffffu, page, 0);
      const bool run = pages_per_tile > 1 && pages == pages_per_tile && page0 + pages <= p.num_pages &&
                       __all_sync(0xffffffffu, lane >= pages || page == page0 + lane);
      if (i >= kStages &&
          !__all_sync(0xffffffffu, bar_wait(which ? v_empty(s) : k_empty(s), ((i / kStages) & 1) ^ 1, p.status)))
        break;
      if (which && i < kStages && pages < pages_per_tile) {
        // First use of this stage by a tile with fewer than 128 keys (the last one): the V rows no
        // TMA fills must be finite, because a probability of zero times a NaN would still poison
        // the sum.  K needs nothing: scores of keys past the end are replaced, not multiplied.
        // (Every CTA used to clear all stages when it started: a microsecond of each CTA's life.)
        const int first = pages * p.page_size;
        for (int db = 0; db < kDBlocks; ++db)
          for (int c = first * 8 + lane; c < kBlockKV * 8; c += 32)
            *reinterpret_cast<uint4*>(gbase + kVOff + (s * kDBlocks + db) * kSliceBytes + c * 16) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
      }
      if (lane == 0) bar_expect_tx(full, (uint32_t)pages * page_bytes * kDBlocks);
      const uint32_t dst = base + (which ? kVOff : kKOff) + s * kDBlocks * kSliceBytes;
      if (run) {
        if (lane < kDBlocks) tma_4d(dst + lane * kSliceBytes, run_map, lane * 64, 0, kv_head, page0, full);
      } else if (lane < pages) {
        const int row = (page * p.num_kv_heads + kv_head) * p.page_size;
        for (int db = 0; db < kDBlocks; ++db)
          tma_2d(dst + db * kSliceBytes + lane * page_bytes, map, db * 64, row, full);
      }
      page = page_next;
      page_next = page_after;
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(p.status, kStatusBadPage);
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- first product: S = Q K^T of tile i into the buffer of the warpgroup that takes it (i & 1) ----
      // M = 128 queries, N = 128 keys, A and B K-major.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlockKV >> 3) << 17) | ((128u >> 4) << 24);
      const uint64_t desc_q = desc_k_major(base + kQOff);
      bool ok = bar_wait(q_full, 0, p.status);
      for (int i = 0; i < num_tiles && ok; ++i) {
        const int s = i % kStages;
        const uint64_t desc_k = desc_k_major(base + kKOff + s * kDBlocks * kSliceBytes);
        ok = bar_wait(k_full(s), (i / kStages) & 1, p.status);
        // The warpgroup has the last of its previous tile's S in registers (it says so some hundred
        // cycles before that tile's P is written).
        if (ok && i >= 2) ok = bar_wait(s_free(i & 1), ((i - 2) >> 1) & 1, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int db = 0; db < kDBlocks; ++db)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ss(tmem_s(i & 1), desc_advance(desc_q, db * kSliceBytes + kk * 32),
                   desc_advance(desc_k, db * kSliceBytes + kk * 32), idesc_s, (db > 0 || kk > 0) ? 1u : 0u);
        mma_commit(s_full(i & 1));
        mma_commit(k_empty(s));
      }
    }
  } else if (warp == 11) {
    if (lane == 0) {
      // ---- second product: O += P V of tile i into its warpgroup's accumulator ----
      // M = 128, N = D, A (P) K-major, B (V) MN-major.
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < num_tiles && ok; ++i) {
        const int g = i & 1, s = i % kStages, b = (i >> 1) % kPBuffers;
        const uint64_t desc_p = desc_k_major(base + kPOff + (g * kPBuffers + b) * kPBytes);
        const uint64_t desc_v = desc_mn_major(base + kVOff + s * kDBlocks * kSliceBytes);
        ok = bar_wait(v_full(s), (i / kStages) & 1, p.status) && bar_wait(p_full(g), (i >> 1) & 1, p.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int ks = 0; ks < kBlockKV / 16; ++ks) {
          // keys ks*16 .. +15: V rows ks * 16; P columns ks * 8 of its tensor-memory tile, or in shared
          // memory slice ks / 4 at byte (ks % 4) * 32
          if (kPInTmem)
            mma_ts(tmem_o(g), tmem_p(g) + ks * 8, desc_advance(desc_v, ks * 16 * 128), idesc_o, (i >= 2 || ks > 0) ? 1u : 0u);
          else
            mma_ss(tmem_o(g), desc_advance(desc_p, (ks / 4) * kSliceBytes + (ks % 4) * 32),
                   desc_advance(desc_v, ks * 16 * 128), idesc_o, (i >= 2 || ks > 0) ? 1u : 0u);
        }
        mma_commit(o_done(g, b));
        mma_commit(v_empty(s));
      }
    }
  } else {
    // ---- softmax and output: in each warpgroup thread r owns query row r ----
    const int r = (warp & 3) * 32 + lane;                      // tensor-memory lane = query row
    const int g = warp >= 6 ? 1 : 0;                           // warpgroup: tiles g, g + 2, ...; dims g * D / 2 ... of the output
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int pos = r < rows ? pos0 + r : -1;
    constexpr int kDimsHere = D / 2;
    const uint32_t s_tile = tmem_s(g), o_acc = tmem_o(g) + lane_addr;
    // P and O are scaled by a reference m_ref: the maximum of the row's first tile, and after that
    // whatever it was, for as long as it serves.  A tile's probabilities are computed against the
    // reference as it stands, in one walk over S that looks at no maximum at all: exponent, sum,
    // round, store.  Only when a row's sum over a tile comes out above kSumLimit (scores far above
    // the reference; an overflow to infinity is such a sum too) does the warp walk the tile for
    // its maximum, move the reference there (O and the running sum are rescaled) and do the tile
    // again.  Every quantity that is scaled by m_ref is scaled alike, and bfloat16 and 32-bit keep
    // their relative precision over that range, so the result does not depend on where the
    // reference stands.
    float m_ref = -INFINITY;
    float l_run = 0.f;
    int done = 0;               // tiles this warpgroup has finished
    bool ok = true;
    // O and the running sum move from reference m_ref to m_to (rows of the warp that need not move have factor 1)
    auto move_reference = [&](float m_to, bool have_o) {
      // a row that was masked so far has m_ref = -inf and an accumulator of zeros: factor 0
      const float factor = m_to == -INFINITY ? 1.f : fast_exp2(m_ref - m_to);
      if (have_o) {
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          float v[32];
          tmem_ld32(o_acc + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) v[c] *= factor;
          tmem_st32(o_acc + c0, v);
        }
        tmem_st_wait();
      }
      l_run *= factor;
      m_ref = m_to;
    };
    for (int i = g; i < num_tiles && ok; i += 2, ++done) {
      const int key0 = k_begin + i * kBlockKV;
      // A P buffer is free once the second product of the tile that used it is complete, and the
      // accumulator may be rescaled once the second product of this warpgroup's previous tile is.
      // That one started when the previous tile's P was written, a moment ago: the wait for it comes
      // as late as it can, before the first store of P (the exponentials of the first 32 columns
      // are made meanwhile), or earlier if the reference has to move.  (With kPBuffers P tiles the
      // store waits for the tile that used the same one.)
      bool o_quiet = done == 0, p_free = done < kPBuffers;
      auto wait_product = [&](int tile) {   // this warpgroup's tile number `tile`
        ok = __all_sync(0xffffffffu, bar_wait(o_done(g, tile % kPBuffers), (tile / kPBuffers) & 1, p.status)) && ok;   // a warp acts as one
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      };
      auto wait_o_quiet = [&]() {
        if (o_quiet) return;
        wait_product(done - 1);
        o_quiet = true;
        p_free = true;
      };
      auto wait_p_free = [&]() {
        if (p_free) return;
        wait_product(done - kPBuffers);
        p_free = true;
        if (kPBuffers == 1) o_quiet = true;
      };
      ok = __all_sync(0xffffffffu, bar_wait(s_full(g), done & 1, p.status));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // A tile that lies wholly before this row's position (and inside its window) needs no mask;
      // in a tile on the diagonal or at a window's edge, column c of the tile is set to -inf
      // (probability 2^-inf = 0) unless c_lo <= c <= c_hi, before anything else looks at it.
      const int c_hi = pos - key0, c_lo = p.window > 0 ? pos - p.window + 1 - key0 : 0;
      const bool warp_all_visible = __all_sync(0xffffffffu, c_hi >= kBlockKV - 1 && c_lo <= 0);
      auto mask = [&](float* sv, int c0) {
        const int hi = c_hi - c0, lo = c_lo - c0;
#pragma unroll
        for (int c = 0; c < 32; ++c) sv[c] = (c <= hi && c >= lo) ? sv[c] : -INFINITY;
      };
      const uint32_t s_row = s_tile + lane_addr;
      unsigned char* p_row = gbase + kPOff + (g * kPBuffers + done % kPBuffers) * kPBytes + (r >> 3) * 1024 + (r & 7) * 128;
      // A row without a reference that sees a key in this tile (its first tile; with a window, the
      // first that reaches into it) gets one from a walk for the maximum before anything else.
      bool walked = __any_sync(0xffffffffu, m_ref == -INFINITY && c_hi >= 0 && c_lo < kBlockKV && c_lo <= c_hi);
      float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll 1
      for (int attempt = 0; attempt < 2; ++attempt) {
        if (walked) {
          float tile_max = -INFINITY;
#pragma unroll 1
          for (int c0 = 0; c0 < kBlockKV; c0 += 32) {
            float sv[32];
            tmem_ld32(s_row + c0, sv);
            tmem_ld_wait();
            if (!warp_all_visible) mask(sv, c0);
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one
#pragma unroll
            for (int c = 0; c < 32; ++c) m4[c & 3] = fmaxf(m4[c & 3], sv[c]);
            tile_max = fmaxf(tile_max, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
          }
          wait_o_quiet();
          // the scale is positive: max and scale commute
          move_reference(fmaxf(m_ref, tile_max * p.scale_log2), done > 0);
        }
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-m_use, -m_use);
        sum2 = make_float2(0.f, 0.f);
        auto store = [&](const float* sv, int c0) {
          uint32_t packed[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(sv[c], sv[c + 1]);
            packed[c >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
          }
          if (kPInTmem) {
            tmem_st16(tmem_p(g) + lane_addr + (c0 >> 1), packed);   // two keys to a column
          } else {
            unsigned char* slice = p_row + (c0 >> 6) * kSliceBytes;
            const int first_chunk = (c0 & 63) >> 3;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(slice + (((first_chunk + q) ^ (r & 7)) << 4)) =
                  make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
          }
        };
        bool again = false;
        // The walk exists twice: for tiles that need no mask, and for the tile on the diagonal or at a
        // window's edge.  Inside one loop the masks' instructions, though jumped over, lay between
        // those of every tile's walk, which runs at the speed its instructions arrive.
        auto walk = [&](auto masked_tag) {
          constexpr bool kMasked = decltype(masked_tag)::value;
          // 32 columns of the row: probabilities against the reference (two columns to an instruction
          // where there is one that takes two), their sum, and P as bfloat16 in the swizzled K-major
          // layout (32 keys = four 16-byte chunks of this row inside slice c0 / 64)
          auto exps = [&](float* sv, int c0, bool masked_already) {
            if (kMasked && !masked_already) mask(sv, c0);
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const float2 x = __ffma2_rn(make_float2(sv[c], sv[c + 1]), scale2, shift2);
              sv[c] = fast_exp2(x.x);
              sv[c + 1] = fast_exp2(x.y);
              sum2 = __fadd2_rn(sum2, make_float2(sv[c], sv[c + 1]));
            }
          };
          // the load of the next 32 columns is in flight during the arithmetic on these (a pipeline of
          // 16-column pieces, one loading, one in the exponentials, one being stored, was slower); two
          // trips of two chunks, not four unrolled: a warp that outruns the instruction cache runs at
          // the speed of instruction fetch
          float sa[32], sb[32];
          tmem_ld32(s_row, sa);
#pragma unroll 1
          for (int c0 = 0; c0 < kBlockKV; c0 += 64) {
            tmem_ld_wait32(sa);
            tmem_ld32(s_row + c0 + 32, sb);
            exps(sa, c0, false);
            if (c0 == 0) wait_p_free();   // before the tile's first store (once in the loop, like everything in it)
            store(sa, c0);
            tmem_ld_wait32(sb);
            const bool last = c0 + 64 >= kBlockKV;
            if (!last) tmem_ld32(s_row + c0 + 64, sa);
            // Once the last columns of S are in registers and it is known that the tile need not be
            // done again against a new reference (never after a walk: then no probability is above
            // 1), S is no longer needed, and the first product of this warpgroup's next tile may
            // overwrite it.  The row's sum over the tile tells, after the last exponentials; or,
            // before them, the sum so far and the largest of the last 32 scores, which costs a
            // fraction of their exponentials.  (Each statement of exps() once in this loop: a second
            // copy of its body for the last chunk cost head size 64 a twentieth of the kernel.)
            if (kReleaseBeforeLastExps && last) {
              if (kMasked) mask(sb, c0 + 32);
              float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one
#pragma unroll
              for (int c = 0; c < 32; ++c) m4[c & 3] = fmaxf(m4[c & 3], sb[c]);
              const float last_max = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
              again = !walked && __any_sync(0xffffffffu, !(sum2.x + sum2.y <= kSumLimit) ||
                                                             fmaf(last_max, p.scale_log2, -m_use) > kLastLimit);
              if (!again) {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                bar_arrive(s_free(g));
              }
            }
            exps(sb, c0 + 32, kReleaseBeforeLastExps && last);
            if (!kReleaseBeforeLastExps && last) {
              again = !walked && __any_sync(0xffffffffu, !(sum2.x + sum2.y <= kSumLimit));
              if (!again) {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                bar_arrive(s_free(g));
              }
            }
            store(sb, c0 + 32);
          }
        };
        if (warp_all_visible)
          walk(std::false_type{});
        else
          walk(std::true_type{});
        if (!again || !ok) break;
        walked = true;
      }
      if (!ok) break;
      l_run += sum2.x + sum2.y;
      if (kPInTmem) tmem_st_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      if (!kPInTmem) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core's proxy
      bar_arrive(p_full(g));
    }
    // this warpgroup's last product
    if (ok && done > 0) {
      ok = bar_wait(o_done(g, (done - 1) % kPBuffers), ((done - 1) / kPBuffers) & 1, p.status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    // The two warpgroups' shares of the row.  Once both have come here every product of the CTA is
    // complete, so the K and V rings are free: each warpgroup writes there the half of the dims
    // that the other will put out (rows padded by one float so that neither writers nor readers
    // conflict), then merges the other's half into its own.
    softmax_sync();
    float* xchg_m = reinterpret_cast<float*>(gbase + kXchgOff);   // [warpgroup][row]
    float* xchg_l = xchg_m + 2 * 128;
    float* xchg_o = reinterpret_cast<float*>(gbase + kKOff);      // [warpgroup][row][D / 2 + 1]
    const bool have = ok && done > 0;
    xchg_m[g * 128 + r] = have ? m_ref : -INFINITY;
    xchg_l[g * 128 + r] = have ? l_run : 0.f;
    float* give = xchg_o + (size_t)(g * 128 + r) * (kDimsHere + 1);
#pragma unroll 1
    for (int c0 = 0; c0 < kDimsHere; c0 += 32) {
      float v[32];
      if (done > 0) {
        tmem_ld32(o_acc + (g ^ 1) * kDimsHere + c0, v);
        tmem_ld_wait();
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) give[c0 + c] = have ? v[c] : 0.f;
    }
    softmax_sync();
    const float m_other = xchg_m[(g ^ 1) * 128 + r], l_other = xchg_l[(g ^ 1) * 128 + r];
    const float m_mine = have ? m_ref : -INFINITY;
    const float m_all = fmaxf(m_mine, m_other);
    const float f_mine = m_mine == -INFINITY ? 0.f : fast_exp2(m_mine - m_all);
    const float f_other = m_other == -INFINITY ? 0.f : fast_exp2(m_other - m_all);
    const float l_all = (have ? l_run : 0.f) * f_mine + l_other * f_other;
    const float* take = xchg_o + (size_t)((g ^ 1) * 128 + r) * (kDimsHere + 1);
    // for a cluster: this CTA's share (sums of both warpgroups, not yet divided), after the exchange area
    float* part_o = reinterpret_cast<float*>(gbase + kShareOff);
    float* part_ml = part_o + kBlockQ * (D + 1);
    const float inv = csize > 1 ? 1.f : (l_all > 0.f ? 1.f / l_all : 0.f);
    __nv_bfloat16* dst = p.out + ((size_t)(token0 + r) * p.num_heads + head) * D + g * kDimsHere;
#pragma unroll 1
    for (int c0 = 0; c0 < kDimsHere; c0 += 32) {
      float v[32];
      if (done > 0) {
        tmem_ld32(o_acc + g * kDimsHere + c0, v);
        tmem_ld_wait();
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = ((have ? v[c] : 0.f) * f_mine + take[c0 + c] * f_other) * inv;
      if (csize > 1) {
#pragma unroll
        for (int c = 0; c < 32; ++c) part_o[r * (D + 1) + g * kDimsHere + c0 + c] = v[c];
      } else if (ok && pos >= 0) {
#pragma unroll
        for (int d = 0; d < 32; d += 8) {
          uint4 raw;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[d + 2 * e], v[d + 2 * e + 1]);
          *reinterpret_cast<uint4*>(dst + c0 + d) = raw;
        }
      }
    }
    if (csize > 1 && g == 0) {
      part_ml[r] = m_all;
      part_ml[kBlockQ + r] = l_all;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (csize > 1) {
    // Merge the CTAs that shared this row tile: each takes a run of rows, reads every CTA's maximum,
    // sum and accumulator for them and writes the rows.
    const float* part_o = reinterpret_cast<const float*>(gbase + kShareOff);
    const float* part_ml = part_o + kBlockQ * (D + 1);
    cluster_sync_all();
    const int rows_each = (rows + (int)csize - 1) / (int)csize;
    const int row_begin = (int)rank * rows_each, row_end = min(rows, row_begin + rows_each);
    // One warp per row: the factors of the CTAs' shares once per row (lane c reads CTA c's maximum and
    // sum), then every lane adds up the shares of its dims.
    for (int row = row_begin + warp; row < row_end; row += kAttnThreads / 32) {
      const bool live = lane < (int)csize;
      const float m_c = live ? ld_peer(part_ml + row, lane) : -INFINITY;
      const float l_c = live ? ld_peer(part_ml + kBlockQ + row, lane) : 0.f;
      float m = m_c;
#pragma unroll
      for (int offset = 4; offset >= 1; offset >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, offset));   // lanes 0-7
      m = __shfl_sync(0xffffffffu, m, 0);
      const float f_c = m_c == -INFINITY ? 0.f : fast_exp2(m_c - m);
      float l = l_c * f_c;
#pragma unroll
      for (int offset = 4; offset >= 1; offset >>= 1) l += __shfl_xor_sync(0xffffffffu, l, offset);
      l = __shfl_sync(0xffffffffu, l, 0);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      float o[D / 32];
#pragma unroll
      for (int j = 0; j < D / 32; ++j) o[j] = 0.f;
      for (int c = 0; c < (int)csize; ++c) {
        const float f = __shfl_sync(0xffffffffu, f_c, c);
#pragma unroll
        for (int j = 0; j < D / 32; ++j) o[j] += ld_peer(part_o + row * (D + 1) + j * 32 + lane, c) * f;
      }
      __nv_bfloat16* dst = p.out + ((size_t)(token0 + row) * p.num_heads + head) * D;
#pragma unroll
      for (int j = 0; j < D / 32; ++j) dst[j * 32 + lane] = __float2bfloat16_rn(o[j] * inv);
    }
    cluster_leave();   // no CTA leaves while a peer may still read its shared memory
  }
}

// ---------------------------------------------------------------------------
// Decode on the tensor cores, operands swapped: one decoded token has at most a few
// query heads per key/value head, far fewer than the 128 rows an MMA wants, so here the
// KEYS are the 128-row operand.  Per tile of 128 keys
//
//   S^T[128 keys, 16 heads] = K_tile (K-major, straight from its pages) . Q^T
//   O^T[D dims, 16 heads]  += V_tile (MN-major, straight from its pages) . P^T
//
// so the tensor core runs full tiles whatever the number of heads, and K and V are used
// in the layout the cache stores.  Softmax thread r owns key r of the tile (tensor-memory
// lane r of S^T); the maximum of a head over the tile's keys is a warp shuffle reduction
// and one exchange between the four warps through shared memory.  In O^T thread r owns
// one dim (for D = 64 the M = 64 accumulator lives in lanes 0-15 of each warp's quarter)
// and keeps the 16 heads' running sums in registers.  The splits of a long context are
// the CTAs of a thread-block cluster and merge through distributed shared memory.
// ---------------------------------------------------------------------------
#ifndef DECODE_STAGES
#define DECODE_STAGES 3
#endif
constexpr int kDecStages = DECODE_STAGES;
constexpr int kDecThreads = 192;                           // producer warp, MMA warp, four softmax warps
constexpr int kDecHeads = 16;                              // query heads of one key/value head per CTA (the MMA's N)
constexpr int kDecQSlice = kDecHeads * 128;                // [16 heads x 64 dims] bf16
constexpr int kDecPBytes = 2 * kDecHeads * 128;            // [16 heads x 128 keys] bf16: two 64-key slices
constexpr int kDecKOff = 0;
constexpr int kDecVOff = kDecKOff + kDecStages * kDBlocks * kSliceBytes;
constexpr int kDecPOff = kDecVOff + kDecStages * kDBlocks * kSliceBytes;
constexpr int kDecQOff = kDecPOff + 2 * kDecPBytes;
constexpr int kDecBarOff = kDecQOff + kDBlocks * kDecQSlice;
constexpr int kDecNumBars = 2 * kDecStages + 7;            // kv_full[], kv_empty[], s_full[2], p_full[2], o_full[2], q_ready
constexpr int kDecXchgOff = (kDecBarOff + 8 * kDecNumBars + 16 + 15) / 16 * 16;   // [2][4 warps][16 heads] tile maxima, [4][16] sums
static_assert(kDecXchgOff % 16 == 0, "the tile maxima are read as float4");
constexpr int kDecOutOff = kDecXchgOff + (2 * 4 * 16 + 4 * 16) * 4;   // cta_o [16][D], cta_m [16], cta_l [16]
constexpr int kDecSmemBytes = kDecOutOff + (16 * D + 32) * 4;
static_assert(kDecSmemBytes <= 227 * 1024, "shared memory of the tcgen05 decode kernel exceeds an SM");
static_assert(kDecQOff % 1024 == 0 && kDecPOff % 1024 == 0, "operand tiles start on a swizzle group");
constexpr int kDecCtasPerSm = (227 * 1024) / (kDecSmemBytes + 1024) < 3 ? (227 * 1024) / (kDecSmemBytes + 1024) : 3;
constexpr int kDecTmemCols = 64;                           // S^T: 2 x 16 columns, O^T tile: 2 x 16 columns
constexpr int kDecMaxSplits = 8;                           // clusters per token, which meet in global memory
constexpr int kDecMaxCluster = 16;                        // above 8: a cluster size the launch has to allow by name

struct TcDecodeParams {
  const int* token_list;    // packed indices of the tokens to process, or null for 0 .. n-1
  const __nv_bfloat16* q;   // [tokens, heads, D]
  const int* block_table;   // [requests, table_width]
  const int* seq_of_token;
  const int* positions;
  __nv_bfloat16* out;       // [tokens, heads, D]
  int* status;
  int num_heads, num_kv_heads, page_size, num_pages, table_width, window;
  float scale_log2;
  // A token's keys split over `splits` clusters, which meet in global memory: every cluster writes its
  // unnormalised share [16 heads][D + 2] (the accumulator, then maximum and sum) to split_out, every
  // CTA counts itself in split_count, and the CTA that finds itself the last adds the shares up.
  int splits;
  float* split_out;         // [launch's (token, kv head, head block)][splits][16][D + 2]
  int* split_count;         // one per (token, kv head, head block); zero between launches
};

// kSplit: several clusters per token (a kernel of its own, so that the one that most steps run
// carries none of its code).
template <bool kSplit>
__global__ void __launch_bounds__(kDecThreads, kDecCtasPerSm)
paged_decode_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                      const __grid_constant__ CUtensorMap run_k, const __grid_constant__ CUtensorMap run_v,
                                      TcDecodeParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = saddr(smem_raw);
  unsigned char* gbase = smem_raw;
  // Every CTA of the grid sees the same alignment, so all leave together (no cluster barrier is left waiting).
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicOr(p.status, kStatusWaitExpired);
    return;
  }
  const uint32_t bars = base + kDecBarOff;
  auto kv_full = [&](int s) { return bars + 8u * s; };
  auto kv_empty = [&](int s) { return bars + 8u * (kDecStages + s); };
  auto s_full = [&](int b) { return bars + 8u * (2 * kDecStages + b); };
  auto p_full = [&](int b) { return bars + 8u * (2 * kDecStages + 2 + b); };
  auto o_full = [&](int b) { return bars + 8u * (2 * kDecStages + 4 + b); };
  const uint32_t q_ready = bars + 8u * (2 * kDecStages + 6);
  const uint32_t tmem_holder = bars + 8 * kDecNumBars;
  volatile uint32_t* tmem_holder_ptr = reinterpret_cast<volatile uint32_t*>(gbase + kDecBarOff + 8 * kDecNumBars);
  float* warp_max_x = reinterpret_cast<float*>(gbase + kDecXchgOff);   // [tile parity][warp][head]
  float* warp_sum_x = warp_max_x + 2 * 4 * 16;                         // [warp][head]
  float* cta_o = reinterpret_cast<float*>(gbase + kDecOutOff);         // [16][D]
  float* cta_m = cta_o + 16 * D;
  float* cta_l = cta_m + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.num_heads / p.num_kv_heads;
  const int head_blocks = (group + kDecHeads - 1) / kDecHeads;
  const int kv_head = blockIdx.y / head_blocks;
  const int head_block = blockIdx.y - kv_head * head_blocks;
  const int first_head = kv_head * group + head_block * kDecHeads;
  const int rows_valid = min(kDecHeads, group - head_block * kDecHeads);
  const uint32_t rank = cluster_rank(), csize = cluster_size();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) {
      bar_init(kv_full(s), 1);
      bar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      bar_init(s_full(b), 1);
      bar_init(p_full(b), 128);
      bar_init(o_full(b), 1);
    }
    bar_init(q_ready, 128);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_holder), "r"(kDecTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // What follows reads only what no kernel of this step writes: the step's own inputs
  // (positions, block tables) and keys and values of earlier steps.  The kernel before this one
  // (which writes this token's query, key and value) may still be running: each thread waits
  // for it where it first needs one of those.
  const int t = p.token_list ? p.token_list[blockIdx.z] : blockIdx.z;
  const int pos = p.positions[t];
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int lo_page = lo / p.page_size * p.page_size;         // tiles start on a page edge
  const int split = kSplit ? (int)(blockIdx.x / csize) : 0;    // which of the token's clusters this is
  const int parts = kSplit ? (int)csize * p.splits : (int)csize;
  int per = (pos + 1 - lo_page + parts - 1) / parts;
  per = (per + kBlockKV - 1) / kBlockKV * kBlockKV;
  const int k_begin = min(pos + 1, lo_page + (split * (int)csize + (int)rank) * per);
  const int k_end = min(pos + 1, k_begin + per);
  const int num_tiles = (k_end - k_begin + kBlockKV - 1) / kBlockKV;
  const int* table = p.block_table + (size_t)p.seq_of_token[t] * p.table_width;
  const int pages_per_tile = kBlockKV / p.page_size;
  const uint32_t page_bytes = (uint32_t)p.page_size * 128u;   // one page of one 64-wide slice

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  pdl_launch_dependents();   // after the tensor-memory allocation, see gemm_tcgen05.cu
  const uint32_t tmem_base = *tmem_holder_ptr;
  auto tmem_s = [&](int b) { return tmem_base + 16u * b; };
  auto tmem_o = [&](int b) { return tmem_base + 32u + 16u * b; };

  float acc[kDecHeads], m_run[kDecHeads], l_thr[kDecHeads];
#pragma unroll
  for (int h = 0; h < kDecHeads; ++h) {
    acc[h] = 0.f;
    m_run[h] = -INFINITY;
    l_thr[h] = 0.f;
  }
  const int r = (warp & 3) * 32 + lane;                        // softmax warps: tensor-memory lane

  if (warp == 0) {
    // ---- producer: lane g fetches page g of a tile ----
    // The block-table entries of a tile are read one tile ahead, so that the round trip to
    // global memory does not sit between a freed stage and its next load.
    bool bad = false;
    auto pages_of = [&](int i) {
      const int key0 = k_begin + i * kBlockKV;
      return min(pages_per_tile, (k_end - key0 + p.page_size - 1) / p.page_size);
    };
    auto page_of = [&](int i) {
      return (i < num_tiles && lane < pages_of(i)) ? table[(k_begin + i * kBlockKV) / p.page_size + lane] : 0;
    };
    int next_page = page_of(0);
    for (int i = 0; i < num_tiles; ++i) {
      const int s = i % kDecStages;
      int page = next_page;
      next_page = page_of(i + 1);
      const int pages = pages_of(i);
      if (i < kDecStages && pages < pages_per_tile) {
        // First use of this stage by a tile with fewer than 128 keys: the V rows no TMA fills must be
        // finite (a probability of zero times a NaN would still poison the sum).  K needs nothing:
        // scores of keys past the end are replaced, not multiplied.
        const int first = pages * p.page_size;
        for (int db = 0; db < kDBlocks; ++db)
          for (int c = first * 8 + lane; c < kBlockKV * 8; c += 32)
            *reinterpret_cast<uint4*>(gbase + kDecVOff + (s * kDBlocks + db) * kSliceBytes + c * 16) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      // Wait for the kernel before this one where a load needs it (the tile with this step's own key
      // and value) and before the first bounded wait that only progress of this kernel's other
      // warps, which need the query, can end: a bounded wait must not run while the wait for
      // another kernel is still open.
      if (i >= kDecStages || k_begin + (i + 1) * kBlockKV > pos) pdl_wait();
      int ok = 1;
      if (i >= kDecStages && lane == 0) ok = bar_wait(kv_empty(s), ((i / kDecStages) & 1) ^ 1, p.status) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (page < 0 || page >= p.num_pages) {
        bad = true;
        page = 0;   // keep the byte count right; the status word fails the step
      }
      __syncwarp();
      if (lane == 0) bar_expect_tx(kv_full(s), (uint32_t)pages * page_bytes * kDBlocks * 2);
      __syncwarp();
      // A tile is one TMA box per page and 64-dim slice, and with small pages the time the TMA unit
      // takes per box is most of a tile's time.  When the tile's pages follow one another in the pool
      // (a context reserved in one go gets such runs), one box of a four-dimensional view of the
      // cache (dims, rows of a page, head, page) brings the whole 128-key slice.
      const int page0 = __shfl_sync(0xffffffffu, page, 0);
      const bool run = pages_per_tile > 1 && pages == pages_per_tile && page0 + pages <= p.num_pages &&
                       __all_sync(0xffffffffu, lane >= pages || page == page0 + lane);
      if (run) {
        if (lane < 2 * kDBlocks) {
          const int db = lane >> 1;
          if (lane & 1)
            tma_4d(base + kDecVOff + (s * kDBlocks + db) * kSliceBytes, &run_v, db * 64, 0, kv_head, page0, kv_full(s));
          else
            tma_4d(base + kDecKOff + (s * kDBlocks + db) * kSliceBytes, &run_k, db * 64, 0, kv_head, page0, kv_full(s));
        }
      } else if (lane < pages) {
        const int row = (page * p.num_kv_heads + kv_head) * p.page_size;
        for (int db = 0; db < kDBlocks; ++db) {
          tma_2d(base + kDecKOff + (s * kDBlocks + db) * kSliceBytes + lane * page_bytes, &map_k, db * 64, row, kv_full(s));
          tma_2d(base + kDecVOff + (s * kDBlocks + db) * kSliceBytes + lane * page_bytes, &map_v, db * 64, row, kv_full(s));
        }
      }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(p.status, kStatusBadPage);
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      // S^T: M = 128 keys, N = 16 heads, both K-major.  O^T: M = D dims (A = V, MN-major), N = 16 heads (B = P^T, K-major).
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kDecHeads >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_o =
          (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(kDecHeads >> 3) << 17) | ((uint32_t)(D >> 4) << 24);
      // The two products are issued as their inputs arrive, whichever comes first: S^T of a
      // tile as soon as its keys have landed (at most one tile ahead of the softmax: S^T exists
      // twice), O^T of a tile as soon as its probabilities are written.  Waiting for the next
      // tile's keys before this tile's second product would hold this tile's stage, and with it
      // the producer, for a whole load.
      int next_qk = 0, next_pv = 0;
      int polls = 0;
      const uint64_t desc_q = desc_k_major(base + kDecQOff);
      pdl_wait();   // the bounded waits below count only while this kernel alone is to be waited for
      if (num_tiles > 0 && !bar_wait(q_ready, 0, p.status)) next_pv = num_tiles;
      while (next_pv < num_tiles) {
        bool progress = false;
        if (next_qk < num_tiles && next_qk <= next_pv + 1) {
          const int s = next_qk % kDecStages;
          if (bar_test(kv_full(s), (next_qk / kDecStages) & 1)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t desc_k = desc_k_major(base + kDecKOff + s * kDBlocks * kSliceBytes);
#pragma unroll
            for (int db = 0; db < kDBlocks; ++db)
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                mma_ss(tmem_s(next_qk & 1), desc_advance(desc_k, db * kSliceBytes + kk * 32),
                       desc_advance(desc_q, db * kDecQSlice + kk * 32), idesc_s, (db > 0 || kk > 0) ? 1u : 0u);
            mma_commit(s_full(next_qk & 1));
            ++next_qk;
            progress = true;
          }
        }
        if (next_pv < next_qk && bar_test(p_full(next_pv & 1), (next_pv >> 1) & 1)) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const int s = next_pv % kDecStages;
          const uint64_t desc_v = desc_mn_major(base + kDecVOff + s * kDBlocks * kSliceBytes);
          const uint64_t desc_p = desc_k_major(base + kDecPOff + (next_pv & 1) * kDecPBytes);
#pragma unroll
          for (int ks = 0; ks < kBlockKV / 16; ++ks)
            mma_ss(tmem_o(next_pv & 1), desc_advance(desc_v, ks * 16 * 128),
                   desc_advance(desc_p, (ks / 4) * (kDecPBytes / 2) + (ks % 4) * 32), idesc_o, ks > 0 ? 1u : 0u);
          mma_commit(kv_empty(s));
          mma_commit(o_full(next_pv & 1));
          ++next_pv;
          progress = true;
        }
        if (progress) {
          polls = 0;
        } else if (++polls > kPolls) {
          atomicOr(p.status, kStatusWaitExpired);
          break;
        }
      }
    }
  } else {
    // ---- softmax: thread r owns key r of each tile and, in O^T, one dim ----
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    float alpha_pending[kDecHeads];
#pragma unroll
    for (int h = 0; h < kDecHeads; ++h) alpha_pending[h] = 1.f;
    bool ok = true;
    // Q^T operand: 16 head rows (zeros beyond the group), K-major with the 128-byte swizzle.
    pdl_wait();
    for (int idx = r; idx < kDecHeads * (D / 8); idx += 128) {
      const int h = idx / (D / 8), c = idx - h * (D / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h < rows_valid) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)t * p.num_heads + first_head + h) * D + c * 8);
      *reinterpret_cast<uint4*>(gbase + kDecQOff + (c >> 3) * kDecQSlice + (h >> 3) * 1024 + (h & 7) * 128 +
                                (((c & 7) ^ (h & 7)) << 4)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    bar_arrive(q_ready);
    auto add_tile = [&](int i) {
      if (!bar_wait_likely_done(o_full(i & 1), (i >> 1) & 1, p.status)) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float v[16];
      tmem_ld16(tmem_o(i & 1) + lane_addr, v);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < kDecHeads; ++h) acc[h] = fmaf(acc[h], alpha_pending[h], v[h]);
      return true;
    };
    // Every softmax warp walks every tile, whatever happens: the four meet inside the loop at a
    // hardware barrier.  After a bounded wait that gave up (the status word then fails the step)
    // nothing is waited for any more and the results are garbage, but the walk goes on to its end.
    for (int i = 0; i < num_tiles; ++i) {
      const int j = k_begin + i * kBlockKV + r;                  // this thread's key
      const bool visible = j >= lo && j < k_end;
      ok = ok && bar_wait_likely_done(s_full(i & 1), (i >> 1) & 1, p.status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sv[16];
      tmem_ld16(tmem_s(i & 1) + lane_addr, sv);
      tmem_ld_wait();
      float* wmax = warp_max_x + ((i & 1) * 4 + (warp & 3)) * 16;
      {
        float red[kDecHeads];
#pragma unroll
        for (int h = 0; h < kDecHeads; ++h) {
          sv[h] = visible ? sv[h] * p.scale_log2 : -INFINITY;
          red[h] = sv[h];
        }
        const float m = warp_reduce16<true>(red, lane);
        if ((lane & 1) == 0) wmax[lane >> 1] = m;
      }
      // the four warps' maxima: a meeting at a named barrier (an mbarrier that all 128 threads
      // arrive at and then wait for took 500 of a tile's 1,640 cycles)
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float4* all_max = reinterpret_cast<const float4*>(warp_max_x + (i & 1) * 4 * 16);   // [warp][head / 4]
      unsigned char* p_col = gbase + kDecPOff + (i & 1) * kDecPBytes + (r >> 6) * (kDecPBytes / 2) + (r & 7) * 2;
      const int key_chunk = (r & 63) >> 3;
      float alpha[kDecHeads];
      // Heads in groups of four, each group straight-line code (a branch per head would put the
      // loads and exponentials of the heads one after the other).  Heads past the group's end
      // inside a started group work on zero queries: finite, and their columns are never read.
#pragma unroll
      for (int g4 = 0; g4 < kDecHeads / 4; ++g4) {
        if (g4 * 4 < rows_valid) {
          const float4 a = all_max[g4], b = all_max[4 + g4], c = all_max[8 + g4], d = all_max[12 + g4];
          const float tile_max[4] = {fmaxf(fmaxf(a.x, b.x), fmaxf(c.x, d.x)), fmaxf(fmaxf(a.y, b.y), fmaxf(c.y, d.y)),
                                     fmaxf(fmaxf(a.z, b.z), fmaxf(c.z, d.z)), fmaxf(fmaxf(a.w, b.w), fmaxf(c.w, d.w))};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = g4 * 4 + e;
            const float m_new = fmaxf(m_run[h], tile_max[e]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = fast_exp2(m_run[h] - m_use);
            m_run[h] = m_new;
            const float pr = fast_exp2(sv[h] - m_use);              // exp2(-inf) = 0 for masked keys
            l_thr[h] = fmaf(l_thr[h], alpha[h], pr);
            *reinterpret_cast<__nv_bfloat16*>(p_col + (h >> 3) * 1024 + (h & 7) * 128 + ((key_chunk ^ (h & 7)) << 4)) =
                __float2bfloat16_rn(pr);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) alpha[g4 * 4 + e] = 1.f;
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P^T is read by the tensor core's proxy
      bar_arrive(p_full(i & 1));
      if (i > 0) ok = ok && add_tile(i - 1);
#pragma unroll
      for (int h = 0; h < kDecHeads; ++h) alpha_pending[h] = alpha[h];
    }
    // This CTA's share: the maxima (every thread holds the same ones; one thread writes them: a
    // branch per head, taken by one lane each, cost this warp more than a microsecond) and the
    // sums over the warp's keys, both while the last product is still running; then the
    // accumulator by (head, dim).
    if (r == 0) {
#pragma unroll
      for (int h = 0; h < kDecHeads; ++h) cta_m[h] = m_run[h];
    }
    float* wsum = warp_sum_x + (warp & 3) * 16;
    const float l = warp_reduce16<false>(l_thr, lane);
    if ((lane & 1) == 0) wsum[lane >> 1] = l;
    if (ok && num_tiles > 0) ok = add_tile(num_tiles - 1);
    const bool holds_dim = D == 128 || lane < 16;                 // M = 64: lanes 0-15 of each quarter
    const int dim = D == 128 ? r : (r >> 5) * 16 + lane;
    if (holds_dim) {
#pragma unroll
      for (int h = 0; h < kDecHeads; ++h) cta_o[h * D + dim] = acc[h];
    }
  }
  pdl_wait();   // every thread, before the output is written (most have passed it already)
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kDecTmemCols) : "memory");
  }
  if (threadIdx.x < 16)
    cta_l[threadIdx.x] = warp_sum_x[threadIdx.x] + warp_sum_x[16 + threadIdx.x] + warp_sum_x[32 + threadIdx.x] +
                         warp_sum_x[48 + threadIdx.x];
  // Merge the CTAs of the cluster: each takes a slice of the (head, dim) elements.  (The CTA meets
  // first, at a barrier that holds a waiting warp in hardware: warps that went on to wait at the
  // cluster barrier each for itself, the producer and MMA warps long before the others, poll
  // there and take issue slots from the softmax warps; a tile then took 1,900 instead of 1,590
  // cycles.)
  cluster_sync_all();
  const int total = rows_valid * D;
  const int slice = (total + (int)csize - 1) / (int)csize;
  const int e_begin = (int)rank * slice, e_end = min(total, e_begin + slice);
  const size_t token_heads = (size_t)t * p.num_heads;
  const int pair = blockIdx.z * gridDim.y + blockIdx.y;
  for (int e = e_begin + threadIdx.x; e < e_end; e += kDecThreads) {
    const int row = e / D, d = e - row * D;
    // Eight peers at a time: all their remote loads first, so that they are in flight together,
    // then the arithmetic.
    float m = -INFINITY, l = 0.f, o = 0.f;
    for (int c0 = 0; c0 < (int)csize; c0 += 8) {
      float mc[8], lc[8], oc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const bool live = c0 + c < (int)csize;
        mc[c] = live ? ld_peer(cta_m + row, c0 + c) : -INFINITY;
        lc[c] = live ? ld_peer(cta_l + row, c0 + c) : 0.f;
        oc[c] = live ? ld_peer(cta_o + e, c0 + c) : 0.f;
      }
      float m_new = m;
#pragma unroll
      for (int c = 0; c < 8; ++c) m_new = fmaxf(m_new, mc[c]);
      const float keep = m == -INFINITY ? 0.f : exp2f(m - m_new);
      l *= keep;
      o *= keep;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float f = mc[c] == -INFINITY ? 0.f : exp2f(mc[c] - m_new);
        l += lc[c] * f;
        o += oc[c] * f;
      }
      m = m_new;
    }
    if (!kSplit) {
      p.out[(token_heads + first_head + row) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    } else {
      float* share = p.split_out + (((size_t)pair * p.splits + split) * kDecHeads + row) * (D + 2);
      share[d] = o;
      if (d == 0) {
        share[D] = m;
        share[D + 1] = l;
      }
    }
  }
  if (!kSplit) {
    cluster_leave();   // no CTA leaves while a peer may still read its shared memory
    return;
  }
  // The peers may go once this CTA has read them; what follows touches global memory only.
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  __syncthreads();
  int* last_flag = reinterpret_cast<int*>(warp_max_x);   // the tile maxima are done with
  if (threadIdx.x == 0) {
    __threadfence();                                     // this CTA's share, before it counts itself
    const int before = atomicAdd(p.split_count + pair, 1);
    const int last = before == parts - 1;
    if (last) p.split_count[pair] = 0;                   // for the next launch: every other CTA has counted itself
    *last_flag = last;
  }
  __syncthreads();
  if (*last_flag) {
    __threadfence();
    const float* shares = p.split_out + (size_t)pair * p.splits * kDecHeads * (D + 2);
    for (int e = threadIdx.x; e < total; e += kDecThreads) {
      const int row = e / D, d = e - row * D;
      // every share's loads at once: one after the other each would wait for the L2
      float mc[kDecMaxSplits], lc[kDecMaxSplits], oc[kDecMaxSplits];
#pragma unroll
      for (int c = 0; c < kDecMaxSplits; ++c) {
        const bool live = c < p.splits;
        const float* share = shares + ((size_t)c * kDecHeads + row) * (D + 2);
        mc[c] = live ? __ldcg(share + D) : -INFINITY;
        lc[c] = live ? __ldcg(share + D + 1) : 0.f;
        oc[c] = live ? __ldcg(share + d) : 0.f;
      }
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < kDecMaxSplits; ++c) m = fmaxf(m, mc[c]);
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int c = 0; c < kDecMaxSplits; ++c) {
        const float f = mc[c] == -INFINITY ? 0.f : exp2f(mc[c] - m);
        l += lc[c] * f;
        o += oc[c] * f;
      }
      p.out[(token_heads + first_head + row) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
  }
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
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

// rows x cols bfloat16, unit stride along cols, box of (64 cols x box_rows), 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t element_strides[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                      element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// The cache [pages, kv_heads, page_size, cols] as a four-dimensional map whose box is one head's 64-dim
// slice of `box_pages` consecutive pages: box_pages * page_size rows land in shared memory one after the other.
static int make_run_map(CUtensorMap* map, const void* base, long long pages, int kv_heads, int page_size, long long cols,
                        int box_pages) {
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return (int)cudaErrorNotSupported;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)pages};
  cuuint64_t strides[3] = {(cuuint64_t)cols * 2, (cuuint64_t)page_size * cols * 2,
                           (cuuint64_t)kv_heads * page_size * cols * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)page_size, 1, (cuuint32_t)box_pages};
  cuuint32_t element_strides[4] = {1, 1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                      element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

extern "C" int einf_attention_tcgen05_head_size() { return D; }

// How many clusters of `cluster` CTAs of the prefill kernel the device holds at once (one CTA fills
// an SM, and the GPCs place fewer clusters than SMs / cluster); 0 on error.
extern "C" int einf_paged_prefill_attention_tcgen05_max_clusters(int cluster) {
  if (cluster < 1 || cluster > 8) return 0;
  if (cudaFuncSetAttribute(paged_prefill_attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(1, 1, cluster);
  config.blockDim = dim3(kAttnThreads);
  config.dynamicSmemBytes = kSmemBytes;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 1;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = cluster;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, paged_prefill_attention_tcgen05_kernel, &config) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

// q, out: [tokens, heads, D]; caches [pages, kv_heads, page_size, D]; tiles: [num_tiles, 4] of 128-row query
// tiles.  page_size must be 8, 16, 32, 64 or 128.
// cluster: CTAs that share one (row tile, head), each with a run of its key tiles: 1 to 8.
extern "C" int einf_paged_prefill_attention_tcgen05(const void* q, const void* k_cache, const void* v_cache,
                                                    const int* block_table, const int* tiles, int num_tiles,
                                                    void* out, int num_tokens, int num_heads, int num_kv_heads,
                                                    int page_size, int num_pages, int table_width, float scale,
                                                    int window, int cluster, int* status, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  if (cluster < 1 || cluster > 8) return (int)cudaErrorInvalidValue;
  if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1)) != 0) return (int)cudaErrorInvalidValue;
  CUtensorMap map_q, map_k, map_v;
  int rc = make_map(&map_q, q, num_tokens, (long long)num_heads * D, kBlockQ);
  if (rc) return rc;
  const long long cache_rows = (long long)num_pages * num_kv_heads * page_size;
  rc = make_map(&map_k, k_cache, cache_rows, D, page_size);
  if (rc) return rc;
  rc = make_map(&map_v, v_cache, cache_rows, D, page_size);
  if (rc) return rc;
  CUtensorMap run_k, run_v;
  rc = make_run_map(&run_k, k_cache, num_pages, num_kv_heads, page_size, D, kBlockKV / page_size);
  if (rc) return rc;
  rc = make_run_map(&run_v, v_cache, num_pages, num_kv_heads, page_size, D, kBlockKV / page_size);
  if (rc) return rc;
  TcAttentionParams p;
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
  cudaError_t e = cudaFuncSetAttribute(paged_prefill_attention_tcgen05_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(num_heads, num_tiles, cluster);
  config.blockDim = dim3(kAttnThreads);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 1;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = cluster;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&config, paged_prefill_attention_tcgen05_kernel, map_q, map_k, map_v, run_k, run_v, p);
}


// Decode: one token per (request); cluster = CTAs that split one token's keys: 1 to 16.
// token_list: packed indices of the num_tokens tokens to process (null: tokens 0 .. num_tokens-1).
// How many clusters of `cluster` CTAs of the decode kernel the device holds at once (what the
// GPCs place, which for clusters of eight one-per-SM CTAs is fewer than SMs / 8); 0 on error.
extern "C" int einf_paged_decode_attention_tcgen05_max_clusters(int cluster) {
  if (cluster < 1 || cluster > kDecMaxCluster) return 0;
  const auto kernel = paged_decode_attention_tcgen05_kernel<false>;   // the two take the same room
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kDecSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (cluster > 8 && cudaFuncSetAttribute(kernel,
                                          cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(cluster, 1, 1);
  config.blockDim = dim3(kDecThreads);
  config.dynamicSmemBytes = kDecSmemBytes;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = cluster;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  // The calculator counts one CTA of this kernel per SM; at head size 64 two fit (kDecCtasPerSm, from
  // the shared memory a CTA takes), and as many clusters more were measured to run at once.
  return clusters * kDecCtasPerSm;
}

extern "C" int einf_paged_decode_attention_tcgen05(const void* q, const void* k_cache, const void* v_cache,
                                                   const int* block_table, const int* seq_of_token,
                                                   const int* positions, const int* token_list, void* out,
                                                   int num_tokens, int num_heads, int num_kv_heads, int page_size,
                                                   int num_pages, int table_width, float scale, int window,
                                                   int cluster, int splits, float* split_out, int* split_count,
                                                   int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (cluster < 1 || cluster > kDecMaxCluster) return (int)cudaErrorInvalidValue;
  if (splits < 1 || splits > kDecMaxSplits || (splits > 1 && (!split_out || !split_count))) return (int)cudaErrorInvalidValue;
  if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1)) != 0) return (int)cudaErrorInvalidValue;
  CUtensorMap map_k, map_v;
  const long long cache_rows = (long long)num_pages * num_kv_heads * page_size;
  int rc = make_map(&map_k, k_cache, cache_rows, D, page_size);
  if (rc) return rc;
  rc = make_map(&map_v, v_cache, cache_rows, D, page_size);
  if (rc) return rc;
  CUtensorMap run_k, run_v;
  rc = make_run_map(&run_k, k_cache, num_pages, num_kv_heads, page_size, D, kBlockKV / page_size);
  if (rc) return rc;
  rc = make_run_map(&run_v, v_cache, num_pages, num_kv_heads, page_size, D, kBlockKV / page_size);
  if (rc) return rc;
  TcDecodeParams p;
  p.token_list = token_list;
  p.q = (const __nv_bfloat16*)q;
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
  p.splits = splits;
  p.split_out = split_out;
  p.split_count = split_count;
  const int head_blocks = (num_heads / num_kv_heads + kDecHeads - 1) / kDecHeads;
  const auto kernel = splits > 1 ? paged_decode_attention_tcgen05_kernel<true> : paged_decode_attention_tcgen05_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes);
  if (e != cudaSuccess) return (int)e;
  // all of the SM's memory as shared memory, so that two CTAs fit at head size 64
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  if (cluster > 8) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(cluster * splits, num_kv_heads * head_blocks, num_tokens);
  config.blockDim = dim3(kDecThreads);
  config.dynamicSmemBytes = kDecSmemBytes;
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
  return (int)cudaLaunchKernelEx(&config, kernel, map_k, map_v, run_k, run_v, p);
}
