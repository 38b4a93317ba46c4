// Token selection from float logits [rows, vocab]: argmax, and temperature
// sampling with top-k, top-p and min-p filters and a counter-based generator.
//
// Semantics follow src/einf/executors/torch/sampler.py:21-102 of the reference:
// greedy rows (temperature 0) take the first largest index; other rows divide
// the logits by the temperature, keep the k largest, keep the smallest set of
// most probable tokens whose mass reaches top_p (the crossing token included),
// drop tokens whose probability is below min_p times the largest, and draw from
// what is left.  Tokens with equal scaled logits stay or go together (the
// reference sorts, so among equal logits it keeps whichever its sort puts first).  The reference seeds a generator with seed + sample_index per
// token; here the uniform number is a hash of (seed, sample_index), so a
// request's stream does not depend on the batch it is in.  Two kernels: a
// thread-block cluster per row that keeps the row in shared memory and finds the
// filters by radix selection (vocabularies up to 390,000), and one CTA per row that
// finds them by bisection on the bit pattern of the scaled logits, 32 passes over
// the row in global memory for each active filter (any vocabulary).
#include "common.cuh"
#include "no_alloc.h"

#include <mutex>

namespace einf {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ float keyed_uniform(unsigned long long seed, unsigned long long index) {
  unsigned long long z = splitmix(seed);
  z = splitmix(z ^ index);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// Block-wide argmax with ties to the lowest index.
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { sv[warp] = v; si[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    v = lane < warps ? sv[lane] : -INFINITY;
    idx = lane < warps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (lane == 0) { sv[0] = v; si[0] = idx; }
  }
  __syncthreads();
  v = sv[0];
  idx = si[0];
}

// Argmax in two steps so that a few rows still fill the GPU: kArgmaxChunks blocks per row
// write their (value, index) into `partial`; the block that finishes last for a row picks
// the winner.  `counters` is zero before the launch and zero after it.
constexpr int kArgmaxChunks = 32;
constexpr int kArgmaxThreads = 256;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ tokens, int vocab,
              float* __restrict__ partial_value, int* __restrict__ partial_index, int* __restrict__ counters) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int is_last;
  pdl_wait();
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int per = (vocab + kArgmaxChunks - 1) / kArgmaxChunks;
  const int begin = chunk * per, end = min(vocab, begin + per);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  block_argmax(best, best_i, sv, si);
  if (threadIdx.x == 0) {
    partial_value[r * kArgmaxChunks + chunk] = best;
    partial_index[r * kArgmaxChunks + chunk] = best_i;
    __threadfence();
    const int done = atomicAdd(counters + r, 1);
    is_last = done == kArgmaxChunks - 1;
    if (is_last) counters[r] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x < 32) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    if (threadIdx.x < kArgmaxChunks) {
      v = __ldcg(partial_value + r * kArgmaxChunks + threadIdx.x);
      idx = __ldcg(partial_index + r * kArgmaxChunks + threadIdx.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (threadIdx.x == 0) tokens[r] = idx == 0x7fffffff ? 0 : idx;
  }
}

struct SampleParams {
  const float* temperature;         // [rows]; 0 = greedy
  const int* top_k;                 // [rows]; 0 = off
  const float* top_p;               // [rows]; 1 = off
  const float* min_p;               // [rows]; 0 = off
  const unsigned long long* seed;   // [rows]
  const long long* sample_index;    // [rows]
};

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int* __restrict__ tokens, int vocab, SampleParams sp) {
  __shared__ float scratch[33];
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float chunk_sums[kSampleThreads];
  __shared__ int winner;
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const float temperature = sp.temperature[r];

  // Largest scaled logit and its index (also the greedy answer).
  const float inv_t = temperature > 0.f ? 1.f / temperature : 1.f;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  block_argmax(best, best_i, sv, si);
  if (temperature <= 0.f) {
    if (threadIdx.x == 0) tokens[r] = best_i == 0x7fffffff ? 0 : best_i;
    return;
  }
  const float max_scaled = best * inv_t;

  // A token is kept iff ordered_key(scaled) >= key_floor and exp(scaled - max) >= min_keep.
  unsigned key_floor = 0u;
  const int top_k = sp.top_k[r];
  if (top_k > 0 && top_k < vocab) {
    // Largest key with count(key >= it) >= k: the key of the k-th largest logit.
    unsigned prefix = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned candidate = prefix | (1u << bit);
      float count = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        count += ordered_key(row[i] * inv_t) >= candidate ? 1.f : 0.f;
      count = block_sum(count, scratch);
      if (count >= (float)top_k) prefix = candidate;
    }
    key_floor = prefix;
  }
  const float top_p = sp.top_p[r];
  if (top_p < 1.f) {
    float mass = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float s = row[i] * inv_t;
      if (ordered_key(s) >= key_floor) mass += expf(s - max_scaled);
    }
    mass = block_sum(mass, scratch);
    const float limit = top_p * mass;
    // Largest key u with mass(kept, key > u) > limit; tokens with key > u stay.
    unsigned low = 0u;
    bool any_false = false;
    {
      float above = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float s = row[i] * inv_t;
        const unsigned key = ordered_key(s);
        if (key >= key_floor && key > 0u) above += expf(s - max_scaled);
      }
      above = block_sum(above, scratch);
      any_false = above > limit;
    }
    if (any_false) {
      for (int bit = 31; bit >= 0; --bit) {
        const unsigned candidate = low | (1u << bit);
        float above = 0.f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
          const float s = row[i] * inv_t;
          const unsigned key = ordered_key(s);
          if (key >= key_floor && key > candidate) above += expf(s - max_scaled);
        }
        above = block_sum(above, scratch);
        if (above > limit) low = candidate;
      }
      if (low + 1u > key_floor) key_floor = low + 1u;
    }
  }
  const float min_keep = sp.min_p[r];

  // Inverse cumulative distribution over the kept tokens in index order: each
  // thread owns one contiguous chunk, so the order of additions is fixed.
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = threadIdx.x * chunk;
  const int end = min(vocab, begin + chunk);
  float local = 0.f;
  for (int i = begin; i < end; ++i) {
    const float s = row[i] * inv_t;
    const float e = expf(s - max_scaled);
    if (ordered_key(s) >= key_floor && e >= min_keep) local += e;
  }
  chunk_sums[threadIdx.x] = local;
  if (threadIdx.x == 0) winner = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < blockDim.x; ++i) total += chunk_sums[i];
    const float u = keyed_uniform(sp.seed[r], (unsigned long long)sp.sample_index[r]);
    const float target = u * total;
    float running = 0.f;
    int owner = -1;
    for (int i = 0; i < blockDim.x; ++i) {
      if (chunk_sums[i] > 0.f) {
        owner = i;  // the last chunk with mass takes the draw if rounding overshoots
        if (running + chunk_sums[i] > target) break;
        running += chunk_sums[i];
      }
    }
    winner = owner;
    scratch[0] = target - running;  // mass to walk inside the winning chunk
  }
  __syncthreads();
  if (threadIdx.x == winner) {
    float remaining = scratch[0];
    int chosen = -1;
    for (int i = begin; i < end; ++i) {
      const float s = row[i] * inv_t;
      const float e = expf(s - max_scaled);
      if (ordered_key(s) >= key_floor && e >= min_keep) {
        chosen = i;
        if (e > remaining) break;
        remaining -= e;
      }
    }
    tokens[r] = chosen < 0 ? best_i : chosen;
  }
  if (winner < 0 && threadIdx.x == 0) tokens[r] = best_i;
}

// ---------------------------------------------------------------------------
// The same draw by a thread-block cluster per row.  The kernel above walks a row 32 times per
// filter with one CTA (a 152,000-token row with top-k and top-p: 2.2 ms, three decode steps).
// Here the eight CTAs of a cluster each keep an eighth of the scaled row in shared memory, so the
// row comes from global memory once, and the filters are found by radix selection: four passes
// of eight bits over a 32-bit rank instead of 32 bisection steps, the 256-bin histograms of the
// CTAs added up through distributed shared memory.
//
// The rank of a token is q = (max - scaled) * 2^24, clamped to 32 bits: smaller is more probable,
// equal scaled logits have equal ranks, and tokens 256 or more below the maximum (whose weight
// is zero in 32-bit anyway) share the last rank.  Unlike the bits of the float itself, whose top
// byte is the same for almost the whole row, the top byte of q spreads a row over dozens of
// bins, so the histogram's atomics do not all meet in one place.
//   top-k keeps q <= Qk,  Qk = max{Q : #(q < Q) < k}          (ties at the k-th value are all kept)
//   top-p keeps q <= Qp,  Qp = max{Q : mass(q < Q) <= top_p * mass}  (among top-k's survivors: a token
//                          stays iff the mass of the strictly more probable ones has not reached the limit)
// Both are "the largest digit whose running total stays within a threshold", byte by byte.  Counts
// and masses are 64-bit integers (a weight is exp(scaled - max) * 2^40), so the order in which
// atomics arrive does not change a sum and the same row always gives the same token.
// The draw itself is the inverse cumulative distribution in index order, as above: CTAs own
// consecutive slices of the row, threads consecutive pieces of a slice, and every sum is made in
// a fixed order.
constexpr int kSampleCluster = 8;
constexpr int kSampleMaxCopies = 16;                                    // copies of a CTA's histogram: one per pair of warps
constexpr int kSampleBase = 2 * 256 * 8 + 256 * 8 + 64 * 4 + 16 * 8;     // hist[2][256], total[256], warp scratch, exchange; then copies[][256], then the slice
constexpr int kSampleMaxSlice = (200 * 1024 - kSampleBase - kSampleMaxCopies * 256 * 8) / 4;   // floats of a slice that fit an SM

__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t peer;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
  return peer;
}
// ordered by the cluster barriers around them
__device__ __forceinline__ unsigned long long ld_peer_u64(const unsigned long long* local, uint32_t rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(peer_address(local, rank)));
  return v;
}
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer_address(local, rank)));
  return v;
}
__device__ __forceinline__ int ld_peer_s32(const int* local, uint32_t rank) {
  int v;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(peer_address(local, rank)));
  return v;
}

__device__ __forceinline__ unsigned rank_of(float scaled, float max_scaled) {
  const float d = (max_scaled - scaled) * 16777216.f;           // >= 0; NaN compares false below and takes the last rank
  return d < 4294967040.f ? (unsigned)d : 0xffffffffu;
}
__device__ __forceinline__ unsigned long long fixed_weight(float scaled, float max_scaled) {
  return (unsigned long long)(expf(scaled - max_scaled) * 1099511627776.f);   // 2^40
}

// One radix selection over the cluster's row: the largest 32-bit Q with total(q < Q) <= threshold,
// where total adds weight(i) over the tokens with q_i <= q_limit.  kMass: weights are fixed-point
// probabilities; otherwise every token weighs 1.
// One pass of a radix selection over the cluster's row.  Among the tokens with q <= q_limit whose
// bits from `match_shift` up equal `prefix` (all of them if match_shift is 32), a histogram of the
// digit (q >> shift) & 255 (or, `saturate`: of min(q >> shift, 255)) is added up over the cluster;
// returns the largest digit whose running total, `below` included, stays within the threshold,
// and moves `below` on to that digit's start.  kMass: a token weighs its fixed-point probability;
// otherwise 1.
template <bool kMass, int kCopies>
__device__ unsigned radix_pass(const float* slice, int n, float max_scaled, unsigned q_limit, int shift, bool saturate,
                               int match_shift, unsigned prefix, unsigned long long threshold,
                               unsigned long long& below, unsigned long long (*hist)[256],
                               unsigned long long (*copies)[256], unsigned long long* total,
                               unsigned long long* carry, int& buffer) {
  unsigned long long* mine = hist[buffer];
  // Atomics to one address take turns, and where most of a row lies in a handful of bins that is
  // most of a pass: every two warps have a histogram of their own (a row of 152,000 tokens: 24 us
  // for such a pass with one histogram per CTA; adding up among the lanes of a warp first, with
  // match.any and a reduction over the matching lanes, took longer than the atomics it saved),
  // added up before the cluster sees it.
  unsigned long long* copy = copies[threadIdx.x >> 6];
  for (int b = threadIdx.x; b < kCopies * 256; b += blockDim.x) copies[0][b] = 0ull;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float s = slice[i];
    const unsigned q = rank_of(s, max_scaled);
    if (q > q_limit || (match_shift < 32 && (q >> match_shift) != prefix)) continue;
    const unsigned digit = saturate ? min(q >> shift, 255u) : (q >> shift) & 255u;
    atomicAdd(&copy[digit], kMass ? fixed_weight(s, max_scaled) : 1ull);
  }
  __syncthreads();
  if (threadIdx.x < 256) {
    unsigned long long sum = 0ull;
#pragma unroll
    for (int j = 0; j < kCopies; ++j) sum += copies[j][threadIdx.x];
    mine[threadIdx.x] = sum;
  }
  __syncthreads();
  cluster_barrier();
  if (threadIdx.x < 256) {
    unsigned long long sum = 0ull;
    for (uint32_t c = 0; c < kSampleCluster; ++c) sum += ld_peer_u64(mine + threadIdx.x, c);
    total[threadIdx.x] = sum;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // lane l owns bins 8l .. 8l+7: running totals in bin order, then the largest bin whose running
    // total (everything below it) stays within the threshold
    const int lane = threadIdx.x;
    unsigned long long own = 0ull;
    for (int b = 0; b < 8; ++b) own += total[lane * 8 + b];
    unsigned long long before = own;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long other = __shfl_up_sync(0xffffffffu, before, o);
      if (lane >= o) before += other;
    }
    before = below + before - own;                      // total below this lane's first bin
    int found = -1;
    unsigned long long found_below = 0ull, running = before;
    for (int b = 0; b < 8; ++b) {
      if (running <= threshold) {
        found = lane * 8 + b;
        found_below = running;
      }
      running += total[lane * 8 + b];
    }
    int best = found;
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    // bin 0 always qualifies while `below` does (it does: a selection starts from 0 <= threshold)
    if (found == best && best >= 0) {
      carry[0] = (unsigned long long)best;
      carry[1] = found_below;
    }
  }
  __syncthreads();
  below = carry[1];
  buffer ^= 1;   // the other histogram next: peers may still be reading this one
  return (unsigned)carry[0];
}

// The largest 32-bit Q with total(q < Q) <= threshold, where total adds the weights of the tokens
// with q_i <= q_limit.  The top byte of q counts whole units below the maximum, and a model's row
// has most of its tokens within a few units of one another: a first pass on that byte would send
// them all to a handful of bins.  So the first pass takes eight bits from bit 21 up (an eighth of a
// unit per bin, the row spread over dozens of bins) with everything from 32 units below the
// maximum on in the last bin; three passes resolve the 21 bits below.  Only a selection that ends
// in that last bin (a k larger than the number of tokens within 32 units of the maximum) is done
// again byte by byte from the top.
template <bool kMass, int kCopies>
__device__ unsigned radix_select(const float* slice, int n, float max_scaled, unsigned q_limit,
                                 unsigned long long threshold, unsigned long long (*hist)[256],
                                 unsigned long long (*copies)[256], unsigned long long* total,
                                 unsigned long long* carry, int& buffer) {
  unsigned long long below = 0ull;   // total of the tokens whose rank lies below the range of the prefix
  auto pass = [&](int shift, bool saturate, int match_shift, unsigned prefix) {
    return radix_pass<kMass, kCopies>(slice, n, max_scaled, q_limit, shift, saturate, match_shift, prefix, threshold, below, hist,
                             copies, total, carry, buffer);
  };
  unsigned prefix = pass(21, true, 32, 0u);
  if (prefix < 255u) {
    prefix = (prefix << 8) | pass(13, false, 21, prefix);
    prefix = (prefix << 8) | pass(5, false, 13, prefix);
    return (prefix << 5) | (pass(0, false, 5, prefix) & 31u);   // the lowest five bits: digits 0 .. 31
  }
  below = 0ull;
  prefix = pass(24, false, 32, 0u);
  prefix = (prefix << 8) | pass(16, false, 24, prefix);
  prefix = (prefix << 8) | pass(8, false, 16, prefix);
  return (prefix << 8) | pass(0, false, 8, prefix);
}

template <int kThreads>
__global__ void __launch_bounds__(kThreads)
sample_cluster_kernel(const float* __restrict__ logits, int* __restrict__ tokens, int vocab, int slice_len, SampleParams sp) {
  extern __shared__ __align__(16) unsigned char sample_smem[];
  auto hist = reinterpret_cast<unsigned long long(*)[256]>(sample_smem);
  unsigned long long* total = reinterpret_cast<unsigned long long*>(sample_smem + 2 * 256 * 8);
  float* wv = reinterpret_cast<float*>(sample_smem + 3 * 256 * 8);          // 32 floats
  int* wi = reinterpret_cast<int*>(wv + 32);                                // 32 ints
  unsigned long long* carry = reinterpret_cast<unsigned long long*>(sample_smem + 3 * 256 * 8 + 64 * 4);   // 2
  unsigned long long* my_mass = carry + 2;                                  // what peers read: fixed-point mass,
  float* my_best = reinterpret_cast<float*>(carry + 3);                     // largest scaled logit,
  int* my_best_i = reinterpret_cast<int*>(carry + 4);                       // its index,
  float* my_total = reinterpret_cast<float*>(carry + 5);                    // kept mass of the final draw
  auto copies = reinterpret_cast<unsigned long long(*)[256]>(sample_smem + 3 * 256 * 8 + 64 * 4 + 16 * 8);
  constexpr int kCopies = kThreads / 64;
  float* slice = reinterpret_cast<float*>(sample_smem + kSampleBase + kCopies * 256 * 8);
  __shared__ float warp_totals[32];

  pdl_wait();
  const int r = blockIdx.x / kSampleCluster;
  const uint32_t rank = cluster_ctarank();
  const float* row = logits + (size_t)r * vocab;
  const float temperature = sp.temperature[r];
  const float inv_t = temperature > 0.f ? 1.f / temperature : 1.f;
  const int first = (int)rank * slice_len;
  const int n = max(0, min(vocab - first, slice_len));

  // The slice, scaled, into shared memory; the largest scaled logit of the row and its first index.
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float raw = row[first + i];
    slice[i] = raw * inv_t;
    if (raw > best) { best = raw; best_i = first + i; }   // indices rise within a thread: the first largest stays
  }
  block_argmax(best, best_i, wv, wi);
  if (threadIdx.x == 0) {
    *my_best = best;
    *my_best_i = best_i;
  }
  cluster_barrier();
  for (uint32_t c = 0; c < kSampleCluster; ++c) {
    const float v = ld_peer_f32(my_best, c);
    const int vi = ld_peer_s32(my_best_i, c);
    if (c == 0 || v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
  }
  if (best_i == 0x7fffffff) best_i = 0;
  if (temperature <= 0.f) {
    if (rank == 0 && threadIdx.x == 0) tokens[r] = best_i;
    cluster_barrier();   // no CTA leaves while a peer may still read its shared memory
    return;
  }
  const float max_scaled = best * inv_t;
  int buffer = 0;
  unsigned q_keep = 0xffffffffu;
  const int top_k = sp.top_k[r];
  if (top_k > 0 && top_k < vocab)
    q_keep = radix_select<false, kCopies>(slice, n, max_scaled, q_keep, (unsigned long long)top_k - 1ull, hist, copies, total, carry, buffer);
  const float top_p = sp.top_p[r];
  if (top_p < 1.f) {
    // the mass of top-k's survivors, then the rank at which the more probable tokens reach top_p of it
    unsigned long long mass = 0ull;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float s = slice[i];
      if (rank_of(s, max_scaled) <= q_keep) mass += fixed_weight(s, max_scaled);
    }
    for (int o = 16; o > 0; o >>= 1) mass += __shfl_xor_sync(0xffffffffu, mass, o);
    __syncthreads();
    if (threadIdx.x == 0) *my_mass = 0ull;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) atomicAdd(my_mass, mass);   // integers: any order, one sum
    __syncthreads();
    cluster_barrier();
    unsigned long long all = 0ull;
    for (uint32_t c = 0; c < kSampleCluster; ++c) all += ld_peer_u64(my_mass, c);
    const unsigned long long limit = (unsigned long long)((double)top_p * (double)all);
    const unsigned q_p = radix_select<true, kCopies>(slice, n, max_scaled, q_keep, limit, hist, copies, total, carry, buffer);
    q_keep = min(q_keep, q_p);
  }
  const float min_keep = sp.min_p[r];

  // Inverse cumulative distribution over the kept tokens in index order.  A thread owns a run of
  // consecutive tokens of the slice; running sums over threads, then over CTAs, in a fixed order.
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int begin = min(n, (int)threadIdx.x * per), end = min(n, begin + per);
  auto weight = [&](int i) {
    const float s = slice[i];
    const float e = expf(s - max_scaled);
    return (rank_of(s, max_scaled) <= q_keep && e >= min_keep) ? e : 0.f;
  };
  float local = 0.f;
  for (int i = begin; i < end; ++i) local += weight(i);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inclusive = local;
  for (int o = 1; o < 32; o <<= 1) {
    const float other = __shfl_up_sync(0xffffffffu, inclusive, o);
    if (lane >= o) inclusive += other;
  }
  if (lane == 31) warp_totals[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    float t = lane < kThreads / 32 ? warp_totals[lane] : 0.f;
    float inc = t;
    for (int o = 1; o < 32; o <<= 1) {
      const float other = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += other;
    }
    warp_totals[lane] = inc - t;            // total of the warps before this one
    if (lane == 31) *my_total = inc;        // this CTA's kept mass
  }
  __syncthreads();
  const float before_thread = warp_totals[warp] + inclusive - local;   // kept mass of this CTA before this thread
  cluster_barrier();
  float before_cta = 0.f, all = 0.f;
  for (uint32_t c = 0; c < kSampleCluster; ++c) {
    const float t = ld_peer_f32(my_total, c);
    if (c < rank) before_cta += t;
    all += t;
  }
  const float u = keyed_uniform(sp.seed[r], (unsigned long long)sp.sample_index[r]);
  const float target = u * all;
  // The CTA that owns the draw: the last one with mass whose running total has not passed the
  // target (so that a draw that rounding pushes past the end still lands on a kept token).
  float running = 0.f;
  int owner = -1;
  for (uint32_t c = 0; c < kSampleCluster; ++c) {
    const float t = ld_peer_f32(my_total, c);
    if (t > 0.f && (owner < 0 || running <= target)) owner = (int)c;
    running += t;
  }
  if (owner < 0) {
    if (rank == 0 && threadIdx.x == 0) tokens[r] = best_i;   // nothing was kept (cannot happen: the maximum always is)
  } else if ((int)rank == owner) {
    const float inside = target - before_cta;
    // the owning thread by the same rule, found by every thread for itself
    const bool mine = local > 0.f && before_thread <= inside;
    // the last such thread: a ballot per warp, the highest warp wins
    __shared__ int owner_thread;
    if (threadIdx.x == 0) owner_thread = -1;
    __syncthreads();
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    if (ballot != 0u && lane == 31 - __clz(ballot)) atomicMax(&owner_thread, (int)threadIdx.x);
    __syncthreads();
    int chosen_thread = owner_thread;
    if (chosen_thread < 0) {
      // rounding put the target before the first kept token of this CTA: the first thread with mass takes it
      const unsigned any = __ballot_sync(0xffffffffu, local > 0.f);
      __shared__ int first_thread;
      if (threadIdx.x == 0) first_thread = 0x7fffffff;
      __syncthreads();
      if (any != 0u && lane == __ffs(any) - 1) atomicMin(&first_thread, (int)threadIdx.x);
      __syncthreads();
      chosen_thread = first_thread;
    }
    if ((int)threadIdx.x == chosen_thread) {
      float remaining = inside - before_thread;
      int chosen = -1;
      for (int i = begin; i < end; ++i) {
        const float e = weight(i);
        if (e > 0.f) {
          chosen = i;
          if (e > remaining) break;
          remaining -= e;
        }
      }
      tokens[r] = chosen < 0 ? best_i : first + chosen;
    }
  }
  cluster_barrier();   // no CTA leaves while a peer may still read its shared memory
}

// The step's report to the host: the sampled tokens and the status word, written by the device
// straight into pinned host memory (one launch instead of two copies on the device and one to
// the host).
__global__ void report_kernel(const int* __restrict__ tokens, int count, const int* __restrict__ status,
                              int* __restrict__ host) {
  for (int i = threadIdx.x; i < count; i += blockDim.x) host[i] = tokens[i];
  if (threadIdx.x == 0) host[count] = status[0];
}

}  // namespace einf

using namespace einf;

// host: pinned host memory of at least count + 1 ints that the device can address (memory
// from cudaHostAlloc is, under unified addressing); refused with an error otherwise.
extern "C" int einf_report(const int* tokens, int count, const int* status, int* host, cudaStream_t stream) {
  if (count < 0) return (int)cudaErrorInvalidValue;
  int* mapped = nullptr;
  cudaError_t e = cudaHostGetDevicePointer((void**)&mapped, host, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return (int)e;
  }
  report_kernel<<<1, 128, 0, stream>>>(tokens, count, status, mapped);
  return (int)cudaGetLastError();
}

// Scratch of einf_argmax for `rows` rows: 32 (value, index) pairs and one counter per row.
extern "C" long long einf_argmax_workspace_bytes(int rows) { return (long long)rows * (kArgmaxChunks * 8 + 4); }

extern "C" int einf_argmax(const float* logits, int* tokens, int rows, int vocab, float* partial_value,
                           int* partial_index, int* counters, cudaStream_t stream) {
  if (rows == 0) return 0;
  return (int)launch_pdl(argmax_kernel, dim3(kArgmaxChunks, rows), kArgmaxThreads, 0, stream, logits, tokens, vocab,
                         partial_value, partial_index, counters);
}

extern "C" int einf_sample(const float* logits, int* tokens, int rows, int vocab, const float* temperature,
                           const int* top_k, const float* top_p, const float* min_p,
                           const unsigned long long* seed, const long long* sample_index,
                           cudaStream_t stream) {
  if (rows == 0) return 0;
  SampleParams sp{temperature, top_k, top_p, min_p, seed, sample_index};
  // A cluster per row where an eighth of a row fits one SM's shared memory (vocabularies up to
  // 390,000); one CTA per row that reads the row from global memory in every pass otherwise.
  const int slice_len = (vocab + kSampleCluster - 1) / kSampleCluster;
  if (slice_len <= kSampleMaxSlice) {
    // 1,024 threads a CTA for a few rows (one CTA fills an SM's registers: the device holds 15
    // clusters at once); 512 threads from 16 rows on, where two CTAs share an SM and 64 rows are
    // three waves instead of five.
    const int threads = rows >= 16 ? 512 : 1024;
    const size_t smem = (size_t)kSampleBase + (size_t)(threads / 64) * 256 * 8 + (size_t)slice_len * sizeof(float);
    auto kernel = threads == 512 ? sample_cluster_kernel<512> : sample_cluster_kernel<1024>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl_cluster(kernel, dim3(rows * kSampleCluster), dim3(threads), smem, kSampleCluster, stream, logits,
                                   tokens, vocab, slice_len, sp);
  }
  sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, tokens, vocab, sp);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// einf_argmax_no_alloc (declared and specified in no_alloc.h): the same kernel as
// einf_argmax, with its scratch in a device array of this file instead of a
// buffer from an allocator.
// ---------------------------------------------------------------------------
namespace {

struct ArgmaxScratch {
  float value[EINF_ARGMAX_NO_ALLOC_MAX_ROWS * kArgmaxChunks];
  int index[EINF_ARGMAX_NO_ALLOC_MAX_ROWS * kArgmaxChunks];
  int counters[EINF_ARGMAX_NO_ALLOC_MAX_ROWS];
};

// One copy per device that loads this library; zero when the module is loaded.
static __device__ __align__(256) unsigned char argmax_scratch[sizeof(ArgmaxScratch)];

constexpr int kMaxDevices = 64;
std::mutex scratch_mutex;
ArgmaxScratch* scratch_of_device[kMaxDevices] = {};

// The device address of argmax_scratch on the current device.  In host code the name
// `argmax_scratch` is only a handle for the runtime, not an address a kernel could use,
// so it is translated once per device and remembered.
cudaError_t scratch_for_current_device(ArgmaxScratch** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(scratch_mutex);
  if (scratch_of_device[device] == nullptr) {
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, argmax_scratch);
    if (e != cudaSuccess) return e;
    scratch_of_device[device] = static_cast<ArgmaxScratch*>(address);
  }
  *out = scratch_of_device[device];
  return cudaSuccess;
}

}  // namespace

extern "C" int einf_argmax_no_alloc(const float* logits, int* tokens, int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || (rows > 0 && (logits == nullptr || tokens == nullptr)))
    return EINF_NO_ALLOC_BAD_ARGUMENT;
  if (rows > EINF_ARGMAX_NO_ALLOC_MAX_ROWS) return EINF_NO_ALLOC_TOO_MANY_ROWS;
  if (rows == 0) return 0;
  ArgmaxScratch* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return (int)e;
  // The kernel leaves its counters at zero, but a call that was cut short would not have:
  // start every call from zero.  The partial pairs are written before they are read.
  e = cudaMemsetAsync(scratch->counters, 0, sizeof(int) * rows, stream);
  if (e != cudaSuccess) return (int)e;
  argmax_kernel<<<dim3(kArgmaxChunks, rows), kArgmaxThreads, 0, stream>>>(logits, tokens, vocab, scratch->value,
                                                                         scratch->index, scratch->counters);
  return (int)cudaGetLastError();
}

extern "C" const char* einf_argmax_no_alloc_strerror(int code) {
  if (code == 0) return "success";
  if (code == EINF_NO_ALLOC_TOO_MANY_ROWS)
    return "einf_argmax_no_alloc: more rows than EINF_ARGMAX_NO_ALLOC_MAX_ROWS (256); its scratch is a fixed "
           "device array, so split the batch or use einf_argmax with a workspace of your own";
  if (code == EINF_NO_ALLOC_BAD_ARGUMENT)
    return "einf_argmax_no_alloc: null pointer, negative row count or non-positive vocabulary size";
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "einf_argmax_no_alloc: unknown error code";
}
