// Token selection from float logits [rows, vocab]: argmax, and temperature
// sampling with top-k, top-p and min-p filters and a counter-based generator.
//
// Semantics follow src/einf/executors/torch/sampler.py:21-102 of the reference:
// greedy rows (temperature 0) take the first largest index; other rows divide
// the logits by the temperature, keep the k largest, keep the smallest set of
// most probable tokens whose mass reaches top_p (the crossing token included),
// drop tokens whose probability is below min_p times the largest, and draw from
// what is left.  The reference seeds a generator with seed + sample_index per
// token; here the uniform number is a hash of (seed, sample_index), so a
// request's stream does not depend on the batch it is in.  The filters are
// found by bisection on the bit pattern of the scaled logits instead of a sort:
// 32 passes over the row for each active filter.
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
