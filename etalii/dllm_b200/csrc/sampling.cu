// Token choice on the device, one block per row of logits.
//   temperature 0: the first index of the largest logit.
//   temperature > 0: z = float(logit / float(T)); p = float(exp(z - max) / sum) with the exponentials and the sum in
//   double; candidates in the total order (p descending, id ascending); top-k keeps the first k, top-p the shortest
//   prefix whose mass reaches it, min-p drops candidates below min_p * p_max; one double in [0,1) from the row's own
//   xoshiro256** state, scaled by the kept mass, picks the first candidate whose running sum exceeds it.
// The order is never materialised: a prefix of it is found by descending the 32 bits of p eight bits at a time
// with counting histograms; masses are summed as 64-bit fixed point (2^-62 units), so every sum is exact integer
// arithmetic, independent of the order of the atomic adds, and a row's choice is reproducible.
// Scratch: one float per logit (the probabilities), given by the caller.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;
constexpr double FX_ONE = 4611686018427387904.0;  // 2^62

enum { FIND_COUNT = 0, FIND_MASS_GE = 1, FIND_MASS_GT = 2 };

struct Found {
  unsigned bits;             // the probability (as bits) of the element at the boundary
  unsigned long long rank;   // how many of the elements with exactly that probability are included (by id), >= 1
  unsigned long long above_count, above_mass, tie_count, tie_mass;
  int ok;
};

struct Shared {
  unsigned count[256];
  unsigned long long mass[256];
  unsigned long long scan_count[256];
  unsigned long long scan_mass[256];
  Found found;
  double reduce_d[32];
  float reduce_f[32];
  int reduce_i[32];
  unsigned tie_counts[THREADS];
};

__device__ __forceinline__ unsigned long long to_fx(float p) { return (unsigned long long)((double)p * FX_ONE); }

// Finds the boundary element of the prefix of the order (p descending, id ascending) at which the count reaches
// `target` (FIND_COUNT), the mass reaches it (FIND_MASS_GE) or exceeds it (FIND_MASS_GT).
__device__ void find_prefix(const float* __restrict__ p, int vocab, int kind, unsigned long long target, Shared& sh) {
  unsigned prefix = 0;
  unsigned long long above_count = 0, above_mass = 0;
  int tid = threadIdx.x;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) { sh.count[tid] = 0; sh.mass[tid] = 0; }
    if (tid == 0) sh.found.ok = 0;
    __syncthreads();
    for (int i = tid; i < vocab; i += THREADS) {
      unsigned bits = __float_as_uint(p[i]);
      if (shift == 24 || (bits >> (shift + 8)) == prefix) {
        unsigned bin = (bits >> shift) & 255u;
        atomicAdd(&sh.count[bin], 1u);
        atomicAdd(&sh.mass[bin], to_fx(p[i]));
      }
    }
    __syncthreads();
    // exclusive suffix sums over the bins (higher bins come first in the order)
    if (tid < 256) { sh.scan_count[tid] = sh.count[tid]; sh.scan_mass[tid] = sh.mass[tid]; }
    __syncthreads();
    for (int step = 1; step < 256; step <<= 1) {
      unsigned long long c = 0, m = 0;
      if (tid < 256 && tid + step < 256) { c = sh.scan_count[tid + step]; m = sh.scan_mass[tid + step]; }
      __syncthreads();
      if (tid < 256) { sh.scan_count[tid] += c; sh.scan_mass[tid] += m; }
      __syncthreads();
    }
    if (tid < 256 && sh.count[tid] > 0) {
      unsigned long long ac = above_count + sh.scan_count[tid] - sh.count[tid];
      unsigned long long am = above_mass + sh.scan_mass[tid] - sh.mass[tid];
      bool hit;
      if (kind == FIND_COUNT) hit = ac < target && target <= ac + sh.count[tid];
      else if (kind == FIND_MASS_GE) hit = am < target && target <= am + sh.mass[tid];
      else hit = am <= target && target < am + sh.mass[tid];
      if (hit) {
        sh.found.ok = 1;
        sh.found.bits = (prefix << 8) | (unsigned)tid;
        sh.found.above_count = ac;
        sh.found.above_mass = am;
        sh.found.tie_count = sh.count[tid];
        sh.found.tie_mass = sh.mass[tid];
      }
    }
    __syncthreads();
    if (!sh.found.ok) return;  // the whole vocabulary does not reach the target
    prefix = sh.found.bits;
    above_count = sh.found.above_count;
    above_mass = sh.found.above_mass;
    __syncthreads();
  }
  if (tid == 0) {
    Found& f = sh.found;
    unsigned long long each = f.tie_count ? f.tie_mass / f.tie_count : 0;
    unsigned long long rank;
    if (kind == FIND_COUNT) rank = target - f.above_count;
    else if (each == 0) rank = 1;
    else if (kind == FIND_MASS_GE) rank = (target - f.above_mass + each - 1) / each;
    else rank = (target - f.above_mass) / each + 1;
    if (rank < 1) rank = 1;
    if (rank > f.tie_count) rank = f.tie_count;
    f.rank = rank;
  }
  __syncthreads();
}

__device__ __forceinline__ unsigned long long rotl64(unsigned long long x, int k) { return (x << k) | (x >> (64 - k)); }

__device__ double next_double(unsigned long long* s) {  // xoshiro256**, top 53 bits times 2^-53
  unsigned long long result = rotl64(s[1] * 5ull, 7) * 9ull;
  unsigned long long t = s[1] << 17;
  s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
  s[2] ^= t;
  s[3] = rotl64(s[3], 45);
  return (double)(result >> 11) * (1.0 / 9007199254740992.0);
}

__device__ double block_sum_d(double v, Shared& sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh.reduce_d[warp] = v;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < THREADS / 32; ++i) total += sh.reduce_d[i];  // same order in every thread
  return total;
}

// (value, index) maximum; ties go to the lower index
__device__ void block_argmax(float& v, int& idx, Shared& sh) {
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) { sh.reduce_f[warp] = v; sh.reduce_i[warp] = idx; }
  __syncthreads();
  v = sh.reduce_f[0]; idx = sh.reduce_i[0];
  for (int i = 1; i < THREADS / 32; ++i) {
    float ov = sh.reduce_f[i];
    int oi = sh.reduce_i[i];
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
}

__global__ void __launch_bounds__(THREADS) sample_kernel(
    int* __restrict__ out_tokens, const float* __restrict__ logits, long long row_stride, int vocab,
    float* __restrict__ scratch, unsigned long long* __restrict__ rng, const int* __restrict__ rng_rows,
    float temperature, int top_k, double top_p, double min_p) {
  __shared__ Shared sh;
  int row = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const float* l = logits + (size_t)row * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  if (temperature == 0.f) {
    for (int i = tid; i < vocab; i += THREADS) {
      float v = l[i];
      if (v > best) { best = v; best_i = i; }
    }
    block_argmax(best, best_i, sh);
    if (tid == 0) out_tokens[row] = best_i == 0x7fffffff ? 0 : best_i;
    return;
  }
  float* p = scratch + (size_t)row * vocab;
  for (int i = tid; i < vocab; i += THREADS) {
    float z = __fdiv_rn(l[i], temperature);
    p[i] = z;
    if (z > best) { best = z; best_i = i; }
  }
  block_argmax(best, best_i, sh);
  double partial = 0.0;
  for (int i = tid; i < vocab; i += THREADS) partial += exp((double)p[i] - (double)best);
  double inverse = 1.0 / block_sum_d(partial, sh);
  for (int i = tid; i < vocab; i += THREADS) p[i] = (float)(exp((double)p[i] - (double)best) * inverse);
  __syncthreads();

  unsigned long long keep = (unsigned long long)vocab;
  if (top_k > 0 && (unsigned long long)top_k < keep) keep = (unsigned long long)top_k;
  if (top_p < 1.0) {
    find_prefix(p, vocab, FIND_MASS_GE, (unsigned long long)(top_p * FX_ONE), sh);
    if (sh.found.ok) {
      unsigned long long n = sh.found.above_count + sh.found.rank;
      if (n < keep) keep = n;
    }
    __syncthreads();
  }
  if (min_p > 0.0) {
    double floor_p = min_p * (double)p[best_i];
    unsigned local = 0;
    for (int i = tid; i < vocab; i += THREADS) local += ((double)p[i] >= floor_p) ? 1u : 0u;
    unsigned long long n = (unsigned long long)block_sum_d((double)local, sh);
    if (n >= 1 && n < keep) keep = n;
  }
  find_prefix(p, vocab, FIND_COUNT, keep, sh);
  unsigned long long each = sh.found.tie_count ? sh.found.tie_mass / sh.found.tie_count : 0;
  unsigned long long total = sh.found.above_mass + sh.found.rank * each;
  __syncthreads();
  unsigned long long* state = rng + (size_t)rng_rows[row] * 4;
  double u;
  if (tid == 0) {
    unsigned long long s[4] = {state[0], state[1], state[2], state[3]};
    u = next_double(s);
    state[0] = s[0]; state[1] = s[1]; state[2] = s[2]; state[3] = s[3];
    sh.reduce_d[0] = u;
  }
  __syncthreads();
  u = sh.reduce_d[0];
  unsigned long long target = (unsigned long long)(u * (double)total);
  if (total > 0 && target >= total) target = total - 1;
  __syncthreads();
  find_prefix(p, vocab, FIND_MASS_GT, target, sh);
  unsigned want_bits;
  unsigned long long want_rank;
  if (sh.found.ok) {
    want_bits = sh.found.bits;
    want_rank = sh.found.rank;
    // never beyond the kept prefix
    unsigned long long position = sh.found.above_count + sh.found.rank;
    if (position > keep) want_rank = keep > sh.found.above_count ? keep - sh.found.above_count : 1;
  } else {  // nothing exceeds the target (all mass is zero): the reference takes the last kept candidate
    __syncthreads();
    find_prefix(p, vocab, FIND_COUNT, keep, sh);
    want_bits = sh.found.bits;
    want_rank = sh.found.rank;
  }
  __syncthreads();
  // the want_rank-th id, ascending, among the elements whose probability has exactly want_bits
  int chunk = (vocab + THREADS - 1) / THREADS;
  int lo = min(tid * chunk, vocab), hi = min(lo + chunk, vocab);
  unsigned mine = 0;
  for (int i = lo; i < hi; ++i) mine += __float_as_uint(p[i]) == want_bits ? 1u : 0u;
  sh.tie_counts[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    unsigned long long seen = 0;
    int owner = THREADS - 1;
    for (int i = 0; i < THREADS; ++i) {
      if (seen + sh.tie_counts[i] >= want_rank) { owner = i; break; }
      seen += sh.tie_counts[i];
    }
    sh.reduce_i[0] = owner;
    sh.found.above_count = seen;
  }
  __syncthreads();
  if (tid == sh.reduce_i[0]) {
    unsigned long long seen = sh.found.above_count;
    int chosen = best_i;
    for (int i = lo; i < hi; ++i) {
      if (__float_as_uint(p[i]) == want_bits && ++seen == want_rank) { chosen = i; break; }
    }
    out_tokens[row] = chosen;
  }
}

__global__ void seed_kernel(unsigned long long* rng, const int* rows, const unsigned long long* seeds, int count) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  unsigned long long state = seeds[i];
  unsigned long long* s = rng + (size_t)rows[i] * 4;
  for (int w = 0; w < 4; ++w) {  // SplitMix64
    state += 0x9E3779B97F4A7C15ull;
    unsigned long long z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    s[w] = z ^ (z >> 31);
  }
}
}  // namespace

// Chooses one token per row of logits[rows, vocab] (row stride given). `scratch` holds rows * vocab floats.
// `rng` holds 4 words of state per sequence; row r uses and advances rng[rng_rows[r]].
DLLM_EXPORT int dllm_sample(int* out_tokens, const float* logits, long long row_stride, int rows, int vocab,
                            float* scratch, unsigned long long* rng, const int* rng_rows, float temperature,
                            int top_k, double top_p, double min_p, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (vocab <= 0 || temperature < 0.f || !(top_p > 0.0) || min_p < 0.0 || top_k < 0) return DLLM_BAD_ARGUMENT;
  if (temperature > 0.f && (scratch == nullptr || rng == nullptr || rng_rows == nullptr)) return DLLM_BAD_ARGUMENT;
  return dllm_launch_pdl(sample_kernel, dim3(rows), dim3(THREADS), 0, stream, out_tokens, logits, row_stride, vocab,
                         scratch, rng, rng_rows, temperature, top_k, top_p, min_p);
}

// rng[rows[i]] = xoshiro256** state from SplitMix64(seeds[i]).
DLLM_EXPORT int dllm_seed_rng(unsigned long long* rng, const int* rows, const unsigned long long* seeds, int count,
                              cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  seed_kernel<<<(count + 127) / 128, 128, 0, stream>>>(rng, rows, seeds, count);
  return dllm_launch_status();
}
