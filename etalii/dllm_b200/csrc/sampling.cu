// Token choice on the device, one block per row of logits.
//   temperature 0: the first index of the largest logit.
//   temperature > 0: z = float(logit / float(T)); p = float(exp(z - max) / sum) with the exponentials and the sum in
//   double; candidates in the total order (p descending, id ascending); top-k keeps the first k, top-p the shortest
//   prefix whose mass reaches it, min-p drops candidates below min_p * p_max; one double in [0,1) from the row's own
//   xoshiro256** state, scaled by the kept mass, picks the first candidate whose running sum exceeds it.
// The order is never materialised: a prefix of it is found by descending the bits of p four at a time with counting
// histograms (private to each thread, then summed in a fixed order); masses are summed as 64-bit fixed point (2^-62
// units), so every sum is exact integer arithmetic and a row's choice is reproducible.
// Scratch, given by the caller: per logit one float (the probability) and one double (the exponential).
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

constexpr int BINS = 16;  // four bits of the key per pass

struct Shared {
  unsigned long long count[BINS];
  unsigned long long mass[BINS];
  unsigned long long part_count[BINS][THREADS / BINS];
  unsigned long long part_mass[BINS][THREADS / BINS];
  Found found;
  double reduce_d[32];
  float reduce_f[32];
  int reduce_i[32];
  unsigned tie_counts[THREADS];
};

// p * 2^62 truncated, for 0 <= p <= 1, by integer shifts of the mantissa (the same value as the double product).
__device__ __forceinline__ unsigned long long to_fx(float p) {
  unsigned bits = __float_as_uint(p);
  int exponent = (int)(bits >> 23) & 255;
  if (exponent == 0) return 0ull;  // zero and subnormals are below 2^-62
  unsigned long long mantissa = (unsigned long long)((bits & 0x7FFFFFu) | 0x800000u);
  int shift = exponent - 88;       // value = mantissa * 2^(exponent - 150); times 2^62
  return shift >= 0 ? mantissa << shift : (shift > -24 ? mantissa >> (-shift) : 0ull);
}

// Finds the boundary element of the prefix of the order (p descending, id ascending) at which the count reaches
// `target` (FIND_COUNT), the mass reaches it (FIND_MASS_GE) or exceeds it (FIND_MASS_GT).
// Probabilities are not negative, so the key is their bits shifted left by one (the sign gone), taken four bits at a
// time from the top. Every thread counts into 16 bins of its own in shared memory (hist_count[bin][thread],
// hist_mass[bin][thread]: no atomics, no bank conflicts: most probabilities share their leading bits and would queue
// on a handful of shared counters), then the bins are summed over the threads in two fixed stages.
__device__ void find_prefix(const float* __restrict__ p, int vocab, int kind, unsigned long long target, Shared& sh,
                            unsigned* __restrict__ hist_count, unsigned long long* __restrict__ hist_mass) {
  unsigned prefix = 0;
  unsigned long long above_count = 0, above_mass = 0;
  int tid = threadIdx.x;
  for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
    for (int bin = 0; bin < BINS; ++bin) {
      hist_count[bin * THREADS + tid] = 0u;
      hist_mass[bin * THREADS + tid] = 0ull;
    }
    if (tid == 0) sh.found.ok = 0;
    for (int i0 = tid; i0 < vocab; i0 += 8 * THREADS) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = i0 + u * THREADS < vocab ? p[i0 + u * THREADS] : -1.f;  // loads first
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        unsigned key = __float_as_uint(v[u]) << 1;
        if (v[u] >= 0.f && (shift == 28 || (key >> (shift + 4)) == prefix)) {
          unsigned bin = (key >> shift) & 15u;
          hist_count[bin * THREADS + tid] += 1u;
          hist_mass[bin * THREADS + tid] += to_fx(v[u]);
        }
      }
    }
    __syncthreads();
    {  // stage 1: thread t adds 16 threads' counters of bin t / 64
      int bin = tid / (THREADS / BINS), strip = tid % (THREADS / BINS);
      unsigned long long c = 0, m = 0;
#pragma unroll
      for (int j = 0; j < BINS; ++j) {
        c += hist_count[bin * THREADS + strip * BINS + j];
        m += hist_mass[bin * THREADS + strip * BINS + j];
      }
      sh.part_count[bin][strip] = c;
      sh.part_mass[bin][strip] = m;
    }
    __syncthreads();
    if (tid < BINS) {  // stage 2: one thread per bin adds the 64 partial sums
      unsigned long long c = 0, m = 0;
      for (int j = 0; j < THREADS / BINS; ++j) { c += sh.part_count[tid][j]; m += sh.part_mass[tid][j]; }
      sh.count[tid] = c;
      sh.mass[tid] = m;
    }
    __syncthreads();
    if (tid == 0) {  // walk the bins from the top of the order
      unsigned long long ac = above_count, am = above_mass;
      for (int bin = BINS - 1; bin >= 0; --bin) {
        unsigned long long c = sh.count[bin], m = sh.mass[bin];
        if (c > 0) {
          bool hit;
          if (kind == FIND_COUNT) hit = ac < target && target <= ac + c;
          else if (kind == FIND_MASS_GE) hit = am < target && target <= am + m;
          else hit = am <= target && target < am + m;
          if (hit) {
            sh.found.ok = 1;
            sh.found.bits = (prefix << 4) | (unsigned)bin;
            sh.found.above_count = ac;
            sh.found.above_mass = am;
            sh.found.tie_count = c;
            sh.found.tie_mass = m;
            break;
          }
        }
        ac += c;
        am += m;
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
    f.bits >>= 1;  // from the key back to the bits of the probability
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

__device__ unsigned long long block_sum_u64(unsigned long long v, Shared& sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* slots = reinterpret_cast<unsigned long long*>(sh.reduce_d);
  __syncthreads();
  if (lane == 0) slots[warp] = v;
  __syncthreads();
  unsigned long long total = 0;
  for (int i = 0; i < THREADS / 32; ++i) total += slots[i];
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
  extern __shared__ __align__(16) unsigned char hist_raw[];  // hist_mass[BINS][THREADS], then hist_count[BINS][THREADS]
  unsigned long long* hist_mass = reinterpret_cast<unsigned long long*>(hist_raw);
  unsigned* hist_count = reinterpret_cast<unsigned*>(hist_mass + BINS * THREADS);
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
  size_t floats = (((size_t)gridDim.x * vocab) + 1) & ~(size_t)1;  // the doubles start 8-byte aligned behind the floats
  double* e = reinterpret_cast<double*>(scratch + floats) + (size_t)row * vocab;
  double partial = 0.0;
  for (int i = tid; i < vocab; i += THREADS) {
    double ex = exp((double)p[i] - (double)best);  // once per logit, kept in double for the division below
    e[i] = ex;
    partial += ex;
  }
  double inverse = 1.0 / block_sum_d(partial, sh);
  unsigned long long all_mass = 0;  // this thread's share of the total mass, in fixed point (exact integer sums)
  for (int i = tid; i < vocab; i += THREADS) {
    float v = (float)(e[i] * inverse);
    p[i] = v;
    all_mass += to_fx(v);
  }
  __syncthreads();

  unsigned long long keep = (unsigned long long)vocab;
  if (top_k > 0 && (unsigned long long)top_k < keep) keep = (unsigned long long)top_k;
  if (top_p < 1.0) {
    find_prefix(p, vocab, FIND_MASS_GE, (unsigned long long)(top_p * FX_ONE), sh, hist_count, hist_mass);
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
  unsigned long long total;
  if (keep >= (unsigned long long)vocab) {  // everything is kept: the total is a plain sum, no search needed
    total = block_sum_u64(all_mass, sh);
  } else {
    find_prefix(p, vocab, FIND_COUNT, keep, sh, hist_count, hist_mass);
    unsigned long long each = sh.found.tie_count ? sh.found.tie_mass / sh.found.tie_count : 0;
    total = sh.found.above_mass + sh.found.rank * each;
  }
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
  find_prefix(p, vocab, FIND_MASS_GT, target, sh, hist_count, hist_mass);
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
    find_prefix(p, vocab, FIND_COUNT, keep, sh, hist_count, hist_mass);
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

// Chooses one token per row of logits[rows, vocab] (row stride given). `scratch` holds 3 * rows * vocab + 2 floats
// (8-byte aligned): the probabilities, then the exponentials as doubles.
// `rng` holds 4 words of state per sequence; row r uses and advances rng[rng_rows[r]].
DLLM_EXPORT int dllm_sample(int* out_tokens, const float* logits, long long row_stride, int rows, int vocab,
                            float* scratch, unsigned long long* rng, const int* rng_rows, float temperature,
                            int top_k, double top_p, double min_p, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (vocab <= 0 || temperature < 0.f || !(top_p > 0.0) || min_p < 0.0 || top_k < 0) return DLLM_BAD_ARGUMENT;
  if (temperature > 0.f && (scratch == nullptr || rng == nullptr || rng_rows == nullptr)) return DLLM_BAD_ARGUMENT;
  size_t smem = temperature > 0.f ? (size_t)BINS * THREADS * (sizeof(unsigned long long) + sizeof(unsigned)) : 0;
  static bool configured = false;
  if (smem && !configured) {
    if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  return dllm_launch_pdl(sample_kernel, dim3(rows), dim3(THREADS), smem, stream, out_tokens, logits, row_stride,
                         vocab, scratch, rng, rng_rows, temperature, top_k, top_p, min_p);
}

// rng[rows[i]] = xoshiro256** state from SplitMix64(seeds[i]).
DLLM_EXPORT int dllm_seed_rng(unsigned long long* rng, const int* rows, const unsigned long long* seeds, int count,
                              cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  seed_kernel<<<(count + 127) / 128, 128, 0, stream>>>(rng, rows, seeds, count);
  return dllm_launch_status();
}
