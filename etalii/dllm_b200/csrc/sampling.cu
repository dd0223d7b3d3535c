// Token choice on the device. A row of logits is the work of a thread-block cluster of 1, 2, 4 or 8 blocks (the fewer
// rows, the more blocks a row gets): the blocks take interleaved stripes of the vocabulary, and every sum or maximum
// over the row goes through distributed shared memory (each block publishes its part, one cluster barrier, every
// block adds the parts in rank order: all blocks hold the same totals and take the same decisions).
//   temperature 0: the first index of the largest logit.
//   temperature > 0: z = float(logit / float(T)); p = float(exp(z - max) / sum) with the exponentials and the sum in
//   double; candidates in the total order (p descending, id ascending); top-k keeps the first k, top-p the shortest
//   prefix whose mass reaches it, min-p drops candidates below min_p * p_max; one double in [0,1) from the row's own
//   xoshiro256** state, scaled by the kept mass, picks the first candidate whose running sum exceeds it.
// The order is never materialised: a prefix of it is found by descending the bits of p four at a time with counting
// histograms (private to each thread, then summed in a fixed order); masses are summed as 64-bit fixed point (2^-62
// units), so every sum is exact integer arithmetic and a row's choice is reproducible. Once at most 32 candidates
// are left under the bits found so far, one warp orders them and the descent ends there. Where a thread's stripe of
// the vocabulary is at most eight logits (up to 65,536 tokens with eight blocks a row), they stay in registers from
// the division by the temperature to the end of the search.
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
constexpr int FEW = 32;   // a search ends by ordering its candidates once this many are left


struct Shared {
  unsigned long long out_u64[2][2 * BINS];  // what this block publishes to its cluster: two sets, used in turn
  double out_d[2];
  float out_f[2];
  int out_i[2];
  unsigned out_u32[2];
  unsigned long long count[BINS];
  unsigned long long mass[BINS];
  unsigned long long part_count[BINS][2];
  unsigned long long part_mass[BINS][2];
  Found found;
  double reduce_d[32];
  float reduce_f[32];
  int reduce_i[32];
  unsigned warp_ties[THREADS / 32];
  unsigned few_n, few_key[FEW], few_sorted[FEW];  // the last candidates of a search (see find_prefix)
};

// ---- the cluster: barrier and reads of the same variable in another block's shared memory
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned remote_addr(const void* local, unsigned rank) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ unsigned long long remote_u64(const unsigned long long* local, unsigned rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote_addr(local, rank)) : "memory");
  return v;
}
__device__ __forceinline__ unsigned remote_u32(const void* local, unsigned rank) {
  unsigned v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote_addr(local, rank)) : "memory");
  return v;
}
// Which of the two sets of published values the next exchange uses. A block may publish into a set again only
// after every block has read it: between two uses of the same set lies the barrier of the exchange in between.
struct Turn {
  int set = 0;
  __device__ __forceinline__ int next() { int s = set; set ^= 1; return s; }
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
// on a handful of shared counters), then the bins are summed over the threads (a fixed tree) and over the blocks of
// the cluster in rank order. Every block walks the same totals and finds the same boundary.
template <int CL>
__device__ __forceinline__ void find_prefix(const float* __restrict__ p, int vocab, int kind, unsigned long long target, Shared& sh,
                            unsigned* __restrict__ hist_count, unsigned long long* __restrict__ hist_mass,
                            unsigned rank, Turn& turn, const float (&kept)[8], bool fits) {
  unsigned prefix = 0;
  unsigned long long above_count = 0, above_mass = 0;
  int tid = threadIdx.x;
  // The thread's bins start at zero and whoever sums them below leaves them at zero again. Where the thread's
  // stripe of the vocabulary is at most eight elements (`fits`), the caller holds them in registers (`kept`, -1 for
  // none) and no pass reads them again.
#pragma unroll
  for (int bin = 0; bin < BINS; ++bin) {
    hist_count[bin * THREADS + tid] = 0u;
    hist_mass[bin * THREADS + tid] = 0ull;
  }
  for (int shift = 28; shift >= 0; shift -= 4) {
    if (tid == 0) sh.found.ok = 0;
    for (int i0 = (int)rank * THREADS + tid; i0 < vocab; i0 += 8 * CL * THREADS) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)  // loads first
        v[u] = fits ? kept[u] : (i0 + u * CL * THREADS < vocab ? p[i0 + u * CL * THREADS] : -1.f);
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
    {  // stage 1: warps 2b and 2b + 1 add bin b over the two halves of the block's threads (lanes stride through
       // the threads, then the warp adds up by shuffles: a fixed tree)
      int warp = tid >> 5, lane = tid & 31;
      int bin = warp >> 1, half = warp & 1;
      unsigned long long c = 0, m = 0;
#pragma unroll
      for (int j = 0; j < THREADS / 64; ++j) {
        int at = bin * THREADS + half * (THREADS / 2) + j * 32 + lane;
        c += hist_count[at];
        m += hist_mass[at];
        hist_count[at] = 0u;  // (every entry is read by exactly one thread: it leaves it empty for the next pass)
        hist_mass[at] = 0ull;
      }
      for (int o = 16; o > 0; o >>= 1) {
        c += __shfl_xor_sync(0xffffffffu, c, o);
        m += __shfl_xor_sync(0xffffffffu, m, o);
      }
      if (lane == 0) { sh.part_count[bin][half] = c; sh.part_mass[bin][half] = m; }
    }
    __syncthreads();
    int set = turn.next();
    if (tid < BINS) {  // stage 2: the block's bins, published to the cluster
      sh.out_u64[set][tid] = sh.part_count[tid][0] + sh.part_count[tid][1];
      sh.out_u64[set][BINS + tid] = sh.part_mass[tid][0] + sh.part_mass[tid][1];
    }
    cluster_sync();
    if (tid < 32) {
      // stage 3 (the first warp): lane b < 16 adds bin b over the cluster, blocks in rank order; then the lanes
      // walk the bins from the top of the order together: lane b needs what lies in the bins above it
      unsigned long long c = 0, m = 0;
      if (tid < BINS) {
#pragma unroll
        for (unsigned r = 0; r < CL; ++r) {
          c += remote_u64(&sh.out_u64[set][tid], r);
          m += remote_u64(&sh.out_u64[set][BINS + tid], r);
        }
      }
      unsigned long long ac = c, am = m;  // inclusive sums over the lanes above and this one
#pragma unroll
      for (int o = 1; o < BINS; o <<= 1) {
        unsigned long long oc = __shfl_down_sync(0xffffffffu, ac, o), om = __shfl_down_sync(0xffffffffu, am, o);
        if (tid + o < BINS) { ac += oc; am += om; }
      }
      ac = above_count + ac - c;  // what lies above this bin
      am = above_mass + am - m;
      bool hit = false;
      if (tid < BINS && c > 0) {
        if (kind == FIND_COUNT) hit = ac < target && target <= ac + c;
        else if (kind == FIND_MASS_GE) hit = am < target && target <= am + m;
        else hit = am <= target && target < am + m;
      }
      // (the ranges of the bins do not overlap: at most one lane hits; with several empty-mass bins tied on a
      // boundary the highest bin is the reference's choice)
      unsigned hits = __ballot_sync(0xffffffffu, hit);
      if (hit && tid == 31 - __clz((int)hits)) {
        sh.found.ok = 1;
        sh.found.bits = (prefix << 4) | (unsigned)tid;
        sh.found.above_count = ac;
        sh.found.above_mass = am;
        sh.found.tie_count = c;
        sh.found.tie_mass = m;
      }
    }
    __syncthreads();
    if (!sh.found.ok) return;  // the whole vocabulary does not reach the target (every block sees the same)
    prefix = sh.found.bits;
    above_count = sh.found.above_count;
    above_mass = sh.found.above_mass;
    bool few = sh.found.tie_count <= (unsigned long long)FEW && shift > 0;
    __syncthreads();
    if (few) {
      // At most 32 candidates are left under this prefix: no need to descend bit by bit. Whoever holds one puts its
      // key on its block's list; every block then reads all lists, orders the keys (descending) in its first warp
      // and walks the groups of equal keys from the top, as the passes above walk bins.
      if (tid == 0) sh.few_n = 0u;
      __syncthreads();
      auto offer = [&](float v) {
        unsigned key = __float_as_uint(v) << 1;
        if (v >= 0.f && (key >> shift) == prefix) sh.few_key[atomicAdd(&sh.few_n, 1u) & (FEW - 1)] = key;
      };
      if (fits) {
#pragma unroll
        for (int u = 0; u < 8; ++u) offer(kept[u]);
      } else {
        for (int i = (int)rank * THREADS + tid; i < vocab; i += CL * THREADS) offer(p[i]);
      }
      cluster_sync();
      if (tid < 32) {
        unsigned key = 0u;
        bool have = false;
        unsigned before = 0;  // the candidates on the lists of lower ranks
#pragma unroll
        for (unsigned r = 0; r < CL; ++r) {
          unsigned n = remote_u32(&sh.few_n, r);
          if (n > (unsigned)FEW) n = FEW;
          if ((unsigned)tid >= before && (unsigned)tid < before + n) {
            key = remote_u32(&sh.few_key[tid - before], r);
            have = true;
          }
          before += n;
        }
        unsigned total = before < 32u ? before : 32u;
        // this candidate's place in the order: the keys above it, and equal keys in lower lanes
        unsigned place = 0;
        for (unsigned j = 0; j < 32u; ++j) {
          unsigned other = __shfl_sync(0xffffffffu, key, (int)j);
          bool other_has = __shfl_sync(0xffffffffu, (int)have, (int)j) != 0;
          if (other_has && (other > key || (other == key && j < (unsigned)tid))) ++place;
        }
        if (have) sh.few_sorted[place] = key;
        __syncwarp();
        if (tid == 0) {
          Found& f = sh.found;
          unsigned long long ac = f.above_count, am = f.above_mass;
          unsigned at = 0;
          bool done = false;
          while (at < total && !done) {
            unsigned k = sh.few_sorted[at];
            unsigned long long c = 1;
            while (at + c < total && sh.few_sorted[at + c] == k) ++c;
            unsigned long long m = c * to_fx(__uint_as_float(k >> 1));
            bool hit;
            if (kind == FIND_COUNT) hit = ac < target && target <= ac + c;
            else if (kind == FIND_MASS_GE) hit = am < target && target <= am + m;
            else hit = am <= target && target < am + m;
            if (hit || at + c >= total) {  // (the bin held the boundary, so a group does; the last one if none says so)
              f.bits = k;
              f.above_count = ac;
              f.above_mass = am;
              f.tie_count = c;
              f.tie_mass = m;
              done = true;
            }
            ac += c;
            am += m;
            at += (unsigned)c;
          }
        }
      }
      __syncthreads();
      break;
    }
  }
  if (tid == 0) {
    Found& f = sh.found;
    f.bits >>= 1;  // from the key back to the bits of the probability
    unsigned long long each = f.tie_count ? f.tie_mass / f.tie_count : 0;
    unsigned long long rank_in_ties;
    if (kind == FIND_COUNT) rank_in_ties = target - f.above_count;
    else if (each == 0) rank_in_ties = 1;
    else if (kind == FIND_MASS_GE) rank_in_ties = (target - f.above_mass + each - 1) / each;
    else rank_in_ties = (target - f.above_mass) / each + 1;
    if (rank_in_ties < 1) rank_in_ties = 1;
    if (rank_in_ties > f.tie_count) rank_in_ties = f.tie_count;
    f.rank = rank_in_ties;
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

// Sums over the cluster: the block's sum first (warps by shuffles, then the warps' sums in warp order), published,
// then the blocks' sums in rank order. Every thread of every block returns the same value.
template <int CL>
__device__ unsigned long long cluster_sum_u64(unsigned long long v, Shared& sh, Turn& turn) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* slots = reinterpret_cast<unsigned long long*>(sh.reduce_d);
  __syncthreads();
  if (lane == 0) slots[warp] = v;
  __syncthreads();
  int set = turn.next();
  if (threadIdx.x == 0) {
    unsigned long long block = 0;
    for (int i = 0; i < THREADS / 32; ++i) block += slots[i];
    sh.out_u64[set][0] = block;
  }
  cluster_sync();
  unsigned long long total = 0;
#pragma unroll
  for (unsigned r = 0; r < CL; ++r) total += remote_u64(&sh.out_u64[set][0], r);
  return total;
}

template <int CL>
__device__ double cluster_sum_d(double v, Shared& sh, Turn& turn) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh.reduce_d[warp] = v;
  __syncthreads();
  int set = turn.next();
  if (threadIdx.x == 0) {
    double block = 0.0;
    for (int i = 0; i < THREADS / 32; ++i) block += sh.reduce_d[i];
    sh.out_d[set] = block;
  }
  cluster_sync();
  double total = 0.0;
#pragma unroll
  for (unsigned r = 0; r < CL; ++r)
    total += __longlong_as_double((long long)remote_u64(reinterpret_cast<unsigned long long*>(&sh.out_d[set]), r));
  return total;
}

// (value, index) maximum over the cluster; ties go to the lower index
template <int CL>
__device__ void cluster_argmax(float& v, int& idx, Shared& sh, Turn& turn) {
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) { sh.reduce_f[warp] = v; sh.reduce_i[warp] = idx; }
  __syncthreads();
  int set = turn.next();
  if (threadIdx.x == 0) {
    float bv = sh.reduce_f[0];
    int bi = sh.reduce_i[0];
    for (int i = 1; i < THREADS / 32; ++i) {
      float ov = sh.reduce_f[i];
      int oi = sh.reduce_i[i];
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    sh.out_f[set] = bv;
    sh.out_i[set] = bi;
  }
  cluster_sync();
  v = __uint_as_float(remote_u32(&sh.out_f[set], 0));
  idx = (int)remote_u32(&sh.out_i[set], 0);
#pragma unroll
  for (unsigned r = 1; r < CL; ++r) {
    float ov = __uint_as_float(remote_u32(&sh.out_f[set], r));
    int oi = (int)remote_u32(&sh.out_i[set], r);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
}

template <int CL>
__global__ void __launch_bounds__(THREADS, 1) sample_kernel(
    int* __restrict__ out_tokens, const float* __restrict__ logits, long long row_stride, int vocab,
    float* __restrict__ scratch, unsigned long long* __restrict__ rng, const int* __restrict__ rng_rows,
    float temperature, int top_k, double top_p, double min_p) {
  __shared__ Shared sh;
  extern __shared__ __align__(16) unsigned char hist_raw[];  // hist_mass[BINS][THREADS], then hist_count[BINS][THREADS]
  unsigned long long* hist_mass = reinterpret_cast<unsigned long long*>(hist_raw);
  unsigned* hist_count = reinterpret_cast<unsigned*>(hist_mass + BINS * THREADS);
  unsigned rank = blockIdx.x;  // cluster dims are (CL, 1, 1) and gridDim.x == CL
  int row = blockIdx.y, rows = gridDim.y, tid = threadIdx.x;
  const int first = (int)rank * THREADS + tid, stride = CL * THREADS;  // this thread's stripe of the vocabulary
  Turn turn;
  pdl_launch_dependents();
  pdl_wait();
  const float* l = logits + (size_t)row * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  if (temperature == 0.f) {
    for (int i = first; i < vocab; i += stride) {
      float v = l[i];
      if (v > best) { best = v; best_i = i; }
    }
    cluster_argmax<CL>(best, best_i, sh, turn);
    if (rank == 0 && tid == 0) out_tokens[row] = best_i == 0x7fffffff ? 0 : best_i;
    cluster_sync();  // nobody leaves while its published values may still be read
    return;
  }
  float* p = scratch + (size_t)row * vocab;
  // A thread's stripe of the vocabulary, where it is at most eight logits, lives in registers from here to the
  // search (the same operations in the same order as the loops that go through global memory otherwise).
  const bool fits = vocab <= 8 * stride;
  float kept[8];
  if (fits) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      int i = first + u * stride;
      kept[u] = -1.f;
      if (i < vocab) {
        float z = __fdiv_rn(l[i], temperature);
        kept[u] = z;
        if (z > best) { best = z; best_i = i; }
      }
    }
  } else {
    for (int i = first; i < vocab; i += stride) {
      float z = __fdiv_rn(l[i], temperature);
      p[i] = z;
      if (z > best) { best = z; best_i = i; }
    }
  }
  cluster_argmax<CL>(best, best_i, sh, turn);
  if (best_i == 0x7fffffff) {
    // no logit of the row is above -inf (all NaN, or every token masked): there is no largest probability to read,
    // so the row gets token 0, as in the greedy path, and nothing below indexes with best_i. Every thread of the
    // cluster holds the same best_i here, so all of them leave together.
    if (rank == 0 && tid == 0) out_tokens[row] = 0;
    cluster_sync();
    return;
  }
  size_t floats = (((size_t)rows * vocab) + 1) & ~(size_t)1;  // the doubles start 8-byte aligned behind the floats
  double* e = reinterpret_cast<double*>(scratch + floats) + (size_t)row * vocab;
  double partial = 0.0;
  unsigned long long all_mass = 0;  // this thread's share of the total mass, in fixed point (exact integer sums)
  if (fits) {
    // (the exponentials wait in the shared memory that the search's histograms take afterwards)
    double* ex = reinterpret_cast<double*>(hist_raw) + tid;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (first + u * stride < vocab) {
        double value = exp((double)kept[u] - (double)best);  // once per logit, kept in double for the division below
        ex[u * THREADS] = value;
        partial += value;
      }
    }
    double inverse = 1.0 / cluster_sum_d<CL>(partial, sh, turn);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      int i = first + u * stride;
      if (i < vocab) {
        float v = (float)(ex[u * THREADS] * inverse);
        p[i] = v;
        kept[u] = v;
        all_mass += to_fx(v);
      } else {
        kept[u] = -1.f;
      }
    }
  } else {
    for (int i = first; i < vocab; i += stride) {
      double ex = exp((double)p[i] - (double)best);
      e[i] = ex;
      partial += ex;
    }
    double inverse = 1.0 / cluster_sum_d<CL>(partial, sh, turn);
    for (int i = first; i < vocab; i += stride) {
      float v = (float)(e[i] * inverse);
      p[i] = v;
      all_mass += to_fx(v);
    }
  }
  __syncthreads();

  unsigned long long keep = (unsigned long long)vocab;
  if (top_k > 0 && (unsigned long long)top_k < keep) keep = (unsigned long long)top_k;
  if (top_p < 1.0) {
    find_prefix<CL>(p, vocab, FIND_MASS_GE, (unsigned long long)(top_p * FX_ONE), sh, hist_count, hist_mass, rank, turn, kept, fits);
    if (sh.found.ok) {
      unsigned long long n = sh.found.above_count + sh.found.rank;
      if (n < keep) keep = n;
    }
    __syncthreads();
  }
  if (min_p > 0.0) {
    cluster_sync();  // the largest probability may have been written by another block of the cluster
    double floor_p = min_p * (double)__ldcg(p + best_i);
    unsigned long long local = 0;
    for (int i = first; i < vocab; i += stride) local += ((double)p[i] >= floor_p) ? 1ull : 0ull;
    unsigned long long n = cluster_sum_u64<CL>(local, sh, turn);
    if (n >= 1 && n < keep) keep = n;
  }
  unsigned long long total;
  if (keep >= (unsigned long long)vocab) {  // everything is kept: the total is a plain sum, no search needed
    total = cluster_sum_u64<CL>(all_mass, sh, turn);
  } else {
    find_prefix<CL>(p, vocab, FIND_COUNT, keep, sh, hist_count, hist_mass, rank, turn, kept, fits);
    unsigned long long each = sh.found.tie_count ? sh.found.tie_mass / sh.found.tie_count : 0;
    total = sh.found.above_mass + sh.found.rank * each;
  }
  __syncthreads();
  // one draw per row: the first block of the cluster advances the row's generator and passes the number on
  // (the others contribute an exact zero to the sum)
  double u = 0.0;
  if (rank == 0 && tid == 0) {
    unsigned long long* state = rng + (size_t)rng_rows[row] * 4;
    unsigned long long s[4] = {state[0], state[1], state[2], state[3]};
    u = next_double(s);
    state[0] = s[0]; state[1] = s[1]; state[2] = s[2]; state[3] = s[3];
  }
  u = cluster_sum_d<CL>(u, sh, turn);
  unsigned long long target = (unsigned long long)(u * (double)total);
  if (total > 0 && target >= total) target = total - 1;
  __syncthreads();
  find_prefix<CL>(p, vocab, FIND_MASS_GT, target, sh, hist_count, hist_mass, rank, turn, kept, fits);
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
    find_prefix<CL>(p, vocab, FIND_COUNT, keep, sh, hist_count, hist_mass, rank, turn, kept, fits);
    want_bits = sh.found.bits;
    want_rank = sh.found.rank;
  }
  // the want_rank-th id, ascending, among the elements whose probability has exactly want_bits: ids in contiguous
  // pieces now, a piece per thread of the cluster (the probabilities of other blocks' stripes are read here)
  cluster_sync();
  int chunk = (vocab + stride - 1) / stride;
  int lo = min(first * chunk, vocab), hi = min(lo + chunk, vocab);
  unsigned mine = 0;
  for (int i = lo; i < hi; ++i) mine += __float_as_uint(__ldcg(p + i)) == want_bits ? 1u : 0u;
  // ties before this thread's piece: in its warp (a scan by shuffles), in the warps before, in the blocks before
  const int warp = tid >> 5, lane = tid & 31;
  unsigned through_me = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned other = __shfl_up_sync(0xffffffffu, through_me, o);
    if (lane >= o) through_me += other;
  }
  if (lane == 31) sh.warp_ties[warp] = through_me;
  __syncthreads();
  unsigned before_warp = 0, block_ties = 0;
  for (int w = 0; w < THREADS / 32; ++w) {
    unsigned ties = sh.warp_ties[w];
    if (w < warp) before_warp += ties;
    block_ties += ties;
  }
  int set = turn.next();
  if (tid == 0) sh.out_u32[set] = block_ties;
  cluster_sync();
  unsigned long long before = 0;  // ties in the blocks of lower rank (their ids are lower)
#pragma unroll
  for (unsigned r = 0; r < CL; ++r)
    if (r < rank) before += remote_u32(&sh.out_u32[set], r);
  before += before_warp + through_me - mine;
  if (before < want_rank && want_rank <= before + mine) {  // true in exactly one thread of the cluster
    unsigned long long seen = before;
    int chosen = best_i;
    for (int i = lo; i < hi; ++i) {
      if (__float_as_uint(__ldcg(p + i)) == want_bits && ++seen == want_rank) { chosen = i; break; }
    }
    out_tokens[row] = chosen;
  }
  cluster_sync();  // nobody leaves while its published values may still be read
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
template <int CL>
int launch(size_t smem, int* out_tokens, const float* logits, long long row_stride, int rows, int vocab, float* scratch,
           unsigned long long* rng, const int* rng_rows, float temperature, int top_k, double top_p, double min_p,
           cudaStream_t stream) {
  static bool configured = false;
  if (smem && !configured) {
    if (cudaFuncSetAttribute(sample_kernel<CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(CL, rows);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = CL;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = dllm_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, sample_kernel<CL>, out_tokens, logits, row_stride, vocab, scratch, rng, rng_rows,
                            temperature, top_k, top_p, min_p) == cudaSuccess
             ? DLLM_OK
             : DLLM_LAUNCH_FAILED;
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
  if (rows > 65535) return DLLM_UNSUPPORTED_SIZE;
  size_t smem = temperature > 0.f ? (size_t)BINS * THREADS * (sizeof(unsigned long long) + sizeof(unsigned)) : 0;
  // blocks per row: as many as keep the whole launch within one wave of the device
  if (rows <= 18) return launch<8>(smem, out_tokens, logits, row_stride, rows, vocab, scratch, rng, rng_rows, temperature, top_k, top_p, min_p, stream);
  if (rows <= 37) return launch<4>(smem, out_tokens, logits, row_stride, rows, vocab, scratch, rng, rng_rows, temperature, top_k, top_p, min_p, stream);
  if (rows <= 74) return launch<2>(smem, out_tokens, logits, row_stride, rows, vocab, scratch, rng, rng_rows, temperature, top_k, top_p, min_p, stream);
  return launch<1>(smem, out_tokens, logits, row_stride, rows, vocab, scratch, rng, rng_rows, temperature, top_k, top_p, min_p, stream);
}

// rng[rows[i]] = xoshiro256** state from SplitMix64(seeds[i]).
DLLM_EXPORT int dllm_seed_rng(unsigned long long* rng, const int* rows, const unsigned long long* seeds, int count,
                              cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  seed_kernel<<<(count + 127) / 128, 128, 0, stream>>>(rng, rows, seeds, count);
  return dllm_launch_status();
}
