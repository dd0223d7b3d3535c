// Prefill attention over the paged cache (bfloat16, head_dim 64 or 128) on the 5th-generation tensor cores. A block
// takes 128 consecutive new tokens of one sequence and one query head and walks the sequence's cache pages (64 keys
// each):
//   softmax warps (0-7): two groups of four warps that take alternate steps (group j % 2 takes step j, with the
//            score, P and output buffers number j % 2), one thread per query: read its row of scores from tensor
//            memory (tcgen05.ld 32x32b), mask, maximum and sum in float32 (no shuffles: the row is the thread's
//            own; the maximum a row subtracts is renewed only when a score exceeds it by 2^8, so most steps read
//            their scores once), write the probabilities as bfloat16 into the swizzled P tile, fetch the group's
//            previous P V and fold it into the float32 output kept in registers: O = O * 2^(m_old - m_new) + P V.
//            At the end the second group hands its maximum, sum and output to the first through shared memory.
//   next warp: one lane issues TMA loads: the query tile once, then a page of keys and a page of values per step
//            into rings of shared-memory stages (128-byte swizzle), signalled by mbarriers;
//   next warp: one lane issues tcgen05.mma for the scores: S_j = Q K_j^T (M = 128 queries, N = 64 keys, K =
//            head_dim) into one of two score buffers in tensor memory, as soon as the buffer is free and the keys
//            are there;
//   last warp: one lane issues tcgen05.mma for the outputs: O_j = P_j V_j (P from shared memory, V read MN-major as
//            it lies in the cache) into one of two output buffers (a lane of its own: issuing a product costs a
//            single thread tens of cycles, and the scores of the next steps must not queue behind a wait for P).
// head_dim 128: operands are two 64-column boxes side by side, the outputs take twice the columns of tensor memory
// and 128 registers of a softmax thread, so there is one softmax group (which then takes every step and alternates
// between the two sets of buffers itself) and the block has seven warps.
// Every wait on an mbarrier is bounded; a role that gives up records a status word and leaves, the block still frees
// its tensor memory and the host raises.
#include "tcgen05.cuh"

namespace {
using namespace tc5;
typedef __nv_bfloat16 bf16;
constexpr int BQ = 128, BKV = 64, STAGES = 4;
constexpr int P_BYTES = BQ * BKV * 2;

template <int HD> struct Shape {
  static constexpr int GROUPS = HD <= 64 ? 2 : 1;             // softmax groups of four warps
  static constexpr int SOFT_WARPS = 4 * GROUPS;
  static constexpr int THREADS = (SOFT_WARPS + 3) * 32;       // + the warps of the three single issuing lanes
  static constexpr int BOXES = HD / 64;                       // 64-column boxes per row of an operand
  static constexpr int Q_BOX = BQ * 128, KV_BOX = BKV * 128;  // bytes of a box: rows of 128 bytes
  static constexpr int Q_BYTES = BOXES * Q_BOX, KV_BYTES = BOXES * KV_BOX;
  // P tiles: with two groups a group would write its next P while its previous product may still read the last
  // one, so each group has two; a single group alternates between the two buffers anyway
  static constexpr int P_TILES = 2 * GROUPS;
  static constexpr size_t SMEM = Q_BYTES + 2 * STAGES * KV_BYTES + P_TILES * P_BYTES + 1024;
  static constexpr unsigned TMEM_COLS = 2 * BKV + 2 * HD <= 256 ? 256 : 512;  // scores 2 x 64, outputs 2 x HD
  static constexpr int EX_LD = HD + 2;  // floats per row of the exchange between the two softmax groups
};

struct Barriers {
  uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  uint64_t s_full[2], s_empty[2], p_full[2], o_full[2], o_empty[2];
};

template <int HD>
__global__ void __launch_bounds__(Shape<HD>::THREADS, 1) prefill_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, bf16* __restrict__ out,
    KvLayout cache, const int* __restrict__ tile_seq, const int* __restrict__ tile_first,
    const int* __restrict__ cu_seqlens, const int* __restrict__ start, const int* __restrict__ slots, int heads,
    float scale_log2, int window, int* __restrict__ status) {
  typedef Shape<HD> S;
  constexpr int GROUPS = S::GROUPS, SOFT_WARPS = S::SOFT_WARPS, Q_BYTES = S::Q_BYTES, KV_BYTES = S::KV_BYTES;
  constexpr unsigned TMEM_COLS = S::TMEM_COLS;
  int tile = blockIdx.x, h = blockIdx.y;
  int q0 = tile_first[tile];
  if (q0 % BQ) return;  // the host lists tiles of 64 tokens; every second one starts a tile of 128
  pdl_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms: 1 KB
  unsigned char* q_s = tiles;
  unsigned char* k_s = q_s + Q_BYTES;
  unsigned char* v_s = k_s + STAGES * KV_BYTES;
  unsigned char* p_s = v_s + STAGES * KV_BYTES;
  __shared__ Barriers bar;
  __shared__ unsigned tmem_base_s;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int b = tile_seq[tile];
  int g = h / (heads / cache.kv_heads);
  int n_new = cu_seqlens[b + 1] - cu_seqlens[b];
  int tok0 = cu_seqlens[b] + q0;           // first token row of this tile in the packed batch
  int rows = min(BQ, n_new - q0);          // queries of this tile that exist
  int pos0 = start[b] + q0;                // absolute position of the tile's first query
  int last_pos = pos0 + rows - 1;
  int kt_end = last_pos / BKV;             // last page any query of the tile sees
  int kt_begin = (window > 0 && pos0 + 1 > window) ? (pos0 + 1 - window) / BKV : 0;
  int steps = kt_end - kt_begin + 1;
  const int* pages = cache.page_table + (size_t)slots[b] * cache.max_pages;

  if (threadIdx.x == 0) {
    mbar_init(&bar.q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar.k_full[s], 1); mbar_init(&bar.k_empty[s], 1);
      mbar_init(&bar.v_full[s], 1); mbar_init(&bar.v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.s_full[i], 1); mbar_init(&bar.s_empty[i], 4);   // the 4 warps of softmax group i
      mbar_init(&bar.p_full[i], 4);
      mbar_init(&bar.o_full[i], 1); mbar_init(&bar.o_empty[i], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == SOFT_WARPS + 1) tmem_alloc(&tmem_base_s, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  unsigned tmem_base = tmem_base_s;
  unsigned tmem_s = tmem_base, tmem_o = tmem_base + 2 * BKV;
  pdl_wait();  // the queries and the newest keys and values come from the kernel before; so does `out`'s last reader

  if (warp == SOFT_WARPS) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
      mbar_expect_tx(&bar.q_full, Q_BYTES);
#pragma unroll
      for (int x = 0; x < S::BOXES; ++x) tma_load_2d(q_s + x * S::Q_BOX, &map_q, &bar.q_full, h * HD + x * 64, tok0);
      for (int j = 0; j < steps; ++j) {
        int s = j % STAGES;
        unsigned parity = ((j / STAGES) - 1) & 1;
        int page = pages[kt_begin + j];
        int row_k = ((page * 2 + 0) * cache.kv_heads + g) * BKV, row_v = ((page * 2 + 1) * cache.kv_heads + g) * BKV;
        if (j >= STAGES && !mbar_wait(&bar.k_empty[s], parity)) { *(volatile int*)status = 12; break; }
        mbar_expect_tx(&bar.k_full[s], KV_BYTES);
#pragma unroll
        for (int x = 0; x < S::BOXES; ++x)
          tma_load_2d(k_s + s * KV_BYTES + x * S::KV_BOX, &map_kv, &bar.k_full[s], x * 64, row_k);
        if (j >= STAGES && !mbar_wait(&bar.v_empty[s], parity)) { *(volatile int*)status = 13; break; }
        mbar_expect_tx(&bar.v_full[s], KV_BYTES);
#pragma unroll
        for (int x = 0; x < S::BOXES; ++x)
          tma_load_2d(v_s + s * KV_BYTES + x * S::KV_BOX, &map_kv, &bar.v_full[s], x * 64, row_v);
      }
    }
  } else if (warp == SOFT_WARPS + 1) {
    if (lane == 0) {
      constexpr unsigned idesc_s = instr_desc(BQ, BKV);
      bool ok = mbar_wait(&bar.q_full, 0);
      if (!ok) *(volatile int*)status = 14;
      unsigned q_addr = smem_u32(q_s);
      for (int i = 0; i < steps && ok; ++i) {  // S_i = Q K_i^T into the score buffer of group i % 2
        int sb = i & 1, s = i % STAGES;
        if (!mbar_wait(&bar.k_full[s], (i / STAGES) & 1)) { *(volatile int*)status = 18; break; }
        if (i >= 2 && !mbar_wait(&bar.s_empty[sb], ((i >> 1) - 1) & 1)) { *(volatile int*)status = 19; break; }
        fence_after_sync();
        unsigned k_addr = smem_u32(k_s + s * KV_BYTES);
#pragma unroll
        for (int x = 0; x < S::BOXES; ++x)  // 64 values of the head per box, 16 per product
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma(tmem_s + (unsigned)(sb * BKV), smem_desc(q_addr + x * S::Q_BOX + k * 32),
                 smem_desc(k_addr + x * S::KV_BOX + k * 32), idesc_s, (x > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(&bar.k_empty[s]);
        tcgen05_commit(&bar.s_full[sb]);
      }
    }
  } else if (warp == SOFT_WARPS + 2) {
    if (lane == 0) {
      constexpr unsigned idesc_o = instr_desc(BQ, 64, true);  // 64 output columns per product: one box of V
      for (int i = 0; i < steps; ++i) {  // O_i = P_i V_i into the output buffer of group i % 2
        int pb = i & 1, s = i % STAGES;
        if (!mbar_wait(&bar.p_full[pb], (i >> 1) & 1)) { *(volatile int*)status = 15; break; }
        if (!mbar_wait(&bar.v_full[s], (i / STAGES) & 1)) { *(volatile int*)status = 16; break; }
        if (i >= 2 && !mbar_wait(&bar.o_empty[pb], ((i >> 1) - 1) & 1)) { *(volatile int*)status = 17; break; }
        fence_after_sync();
        unsigned p_addr = smem_u32(p_s + (i % S::P_TILES) * P_BYTES), v_addr = smem_u32(v_s + s * KV_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
#pragma unroll
          for (int x = 0; x < S::BOXES; ++x)
            umma(tmem_o + (unsigned)(pb * HD + x * 64), smem_desc(p_addr + k * 32),
                 smem_desc(v_addr + x * S::KV_BOX + k * 2048), idesc_o, k > 0 ? 1u : 0u);
        tcgen05_commit(&bar.v_empty[s]);
        tcgen05_commit(&bar.o_full[pb]);
      }
    }
  } else if (warp < SOFT_WARPS) {
    // Step j works in the buffers (scores, P, outputs) number j % 2, for the (j / 2)-th time. With two groups, group
    // wg takes the steps j = wg, wg + 2, ... and so always the same buffers; a single group takes every step.
    int wg = warp >> 2;
    int r = (warp & 3) * 32 + lane;              // this thread's query: row r of the tile, tensor-memory lane r
    int qp = pos0 + r;
    unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    float o[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) o[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, corr_saved = 1.f;
    bool ok = true;
    // fold step i's output into the running one: O = O * corr + P V
    auto consume = [&](int i, float corr) -> bool {
      const int ob = i & 1;
      unsigned o_addr = tmem_o + lane_base + (unsigned)(ob * HD);
      if (!mbar_wait(&bar.o_full[ob], (i >> 1) & 1)) {
        if (lane == 0) *(volatile int*)status = 20;
        return false;
      }
      fence_after_sync();
      unsigned v[2][16];
      tmem_load16_nowait(o_addr, v[0]);
#pragma unroll
      for (int c = 0; c < HD; c += 16) {
        const int cur = (c >> 4) & 1;
        tmem_wait_ld();
        if (c + 16 < HD) tmem_load16_nowait(o_addr + (unsigned)(c + 16), v[cur ^ 1]);
#pragma unroll
        for (int d = 0; d < 16; ++d) o[c + d] = fmaf(o[c + d], corr, __uint_as_float(v[cur][d]));
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.o_empty[ob]);
      return true;
    };
    int taken = 0;  // how many steps this group has taken
    for (int j = wg; j < steps; j += GROUPS, ++taken) {
      const int sb = j & 1;
      unsigned s_addr = tmem_s + lane_base + (unsigned)(sb * BKV);
      unsigned char* p_tile = p_s + (j % S::P_TILES) * P_BYTES;
      if (!mbar_wait(&bar.s_full[sb], (j >> 1) & 1)) {
        if (lane == 0) *(volatile int*)status = 21;
        ok = false;
        break;
      }
      fence_after_sync();
      int key0 = (kt_begin + j) * BKV;
      // a tile with an edge for some row of the block: keys beyond the query, or before its window
      bool edge = key0 + BKV - 1 > pos0 || (window > 0 && key0 < pos0 + BQ - window);
      int key_hi = qp - key0, key_lo = window > 0 ? qp + 1 - window - key0 : -1;  // columns key_lo .. key_hi count
      // (the P tile of this step is free: the product that read it last, P_TILES steps ago, has been consumed)
      // One sweep over the scores gives the probabilities relative to the maximum the row has used so far, and the
      // tile's own maximum on the way. The used maximum need not be the true one: any constant cancels in the
      // quotient, and as long as no score lies more than 8 (in the log2 domain) above it the probabilities stay
      // below 256, which bfloat16 and the float32 sums carry as well as values below 1. Only when a row of the warp
      // exceeds that (mostly in a row's first steps) the warp sweeps again with the new maximum.
      unsigned char* p_row = p_tile + r * 128;  // K-major tile, 128-byte rows, 128-byte swizzle
      auto sweep = [&](float m_use, float& tile_max, float& row_sum) {
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains each: the thread has no one to
        float sum[4] = {0.f, 0.f, 0.f, 0.f};                         // hide behind
        unsigned v[2][16];  // two pieces of 16 columns: one in flight from tensor memory while the other is used
        tmem_load16_nowait(s_addr, v[0]);
#pragma unroll
        for (int c = 0; c < BKV; c += 16) {
          const int cur = (c >> 4) & 1;
          tmem_wait_ld();
          if (c + 16 < BKV) tmem_load16_nowait(s_addr + (unsigned)(c + 16), v[cur ^ 1]);
          float p[16];
          if (edge) {  // (two copies of the loop: the compares cost as much as the rest of an element)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x = (c + i > key_hi || c + i < key_lo) ? -INFINITY : __uint_as_float(v[cur][i]);
              mx[i & 3] = fmaxf(mx[i & 3], x);
              p[i] = fast_exp2(fmaf(x, scale_log2, -m_use));
              sum[i & 3] += p[i];
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x = __uint_as_float(v[cur][i]);
              mx[i & 3] = fmaxf(mx[i & 3], x);
              p[i] = fast_exp2(fmaf(x, scale_log2, -m_use));
              sum[i & 3] += p[i];
            }
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint4 packed;
            __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int i = 0; i < 4; ++i) pk[i] = __floats2bfloat162_rn(p[half * 8 + 2 * i], p[half * 8 + 2 * i + 1]);
            *reinterpret_cast<uint4*>(p_row + ((((c >> 3) + half) ^ (r & 7)) << 4)) = packed;
          }
        }
        tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;  // in the scaled log2 domain
        row_sum = (sum[0] + sum[1]) + (sum[2] + sum[3]);
      };
      float tile_max, row_sum, corr = 1.f;
      sweep(m_run == -INFINITY ? 0.f : m_run, tile_max, row_sum);
      bool over = tile_max > m_run + 8.f;  // (also: the row's first scores, while its maximum is still -inf)
      if (__any_sync(0xffffffffu, over)) {
        // the sweep is a warp's affair (tensor memory is read by whole warps): rows that are not over sweep again
        // with their old maximum and get the same values
        float m_new = over ? fmaxf(m_run, tile_max) : m_run;
        float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen nothing so far
        corr = fast_exp2(m_run - m_use);
        m_run = m_new;
        sweep(m_use, tile_max, row_sum);
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.s_empty[sb]);  // the scores are not needed again: the buffer may be rewritten
      // the group's previous product: it had the time of the sweep to finish
      if (taken >= 1 && !consume(j - GROUPS, corr_saved)) { ok = false; break; }
      corr_saved = corr;
      l_run = l_run * corr + row_sum;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes, read by the tensor cores
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.p_full[sb]);
    }
    if (ok && taken >= 1) ok = consume(wg + (taken - 1) * GROUPS, corr_saved);
    if (GROUPS == 1) {
      if (ok && r < rows) {
        float inv = 1.0f / l_run;
        bf16* dst = out + ((size_t)(tok0 + r) * heads + h) * HD;
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) {
          uint4 w;
          __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            pk[i] = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c * 8) = w;
        }
      }
    } else {
      // every product has been consumed: the shared memory of the key and value stages is free for the exchange
      asm volatile("bar.sync 1, 256;" ::: "memory");
      float* ex = reinterpret_cast<float*>(k_s) + (size_t)r * S::EX_LD;
      if (wg == 1) {
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<float2*>(ex + d) = make_float2(o[d], o[d + 1]);
        ex[HD] = m_run;
        ex[HD + 1] = l_run;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (wg == 0 && ok && r < rows) {
        float m_other = ex[HD], l_other = ex[HD + 1];
        float m = fmaxf(m_run, m_other);
        float m_use = m == -INFINITY ? 0.f : m;
        float mine = fast_exp2(m_run - m_use), theirs = fast_exp2(m_other - m_use);
        float inv = 1.0f / (l_run * mine + l_other * theirs);
        mine *= inv;
        theirs *= inv;
        bf16* dst = out + ((size_t)(tok0 + r) * heads + h) * HD;
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) {
          uint4 w;
          __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            int d = c * 8 + 2 * i;
            float2 other = *reinterpret_cast<const float2*>(ex + d);
            pk[i] = __floats2bfloat162_rn(o[d] * mine + other.x * theirs, o[d + 1] * mine + other.y * theirs);
          }
          *reinterpret_cast<uint4*>(dst + c * 8) = w;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == SOFT_WARPS + 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int HD>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_kv, void* out, const KvLayout& cache, const int* tile_seq,
           const int* tile_first, const int* cu_seqlens, const int* start, const int* slots, int tiles, int heads,
           float scale, int window, int* status, cudaStream_t stream) {
  typedef Shape<HD> S;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)S::SMEM) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  return dllm_launch_pdl(prefill_tcgen05_kernel<HD>, dim3(tiles, heads), dim3(S::THREADS), S::SMEM, stream, map_q,
                         map_kv, (bf16*)out, cache, tile_seq, tile_first, cu_seqlens, start, slots, heads,
                         scale * 1.4426950408889634f, window, status);
}
}  // namespace

// out, q: [tokens, heads * head_dim] bfloat16. tile_seq / tile_first: for each tile of up to 64 new tokens, its
// sequence and the index of its first token among the sequence's new tokens (the kernel pairs them into tiles of
// 128). The keys and values of the new tokens are already in the cache, which holds `cache_pages` pages of 64
// positions. head_dim must be 64 or 128. `status` is a word the device can write; the kernel sets it non-zero if a
// bounded wait ran out.
DLLM_EXPORT int dllm_attention_prefill_tcgen05(void* out, const void* q, int tokens, void* cache_base,
                                               long long cache_pages, const int* page_table, int max_pages,
                                               int page_size, int heads, int kv_heads, int head_dim,
                                               const int* tile_seq, const int* tile_first, const int* cu_seqlens,
                                               const int* start, const int* slots, int tiles, float scale, int window,
                                               int* status, cudaStream_t stream) {
  if (tiles <= 0 || tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || status == nullptr) return DLLM_BAD_ARGUMENT;
  if ((head_dim != 64 && head_dim != 128) || page_size != BKV || heads > 65535 || ((uintptr_t)q & 15) ||
      ((uintptr_t)cache_base & 15) || ((uintptr_t)out & 15) || cache_pages <= 0 ||
      cache_pages * 2 * kv_heads * BKV > 0x7fffffffll)
    return DLLM_UNSUPPORTED_SIZE;
  alignas(64) CUtensorMap map_q, map_kv;
  if (!make_map(&map_q, q, tokens, (long long)heads * head_dim, BQ) ||
      !make_map(&map_kv, cache_base, cache_pages * 2 * kv_heads * BKV, head_dim, BKV))
    return DLLM_LAUNCH_FAILED;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  if (head_dim == 64)
    return launch<64>(map_q, map_kv, out, cache, tile_seq, tile_first, cu_seqlens, start, slots, tiles, heads, scale,
                      window, status, stream);
  return launch<128>(map_q, map_kv, out, cache, tile_seq, tile_first, cu_seqlens, start, slots, tiles, heads, scale,
                     window, status, stream);
}
