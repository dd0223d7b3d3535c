// Decode attention over the paged cache for sequences that bring ONE new token each (bfloat16 cache).
//
// Work is split over (key chunk, kv head, sequence): a block reads the keys and values of its chunk once and serves
// every query head of the group from them (grouped-query sharing), keeping a running maximum and sum in float32.
// Chunks start at fixed multiples of the chunk size, so a sequence's split does not depend on its batch mates. Each
// block writes a partial result (unnormalised output, maximum, sum) to scratch; the block that finishes last for a
// (sequence, kv head) combines that pair's chunks in chunk order (a ticket counter decides who is last; no block
// waits). Blocks whose chunk lies beyond the sequence's length (or before its window) return at once, so one launch
// shape serves every length up to the bound it was sized for (CUDA graphs).
//
// Inside a warp, TPR = pow2ceil(head_dim / 8) lanes share one key row (16 bytes each), so 32 / TPR rows are read at
// once as one contiguous piece of a page. Any head_dim that is a multiple of 8 up to 256 works.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int WARPS = 4;
constexpr int MAX_HEADS_PER_KV = 64;
constexpr int MAX_GROUP = 8;  // most query heads served per pass over the keys

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}

// partial layout: o[(seq * heads + head) * chunks + chunk][head_dim], ml[...][2]; `tickets` holds one counter per
// (sequence, kv head), zero between launches: the block that draws the last ticket of its (sequence, kv head)
// combines the chunks, in chunk order, and puts the counter back to zero. Nobody waits for anybody.
template <int TPR, int G>
__global__ void __launch_bounds__(WARPS * 32) decode_attention_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, unsigned* __restrict__ tickets,
    const bf16* __restrict__ q, KvLayout cache, const int* __restrict__ tok_pos, const int* __restrict__ slots,
    int heads, int chunk, int chunks, float scale, int window) {
  constexpr int ROWS = 32 / TPR;   // key rows a warp reads at once
  constexpr int AHEAD = 4;         // row groups whose keys and values are loaded before any is used
  __shared__ float sm_o[WARPS][G][256];
  __shared__ float sm_ml[WARPS][G][2];
  __shared__ int sm_last;
  __shared__ float sm_m[MAX_HEADS_PER_KV], sm_inv[MAX_HEADS_PER_KV];
  int b = blockIdx.z, g = blockIdx.y, c = blockIdx.x;
  int hd = cache.head_dim, ps = cache.page_size;
  int group = heads / cache.kv_heads;
  pdl_launch_dependents();
  int end = tok_pos[b] + 1;  // positions and slots are written only by the step's last kernel
  int first = (window > 0 && end > window) ? end - window : 0;
  int lo = max(c * chunk, first), hi = min((c + 1) * chunk, end);
  if (lo >= hi) return;
  pdl_wait();  // the queries and this step's keys and values come from the projection kernel before this one
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int sub = lane % TPR, rgroup = lane / TPR;
  bool lane_on = sub * 8 < hd;
  const int* pages = cache.page_table + (size_t)slots[b] * cache.max_pages;
  const bf16* base = (const bf16*)cache.base;
  int per_warp = chunk / WARPS;
  int wlo = max(c * chunk + warp * per_warp, lo), whi = min(c * chunk + (warp + 1) * per_warp, hi);

  for (int h0 = 0; h0 < group; h0 += G) {
    int nh = min(G, group - h0);
    float qf[G][8], acc[G][8], m_run[G], l_run[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      m_run[h] = -INFINITY;
      l_run[h] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { acc[h][i] = 0.f; qf[h][i] = 0.f; }
      if (h < nh && lane_on) {
        uint4 raw = *(const uint4*)(q + ((size_t)b * heads + g * group + h0 + h) * hd + sub * 8);
        unpack8(raw, qf[h]);
      }
    }
    for (int j0 = wlo; j0 < whi; j0 += ROWS * AHEAD) {
      uint4 kraw[AHEAD], vraw[AHEAD];
      bool valid[AHEAD];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        int j = j0 + u * ROWS + rgroup;
        valid[u] = j < whi;
        kraw[u] = make_uint4(0u, 0u, 0u, 0u);
        vraw[u] = kraw[u];
        if (valid[u] && lane_on) {
          int page = pages[j / ps];
          kraw[u] = *(const uint4*)(base + kv_offset(cache, page, 0, g, j % ps) + sub * 8);
          vraw[u] = *(const uint4*)(base + kv_offset(cache, page, 1, g, j % ps) + sub * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        if (j0 + u * ROWS >= whi) break;
        float kf[8], vf[8];
        unpack8(kraw[u], kf);
        unpack8(vraw[u], vf);
#pragma unroll
        for (int h = 0; h < G; ++h) {
          if (h >= nh) break;
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) s = fmaf(qf[h][i], kf[i], s);
#pragma unroll
          for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          s = valid[u] ? s * scale : -INFINITY;
          float tile_max = s;
#pragma unroll
          for (int o = 16; o >= TPR; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
          float m_new = fmaxf(m_run[h], tile_max);
          float p = valid[u] ? __expf(s - m_new) : 0.f;
          float corr = __expf(m_run[h] - m_new);
          float psum = p;
#pragma unroll
          for (int o = 16; o >= TPR; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
          l_run[h] = l_run[h] * corr + psum;
          m_run[h] = m_new;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(p, vf[i], acc[h][i] * corr);
        }
      }
    }
    // add up the row groups of the warp (each holds different keys, the same dimensions)
#pragma unroll
    for (int h = 0; h < G; ++h) {
      if (h >= nh) break;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = acc[h][i];
#pragma unroll
        for (int o = 16; o >= TPR; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[h][i] = v;
      }
      if (rgroup == 0 && lane_on) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_o[warp][h][sub * 8 + i] = acc[h][i];
      }
      if (lane == 0) { sm_ml[warp][h][0] = m_run[h]; sm_ml[warp][h][1] = l_run[h]; }
    }
    __syncthreads();
    // combine the warps in warp order and write the chunk's partial result
    for (int idx = threadIdx.x; idx < nh * hd; idx += WARPS * 32) {
      int h = idx / hd, d = idx % hd;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[w][h][0]);
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        float f = sm_ml[w][h][0] == -INFINITY ? 0.f : __expf(sm_ml[w][h][0] - m);
        o = fmaf(sm_o[w][h][d], f, o);
        l = fmaf(sm_ml[w][h][1], f, l);
      }
      size_t row = ((size_t)b * heads + g * group + h0 + h) * chunks + c;
      part_o[row * hd + d] = o;
      if (d == 0) { part_ml[row * 2] = m; part_ml[row * 2 + 1] = l; }
    }
    __syncthreads();
  }

  // the last block of this (sequence, kv head) to get here combines the chunks
  int c_lo = first / chunk, c_hi = (end + chunk - 1) / chunk;
  __threadfence();   // every thread's partial results are visible device-wide ...
  __syncthreads();   // ... before thread 0 draws the block's ticket
  if (threadIdx.x == 0) {
    unsigned ticket = atomicAdd(&tickets[b * cache.kv_heads + g], 1u);
    sm_last = ticket == (unsigned)(c_hi - c_lo - 1);
    if (sm_last) tickets[b * cache.kv_heads + g] = 0u;
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  // maximum and sum of every query head of the group (a warp per head, lanes over chunks)
  for (int h = warp; h < group; h += WARPS) {
    size_t row0 = ((size_t)b * heads + g * group + h) * chunks;
    float m = -INFINITY;
    for (int cc = c_lo + lane; cc < c_hi; cc += 32) m = fmaxf(m, __ldcg(&part_ml[(row0 + cc) * 2]));
    m = warp_max(m);
    float l = 0.f;  // lane i takes chunks i, i + 32, ...; the lanes are then summed in a fixed tree
    for (int cc = c_lo + lane; cc < c_hi; cc += 32)
      l = fmaf(__ldcg(&part_ml[(row0 + cc) * 2 + 1]), __expf(__ldcg(&part_ml[(row0 + cc) * 2]) - m), l);
    l = warp_sum(l);
    if (lane == 0) { sm_m[h] = m; sm_inv[h] = 1.0f / l; }
  }
  __syncthreads();
  // every (head, dimension) of the group: the chunks in chunk order, loads four ahead
  for (int idx = threadIdx.x; idx < group * hd; idx += WARPS * 32) {
    int h = idx / hd, d = idx % hd;
    size_t row0 = ((size_t)b * heads + g * group + h) * chunks;
    float m = sm_m[h], o = 0.f;
#pragma unroll 4
    for (int cc = c_lo; cc < c_hi; ++cc)
      o = fmaf(__ldcg(&part_o[(row0 + cc) * hd + d]), __expf(__ldcg(&part_ml[(row0 + cc) * 2]) - m), o);
    out[((size_t)b * heads + g * group + h) * hd + d] = __float2bfloat16_rn(o * sm_inv[h]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same split on the tensor cores, for head sizes that are a multiple of 16 up to 128 and chunks of 256 keys:
// each of the block's four warps takes one page of 64 keys, copies its keys and values to shared memory (cp.async)
// and computes scores and output with mma.sync m16n8k16, the 16 rows being the query heads of the kv group (padded
// with zeros). One tile needs no running maximum. The warps are combined in shared memory, then the chunk's partial
// result goes the same way as above (or straight to the output when the sequence has a single chunk).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

constexpr int MMA_CHUNK = 256, TILE_KEYS = 64;

template <int HD>
__global__ void __launch_bounds__(WARPS * 32) decode_attention_mma_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, unsigned* __restrict__ tickets,
    const bf16* __restrict__ q, KvLayout cache, const int* __restrict__ tok_pos, const int* __restrict__ slots,
    int heads, int chunks, float scale_log2, int window) {
  constexpr int LD = HD + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* kv_s = reinterpret_cast<bf16*>(smem_raw);  // per warp: K [64][LD], V [64][LD]
  __shared__ float sm_ml[WARPS][16][2];
  __shared__ int sm_last;
  __shared__ float sm_m[MAX_HEADS_PER_KV], sm_inv[MAX_HEADS_PER_KV];
  int b = blockIdx.z, g = blockIdx.y, c = blockIdx.x;
  int hd = cache.head_dim;
  int group = heads / cache.kv_heads;
  pdl_launch_dependents();
  int end = tok_pos[b] + 1;  // positions and slots are written only by the step's last kernel
  int first = (window > 0 && end > window) ? end - window : 0;
  int lo = max(c * MMA_CHUNK, first), hi = min((c + 1) * MMA_CHUNK, end);
  if (lo >= hi) return;
  int c_lo = first / MMA_CHUNK, c_hi = (end + MMA_CHUNK - 1) / MMA_CHUNK;
  bool single = c_hi - c_lo == 1;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int gq = lane >> 2, tq = lane & 3;
  const int* pages = cache.page_table + (size_t)slots[b] * cache.max_pages;
  int key0 = c * MMA_CHUNK + warp * TILE_KEYS;     // this warp's page of keys
  bool warp_on = key0 < hi && key0 + TILE_KEYS > lo;
  int page = warp_on ? pages[key0 / TILE_KEYS] : 0;
  bf16* k_s = kv_s + (size_t)warp * 2 * TILE_KEYS * LD;
  bf16* v_s = k_s + TILE_KEYS * LD;
  int chunks16 = hd >> 3;
  // Keys and values of earlier steps do not change any more: copy the page before waiting for the kernel that
  // writes this step's row, then (below) read that one row again.
  if (warp_on) {
    const bf16* ksrc = (const bf16*)cache.base + kv_offset(cache, page, 0, g, 0);
    const bf16* vsrc = (const bf16*)cache.base + kv_offset(cache, page, 1, g, 0);
    if (hd == HD) {  // the page is one flat piece: 16-byte piece i goes to row i / (HD/8), column i % (HD/8)
#pragma unroll
      for (int i = 0; i < TILE_KEYS * (HD / 8) / 32; ++i) {
        int idx = lane + 32 * i;
        int dst = (idx / (HD / 8)) * LD + (idx % (HD / 8)) * 8;
        cp_async_16(k_s + dst, ksrc + idx * 8);
        cp_async_16(v_s + dst, vsrc + idx * 8);
      }
    } else {
      for (int idx = lane; idx < TILE_KEYS * (HD / 8); idx += 32) {
        int r = idx / (HD / 8), cc = idx % (HD / 8);
        if (cc < chunks16) {
          cp_async_16(k_s + r * LD + cc * 8, ksrc + (size_t)r * hd + cc * 8);
          cp_async_16(v_s + r * LD + cc * 8, vsrc + (size_t)r * hd + cc * 8);
        } else {
          *reinterpret_cast<uint4*>(k_s + r * LD + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(v_s + r * LD + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  pdl_wait();  // the queries and this step's key and value come from the projection kernel before this one
  int newest = end - 1;
  if (warp_on && newest >= key0 && newest < key0 + TILE_KEYS) {
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncwarp();
    int r = newest - key0;
    const bf16* ksrc = (const bf16*)cache.base + kv_offset(cache, page, 0, g, r);
    const bf16* vsrc = (const bf16*)cache.base + kv_offset(cache, page, 1, g, r);
    for (int cc = lane; cc < chunks16; cc += 32) {
      *reinterpret_cast<uint4*>(k_s + r * LD + cc * 8) = __ldcg(reinterpret_cast<const uint4*>(ksrc + cc * 8));
      *reinterpret_cast<uint4*>(v_s + r * LD + cc * 8) = __ldcg(reinterpret_cast<const uint4*>(vsrc + cc * 8));
    }
    __syncwarp();
  }
  float* red_o = reinterpret_cast<float*>(smem_raw);  // after the products: [WARPS][16][HD] partial outputs

  for (int h0 = 0; h0 < group; h0 += 16) {
    int nh = min(16, group - h0);
    float o_acc[HD / 8][4];
    float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
    if (warp_on) {
      // query fragments straight from global memory: row r of the tile is query head h0 + r of this kv group
      unsigned q_frag[HD / 16][4];
      const bf16* q_lo = q + ((size_t)b * heads + g * group + h0 + gq) * hd;
      const bf16* q_hi = q_lo + (size_t)8 * hd;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        int col = ks * 16 + tq * 2;
        bool in = col < hd;
        q_frag[ks][0] = (gq < nh && in) ? *reinterpret_cast<const unsigned*>(q_lo + col) : 0u;
        q_frag[ks][1] = (gq + 8 < nh && in) ? *reinterpret_cast<const unsigned*>(q_hi + col) : 0u;
        q_frag[ks][2] = (gq < nh && col + 8 < hd) ? *reinterpret_cast<const unsigned*>(q_lo + col + 8) : 0u;
        q_frag[ks][3] = (gq + 8 < nh && col + 8 < hd) ? *reinterpret_cast<const unsigned*>(q_hi + col + 8) : 0u;
      }
      if (h0 == 0) {
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncwarp();
      }
      float s[TILE_KEYS / 8][4];
#pragma unroll
      for (int j = 0; j < TILE_KEYS / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int jp = 0; jp < TILE_KEYS / 16; ++jp) {
          unsigned bfr[4];
          int mat = lane >> 3;
          ldmatrix_x4(bfr, k_s + (jp * 16 + (mat >> 1) * 8 + (lane & 7)) * LD + ks * 16 + (mat & 1) * 8);
          mma_bf16(s[2 * jp], q_frag[ks], bfr[0], bfr[1]);
          mma_bf16(s[2 * jp + 1], q_frag[ks], bfr[2], bfr[3]);
        }
      }
      // masks (keys outside [lo, hi), only in a tile that holds an edge), maximum, probabilities, sum; the
      // scale (with log2 e folded in) is applied inside the exponent: p = 2^(s * scale - max * scale)
      if (key0 < lo || key0 + TILE_KEYS > hi) {
#pragma unroll
        for (int j = 0; j < TILE_KEYS / 8; ++j)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            int key = key0 + j * 8 + tq * 2 + (r & 1);
            if (key < lo || key >= hi) s[j][r] = -INFINITY;
          }
      }
#pragma unroll
      for (int j = 0; j < TILE_KEYS / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) m_row[r >> 1] = fmaxf(m_row[r >> 1], s[j][r]);
      float neg_max[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        m_row[i] = fmaxf(m_row[i], __shfl_xor_sync(0xffffffffu, m_row[i], 1));
        m_row[i] = fmaxf(m_row[i], __shfl_xor_sync(0xffffffffu, m_row[i], 2));
        m_row[i] *= scale_log2;  // from here on the maximum is in the scaled log2 domain, like the partial results
        neg_max[i] = -m_row[i];
      }
      unsigned p_frag[TILE_KEYS / 16][4];
#pragma unroll
      for (int j = 0; j < TILE_KEYS / 8; ++j) {
        float p0 = fast_exp2(fmaf(s[j][0], scale_log2, neg_max[0])), p1 = fast_exp2(fmaf(s[j][1], scale_log2, neg_max[0]));
        float p2 = fast_exp2(fmaf(s[j][2], scale_log2, neg_max[1])), p3 = fast_exp2(fmaf(s[j][3], scale_log2, neg_max[1]));
        l_row[0] += p0 + p1;
        l_row[1] += p2 + p3;
        p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
        p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        l_row[i] += __shfl_xor_sync(0xffffffffu, l_row[i], 1);
        l_row[i] += __shfl_xor_sync(0xffffffffu, l_row[i], 2);
      }
#pragma unroll
      for (int kk = 0; kk < TILE_KEYS / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < HD / 16; ++np) {
          unsigned bfr[4];
          int mat = lane >> 3;
          ldmatrix_x4_trans(bfr, v_s + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * LD + np * 16 + (mat >> 1) * 8);
          mma_bf16(o_acc[2 * np], p_frag[kk], bfr[0], bfr[1]);
          mma_bf16(o_acc[2 * np + 1], p_frag[kk], bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();  // every warp is done with its keys and values: the space becomes the exchange buffer
    if (tq == 0) {
      sm_ml[warp][gq][0] = m_row[0]; sm_ml[warp][gq][1] = l_row[0];
      sm_ml[warp][gq + 8][0] = m_row[1]; sm_ml[warp][gq + 8][1] = l_row[1];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int d = i * 8 + tq * 2;
      float* lo_row = red_o + ((size_t)warp * 16 + gq) * HD + d;
      float* hi_row = red_o + ((size_t)warp * 16 + gq + 8) * HD + d;
      *reinterpret_cast<float2*>(lo_row) = make_float2(o_acc[i][0], o_acc[i][1]);
      *reinterpret_cast<float2*>(hi_row) = make_float2(o_acc[i][2], o_acc[i][3]);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * hd; idx += WARPS * 32) {
      int h = idx / hd, d = idx % hd;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[w][h][0]);
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        float f = sm_ml[w][h][0] == -INFINITY ? 0.f : fast_exp2(sm_ml[w][h][0] - m);
        o = fmaf(red_o[((size_t)w * 16 + h) * HD + d], f, o);
        l = fmaf(sm_ml[w][h][1], f, l);
      }
      size_t head = (size_t)b * heads + g * group + h0 + h;
      if (single) {
        out[head * hd + d] = __float2bfloat16_rn(o / l);
      } else {
        size_t row = head * chunks + c;
        part_o[row * hd + d] = o;
        if (d == 0) { part_ml[row * 2] = m; part_ml[row * 2 + 1] = l; }
      }
    }
    __syncthreads();
    if (h0 + 16 < group && warp_on) {  // the next 16 heads need the keys and values again
      const bf16* ksrc = (const bf16*)cache.base + kv_offset(cache, page, 0, g, 0);
      const bf16* vsrc = (const bf16*)cache.base + kv_offset(cache, page, 1, g, 0);
      for (int idx = lane; idx < TILE_KEYS * (HD / 8); idx += 32) {
        int r = idx / (HD / 8), cc = idx % (HD / 8);
        uint4 kz = make_uint4(0u, 0u, 0u, 0u), vz = kz;
        if (cc < chunks16) {
          kz = *reinterpret_cast<const uint4*>(ksrc + (size_t)r * hd + cc * 8);
          vz = *reinterpret_cast<const uint4*>(vsrc + (size_t)r * hd + cc * 8);
        }
        *reinterpret_cast<uint4*>(k_s + r * LD + cc * 8) = kz;
        *reinterpret_cast<uint4*>(v_s + r * LD + cc * 8) = vz;
      }
      __syncwarp();
    }
  }
  if (single) return;
  // the last block of this (sequence, kv head) combines the chunks (maxima here are in the log2 domain)
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned ticket = atomicAdd(&tickets[b * cache.kv_heads + g], 1u);
    sm_last = ticket == (unsigned)(c_hi - c_lo - 1);
    if (sm_last) {
      tickets[b * cache.kv_heads + g] = 0u;
      __threadfence();
    }
  }
  __syncthreads();
  if (!sm_last) return;
  for (int h = warp; h < group; h += WARPS) {
    size_t row0 = ((size_t)b * heads + g * group + h) * chunks;
    float m = -INFINITY;
    for (int cc = c_lo + lane; cc < c_hi; cc += 32) m = fmaxf(m, __ldcg(&part_ml[(row0 + cc) * 2]));
    m = warp_max(m);
    float l = 0.f;
    for (int cc = c_lo + lane; cc < c_hi; cc += 32)
      l = fmaf(__ldcg(&part_ml[(row0 + cc) * 2 + 1]), fast_exp2(__ldcg(&part_ml[(row0 + cc) * 2]) - m), l);
    l = warp_sum(l);
    if (lane == 0) { sm_m[h] = m; sm_inv[h] = 1.0f / l; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * hd; idx += WARPS * 32) {
    int h = idx / hd, d = idx % hd;
    size_t row0 = ((size_t)b * heads + g * group + h) * chunks;
    float m = sm_m[h], o = 0.f;
#pragma unroll 4
    for (int cc = c_lo; cc < c_hi; ++cc)
      o = fmaf(__ldcg(&part_o[(row0 + cc) * hd + d]), fast_exp2(__ldcg(&part_ml[(row0 + cc) * 2]) - m), o);
    out[((size_t)b * heads + g * group + h) * hd + d] = __float2bfloat16_rn(o * sm_inv[h]);
  }
}

template <int HD>
int launch_mma(void* out, float* part_o, float* part_ml, unsigned* tickets, const void* q, const KvLayout& cache,
               const int* tok_pos, const int* slots, int heads, int chunks, int sequences, float scale, int window,
               cudaStream_t stream) {
  size_t kv_bytes = (size_t)WARPS * 2 * TILE_KEYS * (HD + 8) * sizeof(bf16);
  size_t red_bytes = (size_t)WARPS * 16 * HD * sizeof(float);
  size_t smem = kv_bytes > red_bytes ? kv_bytes : red_bytes;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(decode_attention_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  return dllm_launch_pdl(decode_attention_mma_kernel<HD>, dim3(chunks, cache.kv_heads, sequences), dim3(WARPS * 32),
                         smem, stream, (bf16*)out, part_o, part_ml, tickets, (const bf16*)q, cache, tok_pos, slots,
                         heads, chunks, scale * 1.4426950408889634f, window);
}

int pow2ceil(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}
}  // namespace

// Scratch for the partial results, in floats: sequences * heads * chunks * (head_dim + 2).
DLLM_EXPORT long long dllm_attention_decode_scratch(int sequences, int heads, int head_dim, int chunks) {
  return (long long)sequences * heads * chunks * (head_dim + 2);
}

// out, q: [sequences, heads * head_dim] bfloat16; sequence b's query is the token at tok_pos[b], whose key and value
// are already in the cache. `tickets`: sequences * kv_heads counters, zero before the first launch (the kernel
// leaves them zero). `chunk` keys per block (a multiple of 16, at most 1024); `max_context` bounds the
// lengths this launch must serve (the grid covers max_context / chunk chunks).
DLLM_EXPORT int dllm_attention_decode(void* out, const void* q, void* cache_base, const int* page_table,
                                      int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                      const int* tok_pos, const int* slots, int sequences, float scale, int window,
                                      int chunk, int max_context, float* scratch, unsigned* tickets,
                                      cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return DLLM_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > 256 || (head_dim & 7) || heads / kv_heads > MAX_HEADS_PER_KV)
    return DLLM_UNSUPPORTED_SIZE;
  if (chunk < 16 || chunk > 1024 || chunk % 16 || max_context <= 0 || scratch == nullptr || tickets == nullptr)
    return DLLM_BAD_ARGUMENT;
  int chunks = (max_context + chunk - 1) / chunk;
  if (sequences > 65535 || kv_heads > 65535) return DLLM_UNSUPPORTED_SIZE;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)sequences * heads * chunks * head_dim;
  if (chunk == MMA_CHUNK && head_dim % 16 == 0 && head_dim <= 128 && page_size == TILE_KEYS) {
    unsigned* t = tickets;
    if (head_dim <= 32)
      return launch_mma<32>(out, part_o, part_ml, t, q, cache, tok_pos, slots, heads, chunks, sequences, scale, window, stream);
    if (head_dim <= 64)
      return launch_mma<64>(out, part_o, part_ml, t, q, cache, tok_pos, slots, heads, chunks, sequences, scale, window, stream);
    return launch_mma<128>(out, part_o, part_ml, t, q, cache, tok_pos, slots, heads, chunks, sequences, scale, window, stream);
  }
  dim3 grid(chunks, kv_heads, sequences);
  int tpr = pow2ceil(head_dim / 8);
  int status = DLLM_OK;
  int group = heads / kv_heads;
#define DLLM_LAUNCH_G(T, G)                                                                                     \
  status = dllm_launch_pdl(decode_attention_kernel<T, G>, grid, dim3(WARPS * 32), 0, stream, (bf16*)out, part_o, \
                           part_ml, tickets, (const bf16*)q, cache, tok_pos, slots, heads, chunk, chunks, scale, \
                           window)
#define DLLM_LAUNCH(T)                        \
  if (group <= 1) DLLM_LAUNCH_G(T, 1);        \
  else if (group <= 2) DLLM_LAUNCH_G(T, 2);   \
  else if (group <= 4) DLLM_LAUNCH_G(T, 4);   \
  else DLLM_LAUNCH_G(T, MAX_GROUP)
  switch (tpr) {
    case 1: DLLM_LAUNCH(1); break;
    case 2: DLLM_LAUNCH(2); break;
    case 4: DLLM_LAUNCH(4); break;
    case 8: DLLM_LAUNCH(8); break;
    case 16: DLLM_LAUNCH(16); break;
    case 32: DLLM_LAUNCH(32); break;
    default: return DLLM_UNSUPPORTED_SIZE;
  }
#undef DLLM_LAUNCH
#undef DLLM_LAUNCH_G
  return status;
}
