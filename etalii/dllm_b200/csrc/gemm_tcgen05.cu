// bfloat16 matrix product on the 5th-generation tensor cores: C = A[M,K] * W[N,K]^T, float32 accumulation in tensor
// memory. Blocks are persistent and compute 128 x BN tiles of C, with two accumulators in tensor memory so that one
// tile's epilogue overlaps the next tile's products:
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of 128x64 tiles of A and BNx64
//            tiles of W into a ring of shared-memory stages, signalled by mbarriers (expect_tx / complete_tx);
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN, K=16) four
//            per stage and commits each stage back to the producer (tcgen05.commit -> mbarrier), then commits the
//            whole accumulator to the epilogue;
//   warps 2.. read the accumulator (tcgen05.ld 32x32b, a lane per row; four warps for tiles up to 64 columns, eight
//            for wider ones: two per 32 rows, with half the columns each) and apply the epilogue: store float32 or
//            bfloat16, add into the float32 residual, or SwiGLU on interleaved gate/up columns.
// A product of few tokens can run the other way round (W as the 128-row operand, the tile is C^T), and then also with
// its reduction cut into stretches: a block's work items are (tile, stretch) pairs and every stretch stores its own
// partial result, which a second kernel sums in order (for a W with fewer tiles than the device has multiprocessors).
// Rows of A beyond M and columns of K beyond the matrix are zero-filled by TMA; rows of W beyond N give columns
// that are never stored. No multicast, no clusters. Every wait on an mbarrier is bounded: after the limit the role
// records a status word and leaves, the block still frees its tensor memory, and the host raises.
#include "gemm_common.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc5;
typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BK = 64, UMMA_K = 16;

// DEEP: a ring of nine or ten stages (about 215 KB) for a block that has its multiprocessor to itself: a product
// with no more tiles than the device has multiprocessors and a short reduction then brings a tile's whole operand
// panels in one round trip instead of three.
template <int BN, bool DEEP = false, int EPI_STAGE = 0> struct Shape {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int ACC_COLS = BN < 32 ? 32 : BN;   // columns of one accumulator
  static constexpr int TMEM_COLS = 2 * ACC_COLS;       // two accumulators: a power of two, at least 32
  // about 96 KB a block where that is enough (two blocks share an SM, 2 x TMEM_COLS <= 512 columns); the 256-wide
  // tile takes four 48 KB stages and all of the tensor memory, so one block owns the SM
  // (a 64-wide tile that stages its epilogue gives one of its four stages for it, so that two blocks still fit)
  static constexpr int STAGES = DEEP ? (220 * 1024) / (A_BYTES + B_BYTES)
                                     : (BN >= 256 ? 4 : (BN >= 128 ? 3 : (EPI_STAGE > 0 ? 3 : 4)));
  // (EPI_STAGE: bytes behind the ring through which an epilogue makes its global stores whole lines)
  static constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + B_BYTES) + 1024 + EPI_STAGE;
  static constexpr int BLOCKS_PER_SM = (DEEP || BN >= 256) ? 1 : 2;
  // Epilogue warps: one per quarter of the tensor memory's lanes, or two that take half the columns each. A row's
  // epilogue is a chain of loads and special functions, so wide tiles gain from twice the warps (2048 x 2048 x 8192
  // with the residual: 128-wide 70 against 114 µs, 256-wide 61 against 64); narrow tiles of short products lose
  // (2048 x 576 x 576, 64-wide: 9.5 against 8.6 µs), their blocks being set up and torn down once per tile.
  static constexpr int EPI_WARPS = BN >= 128 ? 8 : 4;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
};

// A persistent block: it takes tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... of the m_tiles x n_tiles grid
// (neighbouring blocks share a tile of W and read different rows of A). The producer's ring of stages runs on across
// tiles; the accumulator alternates between two halves of the block's tensor memory, so the epilogue of one tile
// overlaps the products of the next.
// The SwiGLU epilogue of the 256-wide tile writes 128 bytes of a row per warp: it goes through 4 KB of shared memory
// per warp behind the ring, so that eight lanes write a row's 128 bytes together (see the residual epilogue below).
// The residual epilogue of the 64-wide tile goes through 32 rows x 36 floats per warp: behind the ring, or in the
// ring itself where the block has a single tile (the deep ring: every stage has been read when the accumulator is
// full).
template <int BN, int EPI, bool DEEP> struct EpilogueStage {
  static constexpr int BYTES = (EPI == EPI_SWIGLU && BN == 256 && !DEEP) ? 8 * 4096
                               : ((EPI == EPI_RESIDUAL && BN == 64 && !DEEP) ? 4 * 32 * 36 * 4
                               : ((EPI == EPI_RESIDUAL && BN == 256 && !DEEP) ? 8 * 32 * 20 * 4 : 0));  // (see below)
};

// Item `item` of a block's list: a tile and, where the reduction is cut (k_split > 1), one stretch of its k tiles.
struct WorkItem { int tile, split, kt_begin, kt_end; };
__device__ __forceinline__ WorkItem work_item(int item, int total, int k_tiles, int k_split) {
  if (k_split == 1) return WorkItem{item, 0, 0, k_tiles};
  int split = item / total;
  return WorkItem{item - split * total, split, split * k_tiles / k_split, (split + 1) * k_tiles / k_split};
}

template <int BN, int EPI, bool DEEP, int HD>
__global__ void __launch_bounds__(Shape<BN, DEEP>::THREADS, Shape<BN, DEEP>::BLOCKS_PER_SM) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_w,
                                                               void* __restrict__ c, int M, int N, int K,
                                                               int* __restrict__ status, RopeArgs rope, int m_tiles,
                                                               int n_tiles, int k_split, NormArgs norm) {
  typedef Shape<BN, DEEP, EpilogueStage<BN, EPI, DEEP>::BYTES> S;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms: 1 KB
  __shared__ uint64_t full_bar[S::STAGES], empty_bar[S::STAGES], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_s;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int k_tiles = (K + BK - 1) / BK;
  int total = m_tiles * n_tiles;
  // k_split > 1 (EPI_T_STORE_F32 only): an item is a tile and one of k_split stretches of the reduction; its sums
  // go to part `split` of C, which then holds k_split partial results [N, M] one behind the other
  int items = total * k_split;
  pdl_launch_dependents();  // the next kernel may set itself up (barriers, tensor memory) while this one runs

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], S::EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, (unsigned)S::TMEM_COLS);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  unsigned tmem_base = tmem_base_s;
  if (warp == 0 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }
  pdl_wait();  // everything above touched nothing an earlier kernel writes; from here on this kernel reads and writes

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // k tiles issued so far, over all of this block's tiles
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        WorkItem w = work_item(item, total, k_tiles, k_split);
        int m0 = (w.tile % m_tiles) * BM, n0 = (w.tile / m_tiles) * BN;
        for (int kt = w.kt_begin; kt < w.kt_end; ++kt, ++it) {
          int s = it % S::STAGES;
          if (it >= S::STAGES && !mbar_wait(&empty_bar[s], ((it / S::STAGES) - 1) & 1)) {
            *(volatile int*)status = 2;
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], S::A_BYTES + S::B_BYTES);
          unsigned char* a_dst = tiles + (size_t)s * (S::A_BYTES + S::B_BYTES);
          tma_load_2d(a_dst, &map_a, &full_bar[s], kt * BK, m0);
          tma_load_2d(a_dst + S::A_BYTES, &map_w, &full_bar[s], kt * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned idesc = instr_desc(BM, BN);
      int it = 0, lt = 0;  // k tiles consumed, tiles started
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++lt) {
        int buf = lt & 1;
        if (lt >= 2 && !mbar_wait(&acc_empty[buf], ((lt >> 1) - 1) & 1)) { *(volatile int*)status = 5; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned acc = tmem_base + (unsigned)(buf * S::ACC_COLS);
        WorkItem w = work_item(item, total, k_tiles, k_split);
        for (int kt = w.kt_begin; kt < w.kt_end; ++kt, ++it) {
          int s = it % S::STAGES;
          if (!mbar_wait(&full_bar[s], (it / S::STAGES) & 1)) { *(volatile int*)status = 3; ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned a_addr = smem_u32(tiles + (size_t)s * (S::A_BYTES + S::B_BYTES));
          unsigned b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t adesc = smem_desc(a_addr + k * UMMA_K * 2), bdesc = smem_desc(b_addr + k * UMMA_K * 2);
            umma(acc, adesc, bdesc, idesc, (kt > w.kt_begin || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(&empty_bar[s]);  // the stage is free once these products have read it
        }
        tcgen05_commit(&acc_full[buf]);   // this accumulator is complete once every product so far has finished
      }
    }
  } else {
    // epilogue warps: warp w may read tensor-memory lanes 32 * (w % 4) .. + 31; where there are eight, warps 2..5
    // take the first half of a tile's columns and warps 6..9 the second
    constexpr int HALVES = S::EPI_WARPS / 4;
    int quarter = warp & 3, half = HALVES == 2 ? (warp - 2) >> 2 : 0;
    constexpr int HALF = BN / HALVES;
    int c0 = half * HALF;
    int lt = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++lt) {
      int buf = lt & 1;
      WorkItem w = work_item(item, total, k_tiles, k_split);
      int t = w.tile;
      int m0 = (t % m_tiles) * BM, n_tile = t / m_tiles, n0 = n_tile * BN;
      void* c_part = EPI == EPI_T_STORE_F32 ? (void*)((float*)c + (size_t)w.split * M * N) : c;
      int m = m0 + quarter * 32 + lane;
      // (narrow tiles: the row's old residual values are all asked for before the accumulator is read, so their
      // round trip runs under the wait for the products instead of after it, once per 16 columns)
      constexpr bool EARLY = EPI == EPI_RESIDUAL && BN <= 64;
      // The residual epilogue of the 64-wide tile goes through shared memory, so that the rows it reads and writes
      // in global memory are whole 128-byte lines per eight lanes instead of 16 bytes of 32 different rows per
      // instruction (a thread's accumulator row goes to shared memory, four rows of 32 columns come back per
      // instruction). Measured as links of a chain, with the residual, its copy and the sums of squares: 2048 x 576 x 576
      // 8.3 -> 6.2 µs, 2048 x 576 x 1536 12.9 -> 11.0 µs (the same products with a plain bfloat16 store: 5.9 and 10.8);
      // with 10,946 rows (persistent blocks, the ring in use: the rows are staged behind it, which costs the ring one
      // of its four stages) 33.1 -> 24.1 µs and 42.7 -> 36.0 µs.
      constexpr bool STAGED = EPI == EPI_RESIDUAL && BN == 64;
      const bool staged = STAGED && (N & 3) == 0;
      const int sub = lane >> 3, seg = lane & 7;  // staged: row i * 4 + sub of the warp's 32, floats seg * 4 .. + 3
      float4 old_rows[STAGED ? BN / 32 : 1][STAGED ? 8 : 1];
      if (staged) {
#pragma unroll
        for (int ch = 0; ch < BN / 32; ++ch)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            int mr = m0 + quarter * 32 + i * 4 + sub, nc = n0 + ch * 32 + seg * 4;
            old_rows[STAGED ? ch : 0][STAGED ? i : 0] =
                (mr < M && nc < N) ? *reinterpret_cast<const float4*>((const float*)c + (size_t)mr * N + nc)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
          }
      }
      float4 old[EARLY ? HALF / 4 : 1];
      if (EARLY && !staged && norm.copy_out != nullptr && m < M) {
#pragma unroll
        for (int i = 0; i < HALF / 4; ++i)
          old[i] = n0 + c0 + 4 * i < N
                       ? *reinterpret_cast<const float4*>((const float*)c + (size_t)m * N + n0 + c0 + 4 * i)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      // the token's position and cache page (q/k/v epilogue): a chain of dependent loads that runs under the products
      int pos = 0, page = 0;
      if (EPI == EPI_QKV_ROPE && m < M) {
        pos = rope.tok_pos[m];
        if (rope.write_cache) {
          int slot = rope.slots[rope.tok_seq[m]];
          page = rope.cache.page_table[(size_t)slot * rope.cache.max_pages + pos / rope.cache.page_size];
        }
      }
      // (1 unless the operand is the un-normed copy of the residual; its sums are read while the products run)
      float scale_row = (EPI == EPI_STORE_F32 || EPI == EPI_STORE_T || EPI == EPI_SWIGLU || EPI == EPI_QKV_ROPE)
                            ? row_scale(norm, m, M) : 1.0f;
      if (!mbar_wait(&acc_full[buf], (lt >> 1) & 1)) {
        if (lane == 0) *(volatile int*)status = 4;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      unsigned acc = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * S::ACC_COLS);
      auto release_accumulator = [&]() {  // this warp's last values are in registers: the accumulator may be reused
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      };
      if (EPI == EPI_QKV_ROPE) {
        // The tile is BN / HD whole heads. The thread holds W rotary pairs (i, i + HD / 2) of its token's head at a
        // time: whole heads, one after the other; with eight warps each half of them takes half of the heads where
        // the tile has at least two, else half of the one head's pairs. It rotates them and writes the query, or
        // the key / value into the token's cache row.
        constexpr int HEAD = HD > 0 ? HD : BN;  // (HD is 0 only in instantiations that never take this branch)
        constexpr int SEGS = BN / HEAD;
        constexpr bool SPLIT_HEAD = HALVES == 2 && SEGS == 1 && HEAD >= 64;
        constexpr int W = SPLIT_HEAD ? HEAD / 4 : HEAD / 2;
        int heads = rope.heads, nkv = rope.cache.kv_heads;
        constexpr bool SPLIT_SEGS = HALVES == 2 && SEGS >= 2;
        int seg_begin = SPLIT_SEGS ? half * (SEGS / 2) : 0;
        int seg_end = SPLIT_SEGS ? seg_begin + SEGS / 2 : ((HALVES == 1 || SPLIT_HEAD || half == 0) ? SEGS : 0);
        int first_pair = SPLIT_HEAD ? half * W : 0;
        if (seg_begin >= seg_end) release_accumulator();
#pragma unroll 1
        for (int seg = seg_begin; seg < seg_end; ++seg) {
          float lo[W], hi[W];
#pragma unroll
          for (int col = 0; col < W; col += 16) {
            unsigned v[16];
            tmem_load16(acc + (unsigned)(seg * HEAD + first_pair + col), v);
#pragma unroll
            for (int i = 0; i < 16; ++i) lo[col + i] = __uint_as_float(v[i]) * scale_row;
            tmem_load16(acc + (unsigned)(seg * HEAD + HEAD / 2 + first_pair + col), v);
#pragma unroll
            for (int i = 0; i < 16; ++i) hi[col + i] = __uint_as_float(v[i]) * scale_row;
          }
          if (seg == seg_end - 1) release_accumulator();
          int head = n_tile * SEGS + seg;
          if (m >= M || head >= heads + 2 * nkv || !(head < heads || rope.write_cache)) continue;
          if (rope.table != nullptr && head < heads + nkv) {
            // The table lies pair by pair here, [pair][position]: the 32 tokens of a warp, at consecutive positions in a
            // prompt, then read 256 consecutive bytes per pair. (Position by position, [position][pair], every lane
            // read its own row: 32 lines an instruction, and the rotation cost 5 of the product's 12.5 µs at
            // 2048 x 960 x 576.)
            const float2* cs = rope.table + (size_t)first_pair * rope.table_positions + pos;
#pragma unroll
            for (int i = 0; i < W; ++i) {  // rotary_dim == head_dim here: the partner sits half a head away
              float2 tc = cs[(size_t)i * rope.table_positions];
              float x = lo[i], y = hi[i];
              lo[i] = fmaf(x, tc.x, -(y * tc.y));
              hi[i] = fmaf(x, tc.y, y * tc.x);
            }
          }
          bf16* dst;
          if (head < heads) {
            dst = rope.q_out + ((size_t)m * heads + head) * HEAD;
          } else {
            int which = head < heads + nkv ? 0 : 1;
            int kvh = head - heads - which * nkv;
            dst = (bf16*)rope.cache.base + kv_offset(rope.cache, page, which, kvh, pos % rope.cache.page_size);
          }
#pragma unroll
          for (int i = 0; i < W; i += 8) {
            uint4 o;
            __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) po[j] = __floats2bfloat162_rn(lo[i + 2 * j], lo[i + 2 * j + 1]);
            *reinterpret_cast<uint4*>(dst + first_pair + i) = o;
#pragma unroll
            for (int j = 0; j < 4; ++j) po[j] = __floats2bfloat162_rn(hi[i + 2 * j], hi[i + 2 * j + 1]);
            *reinterpret_cast<uint4*>(dst + HEAD / 2 + first_pair + i) = o;
          }
        }
      } else if (EPI == EPI_SWIGLU && EpilogueStage<BN, EPI, DEEP>::BYTES > 0 && (N & 15) == 0) {
        // SwiGLU, 256-wide tile: the thread's 64 outputs (eight 16-byte pieces) go to its row of the warp's staging
        // space, piece p at place p ^ (row % 8) so that a quarter warp's stores and loads meet different banks; then
        // eight lanes write a row's 128 bytes to global memory together, four rows an instruction.
        unsigned char* stage = tiles + (size_t)S::STAGES * (S::A_BYTES + S::B_BYTES) + (size_t)(warp - 2) * 4096;
#pragma unroll
        for (int cc = 0; cc < HALF; cc += 16) {
          unsigned v[16];
          tmem_load16(acc + (unsigned)(c0 + cc), v);
          if (cc + 16 >= HALF) release_accumulator();
          uint4 o;
          __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            po[i] = __floats2bfloat162_rn(
                silu_for<bf16>(__uint_as_float(v[4 * i]) * scale_row) * (__uint_as_float(v[4 * i + 1]) * scale_row),
                silu_for<bf16>(__uint_as_float(v[4 * i + 2]) * scale_row) * (__uint_as_float(v[4 * i + 3]) * scale_row));
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((((cc >> 4)) ^ (lane & 7)) << 4)) = o;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          int row = i * 4 + (lane >> 3), piece = lane & 7;
          uint4 o = *reinterpret_cast<const uint4*>(stage + row * 128 + ((piece ^ (row & 7)) << 4));
          int mr = m0 + quarter * 32 + row, nc = n0 + c0 + piece * 16;  // (the piece's first accumulator column)
          if (mr < M && nc < N) *reinterpret_cast<uint4*>((bf16*)c + (size_t)mr * (N / 2) + (nc >> 1)) = o;
        }
        __syncwarp();  // (the block's next tile overwrites the staged rows)
      } else if (EPI == EPI_RESIDUAL && BN == 256 && !DEEP && (N & 3) == 0) {
        // The residual epilogue of the 256-wide tile, through shared memory as well: 16 columns at a time (there is
        // room for 32 rows x 20 floats per warp behind four stages of 48 KB), four lanes a row, eight rows an
        // instruction; the old values of the next 32 columns are asked for before these are summed. Measured as links
        // of a chain, with the copy and the sums of squares: 2048 x 2048 x 2048 27.0 µs (a plain bfloat16 store of
        // the same product: 15.2) -> 20.7 µs, 2048 x 4096 x 4096 74.8 µs (53.5) -> 66.5 µs.
        constexpr int LD = 20, CHUNKS = HALF / 16;
        float* st = reinterpret_cast<float*>(tiles + (size_t)S::STAGES * (S::A_BYTES + S::B_BYTES)) +
                    (size_t)(warp - 2) * 32 * LD;
        const int sub8 = lane >> 2, seg4 = lane & 3;  // row i * 8 + sub8 of the warp's 32, floats seg4 * 4 .. + 3
        float squares[4] = {0.f, 0.f, 0.f, 0.f};
        float4 old_now[2][4], old_next[2][4];
        auto ask = [&](float4 (*into)[4], int chunk0) {
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              int mr = m0 + quarter * 32 + i * 8 + sub8, nc = n0 + c0 + (chunk0 + h) * 16 + seg4 * 4;
              into[h][i] = (mr < M && nc < N) ? *reinterpret_cast<const float4*>((const float*)c + (size_t)mr * N + nc)
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        ask(old_now, 0);
#pragma unroll
        for (int pair = 0; pair < CHUNKS / 2; ++pair) {
          if (pair + 1 < CHUNKS / 2) ask(old_next, 2 * pair + 2);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            int chunk = 2 * pair + h;
            unsigned v[16];
            tmem_load16(acc + (unsigned)(c0 + chunk * 16), v);
            if (chunk == CHUNKS - 1) release_accumulator();
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4*>(st + lane * LD + i) =
                  make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                              __uint_as_float(v[i + 3]));
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              int row = i * 8 + sub8, mr = m0 + quarter * 32 + row, nc = n0 + c0 + chunk * 16 + seg4 * 4;
              float4 a = *reinterpret_cast<const float4*>(st + row * LD + seg4 * 4);
              if (mr < M && nc < N) {
                float4 r = old_now[h][i];
                r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
                *reinterpret_cast<float4*>((float*)c + (size_t)mr * N + nc) = r;
                if (norm.copy_out != nullptr) {
                  __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
                  *reinterpret_cast<uint2*>(norm.copy_out + (size_t)mr * N + nc) =
                      make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
                  squares[i] = fmaf(r.x, r.x, fmaf(r.y, r.y, fmaf(r.z, r.z, fmaf(r.w, r.w, squares[i]))));
                }
              }
            }
            __syncwarp();  // (the next 16 columns overwrite the staged rows)
          }
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) old_now[h][i] = old_next[h][i];
        }
        if (norm.ssq_out != nullptr) {  // a row's four lanes, summed in a fixed order
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float v = squares[i];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            int mr = m0 + quarter * 32 + i * 8 + sub8;
            if (seg4 == 0 && mr < M) norm.ssq_out[(size_t)(HALVES * n_tile + half) * M + mr] = v;
          }
        }
      } else if (staged) {
        constexpr int LD = 36;  // floats per staged row: 16-byte pieces, rows of a quarter warp in different banks
        float* st = reinterpret_cast<float*>(DEEP ? tiles : tiles + (size_t)S::STAGES * (S::A_BYTES + S::B_BYTES)) +
                    (size_t)(warp - 2) * 32 * LD;
        float squares[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) squares[i] = 0.f;
#pragma unroll
        for (int ch = 0; ch < BN / 32; ++ch) {
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            unsigned v[16];
            tmem_load16(acc + (unsigned)(ch * 32 + part * 16), v);
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4*>(st + lane * LD + part * 16 + i) =
                  make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                              __uint_as_float(v[i + 3]));
          }
          if (ch == BN / 32 - 1) release_accumulator();
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            int row = i * 4 + sub, mr = m0 + quarter * 32 + row, nc = n0 + ch * 32 + seg * 4;
            float4 a = *reinterpret_cast<const float4*>(st + row * LD + seg * 4);
            if (mr < M && nc < N) {
              float4 r = old_rows[STAGED ? ch : 0][STAGED ? i : 0];
              r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
              *reinterpret_cast<float4*>((float*)c + (size_t)mr * N + nc) = r;
              if (norm.copy_out != nullptr) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
                *reinterpret_cast<uint2*>(norm.copy_out + (size_t)mr * N + nc) =
                    make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
                squares[i] = fmaf(r.x, r.x, fmaf(r.y, r.y, fmaf(r.z, r.z, fmaf(r.w, r.w, squares[i]))));
              }
            }
          }
          __syncwarp();  // (the next 32 columns overwrite the staged rows)
        }
        if (norm.ssq_out != nullptr) {  // a row's eight lanes, summed in a fixed order
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float v = squares[i];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            int mr = m0 + quarter * 32 + i * 4 + sub;
            if (seg == 0 && mr < M) norm.ssq_out[(size_t)n_tile * M + mr] = v;
          }
        }
      } else {
        float ssq = 0.f;  // EPI_RESIDUAL with norm.copy_out: the squares of the new residual values of this half tile
#pragma unroll
        for (int cc = 0; cc < HALF; cc += 16) {
          int col = c0 + cc;
          unsigned v[16];
          tmem_load16(acc + (unsigned)col, v);
          if (cc + 16 >= HALF) release_accumulator();
          float f[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(v[i]) * scale_row;
          if (EPI == EPI_RESIDUAL && norm.copy_out != nullptr) {
            // the residual sum, its bfloat16 copy and its squares (N is a multiple of 16 in this mode)
            int n = n0 + col;
            if (m < M && n < N) {
              float* __restrict__ dst = (float*)c + (size_t)m * N + n;
              float4 r[4];
#pragma unroll
              for (int i = 0; i < 4; ++i)
                r[i] = EARLY ? old[EARLY ? cc / 4 + i : 0] : *reinterpret_cast<const float4*>(dst + 4 * i);
              unsigned pk[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                r[i].x += f[4 * i]; r[i].y += f[4 * i + 1]; r[i].z += f[4 * i + 2]; r[i].w += f[4 * i + 3];
                ssq = fmaf(r[i].x, r[i].x, ssq); ssq = fmaf(r[i].y, r[i].y, ssq);
                ssq = fmaf(r[i].z, r[i].z, ssq); ssq = fmaf(r[i].w, r[i].w, ssq);
                __nv_bfloat162 lo = __floats2bfloat162_rn(r[i].x, r[i].y), hi = __floats2bfloat162_rn(r[i].z, r[i].w);
                pk[2 * i] = *reinterpret_cast<unsigned*>(&lo);
                pk[2 * i + 1] = *reinterpret_cast<unsigned*>(&hi);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(dst + 4 * i) = r[i];
              uint4* __restrict__ copy = reinterpret_cast<uint4*>(norm.copy_out + (size_t)m * N + n);
              copy[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              copy[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
          } else if (EPI >= EPI_T_STORE_F32) {
            epilogue_col16<EPI, bf16>(c_part, m, n0 + col, M, N, f);  // the tile is C^T
          } else {
            epilogue_row16<EPI, bf16>(c, m, n0 + col, M, N, f);
          }
        }
        // (a part per warp's share of the tile's columns: the reader sums parts in order, whoever wrote them)
        if (EPI == EPI_RESIDUAL && norm.ssq_out != nullptr && m < M)
          norm.ssq_out[(size_t)(HALVES * n_tile + half) * M + m] = ssq;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    tmem_dealloc(tmem_base, (unsigned)S::TMEM_COLS);
  }
}

template <int BN, int EPI, bool DEEP, int HD>
int launch_shape(void* c, const CUtensorMap& map_a, const CUtensorMap& map_w, int M, int N, int K, int* status,
                 cudaStream_t stream, const RopeArgs& rope, int m_tiles, int n_tiles, int sms, const NormArgs& norm,
                 int k_split = 1) {
  typedef Shape<BN, DEEP, EpilogueStage<BN, EPI, DEEP>::BYTES> S;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, DEEP, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)S::SMEM) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  long long total = (long long)m_tiles * n_tiles * k_split;
  int blocks = sms * S::BLOCKS_PER_SM;
  if (blocks > total) blocks = (int)total;
  return dllm_launch_pdl(gemm_tcgen05_kernel<BN, EPI, DEEP, HD>, dim3(blocks), dim3(S::THREADS), S::SMEM, stream, map_a, map_w,
                         c, M, N, K, status, rope, m_tiles, n_tiles, k_split, norm);
}

template <int BN, int EPI, int HD = 0>
int launch(void* c, const void* a, const void* w, int M, int N, int K, int* status, cudaStream_t stream,
           const RopeArgs& rope = RopeArgs{}, const NormArgs& norm = NormArgs{}, int k_split = 1) {
  alignas(64) CUtensorMap map_a, map_w;
  if (!make_map(&map_a, a, M, K, BM) || !make_map(&map_w, w, N, K, BN)) return DLLM_LAUNCH_FAILED;
  int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  long long total = (long long)m_tiles * n_tiles;
  if (total * k_split > 0x7fffffff) return DLLM_UNSUPPORTED_SIZE;
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      return DLLM_LAUNCH_FAILED;
  }
  constexpr bool CAN_DEEP = BN == 64 && EPI <= EPI_QKV_ROPE;  // (the shapes where it was measured to pay)
  if (CAN_DEEP && total <= sms && K > 4 * BK)
    return launch_shape<BN, EPI, CAN_DEEP, HD>(c, map_a, map_w, M, N, K, status, stream, rope, m_tiles, n_tiles, sms,
                                               norm);
  return launch_shape<BN, EPI, false, HD>(c, map_a, map_w, M, N, K, status, stream, rope, m_tiles, n_tiles, sms, norm,
                                          k_split);
}

template <int BN>
int dispatch(void* c, const void* a, const void* w, int M, int N, int K, int epilogue, int* status,
             cudaStream_t stream, const NormArgs& norm = NormArgs{}, int k_split = 1) {
  switch (epilogue) {
    case EPI_STORE_F32: return launch<BN, EPI_STORE_F32>(c, a, w, M, N, K, status, stream, RopeArgs{}, norm);
    case EPI_STORE_T: return launch<BN, EPI_STORE_T>(c, a, w, M, N, K, status, stream, RopeArgs{}, norm);
    case EPI_RESIDUAL: return launch<BN, EPI_RESIDUAL>(c, a, w, M, N, K, status, stream, RopeArgs{}, norm);
    case EPI_SWIGLU: return launch<BN, EPI_SWIGLU>(c, a, w, M, N, K, status, stream, RopeArgs{}, norm);
    case EPI_T_STORE_F32:
      return launch<BN, EPI_T_STORE_F32>(c, a, w, M, N, K, status, stream, RopeArgs{}, NormArgs{}, k_split);
    case EPI_T_STORE_T: return launch<BN, EPI_T_STORE_T>(c, a, w, M, N, K, status, stream);
    case EPI_T_RESIDUAL: return launch<BN, EPI_T_RESIDUAL>(c, a, w, M, N, K, status, stream);
    case EPI_T_SWIGLU: return launch<BN, EPI_T_SWIGLU>(c, a, w, M, N, K, status, stream);
    default: return DLLM_BAD_ARGUMENT;
  }
}
}  // namespace

// C = A[M,K] * W[N,K]^T (bfloat16, float32 accumulation in tensor memory). K must be a multiple of 8 (16-byte row
// pitch for TMA), N even for the SwiGLU epilogue, and A and W 16-byte aligned. `tile_n`: 32, 64 or 128 columns of C per block (0 chooses).
// `status` is a word the device can write (device or pinned host memory); the kernel sets it non-zero if one of its
// bounded waits ran out (2: producer, 3: product issuer, 4: epilogue).
// Epilogues 5..8 are 0..3 for a product taken the other way round: the caller passes W as A (M = output features)
// and the activations as W (N = tokens), and C is still [tokens, features]; for a few tokens and a large W this
// streams W through 128-row tiles once instead of re-reading it for every 128 rows of a mostly empty tile of tokens.
static int gemm_entry(void* c, const void* a, const void* w, int M, int N, int K, int epilogue, int tile_n,
                      int* status, cudaStream_t stream, const NormArgs& norm, int* n_tiles_out, int k_split = 1) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (k_split < 1 || k_split > 32 || k_split > (K + BK - 1) / BK || (k_split > 1 && epilogue != EPI_T_STORE_F32))
    return DLLM_BAD_ARGUMENT;
  if (K <= 0 || (K & 7) || ((N & 1) && epilogue == EPI_SWIGLU) || ((M & 1) && epilogue == EPI_T_SWIGLU) ||
      ((uintptr_t)a & 15) || ((uintptr_t)w & 15) || status == nullptr)
    return DLLM_UNSUPPORTED_SIZE;
  if (tile_n == 0) {
    long long m_tiles = (M + BM - 1) / BM;
    long long tiles256 = m_tiles * ((N + 255) / 256);
    if (M <= 256) tile_n = 32;  // few rows: many narrow tiles
    // enough 256-wide tiles to give every multiprocessor one: the widest tile reuses A most (measured: 1.0 to 1.4
    // PFLOP/s from K = 2048 up, against 0.6 to 1.2 for the 128-wide tile; at K = 576, 2048 x 3072 with SwiGLU:
    // 11.5 µs against 12.7 and 13.5 for 128 and 64)
    else if (N % 256 == 0 && tiles256 >= 128) tile_n = 256;
    else if (N % 128 == 0 && N >= 2048 && K >= 1024) tile_n = 128;
    // (32-wide tiles for a narrow output, 2048 x 576, are 0.2 to 0.5 µs faster alone and slower in a step: twice
    // the parts of the rows' sums of squares for the next product to read)
    else tile_n = 64;
  }
  if (n_tiles_out != nullptr)  // (a part per epilogue warp's share of a tile: see the epilogue)
    *n_tiles_out = (tile_n >= 128 ? 2 : 1) * ((N + tile_n - 1) / tile_n);
  switch (tile_n) {
    case 32: return dispatch<32>(c, a, w, M, N, K, epilogue, status, stream, norm, k_split);
    case 64: return dispatch<64>(c, a, w, M, N, K, epilogue, status, stream, norm, k_split);
    case 128: return dispatch<128>(c, a, w, M, N, K, epilogue, status, stream, norm, k_split);
    case 256: return dispatch<256>(c, a, w, M, N, K, epilogue, status, stream, norm, k_split);
    default: return DLLM_BAD_ARGUMENT;
  }
}

DLLM_EXPORT int dllm_gemm_tcgen05(void* c, const void* a, const void* w, int M, int N, int K, int epilogue, int tile_n,
                                  int* status, cudaStream_t stream) {
  return gemm_entry(c, a, w, M, N, K, epilogue, tile_n, status, stream, NormArgs{}, nullptr);
}

// A product of few tokens with a W of few rows and a long reduction, the other way round as epilogues 5..8 and with the
// reduction cut into `k_split` stretches so that the device's multiprocessors all stream a part of W:
// parts[s][tokens, features] (float32, k_split of them one behind the other) = X W^T over stretch s of the k tiles.
// `w` is [features, K], `x` is [tokens, K]; the caller sums the parts in order (dllm_sum_parts_residual).
DLLM_EXPORT int dllm_gemm_tcgen05_split(float* parts, const void* w, const void* x, int features, int tokens, int K,
                                        int k_split, int tile_n, int* status, cudaStream_t stream) {
  if (tile_n != 32 && tile_n != 64) return DLLM_BAD_ARGUMENT;
  return gemm_entry(parts, w, x, features, tokens, K, EPI_T_STORE_F32, tile_n, status, stream, NormArgs{}, nullptr,
                    k_split);
}

// The same product with an RMSNorm folded around it (see NormArgs in gemm_common.cuh), for prefill-sized steps.
// `a` is the bfloat16 copy of the un-normed residual rows, `w` carries the norm's weight in its columns, and every
// row of the result is scaled by 1 / sqrt(sum of its `parts_in` sums of squares / K + eps) before the epilogue
// (store float32, store bfloat16 or SwiGLU).
DLLM_EXPORT int dllm_gemm_tcgen05_normed(void* c, const void* a, const void* w, int M, int N, int K, int epilogue,
                                         const float* ssq_in, int parts_in, float eps, int* status,
                                         cudaStream_t stream) {
  if (ssq_in == nullptr || parts_in <= 0 || (epilogue != EPI_STORE_F32 && epilogue != EPI_STORE_T &&
                                             epilogue != EPI_SWIGLU))
    return DLLM_BAD_ARGUMENT;
  NormArgs norm{ssq_in, parts_in, 1.0f / (float)K, eps, nullptr, nullptr};
  return gemm_entry(c, a, w, M, N, K, epilogue, 0, status, stream, norm, nullptr);
}

// x[M,N] (float32) += A W^T, and for the norm that reads x next: copy_out[M,N] = bfloat16(new x) and
// ssq_out[tile][m] = the sum of the squares of row m's new values in column tile `tile`; *parts_out = the number of
// parts, two a column tile (what the reader passes as parts_in). N must be a multiple of 16; ssq_out holds
// M * ceil(N / 16) floats at least.
DLLM_EXPORT int dllm_gemm_tcgen05_residual_norm(void* x, void* copy_out, float* ssq_out, int* parts_out, const void* a,
                                                const void* w, int M, int N, int K, int* status,
                                                cudaStream_t stream) {
  if (copy_out == nullptr || ssq_out == nullptr || parts_out == nullptr) return DLLM_BAD_ARGUMENT;
  if ((N & 15) || ((uintptr_t)copy_out & 15) || ((uintptr_t)x & 15)) return DLLM_UNSUPPORTED_SIZE;
  NormArgs norm{nullptr, 0, 0.f, 0.f, ssq_out, (bf16*)copy_out};
  return gemm_entry(x, a, w, M, N, K, EPI_RESIDUAL, 0, status, stream, norm, parts_out);
}

// The q/k/v projection of a prefill-sized step in one kernel: W is [(heads + 2 kv_heads) * head_dim, K], every tile
// of the product is one or several whole heads (head_dim 32, 64 or 128; rotary_dim equal to head_dim, or no table), its epilogue
// rotates q and k by the table's angle for each token's position and writes q to q_out and k, v into the paged cache.
// The table is laid out pair by pair: [rotary_dim / 2][table_positions](cos, sin).
static int qkv_rope_entry(const void* a, const void* w, int M, int K, void* q_out, void* cache_base,
                          const int* page_table, int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                          const float* table, int rotary_dim, int table_positions, const int* tok_seq,
                          const int* tok_pos, const int* slots, int write_cache, int* status, cudaStream_t stream,
                          const NormArgs& norm) {
  if (M <= 0) return DLLM_OK;
  if (table != nullptr && table_positions <= 0) return DLLM_BAD_ARGUMENT;
  if (K <= 0 || (K & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15) || status == nullptr || heads <= 0 ||
      kv_heads <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  if ((head_dim != 32 && head_dim != 64 && head_dim != 128) || (table != nullptr && rotary_dim != head_dim))
    return DLLM_UNSUPPORTED_SIZE;
  RopeArgs rope{(bf16*)q_out, KvLayout{cache_base, page_table, max_pages, page_size, kv_heads, head_dim},
                (const float2*)table, table ? rotary_dim : 0, heads, tok_seq, tok_pos, slots, write_cache, -1,
                table_positions};
  int N = (heads + 2 * kv_heads) * head_dim;
  // a tile is one head, or four heads of 64 / two of 128 where the product is large enough to fill the device with
  // the wide tiles (which reuse A four times as often: 1.0 to 1.2 PFLOP/s against 0.6)
  bool wide = M >= 1024 && K >= 1024 && (long long)((M + BM - 1) / BM) * ((N + 255) / 256) >= 64;
  switch (head_dim) {
    case 32: return launch<32, EPI_QKV_ROPE, 32>(nullptr, a, w, M, N, K, status, stream, rope, norm);
    case 64:
      if (wide) return launch<256, EPI_QKV_ROPE, 64>(nullptr, a, w, M, N, K, status, stream, rope, norm);
      return launch<64, EPI_QKV_ROPE, 64>(nullptr, a, w, M, N, K, status, stream, rope, norm);
    default:
      if (wide) return launch<256, EPI_QKV_ROPE, 128>(nullptr, a, w, M, N, K, status, stream, rope, norm);
      return launch<128, EPI_QKV_ROPE, 128>(nullptr, a, w, M, N, K, status, stream, rope, norm);
  }
}

DLLM_EXPORT int dllm_gemm_tcgen05_qkv_rope(const void* a, const void* w, int M, int K, void* q_out, void* cache_base,
                                           const int* page_table, int max_pages, int page_size, int heads,
                                           int kv_heads, int head_dim, const float* table, int rotary_dim,
                                           int table_positions, const int* tok_seq, const int* tok_pos,
                                           const int* slots, int write_cache, int* status, cudaStream_t stream) {
  return qkv_rope_entry(a, w, M, K, q_out, cache_base, page_table, max_pages, page_size, heads, kv_heads, head_dim,
                        table, rotary_dim, table_positions, tok_seq, tok_pos, slots, write_cache, status, stream,
                        NormArgs{});
}

// The same with the RMSNorm folded around it: `a` is the bfloat16 copy of the un-normed residual rows, `w` carries
// the norm's weight in its columns, rows are scaled by 1 / sqrt(sum of parts / K + eps) before rotation and stores.
DLLM_EXPORT int dllm_gemm_tcgen05_qkv_rope_normed(const void* a, const void* w, int M, int K, void* q_out,
                                                  void* cache_base, const int* page_table, int max_pages,
                                                  int page_size, int heads, int kv_heads, int head_dim,
                                                  const float* table, int rotary_dim, int table_positions,
                                                  const int* tok_seq, const int* tok_pos, const int* slots,
                                                  int write_cache, const float* ssq_in, int parts_in, float eps,
                                                  int* status, cudaStream_t stream) {
  if (ssq_in == nullptr || parts_in <= 0 || K <= 0) return DLLM_BAD_ARGUMENT;
  NormArgs norm{ssq_in, parts_in, 1.0f / (float)K, eps, nullptr, nullptr};
  return qkv_rope_entry(a, w, M, K, q_out, cache_base, page_table, max_pages, page_size, heads, kv_heads, head_dim,
                        table, rotary_dim, table_positions, tok_seq, tok_pos, slots, write_cache, status, stream, norm);
}
