// Embedding gather, RMSNorm (optionally of gathered rows), rotary position encoding fused with the cache write,
// and the residual add. The residual stream is float32 in both precisions; norms and rotations are computed in
// float32 and rounded once to the output type.
#include "common.cuh"

// ---- embedding: x[r, :] = float(table[token_r, :]) ----------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ tokens,
                             int hidden, int vocab, int* __restrict__ status) {
  int row = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  int token = tokens[row];
  if (token < 0 || token >= vocab) {  // refused, never read out of range
    if (threadIdx.x == 0) *(volatile int*)status = 64;  // (a word in device or pinned host memory)
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)row * hidden + i] = 0.f;
    return;
  }
  const T* src = table + (size_t)token * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)row * hidden + i] = to_float(src[i]);
}

DLLM_EXPORT int dllm_embed(float* out, const void* table, const int* tokens, int rows, int hidden, int vocab,
                           int dtype, int* status, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (hidden <= 0 || vocab <= 0) return DLLM_BAD_ARGUMENT;
  int threads = hidden >= 256 ? 256 : 64;
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(embed_kernel<float>, dim3(rows), dim3(threads), 0, stream, out, (const float*)table,
                           tokens, hidden, vocab, status);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(embed_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, out,
                           (const __nv_bfloat16*)table, tokens, hidden, vocab, status);
  return DLLM_BAD_ARGUMENT;
}

// ---- RMSNorm: out[r] = x[rows ? rows[r] : r] * (1 / sqrt(mean(x^2) + eps)) * w ---------------------------------------
// One block per row; each thread sums a strided part, then a fixed-order block reduction, so a row's result does not
// depend on which other rows are in the launch.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ weight,
                               const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float partial[32];
  int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = src[i];
    sum = fmaf(v, v, sum);
  }
  sum = warp_sum(sum);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float v = lane < warps ? partial[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) partial[0] = 1.0f / sqrtf(v / (float)hidden + eps);
  }
  __syncthreads();
  float inv = partial[0];
  T* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<T>(src[i] * inv * weight[i]);
}

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
  *reinterpret_cast<uint2*>(dst) = packed;
}

// Narrow rows (hidden a multiple of 4, at most 4096 floats): one warp per row, the row kept in registers between
// the sum and the scaling, 16-byte loads. Lane l holds floats 4*(l + 32*i) ..; the sum is a fixed tree.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                           const float* __restrict__ weight,
                                                           const int* __restrict__ rows, int n_rows, int hidden,
                                                           float eps) {
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * hidden);
  int vecs = hidden >> 2;
  float4 v[32];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      v[i] = src[idx];
      sum = fmaf(v[i].x, v[i].x, sum); sum = fmaf(v[i].y, v[i].y, sum);
      sum = fmaf(v[i].z, v[i].z, sum); sum = fmaf(v[i].w, v[i].w, sum);
    }
  }
  sum = warp_sum(sum);
  float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
  const float4* wv = reinterpret_cast<const float4*>(weight);
  T* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      float4 w4 = wv[idx];
      store4(dst + 4 * idx, v[i].x * inv * w4.x, v[i].y * inv * w4.y, v[i].z * inv * w4.z, v[i].w * inv * w4.w);
    }
  }
}

DLLM_EXPORT int dllm_rmsnorm(void* out, const float* x, const float* weight, const int* rows, int n_rows, int hidden,
                             float eps, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return DLLM_OK;
  if (hidden <= 0) return DLLM_BAD_ARGUMENT;
  if ((hidden & 3) == 0 && hidden <= 4096) {  // whatever the number of rows, so a row has the same bits everywhere
    int blocks = (n_rows + 7) / 8;
    if (out_dtype == DLLM_F32)
      return dllm_launch_pdl(rmsnorm_warp_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, x, weight, rows,
                             n_rows, hidden, eps);
    if (out_dtype == DLLM_BF16)
      return dllm_launch_pdl(rmsnorm_warp_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                             (__nv_bfloat16*)out, x, weight, rows, n_rows, hidden, eps);
    return DLLM_BAD_ARGUMENT;
  }
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == DLLM_F32)
    rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>((float*)out, x, weight, rows, hidden, eps);
  else if (out_dtype == DLLM_BF16)
    rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>((__nv_bfloat16*)out, x, weight, rows, hidden, eps);
  else
    return DLLM_BAD_ARGUMENT;
  return dllm_launch_status();
}

// ---- what a norm folded around the next product needs of the first rows of a step -------------------------------
// copy[r] = bfloat16(x[r]) and ssq[r] = sum of x[r]^2 (one part a row): a warp a row, any width that is a multiple
// of 4 (see NormArgs in gemm_common.cuh; later rows come from the epilogue of the products that write the residual).
__global__ void __launch_bounds__(256) cast_ssq_kernel(__nv_bfloat16* __restrict__ copy, float* __restrict__ ssq,
                                                       const float* __restrict__ x, int n_rows, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)r * hidden);
  float sum = 0.f;
  for (int idx = lane; idx < (hidden >> 2); idx += 32) {
    float4 v = src[idx];
    sum = fmaf(v.x, v.x, sum); sum = fmaf(v.y, v.y, sum);
    sum = fmaf(v.z, v.z, sum); sum = fmaf(v.w, v.w, sum);
    store4(copy + (size_t)r * hidden + 4 * idx, v.x, v.y, v.z, v.w);
  }
  sum = warp_sum(sum);
  if (lane == 0) ssq[r] = sum;
}

DLLM_EXPORT int dllm_cast_ssq(void* copy, float* ssq, const float* x, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return DLLM_OK;
  if (hidden <= 0 || (hidden & 3) || copy == nullptr || ssq == nullptr) return DLLM_UNSUPPORTED_SIZE;
  return dllm_launch_pdl(cast_ssq_kernel, dim3((n_rows + 7) / 8), dim3(256), 0, stream, (__nv_bfloat16*)copy, ssq, x,
                         n_rows, hidden);
}

// ---- rotary encoding + cache write --------------------------------------------------------------------------------
// qkv is the float32 output of the fused q/k/v projection, [tokens, (heads + 2 kv_heads) * head_dim]. Queries and
// keys rotate pairs (i, i + rotary_dim/2) by the angle whose cosine and sine the table holds for the token's
// position; dimensions beyond rotary_dim pass through. Queries go to q_out, keys and values into the token's
// place in the paged cache (page_table[slot][pos / page_size], row pos % page_size). With parts > 1, qkv is that
// many partial results of the projection, `part_stride` floats apart, and a value is their sum in order.
template <typename T>
__global__ void rope_cache_kernel(const float* __restrict__ qkv, T* __restrict__ q_out, KvLayout cache,
                                  const float2* __restrict__ table, int rotary_dim, int heads,
                                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                  const int* __restrict__ slots, int write_cache, int parts, size_t part_stride) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x, h = blockIdx.y;
  int hd = cache.head_dim, nkv = cache.kv_heads;
  if (!write_cache && h >= heads) return;
  int pos = tok_pos[t];
  const float* src = qkv + ((size_t)t * (heads + 2 * nkv) + h) * hd;
  T* dst;
  bool rotate = h < heads + nkv && table != nullptr;
  if (h < heads) {
    dst = q_out + ((size_t)t * heads + h) * hd;
  } else {
    int which = h < heads + nkv ? 0 : 1;
    int g = h - heads - which * nkv;
    int slot = slots[tok_seq[t]];
    int page = cache.page_table[(size_t)slot * cache.max_pages + pos / cache.page_size];
    dst = (T*)cache.base + kv_offset(cache, page, which, g, pos % cache.page_size);
  }
  int half = rotary_dim / 2;
  auto value = [&](int i) {
    float sum = src[i];
    for (int p = 1; p < parts; ++p) sum += src[(size_t)p * part_stride + i];
    return sum;
  };
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    float v = value(i);
    if (rotate && i < rotary_dim) {
      int j = i < half ? i : i - half;
      float2 cs = table[(size_t)pos * half + j];
      float a = value(j), b = value(j + half);
      v = i < half ? fmaf(a, cs.x, -(b * cs.y)) : fmaf(a, cs.y, b * cs.x);
    }
    dst[i] = from_float<T>(v);
  }
}

DLLM_EXPORT int dllm_rope_cache_write(const float* qkv, void* q_out, void* cache_base, const int* page_table,
                                      int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                      const float* table, int rotary_dim, const int* tok_seq, const int* tok_pos,
                                      const int* slots, int tokens, int write_cache, int dtype, int parts,
                                      long long part_stride, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || head_dim <= 0 || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) ||
      parts < 1 || part_stride < 0)
    return DLLM_BAD_ARGUMENT;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  dim3 grid(tokens, heads + 2 * kv_heads);
  int threads = head_dim >= 128 ? 128 : (head_dim > 32 ? 64 : 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(rope_cache_kernel<float>, grid, dim3(threads), 0, stream, qkv, (float*)q_out, cache,
                           (const float2*)table, rotary_dim, heads, tok_seq, tok_pos, slots, write_cache, parts,
                           (size_t)part_stride);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(rope_cache_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, qkv,
                           (__nv_bfloat16*)q_out, cache, (const float2*)table, rotary_dim, heads, tok_seq, tok_pos,
                           slots, write_cache, parts, (size_t)part_stride);
  return DLLM_BAD_ARGUMENT;
}

// ---- residual += update (float32 sum) -----------------------------------------------------------------------------
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ residual, const T* __restrict__ update, size_t count) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) residual[i] += to_float(update[i]);
}

DLLM_EXPORT int dllm_add_residual(float* residual, const void* update, long long count, int dtype,
                                  cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  unsigned blocks = (unsigned)((count + 255) / 256);
  if (dtype == DLLM_F32)
    add_residual_kernel<float><<<blocks, 256, 0, stream>>>(residual, (const float*)update, (size_t)count);
  else if (dtype == DLLM_BF16)
    add_residual_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(residual, (const __nv_bfloat16*)update,
                                                                    (size_t)count);
  else
    return DLLM_BAD_ARGUMENT;
  return dllm_launch_status();
}

// ---- residual += parts[0] + parts[1] + ... (the partial results of a product whose reduction was cut) ------------
// parts holds `k_split` float32 arrays of `count` values one behind the other; they are summed in that order, then
// added to the residual. count must be a multiple of 4 and the arrays 16-byte aligned.
__global__ void __launch_bounds__(256) sum_parts_residual_kernel(float* __restrict__ residual,
                                                                 const float* __restrict__ parts, int k_split,
                                                                 size_t count) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= count) return;
  float4 old = *reinterpret_cast<const float4*>(residual + i);
  float4 sum = __ldcg(reinterpret_cast<const float4*>(parts + i));
  for (int s = 1; s < k_split; ++s) {
    float4 p = __ldcg(reinterpret_cast<const float4*>(parts + (size_t)s * count + i));
    sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
  }
  old.x += sum.x; old.y += sum.y; old.z += sum.z; old.w += sum.w;
  *reinterpret_cast<float4*>(residual + i) = old;
}

DLLM_EXPORT int dllm_sum_parts_residual(float* residual, const float* parts, int k_split, long long count,
                                        cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  if (k_split < 1 || (count & 3) || ((uintptr_t)residual & 15) || ((uintptr_t)parts & 15)) return DLLM_UNSUPPORTED_SIZE;
  unsigned blocks = (unsigned)((count / 4 + 255) / 256);
  return dllm_launch_pdl(sum_parts_residual_kernel, dim3(blocks), dim3(256), 0, stream, residual, parts, k_split,
                         (size_t)count);
}

// ---- decode feedback: the chosen tokens become the next step's input, positions move on by one -------------------
// Lets single-token steps follow one another on the device without the host: tokens[b] = chosen[b], positions and
// cached lengths + 1, and the chosen tokens are appended to `history` ([capacity, batch]) at row *counter.
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ tok_pos, int* __restrict__ start,
                                      const int* __restrict__ chosen, int* __restrict__ history,
                                      int* __restrict__ counter, int batch, int capacity) {
  pdl_wait();
  int row = *counter;
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    int token = chosen[b];
    tokens[b] = token;
    tok_pos[b] += 1;
    start[b] += 1;
    if (row < capacity) history[(size_t)row * batch + b] = token;
  }
  __syncthreads();
  if (threadIdx.x == 0) *counter = row + 1;
}

DLLM_EXPORT int dllm_decode_advance(int* tokens, int* tok_pos, int* start, const int* chosen, int* history,
                                    int* counter, int batch, int capacity, cudaStream_t stream) {
  if (batch <= 0) return DLLM_OK;
  return dllm_launch_pdl(decode_advance_kernel, dim3(1), dim3(256), 0, stream, tokens, tok_pos, start, chosen,
                         history, counter, batch, capacity);
}

// A copy from pinned host memory to the device on the given stream (the host side of a step makes two small ones: the
// step's metadata and the page-table rows that changed; through this entry point each costs the host a few
// microseconds less than through the tensor library's dispatch).
DLLM_EXPORT int dllm_copy_to_device(void* dst, const void* src, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return DLLM_OK;
  if (dst == nullptr || src == nullptr) return DLLM_BAD_ARGUMENT;
  return cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream) == cudaSuccess ? DLLM_OK
                                                                                                 : DLLM_LAUNCH_FAILED;
}

// Takes token ids out of the choice while an output is shorter than it has to be: logits[row, ids[i]] = -inf for
// every row, if *produced + *steps < min_tokens (`produced`: tokens every sequence of the batch has so far when a run
// of steps begins; `steps`: the steps of that run so far, or null). A probability of exactly zero is never drawn and
// never the largest, so what is chosen is what a choice among the other tokens alone would choose.
__global__ void mask_tokens_kernel(float* __restrict__ logits, int rows, int vocab, const int* __restrict__ ids,
                                   int n_ids, const int* __restrict__ produced, const int* __restrict__ steps,
                                   int min_tokens) {
  pdl_wait();
  int have = *produced + (steps != nullptr ? *steps : 0);
  if (have >= min_tokens) return;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * n_ids; i += gridDim.x * blockDim.x) {
    int id = ids[i % n_ids];
    if (id >= 0 && id < vocab) logits[(size_t)(i / n_ids) * vocab + id] = -INFINITY;
  }
}

DLLM_EXPORT int dllm_mask_tokens(float* logits, int rows, int vocab, const int* ids, int n_ids, const int* produced,
                                 const int* steps, int min_tokens, cudaStream_t stream) {
  if (rows <= 0 || n_ids <= 0 || min_tokens <= 0) return DLLM_OK;
  if (vocab <= 0 || logits == nullptr || ids == nullptr || produced == nullptr) return DLLM_BAD_ARGUMENT;
  return dllm_launch_pdl(mask_tokens_kernel, dim3(1), dim3(256), 0, stream, logits, rows, vocab, ids, n_ids, produced,
                         steps, min_tokens);
}
