// What sits between an attention's input projection and its score kernel, for layouts the fused
// q/k/v epilogues do not cover.  Float32 arithmetic, one rounding on the way out.
//
//   hfee_rope_norm_cache        per head: rotate `rope_dim` dimensions that start anywhere in the head
//                               (dimension i with i + rope_dim/2), then optionally divide the head by its
//                               root mean square (no weight); queries to a buffer whose head stride and
//                               offset may differ from the source's, keys into their cache page at an
//                               offset within the cached vector, values copied to theirs.  Key and value
//                               sizes are independent.
//   hfee_latent_norm_rope_cache one token's down-projections of a latent attention: the query latent
//                               RMS-normed with its weight into a buffer, the key/value latent RMS-normed
//                               with its weight into the leading dimensions of the token's cached vector,
//                               the rotated tail behind it.
//   hfee_attention_prepare     one token's [q | k | v] projection on its way to the score kernel: a bias per column
//                               (each optional), an RMS norm with a weight over the whole query and the whole key
//                               projection (all heads at once; optional), then the rotation of the first `rope_dim`
//                               dimensions of every query and key head, pairing dimension i with i + rope_dim/2 or
//                               2i with 2i + 1; queries to a buffer, keys and values to their cache pages.  Key and
//                               value sizes are independent.  One block per token, the row in shared memory.
#include "common.cuh"

namespace {

constexpr int RN_WARPS = 4;
constexpr int RN_MAX_LEN = 640;
constexpr int RN_PER_LANE = RN_MAX_LEN / 32;

struct HeadGroup {
  int count;          // heads of this kind
  int src_off;        // column of head 0 in the source row
  int src_stride;     // columns from one head to the next
  int len;            // dimensions taken per head
  int rope_off;       // first rotated dimension within the head (ignored without a table)
  int dst_off;        // where the head's dimensions start in the destination vector
  int dst_stride;     // query buffer: columns from one head to the next; pools: unused
};

// x[d] of a head after rotation; the partner dimension is read from the source as well
template <typename T>
__device__ __forceinline__ float rotated(const T* __restrict__ x, int d, int rope_off, int rope_dim,
                                         const float* __restrict__ cs) {
  const float v = to_f32<T>(x[d]);
  const int half = rope_dim >> 1, r = d - rope_off;
  if (cs == nullptr || r < 0 || r >= rope_dim) return v;
  if (r < half) return v * cs[2 * r] - to_f32<T>(x[d + half]) * cs[2 * r + 1];
  const int i = r - half;
  return v * cs[2 * i] + to_f32<T>(x[d - half]) * cs[2 * i + 1];
}

// PER_LANE: dimensions of a head per lane (heads of at most 32 * PER_LANE dimensions)
template <typename T, int PER_LANE>
__global__ void __launch_bounds__(RN_WARPS * 32)
rope_norm_cache_kernel(const T* __restrict__ src, long long ld_src, int n, const float* __restrict__ cs, int rope_dim,
                       float norm_eps, const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                       HeadGroup qg, T* __restrict__ q_out, long long ld_q, HeadGroup kg, T* __restrict__ k_pool,
                       PagedCache kc, HeadGroup vg, T* __restrict__ v_pool, PagedCache vc) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_token = qg.count + kg.count + vg.count;
  const unsigned task = blockIdx.x * RN_WARPS + warp;          // the launcher keeps n * per_token below 2^31
  if (task >= (unsigned)n * (unsigned)per_token) return;
  const int i = (int)(task / (unsigned)per_token);
  int h = (int)(task - (unsigned)i * (unsigned)per_token);
  const T* row = src + (long long)i * ld_src;
  const float* csr = cs != nullptr ? cs + (long long)i * rope_dim : nullptr;
  HeadGroup g;
  T* dst;
  bool norm = norm_eps >= 0.f;
  if (h < qg.count) {
    g = qg;
    dst = q_out + (long long)i * ld_q + (long long)h * g.dst_stride + g.dst_off;
  } else if (h < qg.count + kg.count) {
    h -= qg.count;
    g = kg;
    dst = k_pool + paged_offset(kc, slot_of_token[i], positions[i], h) + g.dst_off;
  } else {
    h -= qg.count + kg.count;
    g = vg;
    dst = v_pool + paged_offset(vc, slot_of_token[i], positions[i], h) + g.dst_off;
    norm = false;
    csr = nullptr;
  }
  const T* x = row + g.src_off + (long long)h * g.src_stride;
  float v[PER_LANE];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int d = lane + 32 * j;
    v[j] = d < g.len ? rotated<T>(x, d, g.rope_off, rope_dim, csr) : 0.f;
    ss = fmaf(v[j], v[j], ss);
  }
  float scale = 1.f;
  if (norm) scale = 1.0f / sqrtf(warp_sum(ss) / (float)g.len + norm_eps);
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int d = lane + 32 * j;
    if (d < g.len) dst[d] = from_f32<T>(v[j] * scale);
  }
}

constexpr int LT_THREADS = 128;

__device__ __forceinline__ float block_sum_lt(float v, float* partial) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < LT_THREADS / 32; ++i) total += partial[i];
  return total;
}

template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
latent_norm_rope_cache_kernel(const T* __restrict__ proj, long long ld, int q_off, int q_rank, int kv_off, int kv_rank,
                              int rot_dim, const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                              const float* __restrict__ cs, const int* __restrict__ positions,
                              const int* __restrict__ slot_of_token, T* __restrict__ cq_out, long long ld_cq,
                              T* __restrict__ k_pool, PagedCache kc, int write_cache) {
  __shared__ float partial[LT_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x;
  const T* row = proj + (long long)i * ld;
  {
    const T* x = row + q_off;
    float ss = 0.f;
    for (int d = threadIdx.x; d < q_rank; d += LT_THREADS) { const float v = to_f32<T>(x[d]); ss = fmaf(v, v, ss); }
    const float scale = 1.0f / sqrtf(block_sum_lt(ss, partial) / (float)q_rank + eps);
    T* dst = cq_out + (long long)i * ld_cq;
    for (int d = threadIdx.x; d < q_rank; d += LT_THREADS) dst[d] = from_f32<T>(to_f32<T>(x[d]) * scale * wq[d]);
  }
  if (!write_cache) return;
  {
    const T* x = row + kv_off;
    float ss = 0.f;
    for (int d = threadIdx.x; d < kv_rank; d += LT_THREADS) { const float v = to_f32<T>(x[d]); ss = fmaf(v, v, ss); }
    const float scale = 1.0f / sqrtf(block_sum_lt(ss, partial) / (float)kv_rank + eps);
    T* dst = k_pool + paged_offset(kc, slot_of_token[i], positions[i], 0);
    for (int d = threadIdx.x; d < kv_rank; d += LT_THREADS) dst[d] = from_f32<T>(to_f32<T>(x[d]) * scale * wkv[d]);
    const float* csr = cs + (long long)i * rot_dim;
    for (int d = threadIdx.x; d < rot_dim; d += LT_THREADS)
      dst[kv_rank + d] = from_f32<T>(rotated<T>(x + kv_rank, d, 0, rot_dim, csr));
  }
}


constexpr int AP_THREADS = 128;

__device__ __forceinline__ float block_sum_ap(float v, float* partial) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < AP_THREADS / 32; ++i) total += partial[i];
  return total;
}

// element d of a head of `len` dimensions in shared memory after the rotation
__device__ __forceinline__ float rotated_s(const float* __restrict__ x, int d, int rope_dim, int interleaved,
                                           const float* __restrict__ cs) {
  const float v = x[d];
  if (cs == nullptr || d >= rope_dim) return v;
  if (interleaved) {
    const int i = d >> 1;
    return (d & 1) ? v * cs[2 * i] + x[d - 1] * cs[2 * i + 1] : v * cs[2 * i] - x[d + 1] * cs[2 * i + 1];
  }
  const int half = rope_dim >> 1;
  if (d < half) return v * cs[2 * d] - x[d + half] * cs[2 * d + 1];
  return v * cs[2 * (d - half)] + x[d - half] * cs[2 * (d - half) + 1];
}

template <typename T>
__global__ void __launch_bounds__(AP_THREADS)
attention_prepare_kernel(const T* __restrict__ src, long long ld_src, int q_off, int k_off, int v_off,
                         const float* __restrict__ bq, const float* __restrict__ bk, const float* __restrict__ bv,
                         const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                         const float* __restrict__ cs, int rope_dim, int interleaved,
                         const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                         T* __restrict__ q_out, long long ld_q, T* __restrict__ k_pool, PagedCache kc,
                         T* __restrict__ v_pool, PagedCache vc, int heads, int key_dim) {
  extern __shared__ float row_s[];            // [q_cols | k_cols | v_cols]
  __shared__ float partial[AP_THREADS / 32];
  const int i = blockIdx.x;
  const int pos = positions[i], slot = slot_of_token[i];
  pdl_wait();
  pdl_launch_dependents();
  const bool write = k_pool != nullptr;
  const int q_cols = heads * key_dim, k_cols = write ? kc.kv_heads * key_dim : 0, v_cols = write ? vc.kv_heads * vc.head_dim : 0;
  const T* row = src + (long long)i * ld_src;
  float* qs = row_s;
  float* ks = qs + q_cols;
  float* vs = ks + k_cols;
  float ssq = 0.f, ssk = 0.f;
  for (int c = threadIdx.x; c < q_cols; c += AP_THREADS) {
    const float v = to_f32<T>(row[q_off + c]) + (bq != nullptr ? bq[c] : 0.f);
    qs[c] = v;
    ssq = fmaf(v, v, ssq);
  }
  for (int c = threadIdx.x; c < k_cols; c += AP_THREADS) {
    const float v = to_f32<T>(row[k_off + c]) + (bk != nullptr ? bk[c] : 0.f);
    ks[c] = v;
    ssk = fmaf(v, v, ssk);
  }
  for (int c = threadIdx.x; c < v_cols; c += AP_THREADS) vs[c] = to_f32<T>(row[v_off + c]) + (bv != nullptr ? bv[c] : 0.f);
  if (wq != nullptr) {
    const float scale = 1.0f / sqrtf(block_sum_ap(ssq, partial) / (float)q_cols + eps);
    for (int c = threadIdx.x; c < q_cols; c += AP_THREADS) qs[c] = qs[c] * scale * wq[c];      // a thread's own columns
  }
  if (wk != nullptr && write) {
    const float scale = 1.0f / sqrtf(block_sum_ap(ssk, partial) / (float)k_cols + eps);
    for (int c = threadIdx.x; c < k_cols; c += AP_THREADS) ks[c] = ks[c] * scale * wk[c];
  }
  __syncthreads();
  const float* csr = cs != nullptr ? cs + (long long)i * rope_dim : nullptr;
  T* qrow = q_out + (long long)i * ld_q;
  for (int c = threadIdx.x; c < q_cols; c += AP_THREADS) {
    const int h = c / key_dim, d = c - h * key_dim;
    qrow[c] = from_f32<T>(rotated_s(qs + h * key_dim, d, rope_dim, interleaved, csr));
  }
  if (!write) return;
  for (int c = threadIdx.x; c < k_cols; c += AP_THREADS) {
    const int g = c / key_dim, d = c - g * key_dim;
    k_pool[paged_offset(kc, slot, pos, g) + d] = from_f32<T>(rotated_s(ks + g * key_dim, d, rope_dim, interleaved, csr));
  }
  const int vd = vc.head_dim;
  for (int c = threadIdx.x; c < v_cols; c += AP_THREADS) {
    const int g = c / vd, d = c - g * vd;
    v_pool[paged_offset(vc, slot, pos, g) + d] = from_f32<T>(vs[c]);
  }
}

template <typename T>
int launch_rope_norm(const void* src, long long ld_src, int n, const float* cs, int rope_dim, float norm_eps,
                     const int* positions, const int* slot_of_token, const HeadGroup& qg, void* q_out, long long ld_q,
                     const HeadGroup& kg, void* k_pool, const PagedCache& kc, const HeadGroup& vg, void* v_pool,
                     const PagedCache& vc, cudaStream_t stream) {
  const long long tasks = (long long)n * (qg.count + kg.count + vg.count);
  if (tasks == 0) return HFEE_OK;
  if (tasks >= (1ll << 31)) return hfee_fail(HFEE_ERR_ARG, "rope_norm_cache: %lld (token, head) pairs exceed one launch", tasks);
  const unsigned blocks = (unsigned)((tasks + RN_WARPS - 1) / RN_WARPS);
  int longest = 0;
  if (qg.count) longest = qg.len;
  if (kg.count && kg.len > longest) longest = kg.len;
  if (vg.count && vg.len > longest) longest = vg.len;
#define HFEE_RN(P)                                                                                                          \
  hfee_launch(rope_norm_cache_kernel<T, P>, dim3(blocks), dim3(RN_WARPS * 32), 0, stream, (const T*)src, ld_src, n, cs, rope_dim, \
              norm_eps, positions, slot_of_token, qg, (T*)q_out, ld_q, kg, (T*)k_pool, kc, vg, (T*)v_pool, vc)
  if (longest <= 32) HFEE_RN(1);
  else if (longest <= 64) HFEE_RN(2);
  else if (longest <= 128) HFEE_RN(4);
  else if (longest <= 256) HFEE_RN(8);
  else HFEE_RN(RN_PER_LANE);
#undef HFEE_RN
  return hfee_check_launch("rope_norm_cache");
}

}  // namespace

// q_out, k_pool and v_pool may each be null: that kind of head is then skipped.  norm_eps < 0: no norm.
// cs: [n, rope_dim / 2, 2] cosines and sines of the step's tokens, or null for no rotation.
HFEE_API int hfee_rope_norm_cache(const void* src, long long ld_src, int dtype, int n, const float* cs, int rope_dim,
                                  float norm_eps, const int* positions, const int* slot_of_token,
                                  int heads, int q_src_off, int q_src_stride, int q_len, int q_rope_off, void* q_out,
                                  long long ld_q, int q_dst_off, int q_dst_stride,
                                  int kv_heads, int k_src_off, int k_src_stride, int k_len, int k_rope_off, void* k_pool,
                                  int k_pool_dim, int k_dst_off,
                                  int v_src_off, int v_src_stride, int v_len, void* v_pool, int v_pool_dim,
                                  const int* block_table, int max_pages, int page_size, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(q_len <= RN_MAX_LEN && k_len <= RN_MAX_LEN && v_len <= RN_MAX_LEN, "rope_norm_cache: a head is longer than %d",
               RN_MAX_LEN);
  HFEE_REQUIRE(rope_dim >= 0 && rope_dim % 2 == 0, "rope_norm_cache: rope_dim %d must be even", rope_dim);
  HeadGroup qg{q_out != nullptr ? heads : 0, q_src_off, q_src_stride, q_len, q_rope_off, q_dst_off, q_dst_stride};
  HeadGroup kg{k_pool != nullptr ? kv_heads : 0, k_src_off, k_src_stride, k_len, k_rope_off, k_dst_off, 0};
  HeadGroup vg{v_pool != nullptr ? kv_heads : 0, v_src_off, v_src_stride, v_len, 0, 0, 0};
  if (cs != nullptr) {
    HFEE_REQUIRE(qg.count == 0 || (q_rope_off >= 0 && q_rope_off + rope_dim <= q_len), "rope_norm_cache: rotated query dimensions leave the head");
    HFEE_REQUIRE(kg.count == 0 || (k_rope_off >= 0 && k_rope_off + rope_dim <= k_len), "rope_norm_cache: rotated key dimensions leave the head");
  }
  PagedCache kc{}, vc{};
  if (kg.count) {
    HFEE_REQUIRE(k_dst_off + k_len <= k_pool_dim, "rope_norm_cache: key does not fit its cached vector");
    HFEE_REQUIRE(make_paged_cache(&kc, block_table, max_pages, page_size, kv_heads, k_pool_dim), "page_size %d must be a power of two", page_size);
  }
  if (vg.count) {
    HFEE_REQUIRE(v_len <= v_pool_dim, "rope_norm_cache: value does not fit its cached vector");
    HFEE_REQUIRE(make_paged_cache(&vc, block_table, max_pages, page_size, kv_heads, v_pool_dim), "page_size %d must be a power of two", page_size);
  }
  if (dtype == HFEE_F32)
    return launch_rope_norm<float>(src, ld_src, n, cs, rope_dim, norm_eps, positions, slot_of_token, qg, q_out, ld_q, kg, k_pool, kc, vg, v_pool, vc, stream);
  if (dtype == HFEE_BF16)
    return launch_rope_norm<__nv_bfloat16>(src, ld_src, n, cs, rope_dim, norm_eps, positions, slot_of_token, qg, q_out, ld_q, kg, k_pool, kc, vg, v_pool, vc, stream);
  return hfee_fail(HFEE_ERR_ARG, "rope_norm_cache: unknown dtype %d", dtype);
}

// src rows hold the query projection at q_off (heads * key_dim columns), the key projection at k_off (kv_heads *
// key_dim) and the value projection at v_off (kv_heads * value_dim).  bq, bk, bv: a bias per column (float32, each may
// be null); wq, wk: weights of an RMS norm over the whole query / key projection (null: no norm); cs: [n, rope_dim/2,
// 2] cosines and sines (null: no rotation); interleaved: pairs (2i, 2i+1) instead of (i, i + rope_dim/2).  k_pool null:
// queries only (a run that reads a cache another run filled).
HFEE_API int hfee_attention_prepare(const void* src, long long ld_src, int dtype, int n, int q_off, int k_off, int v_off,
                                    const float* bq, const float* bk, const float* bv, const float* wq, const float* wk,
                                    float eps, const float* cs, int rope_dim, int interleaved, const int* positions,
                                    const int* slot_of_token, void* q_out, long long ld_q, void* k_pool, void* v_pool,
                                    const int* block_table, int max_pages, int page_size, int heads, int kv_heads,
                                    int key_dim, int value_dim, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(heads > 0 && kv_heads > 0 && key_dim > 0 && value_dim > 0, "attention_prepare: bad sizes");
  HFEE_REQUIRE(rope_dim >= 0 && rope_dim % 2 == 0 && rope_dim <= key_dim,
               "attention_prepare: rope_dim %d must be even and at most the key size %d", rope_dim, key_dim);
  HFEE_REQUIRE((k_pool == nullptr) == (v_pool == nullptr), "attention_prepare: keys and values are cached together");
  HFEE_REQUIRE(ld_q >= (long long)heads * key_dim, "attention_prepare: ld_q is too small");
  PagedCache kc{}, vc{};
  HFEE_REQUIRE(make_paged_cache(&kc, block_table, max_pages, page_size, kv_heads, key_dim), "page_size %d must be a power of two", page_size);
  make_paged_cache(&vc, block_table, max_pages, page_size, kv_heads, value_dim);
  const size_t smem = sizeof(float) * ((size_t)heads * key_dim + (k_pool != nullptr ? (size_t)kv_heads * (key_dim + value_dim) : 0));
  HFEE_REQUIRE(smem <= 48 * 1024, "attention_prepare: a token's projections (%zu bytes as float32) exceed 48 KB", smem);
  if (cs == nullptr) rope_dim = 0;
  if (dtype == HFEE_F32)
    hfee_launch(attention_prepare_kernel<float>, dim3(n), dim3(AP_THREADS), smem, stream, (const float*)src, ld_src, q_off, k_off, v_off,
                bq, bk, bv, wq, wk, eps, cs, rope_dim, interleaved, positions, slot_of_token, (float*)q_out, ld_q, (float*)k_pool, kc,
                (float*)v_pool, vc, heads, key_dim);
  else if (dtype == HFEE_BF16)
    hfee_launch(attention_prepare_kernel<__nv_bfloat16>, dim3(n), dim3(AP_THREADS), smem, stream, (const __nv_bfloat16*)src, ld_src,
                q_off, k_off, v_off, bq, bk, bv, wq, wk, eps, cs, rope_dim, interleaved, positions, slot_of_token,
                (__nv_bfloat16*)q_out, ld_q, (__nv_bfloat16*)k_pool, kc, (__nv_bfloat16*)v_pool, vc, heads, key_dim);
  else
    return hfee_fail(HFEE_ERR_ARG, "attention_prepare: unknown dtype %d", dtype);
  return hfee_check_launch("attention_prepare");
}

// proj rows hold the query latent at q_off (q_rank columns) and [key/value latent | tail to rotate] at kv_off
// (kv_rank + rot_dim columns).  The cached vector of a token is [normed latent | rotated tail] (one "head").
HFEE_API int hfee_latent_norm_rope_cache(const void* proj, long long ld, int dtype, int n, int q_off, int q_rank, int kv_off,
                                         int kv_rank, int rot_dim, const float* wq, const float* wkv, float eps,
                                         const float* cs, const int* positions, const int* slot_of_token, void* cq_out,
                                         long long ld_cq, void* k_pool, const int* block_table, int max_pages,
                                         int page_size, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(q_rank > 0 && kv_rank > 0 && rot_dim > 0 && rot_dim % 2 == 0, "latent_norm_rope_cache: bad sizes");
  HFEE_REQUIRE(cs != nullptr || k_pool == nullptr, "latent_norm_rope_cache: the rotated tail needs its table");
  PagedCache kc{};
  if (k_pool != nullptr)
    HFEE_REQUIRE(make_paged_cache(&kc, block_table, max_pages, page_size, 1, kv_rank + rot_dim), "page_size %d must be a power of two", page_size);
  if (dtype == HFEE_F32)
    hfee_launch(latent_norm_rope_cache_kernel<float>, dim3(n), dim3(LT_THREADS), 0, stream, (const float*)proj, ld, q_off, q_rank,
                kv_off, kv_rank, rot_dim, wq, wkv, eps, cs, positions, slot_of_token, (float*)cq_out, ld_cq, (float*)k_pool, kc,
                k_pool != nullptr ? 1 : 0);
  else if (dtype == HFEE_BF16)
    hfee_launch(latent_norm_rope_cache_kernel<__nv_bfloat16>, dim3(n), dim3(LT_THREADS), 0, stream, (const __nv_bfloat16*)proj, ld,
                q_off, q_rank, kv_off, kv_rank, rot_dim, wq, wkv, eps, cs, positions, slot_of_token, (__nv_bfloat16*)cq_out, ld_cq,
                (__nv_bfloat16*)k_pool, kc, k_pool != nullptr ? 1 : 0);
  else
    return hfee_fail(HFEE_ERR_ARG, "latent_norm_rope_cache: unknown dtype %d", dtype);
  return hfee_check_launch("latent_norm_rope_cache");
}
