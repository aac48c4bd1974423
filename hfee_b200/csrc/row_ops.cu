// Row kernels on the float32 residual stream: a hashed bigram embedding, layer norm, and a bias per column.
//
//   hfee_embed_bigram     out[i,:] = table[token_i,:] + pairs[row_i,:] (float32), row_i = (previous token * mul_prev +
//                         token_i * mul_cur) mod buckets, and row `buckets` for a request's first token.  The previous
//                         token of a portion's first token is the request's last token of an earlier step, kept per
//                         request slot in `last_token`.
//   hfee_remember_tokens  last_token[slot of request r] = the last token request r brought in this step.
//   hfee_layernorm        out[r,:] = (x[row(r),:] - mean) / sqrt(var + eps) * w, var = mean of squared deviations;
//                         one block per row, the row kept in registers between the passes where it fits;
//                         `residual_add` (optional, float32 [n, width], not with `rows`) is added to x first and the
//                         sum stored back to x: a sublayer's residual update and the next norm in one pass.
//   hfee_add_bias         x[r, c] += bias[c].
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

template <int THREADS>
__device__ __forceinline__ float block_total(float v, float* partial) {
  v = warp_sum(v);
  __syncthreads();                       // partial may still be read from an earlier call
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += partial[i];       // fixed order
  return total;
}

__device__ __forceinline__ int token_at(const int* __restrict__ tokens, const int* __restrict__ slot_of_token,
                                        const int* __restrict__ feedback, int i) {
  int tok = tokens[i];
  if (tok < 0 && feedback != nullptr) tok = feedback[slot_of_token[i]];
  return tok;
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
embed_bigram_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int* __restrict__ tokens,
                    const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                    const int* __restrict__ feedback, const int* __restrict__ last_token, float* __restrict__ out,
                    int width, int vocab, int buckets, long long mul_prev, long long mul_cur) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x;
  const int tok = token_at(tokens, slot_of_token, feedback, i);
  const int slot = slot_of_token[i];
  int row = buckets;
  if (positions[i] > 0) {
    // the token in front: the one before it in this step if that belongs to the same request, else what the
    // request's earlier step left
    const int prev = (i > 0 && slot_of_token[i - 1] == slot) ? token_at(tokens, slot_of_token, feedback, i - 1) : last_token[slot];
    row = (int)(((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets);
    if (row < 0) row += buckets;
  }
  const bool ok = tok >= 0 && tok < vocab;
  const T* a = table + (long long)(ok ? tok : 0) * width;
  const T* b = pairs + (long long)row * width;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS)
    out[(long long)i * width + c] = ok ? to_f32<T>(a[c]) + to_f32<T>(b[c]) : 0.f;
}

__global__ void remember_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ slot_of_token,
                                       const int* __restrict__ feedback, const int* __restrict__ cu_tokens,
                                       const int* __restrict__ slots, int requests, int* __restrict__ last_token) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= requests) return;
  const int end = cu_tokens[r + 1];
  if (end > cu_tokens[r]) last_token[slots[r]] = token_at(tokens, slot_of_token, feedback, end - 1);
}

// PER: values of the row per thread that stay in registers (rows up to ROW_THREADS * PER wide); wider rows are read
// three times.
template <typename TOut, int PER>
__global__ void __launch_bounds__(ROW_THREADS)
layernorm_kernel(float* __restrict__ x, const float* __restrict__ residual_add, const float* __restrict__ w,
                 const int* __restrict__ rows, TOut* __restrict__ out, long long ld_o, int width, float eps) {
  __shared__ float partial[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  float* xr = x + (long long)(rows ? rows[r] : r) * width;
  const float* ar = residual_add != nullptr ? residual_add + (long long)r * width : nullptr;
  TOut* orow = out + (long long)r * ld_o;
  const bool fits = width <= ROW_THREADS * PER;
  float v[PER];
  float sum = 0.f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = threadIdx.x + j * ROW_THREADS;
      v[j] = 0.f;
      if (c < width) {
        v[j] = xr[c];
        if (ar != nullptr) { v[j] += ar[c]; xr[c] = v[j]; }
      }
      sum += v[j];
    }
  } else {
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
      float t = xr[c];
      if (ar != nullptr) { t += ar[c]; xr[c] = t; }
      sum += t;
    }
  }
  const float mean = block_total<ROW_THREADS>(sum, partial) / (float)width;
  float ss = 0.f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = threadIdx.x + j * ROW_THREADS;
      const float d = c < width ? v[j] - mean : 0.f;
      ss = fmaf(d, d, ss);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) { const float d = xr[c] - mean; ss = fmaf(d, d, ss); }
  }
  const float scale = 1.0f / sqrtf(block_total<ROW_THREADS>(ss, partial) / (float)width + eps);
  if (fits) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = threadIdx.x + j * ROW_THREADS;
      if (c < width) orow[c] = from_f32<TOut>((v[j] - mean) * scale * w[c]);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) orow[c] = from_f32<TOut>((xr[c] - mean) * scale * w[c]);
  }
}

// The same for widths that are multiples of 4 with 16-byte accesses: a thread owns the pieces tid, tid + ROW_THREADS, ...,
// NCH of them (rows of at most ROW_THREADS * 4 * NCH values), all requested before the first is used and kept in
// registers between the passes.
template <typename TOut, int NCH>
__global__ void __launch_bounds__(ROW_THREADS)
layernorm_vec_kernel(float* __restrict__ x, const float* __restrict__ residual_add, const float* __restrict__ w,
                     const int* __restrict__ rows, TOut* __restrict__ out, long long ld_o, int width, float eps) {
  __shared__ float partial[ROW_THREADS / 32];
  const int r = blockIdx.x, tid = threadIdx.x;
  float4 wv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (tid + j * ROW_THREADS) * 4;
    wv[j] = c < width ? __ldg(reinterpret_cast<const float4*>(w + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int src_row = rows ? rows[r] : r;
  pdl_wait();
  pdl_launch_dependents();
  float* xr = x + (long long)src_row * width;
  const float* ar = residual_add != nullptr ? residual_add + (long long)r * width : nullptr;
  float4 v[NCH];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (tid + j * ROW_THREADS) * 4;
    v[j] = c < width ? *reinterpret_cast<const float4*>(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (ar != nullptr) {
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = (tid + j * ROW_THREADS) * 4;
      if (c < width) {
        const float4 a = *reinterpret_cast<const float4*>(ar + c);
        v[j].x += a.x; v[j].y += a.y; v[j].z += a.z; v[j].w += a.w;
        *reinterpret_cast<float4*>(xr + c) = v[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  const float mean = block_total<ROW_THREADS>(sum, partial) / (float)width;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (tid + j * ROW_THREADS) * 4;
    if (c < width) {
      const float a = v[j].x - mean, b = v[j].y - mean, cc = v[j].z - mean, d = v[j].w - mean;
      ss = fmaf(a, a, ss); ss = fmaf(b, b, ss); ss = fmaf(cc, cc, ss); ss = fmaf(d, d, ss);
    }
  }
  const float scale = 1.0f / sqrtf(block_total<ROW_THREADS>(ss, partial) / (float)width + eps);
  TOut* orow = out + (long long)r * ld_o;
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (tid + j * ROW_THREADS) * 4;
    if (c >= width) continue;
    const float o0 = (v[j].x - mean) * scale * wv[j].x, o1 = (v[j].y - mean) * scale * wv[j].y;
    const float o2 = (v[j].z - mean) * scale * wv[j].z, o3 = (v[j].w - mean) * scale * wv[j].w;
    if constexpr (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(orow) + c) = make_float4(o0, o1, o2, o3);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(orow) + c) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

__global__ void add_bias_vec_kernel(float4* __restrict__ x, long long ld4, const float4* __restrict__ bias, int cols4, long long total4) {
  pdl_wait();
  pdl_launch_dependents();
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total4) return;
  const long long r = e / cols4;
  const int c = (int)(e - r * cols4);
  float4 v = x[r * ld4 + c];
  const float4 b = __ldg(bias + c);
  v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  x[r * ld4 + c] = v;
}

__global__ void add_bias_kernel(float* __restrict__ x, long long ld, const float* __restrict__ bias, int cols, long long total) {
  pdl_wait();
  pdl_launch_dependents();
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long r = e / cols;
  const int c = (int)(e - r * cols);
  x[r * ld + c] += bias[c];
}

template <typename TOut>
void launch_layernorm(float* x, const float* residual_add, const float* w, const int* rows, void* out, long long ld_o, int n,
                      int width, float eps, cudaStream_t stream) {
  const bool vec = width % 4 == 0 && ld_o % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                   (residual_add == nullptr || (uintptr_t)residual_add % 16 == 0);
  if (vec && width <= ROW_THREADS * 4 * 2)
    hfee_launch(layernorm_vec_kernel<TOut, 2>, dim3(n), dim3(ROW_THREADS), 0, stream, x, residual_add, w, rows, (TOut*)out, ld_o, width, eps);
  else if (vec && width <= ROW_THREADS * 4 * 8)
    hfee_launch(layernorm_vec_kernel<TOut, 8>, dim3(n), dim3(ROW_THREADS), 0, stream, x, residual_add, w, rows, (TOut*)out, ld_o, width, eps);
  else if (width <= ROW_THREADS * 4)
    hfee_launch(layernorm_kernel<TOut, 4>, dim3(n), dim3(ROW_THREADS), 0, stream, x, residual_add, w, rows, (TOut*)out, ld_o, width, eps);
  else
    hfee_launch(layernorm_kernel<TOut, 16>, dim3(n), dim3(ROW_THREADS), 0, stream, x, residual_add, w, rows, (TOut*)out, ld_o, width, eps);
}

}  // namespace

HFEE_API int hfee_embed_bigram(const void* table, const void* pairs, int dtype, const int* tokens, const int* positions,
                               const int* slot_of_token, const int* feedback, const int* last_token, float* out, int n,
                               int width, int vocab, int buckets, long long mul_prev, long long mul_cur,
                               cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && vocab > 0 && buckets > 0, "embed_bigram: bad sizes");
  HFEE_REQUIRE(mul_prev >= 0 && mul_cur >= 0 && mul_prev < (1ll << 31) && mul_cur < (1ll << 31), "embed_bigram: multipliers outside 0..2^31");
  if (dtype == HFEE_F32)
    hfee_launch(embed_bigram_kernel<float>, dim3(n), dim3(ROW_THREADS), 0, stream, (const float*)table, (const float*)pairs, tokens,
                positions, slot_of_token, feedback, last_token, out, width, vocab, buckets, mul_prev, mul_cur);
  else if (dtype == HFEE_BF16)
    hfee_launch(embed_bigram_kernel<__nv_bfloat16>, dim3(n), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)table,
                (const __nv_bfloat16*)pairs, tokens, positions, slot_of_token, feedback, last_token, out, width, vocab, buckets,
                mul_prev, mul_cur);
  else
    return hfee_fail(HFEE_ERR_ARG, "embed_bigram: unknown dtype %d", dtype);
  return hfee_check_launch("embed_bigram");
}

HFEE_API int hfee_remember_tokens(const int* tokens, const int* slot_of_token, const int* feedback, const int* cu_tokens,
                                  const int* slots, int requests, int* last_token, cudaStream_t stream) {
  if (requests == 0) return HFEE_OK;
  hfee_launch(remember_tokens_kernel, dim3((requests + 63) / 64), dim3(64), 0, stream, tokens, slot_of_token, feedback, cu_tokens,
              slots, requests, last_token);
  return hfee_check_launch("remember_tokens");
}

HFEE_API int hfee_layernorm(float* x, const float* residual_add, const float* w, const int* rows, void* out, long long ld_o,
                            int dtype, int n, int width, float eps, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && ld_o >= width, "layernorm: bad sizes");
  HFEE_REQUIRE(residual_add == nullptr || rows == nullptr, "layernorm: a residual update does not go with gathered rows");
  if (dtype == HFEE_F32) launch_layernorm<float>(x, residual_add, w, rows, out, ld_o, n, width, eps, stream);
  else if (dtype == HFEE_BF16) launch_layernorm<__nv_bfloat16>(x, residual_add, w, rows, out, ld_o, n, width, eps, stream);
  else return hfee_fail(HFEE_ERR_ARG, "layernorm: unknown dtype %d", dtype);
  return hfee_check_launch("layernorm");
}

HFEE_API int hfee_add_bias(float* x, long long ld, const float* bias, int rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return HFEE_OK;
  HFEE_REQUIRE(rows > 0 && cols > 0 && ld >= cols, "add_bias: bad sizes");
  const long long total = (long long)rows * cols;
  if (cols % 4 == 0 && ld % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)bias % 16 == 0) {
    hfee_launch(add_bias_vec_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (float4*)x, ld / 4, (const float4*)bias,
                cols / 4, total / 4);
    return hfee_check_launch("add_bias");
  }
  hfee_launch(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, ld, bias, cols, total);
  return hfee_check_launch("add_bias");
}
