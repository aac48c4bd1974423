// Row-wise pieces of layers that gate or norm a sublayer's output, all in float32 arithmetic:
//
//   hfee_rmsnorm_add      residual += y / sqrt(mean(y^2) + eps) * w          (a norm on a sublayer's output)
//   hfee_norm_gate        out = [x / sqrt(mean(x^2) + eps) * w] * sigmoid(g)  (the norm is optional)
//   hfee_gated_act        out = act(gate) * up, act = SiLU or tanh-GELU
//   hfee_scale_f32        x *= alpha
//   hfee_cast_rows        out = x rounded to the activations' type (what a matrix product reads of the residual stream)
//   hfee_qk_norm_rope_cache   RMS norm over a token's whole query (and key) projection, rotary on the
//                         leading dimensions of every head, keys into their cache page, and the
//                         values' page filled with the keys as projected (v_offset < 0) or with the
//                         columns of the row that start at v_offset
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* partial) {
  v = warp_sum(v);
  __syncthreads();                                   // partial may still be read from a call before
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < ROW_THREADS / 32; ++i) total += partial[i];
  return total;
}

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.f / (1.f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_add_kernel(const float* __restrict__ y, long long ld_y, const float* __restrict__ w,
                   float* __restrict__ residual, int width, float eps, int add_unit, T* __restrict__ cast_out,
                   long long ld_c) {
  __shared__ float partial[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const float* yr = y + (long long)blockIdx.x * ld_y;
  float* rr = residual + (long long)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) ss = fmaf(yr[c], yr[c], ss);
  const float scale = 1.0f / sqrtf(block_sum(ss, partial) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
    const float r = rr[c] + yr[c] * scale * (add_unit ? 1.f + w[c] : w[c]);
    rr[c] = r;
    if (cast_out != nullptr) cast_out[(long long)blockIdx.x * ld_c + c] = from_f32<T>(r);
  }
}

// The same for widths that are multiples of 4 and at most ROW_THREADS * 4 * NCH: 16-byte accesses, the row of y
// and of the residual requested at once and kept in registers between the two passes.
template <typename T, int NCH>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_add_vec_kernel(const float* __restrict__ y, long long ld_y, const float* __restrict__ w,
                       float* __restrict__ residual, int width, float eps, int add_unit, T* __restrict__ cast_out,
                       long long ld_c) {
  __shared__ float partial[ROW_THREADS / 32];
  float4 wv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * ROW_THREADS) * 4;
    wv[j] = c < width ? __ldg(reinterpret_cast<const float4*>(w + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  pdl_launch_dependents();
  const float* yr = y + (long long)blockIdx.x * ld_y;
  float* rr = residual + (long long)blockIdx.x * width;
  float4 yv[NCH], rv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * ROW_THREADS) * 4;
    yv[j] = c < width ? *reinterpret_cast<const float4*>(yr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    rv[j] = c < width ? *reinterpret_cast<const float4*>(rr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NCH; ++j) ss = fmaf(yv[j].x, yv[j].x, fmaf(yv[j].y, yv[j].y, fmaf(yv[j].z, yv[j].z, fmaf(yv[j].w, yv[j].w, ss))));
  const float scale = 1.0f / sqrtf(block_sum(ss, partial) / (float)width + eps);
  const float unit = add_unit ? 1.f : 0.f;
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * ROW_THREADS) * 4;
    if (c >= width) continue;
    float4 r = rv[j];
    r.x += yv[j].x * scale * (wv[j].x + unit);
    r.y += yv[j].y * scale * (wv[j].y + unit);
    r.z += yv[j].z * scale * (wv[j].z + unit);
    r.w += yv[j].w * scale * (wv[j].w + unit);
    *reinterpret_cast<float4*>(rr + c) = r;
    if (cast_out != nullptr) {
      T* dst = cast_out + (long long)blockIdx.x * ld_c + c;
      dst[0] = from_f32<T>(r.x); dst[1] = from_f32<T>(r.y); dst[2] = from_f32<T>(r.z); dst[3] = from_f32<T>(r.w);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
norm_gate_kernel(const float* __restrict__ x, long long ld_x, const float* __restrict__ w, float eps,
                 const T* __restrict__ gate, long long ld_g, T* __restrict__ out, long long ld_o, int width) {
  __shared__ float partial[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const float* xr = x + (long long)blockIdx.x * ld_x;
  const T* gr = gate + (long long)blockIdx.x * ld_g;
  T* orow = out + (long long)blockIdx.x * ld_o;
  float scale = 1.f;
  if (w != nullptr) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += ROW_THREADS) ss = fmaf(xr[c], xr[c], ss);
    scale = 1.0f / sqrtf(block_sum(ss, partial) / (float)width + eps);
  }
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
    const float v = w != nullptr ? xr[c] * scale * w[c] : xr[c];
    orow[c] = from_f32<T>(v * sigmoid_f32(to_f32<T>(gr[c])));
  }
}

// four consecutive activations at once (rows that 8- or 16-byte accesses can read)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// norm_gate for widths that are multiples of 4 and at most ROW_THREADS * 4 * NCH, the row kept in registers
template <typename T, int NCH>
__global__ void __launch_bounds__(ROW_THREADS)
norm_gate_vec_kernel(const float* __restrict__ x, long long ld_x, const float* __restrict__ w, float eps,
                     const T* __restrict__ gate, long long ld_g, T* __restrict__ out, long long ld_o, int width) {
  __shared__ float partial[ROW_THREADS / 32];
  float4 wv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * ROW_THREADS) * 4;
    wv[j] = (w != nullptr && c < width) ? __ldg(reinterpret_cast<const float4*>(w + c)) : make_float4(1.f, 1.f, 1.f, 1.f);
  }
  pdl_wait();
  pdl_launch_dependents();
  const float* xr = x + (long long)blockIdx.x * ld_x;
  const T* gr = gate + (long long)blockIdx.x * ld_g;
  T* orow = out + (long long)blockIdx.x * ld_o;
  float4 xv[NCH], gv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * ROW_THREADS) * 4;
    xv[j] = c < width ? load4(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    gv[j] = c < width ? load4(gr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float scale = 1.f;
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) ss = fmaf(xv[j].x, xv[j].x, fmaf(xv[j].y, xv[j].y, fmaf(xv[j].z, xv[j].z, fmaf(xv[j].w, xv[j].w, ss))));
    scale = 1.0f / sqrtf(block_sum(ss, partial) / (float)width + eps);
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * ROW_THREADS) * 4;
    if (c >= width) continue;
    float4 o;
    o.x = xv[j].x * scale * wv[j].x * sigmoid_f32(gv[j].x);
    o.y = xv[j].y * scale * wv[j].y * sigmoid_f32(gv[j].y);
    o.z = xv[j].z * scale * wv[j].z * sigmoid_f32(gv[j].z);
    o.w = xv[j].w * scale * wv[j].w * sigmoid_f32(gv[j].w);
    store4(orow + c, o);
  }
}

enum GateActivation { GA_SILU = 0, GA_GELU_TANH = 1 };

__device__ __forceinline__ float gate_activation(float z, int act) {
  if (act == GA_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, long long ld_gu, T* __restrict__ h, long long ld_h, int n,
                                 int inter, int granule, int act) {
  pdl_wait();
  pdl_launch_dependents();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * inter) return;
  int i = (int)(idx / inter), c = (int)(idx % inter);
  long long gcol = (long long)(c / granule) * 2 * granule + c % granule;
  float g = to_f32<T>(gu[(long long)i * ld_gu + gcol]);
  float u = to_f32<T>(gu[(long long)i * ld_gu + gcol + granule]);
  h[(long long)i * ld_h + c] = from_f32<T>(gate_activation(g, act) * u);
}

__global__ void scale_kernel(float* __restrict__ x, long long ld, int cols, long long total, float alpha) {
  pdl_wait();
  pdl_launch_dependents();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  x[(idx / cols) * ld + idx % cols] *= alpha;
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long ld_o, int cols, long long total) {
  pdl_wait();
  pdl_launch_dependents();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  out[(idx / cols) * ld_o + idx % cols] = from_f32<T>(x[idx]);
}

// One block per token.  qk row: [heads * hd query values | kv_heads * hd key values].
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
qk_norm_rope_cache_kernel(const T* __restrict__ qk, long long ld_qk, const float* __restrict__ wq,
                          const float* __restrict__ wk, float eps, const float2* __restrict__ cs, int rope_dim,
                          const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                          T* __restrict__ q_out, long long ld_q, T* __restrict__ k_pool, T* __restrict__ v_pool,
                          PagedCache cache, int heads, int v_offset) {
  __shared__ float partial[ROW_THREADS / 32];
  const int i = blockIdx.x;
  const int pos = positions[i], slot = slot_of_token[i];
  pdl_wait();
  pdl_launch_dependents();
  const int hd = cache.head_dim, half = rope_dim / 2;
  const int q_cols = heads * hd, k_cols = cache.kv_heads * hd;
  const T* row = qk + (long long)i * ld_qk;
  const float2* csr = cs != nullptr ? cs + (long long)i * half : nullptr;

  // a warp takes whole heads (no division per element; the key's page is looked up once per head)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int WARPS = ROW_THREADS / 32;
  float ss = 0.f;
  for (int c = threadIdx.x; c < q_cols; c += ROW_THREADS) { const float v = to_f32<T>(row[c]); ss = fmaf(v, v, ss); }
  const float q_scale = wq != nullptr ? 1.0f / sqrtf(block_sum(ss, partial) / (float)q_cols + eps) : 1.f;
  for (int h = warp; h < heads; h += WARPS) {
    const T* in = row + (long long)h * hd;
    const float* wh = wq != nullptr ? wq + (long long)h * hd : nullptr;
    T* dst = q_out + (long long)i * ld_q + (long long)h * hd;
    for (int d = lane; d < hd; d += 32) {
      float val = to_f32<T>(in[d]) * q_scale * (wh != nullptr ? wh[d] : 1.f);
      if (csr != nullptr && d < rope_dim) {
        const int p = d < half ? d + half : d - half;               // the dimension this one is paired with
        const float other = to_f32<T>(in[p]) * q_scale * (wh != nullptr ? wh[p] : 1.f);
        const float2 t = csr[d < half ? d : d - half];              // (cos, sin) of the pair's angle
        val = d < half ? val * t.x - other * t.y : val * t.x + other * t.y;
      }
      dst[d] = from_f32<T>(val);
    }
  }
  if (k_pool == nullptr) return;
  const T* krow = row + q_cols;
  ss = 0.f;
  for (int c = threadIdx.x; c < k_cols; c += ROW_THREADS) { const float v = to_f32<T>(krow[c]); ss = fmaf(v, v, ss); }
  const float k_scale = wk != nullptr ? 1.0f / sqrtf(block_sum(ss, partial) / (float)k_cols + eps) : 1.f;
  for (int g = warp; g < cache.kv_heads; g += WARPS) {
    const T* in = krow + (long long)g * hd;
    const float* wh = wk != nullptr ? wk + (long long)g * hd : nullptr;
    const long long at = paged_offset(cache, slot, pos, g);
    for (int d = lane; d < hd; d += 32) {
      const T raw = in[d];
      float val = to_f32<T>(raw) * k_scale * (wh != nullptr ? wh[d] : 1.f);
      if (csr != nullptr && d < rope_dim) {
        const int p = d < half ? d + half : d - half;
        const float other = to_f32<T>(in[p]) * k_scale * (wh != nullptr ? wh[p] : 1.f);
        const float2 t = csr[d < half ? d : d - half];
        val = d < half ? val * t.x - other * t.y : val * t.x + other * t.y;
      }
      k_pool[at + d] = from_f32<T>(val);
      if (v_pool != nullptr) v_pool[at + d] = v_offset >= 0 ? row[v_offset + (long long)g * hd + d] : raw;
    }
  }
}

}  // namespace

namespace {
template <typename T>
void launch_rmsnorm_add(const float* y, long long ld_y, const float* w, float* residual, int n, int width, float eps,
                        int add_unit, void* cast_out, long long ld_c, cudaStream_t stream) {
  const bool vec = width % 4 == 0 && ld_y % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)residual % 16 == 0 &&
                   (uintptr_t)w % 16 == 0;
  if (vec && width <= ROW_THREADS * 4 * 2)
    hfee_launch(rmsnorm_add_vec_kernel<T, 2>, dim3(n), dim3(ROW_THREADS), 0, stream, y, ld_y, w, residual, width, eps, add_unit, (T*)cast_out, ld_c);
  else if (vec && width <= ROW_THREADS * 4 * 8)
    hfee_launch(rmsnorm_add_vec_kernel<T, 8>, dim3(n), dim3(ROW_THREADS), 0, stream, y, ld_y, w, residual, width, eps, add_unit, (T*)cast_out, ld_c);
  else
    hfee_launch(rmsnorm_add_kernel<T>, dim3(n), dim3(ROW_THREADS), 0, stream, y, ld_y, w, residual, width, eps, add_unit, (T*)cast_out, ld_c);
}
}  // namespace

namespace {
// residual += y / sqrt(mean(y^2) + eps) * w, then out = residual / sqrt(mean(residual^2) + eps2) * w2: the norm on a
// sublayer's output and the norm in front of the next sublayer in one pass over the row (kept in shared memory).
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_add_norm_kernel(const float* __restrict__ y, long long ld_y, const float* __restrict__ w, float* __restrict__ residual,
                        int width, float eps, int add_unit, const float* __restrict__ w2, float eps2, int add_unit2,
                        T* __restrict__ out, long long ld_o) {
  extern __shared__ float row_s[];
  __shared__ float partial[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const float* yr = y + (long long)blockIdx.x * ld_y;
  float* rr = residual + (long long)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
    const float v = yr[c];
    row_s[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float scale = 1.0f / sqrtf(block_sum(ss, partial) / (float)width + eps);
  float ss2 = 0.f;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
    const float r = rr[c] + row_s[c] * scale * (add_unit ? 1.f + w[c] : w[c]);
    rr[c] = r;
    row_s[c] = r;
    ss2 = fmaf(r, r, ss2);
  }
  const float scale2 = 1.0f / sqrtf(block_sum(ss2, partial) / (float)width + eps2);
  T* orow = out + (long long)blockIdx.x * ld_o;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS)
    orow[c] = from_f32<T>(row_s[c] * scale2 * (add_unit2 ? 1.f + w2[c] : w2[c]));
}
}  // namespace

HFEE_API int hfee_rmsnorm_add_norm(const float* y, long long ld_y, const float* w, float* residual, int n, int width,
                                   float eps, int add_unit, const float* w2, float eps2, int add_unit2, void* out,
                                   long long ld_o, int out_dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && ld_y >= width && ld_o >= width, "rmsnorm_add_norm: bad sizes");
  HFEE_REQUIRE((size_t)width * sizeof(float) <= 48 * 1024, "rmsnorm_add_norm: width %d does not fit shared memory", width);
  const size_t smem = (size_t)width * sizeof(float);
  if (out_dtype == HFEE_BF16)
    hfee_launch(rmsnorm_add_norm_kernel<__nv_bfloat16>, dim3(n), dim3(ROW_THREADS), smem, stream, y, ld_y, w, residual, width, eps,
                add_unit, w2, eps2, add_unit2, (__nv_bfloat16*)out, ld_o);
  else if (out_dtype == HFEE_F32)
    hfee_launch(rmsnorm_add_norm_kernel<float>, dim3(n), dim3(ROW_THREADS), smem, stream, y, ld_y, w, residual, width, eps, add_unit,
                w2, eps2, add_unit2, (float*)out, ld_o);
  else
    return hfee_fail(HFEE_ERR_ARG, "rmsnorm_add_norm: unknown dtype %d", out_dtype);
  return hfee_check_launch("rmsnorm_add_norm");
}

// residual += norm(y); with cast_out the new residual row is also written there in the activations' type
HFEE_API int hfee_rmsnorm_add(const float* y, long long ld_y, const float* w, float* residual, int n, int width,
                              float eps, int add_unit, void* cast_out, long long ld_c, int cast_dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && ld_y >= width, "rmsnorm_add: bad sizes");
  HFEE_REQUIRE(cast_out == nullptr || ld_c >= width, "rmsnorm_add: ld_c=%lld is too small", ld_c);
  if (cast_out != nullptr && cast_dtype == HFEE_BF16)
    launch_rmsnorm_add<__nv_bfloat16>(y, ld_y, w, residual, n, width, eps, add_unit, cast_out, ld_c, stream);
  else if (cast_out == nullptr || cast_dtype == HFEE_F32)
    launch_rmsnorm_add<float>(y, ld_y, w, residual, n, width, eps, add_unit, cast_out, ld_c, stream);
  else
    return hfee_fail(HFEE_ERR_ARG, "rmsnorm_add: unknown dtype %d", cast_dtype);
  return hfee_check_launch("rmsnorm_add");
}

HFEE_API int hfee_norm_gate(const float* x, long long ld_x, const float* w, float eps, const void* gate, long long ld_g,
                            void* out, long long ld_o, int n, int width, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && ld_x >= width && ld_g >= width && ld_o >= width, "norm_gate: bad sizes");
  const size_t elem = dtype == HFEE_F32 ? 4 : 2;
  const bool vec = width % 4 == 0 && ld_x % 4 == 0 && ld_g % 4 == 0 && ld_o % 4 == 0 && (uintptr_t)x % 16 == 0 &&
                   (w == nullptr || (uintptr_t)w % 16 == 0) && (uintptr_t)gate % (4 * elem) == 0 &&
                   (uintptr_t)out % (4 * elem) == 0 && width <= ROW_THREADS * 4 * 8;
#define HFEE_NG(T)                                                                                                        \
  do {                                                                                                                    \
    if (vec && width <= ROW_THREADS * 4 * 2)                                                                              \
      hfee_launch(norm_gate_vec_kernel<T, 2>, dim3(n), dim3(ROW_THREADS), 0, stream, x, ld_x, w, eps, (const T*)gate, ld_g, (T*)out, ld_o, width); \
    else if (vec)                                                                                                         \
      hfee_launch(norm_gate_vec_kernel<T, 8>, dim3(n), dim3(ROW_THREADS), 0, stream, x, ld_x, w, eps, (const T*)gate, ld_g, (T*)out, ld_o, width); \
    else                                                                                                                  \
      hfee_launch(norm_gate_kernel<T>, dim3(n), dim3(ROW_THREADS), 0, stream, x, ld_x, w, eps, (const T*)gate, ld_g, (T*)out, ld_o, width);        \
  } while (0)
  if (dtype == HFEE_F32) HFEE_NG(float);
  else if (dtype == HFEE_BF16) HFEE_NG(__nv_bfloat16);
  else return hfee_fail(HFEE_ERR_ARG, "norm_gate: unknown dtype %d", dtype);
#undef HFEE_NG
  return hfee_check_launch("norm_gate");
}

HFEE_API int hfee_gated_act(const void* gu, long long ld_gu, void* h, long long ld_h, int n, int inter, int granule,
                            int act, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && inter > 0 && ld_gu >= 2 * inter && ld_h >= inter, "gated_act: bad sizes");
  HFEE_REQUIRE(granule > 0 && inter % granule == 0, "gated_act: granule %d does not divide %d", granule, inter);
  HFEE_REQUIRE(act == GA_SILU || act == GA_GELU_TANH, "gated_act: unknown activation %d", act);
  long long total = (long long)n * inter;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == HFEE_F32)
    hfee_launch(gated_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, ld_gu, (float*)h, ld_h, n, inter, granule, act);
  else if (dtype == HFEE_BF16)
    hfee_launch(gated_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, ld_gu, (__nv_bfloat16*)h, ld_h, n, inter, granule, act);
  else
    return hfee_fail(HFEE_ERR_ARG, "gated_act: unknown dtype %d", dtype);
  return hfee_check_launch("gated_act");
}

HFEE_API int hfee_scale_f32(float* x, long long ld, int rows, int cols, float alpha, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return HFEE_OK;
  HFEE_REQUIRE(rows > 0 && cols > 0 && ld >= cols, "scale: bad sizes");
  long long total = (long long)rows * cols;
  hfee_launch(scale_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, ld, cols, total, alpha);
  return hfee_check_launch("scale");
}

HFEE_API int hfee_cast_rows(const float* x, void* out, long long ld_o, int rows, int cols, int dtype, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return HFEE_OK;
  HFEE_REQUIRE(rows > 0 && cols > 0 && ld_o >= cols, "cast_rows: bad sizes");
  long long total = (long long)rows * cols;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == HFEE_F32)
    hfee_launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (float*)out, ld_o, cols, total);
  else if (dtype == HFEE_BF16)
    hfee_launch(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, ld_o, cols, total);
  else
    return hfee_fail(HFEE_ERR_ARG, "cast_rows: unknown dtype %d", dtype);
  return hfee_check_launch("cast_rows");
}

HFEE_API int hfee_qk_norm_rope_cache(const void* qk, long long ld_qk, const float* wq, const float* wk, float eps,
                                     const float* cs, int rope_dim, const int* positions, const int* slot_of_token,
                                     void* q_out, long long ld_q, void* k_pool, void* v_pool, const int* block_table,
                                     int max_pages, int page_size, int n, int heads, int kv_heads, int head_dim,
                                     int v_offset, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && heads > 0 && kv_heads > 0 && head_dim > 0, "qk_norm_rope_cache: bad sizes");
  HFEE_REQUIRE(rope_dim >= 0 && rope_dim % 2 == 0 && rope_dim <= head_dim,
               "qk_norm_rope_cache: rope_dim %d must be even and at most head_dim %d", rope_dim, head_dim);
  HFEE_REQUIRE(ld_q >= (long long)heads * head_dim && ld_qk >= (long long)heads * head_dim + (k_pool ? (long long)kv_heads * head_dim : 0),
               "qk_norm_rope_cache: a leading dimension is too small");
  PagedCache c;
  HFEE_REQUIRE(make_paged_cache(&c, block_table, max_pages, page_size, kv_heads, head_dim),
               "page_size %d must be a power of two", page_size);
  const float2* cs2 = (const float2*)cs;
  if (dtype == HFEE_F32)
    hfee_launch(qk_norm_rope_cache_kernel<float>, dim3(n), dim3(ROW_THREADS), 0, stream, (const float*)qk, ld_qk, wq, wk, eps, cs2,
                rope_dim, positions, slot_of_token, (float*)q_out, ld_q, (float*)k_pool, (float*)v_pool, c, heads, v_offset);
  else if (dtype == HFEE_BF16)
    hfee_launch(qk_norm_rope_cache_kernel<__nv_bfloat16>, dim3(n), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)qk, ld_qk, wq, wk,
                eps, cs2, rope_dim, positions, slot_of_token, (__nv_bfloat16*)q_out, ld_q, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, c, heads, v_offset);
  else
    return hfee_fail(HFEE_ERR_ARG, "qk_norm_rope_cache: unknown dtype %d", dtype);
  return hfee_check_launch("qk_norm_rope_cache");
}

// ---------------------------------------------------------------------------------------------------------------
//   hfee_head_norm_gate   per (token, head): out = x / sqrt(mean_head(x^2) + eps) * w[d] * act(gate) * out_scale, the weight
//                         [head_dim] shared by the heads, or [heads * head_dim] (w_head_stride = head_dim); act = sigmoid or SiLU
//   hfee_unary_act        out = act(x) element by element; act = relu(x)^2
//   hfee_head_gate        x[i, h, :] *= sigmoid(gate[i, h]): one gate number per head
namespace {

constexpr int HG_SIGMOID = 0, HG_SILU = 1;
constexpr int UA_RELU2 = 0;

template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ x, long long ld_x, const float* __restrict__ w, float eps,
                      const T* __restrict__ gate, long long ld_g, T* __restrict__ out, long long ld_o, int n, int heads,
                      int head_dim, int act, int w_head_stride, float out_scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const unsigned task = blockIdx.x * 4 + (threadIdx.x >> 5);   // the launcher keeps n * heads below 2^31
  if (task >= (unsigned)n * (unsigned)heads) return;
  const int i = (int)(task / (unsigned)heads), h = (int)(task - (unsigned)i * (unsigned)heads);
  const float* xr = x + (long long)i * ld_x + (long long)h * head_dim;
  const T* gr = gate + (long long)i * ld_g + (long long)h * head_dim;
  T* orow = out + (long long)i * ld_o + (long long)h * head_dim;
  float ss = 0.f;
  for (int d = lane; d < head_dim; d += 32) ss = fmaf(xr[d], xr[d], ss);
  const float scale = out_scale / sqrtf(warp_sum(ss) / (float)head_dim + eps);
  const float* wh = w + (long long)h * w_head_stride;
  for (int d = lane; d < head_dim; d += 32) {
    const float g = to_f32<T>(gr[d]);
    const float s = sigmoid_f32(g);
    orow[d] = from_f32<T>(xr[d] * scale * wh[d] * (act == HG_SILU ? g * s : s));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
unary_act_kernel(const T* __restrict__ x, long long ld_x, T* __restrict__ out, long long ld_o, int cols, long long total, int act) {
  pdl_wait();
  pdl_launch_dependents();
  const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
  if (e >= total) return;
  const long long r = e / cols;
  const int c = (int)(e - r * cols);
  const float v = fmaxf(to_f32<T>(x[r * ld_x + c]), 0.f);
  out[r * ld_o + c] = from_f32<T>(v * v);
}

template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ x, long long ld_x, const T* __restrict__ gate, long long ld_g, int heads, int head_dim,
                 long long total) {
  pdl_wait();
  pdl_launch_dependents();
  const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
  if (e >= total) return;
  const int cols = heads * head_dim;
  const long long r = e / cols;
  const int c = (int)(e - r * cols);
  const float g = sigmoid_f32(to_f32<T>(gate[r * ld_g + c / head_dim]));
  x[r * ld_x + c] = from_f32<T>(to_f32<T>(x[r * ld_x + c]) * g);
}

}  // namespace

HFEE_API int hfee_head_norm_gate_scaled(const float* x, long long ld_x, const float* w, int w_per_head, float eps, const void* gate,
                                        long long ld_g, void* out, long long ld_o, int n, int heads, int head_dim, int act,
                                        float out_scale, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  const int w_head_stride = w_per_head ? head_dim : 0;
  const long long width = (long long)heads * head_dim;
  HFEE_REQUIRE(n > 0 && heads > 0 && head_dim > 0 && ld_x >= width && ld_g >= width && ld_o >= width, "head_norm_gate: bad sizes");
  HFEE_REQUIRE(act == HG_SIGMOID || act == HG_SILU, "head_norm_gate: unknown gate activation %d", act);
  HFEE_REQUIRE((long long)n * heads < (1ll << 31), "head_norm_gate: too many (token, head) pairs for one launch");
  const unsigned blocks = (unsigned)(((long long)n * heads + 3) / 4);
  if (dtype == HFEE_F32)
    hfee_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, stream, x, ld_x, w, eps, (const float*)gate, ld_g, (float*)out, ld_o, n, heads, head_dim, act, w_head_stride, out_scale);
  else if (dtype == HFEE_BF16)
    hfee_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, x, ld_x, w, eps, (const __nv_bfloat16*)gate, ld_g, (__nv_bfloat16*)out, ld_o, n, heads, head_dim, act, w_head_stride, out_scale);
  else
    return hfee_fail(HFEE_ERR_ARG, "head_norm_gate: unknown dtype %d", dtype);
  return hfee_check_launch("head_norm_gate");
}

HFEE_API int hfee_head_norm_gate(const float* x, long long ld_x, const float* w, float eps, const void* gate, long long ld_g,
                                 void* out, long long ld_o, int n, int heads, int head_dim, int act, int dtype,
                                 cudaStream_t stream) {
  return hfee_head_norm_gate_scaled(x, ld_x, w, 0, eps, gate, ld_g, out, ld_o, n, heads, head_dim, act, 1.f, dtype, stream);
}

HFEE_API int hfee_unary_act(const void* x, long long ld_x, void* out, long long ld_o, int rows, int cols, int act, int dtype,
                            cudaStream_t stream) {
  if (rows == 0 || cols == 0) return HFEE_OK;
  HFEE_REQUIRE(rows > 0 && cols > 0 && ld_x >= cols && ld_o >= cols, "unary_act: bad sizes");
  HFEE_REQUIRE(act == UA_RELU2, "unary_act: unknown activation %d", act);
  const long long total = (long long)rows * cols;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == HFEE_F32)
    hfee_launch(unary_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, ld_x, (float*)out, ld_o, cols, total, act);
  else if (dtype == HFEE_BF16)
    hfee_launch(unary_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, ld_x, (__nv_bfloat16*)out, ld_o, cols, total, act);
  else
    return hfee_fail(HFEE_ERR_ARG, "unary_act: unknown dtype %d", dtype);
  return hfee_check_launch("unary_act");
}

HFEE_API int hfee_head_gate(void* x, long long ld_x, const void* gate, long long ld_g, int n, int heads, int head_dim, int dtype,
                            cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && heads > 0 && head_dim > 0 && ld_x >= (long long)heads * head_dim && ld_g >= heads, "head_gate: bad sizes");
  const long long total = (long long)n * heads * head_dim;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == HFEE_F32)
    hfee_launch(head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, ld_x, (const float*)gate, ld_g, heads, head_dim, total);
  else if (dtype == HFEE_BF16)
    hfee_launch(head_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, ld_x, (const __nv_bfloat16*)gate, ld_g, heads, head_dim, total);
  else
    return hfee_fail(HFEE_ERR_ARG, "head_gate: unknown dtype %d", dtype);
  return hfee_check_launch("head_gate");
}
