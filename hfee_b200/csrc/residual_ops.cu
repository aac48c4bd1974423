// Row kernels around the residual stream of designs that scale, average or cap it.
//
//   hfee_add_sinusoid      x[t, 2i] += sin(p_t * base^(-2i/width)), x[t, 2i+1] += cos(same): absolute positions
//                          as sines and cosines over the whole width (angles in float64).
//   hfee_softcap           x = cap * tanh(x / cap), float32 in place (logit capping).
//   hfee_clamped_glu       out = g * sigmoid(alpha * g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit),
//                          over a [gate | up] projection laid out in groups of `granule` columns.
//   hfee_scaled_add_norm   residual += m * y; out = residual / sqrt(mean(residual^2) + eps) * w: a sublayer's scaled
//                          output joins the stream and the next sublayer's input leaves in the same pass (out null:
//                          the sum alone).
//   hfee_depth_average     r = residual (+ m * y); history[index + 1] = r;
//                          residual = sum_(j <= index) a[j] * history[j] + a[index + 1] * r: what the next layer
//                          reads is a learned mix of the embedding output and every layer's result so far.
//
// All arithmetic is float32 (angles float64); `T` is the dtype of activations that leave for a matrix product.
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

__global__ void __launch_bounds__(ROW_THREADS)
add_sinusoid_kernel(float* __restrict__ x, const int* __restrict__ positions, int width, double log2_base) {
  const int t = blockIdx.x;
  const int p = positions[t];             // host-written batch layout
  pdl_wait();
  pdl_launch_dependents();
  float* row = x + (long long)t * width;
  const int pairs = (width + 1) / 2;
  for (int i = threadIdx.x; i < pairs; i += ROW_THREADS) {
    const double freq = exp2(-(2.0 * i / (double)width) * log2_base);
    double s, c;
    sincos((double)p * freq, &s, &c);
    row[2 * i] += (float)s;
    if (2 * i + 1 < width) row[2 * i + 1] += (float)c;
  }
}

constexpr int SOFTCAP_COLS = 4 * ROW_THREADS;

__global__ void __launch_bounds__(ROW_THREADS)
softcap_kernel(float* __restrict__ x, long long ld, int cols, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  float* row = x + (long long)blockIdx.x * ld;
  const float inv = 1.f / cap;
  // blockIdx.y: the row's columns in pieces of SOFTCAP_COLS, so that a few rows of a large vocabulary still fill the GPU
  const int c0 = blockIdx.y * SOFTCAP_COLS, c1 = min(cols, c0 + SOFTCAP_COLS);
  for (int c = c0 + threadIdx.x; c < c1; c += ROW_THREADS) row[c] = cap * tanhf(row[c] * inv);
}

__device__ __forceinline__ float clamped_glu(float gate, float up, float limit, float alpha, float shift) {
  const float g = fminf(gate, limit);
  const float u = fminf(fmaxf(up, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + shift);
}

constexpr int GLU_SPAN = 4 * ROW_THREADS;

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
clamped_glu_kernel(const T* __restrict__ gate_up, long long ld_in, T* __restrict__ out, long long ld_out, int inner,
                   int granule, float limit, float alpha, float shift) {
  pdl_wait();
  pdl_launch_dependents();
  const T* in = gate_up + (long long)blockIdx.x * ld_in;
  T* o = out + (long long)blockIdx.x * ld_out;
  // a block owns a span of GLU_SPAN columns of its row, so that a few rows (a decode step) still fill the SMs
  const int end = min(inner, (int)(blockIdx.y + 1) * GLU_SPAN);
  for (int c = blockIdx.y * GLU_SPAN + threadIdx.x; c < end; c += ROW_THREADS) {
    const int at = (c / granule) * 2 * granule + c % granule;
    o[c] = from_f32<T>(clamped_glu(to_f32<T>(in[at]), to_f32<T>(in[at + granule]), limit, alpha, shift));
  }
}

__device__ __forceinline__ float block_sum(float v, float* shared) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) shared[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < ROW_THREADS / 32; ++w) total += shared[w];      // the same order in every thread
  return total;
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
scaled_add_norm_kernel(const float* __restrict__ y, float m, float* __restrict__ residual, const float* __restrict__ w,
                       float eps, T* __restrict__ out, long long ld_out, int width) {
  __shared__ float partial[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const float* yr = y + (long long)blockIdx.x * width;
  float* rr = residual + (long long)blockIdx.x * width;
  float sq = 0.f;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
    const float v = fmaf(m, yr[c], rr[c]);
    rr[c] = v;
    sq = fmaf(v, v, sq);
  }
  if (out == nullptr) return;            // the sum alone (the same for every thread of the launch)
  const float inv = 1.f / sqrtf(block_sum(sq, partial) / (float)width + eps);
  T* o = out + (long long)blockIdx.x * ld_out;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) o[c] = from_f32<T>(rr[c] * inv * w[c]);   // the thread's own writes
}

constexpr int MAX_DEPTH = 256;

__global__ void __launch_bounds__(ROW_THREADS)
depth_average_kernel(float* __restrict__ residual, const float* __restrict__ y, float m, float* __restrict__ history,
                     long long entry_stride, const float* __restrict__ a, int index, int width) {
  __shared__ float a_s[MAX_DEPTH + 2];
  for (int j = threadIdx.x; j < index + 2; j += ROW_THREADS) a_s[j] = a[j];      // weights: never written by a kernel
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  const long long row = (long long)blockIdx.x * width;
  for (int c = threadIdx.x; c < width; c += ROW_THREADS) {
    float r = residual[row + c];
    if (y != nullptr) r = fmaf(m, y[row + c], r);
    history[(long long)(index + 1) * entry_stride + row + c] = r;
    float acc = 0.f;
    for (int j = 0; j <= index; ++j) acc = fmaf(a_s[j], history[(long long)j * entry_stride + row + c], acc);
    residual[row + c] = fmaf(a_s[index + 1], r, acc);
  }
}

}  // namespace

HFEE_API int hfee_add_sinusoid(float* x, const int* positions, int n, int width, float base, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && base > 1.f, "add_sinusoid: bad sizes or base");
  hfee_launch(add_sinusoid_kernel, dim3(n), dim3(ROW_THREADS), 0, stream, x, positions, width, log2((double)base));
  return hfee_check_launch("add_sinusoid");
}

HFEE_API int hfee_softcap(float* x, long long ld, int rows, int cols, float cap, cudaStream_t stream) {
  if (rows == 0) return HFEE_OK;
  HFEE_REQUIRE(rows > 0 && cols > 0 && ld >= cols && cap > 0.f, "softcap: bad sizes or cap");
  HFEE_REQUIRE((cols + SOFTCAP_COLS - 1) / SOFTCAP_COLS <= 65535, "softcap: %d columns are too many", cols);
  hfee_launch(softcap_kernel, dim3(rows, (cols + SOFTCAP_COLS - 1) / SOFTCAP_COLS), dim3(ROW_THREADS), 0, stream, x, ld, cols, cap);
  return hfee_check_launch("softcap");
}

HFEE_API int hfee_clamped_glu(const void* gate_up, long long ld_in, void* out, long long ld_out, int n, int inner, int granule,
                              float limit, float alpha, float shift, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && inner > 0 && granule > 0 && inner % granule == 0, "clamped_glu: inner %d is not a multiple of the granule %d", inner, granule);
  HFEE_REQUIRE(ld_in >= 2 * inner && ld_out >= inner && limit > 0.f, "clamped_glu: a row stride is too small or the limit is not positive");
  if (dtype == HFEE_F32)
    hfee_launch(clamped_glu_kernel<float>, dim3(n, (inner + GLU_SPAN - 1) / GLU_SPAN), dim3(ROW_THREADS), 0, stream, (const float*)gate_up, ld_in, (float*)out, ld_out,
                inner, granule, limit, alpha, shift);
  else if (dtype == HFEE_BF16)
    hfee_launch(clamped_glu_kernel<__nv_bfloat16>, dim3(n, (inner + GLU_SPAN - 1) / GLU_SPAN), dim3(ROW_THREADS), 0, stream, (const __nv_bfloat16*)gate_up, ld_in,
                (__nv_bfloat16*)out, ld_out, inner, granule, limit, alpha, shift);
  else
    return hfee_fail(HFEE_ERR_ARG, "clamped_glu: unknown dtype %d", dtype);
  return hfee_check_launch("clamped_glu");
}

HFEE_API int hfee_scaled_add_norm(const float* y, float m, float* residual, const float* w, float eps, void* out, long long ld_out,
                                  int n, int width, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && (out == nullptr || (ld_out >= width && w != nullptr)), "scaled_add_norm: bad sizes");
  if (dtype == HFEE_F32)
    hfee_launch(scaled_add_norm_kernel<float>, dim3(n), dim3(ROW_THREADS), 0, stream, y, m, residual, w, eps, (float*)out, ld_out, width);
  else if (dtype == HFEE_BF16)
    hfee_launch(scaled_add_norm_kernel<__nv_bfloat16>, dim3(n), dim3(ROW_THREADS), 0, stream, y, m, residual, w, eps,
                (__nv_bfloat16*)out, ld_out, width);
  else
    return hfee_fail(HFEE_ERR_ARG, "scaled_add_norm: unknown dtype %d", dtype);
  return hfee_check_launch("scaled_add_norm");
}

// history: [entries][entry_stride] float32 with entry_stride >= n * width; a: index + 2 weights; y may be null.
HFEE_API int hfee_depth_average(float* residual, const float* y, float m, float* history, long long entry_stride, const float* a,
                                int index, int n, int width, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && index >= 0 && index < MAX_DEPTH, "depth_average: layer index %d is outside 0..%d", index, MAX_DEPTH - 1);
  HFEE_REQUIRE(entry_stride >= (long long)n * width, "depth_average: the history's entries are too small");
  hfee_launch(depth_average_kernel, dim3(n), dim3(ROW_THREADS), 0, stream, residual, y, m, history, entry_stride, a, index, width);
  return hfee_check_launch("depth_average");
}
