// Elementwise linear recurrences S_t = a_t S_(t-1) + b_t with a per-request state in float32.
//
//   hfee_mingru          z = sigmoid(pz + bz), u = px + bx, c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
//                        S_t = (1 - z) S_(t-1) + z c per channel; out = S_t * silu(g) in the activations' dtype.
//   hfee_selective_scan  dt = softplus(pdt + dt_bias), A = -exp(A_log); per channel c and state entry n
//                        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;
//                        out = y * silu(z) * out_scale.
//
// Both walk a request's tokens of the step from the state its slot holds and leave the new state there, so a
// prompt may be cut anywhere.  A portion is split among the warps of a CTA in equal runs of tokens: every warp
// first reduces its run to the pair (product of a, value reached from zero), the pairs of the runs in front are
// applied in order to the slot's state, and the run is walked again from the state that gives, this time with
// outputs.  With one warp (decode steps, short portions) the first two phases fall away.  All arithmetic on
// gates, step sizes, decays and states is float32; T is the dtype of the projections and of the output.
#include "common.cuh"

namespace {

constexpr int MAX_WARPS = 32;

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f32(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// The run of tokens [lo, hi) of warp `warp` among `warps` for a portion of `count` tokens.
__device__ __forceinline__ void token_run(int count, int warps, int warp, int* lo, int* hi) {
  const int len = (count + warps - 1) / warps;
  *lo = min(count, warp * len);
  *hi = min(count, *lo + len);
}

// ---------------------------------------------------------------------------------------------- minGRU
template <typename T>
__global__ void mingru_kernel(const T* __restrict__ proj, long long ld, int z_off, int x_off, int g_off,
                              const float* __restrict__ z_bias, const float* __restrict__ x_bias, float* __restrict__ state,
                              const int* __restrict__ cu_tokens, const int* __restrict__ slots, T* __restrict__ out,
                              long long ld_out, int channels, int write_state) {
  __shared__ float run_a[MAX_WARPS][32], run_b[MAX_WARPS][32];
  const int req = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;        // host-written batch layout
  const int slot = slots[req];
  const bool live = c < channels;
  const float bz = live ? z_bias[c] : 0.f, bx = live ? x_bias[c] : 0.f;       // weights
  pdl_wait();
  pdl_launch_dependents();
  int lo, hi;
  token_run(count, warps, warp, &lo, &hi);
  const T* rows = proj + (long long)begin * ld;
  if (warps > 1) {
    float a = 1.f, b = 0.f;
    if (live) {
#pragma unroll 4
      for (int t = lo; t < hi; ++t) {
        const T* row = rows + (long long)t * ld;
        const float z = sigmoid_f32(to_f32<T>(row[z_off + c]) + bz);
        const float u = to_f32<T>(row[x_off + c]) + bx;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f32(u);
        a *= 1.f - z;
        b = fmaf(1.f - z, b, z * cand);
      }
    }
    run_a[warp][lane] = a;
    run_b[warp][lane] = b;
    __syncthreads();
  }
  if (!live) return;
  float* st = state + (long long)slot * channels + c;
  float S = *st;
  for (int w = 0; w < warp; ++w) S = fmaf(run_a[w][lane], S, run_b[w][lane]);
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    const T* row = rows + (long long)t * ld;
    const float z = sigmoid_f32(to_f32<T>(row[z_off + c]) + bz);
    const float u = to_f32<T>(row[x_off + c]) + bx;
    const float cand = u >= 0.f ? u + 0.5f : sigmoid_f32(u);
    S = fmaf(1.f - z, S, z * cand);
    const float g = to_f32<T>(row[g_off + c]);
    out[(long long)(begin + t) * ld_out + c] = from_f32<T>(S * g * sigmoid_f32(g));
  }
  if (write_state && hi == count && lo < hi) *st = S;
}

// ---------------------------------------------------------------------------------------------- selective scan
// LANES threads share a channel and hold NS state entries each (entry n = part + LANES * j).
template <typename T, int NS>
__global__ void selective_scan_kernel(const T* __restrict__ x, long long ld_x, const float* __restrict__ dt_proj, long long ld_dt,
                                      const T* __restrict__ bc, long long ld_bc, int b_off, int c_off,
                                      const T* __restrict__ z, long long ld_z, const float* __restrict__ a_log,
                                      const float* __restrict__ d_skip, const float* __restrict__ dt_bias,
                                      float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                                      T* __restrict__ out, long long ld_out, int channels, int n_state, int lanes, float out_scale,
                                      int write_state) {
  extern __shared__ float runs[];          // [warps][2][NS][32]
  const int req = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int per_warp = 32 / lanes;
  const int part = lane % lanes;
  const int c = blockIdx.x * per_warp + lane / lanes;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;        // host-written batch layout
  const int slot = slots[req];
  const bool live = c < channels;
  float A[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = part + lanes * j;
    A[j] = (live && n < n_state) ? -expf(a_log[(long long)c * n_state + n]) : 0.f;      // weights
  }
  const float bias = live ? dt_bias[c] : 0.f, skip = live ? d_skip[c] : 0.f;
  pdl_wait();
  pdl_launch_dependents();
  int lo, hi;
  token_run(count, warps, warp, &lo, &hi);
  const int cc = live ? c : 0;             // dead lanes read a valid address and write nothing
  if (warps > 1) {
    float dt_sum = 0.f, b[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) b[j] = 0.f;
    for (int t = lo; t < hi; ++t) {
      const long long row = begin + t;
      const float dt = softplus_f32(dt_proj[row * ld_dt + cc] + bias);
      const float dx = dt * to_f32<T>(x[row * ld_x + cc]);
      dt_sum += dt;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        const int n = part + lanes * j;
        const float Bn = n < n_state ? to_f32<T>(bc[row * ld_bc + b_off + n]) : 0.f;
        b[j] = fmaf(expf(dt * A[j]), b[j], dx * Bn);
      }
    }
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      runs[((warp * 2 + 0) * NS + j) * 32 + lane] = expf(dt_sum * A[j]);
      runs[((warp * 2 + 1) * NS + j) * 32 + lane] = b[j];
    }
    __syncthreads();
  }
  float S[NS];
  float* st = state + ((long long)slot * channels + cc) * n_state;
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = part + lanes * j;
    S[j] = (live && n < n_state) ? st[n] : 0.f;
  }
  for (int w = 0; w < warp; ++w) {
#pragma unroll
    for (int j = 0; j < NS; ++j)
      S[j] = fmaf(runs[((w * 2 + 0) * NS + j) * 32 + lane], S[j], runs[((w * 2 + 1) * NS + j) * 32 + lane]);
  }
  for (int t = lo; t < hi; ++t) {
    const long long row = begin + t;
    const float dt = softplus_f32(dt_proj[row * ld_dt + cc] + bias);
    const float xv = to_f32<T>(x[row * ld_x + cc]);
    const float dx = dt * xv;
    float y = 0.f;
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int n = part + lanes * j;
      const bool in = n < n_state;
      const float Bn = in ? to_f32<T>(bc[row * ld_bc + b_off + n]) : 0.f;
      const float Cn = in ? to_f32<T>(bc[row * ld_bc + c_off + n]) : 0.f;
      S[j] = fmaf(expf(dt * A[j]), S[j], dx * Bn);
      y = fmaf(S[j], Cn, y);
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (live && part == 0) {
      const float g = to_f32<T>(z[row * ld_z + c]);
      out[row * ld_out + c] = from_f32<T>(fmaf(skip, xv, y) * g * sigmoid_f32(g) * out_scale);
    }
  }
  if (write_state && live && hi == count && lo < hi) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int n = part + lanes * j;
      if (n < n_state) st[n] = S[j];
    }
  }
}

int warps_for(int max_new, int most) {
  int w = (max_new + 15) / 16;            // runs of 16 tokens and more
  if (w < 1) w = 1;
  return w > most ? most : w;
}

template <typename T>
int launch_mingru(const void* proj, long long ld, int z_off, int x_off, int g_off, const float* z_bias, const float* x_bias,
                  float* state, const int* cu_tokens, const int* slots, void* out, long long ld_out, int requests, int max_new,
                  int channels, int write_state, cudaStream_t stream) {
  const int warps = warps_for(max_new, MAX_WARPS);
  hfee_launch(mingru_kernel<T>, dim3((channels + 31) / 32, requests), dim3(32 * warps), 0, stream, (const T*)proj, ld, z_off, x_off,
              g_off, z_bias, x_bias, state, cu_tokens, slots, (T*)out, ld_out, channels, write_state);
  return hfee_check_launch("mingru");
}

template <typename T, int NS>
int launch_scan_ns(const void* x, long long ld_x, const float* dt_proj, long long ld_dt, const void* bc, long long ld_bc, int b_off,
                   int c_off, const void* z, long long ld_z, const float* a_log, const float* d_skip, const float* dt_bias,
                   float* state, const int* cu_tokens, const int* slots, void* out, long long ld_out, int requests, int max_new,
                   int channels, int n_state, int lanes, float out_scale, int write_state, cudaStream_t stream) {
  const int warps = warps_for(max_new, NS <= 4 ? MAX_WARPS : 8);
  const size_t smem = warps > 1 ? (size_t)warps * 2 * NS * 32 * sizeof(float) : 0;
  const int per_warp = 32 / lanes;
  hfee_launch(selective_scan_kernel<T, NS>, dim3((channels + per_warp - 1) / per_warp, requests), dim3(32 * warps), smem, stream,
              (const T*)x, ld_x, dt_proj, ld_dt, (const T*)bc, ld_bc, b_off, c_off, (const T*)z, ld_z, a_log, d_skip, dt_bias, state,
              cu_tokens, slots, (T*)out, ld_out, channels, n_state, lanes, out_scale, write_state);
  return hfee_check_launch("selective_scan");
}

}  // namespace

// proj: [n, >= 3 * channels] with z, x, g at their column offsets; state: [slots, channels] float32.
HFEE_API int hfee_mingru(const void* proj, long long ld, int z_off, int x_off, int g_off, const float* z_bias, const float* x_bias,
                         float* state, const int* cu_tokens, const int* slots, void* out, long long ld_out, int requests, int max_new,
                         int channels, int write_state, int dtype, cudaStream_t stream) {
  if (requests == 0 || max_new == 0) return HFEE_OK;
  HFEE_REQUIRE(requests > 0 && max_new > 0 && channels > 0 && ld_out >= channels, "mingru: bad sizes");
  HFEE_REQUIRE(z_off >= 0 && x_off >= 0 && g_off >= 0 && ld >= channels, "mingru: bad offsets");
  if (dtype == HFEE_F32)
    return launch_mingru<float>(proj, ld, z_off, x_off, g_off, z_bias, x_bias, state, cu_tokens, slots, out, ld_out, requests, max_new,
                                channels, write_state, stream);
  if (dtype == HFEE_BF16)
    return launch_mingru<__nv_bfloat16>(proj, ld, z_off, x_off, g_off, z_bias, x_bias, state, cu_tokens, slots, out, ld_out, requests,
                                        max_new, channels, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "mingru: unknown dtype %d", dtype);
}

// x, z, out: [n, channels] (row strides of their own); dt_proj: [n, channels] float32, the step-size projection in front of
// its bias and softplus; bc: rows holding B at b_off and C at c_off, n_state entries each; a_log: [channels, n_state];
// state: [slots, channels, n_state] float32.
HFEE_API int hfee_selective_scan(const void* x, long long ld_x, const float* dt_proj, long long ld_dt, const void* bc, long long ld_bc,
                                 int b_off, int c_off, const void* z, long long ld_z, const float* a_log, const float* d_skip,
                                 const float* dt_bias, float* state, const int* cu_tokens, const int* slots, void* out,
                                 long long ld_out, int requests, int max_new, int channels, int n_state, float out_scale,
                                 int write_state, int dtype, cudaStream_t stream) {
  if (requests == 0 || max_new == 0) return HFEE_OK;
  HFEE_REQUIRE(requests > 0 && max_new > 0 && channels > 0, "selective_scan: bad sizes");
  HFEE_REQUIRE(n_state >= 1 && n_state <= 512, "selective_scan: state size %d is outside 1..512", n_state);
  HFEE_REQUIRE(ld_x >= channels && ld_dt >= channels && ld_z >= channels && ld_out >= channels, "selective_scan: a row stride is too small");
  int lanes = 1;
  while (lanes < 32 && lanes * 4 < n_state) lanes *= 2;      // four state entries a thread where 32 lanes allow it
  const int ns = (n_state + lanes - 1) / lanes;
#define HFEE_SCAN(T, NS)                                                                                                        \
  return launch_scan_ns<T, NS>(x, ld_x, dt_proj, ld_dt, bc, ld_bc, b_off, c_off, z, ld_z, a_log, d_skip, dt_bias, state, cu_tokens, \
                               slots, out, ld_out, requests, max_new, channels, n_state, lanes, out_scale, write_state, stream)
  if (dtype == HFEE_F32) {
    if (ns <= 4) HFEE_SCAN(float, 4);
    HFEE_SCAN(float, 16);
  }
  if (dtype == HFEE_BF16) {
    if (ns <= 4) HFEE_SCAN(__nv_bfloat16, 4);
    HFEE_SCAN(__nv_bfloat16, 16);
  }
#undef HFEE_SCAN
  return hfee_fail(HFEE_ERR_ARG, "selective_scan: unknown dtype %d", dtype);
}
