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
#include <cstdint>

namespace {

constexpr int MAX_WARPS = 32;

// Gates and step sizes of the bfloat16 models come from projections that carry 8 significant bits, so their
// instances take the hardware's approximate exponential, logarithm and reciprocal (float32, about 2 units in the last
// place); the float32 instances keep the exact functions.
template <typename T> struct Fn {
  static __device__ __forceinline__ float sigmoid(float v) { return 1.f / (1.f + expf(-v)); }
  static __device__ __forceinline__ float softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }
  static __device__ __forceinline__ float decay_rate(float a) { return a; }                 // decay = exp(dt * rate)
  static __device__ __forceinline__ float decay(float dt, float rate) { return expf(dt * rate); }
};
template <> struct Fn<__nv_bfloat16> {
  static __device__ __forceinline__ float sigmoid(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }
  static __device__ __forceinline__ float softplus(float v) {
    const float e = __expf(v);
    return v > 20.f ? v : (v < -15.f ? e : __logf(1.f + e));      // 1 + e rounds to 1 below: ln(1 + e) = e there
  }
  static __device__ __forceinline__ float decay_rate(float a) { return a * 1.4426950408889634f; }
  static __device__ __forceinline__ float decay(float dt, float rate) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(dt * rate));
    return r;
  }
};

// The run of tokens [lo, hi) of run `run` among `runs` for a portion of `count` tokens.
__device__ __forceinline__ void token_run(int count, int runs, int run, int* lo, int* hi) {
  const int len = (count + runs - 1) / runs;
  *lo = min(count, run * len);
  *hi = min(count, *lo + len);
}

// ---------------------------------------------------------------------------------------------- minGRU
// A CTA owns CH channels (32, or 16 when that fills more of the GPU); a warp walks 32 / CH runs of tokens at once.
template <typename T, int CH>
__global__ void mingru_kernel(const T* __restrict__ proj, long long ld, int z_off, int x_off, int g_off,
                              const float* __restrict__ z_bias, const float* __restrict__ x_bias, float* __restrict__ state,
                              const int* __restrict__ cu_tokens, const int* __restrict__ slots, T* __restrict__ out,
                              long long ld_out, int channels, int write_state) {
  constexpr int SUB = 32 / CH;
  __shared__ float run_a[MAX_WARPS * SUB][CH], run_b[MAX_WARPS * SUB][CH];
  const int req = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int ch = lane % CH, run = warp * SUB + lane / CH, runs = warps * SUB;
  const int c = blockIdx.x * CH + ch;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;        // host-written batch layout
  const int slot = slots[req];
  const bool live = c < channels;
  const float bz = live ? z_bias[c] : 0.f, bx = live ? x_bias[c] : 0.f;       // weights
  pdl_wait();
  pdl_launch_dependents();
  int lo, hi;
  token_run(count, runs, run, &lo, &hi);
  const T* rows = proj + (long long)begin * ld + (live ? c : 0);
  if (runs > 1) {
    float a = 1.f, b = 0.f;
    if (live) {
#pragma unroll 4
      for (int t = lo; t < hi; ++t) {
        const T* row = rows + (long long)t * ld;
        const float z = Fn<T>::sigmoid(to_f32<T>(row[z_off]) + bz);
        const float u = to_f32<T>(row[x_off]) + bx;
        const float cand = u >= 0.f ? u + 0.5f : Fn<T>::sigmoid(u);
        a *= 1.f - z;
        b = fmaf(1.f - z, b, z * cand);
      }
    }
    run_a[run][ch] = a;
    run_b[run][ch] = b;
    __syncthreads();
  }
  if (!live) return;
  float* st = state + (long long)slot * channels + c;
  float S = *st;
  for (int w = 0; w < run; ++w) S = fmaf(run_a[w][ch], S, run_b[w][ch]);
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    const T* row = rows + (long long)t * ld;
    const float z = Fn<T>::sigmoid(to_f32<T>(row[z_off]) + bz);
    const float u = to_f32<T>(row[x_off]) + bx;
    const float cand = u >= 0.f ? u + 0.5f : Fn<T>::sigmoid(u);
    S = fmaf(1.f - z, S, z * cand);
    const float g = to_f32<T>(row[g_off]);
    out[(long long)(begin + t) * ld_out + c] = from_f32<T>(S * g * Fn<T>::sigmoid(g));
  }
  if (write_state && hi == count && lo < hi) *st = S;
}

// ---------------------------------------------------------------------------------------------- selective scan
// LANES threads share a channel and hold NS state entries each (entries part * NS .. part * NS + NS - 1).  Tokens are
// taken TB at a time: everything the TB tokens read is requested first, so a warp waits for memory once per TB tokens.
constexpr int SCAN_MAX_WARPS = 16;

// NS entries of B or C from `p` (the row's first entry) starting at entry n0, as float32; entries from n_state on are zero.
template <typename T, int NS, bool VEC> struct Entries {
  T v[NS];
  __device__ __forceinline__ void load(const T* p, int n0, int n_state) {
#pragma unroll
    for (int j = 0; j < NS; ++j) v[j] = n0 + j < n_state ? p[n0 + j] : from_f32<T>(0.f);
  }
  __device__ __forceinline__ float get(int j) const { return to_f32<T>(v[j]); }
};
// four bfloat16 entries in one 8-byte request (rows, offsets and n_state multiples of four)
template <> struct Entries<__nv_bfloat16, 4, true> {
  uint2 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p, int n0, int n_state) {
    v = n0 < n_state ? *reinterpret_cast<const uint2*>(p + n0) : make_uint2(0u, 0u);
  }
  __device__ __forceinline__ float get(int j) const {
    const unsigned w = j < 2 ? v.x : v.y;
    return __uint_as_float((j & 1) ? (w & 0xffff0000u) : (w << 16));
  }
};

template <typename T, int NS, bool VEC>
__global__ void __launch_bounds__(NS <= 4 ? 32 * SCAN_MAX_WARPS : 256, NS <= 4 ? 2 : 1)
selective_scan_kernel(const T* __restrict__ x, int ld_x, const float* __restrict__ dt_proj, int ld_dt,
                      const T* __restrict__ bc, int ld_bc, int b_off, int c_off,
                      const T* __restrict__ z, int ld_z, const float* __restrict__ a_log,
                      const float* __restrict__ d_skip, const float* __restrict__ dt_bias,
                      float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                      T* __restrict__ out, int ld_out, int channels, int n_state, int lanes, float out_scale,
                      int write_state) {
  constexpr int TB = NS <= 4 ? 2 : 1;      // two CTAs of 16 warps an SM hold no more in 64 registers
  extern __shared__ float runs[];          // [warps][2][NS][32]
  const int req = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int per_warp = 32 / lanes;
  const int part = lane % lanes, n0 = part * NS;
  const int c = blockIdx.x * per_warp + lane / lanes;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;        // host-written batch layout
  const int slot = slots[req];
  const bool live = c < channels;
  const int cc = live ? c : 0;             // dead lanes read a valid address and write nothing
  float A[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j)
    A[j] = (live && n0 + j < n_state) ? Fn<T>::decay_rate(-expf(a_log[(long long)cc * n_state + n0 + j])) : 0.f;      // weights
  const float bias = live ? dt_bias[c] : 0.f, skip = live ? d_skip[c] : 0.f;
  pdl_wait();
  pdl_launch_dependents();
  int lo, hi;
  token_run(count, warps, warp, &lo, &hi);
  const float* dt_p = dt_proj + (long long)begin * ld_dt + cc;
  const T* x_p = x + (long long)begin * ld_x + cc;
  const T* z_p = z + (long long)begin * ld_z + cc;
  const T* b_p = bc + (long long)begin * ld_bc + b_off;
  const T* c_p = bc + (long long)begin * ld_bc + c_off;
  T* out_p = out + (long long)begin * ld_out + cc;
  if (warps > 1) {
    float dt_sum = 0.f, b[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) b[j] = 0.f;
    for (int t0 = lo; t0 < hi; t0 += TB) {
      float dt_raw[TB];
      T x_raw[TB];
      Entries<T, NS, VEC> B[TB];
#pragma unroll
      for (int k = 0; k < TB; ++k) {
        const int t = min(t0 + k, hi - 1);          // offsets inside a request's rows fit 32 bits (checked at the launch)
        dt_raw[k] = dt_p[t * ld_dt];
        x_raw[k] = x_p[t * ld_x];
        B[k].load(b_p + t * ld_bc, n0, n_state);
      }
#pragma unroll
      for (int k = 0; k < TB; ++k) {
        if (t0 + k < hi) {
          const float dt = Fn<T>::softplus(dt_raw[k] + bias);
          const float dx = dt * to_f32<T>(x_raw[k]);
          dt_sum += dt;
#pragma unroll
          for (int j = 0; j < NS; ++j) b[j] = fmaf(Fn<T>::decay(dt, A[j]), b[j], dx * B[k].get(j));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      runs[((warp * 2 + 0) * NS + j) * 32 + lane] = Fn<T>::decay(dt_sum, A[j]);
      runs[((warp * 2 + 1) * NS + j) * 32 + lane] = b[j];
    }
    __syncthreads();
  }
  float S[NS];
  float* st = state + ((long long)slot * channels + cc) * n_state;
#pragma unroll
  for (int j = 0; j < NS; ++j) S[j] = (live && n0 + j < n_state) ? st[n0 + j] : 0.f;
  for (int w = 0; w < warp; ++w) {
#pragma unroll
    for (int j = 0; j < NS; ++j)
      S[j] = fmaf(runs[((w * 2 + 0) * NS + j) * 32 + lane], S[j], runs[((w * 2 + 1) * NS + j) * 32 + lane]);
  }
  for (int t0 = lo; t0 < hi; t0 += TB) {
    float dt_raw[TB];
    T x_raw[TB], z_raw[TB];
    Entries<T, NS, VEC> B[TB], C[TB];
#pragma unroll
    for (int k = 0; k < TB; ++k) {
      const int t = min(t0 + k, hi - 1);
      dt_raw[k] = dt_p[t * ld_dt];
      x_raw[k] = x_p[t * ld_x];
      z_raw[k] = z_p[t * ld_z];
      B[k].load(b_p + t * ld_bc, n0, n_state);
      C[k].load(c_p + t * ld_bc, n0, n_state);
    }
#pragma unroll
    for (int k = 0; k < TB; ++k) {
      if (t0 + k < hi) {             // the same for the whole warp
        const float dt = Fn<T>::softplus(dt_raw[k] + bias);
        const float xv = to_f32<T>(x_raw[k]);
        const float dx = dt * xv;
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < NS; ++j) {
          S[j] = fmaf(Fn<T>::decay(dt, A[j]), S[j], dx * B[k].get(j));
          y = fmaf(S[j], C[k].get(j), y);
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (live && part == 0) {
          const float g = to_f32<T>(z_raw[k]);
          out_p[(t0 + k) * ld_out] = from_f32<T>(fmaf(skip, xv, y) * g * Fn<T>::sigmoid(g) * out_scale);
        }
      }
    }
  }
  if (write_state && live && hi == count && lo < hi) {
#pragma unroll
    for (int j = 0; j < NS; ++j)
      if (n0 + j < n_state) st[n0 + j] = S[j];
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
  // half-warps of 16 channels and two runs of tokens a warp while CTAs of 32 channels would leave SMs idle
  if (max_new >= 32 && (long long)((channels + 31) / 32) * requests < 128) {
    const int warps = warps_for((max_new + 1) / 2, MAX_WARPS);
    hfee_launch(mingru_kernel<T, 16>, dim3((channels + 15) / 16, requests), dim3(32 * warps), 0, stream, (const T*)proj, ld, z_off,
                x_off, g_off, z_bias, x_bias, state, cu_tokens, slots, (T*)out, ld_out, channels, write_state);
  } else {
    const int warps = warps_for(max_new, MAX_WARPS);
    hfee_launch(mingru_kernel<T, 32>, dim3((channels + 31) / 32, requests), dim3(32 * warps), 0, stream, (const T*)proj, ld, z_off,
                x_off, g_off, z_bias, x_bias, state, cu_tokens, slots, (T*)out, ld_out, channels, write_state);
  }
  return hfee_check_launch("mingru");
}

template <typename T, int NS>
int launch_scan_ns(const void* x, long long ld_x, const float* dt_proj, long long ld_dt, const void* bc, long long ld_bc, int b_off,
                   int c_off, const void* z, long long ld_z, const float* a_log, const float* d_skip, const float* dt_bias,
                   float* state, const int* cu_tokens, const int* slots, void* out, long long ld_out, int requests, int max_new,
                   int channels, int n_state, int lanes, float out_scale, int write_state, cudaStream_t stream) {
  const int warps = warps_for(max_new, NS <= 4 ? SCAN_MAX_WARPS : 8);
  const size_t smem = warps > 1 ? (size_t)warps * 2 * NS * 32 * sizeof(float) : 0;
  const int per_warp = 32 / lanes;
  const dim3 grid((channels + per_warp - 1) / per_warp, requests), block(32 * warps);
  // 8-byte requests for a thread's four bfloat16 entries of B and of C where every one of them is aligned
  const bool vec = sizeof(T) == 2 && NS == 4 && n_state % 4 == 0 && b_off % 4 == 0 && c_off % 4 == 0 && ld_bc % 4 == 0 &&
                   (uintptr_t)bc % 8 == 0;
#define HFEE_SCAN_LAUNCH(VEC)                                                                                                \
  hfee_launch(selective_scan_kernel<T, NS, VEC>, grid, block, smem, stream, (const T*)x, (int)ld_x, dt_proj, (int)ld_dt,       \
              (const T*)bc, (int)ld_bc, b_off, c_off, (const T*)z, (int)ld_z, a_log, d_skip, dt_bias, state, cu_tokens, slots,  \
              (T*)out, (int)ld_out,                                                                                       \
              channels, n_state, lanes, out_scale, write_state)
  if (vec) HFEE_SCAN_LAUNCH(true);
  else HFEE_SCAN_LAUNCH(false);
#undef HFEE_SCAN_LAUNCH
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
  {
    long long widest = ld_x > ld_dt ? ld_x : ld_dt;
    for (long long ld : {ld_bc, ld_z, ld_out}) widest = ld > widest ? ld : widest;
    HFEE_REQUIRE(widest * max_new < (1ll << 31), "selective_scan: %d rows of %lld entries pass 32-bit offsets", max_new, widest);
  }
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
