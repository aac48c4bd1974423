// The gated delta rule on a matrix state per head, and the short convolution with activation in front of it.
//
//   hfee_conv_act     y[t, c] = act(sum_j w[c, j] * x[t - taps + 1 + j, c]) per request, inputs in front of the step's
//                     tokens taken from the request's state (its last taps - 1 inputs, zeros for a fresh request),
//                     which is renewed.  x is a slice of a projection (any row stride, either dtype); arithmetic and
//                     state are float32.
//   hfee_delta_rule   per request and head, with S [dim, vdim] float32 carried from step to step:
//                         S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//                     q and k are first made unit vectors (x / sqrt(sum x^2 + 1e-6); q also times dim^-1/2),
//                     beta_t = sigmoid(b_t), g_t = exp(-exp(A_log) * softplus(a_t + dt_bias)), all float32.
//                     Columns of S evolve independently: S[:, j] <- g S[:, j] + k * beta (v_j - g S[:, j].k), so a
//                     block owns DR_COLS columns of one (request, head), a warp one column (each lane keeps dim / 32
//                     of its entries in registers), and the tokens of the step are taken in tiles of DR_TILE, each
//                     solved at once (see the kernel): the result depends on how a prompt was cut only through the
//                     order of float32 sums.
#include "common.cuh"

namespace {

constexpr int CA_MAX_TAPS = 8;
constexpr int CA_TOKENS = 16;
constexpr int CA_THREADS = 128;
constexpr int CA_OUT = 1, CA_STATE = 2;
constexpr int ACT_NONE = 0, ACT_SILU = 1;

// CH = channels per thread: 2 (one 4- or 8-byte access for both) for even widths and row strides, else 1.
template <typename T, int CH> struct ChanIO;
template <typename T> struct ChanIO<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = to_f32<T>(*p); }
  static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { *p = from_f32<T>(v[0]); }
};
template <> struct ChanIO<float, 2> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[2]) { const float2 t = *reinterpret_cast<const float2*>(p); v[0] = t.x; v[1] = t.y; }
  static __device__ __forceinline__ void store(float* p, const float (&v)[2]) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
};
template <> struct ChanIO<__nv_bfloat16, 2> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[2]) {
    const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p);
    v[0] = __bfloat162float(t.x); v[1] = __bfloat162float(t.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[2]) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]); }
};

// values that are rounded to bfloat16 on the way out take the fast exponential and division
template <typename T> __device__ __forceinline__ float silu_out(float z);
template <> __device__ __forceinline__ float silu_out<float>(float z) { return z / (1.f + expf(-z)); }
template <> __device__ __forceinline__ float silu_out<__nv_bfloat16>(float z) { return __fdividef(z, 1.f + __expf(-z)); }

// MAXT: the most taps this instance takes (4 or CA_MAX_TAPS): the window and the weights live in registers
template <typename T, int CH, int MAXT>
__global__ void __launch_bounds__(CA_THREADS)
conv_act_kernel(const T* __restrict__ x, long long ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots, T* __restrict__ out, long long ld_out,
                int width, int taps, int act, int mode) {
  const int req = blockIdx.y;
  const int c = (blockIdx.z * CA_THREADS + threadIdx.x) * CH;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;     // host-written batch layout
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0 || c >= width) return;
  const int hist = taps - 1;
  const int first = (mode == CA_STATE) ? ((count - 1) / CA_TOKENS) * CA_TOKENS : blockIdx.x * CA_TOKENS;
  if (first >= count) return;
  const int last = min(count, first + CA_TOKENS);
  float* st = state + (long long)slot * hist * width + c;                    // st[s * width]: input at index s - hist
  const T* xc = x + (long long)begin * ld_x + c;
  float wv[CH][MAXT], win[MAXT][CH], bv[CH];
#pragma unroll
  for (int k = 0; k < CH; ++k) bv[k] = bias != nullptr ? bias[c + k] : 0.f;
#pragma unroll
  for (int j = 0; j < MAXT; ++j) {
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      wv[k][j] = j < taps ? w[(long long)(c + k) * taps + j] : 0.f;
      win[j][k] = 0.f;
    }
    if (j < hist) {
      const int s = first - hist + j;
      if (s >= 0) ChanIO<T, CH>::load(xc + (long long)s * ld_x, win[j]);
      else ChanIO<float, CH>::load(st + (long long)(hist + s) * width, win[j]);
    }
  }
  if (mode & CA_OUT) {
    float xin[CA_TOKENS][CH];                 // the run's inputs, requested together
#pragma unroll
    for (int i = 0; i < CA_TOKENS; ++i) {
#pragma unroll
      for (int k = 0; k < CH; ++k) xin[i][k] = 0.f;
      if (first + i < last) ChanIO<T, CH>::load(xc + (long long)(first + i) * ld_x, xin[i]);
    }
#pragma unroll
    for (int i = 0; i < CA_TOKENS; ++i) {
      const int t = first + i;
      if (t >= last) break;
      float o[CH];
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        float acc = bv[k];
#pragma unroll
        for (int j = 0; j < MAXT; ++j) {
          const float in = (j == hist) ? xin[i][k] : win[j][k];
          if (j < taps) acc = fmaf(wv[k][j], in, acc);
        }
        o[k] = act == ACT_SILU ? silu_out<T>(acc) : acc;
      }
      ChanIO<T, CH>::store(out + (long long)(begin + t) * ld_out + c, o);
#pragma unroll
      for (int j = 0; j + 1 < MAXT; ++j)
#pragma unroll
        for (int k = 0; k < CH; ++k) win[j][k] = (j + 1 == hist) ? xin[i][k] : win[j + 1][k];
    }
  }
  if ((mode & CA_STATE) && last == count) {
    // new st[s] = input at index count - hist + s; a negative index lies in the old state, at a higher
    // place than the one being written, so ascending order reads before it overwrites
    for (int s = 0; s < hist; ++s) {
      const int idx = count - hist + s;
      float v[CH];
      if (idx >= 0) ChanIO<T, CH>::load(xc + (long long)idx * ld_x, v);
      else ChanIO<float, CH>::load(st + (long long)(hist + idx) * width, v);
      ChanIO<float, CH>::store(st + (long long)s * width, v);
    }
  }
}

template <typename T, int CH>
int launch_conv_act_ch(const void* x, long long ld_x, const float* w, const float* bias, float* state, const int* cu_tokens, const int* slots,
                       void* out, long long ld_out, int requests, int max_new, int width, int taps, int act, int write_state,
                       cudaStream_t stream) {
  const unsigned runs = (unsigned)((max_new + CA_TOKENS - 1) / CA_TOKENS);
  const unsigned cz = (unsigned)((width / CH + CA_THREADS - 1) / CA_THREADS);
  const bool together = write_state && runs == 1 && taps > 1;
  auto kernel = taps <= 4 ? conv_act_kernel<T, CH, 4> : conv_act_kernel<T, CH, CA_MAX_TAPS>;
  hfee_launch(kernel, dim3(runs, requests, cz), dim3(CA_THREADS), 0, stream, (const T*)x, ld_x, w, bias, state, cu_tokens,
              slots, (T*)out, ld_out, width, taps, act, together ? (CA_OUT | CA_STATE) : CA_OUT);
  if (write_state && !together && taps > 1)
    hfee_launch(kernel, dim3(1, requests, cz), dim3(CA_THREADS), 0, stream, (const T*)x, ld_x, w, bias, state, cu_tokens,
                slots, (T*)out, ld_out, width, taps, act, CA_STATE);
  return hfee_check_launch("conv_act");
}

template <typename T>
int launch_conv_act(const void* x, long long ld_x, const float* w, const float* bias, float* state, const int* cu_tokens, const int* slots,
                    void* out, long long ld_out, int requests, int max_new, int width, int taps, int act, int write_state,
                    cudaStream_t stream) {
  const bool pairs = width % 2 == 0 && ld_x % 2 == 0 && ld_out % 2 == 0 && (uintptr_t)x % (2 * sizeof(T)) == 0 &&
                     (uintptr_t)out % (2 * sizeof(T)) == 0 && (uintptr_t)state % 8 == 0;
  if (pairs)
    return launch_conv_act_ch<T, 2>(x, ld_x, w, bias, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, act, write_state, stream);
  return launch_conv_act_ch<T, 1>(x, ld_x, w, bias, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, act, write_state, stream);
}

// ---------------------------------------------------------------------------------------------------------------
constexpr int DR_COLS = 8;                   // columns of the state per block: one warp each
constexpr int DR_THREADS = DR_COLS * 32;
constexpr int DR_TILE = 16;                  // tokens solved at once
constexpr int DR_MAX_DIM = 256;

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct DeltaArgs {
  long long ld_qkv, ld_ba, ld_out;
  int q_off, k_off, v_off;         // columns of head 0 in a row of the q/k/v buffer
  int b_off, a_off;                // columns of head 0's write strength and decay inputs
  int heads, qk_heads, dim, vdim;
  int write_state;
  int vec;                         // rows of q and k can be fetched in 16-byte pieces
};

// A tile's queries and keys on their way from global memory to shared memory: fetched into registers one tile ahead, so
// that the loads are in flight while the tile before is being solved.
template <typename T, int R>
struct TileFetch {
  static constexpr int VEC = 16 / sizeof(T);
  static constexpr int ROW = 32 * R / VEC;                                   // pieces per row of q (or k)
  static constexpr int QK = 2 * DR_TILE * ROW;
  static constexpr int PER = (QK + DR_THREADS - 1) / DR_THREADS;
  uint4 qk[PER];
};
template <typename T> __device__ __forceinline__ void unpack16(const uint4& raw, float* dst);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& raw, float* dst) {
  dst[0] = __uint_as_float(raw.x); dst[1] = __uint_as_float(raw.y); dst[2] = __uint_as_float(raw.z); dst[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& raw, float* dst) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dst[2 * i] = __uint_as_float(w[i] << 16);
    dst[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// R: state entries per lane (dim <= 32 * R).
//
// A tile of up to DR_TILE tokens is solved at once.  With L_t the sum of log g over the tile's tokens up to t and S_0
// the state in front of the tile,
//     u_t = beta_t (v_t - e^{L_t} S_0^T k_t) - sum_{j<t} A[t][j] u_j,      A[t][j] = beta_t e^{L_t - L_j} (k_j . k_t)
//     o_t = e^{L_t} S_0^T q_t + sum_{j<=t} B[t][j] u_j,                    B[t][j] = e^{L_t - L_j} (k_j . q_t)
//     S   = e^{L_last} S_0 + sum_j e^{L_last - L_j} k_j u_j^T
// which is the recurrence written out.  A and B are the same for every column and are computed once per block.  A warp
// owns one column: its lanes share the column's entries, the 32 products S_0^T k_t and S_0^T q_t are reduced across
// the lanes so that lane t ends with the first of token t and lane 16 + t with the second, and one loop over j then
// broadcasts u_j from lane j, lets the lanes below 16 finish their u_t, those above their o_t, and all of them add
// k_j u_j to their entries of S.
template <typename T, int R>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const T* __restrict__ qkv, const T* __restrict__ ba, const float* __restrict__ a_log,
                  const float* __restrict__ dt_bias, float* __restrict__ state, const int* __restrict__ cu_tokens,
                  const int* __restrict__ slots, float* __restrict__ out, DeltaArgs p) {
  constexpr int DP = 32 * R + 1;             // padded key size; odd, so that rows of a tile start in different banks
  extern __shared__ float smem[];
  float* q_s = smem;                         // [DR_TILE][DP]
  float* k_s = q_s + DR_TILE * DP;           // [DR_TILE][DP]
  __shared__ float v_s[DR_TILE][DR_COLS], o_s[DR_TILE][DR_COLS], beta_s[DR_TILE], raw_s[DR_TILE], lg_s[DR_TILE], el_s[DR_TILE],
      er_s[DR_TILE];
  __shared__ float C_s[2 * DR_TILE][DR_TILE + 1];      // rows t: -A[t][.]; rows 16 + t: B[t][.]
  const int req = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * DR_COLS;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col = col0 + warp;
  const int kh = h / (p.heads / p.qk_heads);
  const int dim = p.dim, vdim = p.vdim;
  float* sp = state + (((long long)slot * p.heads + h) * dim) * vdim + col;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    S[r] = (i < dim && col < vdim) ? sp[(long long)i * vdim] : 0.f;
  }
  const float rate = expf(a_log[h]), bias = dt_bias[h];
  const float q_scale = 1.0f / sqrtf((float)dim);
  if (count == 1) {
    // a decoded token: the recurrence itself, every warp on its own (no tables, no barriers)
    const T* row = qkv + (long long)begin * p.ld_qkv + (long long)kh * dim;
    float kk[R], qq[R];
    float sk = 0.f, sq = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = lane + 32 * r;
      kk[r] = i < dim ? to_f32<T>(row[p.k_off + i]) : 0.f;
      qq[r] = i < dim ? to_f32<T>(row[p.q_off + i]) : 0.f;
      sk = fmaf(kk[r], kk[r], sk);
      sq = fmaf(qq[r], qq[r], sq);
    }
    const float k_scale = 1.0f / sqrtf(warp_sum(sk) + 1e-6f), qn_scale = q_scale / sqrtf(warp_sum(sq) + 1e-6f);
    float pk = 0.f, pq = 0.f, kq = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      kk[r] *= k_scale;
      qq[r] *= qn_scale;
      pk = fmaf(S[r], kk[r], pk);
      pq = fmaf(S[r], qq[r], pq);
      kq = fmaf(kk[r], qq[r], kq);
    }
    pk = warp_sum(pk); pq = warp_sum(pq); kq = warp_sum(kq);
    const T* gates = ba + (long long)begin * p.ld_ba;
    const float beta = 1.f / (1.f + expf(-to_f32<T>(gates[p.b_off + h])));
    const float g = expf(-rate * softplus_f32(to_f32<T>(gates[p.a_off + h]) + bias));
    const float v = col < vdim ? to_f32<T>(qkv[(long long)begin * p.ld_qkv + p.v_off + (long long)h * vdim + col]) : 0.f;
    const float u = beta * (v - g * pk);
    if (lane == 0 && col < vdim) out[(long long)begin * p.ld_out + (long long)h * vdim + col] = fmaf(kq, u, g * pq);
    if (p.write_state) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        if (i < dim && col < vdim) sp[(long long)i * vdim] = fmaf(kk[r], u, g * S[r]);
      }
    }
    return;
  }
  using F = TileFetch<T, R>;
  F pf;
  auto fetch = [&](int first) {
    const int rows = min(DR_TILE, count - first);
    const long long at = begin + first;
#pragma unroll
    for (int i = 0; i < F::PER; ++i) {
      const int pi = tid + i * DR_THREADS;
      const int which = pi / (DR_TILE * F::ROW), rem = pi - which * (DR_TILE * F::ROW);
      const int t = rem / F::ROW, c = (rem - t * F::ROW) * F::VEC;
      pf.qk[i] = make_uint4(0u, 0u, 0u, 0u);
      if (pi < F::QK && t < rows && c < dim)
        pf.qk[i] = *reinterpret_cast<const uint4*>(qkv + (at + t) * p.ld_qkv + (which ? p.k_off : p.q_off) + (long long)kh * dim + c);
    }
  };
  if (p.vec) fetch(0);

  for (int tile0 = 0; tile0 < count; tile0 += DR_TILE) {
    const int tt = min(DR_TILE, count - tile0);
    const long long tok0 = begin + tile0;
    if (p.vec) {
      // this tile's queries and keys are in registers already; the next tile's are requested before this one is used
#pragma unroll
      for (int i = 0; i < F::PER; ++i) {
        const int pi = tid + i * DR_THREADS;
        if (pi < F::QK) {
          const int which = pi / (DR_TILE * F::ROW), rem = pi - which * (DR_TILE * F::ROW);
          const int t = rem / F::ROW, c = (rem - t * F::ROW) * F::VEC;
          float vals[F::VEC];
          unpack16<T>(pf.qk[i], vals);
          float* dst = (which ? k_s : q_s) + t * DP + c;
#pragma unroll
          for (int e = 0; e < F::VEC; ++e) dst[e] = vals[e];
        }
      }
      if (tile0 + DR_TILE < count) fetch(tile0 + DR_TILE);
    } else {
      for (int e = tid; e < DR_TILE * DP; e += DR_THREADS) {
        const int t = e / DP, d = e - t * DP;
        const bool in = t < tt && d < dim;
        const T* row = qkv + (tok0 + (in ? t : 0)) * p.ld_qkv + (long long)kh * dim + (in ? d : 0);
        q_s[e] = in ? to_f32<T>(row[p.q_off]) : 0.f;
        k_s[e] = in ? to_f32<T>(row[p.k_off]) : 0.f;
      }
    }
    if (tid < DR_TILE * DR_COLS) {
      const int t = tid / DR_COLS, c = tid - t * DR_COLS;
      v_s[t][c] = (t < tt && col0 + c < vdim) ? to_f32<T>(qkv[(tok0 + t) * p.ld_qkv + p.v_off + (long long)h * vdim + col0 + c]) : 0.f;
    } else if (tid < DR_TILE * DR_COLS + tt) {
      const int t = tid - DR_TILE * DR_COLS;
      const T* row = ba + (tok0 + t) * p.ld_ba;
      beta_s[t] = 1.f / (1.f + expf(-to_f32<T>(row[p.b_off + h])));
      raw_s[t] = -rate * softplus_f32(to_f32<T>(row[p.a_off + h]) + bias);          // log g
    }
    __syncthreads();
    for (int vid = warp; vid < 2 * tt; vid += DR_COLS) {
      float* vec = vid < tt ? q_s + vid * DP : k_s + (vid - tt) * DP;
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(vec[d], vec[d], ss);
      const float scale = (vid < tt ? q_scale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
      for (int d = lane; d < dim; d += 32) vec[d] *= scale;
    }
    if (tid < tt) {                           // L_t, e^{L_t} and e^{L_last - L_t}
      float mine = 0.f, all = 0.f;
      for (int t = 0; t < tt; ++t) {
        all += raw_s[t];
        if (t == tid) mine = all;
      }
      lg_s[tid] = mine;
      el_s[tid] = expf(mine);
      er_s[tid] = expf(all - mine);
    }
    __syncthreads();
    // the tables: thread e takes the pair (t, j) = (e / 16, e % 16) of A, thread 256 + e that of B
    for (int e = tid; e < 2 * DR_TILE * DR_TILE; e += DR_THREADS) {
      const int row = e / DR_TILE, j = e - row * DR_TILE;
      const int t = row & (DR_TILE - 1);
      const bool second = row >= DR_TILE;
      float c = 0.f;
      if (t < tt && (second ? j <= t : j < t)) {
        const float* kj = k_s + j * DP;
        const float* xt = (second ? q_s : k_s) + t * DP;
        float d0 = 0.f, d1 = 0.f;
        int d = 0;
        for (; d + 1 < dim; d += 2) {
          d0 = fmaf(kj[d], xt[d], d0);
          d1 = fmaf(kj[d + 1], xt[d + 1], d1);
        }
        if (d < dim) d0 = fmaf(kj[d], xt[d], d0);
        const float dec = expf(lg_s[t] - lg_s[j]);
        c = second ? dec * (d0 + d1) : -beta_s[t] * dec * (d0 + d1);
      }
      C_s[row][j] = c;
    }
    // S_0^T k_t (values 0..15) and S_0^T q_t (values 16..31) for this column: partial sums per lane, then a
    // reduction across the lanes that leaves value l complete in lane l
    float val[2 * DR_TILE];
#pragma unroll
    for (int t = 0; t < DR_TILE; ++t) {
      float sk = 0.f, sq = 0.f;
      const float* kt = k_s + t * DP + lane;
      const float* qt = q_s + t * DP + lane;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        sk = fmaf(S[r], kt[32 * r], sk);
        sq = fmaf(S[r], qt[32 * r], sq);
      }
      val[t] = sk;
      val[DR_TILE + t] = sq;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < off; ++i) {
        const float send = upper ? val[i] : val[i + off];
        const float keep = upper ? val[i + off] : val[i];
        val[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
    __syncthreads();
    const int t_mine = lane & (DR_TILE - 1);
    float x = 0.f;
    if (t_mine < tt) x = lane < DR_TILE ? beta_s[t_mine] * (v_s[t_mine][warp] - el_s[t_mine] * val[0]) : el_s[t_mine] * val[0];
    const float carry = el_s[tt - 1];
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] *= carry;
#pragma unroll
    for (int j = 0; j < DR_TILE; ++j) {
      if (j < tt) {
        const float uj = __shfl_sync(0xffffffffu, x, j);
        x = fmaf(C_s[lane][j], uj, x);
        const float w = uj * er_s[j];
        const float* kj = k_s + j * DP + lane;
#pragma unroll
        for (int r = 0; r < R; ++r) S[r] = fmaf(kj[32 * r], w, S[r]);
      }
    }
    if (lane >= DR_TILE && t_mine < tt) o_s[t_mine][warp] = x;
    __syncthreads();
    if (tid < tt * DR_COLS) {
      const int t = tid / DR_COLS, c = tid - t * DR_COLS;
      if (col0 + c < vdim) out[(tok0 + t) * p.ld_out + (long long)h * vdim + col0 + c] = o_s[t][c];
    }
  }
  if (p.write_state) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = lane + 32 * r;
      if (i < dim && col < vdim) sp[(long long)i * vdim] = S[r];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same in two kernels, for steps with portions of several tokens: everything that does not depend on the state is
// computed for all tiles at once by `delta_prepare` (unit vectors, beta, the running log-decays and the tables: one
// block per tile and head), and `delta_solve` walks a request's tiles with what is left: the products with S_0, the
// substitution and the update of S.  A tile's place in the workspace is (first token of the tile) / 16 + request, which
// differs for any two tiles of a step.
constexpr int DW_HEAD = 2 * DR_TILE * DR_TILE + 3 * DR_TILE;       // tables, e^L, e^(L_last - L), beta

__host__ __device__ inline int dw_dim(int dim) { return (dim + 3) / 4 * 4; }
__host__ __device__ inline long long dw_qk_floats(int dim) { return 2ll * DR_TILE * dw_dim(dim); }

template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const T* __restrict__ qkv, const T* __restrict__ ba, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, const int* __restrict__ cu_tokens, float* __restrict__ ws_head,
                     float* __restrict__ ws_qk, DeltaArgs p) {
  extern __shared__ float smem[];
  const int dim = p.dim, DP = dim + 1, DPW = dw_dim(dim);
  float* q_s = smem;
  float* k_s = q_s + DR_TILE * DP;
  __shared__ float beta_s[DR_TILE], raw_s[DR_TILE], lg_s[DR_TILE];
  const int req = blockIdx.z, h = blockIdx.y, tile0 = blockIdx.x * DR_TILE;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  pdl_wait();
  pdl_launch_dependents();
  if (tile0 >= count) return;
  const int tt = min(DR_TILE, count - tile0);
  const long long tok0 = begin + tile0;
  const long long place = tok0 / DR_TILE + req;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = p.heads / p.qk_heads, kh = h / group;
  for (int e = tid; e < DR_TILE * DP; e += 128) {
    const int t = e / DP, d = e - t * DP;
    const bool in = t < tt && d < dim;
    const T* row = qkv + (tok0 + (in ? t : 0)) * p.ld_qkv + (long long)kh * dim + (in ? d : 0);
    q_s[e] = in ? to_f32<T>(row[p.q_off]) : 0.f;
    k_s[e] = in ? to_f32<T>(row[p.k_off]) : 0.f;
  }
  if (tid < DR_TILE) {
    float b = 0.f, r = 0.f;
    if (tid < tt) {
      const T* row = ba + (tok0 + tid) * p.ld_ba;
      b = 1.f / (1.f + expf(-to_f32<T>(row[p.b_off + h])));
      r = -expf(a_log[h]) * softplus_f32(to_f32<T>(row[p.a_off + h]) + dt_bias[h]);
    }
    beta_s[tid] = b;
    raw_s[tid] = r;
  }
  __syncthreads();
  const float q_scale = 1.0f / sqrtf((float)dim);
  for (int vid = warp; vid < 2 * tt; vid += 4) {
    float* vec = vid < tt ? q_s + vid * DP : k_s + (vid - tt) * DP;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(vec[d], vec[d], ss);
    const float scale = (vid < tt ? q_scale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
    for (int d = lane; d < dim; d += 32) vec[d] *= scale;
  }
  float* wh = ws_head + (place * p.heads + h) * DW_HEAD;
  if (tid < DR_TILE) {
    float mine = 0.f, all = 0.f;
    for (int t = 0; t < tt; ++t) {
      all += raw_s[t];
      if (t == tid) mine = all;
    }
    lg_s[tid] = mine;
    wh[2 * DR_TILE * DR_TILE + tid] = tid < tt ? expf(mine) : 0.f;
    wh[2 * DR_TILE * DR_TILE + DR_TILE + tid] = tid < tt ? expf(all - mine) : 0.f;
    wh[2 * DR_TILE * DR_TILE + 2 * DR_TILE + tid] = beta_s[tid];
  }
  __syncthreads();
  for (int e = tid; e < 2 * DR_TILE * DR_TILE; e += 128) {
    const int row = e / DR_TILE, j = e - row * DR_TILE;
    const int t = row & (DR_TILE - 1);
    const bool second = row >= DR_TILE;
    float c = 0.f;
    if (t < tt && (second ? j <= t : j < t)) {
      const float* kj = k_s + j * DP;
      const float* xt = (second ? q_s : k_s) + t * DP;
      float d0 = 0.f, d1 = 0.f;
      int d = 0;
      for (; d + 1 < dim; d += 2) {
        d0 = fmaf(kj[d], xt[d], d0);
        d1 = fmaf(kj[d + 1], xt[d + 1], d1);
      }
      if (d < dim) d0 = fmaf(kj[d], xt[d], d0);
      const float dec = expf(lg_s[t] - lg_s[j]);
      c = second ? dec * (d0 + d1) : -beta_s[t] * dec * (d0 + d1);
    }
    wh[e] = c;
  }
  if (h % group == 0) {
    float* wq = ws_qk + (place * p.qk_heads + kh) * dw_qk_floats(dim);
    for (int e = tid; e < DR_TILE * DPW; e += 128) {
      const int t = e / DPW, d = e - t * DPW;
      wq[e] = d < dim ? q_s[t * DP + d] : 0.f;
      wq[DR_TILE * DPW + e] = d < dim ? k_s[t * DP + d] : 0.f;
    }
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(DR_THREADS)
delta_solve_kernel(const T* __restrict__ qkv, const float* __restrict__ ws_head, const float* __restrict__ ws_qk,
                   float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                   float* __restrict__ out, DeltaArgs p) {
  extern __shared__ __align__(16) float smem[];
  const int dim = p.dim, vdim = p.vdim, DPW = dw_dim(dim);
  float* q_s = smem;                         // [DR_TILE][DPW]
  float* k_s = q_s + DR_TILE * DPW;          // [DR_TILE][DPW]
  __shared__ float v_s[DR_TILE][DR_COLS], o_s[DR_TILE][DR_COLS], el_s[DR_TILE], er_s[DR_TILE], beta_s[DR_TILE];
  __shared__ float C_s[2 * DR_TILE][DR_TILE + 1];
  constexpr int PER = (2 * DR_TILE * 32 * R / 4 + DR_THREADS - 1) / DR_THREADS;      // float4 pieces of q and k per thread
  const int req = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * DR_COLS;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col = col0 + warp;
  const int kh = h / (p.heads / p.qk_heads);
  float* sp = state + (((long long)slot * p.heads + h) * dim) * vdim + col;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    S[r] = (i < dim && col < vdim) ? sp[(long long)i * vdim] : 0.f;
  }
  const int qk_pieces = 2 * DR_TILE * DPW / 4;
  float4 pre_qk[PER], pre_head;
  float pre_v;
  auto fetch = [&](int first) {
    const long long tok = begin + first, place = tok / DR_TILE + req;
    const float4* src = reinterpret_cast<const float4*>(ws_qk + (place * p.qk_heads + kh) * dw_qk_floats(dim));
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int pi = tid + i * DR_THREADS;
      pre_qk[i] = pi < qk_pieces ? src[pi] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pre_head = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid < DW_HEAD / 4) pre_head = reinterpret_cast<const float4*>(ws_head + (place * p.heads + h) * DW_HEAD)[tid];
    pre_v = 0.f;
    if (tid < DR_TILE * DR_COLS) {
      const int t = tid / DR_COLS, c = tid - t * DR_COLS;
      if (first + t < count && col0 + c < vdim)
        pre_v = to_f32<T>(qkv[(tok + t) * p.ld_qkv + p.v_off + (long long)h * vdim + col0 + c]);
    }
  };
  fetch(0);
  for (int tile0 = 0; tile0 < count; tile0 += DR_TILE) {
    const int tt = min(DR_TILE, count - tile0);
    const long long tok0 = begin + tile0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int pi = tid + i * DR_THREADS;
      if (pi < qk_pieces) reinterpret_cast<float4*>(q_s)[pi] = pre_qk[i];     // q rows, then k rows, as in the workspace
    }
    if (tid < DW_HEAD / 4) {
      const float vals[4] = {pre_head.x, pre_head.y, pre_head.z, pre_head.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int at = 4 * tid + e;
        if (at < 2 * DR_TILE * DR_TILE) C_s[at / DR_TILE][at % DR_TILE] = vals[e];
        else if (at < 2 * DR_TILE * DR_TILE + DR_TILE) el_s[at - 2 * DR_TILE * DR_TILE] = vals[e];
        else if (at < 2 * DR_TILE * DR_TILE + 2 * DR_TILE) er_s[at - 2 * DR_TILE * DR_TILE - DR_TILE] = vals[e];
        else beta_s[at - 2 * DR_TILE * DR_TILE - 2 * DR_TILE] = vals[e];
      }
    }
    if (tid < DR_TILE * DR_COLS) v_s[tid / DR_COLS][tid % DR_COLS] = pre_v;
    if (tile0 + DR_TILE < count) fetch(tile0 + DR_TILE);
    __syncthreads();
    float val[2 * DR_TILE];
#pragma unroll
    for (int t = 0; t < DR_TILE; ++t) {
      float sk = 0.f, sq = 0.f;
      const float* kt = k_s + t * DPW + lane;
      const float* qt = q_s + t * DPW + lane;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (lane + 32 * r < DPW) {
          sk = fmaf(S[r], kt[32 * r], sk);
          sq = fmaf(S[r], qt[32 * r], sq);
        }
      }
      val[t] = sk;
      val[DR_TILE + t] = sq;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < off; ++i) {
        const float send = upper ? val[i] : val[i + off];
        const float keep = upper ? val[i + off] : val[i];
        val[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
    const int t_mine = lane & (DR_TILE - 1);
    float x = 0.f;
    if (t_mine < tt) x = lane < DR_TILE ? beta_s[t_mine] * (v_s[t_mine][warp] - el_s[t_mine] * val[0]) : el_s[t_mine] * val[0];
    const float carry = el_s[tt - 1];
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] *= carry;
#pragma unroll
    for (int j = 0; j < DR_TILE; ++j) {
      if (j < tt) {
        const float uj = __shfl_sync(0xffffffffu, x, j);
        x = fmaf(C_s[lane][j], uj, x);
        const float w = uj * er_s[j];
        const float* kj = k_s + j * DPW + lane;
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (lane + 32 * r < DPW) S[r] = fmaf(kj[32 * r], w, S[r]);
      }
    }
    if (lane >= DR_TILE && t_mine < tt) o_s[t_mine][warp] = x;
    __syncthreads();
    if (tid < tt * DR_COLS) {
      const int t = tid / DR_COLS, c = tid - t * DR_COLS;
      if (col0 + c < vdim) out[(tok0 + t) * p.ld_out + (long long)h * vdim + col0 + c] = o_s[t][c];
    }
  }
  if (p.write_state) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = lane + 32 * r;
      if (i < dim && col < vdim) sp[(long long)i * vdim] = S[r];
    }
  }
}

template <typename T, int R>
int launch_solve_r(const void* qkv, const float* ws_head, const float* ws_qk, float* state, const int* cu_tokens,
                   const int* slots, float* out, const DeltaArgs& p, int requests, cudaStream_t stream) {
  const size_t smem = (size_t)2 * DR_TILE * dw_dim(p.dim) * sizeof(float);
  hfee_launch(delta_solve_kernel<T, R>, dim3((unsigned)((p.vdim + DR_COLS - 1) / DR_COLS), (unsigned)p.heads, (unsigned)requests),
              dim3(DR_THREADS), smem, stream, (const T*)qkv, ws_head, ws_qk, state, cu_tokens, slots, out, p);
  return hfee_check_launch("delta_solve");
}

template <typename T>
int launch_prepared(const void* qkv, const void* ba, const float* a_log, const float* dt_bias, float* state,
                    const int* cu_tokens, const int* slots, float* out, const DeltaArgs& p, int requests, int max_new,
                    float* ws_head, float* ws_qk, cudaStream_t stream) {
  const size_t smem = (size_t)2 * DR_TILE * (p.dim + 1) * sizeof(float);
  hfee_launch(delta_prepare_kernel<T>, dim3((unsigned)((max_new + DR_TILE - 1) / DR_TILE), (unsigned)p.heads, (unsigned)requests),
              dim3(128), smem, stream, (const T*)qkv, (const T*)ba, a_log, dt_bias, cu_tokens, ws_head, ws_qk, p);
  int rc = hfee_check_launch("delta_prepare");
  if (rc != HFEE_OK) return rc;
  const int r = (p.dim + 31) / 32;
  if (r <= 1) return launch_solve_r<T, 1>(qkv, ws_head, ws_qk, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 2) return launch_solve_r<T, 2>(qkv, ws_head, ws_qk, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 4) return launch_solve_r<T, 4>(qkv, ws_head, ws_qk, state, cu_tokens, slots, out, p, requests, stream);
  return launch_solve_r<T, 8>(qkv, ws_head, ws_qk, state, cu_tokens, slots, out, p, requests, stream);
}

template <typename T, int R>
int launch_delta_r(const void* qkv, const void* ba, const float* a_log, const float* dt_bias, float* state,
                   const int* cu_tokens, const int* slots, float* out, const DeltaArgs& p, int requests, cudaStream_t stream) {
  const size_t smem = (size_t)2 * DR_TILE * (32 * R + 1) * sizeof(float);
  hfee_launch(delta_rule_kernel<T, R>, dim3((unsigned)((p.vdim + DR_COLS - 1) / DR_COLS), (unsigned)p.heads, (unsigned)requests),
              dim3(DR_THREADS), smem, stream, (const T*)qkv, (const T*)ba, a_log, dt_bias, state, cu_tokens, slots, out, p);
  return hfee_check_launch("delta_rule");
}

template <typename T>
int launch_delta(const void* qkv, const void* ba, const float* a_log, const float* dt_bias, float* state,
                 const int* cu_tokens, const int* slots, float* out, const DeltaArgs& p, int requests, cudaStream_t stream) {
  const int r = (p.dim + 31) / 32;
  if (r <= 1) return launch_delta_r<T, 1>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 2) return launch_delta_r<T, 2>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 4) return launch_delta_r<T, 4>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  return launch_delta_r<T, 8>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
}

}  // namespace

// Launches one kernel, or two when a portion is longer than one run of tokens and the state is written.
HFEE_API int hfee_conv_act_launches(int max_new, int taps, int write_state) {
  return (write_state && taps > 1 && max_new > CA_TOKENS) ? 2 : 1;
}

// act: 0 none, 1 SiLU.  state: [slots, taps - 1, width] float32.  bias: [width] added in front of the activation, or null.
HFEE_API int hfee_conv_act(const void* x, long long ld_x, int dtype, const float* w, const float* bias, float* state, const int* cu_tokens,
                           const int* slots, void* out, long long ld_out, int requests, int max_new, int width, int taps,
                           int act, int write_state, cudaStream_t stream) {
  if (requests == 0 || max_new == 0) return HFEE_OK;
  HFEE_REQUIRE(requests > 0 && max_new > 0 && width > 0, "conv_act: bad sizes");
  HFEE_REQUIRE(taps >= 1 && taps <= CA_MAX_TAPS, "conv_act: taps %d is outside 1..%d", taps, CA_MAX_TAPS);
  HFEE_REQUIRE(ld_x >= width && ld_out >= width, "conv_act: a row stride is too small");
  HFEE_REQUIRE(act == ACT_NONE || act == ACT_SILU, "conv_act: unknown activation %d", act);
  if (dtype == HFEE_F32)
    return launch_conv_act<float>(x, ld_x, w, bias, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, act, write_state, stream);
  if (dtype == HFEE_BF16)
    return launch_conv_act<__nv_bfloat16>(x, ld_x, w, bias, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, act, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "conv_act: unknown dtype %d", dtype);
}

// Floats of workspace the two-kernel form needs for a step of n_tokens tokens in `requests` requests.
HFEE_API long long hfee_delta_rule_workspace(int requests, int n_tokens, int heads, int qk_heads, int dim) {
  const long long places = n_tokens / DR_TILE + requests + 1;
  return places * ((long long)heads * DW_HEAD + (long long)qk_heads * dw_qk_floats(dim));
}

// With a workspace (see hfee_delta_rule_workspace) and a portion of more than one token in the step (max_new > 1), the
// step runs as two kernels (delta_prepare, delta_solve); else as one.
// qkv rows: head g's query at q_off + g * dim, its key at k_off + g * dim (g < qk_heads; head h of `heads` uses
// g = h / (heads / qk_heads)), head h's value at v_off + h * vdim.  ba rows: b_off + h and a_off + h.
// state: [slots, heads, dim, vdim] float32.  out: float32 [n, heads * vdim].
HFEE_API int hfee_delta_rule(const void* qkv, long long ld_qkv, int q_off, int k_off, int v_off, const void* ba,
                             long long ld_ba, int b_off, int a_off, int dtype, const float* a_log, const float* dt_bias,
                             float* state, const int* cu_tokens, const int* slots, float* out, long long ld_out,
                             int requests, int heads, int qk_heads, int dim, int vdim, int write_state, int n_tokens,
                             int max_new, float* workspace, long long workspace_floats, cudaStream_t stream) {
  if (requests == 0) return HFEE_OK;
  HFEE_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0, "delta_rule: heads %d must be a multiple of %d", heads, qk_heads);
  HFEE_REQUIRE(dim > 0 && dim <= DR_MAX_DIM && vdim > 0, "delta_rule: key size %d is outside 1..%d", dim, DR_MAX_DIM);
  const int vec_elems = dtype == HFEE_F32 ? 4 : 8;
  const int vec = dim % vec_elems == 0 && ld_qkv % vec_elems == 0 && q_off % vec_elems == 0 && k_off % vec_elems == 0 &&
                  (uintptr_t)qkv % 16 == 0;
  DeltaArgs p{ld_qkv, ld_ba, ld_out, q_off, k_off, v_off, b_off, a_off, heads, qk_heads, dim, vdim, write_state, vec};
  if (workspace != nullptr && max_new > 1) {
    // portions of several tokens: the state-independent part of every tile first, in parallel
    HFEE_REQUIRE(workspace_floats >= hfee_delta_rule_workspace(requests, n_tokens, heads, qk_heads, dim) && (uintptr_t)workspace % 16 == 0,
                 "delta_rule: the workspace is too small or not 16-byte aligned");
    const long long places = n_tokens / DR_TILE + requests + 1;
    float* ws_head = workspace;
    float* ws_qk = workspace + places * heads * DW_HEAD;
    if (dtype == HFEE_F32)
      return launch_prepared<float>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, max_new, ws_head, ws_qk, stream);
    if (dtype == HFEE_BF16)
      return launch_prepared<__nv_bfloat16>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, max_new, ws_head, ws_qk, stream);
    return hfee_fail(HFEE_ERR_ARG, "delta_rule: unknown dtype %d", dtype);
  }
  if (dtype == HFEE_F32)
    return launch_delta<float>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (dtype == HFEE_BF16)
    return launch_delta<__nv_bfloat16>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  return hfee_fail(HFEE_ERR_ARG, "delta_rule: unknown dtype %d", dtype);
}
