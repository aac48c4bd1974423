// Linear attention whose matrix state is gated by the token, with a float32 state per (request, head):
//
//   channel decay      S_t = diag(a_t) S_(t-1) + k_t v_t^T            a_t = sigmoid(z_t)^(1/tau) per key channel
//                      o_t = S_t^T q_t
//
//   exponential gates  m_t = max(f_t + m_(t-1), i_t)                  i_t = cap tanh(x_i / cap), f_t = logsigmoid(cap tanh(x_f / cap))
//                      S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T          (n_t the same with k_t alone)
//                      o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
//
// S: [dim][vdim], n: [dim], m: one number; all zero for a fresh request.  q (times q_scale), k and v are slices of one
// projection buffer (type T); the gates' pre-activations z, x_i, x_f are float32, and so are the decays, their
// logarithms and exponentials, the states, every product and o.
//
// hfee_gated_recurrence walks a request's tokens one after the other.  A thread keeps GR_ROWS rows
// of two state columns in registers (a staged q, k or decay is read from shared memory once for both); a warp covers
// GR_COLS = 64 columns of those rows, a block all rows (blockDim.y row groups whose partial outputs meet in shared
// memory in a fixed order) of 64 columns; blockIdx = (head, request, column tile).
// Lane j of row group g also keeps n[g * 32 + j].  Tokens are staged GR_STAGE at a time; the scalar recurrence of
// the running maximum is walked by one thread per stage.  The order of the sums does not depend on how a prompt was
// cut, and a state is what the tokens before left, so neither does a position's output.
//
// hfee_gated_recurrence_chunked is the prompt path: both recurrences are linear in the state once the gates are known,
// S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T, so runs of GC_T tokens work side by side.  (0, exponential gates only) one warp
// per (request, head) computes every token's (a_t, b_t, e^(-m_t)) with a warp scan over the maps m -> max(m + f, i),
// which compose; (1) every run walks its tokens from a zero state and leaves its sum and the product of its decays; (2)
// per (request, head) the states in front of every run, in order, and the request's new state; (3) every run walks its
// tokens again from the state in front of it and writes the outputs.  The same recurrence in another association.
#include "common.cuh"

namespace {

constexpr int GR_ROWS = 32;
constexpr int GR_LANES = 32;         // threads of a row group: one warp
constexpr int GR_NC = 2;             // state columns per thread (lane j: columns j and j + 32 of the block's 64)
constexpr int GR_COLS = GR_LANES * GR_NC;
constexpr int GR_STAGE = 8;
constexpr int GR_MAX_DIM = 256;
constexpr int GC_T = 64;             // tokens of a run of the chunked path
enum Pass { PASS_WHOLE = 0, PASS_LOCAL = 1, PASS_OUT = 2 };

enum Mode { MODE_CHANNEL_DECAY = 0, MODE_EXP_GATES = 1 };

__device__ __forceinline__ float log_sigmoid_f32(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

struct RecurrenceArgs {
  long long ld;                 // of q, k, v
  const float* pre;             // channel decay: z [n, heads * dim]; exponential gates: [n, 2 * heads] = x_i then x_f
  long long ld_pre;
  const float* bias;            // added to `pre` column by column; may be null
  float p0;                     // channel decay: 1 / tau; exponential gates: cap
  float q_scale;
  float* state;                 // [slots, heads, dim, vdim]
  float* norm_state;            // [slots, heads, dim]       (exponential gates)
  float* max_state;             // [slots, heads]            (exponential gates)
  const int* cu_tokens;
  const int* slots;
  float* out;
  long long ld_o;
  int heads, dim, vdim, write_state;
  // chunked path: the runs of all requests are numbered in batch order
  int requests;
  float* run_state;             // [runs, heads, dim, vdim]: a run's own sum (pass 1), then the state in front of it (pass 2)
  float* run_norm;              // [runs, heads, dim]        the same for n (exponential gates)
  float* run_decay;             // [runs, heads, dim]        product of the run's decays per key channel
  const float* gates;           // [3][n_tokens, heads]: a_t, b_t, e^(-m_t) (exponential gates)
  long long gate_stride;        // n_tokens * heads
  int decays_given;             // channel decay: `pre` holds the decays themselves (the chunked path computes them once)
};

__device__ __forceinline__ int runs_of(int count) { return (count + GC_T - 1) / GC_T; }

// (request, run within it) of run `number`; false if there is no such run
__device__ __forceinline__ bool find_run(const int* __restrict__ cu_tokens, int requests, int number, int* req, int* run) {
  int base = 0;
  for (int r = 0; r < requests; ++r) {
    const int c = runs_of(cu_tokens[r + 1] - cu_tokens[r]);
    if (number < base + c) { *req = r; *run = number - base; return true; }
    base += c;
  }
  return false;
}

template <typename T, int MODE, int PASS>
__global__ void __launch_bounds__(GR_LANES * (GR_MAX_DIM / GR_ROWS), 2)
gated_recurrence_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, RecurrenceArgs p) {
  extern __shared__ __align__(16) float smem[];
  __shared__ float a_s[GR_STAGE], b_s[GR_STAGE], em_s[GR_STAGE];
  __shared__ float m_cur;
  const int head = blockIdx.x;
  int req = blockIdx.y, run = 0;
  if constexpr (PASS != PASS_WHOLE) {
    if (!find_run(p.cu_tokens, p.requests, blockIdx.y, &req, &run)) return;
  }
  const int groups = blockDim.y, dim_pad = groups * GR_ROWS;
  const int j = threadIdx.x, g = threadIdx.y;
  const int col = blockIdx.z * GR_COLS + j;            // and col + 32
  const int tid = g * GR_LANES + j, threads = GR_LANES * groups;
  const int heads = p.heads, dim = p.dim, vdim = p.vdim;
  float* qs = smem;                                   // [GR_STAGE][dim_pad]
  float* ks = qs + GR_STAGE * dim_pad;                // [GR_STAGE][dim_pad]
  float* vs = ks + GR_STAGE * dim_pad;                // [GR_STAGE][GR_COLS]
  float* part = vs + GR_STAGE * GR_COLS;              // [GR_STAGE][groups][GR_COLS]
  float* part_n = part + GR_STAGE * groups * GR_COLS; // [GR_STAGE][groups]
  float* as = part_n + GR_STAGE * groups;             // [GR_STAGE][dim_pad]   (channel decay)
  int begin = p.cu_tokens[req], count = p.cu_tokens[req + 1] - begin;
  if constexpr (PASS != PASS_WHOLE) {
    begin += run * GC_T;
    count = min(GC_T, count - run * GC_T);
  }
  const int slot = p.slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;

  // where the state comes from and goes to: the request's slot, or the run's place in the workspace
  const long long place = PASS == PASS_WHOLE ? (long long)slot * heads + head : (long long)blockIdx.y * heads + head;
  float* S_g = (PASS == PASS_WHOLE ? p.state : p.run_state) + (place * dim) * vdim;
  float* n_g = (PASS == PASS_WHOLE ? p.norm_state : p.run_norm) + place * dim;
  float S[GR_NC][GR_ROWS];
#pragma unroll
  for (int c = 0; c < GR_NC; ++c)
#pragma unroll
    for (int i = 0; i < GR_ROWS; ++i) {
      const int row = g * GR_ROWS + i;
      S[c][i] = (PASS != PASS_LOCAL && row < dim && col + c * GR_LANES < vdim) ? S_g[(long long)row * vdim + col + c * GR_LANES] : 0.f;
    }
  float n_own = 0.f;                                  // n[g * GR_ROWS + j]
  float decay_own = 1.f;                              // PASS_LOCAL: product of the run's decays of that row
  const int own_row = g * GR_ROWS + j;
  if constexpr (MODE == MODE_EXP_GATES) {
    if (PASS != PASS_LOCAL && own_row < dim) n_own = n_g[own_row];
    if (PASS == PASS_WHOLE && tid == 0) m_cur = p.max_state[(long long)slot * heads + head];
  }
  // A block has as many threads as a staged token has (padded) key channels: thread `tid` brings channel `tid` of every
  // token of a stage, and its share of the stage's values.
  const bool live_d = tid < dim;
  const int chan = head * dim + tid;
  const float z_bias = (MODE == MODE_CHANNEL_DECAY && live_d && !p.decays_given && p.bias != nullptr) ? p.bias[chan] : 0.f;
  for (int t0 = 0; t0 < count; t0 += GR_STAGE) {
    const int nt = min(GR_STAGE, count - t0);
    __syncthreads();                                  // the stage before is used up
#pragma unroll
    for (int t = 0; t < GR_STAGE; ++t) {
      if (t < nt) {
        const int e = t * dim_pad + tid;
        const long long at = (long long)(begin + t0 + t) * p.ld + chan;
        qs[e] = live_d ? to_f32<T>(q[at]) * p.q_scale : 0.f;
        ks[e] = live_d ? to_f32<T>(k[at]) : 0.f;
        if constexpr (MODE == MODE_CHANNEL_DECAY) {    // a decay, or the gate's pre-activation it comes from
          float a = 1.f;
          if (live_d) {
            a = p.pre[(long long)(begin + t0 + t) * p.ld_pre + chan];
            if (!p.decays_given) a = expf(log_sigmoid_f32(a + z_bias) * p.p0);
          }
          as[e] = a;
        }
      }
    }
    for (int e = tid; e < nt * GR_COLS; e += threads) {
      const int t = e / GR_COLS, c = blockIdx.z * GR_COLS + e % GR_COLS;
      vs[e] = c < vdim ? to_f32<T>(v[(long long)(begin + t0 + t) * p.ld + (long long)head * vdim + c]) : 0.f;
    }
    if constexpr (MODE == MODE_EXP_GATES && PASS != PASS_WHOLE) {
      if (tid < nt) {                                 // the gates were computed for every token beforehand
        const long long at = (long long)(begin + t0 + tid) * heads + head;
        a_s[tid] = p.gates[at];
        b_s[tid] = p.gates[p.gate_stride + at];
        em_s[tid] = p.gates[2 * p.gate_stride + at];
      }
    }
    if constexpr (MODE == MODE_EXP_GATES && PASS == PASS_WHOLE) {
      if (tid == 0) {
        float m = m_cur;
        const float cap = p.p0;
        for (int t = 0; t < nt; ++t) {
          const float* pre = p.pre + (long long)(begin + t0 + t) * p.ld_pre;
          const float xi = pre[head] + (p.bias != nullptr ? p.bias[head] : 0.f);
          const float xf = pre[heads + head] + (p.bias != nullptr ? p.bias[heads + head] : 0.f);
          const float ig = cap * tanhf(xi / cap);
          const float fg = log_sigmoid_f32(cap * tanhf(xf / cap));
          const float m_new = fmaxf(fg + m, ig);
          a_s[t] = expf(fg + m - m_new);
          b_s[t] = expf(ig - m_new);
          em_s[t] = expf(-m_new);
          m = m_new;
        }
        m_cur = m;
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float vv = vs[t * GR_COLS + j], vw = vs[t * GR_COLS + GR_LANES + j];
      const float4* k4 = reinterpret_cast<const float4*>(ks + t * dim_pad + g * GR_ROWS);
      const float4* q4 = reinterpret_cast<const float4*>(qs + t * dim_pad + g * GR_ROWS);
      float acc = 0.f, acd = 0.f;
      if constexpr (MODE == MODE_CHANNEL_DECAY) {
        const float4* a4 = reinterpret_cast<const float4*>(as + t * dim_pad + g * GR_ROWS);
#pragma unroll
        for (int i = 0; i < GR_ROWS / 4; ++i) {
          const float4 kk = k4[i], qq = q4[i], aa = a4[i];
          S[0][4 * i + 0] = fmaf(aa.x, S[0][4 * i + 0], kk.x * vv);  acc = fmaf(S[0][4 * i + 0], qq.x, acc);
          S[0][4 * i + 1] = fmaf(aa.y, S[0][4 * i + 1], kk.y * vv);  acc = fmaf(S[0][4 * i + 1], qq.y, acc);
          S[0][4 * i + 2] = fmaf(aa.z, S[0][4 * i + 2], kk.z * vv);  acc = fmaf(S[0][4 * i + 2], qq.z, acc);
          S[0][4 * i + 3] = fmaf(aa.w, S[0][4 * i + 3], kk.w * vv);  acc = fmaf(S[0][4 * i + 3], qq.w, acc);
          S[1][4 * i + 0] = fmaf(aa.x, S[1][4 * i + 0], kk.x * vw);  acd = fmaf(S[1][4 * i + 0], qq.x, acd);
          S[1][4 * i + 1] = fmaf(aa.y, S[1][4 * i + 1], kk.y * vw);  acd = fmaf(S[1][4 * i + 1], qq.y, acd);
          S[1][4 * i + 2] = fmaf(aa.z, S[1][4 * i + 2], kk.z * vw);  acd = fmaf(S[1][4 * i + 2], qq.z, acd);
          S[1][4 * i + 3] = fmaf(aa.w, S[1][4 * i + 3], kk.w * vw);  acd = fmaf(S[1][4 * i + 3], qq.w, acd);
        }
        if constexpr (PASS == PASS_LOCAL) decay_own *= as[t * dim_pad + own_row];
      } else {
        const float a = a_s[t], bv = b_s[t] * vv, bw = b_s[t] * vw;
#pragma unroll
        for (int i = 0; i < GR_ROWS / 4; ++i) {
          const float4 kk = k4[i], qq = q4[i];
          S[0][4 * i + 0] = fmaf(a, S[0][4 * i + 0], kk.x * bv);  acc = fmaf(S[0][4 * i + 0], qq.x, acc);
          S[0][4 * i + 1] = fmaf(a, S[0][4 * i + 1], kk.y * bv);  acc = fmaf(S[0][4 * i + 1], qq.y, acc);
          S[0][4 * i + 2] = fmaf(a, S[0][4 * i + 2], kk.z * bv);  acc = fmaf(S[0][4 * i + 2], qq.z, acc);
          S[0][4 * i + 3] = fmaf(a, S[0][4 * i + 3], kk.w * bv);  acc = fmaf(S[0][4 * i + 3], qq.w, acc);
          S[1][4 * i + 0] = fmaf(a, S[1][4 * i + 0], kk.x * bw);  acd = fmaf(S[1][4 * i + 0], qq.x, acd);
          S[1][4 * i + 1] = fmaf(a, S[1][4 * i + 1], kk.y * bw);  acd = fmaf(S[1][4 * i + 1], qq.y, acd);
          S[1][4 * i + 2] = fmaf(a, S[1][4 * i + 2], kk.z * bw);  acd = fmaf(S[1][4 * i + 2], qq.z, acd);
          S[1][4 * i + 3] = fmaf(a, S[1][4 * i + 3], kk.w * bw);  acd = fmaf(S[1][4 * i + 3], qq.w, acd);
        }
        n_own = fmaf(a, n_own, b_s[t] * ks[t * dim_pad + own_row]);
        if constexpr (PASS == PASS_LOCAL) decay_own *= a;
        if constexpr (PASS != PASS_LOCAL) {
          const float nq = warp_sum(n_own * qs[t * dim_pad + own_row]);
          if (j == 0) part_n[t * groups + g] = nq;
        }
      }
      if constexpr (PASS != PASS_LOCAL) {
        part[(t * groups + g) * GR_COLS + j] = acc;
        part[(t * groups + g) * GR_COLS + GR_LANES + j] = acd;
      }
    }
    if constexpr (PASS == PASS_LOCAL) continue;       // a run's own sum: no outputs
    __syncthreads();
    for (int e = tid; e < nt * GR_COLS; e += threads) {
      const int t = e / GR_COLS, jj = e % GR_COLS, c = blockIdx.z * GR_COLS + jj;
      float sum = 0.f;
      for (int gg = 0; gg < groups; ++gg) sum += part[(t * groups + gg) * GR_COLS + jj];
      if constexpr (MODE == MODE_EXP_GATES) {
        float nq = 0.f;
        for (int gg = 0; gg < groups; ++gg) nq += part_n[t * groups + gg];
        sum /= fmaxf(fabsf(nq), em_s[t]) + 1e-6f;
      }
      if (c < vdim) p.out[(long long)(begin + t0 + t) * p.ld_o + (long long)head * vdim + c] = sum;
    }
  }
  if constexpr (PASS == PASS_OUT) return;
  if (PASS == PASS_LOCAL || p.write_state) {
#pragma unroll
    for (int c = 0; c < GR_NC; ++c)
#pragma unroll
      for (int i = 0; i < GR_ROWS; ++i) {
        const int row = g * GR_ROWS + i;
        if (row < dim && col + c * GR_LANES < vdim) S_g[(long long)row * vdim + col + c * GR_LANES] = S[c][i];
      }
    if (blockIdx.z == 0) {
      if constexpr (MODE == MODE_EXP_GATES) {
        if (own_row < dim) n_g[own_row] = n_own;
        if (PASS == PASS_WHOLE && tid == 0) p.max_state[(long long)slot * heads + head] = m_cur;
      }
      if constexpr (PASS == PASS_LOCAL) {
        if (own_row < dim) p.run_decay[place * dim + own_row] = decay_own;
      }
    }
  }
}

// pre[t, c] <- sigmoid(pre[t, c] + bias[c])^p0: every token's decays, once for all passes and column tiles.
__global__ void __launch_bounds__(256)
channel_decays_kernel(float* __restrict__ pre, long long ld_pre, const float* __restrict__ bias, float p0, int cols, long long total) {
  pdl_wait();
  pdl_launch_dependents();
  const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
  if (e >= total) return;
  const long long r = e / cols;
  const int c = (int)(e - r * cols);
  float* at = pre + r * ld_pre + c;
  *at = expf(log_sigmoid_f32(*at + (bias != nullptr ? bias[c] : 0.f)) * p0);
}

// Every token's gates of the exponential recurrence, one warp per (request, head).  The running maximum is the map
// m -> max(m + f_t, i_t) applied token after token; two such maps compose to one of the same form, (f, i) then (f', i')
// = (f + f', max(i + f', i')), so a warp scans 32 tokens at a time.
__global__ void __launch_bounds__(128)
memory_gates_kernel(const float* __restrict__ pre, long long ld_pre, const float* __restrict__ bias, float cap,
                    float* __restrict__ max_state, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int requests,
                    int heads, float* __restrict__ gates, long long gate_stride, int write_state) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int task = blockIdx.x * 4 + warp;
  if (task >= requests * heads) return;
  const int req = task / heads, head = task - req * heads;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;
  float m = max_state[(long long)slot * heads + head];
  const float bi = bias != nullptr ? bias[head] : 0.f, bf = bias != nullptr ? bias[heads + head] : 0.f;
  constexpr int AHEAD = 4;                             // groups of 32 tokens whose pre-activations are requested together
  float xi[AHEAD], xf[AHEAD];
  for (int t0 = 0; t0 < count; t0 += 32) {
    const int t = t0 + lane;
    const bool live = t < count;
    const int u = (t0 / 32) % AHEAD;
    if (u == 0) {
#pragma unroll
      for (int i = 0; i < AHEAD; ++i) {
        const int ti = t + 32 * i;
        const float* row = pre + (long long)(begin + min(ti, count - 1)) * ld_pre;
        xi[i] = row[head];
        xf[i] = row[heads + head];
      }
    }
    float ig = -INFINITY, fg = 0.f;                    // a dead lane is the identity map
    if (live) {
      float vi = xi[0], vf = xf[0];
#pragma unroll
      for (int i = 1; i < AHEAD; ++i)
        if (u == i) { vi = xi[i]; vf = xf[i]; }
      ig = cap * tanhf((vi + bi) / cap);
      fg = log_sigmoid_f32(cap * tanhf((vf + bf) / cap));
    }
    float F = fg, I = ig;                              // the maps of tokens t0 .. t composed
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) { I = fmaxf(Ip + F, I); F = Fp + F; }
    }
    const float m_t = fmaxf(m + F, I);
    float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
    if (lane == 0) m_prev = m;
    if (live) {
      const long long at = (long long)(begin + t) * heads + head;
      gates[at] = expf(fg + m_prev - m_t);
      gates[gate_stride + at] = expf(ig - m_t);
      gates[2 * gate_stride + at] = expf(-m_t);
    }
    m = __shfl_sync(0xffffffffu, m_t, min(31, count - 1 - t0));
  }
  if (write_state && lane == 0) max_state[(long long)slot * heads + head] = m;
}

// The states in front of every run of a request, in order: run_state[run] holds the run's own sum on entry and the
// state in front of the run on exit; the request's state moves to behind its last run.  One thread per state element.
__global__ void __launch_bounds__(256)
recurrence_carry_kernel(RecurrenceArgs p, int with_norm) {
  const int head = blockIdx.x, req = blockIdx.y;
  const int count = p.cu_tokens[req + 1] - p.cu_tokens[req];
  const int slot = p.slots[req];
  int first = 0;
  for (int r = 0; r < req; ++r) first += runs_of(p.cu_tokens[r + 1] - p.cu_tokens[r]);
  const int runs = runs_of(count);
  pdl_wait();
  pdl_launch_dependents();
  const long long elements = (long long)p.dim * p.vdim;
  const long long e = (long long)blockIdx.z * 256 + threadIdx.x;
  if (e < elements) {
    const int row = (int)(e / p.vdim);
    float* S_g = p.state + ((long long)slot * p.heads + head) * elements + e;
    float S = *S_g;
    for (int c0 = 0; c0 < runs; c0 += 8) {              // eight runs' sums and decays are requested together
      float own[8], dec[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const long long place = (long long)(first + min(c0 + i, runs - 1)) * p.heads + head;
        own[i] = p.run_state[place * elements + e];
        dec[i] = p.run_decay[place * p.dim + row];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (c0 + i < runs) {
          p.run_state[((long long)(first + c0 + i) * p.heads + head) * elements + e] = S;
          S = fmaf(dec[i], S, own[i]);
        }
      }
    }
    if (p.write_state && runs > 0) *S_g = S;
  }
  if (with_norm && e < p.dim) {
    float* n_g = p.norm_state + ((long long)slot * p.heads + head) * p.dim + e;
    float nv = *n_g;
    for (int c = 0; c < runs; ++c) {
      const long long place = (long long)(first + c) * p.heads + head;
      float* w = p.run_norm + place * p.dim + e;
      const float own = *w;
      *w = nv;
      nv = fmaf(p.run_decay[place * p.dim + e], nv, own);
    }
    if (p.write_state && runs > 0) *n_g = nv;
  }
}

template <typename T, int PASS>
int launch_recurrence(int mode, const void* q, const void* k, const void* v, const RecurrenceArgs& p, int grid_y,
                      cudaStream_t stream) {
  const int groups = (p.dim + GR_ROWS - 1) / GR_ROWS, dim_pad = groups * GR_ROWS;
  const dim3 grid(p.heads, grid_y, (p.vdim + GR_COLS - 1) / GR_COLS), block(GR_LANES, groups);
  size_t floats = (size_t)GR_STAGE * (2 * dim_pad + GR_COLS + groups * GR_COLS + groups);
  if (mode == MODE_CHANNEL_DECAY) floats += (size_t)GR_STAGE * dim_pad;
  const size_t smem = floats * sizeof(float);
  if (mode == MODE_CHANNEL_DECAY)
    hfee_launch(gated_recurrence_kernel<T, MODE_CHANNEL_DECAY, PASS>, grid, block, smem, stream, (const T*)q, (const T*)k, (const T*)v, p);
  else
    hfee_launch(gated_recurrence_kernel<T, MODE_EXP_GATES, PASS>, grid, block, smem, stream, (const T*)q, (const T*)k, (const T*)v, p);
  return hfee_check_launch("gated_recurrence");
}

template <typename T>
int launch_chunked(int mode, const void* q, const void* k, const void* v, RecurrenceArgs p, const float* pre, long long ld_pre,
                   const float* bias, float cap, int n_tokens, int max_runs, cudaStream_t stream) {
  if (mode == MODE_CHANNEL_DECAY) {                  // `pre` is scratch of the caller's: the decays take the gates' place
    const int cols = p.heads * p.dim;
    const long long total = (long long)n_tokens * cols;
    hfee_launch(channel_decays_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (float*)pre, ld_pre, bias, p.p0, cols, total);
    int rc = hfee_check_launch("channel_decays");
    if (rc != HFEE_OK) return rc;
    p.decays_given = 1;
  }
  if (mode == MODE_EXP_GATES) {
    hfee_launch(memory_gates_kernel, dim3((p.requests * p.heads + 3) / 4), dim3(128), 0, stream, pre, ld_pre, bias, cap, p.max_state,
                p.cu_tokens, p.slots, p.requests, p.heads, (float*)p.gates, p.gate_stride, p.write_state);
    int rc = hfee_check_launch("memory_gates");
    if (rc != HFEE_OK) return rc;
  }
  int rc = launch_recurrence<T, PASS_LOCAL>(mode, q, k, v, p, max_runs, stream);
  if (rc != HFEE_OK) return rc;
  const long long elements = (long long)p.dim * p.vdim;
  hfee_launch(recurrence_carry_kernel, dim3(p.heads, p.requests, (unsigned)((elements + 255) / 256)), dim3(256), 0, stream, p,
              mode == MODE_EXP_GATES ? 1 : 0);
  rc = hfee_check_launch("recurrence_carry");
  if (rc != HFEE_OK) return rc;
  return launch_recurrence<T, PASS_OUT>(mode, q, k, v, p, max_runs, stream);
}

}  // namespace

// mode 0 (channel decay): pre = z [n, heads * dim] float32 (+ bias [heads * dim] or null), p0 = 1 / tau; norm_state and
// max_state are unused.  mode 1 (exponential gates): pre [n, 2 * heads] float32 = the input gates' pre-activations, then
// the forget gates' (+ bias [2 * heads] or null), p0 = cap.  q, k: heads * dim columns, v: heads * vdim columns of rows
// with the stride ld; out [n, heads * vdim] float32.  Requests without tokens in this step are skipped.
HFEE_API int hfee_gated_recurrence(int mode, const void* q, const void* k, const void* v, long long ld, int dtype,
                                   const float* pre, long long ld_pre, const float* bias, float p0, float q_scale,
                                   float* state, float* norm_state, float* max_state, const int* cu_tokens,
                                   const int* slots, float* out, long long ld_o, int requests, int heads, int dim,
                                   int vdim, int write_state, cudaStream_t stream) {
  if (requests == 0) return HFEE_OK;
  HFEE_REQUIRE(mode == MODE_CHANNEL_DECAY || mode == MODE_EXP_GATES, "gated_recurrence: unknown mode %d", mode);
  HFEE_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && dim <= GR_MAX_DIM, "gated_recurrence: key size %d is outside 1..%d", dim, GR_MAX_DIM);
  HFEE_REQUIRE(requests <= 65535 && (vdim + GR_COLS - 1) / GR_COLS <= 65535, "gated_recurrence: too many requests or columns for one grid");
  HFEE_REQUIRE(ld_o >= (long long)heads * vdim, "gated_recurrence: ld_o is too small");
  HFEE_REQUIRE(mode == MODE_CHANNEL_DECAY ? ld_pre >= (long long)heads * dim : ld_pre >= 2 * heads, "gated_recurrence: ld_pre is too small");
  HFEE_REQUIRE(mode == MODE_CHANNEL_DECAY || (norm_state != nullptr && max_state != nullptr), "gated_recurrence: exponential gates need their normaliser and maximum states");
  HFEE_REQUIRE(p0 > 0.f, "gated_recurrence: the temperature or cap must be positive");
  RecurrenceArgs p{ld, pre, ld_pre, bias, p0, q_scale, state, norm_state, max_state, cu_tokens, slots, out, ld_o, heads, dim, vdim, write_state,
                   requests, nullptr, nullptr, nullptr, nullptr, 0, 0};
  if (dtype == HFEE_F32) return launch_recurrence<float, PASS_WHOLE>(mode, q, k, v, p, requests, stream);
  if (dtype == HFEE_BF16) return launch_recurrence<__nv_bfloat16, PASS_WHOLE>(mode, q, k, v, p, requests, stream);
  return hfee_fail(HFEE_ERR_ARG, "gated_recurrence: unknown dtype %d", dtype);
}

// Floats of workspace the chunked path needs for a step of at most n_tokens tokens of at most `requests` requests.
HFEE_API long long hfee_gated_recurrence_workspace(int requests, int n_tokens, int heads, int dim, int vdim) {
  const long long runs = n_tokens / GC_T + requests;
  return runs * heads * ((long long)dim * vdim + 2 * dim) + 3ll * n_tokens * heads;
}

// The same result as hfee_gated_recurrence for steps with long portions; `workspace` holds
// hfee_gated_recurrence_workspace(requests, n_tokens, ...) floats.  With the channel decay, `pre` is overwritten (by the
// decays).
HFEE_API int hfee_gated_recurrence_chunked(int mode, const void* q, const void* k, const void* v, long long ld, int dtype,
                                           float* pre, long long ld_pre, const float* bias, float p0, float q_scale,
                                           float* state, float* norm_state, float* max_state, const int* cu_tokens,
                                           const int* slots, float* out, long long ld_o, int requests, int n_tokens, int heads,
                                           int dim, int vdim, int write_state, float* workspace, long long workspace_floats,
                                           cudaStream_t stream) {
  if (requests == 0 || n_tokens == 0) return HFEE_OK;
  HFEE_REQUIRE(mode == MODE_CHANNEL_DECAY || mode == MODE_EXP_GATES, "gated_recurrence: unknown mode %d", mode);
  HFEE_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && dim <= GR_MAX_DIM, "gated_recurrence: key size %d is outside 1..%d", dim, GR_MAX_DIM);
  HFEE_REQUIRE(ld_o >= (long long)heads * vdim, "gated_recurrence: ld_o is too small");
  HFEE_REQUIRE(mode == MODE_CHANNEL_DECAY ? ld_pre >= (long long)heads * dim : ld_pre >= 2 * heads, "gated_recurrence: ld_pre is too small");
  HFEE_REQUIRE(mode == MODE_CHANNEL_DECAY || (norm_state != nullptr && max_state != nullptr), "gated_recurrence: exponential gates need their normaliser and maximum states");
  HFEE_REQUIRE(p0 > 0.f, "gated_recurrence: the temperature or cap must be positive");
  const long long max_runs = n_tokens / GC_T + requests;
  HFEE_REQUIRE(max_runs <= 65535 && requests <= 65535, "gated_recurrence: too many runs for one grid");
  HFEE_REQUIRE(workspace != nullptr && workspace_floats >= hfee_gated_recurrence_workspace(requests, n_tokens, heads, dim, vdim),
               "gated_recurrence: the workspace is too small");
  RecurrenceArgs p{ld, pre, ld_pre, bias, p0, q_scale, state, norm_state, max_state, cu_tokens, slots, out, ld_o, heads, dim, vdim, write_state,
                   requests, nullptr, nullptr, nullptr, nullptr, 0, 0};
  p.run_state = workspace;
  p.run_norm = p.run_state + max_runs * heads * dim * vdim;
  p.run_decay = p.run_norm + max_runs * heads * dim;
  p.gates = p.run_decay + max_runs * heads * dim;
  p.gate_stride = (long long)n_tokens * heads;
  if (dtype == HFEE_F32) return launch_chunked<float>(mode, q, k, v, p, pre, ld_pre, bias, p0, n_tokens, (int)max_runs, stream);
  if (dtype == HFEE_BF16) return launch_chunked<__nv_bfloat16>(mode, q, k, v, p, pre, ld_pre, bias, p0, n_tokens, (int)max_runs, stream);
  return hfee_fail(HFEE_ERR_ARG, "gated_recurrence: unknown dtype %d", dtype);
}
