// Routed mixture of small gated experts: router, plan, the experts' two products over the tokens that chose them,
// and the weighted sum.
//
//   hfee_moe_route     scores = softmax(logits) over all experts (float32); the `top` largest per token (ties: the lower
//                      expert), their weights = score * scale (not renormalised).
//   hfee_moe_plan      orders the (token, choice) pairs by expert: offsets[e] .. offsets[e + 1] are the places of expert
//                      e's pairs, sorted[place] = token * top + choice; the places are cut into tiles of MOE_TILE rows
//                      that never span two experts (tile_expert, tile_row; unused tiles carry expert -1).
//   hfee_moe_gate_up   hidden[place] = act(W_gate[e] x, W_up[e] x) for every place of every expert, x gathered by token.
//   hfee_moe_down      pair_out[sorted[place]] = W_down[e] hidden[place] (float32).
//   hfee_moe_combine   y[t] (+)= sum_k weight[t, k] * pair_out[t * top + k].
//
// For the tensor cores the places are laid out in tiles of as many rows as a product's tile has, every expert
// starting at a tile's border (hfee_moe_plan_tiles), the tokens' rows are copied to their places
// (hfee_moe_gather_rows), the two products run as grouped products over those tiles (each tile against its expert's
// matrix), and hfee_moe_combine finds a pair's row through place_of_pair.  Rows between an expert's last pair and
// the next border hold whatever the buffer held; a row of a product depends on that row alone, and nothing reads them.
//
// Everything the launches depend on (grids, buffers) follows from the number of tokens alone; counts and places
// live in device memory, so a step replays from a CUDA graph.  A pair's result is computed by one thread block
// with k summed in order and does not depend on its place, so the order inside an expert (which the plan's atomic
// counters leave open) cannot show.  Gated activation: g = min(gate, limit), u = clamp(up, -limit, limit),
// g * sigmoid(alpha * g) * (u + shift); an infinite limit, alpha = 1 and shift = 0 give silu(gate) * up.
#include "common.cuh"

namespace {

constexpr int MOE_TILE = 32;         // rows (pairs) of a tile
constexpr int COLS = 64;             // output columns of a tile
constexpr int KSTEP = 32;
constexpr int THREADS = 256;
constexpr int PLAN_THREADS = 1024;
constexpr int MAX_EXPERTS = 1024;

__global__ void moe_route_kernel(const float* __restrict__ logits, int experts, int top, float scale, int* __restrict__ choice,
                                 float* __restrict__ weight, int n) {
  extern __shared__ float score_s[];       // [warps][experts]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n) return;
  float* s = score_s + (long long)warp * experts;
  const float* z = logits + (long long)t * experts;
  float m = -INFINITY;
  for (int e = lane; e < experts; e += 32) m = fmaxf(m, z[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float p = expf(z[e] - m);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -1.f;
    int at = experts;
    for (int e = lane; e < experts; e += 32)
      if (s[e] > best) { best = s[e]; at = e; }            // ascending e: the lowest index wins a tie within the lane
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (lane == 0) {
      choice[(long long)t * top + k] = at;
      weight[(long long)t * top + k] = best / sum * scale;
      s[at] = -2.f;
    }
    __syncwarp();
  }
}

// Router with sigmoid scores and a choice limited to groups of experts: s = sigmoid(logit); the experts form `groups`
// equal groups of neighbours, a group's score is the sum of its two largest s (of its only one, if it has one expert),
// only experts of the `keep` best groups (ties: the lower group) can be chosen; the `top` largest s among those (ties:
// the lower expert); weights = s / (sum of the chosen s + 1e-20) * scale.  One warp per token; logits rows have the
// stride ld (columns behind `experts` are not the router's).
__global__ void moe_route_grouped_kernel(const float* __restrict__ logits, int ld, int experts, int top, int groups, int keep,
                                         float scale, int* __restrict__ choice, float* __restrict__ weight, int n) {
  extern __shared__ float score_s[];       // [warps][experts + groups]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n) return;
  float* s = score_s + (long long)warp * (experts + groups);
  float* gs = s + experts;
  const float* z = logits + (long long)t * ld;
  for (int e = lane; e < experts; e += 32) s[e] = 1.f / (1.f + expf(-z[e]));
  __syncwarp();
  const int size = experts / groups;
  for (int g = lane; g < groups; g += 32) {
    float a = -1.f, b = -1.f;                  // the two largest of the group
    for (int e = g * size; e < (g + 1) * size; ++e) {
      const float v = s[e];
      if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
    }
    gs[g] = a + (size > 1 ? b : 0.f);
  }
  __syncwarp();
  // strike the groups that are not among the `keep` best: a group is kept if fewer than `keep` groups beat it
  for (int g = lane; g < groups; g += 32) {
    int better = 0;
    for (int o = 0; o < groups; ++o) better += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
    if (better >= keep)
      for (int e = g * size; e < (g + 1) * size; ++e) s[e] = -2.f;
  }
  __syncwarp();
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -1.f;
    int at = experts;
    for (int e = lane; e < experts; e += 32)
      if (s[e] > best) { best = s[e]; at = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    sum += best;
    if (lane == 0) {
      choice[(long long)t * top + k] = at;
      weight[(long long)t * top + k] = best;
      s[at] = -2.f;
    }
    __syncwarp();
  }
  if (lane < top) weight[(long long)t * top + lane] = weight[(long long)t * top + lane] / (sum + 1e-20f) * scale;
  for (int k = 32 + lane; k < top; k += 32) weight[(long long)t * top + k] = weight[(long long)t * top + k] / (sum + 1e-20f) * scale;
}

__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ choice, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ sorted,
                int* __restrict__ tile_expert, int* __restrict__ tile_row, int max_tiles) {
  __shared__ int count[MAX_EXPERTS], cursor[MAX_EXPERTS], first_tile[MAX_EXPERTS + 1], off_s[MAX_EXPERTS + 1];
  for (int e = threadIdx.x; e < experts; e += PLAN_THREADS) count[e] = cursor[e] = 0;
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += PLAN_THREADS) atomicAdd(&count[choice[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, tile = 0;
    for (int e = 0; e < experts; ++e) {
      off_s[e] = off;
      first_tile[e] = tile;
      off += count[e];
      tile += (count[e] + MOE_TILE - 1) / MOE_TILE;
    }
    off_s[experts] = off;
    first_tile[experts] = tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += PLAN_THREADS) offsets[e] = off_s[e];
  for (int e = threadIdx.x; e < experts; e += PLAN_THREADS)
    for (int j = first_tile[e]; j < first_tile[e + 1]; ++j) {
      tile_expert[j] = e;
      tile_row[j] = off_s[e] + (j - first_tile[e]) * MOE_TILE;
    }
  for (int j = first_tile[experts] + threadIdx.x; j < max_tiles; j += PLAN_THREADS) tile_expert[j] = -1;
  for (int i = threadIdx.x; i < pairs; i += PLAN_THREADS) {
    const int e = choice[i];
    sorted[off_s[e] + atomicAdd(&cursor[e], 1)] = i;
  }
}

// Places in tiles of tile_rows rows: expert e's pairs lie from first_tile[e] * tile_rows on.  place_of_pair[pair] is the
// pair's row, row_pair[row] the pair of a row (-1: none), tile_group[tile] the tile's expert (-1: unused).
__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_tiles_kernel(const int* __restrict__ choice, int pairs, int experts, int tile_rows, int* __restrict__ place_of_pair,
                      int* __restrict__ row_pair, int* __restrict__ tile_group, int max_tiles) {
  __shared__ int count[MAX_EXPERTS], cursor[MAX_EXPERTS], first_tile[MAX_EXPERTS + 1];
  for (int e = threadIdx.x; e < experts; e += PLAN_THREADS) count[e] = cursor[e] = 0;
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += PLAN_THREADS) atomicAdd(&count[choice[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < experts; ++e) {
      first_tile[e] = tile;
      tile += (count[e] + tile_rows - 1) / tile_rows;
    }
    first_tile[experts] = tile;
  }
  __syncthreads();
  const int used = first_tile[experts];
  for (int e = threadIdx.x; e < experts; e += PLAN_THREADS)
    for (int j = first_tile[e]; j < first_tile[e + 1]; ++j) tile_group[j] = e;
  for (int j = used + threadIdx.x; j < max_tiles; j += PLAN_THREADS) tile_group[j] = -1;
  for (long long r = threadIdx.x; r < (long long)used * tile_rows; r += PLAN_THREADS) row_pair[r] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += PLAN_THREADS) {
    const int e = choice[i];
    const int row = first_tile[e] * tile_rows + atomicAdd(&cursor[e], 1);
    place_of_pair[i] = row;
    row_pair[row] = i;
  }
}

// xg[row] = x[row_pair[row] / top] for the rows of used tiles that hold a pair; 16 bytes per thread and step.
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const uint4* __restrict__ x, long long ld_x16, int top, const int* __restrict__ row_pair,
                       const int* __restrict__ tile_group, int tile_rows, uint4* __restrict__ xg, long long ld_g16, int width16) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  if (tile_group[row / tile_rows] < 0) return;
  const int pair = row_pair[row];
  if (pair < 0) return;
  const uint4* src = x + (long long)(pair / top) * ld_x16;
  uint4* dst = xg + (long long)row * ld_g16;
  for (int i = threadIdx.x; i < width16; i += 128) dst[i] = src[i];
}

__device__ __forceinline__ float clamped_glu(float gate, float up, float limit, float alpha, float shift) {
  const float g = fminf(gate, limit);
  const float u = fminf(fmaxf(up, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + shift);
}

// One tile: MOE_TILE rows x COLS columns, 256 threads, thread (ty = tid / 16, tx = tid % 16) owns rows ty, ty + 16 and
// columns tx + 16 j (j < 4); k in steps of KSTEP through shared memory, summed in order.
template <typename T, bool GATED>
__global__ void __launch_bounds__(THREADS)
moe_expert_kernel(const T* __restrict__ a, long long ld_a, int top, const T* __restrict__ w1, const T* __restrict__ w2,
                  long long expert_stride, int n_out, int k_dim, const int* __restrict__ offsets, const int* __restrict__ sorted,
                  const int* __restrict__ tile_expert, const int* __restrict__ tile_row, T* __restrict__ hidden,
                  float* __restrict__ pair_out, long long ld_out, float limit, float alpha, float shift) {
  __shared__ float a_s[MOE_TILE][KSTEP + 1], w1_s[COLS][KSTEP + 1], w2_s[GATED ? COLS : 1][KSTEP + 1];
  __shared__ int row_src[MOE_TILE], row_dst[MOE_TILE];
  pdl_wait();
  pdl_launch_dependents();
  const int expert = tile_expert[blockIdx.x];
  if (expert < 0) return;
  const int row0 = tile_row[blockIdx.x];
  const int rows = min(MOE_TILE, offsets[expert + 1] - row0);
  const int col0 = blockIdx.y * COLS;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  if (tid < MOE_TILE) {
    const int pair = tid < rows ? sorted[row0 + tid] : -1;
    // first product: rows are gathered by token and go to their place; second: rows lie at their place and go to their pair
    row_src[tid] = GATED ? (pair < 0 ? -1 : pair / top) : (tid < rows ? row0 + tid : -1);
    row_dst[tid] = GATED ? (tid < rows ? row0 + tid : -1) : pair;
  }
  __syncthreads();
  const T* w1e = w1 + (long long)expert * expert_stride;
  const T* w2e = GATED ? w2 + (long long)expert * expert_stride : nullptr;
  float acc1[2][4], acc2[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc1[i][j] = acc2[i][j] = 0.f;
  for (int k0 = 0; k0 < k_dim; k0 += KSTEP) {
    for (int i = tid; i < MOE_TILE * KSTEP; i += THREADS) {
      const int r = i / KSTEP, k = i % KSTEP;
      const int src = row_src[r];
      a_s[r][k] = (src >= 0 && k0 + k < k_dim) ? to_f32<T>(a[(long long)src * ld_a + k0 + k]) : 0.f;
    }
    for (int i = tid; i < COLS * KSTEP; i += THREADS) {
      const int c = i / KSTEP, k = i % KSTEP;
      const bool in = col0 + c < n_out && k0 + k < k_dim;
      w1_s[c][k] = in ? to_f32<T>(w1e[(long long)(col0 + c) * k_dim + k0 + k]) : 0.f;
      if constexpr (GATED) w2_s[c][k] = in ? to_f32<T>(w2e[(long long)(col0 + c) * k_dim + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < KSTEP; ++k) {
      const float a0 = a_s[ty][k], a1 = a_s[ty + 16][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b1 = w1_s[tx + 16 * j][k];
        acc1[0][j] = fmaf(a0, b1, acc1[0][j]);
        acc1[1][j] = fmaf(a1, b1, acc1[1][j]);
        if constexpr (GATED) {
          const float b2 = w2_s[tx + 16 * j][k];
          acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
          acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int dst = row_dst[ty + 16 * i];
    if (dst < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx + 16 * j;
      if (c >= n_out) continue;
      if constexpr (GATED) hidden[(long long)dst * ld_out + c] = from_f32<T>(clamped_glu(acc1[i][j], acc2[i][j], limit, alpha, shift));
      else pair_out[(long long)dst * ld_out + c] = acc1[i][j];
    }
  }
}

__global__ void __launch_bounds__(THREADS)
moe_combine_kernel(const float* __restrict__ pair_out, const float* __restrict__ weight, const int* __restrict__ place, int top,
                   float* __restrict__ y, int width, int accumulate,      // place: the row of each pair (null: the pair's index)
                   const float* __restrict__ extra, const float* __restrict__ extra_gate, long long ld_gate) {
  pdl_wait();
  pdl_launch_dependents();
  const long long t = blockIdx.x;
  // extra [n, width]: one more term per token (an expert every token uses), times sigmoid(extra_gate[t * ld_gate])
  const float eg = extra != nullptr ? (extra_gate != nullptr ? 1.f / (1.f + expf(-extra_gate[t * ld_gate])) : 1.f) : 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float acc = accumulate ? y[t * width + c] : 0.f;
    if (extra != nullptr) acc = fmaf(eg, extra[t * width + c], acc);
    for (int k = 0; k < top; ++k) {
      const long long row = place ? place[t * top + k] : t * top + k;
      acc = fmaf(weight[t * top + k], pair_out[row * width + c], acc);
    }
    y[t * width + c] = acc;
  }
}

template <typename T>
int launch_experts(bool gated, const void* a, long long ld_a, int top, const void* w1, const void* w2, long long expert_stride,
                   int n_out, int k_dim, const int* offsets, const int* sorted, const int* tile_expert, const int* tile_row,
                   void* hidden, float* pair_out, long long ld_out, float limit, float alpha, float shift, int max_tiles, cudaStream_t stream) {
  dim3 grid(max_tiles, (n_out + COLS - 1) / COLS);
  if (gated)
    hfee_launch(moe_expert_kernel<T, true>, grid, dim3(THREADS), 0, stream, (const T*)a, ld_a, top, (const T*)w1, (const T*)w2,
                expert_stride, n_out, k_dim, offsets, sorted, tile_expert, tile_row, (T*)hidden, pair_out, ld_out, limit, alpha, shift);
  else
    hfee_launch(moe_expert_kernel<T, false>, grid, dim3(THREADS), 0, stream, (const T*)a, ld_a, top, (const T*)w1, (const T*)w2,
                expert_stride, n_out, k_dim, offsets, sorted, tile_expert, tile_row, (T*)hidden, pair_out, ld_out, limit, alpha, shift);
  return hfee_check_launch(gated ? "moe_gate_up" : "moe_down");
}

}  // namespace

HFEE_API int hfee_moe_tile_rows() { return MOE_TILE; }

HFEE_API int hfee_moe_route(const float* logits, int n, int experts, int top, float scale, int* choice, float* weight,
                            cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && experts >= 1 && experts <= MAX_EXPERTS, "moe_route: %d experts are outside 1..%d", experts, MAX_EXPERTS);
  HFEE_REQUIRE(top >= 1 && top <= experts, "moe_route: top %d is outside 1..%d", top, experts);
  const int warps = 4;
  hfee_launch(moe_route_kernel, dim3((n + warps - 1) / warps), dim3(32 * warps), (size_t)warps * experts * sizeof(float), stream,
              logits, experts, top, scale, choice, weight, n);
  return hfee_check_launch("moe_route");
}

// offsets: [experts + 1]; sorted: [pairs]; tile_expert, tile_row: [max_tiles], max_tiles >= pairs / MOE_TILE + experts.
HFEE_API int hfee_moe_plan(const int* choice, int pairs, int experts, int* offsets, int* sorted, int* tile_expert, int* tile_row,
                           int max_tiles, cudaStream_t stream) {
  if (pairs == 0) return HFEE_OK;
  HFEE_REQUIRE(pairs > 0 && experts >= 1 && experts <= MAX_EXPERTS, "moe_plan: bad sizes");
  HFEE_REQUIRE(max_tiles >= (pairs + MOE_TILE - 1) / MOE_TILE + experts - 1, "moe_plan: room for %d tiles is too little", max_tiles);
  hfee_launch(moe_plan_kernel, dim3(1), dim3(PLAN_THREADS), 0, stream, choice, pairs, experts, offsets, sorted, tile_expert, tile_row,
              max_tiles);
  return hfee_check_launch("moe_plan");
}

// x: [n, width] tokens; w_gate, w_up: [experts, inner, width]; hidden: [pairs, inner] by place.
// expert_stride: elements from one expert's w_gate (and w_up) to the next one's.
HFEE_API int hfee_moe_gate_up(const void* x, long long ld_x, int top, const void* w_gate, const void* w_up, long long expert_stride,
                              int inner, int width, const int* offsets, const int* sorted, const int* tile_expert, const int* tile_row, void* hidden,
                              long long ld_hidden, float limit, float alpha, float shift, int max_tiles, int dtype, cudaStream_t stream) {
  if (max_tiles == 0) return HFEE_OK;
  HFEE_REQUIRE(inner > 0 && width > 0 && top > 0 && ld_x >= width && ld_hidden >= inner && limit > 0.f &&
               expert_stride >= (long long)inner * width, "moe_gate_up: bad sizes");
  if (dtype == HFEE_F32)
    return launch_experts<float>(true, x, ld_x, top, w_gate, w_up, expert_stride, inner, width, offsets, sorted, tile_expert,
                                 tile_row, hidden, nullptr, ld_hidden, limit, alpha, shift, max_tiles, stream);
  if (dtype == HFEE_BF16)
    return launch_experts<__nv_bfloat16>(true, x, ld_x, top, w_gate, w_up, expert_stride, inner, width, offsets, sorted,
                                         tile_expert, tile_row, hidden, nullptr, ld_hidden, limit, alpha, shift, max_tiles, stream);
  return hfee_fail(HFEE_ERR_ARG, "moe_gate_up: unknown dtype %d", dtype);
}

// hidden: [pairs, inner] by place; w_down: [experts, width, inner]; pair_out: [pairs, width] float32 by pair.
HFEE_API int hfee_moe_down(const void* hidden, long long ld_hidden, int top, const void* w_down, int inner, int width,
                           const int* offsets, const int* sorted, const int* tile_expert, const int* tile_row, float* pair_out,
                           int max_tiles, int dtype, cudaStream_t stream) {
  if (max_tiles == 0) return HFEE_OK;
  HFEE_REQUIRE(inner > 0 && width > 0 && top > 0 && ld_hidden >= inner, "moe_down: bad sizes");
  if (dtype == HFEE_F32)
    return launch_experts<float>(false, hidden, ld_hidden, top, w_down, nullptr, (long long)inner * width, width, inner, offsets, sorted,
                                 tile_expert, tile_row, nullptr, pair_out, width, 0.f, 0.f, 0.f, max_tiles, stream);
  if (dtype == HFEE_BF16)
    return launch_experts<__nv_bfloat16>(false, hidden, ld_hidden, top, w_down, nullptr, (long long)inner * width, width, inner, offsets,
                                         sorted, tile_expert, tile_row, nullptr, pair_out, width, 0.f, 0.f, 0.f, max_tiles, stream);
  return hfee_fail(HFEE_ERR_ARG, "moe_down: unknown dtype %d", dtype);
}

HFEE_API int hfee_moe_combine_extra(const float* pair_out, const float* weight, const int* place, int n, int top, float* y, int width,
                                    int accumulate, const float* extra, const float* extra_gate, long long ld_gate,
                                    cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  HFEE_REQUIRE(extra != nullptr || extra_gate == nullptr, "moe_combine: a gate without the term it gates");
  hfee_launch(moe_combine_kernel, dim3(n), dim3(THREADS), 0, stream, pair_out, weight, place, top, y, width, accumulate, extra,
              extra_gate, ld_gate);
  return hfee_check_launch("moe_combine");
}

HFEE_API int hfee_moe_combine(const float* pair_out, const float* weight, const int* place, int n, int top, float* y, int width,
                              int accumulate, cudaStream_t stream) {
  return hfee_moe_combine_extra(pair_out, weight, place, n, top, y, width, accumulate, nullptr, nullptr, 0, stream);
}

// logits: [n, ld] float32 of which the first `experts` columns are the router's.
HFEE_API int hfee_moe_route_grouped(const float* logits, long long ld, int n, int experts, int top, int groups, int keep, float scale,
                                    int* choice, float* weight, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(experts >= 1 && experts <= MAX_EXPERTS && groups >= 1 && experts % groups == 0 && keep >= 1 && keep <= groups,
               "moe_route_grouped: %d experts in %d groups of which %d are kept", experts, groups, keep);
  HFEE_REQUIRE(top >= 1 && top <= keep * (experts / groups), "moe_route_grouped: top %d exceeds the experts of the kept groups", top);
  HFEE_REQUIRE(ld >= experts, "moe_route_grouped: ld is too small");
  const int warps = 4;
  hfee_launch(moe_route_grouped_kernel, dim3((n + warps - 1) / warps), dim3(warps * 32), (size_t)warps * (experts + groups) * sizeof(float),
              stream, logits, (int)ld, experts, top, groups, keep, scale, choice, weight, n);
  return hfee_check_launch("moe_route_grouped");
}

// place_of_pair: [pairs]; row_pair: [max_tiles * tile_rows]; tile_group: [max_tiles], max_tiles >= pairs / tile_rows +
// min(experts, pairs).
HFEE_API int hfee_moe_plan_tiles(const int* choice, int pairs, int experts, int tile_rows, int* place_of_pair, int* row_pair,
                                 int* tile_group, int max_tiles, cudaStream_t stream) {
  if (pairs == 0) return HFEE_OK;
  HFEE_REQUIRE(pairs > 0 && experts >= 1 && experts <= MAX_EXPERTS && tile_rows > 0, "moe_plan_tiles: bad sizes");
  HFEE_REQUIRE(max_tiles >= pairs / tile_rows + (experts < pairs ? experts : pairs), "moe_plan_tiles: room for %d tiles is too little", max_tiles);
  hfee_launch(moe_plan_tiles_kernel, dim3(1), dim3(PLAN_THREADS), 0, stream, choice, pairs, experts, tile_rows, place_of_pair, row_pair,
              tile_group, max_tiles);
  return hfee_check_launch("moe_plan_tiles");
}

// x: [n, width] tokens; xg: [max_tiles * tile_rows, width] by place.  16-bit elements, rows of whole 16-byte pieces.
HFEE_API int hfee_moe_gather_rows(const void* x, long long ld_x, int top, const int* row_pair, const int* tile_group, int tile_rows,
                                  void* xg, long long ld_g, int width, int max_tiles, cudaStream_t stream) {
  if (max_tiles == 0) return HFEE_OK;
  HFEE_REQUIRE(width > 0 && width % 8 == 0 && ld_x % 8 == 0 && ld_g % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)xg % 16 == 0),
               "moe_gather_rows: rows must be whole 16-byte pieces");
  hfee_launch(moe_gather_rows_kernel, dim3((unsigned)(max_tiles * tile_rows)), dim3(128), 0, stream, (const uint4*)x, ld_x / 8, top,
              row_pair, tile_group, tile_rows, (uint4*)xg, ld_g / 8, width / 8);
  return hfee_check_launch("moe_gather_rows");
}
