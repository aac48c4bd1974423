// Causal grouped-query attention over the paged cache on the CUDA cores, float32
// arithmetic, for any head size: one warp per (token, query head).
//
// The keys a token sees are the positions lo..pos of its own request, lo = 0 or
// pos+1-window.  They are visited in blocks of 32 counted from lo with an online
// softmax, so the result at a position depends neither on how the tokens were cut
// into steps nor on which pages hold them.  This kernel is the attention of the
// true 32-bit path and the fallback of the bfloat16 path.
//
// Options beside the plain softmax over a causal window: `chunk` > 0 hides every key whose
// position lies in another block of `chunk` positions than the query's (blocks counted from
// position 0 of the request); SIGMOID replaces the softmax by unnormalised weights
// sigmoid(score * head_scale[h] + head_bias[h]) (either array may be missing); `gate` multiplies
// the output element by element with sigmoid(gate[token, head * vd + d]), or, with GATE_PER_HEAD, every
// element of head h with the one number sigmoid(gate[token, h]).  The values may have another size than the
// keys (`vcache.head_dim`), and with v_pool == k_pool and a value size of at most the key size they are the
// leading dimensions of the cached keys (a latent cache: one vector per token serves as key and as value).
// Reference: hostfog/hfee internal/llm/forward.go:146-178 (scores scaled after the
// dot, softmax over 0..pos, weighted sum of values), internal/ggml/ops.go:136-150.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 640;      // key size
constexpr int MAX_VD = 512;      // value size
constexpr int GATE_NONE = 0, GATE_ELEMENT = 1, GATE_PER_HEAD = 2;

template <typename T, bool SIGMOID>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, PagedCache cache, PagedCache vcache, int vd,
                      const int* __restrict__ positions,
                      const int* __restrict__ slot_of_token, T* __restrict__ out, int ld_o, int n, int heads,
                      float scale, int window, int chunk, const float* __restrict__ head_scale,
                      const float* __restrict__ head_bias, const T* __restrict__ gate, long long ld_gate,
                      int gate_mode, const float* __restrict__ dist_r1, const float* __restrict__ dist_r2, float out_scale,
                      const float* __restrict__ sink) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float q_s[WARPS][MAX_HD];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long task = (long long)blockIdx.x * WARPS + warp;
  if (task >= (long long)n * heads) return;
  int i = (int)(task / heads), h = (int)(task % heads);
  int hd = cache.head_dim;
  int kvh = h / (heads / cache.kv_heads);
  int pos = positions[i], slot = slot_of_token[i];
  int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
  const float h_scale = (SIGMOID && head_scale != nullptr) ? head_scale[h] : 1.f;
  const float h_bias = (SIGMOID && head_bias != nullptr) ? head_bias[h] : 0.f;
  const float r1 = dist_r1 != nullptr ? dist_r1[h] : 0.f, r2 = dist_r1 != nullptr ? dist_r2[h] : 0.f;

  const T* qrow = q + (long long)i * ld_q + (long long)h * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32<T>(qrow[d]);
  __syncwarp();

  constexpr int DPL = MAX_VD / 32;     // output dims per lane
  float o[DPL];
#pragma unroll
  for (int j = 0; j < DPL; ++j) o[j] = 0.f;
  // a sink is one more term exp(sink[h]) of the denominator that has no key and no value
  float m = (!SIGMOID && sink != nullptr) ? sink[h] : -INFINITY, l = (!SIGMOID && sink != nullptr) ? 1.f : 0.f;

  for (int base = lo; base <= pos; base += 32) {
    int key = base + lane;
    float s = -INFINITY;
    if (key <= pos) {
      const T* kr = k_pool + paged_offset(cache, slot, key, kvh);
      float acc = 0.f;
      for (int d = 0; d < hd; ++d) acc = fmaf(q_s[warp][d], to_f32<T>(kr[d]), acc);
      s = acc * scale;
      if (dist_r1 != nullptr) s -= r1 * log1pf(r2 * (float)(pos - key));
    }
    float p;
    if constexpr (SIGMOID) {
      p = key <= pos ? 1.f / (1.f + expf(-(s * h_scale + h_bias))) : 0.f;
    } else {
      float m_new = fmaxf(m, warp_max(s));
      p = key <= pos ? expf(s - m_new) : 0.f;
      float alpha = expf(m - m_new);          // exp(-inf) = 0 on the first block
      l = l * alpha + warp_sum(p);
#pragma unroll
      for (int j = 0; j < DPL; ++j) o[j] *= alpha;
      m = m_new;
    }
    int count = min(32, pos + 1 - base);
    for (int t = 0; t < count; ++t) {
      float pt = __shfl_sync(0xffffffffu, p, t);
      const T* vr = v_pool + paged_offset(vcache, slot, base + t, kvh);
#pragma unroll
      for (int j = 0; j < DPL; ++j) {
        int d = lane + 32 * j;
        if (d < vd) o[j] = fmaf(pt, to_f32<T>(vr[d]), o[j]);
      }
    }
  }
  T* orow = out + (long long)i * ld_o + (long long)h * vd;
  float inv = (SIGMOID ? 1.f : 1.f / l) * out_scale;
  const T* grow = gate_mode == GATE_ELEMENT ? gate + (long long)i * ld_gate + (long long)h * vd : nullptr;
  if (gate_mode == GATE_PER_HEAD) inv *= 1.f / (1.f + expf(-to_f32<T>(gate[(long long)i * ld_gate + h])));
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    int d = lane + 32 * j;
    if (d < vd) {
      float v = o[j] * inv;
      if (grow != nullptr) v *= 1.f / (1.f + expf(-to_f32<T>(grow[d])));
      orow[d] = from_f32<T>(v);
    }
  }
}

}  // namespace

namespace {
template <typename T>
void launch_simt(const void* q, int ld_q, const void* k_pool, const void* v_pool, const PagedCache& c, const PagedCache& vc,
                 int vd, const int* positions,
                 const int* slot_of_token, void* out, int ld_o, int n, int heads, float scale, int window, int chunk,
                 int sigmoid, const float* head_scale, const float* head_bias, const void* gate, long long ld_gate,
                 int gate_mode, const float* dist_r1, const float* dist_r2, float out_scale, const float* sink, cudaStream_t stream) {
  long long tasks = (long long)n * heads;
  unsigned blocks = (unsigned)((tasks + WARPS - 1) / WARPS);
  if (sigmoid)
    hfee_launch(attention_simt_kernel<T, true>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const T*)q, ld_q, (const T*)k_pool,
                (const T*)v_pool, c, vc, vd, positions, slot_of_token, (T*)out, ld_o, n, heads, scale, window, chunk, head_scale,
                head_bias, (const T*)gate, ld_gate, gate_mode, dist_r1, dist_r2, out_scale, sink);
  else
    hfee_launch(attention_simt_kernel<T, false>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const T*)q, ld_q, (const T*)k_pool,
                (const T*)v_pool, c, vc, vd, positions, slot_of_token, (T*)out, ld_o, n, heads, scale, window, chunk, head_scale,
                head_bias, (const T*)gate, ld_gate, gate_mode, dist_r1, dist_r2, out_scale, sink);
}
}  // namespace

// weights: 0 = softmax over the visible keys, 1 = sigmoid(score * head_scale[h] + head_bias[h]) per key.
// value_dim: size of a value; v_pool is [pages][kv_heads][page_size][value_dim], or, with values_in_keys, the key
// pool itself, whose leading value_dim dimensions are the values.  gate_mode: 0 none, 1 one number per output
// element ([n, heads * value_dim]), 2 one number per head ([n, heads]); the output is multiplied by its sigmoid.
// dist_r1, dist_r2 (per head, or both null): r1[h] * ln(1 + r2[h] * (query position - key position)) is taken off the
// score before the softmax.  out_scale multiplies the output.  sink (per head, or null): the softmax's denominator also
// holds exp(sink[h]).
HFEE_API int hfee_attention_simt_sink(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                          const int* block_table, int max_pages, int page_size, const int* positions,
                                          const int* slot_of_token, void* out, int ld_o, int n, int heads, int kv_heads,
                                          int head_dim, int value_dim, int values_in_keys, float scale, int window,
                                          int chunk, int weights, const float* head_scale, const float* head_bias,
                                          const void* gate, long long ld_gate, int gate_mode, const float* dist_r1,
                                          const float* dist_r2, float out_scale, const float* sink, int dtype,
                                          cudaStream_t stream) {
  HFEE_REQUIRE(sink == nullptr || weights == 0, "attention_simt: a sink goes with the softmax");
  HFEE_REQUIRE((dist_r1 == nullptr) == (dist_r2 == nullptr), "attention_simt: the distance penalty needs both of its arrays");
  HFEE_REQUIRE(dist_r1 == nullptr || weights == 0, "attention_simt: the distance penalty goes with the softmax");
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(head_dim > 0 && head_dim <= MAX_HD, "attention_simt: head_dim %d is outside 1..%d", head_dim, MAX_HD);
  HFEE_REQUIRE(value_dim > 0 && value_dim <= MAX_VD, "attention_simt: value_dim %d is outside 1..%d", value_dim, MAX_VD);
  HFEE_REQUIRE(!values_in_keys || value_dim <= head_dim, "attention_simt: values inside keys need value_dim <= head_dim");
  HFEE_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
               "attention_simt: heads %d must be a multiple of kv_heads %d", heads, kv_heads);
  HFEE_REQUIRE(page_size > 0 && max_pages > 0, "attention_simt: bad cache sizes");
  HFEE_REQUIRE(window >= 0 && chunk >= 0 && (weights == 0 || weights == 1), "attention_simt: bad mask or weight option");
  HFEE_REQUIRE(gate_mode >= GATE_NONE && gate_mode <= GATE_PER_HEAD && (gate_mode == GATE_NONE) == (gate == nullptr),
               "attention_simt: gate and gate_mode %d do not fit", gate_mode);
  HFEE_REQUIRE(gate_mode != GATE_ELEMENT || ld_gate >= (long long)heads * value_dim, "attention_simt: ld_gate is too small");
  HFEE_REQUIRE(gate_mode != GATE_PER_HEAD || ld_gate >= heads, "attention_simt: ld_gate is too small");
  PagedCache c, vc;
  HFEE_REQUIRE(make_paged_cache(&c, block_table, max_pages, page_size, kv_heads, head_dim),
               "page_size %d must be a power of two", page_size);
  if (values_in_keys) {
    vc = c;
    v_pool = k_pool;
  } else {
    make_paged_cache(&vc, block_table, max_pages, page_size, kv_heads, value_dim);
  }
  if (dtype == HFEE_F32)
    launch_simt<float>(q, ld_q, k_pool, v_pool, c, vc, value_dim, positions, slot_of_token, out, ld_o, n, heads, scale,
                       window, chunk, weights, head_scale, head_bias, gate, ld_gate, gate_mode, dist_r1, dist_r2, out_scale, sink, stream);
  else if (dtype == HFEE_BF16)
    launch_simt<__nv_bfloat16>(q, ld_q, k_pool, v_pool, c, vc, value_dim, positions, slot_of_token, out, ld_o, n, heads,
                               scale, window, chunk, weights, head_scale, head_bias, gate, ld_gate, gate_mode, dist_r1, dist_r2,
                               out_scale, sink, stream);
  else
    return hfee_fail(HFEE_ERR_ARG, "attention_simt: unknown dtype %d", dtype);
  return hfee_check_launch("attention_simt");
}

HFEE_API int hfee_attention_simt_distance(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                          const int* block_table, int max_pages, int page_size, const int* positions,
                                          const int* slot_of_token, void* out, int ld_o, int n, int heads, int kv_heads,
                                          int head_dim, int value_dim, int values_in_keys, float scale, int window,
                                          int chunk, int weights, const float* head_scale, const float* head_bias,
                                          const void* gate, long long ld_gate, int gate_mode, const float* dist_r1,
                                          const float* dist_r2, float out_scale, int dtype, cudaStream_t stream) {
  return hfee_attention_simt_sink(q, ld_q, k_pool, v_pool, block_table, max_pages, page_size, positions, slot_of_token, out,
                                  ld_o, n, heads, kv_heads, head_dim, value_dim, values_in_keys, scale, window, chunk,
                                  weights, head_scale, head_bias, gate, ld_gate, gate_mode, dist_r1, dist_r2, out_scale,
                                  nullptr, dtype, stream);
}

HFEE_API int hfee_attention_simt_general(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                         const int* block_table, int max_pages, int page_size, const int* positions,
                                         const int* slot_of_token, void* out, int ld_o, int n, int heads, int kv_heads,
                                         int head_dim, int value_dim, int values_in_keys, float scale, int window,
                                         int chunk, int weights, const float* head_scale, const float* head_bias,
                                         const void* gate, long long ld_gate, int gate_mode, int dtype,
                                         cudaStream_t stream) {
  return hfee_attention_simt_distance(q, ld_q, k_pool, v_pool, block_table, max_pages, page_size, positions, slot_of_token,
                                      out, ld_o, n, heads, kv_heads, head_dim, value_dim, values_in_keys, scale, window,
                                      chunk, weights, head_scale, head_bias, gate, ld_gate, gate_mode, nullptr, nullptr,
                                      1.f, dtype, stream);
}

HFEE_API int hfee_attention_simt_masked(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                        const int* block_table, int max_pages, int page_size, const int* positions,
                                        const int* slot_of_token, void* out, int ld_o, int n, int heads, int kv_heads,
                                        int head_dim, float scale, int window, int chunk, int weights,
                                        const float* head_scale, const float* head_bias, const void* gate,
                                        long long ld_gate, int dtype, cudaStream_t stream) {
  HFEE_REQUIRE(head_dim > 0 && head_dim <= MAX_VD, "attention_simt: head_dim %d is outside 1..%d", head_dim, MAX_VD);
  return hfee_attention_simt_general(q, ld_q, k_pool, v_pool, block_table, max_pages, page_size, positions, slot_of_token,
                                     out, ld_o, n, heads, kv_heads, head_dim, head_dim, 0, scale, window, chunk, weights,
                                     head_scale, head_bias, gate, ld_gate, gate != nullptr ? GATE_ELEMENT : GATE_NONE,
                                     dtype, stream);
}

HFEE_API int hfee_attention_simt(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                 const int* block_table, int max_pages, int page_size, const int* positions,
                                 const int* slot_of_token, void* out, int ld_o, int n, int heads, int kv_heads,
                                 int head_dim, float scale, int window, int dtype, cudaStream_t stream) {
  return hfee_attention_simt_masked(q, ld_q, k_pool, v_pool, block_table, max_pages, page_size, positions, slot_of_token,
                                    out, ld_o, n, heads, kv_heads, head_dim, scale, window, 0, 0, nullptr, nullptr,
                                    nullptr, 0, dtype, stream);
}
