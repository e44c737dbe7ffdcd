/*
 * moe_oracle.c - CPU restatement of the reference's fused MXFP4 MoE layer.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing the library ships may call, link or load
 * this file; it exists so the CUDA path can be checked against an independent
 * statement of the reference algorithm (and timed as the CPU baseline).
 *
 * Each function names the reference code it follows (paths are relative to the
 * reference project root). Parity is PINNED: tests compare this file against
 * the reference's own moe_fused.cpp / dist_moe.cpp compiled in place (see the
 * Makefile next to this file) bit for bit, and against the analytic
 * known-answer cases of tests/kernels/moe/test_moe_fused.cpp,
 * test_moe_align_oracle.cpp and test_dist_moe.cpp.
 *
 * The routing functions at the bottom have no CPU counterpart in the reference
 * (its routers are GPU-only Triton/Gluon ops); they restate
 * src/python/vkernels/torch_ops/tokenspeed_amd/routing.py and glm_router.py
 * and are "parity unpinned" against reference code; they are pinned only to
 * golden vectors generated from a torch-eager statement of the same formulas.
 *
 * Arithmetic contract (src/c/CMakeLists.txt:8-11): compile with
 * -ffp-contract=off. The summation order below reproduces the reference's:
 * a 64-long sequential fp32 dot per K block, then one add into the running
 * accumulator (moe_fused.cpp:315-325).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define VKO_BM 16 /* rows per routed block (moe_fused.cpp:245) */
#define VKO_BK 64 /* K elements per partial dot (moe_fused.cpp:247) */

#if defined(__GNUC__) && defined(__x86_64__) && !defined(VKO_NO_CLONES)
#define VKO_HOT __attribute__((target_clones("avx2", "default")))
#else
#define VKO_HOT
#endif

/* ------------------------------------------------------------------ */
/* scalar helpers                                                       */
/* ------------------------------------------------------------------ */

static inline float bits_to_f32(uint32_t b) {
  float f;
  memcpy(&f, &b, sizeof f);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t b;
  memcpy(&b, &f, sizeof b);
  return b;
}

/* Round-to-nearest-even fp32 -> bf16 by integer arithmetic on the bit pattern
 * (moe_fused.cpp:41-45). NaN/inf take the same integer path as the reference. */
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t b = f32_to_bits(f);
  b += 0x7FFFu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
static inline float bf16_to_f32(uint16_t v) { return bits_to_f32((uint32_t)v << 16); }

/* E2M1 nibble -> fp32. The reference's table is NOT the OCP one: magnitudes
 * {0, 0.25, 1, 1.5, 2, 3, inf, NaN} (moe_fused.cpp:24-39). The NaN code carries
 * no sign. */
static inline float e2m1_value(unsigned nib) {
  static const uint32_t mag[8] = {0x00000000u, 0x3E800000u, 0x3F800000u, 0x3FC00000u,
                                  0x40000000u, 0x40400000u, 0x7F800000u, 0x7FC00000u};
  unsigned m = nib & 7u;
  uint32_t b = mag[m];
  if ((nib & 8u) && m != 7u) b |= 0x80000000u;
  return bits_to_f32(b);
}

/* ue8m0 scale byte -> fp32: 0xFF -> 0, 0x00 -> 2^-127 (subnormal), else 2^(s-127)
 * (moe_fused.cpp:50-64). */
static inline float ue8m0_value(uint8_t s) {
  if (s == 0xFFu) return 0.0f;
  if (s == 0u) return bits_to_f32(0x00400000u);
  return bits_to_f32((uint32_t)s << 23);
}

float vko_e2m1_value(int nibble) { return e2m1_value((unsigned)nibble & 15u); }
float vko_ue8m0_value(int s) { return ue8m0_value((uint8_t)s); }

/* dst[i] = RNE-bf16(src[i]) (dist_moe.cpp:334-343). */
void vko_round_bf16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_rne(src[i]);
}

/* ------------------------------------------------------------------ */
/* weight dequantisation                                                */
/* ------------------------------------------------------------------ */

/* One row of K packed weights -> K bf16 values held as float.
 * value = bf16(fp32(nibble) * fp32(scale)); low nibble is the even k
 * (moe_fused.cpp:153-171). */
static inline void dequant_row(const uint8_t* packed, const uint8_t* scale, int K, int group,
                               float* out) {
  for (int k = 0; k < K; k += 2) {
    float sc = ue8m0_value(scale[k / group]);
    uint8_t pb = packed[k >> 1];
    out[k] = bf16_to_f32(f32_to_bf16_rne(e2m1_value(pb & 15u) * sc));
    out[k + 1] = bf16_to_f32(f32_to_bf16_rne(e2m1_value(pb >> 4) * sc));
  }
}

/* [N, K/2] packed + [N, K/group] scales -> out[K][N] bf16 (transposed), with
 * the reference's stride arguments (moe_fused.cpp:141-201; both of its
 * variants produce these bits). */
void vko_dequant_weight_tile(const uint8_t* packed, const uint8_t* scale, uint16_t* out_bf16, int N,
                             int K, int group_size, int stride_packed, int stride_scale_n,
                             int stride_scale_k) {
  for (int n = 0; n < N; ++n) {
    for (int k = 0; k < K; ++k) {
      uint8_t pb = packed[(size_t)n * stride_packed + (k >> 1)];
      unsigned nib = (k & 1) ? (pb >> 4) : (pb & 15u);
      float sc = ue8m0_value(scale[(size_t)n * stride_scale_n + (size_t)(k / group_size) * stride_scale_k]);
      out_bf16[(size_t)k * N + n] = f32_to_bf16_rne(e2m1_value(nib) * sc);
    }
  }
}

/* ------------------------------------------------------------------ */
/* block GEMM core                                                      */
/* ------------------------------------------------------------------ */

/* acc[m] = sum over K blocks of (sequential 64-long dot), for the 16 rows of
 * one routed block against one weight row. at is the block's activations
 * transposed to [K][16] so the 16 independent row sums vectorise without
 * changing any single row's summation order. */
VKO_HOT static void block_row_dot(const float* at, const float* wrow, int K, float* acc) {
  for (int m = 0; m < VKO_BM; ++m) acc[m] = 0.0f;
  for (int kb = 0; kb < K; kb += VKO_BK) {
    float dot[VKO_BM];
    for (int m = 0; m < VKO_BM; ++m) dot[m] = 0.0f;
    for (int k = kb; k < kb + VKO_BK; ++k) {
      const float w = wrow[k];
      const float* a = at + (size_t)k * VKO_BM;
      for (int m = 0; m < VKO_BM; ++m) dot[m] += a[m] * w;
    }
    for (int m = 0; m < VKO_BM; ++m) acc[m] += dot[m];
  }
}

/* Generic "rows of a routed block times an expert's weight rows" stage shared
 * by the gate/up and down GEMMs.
 *   src_is_sorted = 0: activations are gathered from src[token = flat / top_k]
 *                      (gate/up, moe_fused.cpp:288-299)
 *   src_is_sorted = 1: activations are read at the sorted row itself
 *                      (down, moe_fused.cpp:469-480)
 * dst[EM, n_out] receives raw fp32 accumulators; padding rows of a live block
 * receive 0 and blocks whose expert id is negative are left untouched
 * (moe_fused.cpp:274-275,354-362). */
static void grouped_gemm(const uint16_t* src, int src_stride, int k_base, int src_is_sorted,
                         const uint8_t* w, const uint8_t* w_scale, const int32_t* sorted_ids,
                         const int32_t* expert_ids, float* dst, int M, int top_k, int EM, int K,
                         int n_out, int group) {
  const int N = M * top_k;
  const int n_blocks = EM / VKO_BM;
  const size_t w_expert = (size_t)n_out * (size_t)(K / 2);
  const size_t s_expert = (size_t)n_out * (size_t)(K / group);
#pragma omp parallel
  {
    float* at = (float*)malloc(sizeof(float) * (size_t)K * VKO_BM);
    float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(dynamic, 1)
    for (int mb = 0; mb < n_blocks; ++mb) {
      const int e = expert_ids[mb];
      if (e < 0) continue;
      const int r0 = mb * VKO_BM;
      int real[VKO_BM];
      for (int m = 0; m < VKO_BM; ++m) {
        const int flat = sorted_ids[r0 + m];
        real[m] = flat < N;
        const uint16_t* row = NULL;
        if (real[m]) {
          const size_t r = src_is_sorted ? (size_t)(r0 + m) : (size_t)(flat / top_k);
          row = src + r * (size_t)src_stride + k_base;
        }
        for (int k = 0; k < K; ++k) at[(size_t)k * VKO_BM + m] = row ? bf16_to_f32(row[k]) : 0.0f;
      }
      for (int n = 0; n < n_out; ++n) {
        dequant_row(w + (size_t)e * w_expert + (size_t)n * (K / 2),
                    w_scale + (size_t)e * s_expert + (size_t)n * (K / group), K, group, wrow);
        float acc[VKO_BM];
        block_row_dot(at, wrow, K, acc);
        for (int m = 0; m < VKO_BM; ++m)
          dst[(size_t)(r0 + m) * n_out + n] = real[m] ? acc[m] : 0.0f;
      }
    }
    free(at);
    free(wrow);
  }
}

/* Stage 0a: gate_up[EM, 2*ispp] = gather(A) @ w13^T (moe_fused.cpp:235-365).
 * Weight row n of w13 is output column n: gate rows first, then up rows. */
void vko_moe_gateup(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                    const int32_t* sorted_ids, const int32_t* expert_ids, float* gate_up, int M,
                    int a_stride, int k_base, int hidden_k, int ispp, int top_k, int EM,
                    int group_size) {
  grouped_gemm(A, a_stride, k_base, 0, w13, w13_scale, sorted_ids, expert_ids, gate_up, M, top_k,
               EM, hidden_k, 2 * ispp, group_size);
}

/* One (gate, up) pair through the epilogue (moe_fused.cpp:206-226). */
static inline float act_value(int activation, float g, float u, float limit, float beta,
                              float linear_beta) {
  if (activation == 1) { /* SiTU */
    float sig = 1.0f / (1.0f + expf(-g));
    float go = beta * tanhf(g / beta) * sig;
    float uo = (linear_beta > 0.0f) ? linear_beta * tanhf(u / linear_beta) : u;
    return go * uo;
  }
  if (limit > 0.0f) {
    if (g > limit) g = limit;
    if (u > limit) u = limit;
    if (u < -limit) u = -limit;
  }
  float silu = g / (1.0f + expf(-g));
  return silu * u;
}

/* Stage 0b: bias + activation, ONE rounding to bf16; padding rows and dead
 * blocks are never written (moe_fused.cpp:370-422). */
void vko_moe_act_epilogue(const float* gate_up, const float* b13, uint16_t* act,
                          const int32_t* sorted_ids, const int32_t* expert_ids, int M, int top_k,
                          int EM, int ispp, float swiglu_limit, int activation, float beta,
                          float linear_beta) {
  const int N = M * top_k;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < EM; ++r) {
    const int e = expert_ids[r / VKO_BM];
    if (e < 0 || sorted_ids[r] >= N) continue;
    const float* gu = gate_up + (size_t)r * 2 * ispp;
    for (int n = 0; n < ispp; ++n) {
      float g = gu[n], u = gu[ispp + n];
      if (b13) {
        g += b13[(size_t)e * 2 * ispp + n];
        u += b13[(size_t)e * 2 * ispp + ispp + n];
      }
      act[(size_t)r * ispp + n] =
          f32_to_bf16_rne(act_value(activation, g, u, swiglu_limit, beta, linear_beta));
    }
  }
}

/* Stage 1a: partial[EM, hidden] = act @ w2^T (moe_fused.cpp:427-518). */
void vko_moe_down(const uint16_t* act, const uint8_t* w2, const uint8_t* w2_scale,
                  const int32_t* sorted_ids, const int32_t* expert_ids, float* partial, int M,
                  int a_stride, int k_base, int ispp_k, int hidden, int top_k, int EM,
                  int group_size) {
  grouped_gemm(act, a_stride, k_base, 1, w2, w2_scale, sorted_ids, expert_ids, partial, M, top_k,
               EM, ispp_k, hidden, group_size);
}

/* Stage 1b: out[token] += (partial + b2) * weight, rows visited in sorted
 * order so each token accumulates its experts in ascending row order
 * (moe_fused.cpp:523-564). Threads split the columns, never the rows, which
 * keeps every output element's addition order. */
void vko_moe_combine(const float* partial, const float* b2, const float* topk_w_sorted,
                     const int32_t* sorted_ids, const int32_t* expert_ids, float* out, int M,
                     int hidden, int top_k, int EM) {
  const int N = M * top_k;
  const int chunk = 64;
#pragma omp parallel for schedule(static)
  for (int c0 = 0; c0 < hidden; c0 += chunk) {
    const int c1 = c0 + chunk < hidden ? c0 + chunk : hidden;
    for (int r = 0; r < EM; ++r) {
      const int e = expert_ids[r / VKO_BM];
      if (e < 0) continue;
      const int flat = sorted_ids[r];
      if (flat >= N) continue;
      const float wgt = topk_w_sorted[r];
      float* o = out + (size_t)(flat / top_k) * hidden;
      const float* p = partial + (size_t)r * hidden;
      for (int c = c0; c < c1; ++c) {
        float v = p[c];
        if (b2) v += b2[(size_t)e * hidden + c];
        v *= wgt;
        o[c] += v;
      }
    }
  }
}

/* The four stages composed (moe_fused.cpp:569-603). Returns 0, or -1 when the
 * fp32 temporaries cannot be allocated. If gate_up_dbg / partial_dbg are
 * non-NULL the raw accumulators are left there for the caller to inspect. */
int vko_fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                        const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                        const float* topk_w_sorted, const int32_t* expert_ids,
                        uint16_t* act_scratch, float* out, int M, int hidden, int ispp, int top_k,
                        int EM, int group_size, float swiglu_limit, int activation, float beta,
                        float linear_beta, const float* b13, const float* b2) {
  float* gate_up = (float*)malloc(sizeof(float) * (size_t)(EM > 0 ? EM : 1) * 2 * ispp);
  float* partial = (float*)malloc(sizeof(float) * (size_t)(EM > 0 ? EM : 1) * hidden);
  if (!gate_up || !partial) {
    free(gate_up);
    free(partial);
    return -1;
  }
  vko_moe_gateup(A, w13, w13_scale, sorted_ids, expert_ids, gate_up, M, hidden, 0, hidden, ispp,
                 top_k, EM, group_size);
  vko_moe_act_epilogue(gate_up, b13, act_scratch, sorted_ids, expert_ids, M, top_k, EM, ispp,
                       swiglu_limit, activation, beta, linear_beta);
  vko_moe_down(act_scratch, w2, w2_scale, sorted_ids, expert_ids, partial, M, ispp, 0, ispp,
               hidden, top_k, EM, group_size);
  vko_moe_combine(partial, b2, topk_w_sorted, sorted_ids, expert_ids, out, M, hidden, top_k, EM);
  free(gate_up);
  free(partial);
  return 0;
}

/* ------------------------------------------------------------------ */
/* alignment                                                            */
/* ------------------------------------------------------------------ */

/* Shared body of the two alignment contracts below. */
static int align_impl(const int32_t* topk_ids, const int32_t* expert_map, int N, int block_size,
                      int num_experts, int local_n, int32_t* sorted_ids, int32_t* expert_ids,
                      int cap_rows) {
  int* count = (int*)calloc((size_t)(local_n > 0 ? local_n : 1), sizeof(int));
  int* start = (int*)calloc((size_t)(local_n > 0 ? local_n : 1), sizeof(int));
  for (int i = 0; i < N; ++i) {
    int e = topk_ids[i];
    if (e < 0 || e >= num_experts) continue;
    if (expert_map) e = expert_map[e];
    if (e < 0 || e >= local_n) continue;
    count[e]++;
  }
  int EM = 0, blk = 0;
  for (int e = 0; e < local_n; ++e) {
    start[e] = EM;
    const int nb = (count[e] + block_size - 1) / block_size;
    for (int b = 0; b < nb; ++b, ++blk)
      if (cap_rows < 0 || (blk + 1) * block_size <= cap_rows) expert_ids[blk] = e;
    EM += nb * block_size;
  }
  const int lim = cap_rows < 0 ? EM : (EM < cap_rows ? EM : cap_rows);
  for (int i = 0; i < lim; ++i) sorted_ids[i] = N;
  for (int i = 0; i < N; ++i) {
    int e = topk_ids[i];
    if (e < 0 || e >= num_experts) continue;
    if (expert_map) e = expert_map[e];
    if (e < 0 || e >= local_n) continue;
    const int pos = start[e]++;
    if (cap_rows < 0 || pos < cap_rows) sorted_ids[pos] = i;
  }
  free(count);
  free(start);
  return EM;
}

/* Host alignment (moe_fused.cpp:609-661): flat indices grouped by expert in
 * ascending expert order, ascending flat index inside an expert, each expert
 * padded to block_size with the sentinel N = M*top_k; ids outside [0, E) are
 * dropped; returns EM (0 when nothing routes). */
int vko_moe_align_block_size(const int32_t* topk_ids, int M, int top_k, int block_size,
                             int num_experts, int32_t* sorted_ids, int32_t* expert_ids) {
  return align_impl(topk_ids, NULL, M * top_k, block_size, num_experts, num_experts, sorted_ids,
                    expert_ids, -1);
}

/* Device-alignment contract (moe_fused.hip:1983-2099 and
 * vllm_experts.py:297-372): optional global->local expert_map (-1 = skip),
 * local expert ids in expert_ids, every entry of sorted_ids[max_EM] /
 * expert_ids[max_EM/block_size] written (sentinels N / -1 beyond the real
 * rows), and an empty routing reports EM = block_size. */
int vko_moe_align_block_size_map(const int32_t* topk_ids, const int32_t* expert_map, int M,
                                 int top_k, int block_size, int num_experts, int local_n,
                                 int max_EM, int32_t* sorted_ids, int32_t* expert_ids) {
  const int N = M * top_k;
  for (int i = 0; i < max_EM; ++i) sorted_ids[i] = N;
  for (int i = 0; i < max_EM / block_size; ++i) expert_ids[i] = -1;
  int EM = align_impl(topk_ids, expert_map, N, block_size, num_experts, local_n, sorted_ids,
                      expert_ids, max_EM);
  if (EM == 0) EM = block_size;
  if (EM > max_EM) EM = max_EM;
  return EM;
}

/* ------------------------------------------------------------------ */
/* expert parallelism                                                   */
/* ------------------------------------------------------------------ */

/* Contiguous expert range of one rank: E/ep each, the first E%ep ranks take
 * one more (dist_moe.cpp:225-240). Returns 0, or -1 on a bad argument (the
 * reference throws invalid_argument there). */
int vko_moe_ep_plan(int num_experts, int ep, int rank, int* expert_begin, int* expert_end) {
  if (ep <= 0 || rank < 0 || rank >= ep || num_experts < ep) return -1;
  const int base = num_experts / ep, rem = num_experts % ep;
  const int begin = rank * base + (rank < rem ? rank : rem);
  *expert_begin = begin;
  *expert_end = begin + base + (rank < rem ? 1 : 0);
  return 0;
}

/* Local aligned layout of one rank: keep the (token, slot) pairs whose expert
 * is in [begin, end), align them, report LOCAL expert ids
 * (dist_moe.cpp:242-274). Buffers must hold M*top_k + (end-begin)*block_size
 * rows. Returns the local EM. */
int vko_moe_ep_dispatch(const int32_t* topk_ids, int M, int top_k, int num_experts,
                        int block_size, int expert_begin, int expert_end, int32_t* sorted_ids,
                        int32_t* expert_ids) {
  const int N = M * top_k;
  int32_t* masked = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N > 0 ? N : 1));
  for (int i = 0; i < N; ++i) {
    const int e = topk_ids[i];
    masked[i] = (e >= expert_begin && e < expert_end) ? e : -1;
  }
  const int EM =
      vko_moe_align_block_size(masked, M, top_k, block_size, num_experts, sorted_ids, expert_ids);
  for (int b = 0; b < EM / block_size; ++b)
    if (expert_ids[b] >= 0) expert_ids[b] -= expert_begin;
  free(masked);
  return EM;
}

/* ------------------------------------------------------------------ */
/* routing (no CPU counterpart in the reference; see the file header)   */
/* ------------------------------------------------------------------ */

/* logits[t, e] = sum_k fp32(x[t, k]) * Wr[e, k], fp32, k ascending. */
void vko_router_logits(const uint16_t* x, const float* wr, float* logits, int T, int H, int E) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    for (int e = 0; e < E; ++e) {
      float acc = 0.0f;
      const uint16_t* xr = x + (size_t)t * H;
      const float* w = wr + (size_t)e * H;
      for (int k = 0; k < H; ++k) acc += bf16_to_f32(xr[k]) * w[k];
      logits[(size_t)t * E + e] = acc;
    }
  }
}

/* k rounds of "largest remaining choice, lowest index on ties"
 * (routing.py:112-120, glm_router.py:70-76). */
static void pick_topk(const float* choice, int E, int k, int32_t* ids, unsigned char* used) {
  memset(used, 0, (size_t)E);
  for (int r = 0; r < k; ++r) {
    int best = -1;
    for (int e = 0; e < E; ++e) {
      if (used[e]) continue;
      if (best < 0 || choice[e] > choice[best]) best = e;
    }
    ids[r] = best;
    if (best >= 0) used[best] = 1;
  }
}

/* Smallest relative gap that decides the pick: between consecutive picks
 * (their ORDER is part of the result) and between the last pick and the best
 * unpicked entry. Inputs whose margin is below a few fp32 ulps cannot be
 * compared index-for-index across implementations that sum in another order. */
static float pick_margin(const float* choice, int E, int k, const int32_t* id,
                         const unsigned char* used) {
  float m = INFINITY;
  float next = -INFINITY;
  for (int e = 0; e < E; ++e)
    if (!used[e] && choice[e] > next) next = choice[e];
  if (k < E) {
    float kth = choice[id[k - 1]];
    m = (kth - next) / fmaxf(fabsf(kth), 1e-30f);
  }
  for (int r = 0; r + 1 < k; ++r) {
    float d = (choice[id[r]] - choice[id[r + 1]]) / fmaxf(fabsf(choice[id[r]]), 1e-30f);
    if (d < m) m = d;
  }
  return m;
}

/* Softmax top-k (routing.py:58-145): full-row softmax, selection on
 * score (+ bias), weight = unbiased score, optional renormalisation by the
 * selected sum (0 -> 1), then * scaling. margin (optional, [T]) receives the
 * relative gap between the k-th and (k+1)-th selection value. */
void vko_route_softmax_topk(const float* logits, const float* bias, int T, int E, int k,
                            int renorm, float scaling, int32_t* ids, float* w, float* margin) {
#pragma omp parallel
  {
    float* score = (float*)malloc(sizeof(float) * (size_t)E);
    float* choice = (float*)malloc(sizeof(float) * (size_t)E);
    unsigned char* used = (unsigned char*)malloc((size_t)E);
#pragma omp for schedule(static)
    for (int t = 0; t < T; ++t) {
      const float* l = logits + (size_t)t * E;
      float mx = l[0];
      for (int e = 1; e < E; ++e) mx = l[e] > mx ? l[e] : mx;
      float den = 0.0f;
      for (int e = 0; e < E; ++e) {
        score[e] = expf(l[e] - mx);
        den += score[e];
      }
      for (int e = 0; e < E; ++e) {
        score[e] = score[e] / den;
        choice[e] = bias ? score[e] + bias[e] : score[e];
      }
      int32_t* id = ids + (size_t)t * k;
      float* wt = w + (size_t)t * k;
      pick_topk(choice, E, k, id, used);
      float sum = 0.0f;
      for (int r = 0; r < k; ++r) {
        wt[r] = score[id[r]];
        sum += wt[r];
      }
      if (renorm) {
        if (sum == 0.0f) sum = 1.0f;
        for (int r = 0; r < k; ++r) wt[r] = wt[r] / sum;
      }
      for (int r = 0; r < k; ++r) wt[r] *= scaling;
      if (margin) margin[t] = pick_margin(choice, E, k, id, used);
    }
    free(score);
    free(choice);
    free(used);
  }
}

/* Sigmoid + bias, group-limited top-k (DeepSeek-V3 "noaux_tc" convention; the
 * per-expert part follows glm_router.py:184-201, the group step is this
 * build's choice because the reference declines n_group != 1,
 * glm_router.py:120-125):
 *   score  = 1 / (1 + exp(-logit))          choice = score + bias
 *   group score = sum of the two largest choice values in the group
 *   keep the topk_group best groups (lowest index on ties)
 *   pick k experts by choice inside the kept groups (lowest index on ties,
 *   descending order), weight = unbiased score
 *   renorm: w / (sum + 1e-20); then * scaling. */
void vko_route_sigmoid_group_topk(const float* logits, const float* bias, int T, int E, int k,
                                  int n_group, int topk_group, int renorm, float scaling,
                                  int32_t* ids, float* w, float* margin) {
  const int gs = E / n_group;
#pragma omp parallel
  {
    float* score = (float*)malloc(sizeof(float) * (size_t)E);
    float* choice = (float*)malloc(sizeof(float) * (size_t)E);
    float* gscore = (float*)malloc(sizeof(float) * (size_t)n_group);
    int32_t* gsel = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_group);
    unsigned char* used = (unsigned char*)malloc((size_t)(E > n_group ? E : n_group));
#pragma omp for schedule(static)
    for (int t = 0; t < T; ++t) {
      const float* l = logits + (size_t)t * E;
      for (int e = 0; e < E; ++e) {
        score[e] = 1.0f / (1.0f + expf(-l[e]));
        choice[e] = score[e] + (bias ? bias[e] : 0.0f);
      }
      float gmargin = INFINITY;
      if (n_group > 1) {
        for (int g = 0; g < n_group; ++g) {
          float a = -INFINITY, b = -INFINITY; /* a >= b: two largest */
          for (int e = g * gs; e < (g + 1) * gs; ++e) {
            const float c = choice[e];
            if (c > a) {
              b = a;
              a = c;
            } else if (c > b) {
              b = c;
            }
          }
          gscore[g] = (gs >= 2) ? a + b : a;
        }
        pick_topk(gscore, n_group, topk_group, gsel, used);
        if (topk_group < n_group) {
          float next = -INFINITY;
          for (int g = 0; g < n_group; ++g)
            if (!used[g] && gscore[g] > next) next = gscore[g];
          float kth = gscore[gsel[topk_group - 1]];
          gmargin = (kth - next) / fmaxf(fabsf(kth), 1e-30f);
        }
        for (int g = 0; g < n_group; ++g)
          if (!used[g])
            for (int e = g * gs; e < (g + 1) * gs; ++e) choice[e] = -INFINITY;
      }
      int32_t* id = ids + (size_t)t * k;
      float* wt = w + (size_t)t * k;
      pick_topk(choice, E, k, id, used);
      float sum = 0.0f;
      for (int r = 0; r < k; ++r) {
        wt[r] = score[id[r]];
        sum += wt[r];
      }
      if (renorm)
        for (int r = 0; r < k; ++r) wt[r] = wt[r] / (sum + 1.0e-20f);
      for (int r = 0; r < k; ++r) wt[r] *= scaling;
      if (margin) {
        float m = pick_margin(choice, E, k, id, used);
        margin[t] = m < gmargin ? m : gmargin;
      }
    }
    free(score);
    free(choice);
    free(gscore);
    free(gsel);
    free(used);
  }
}

int vko_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void vko_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
