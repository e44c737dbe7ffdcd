// moe_prep.cuh - device building blocks shared by the routing and alignment kernels: the
// per-token router (one warp), and the stable counting sort by expert of one 1024-entry chunk.
#pragma once

#include "common.cuh"

namespace vkernels::kernels::cuda {
namespace prep {

// One warp per token. Expert e lives in lane e % 32, slot e / 32.
constexpr int kMaxSlots = 32;  // E <= 1024

struct Best {
  float v;
  int i;
};
// larger value wins; equal values: lower index wins
__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    Best o{__shfl_xor_sync(0xFFFFFFFFu, x.v, d), __shfl_xor_sync(0xFFFFFFFFu, x.i, d)};
    x = better(x, o);
  }
  return x;
}

// Routing of ONE token by a whole warp (expert e lives in lane e % 32, slot e / 32): softmax or
// sigmoid (+ bias, optionally group-limited) scores, k rounds of arg-max with removal (lowest
// index on ties), renormalisation, scaling; writes ids / w [k + n_shared] for the token.
template <int SLOTS>
__device__ __forceinline__ void route_token(const float* __restrict__ l, const float* __restrict__ bias, int E, int k,
                                            int sigmoid, int n_group, int topk_group, int renorm, float scaling,
                                            int n_shared, int lane, int32_t* __restrict__ ids_t, float* __restrict__ w_t) {
  const float NEG = -INFINITY;
  float score[SLOTS], choice[SLOTS];
  if (!sigmoid) {
    float mx = NEG;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      score[s] = (e < E) ? l[e] : NEG;
      mx = fmaxf(mx, score[s]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, d));
    float den = 0.0f;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      score[s] = (e < E) ? expf(score[s] - mx) : 0.0f;
      den += score[s];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) den += __shfl_xor_sync(0xFFFFFFFFu, den, d);
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      score[s] = score[s] / den;
      choice[s] = (e < E) ? (bias ? score[s] + bias[e] : score[s]) : NEG;
    }
  } else {
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      if (e < E) {
        score[s] = 1.0f / (1.0f + expf(-l[e]));
        choice[s] = score[s] + (bias ? bias[e] : 0.0f);
      } else {
        score[s] = 0.0f;
        choice[s] = NEG;
      }
    }
    if (n_group > 1) {
      const int gs = E / n_group;
      // group score = sum of the two largest choices of the group
      // (lane g keeps group g's score; n_group <= 32)
      float my_gscore = NEG;
      for (int g = 0; g < n_group; ++g) {
        float a = NEG, b = NEG;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
          const int e = s * 32 + lane;
          if (e < E && e / gs == g) {
            const float c = choice[s];
            if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
          }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
          const float oa = __shfl_xor_sync(0xFFFFFFFFu, a, d);
          const float ob = __shfl_xor_sync(0xFFFFFFFFu, b, d);
          // merge two (largest, second) pairs
          const float na = fmaxf(a, oa);
          const float nb = fmaxf(fminf(a, oa), fmaxf(b, ob));
          a = na;
          b = nb;
        }
        const float gsc = (gs >= 2) ? a + b : a;
        if (lane == g) my_gscore = gsc;
      }
      unsigned keep = 0;  // bit g set = group g stays eligible
      for (int r = 0; r < topk_group; ++r) {
        // a taken group competes with index INT_MAX so it cannot win again
        const bool open = lane < n_group && !((keep >> lane) & 1u);
        Best x = warp_best(Best{open ? my_gscore : NEG, open ? lane : 0x7FFFFFFF});
        if (x.i < n_group) keep |= 1u << x.i;
      }
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (e < E && !((keep >> (e / gs)) & 1u)) choice[s] = NEG;
      }
    }
  }
  // k rounds of arg-max with removal
  const int kk = k + n_shared;
  float sum = 0.0f;
  float my_w = 0.0f;  // lane r keeps the weight of pick r (k <= 32)
  int my_id = 0;
  unsigned used = 0;  // bit s set = this lane's slot s already picked
  for (int r = 0; r < k; ++r) {
    Best x{NEG, 0x7FFFFFFF};
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int e = s * 32 + lane;
      if (e < E && !((used >> s) & 1u)) x = better(x, Best{choice[s], e});
    }
    x = warp_best(x);
    float sc = 0.0f;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s)
      if (s * 32 + lane == x.i) {
        used |= 1u << s;
        sc = score[s];
      }
    sc = __shfl_sync(0xFFFFFFFFu, sc, x.i & 31);
    sum += sc;  // same order on every lane: pick 0, pick 1, ...
    if (lane == r) {
      my_w = sc;
      my_id = x.i;
    }
  }
  if (renorm) {
    if (sigmoid) {
      my_w = my_w / (sum + 1.0e-20f);
    } else {
      if (sum == 0.0f) sum = 1.0f;
      my_w = my_w / sum;
    }
  }
  my_w *= scaling;
  if (lane < k) {
    ids_t[lane] = my_id;
    w_t[lane] = my_w;
  } else if (lane < kk) {
    ids_t[lane] = E + (lane - k);
    w_t[lane] = 1.0f;
  }
}

constexpr int kChunk = 1024;   // entries per chunk = threads per CTA
constexpr int kWarps = kChunk / 32;

__device__ __forceinline__ int local_expert(const int32_t* topk_ids, const int32_t* expert_map,
                                            int i, int N, int num_experts, int local_n) {
  if (i >= N) return -1;
  int e = topk_ids[i];
  if (e < 0 || e >= num_experts) return -1;
  if (expert_map != nullptr) e = expert_map[e];
  return (e < 0 || e >= local_n) ? -1 : e;
}

// Rank of each thread's entry among the chunk's entries with the same expert
// (entries ordered by thread index), plus the chunk histogram in hist[0][*].
//   warp_hist: [kWarps + 1][local_n] ints of shared memory.
// On return warp_hist[w][e] = number of entries of expert e in warps < w and
// warp_hist[kWarps][e] = the chunk total.
__device__ __forceinline__ int chunk_rank(int le, int local_n, int* warp_hist) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < (kWarps + 1) * local_n; i += kChunk) warp_hist[i] = 0;
  __syncthreads();
  // peers = lanes of this warp holding the same expert (le = -1 groups too, ignored below)
  const unsigned peers = __match_any_sync(0xFFFFFFFFu, le);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (le >= 0 && rank_in_warp == 0) warp_hist[warp * local_n + le] = __popc(peers);
  __syncthreads();
  // exclusive scan over warps, one thread per expert
  for (int e = tid; e < local_n; e += kChunk) {
    int run = 0;
    for (int w = 0; w < kWarps; ++w) {
      int c = warp_hist[w * local_n + e];
      warp_hist[w * local_n + e] = run;
      run += c;
    }
    warp_hist[kWarps * local_n + e] = run;
  }
  __syncthreads();
  return le >= 0 ? warp_hist[warp * local_n + le] + rank_in_warp : 0;
}

// Exclusive scan of padded expert sizes by one CTA; writes expert_ids for the
// real blocks, the row offset of every expert, and *out_em.
//   count[e] : entries of expert e (shared or global)
//   offset[e]: receives the first sorted row of expert e
__device__ __forceinline__ void scan_experts(const int* count, int* offset, int local_n,
                                             int block_size, int max_EM, int32_t* expert_ids,
                                             int32_t* out_em, int* s_tmp /* [kChunk] */) {
  const int tid = threadIdx.x;
  // each thread owns a contiguous slice of experts
  const int per = (local_n + kChunk - 1) / kChunk;
  const int e0 = tid * per, e1 = min(local_n, e0 + per);
  int mine = 0;
  for (int e = e0; e < e1; ++e) mine += ((count[e] + block_size - 1) / block_size) * block_size;
  // inclusive scan over the 1024 per-thread sums: shuffles inside each warp, then the 32 warp
  // totals by the first warp (two barriers instead of one per doubling step)
  const int lane_ = tid & 31, warp_ = tid >> 5;
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if (lane_ >= d) incl += v;
  }
  if (lane_ == 31) s_tmp[warp_] = incl;
  __syncthreads();
  if (warp_ == 0) {
    int t = s_tmp[lane_];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xFFFFFFFFu, t, d);
      if (lane_ >= d) t += v;
    }
    s_tmp[32 + lane_] = t;   // inclusive totals of warps 0..lane
  }
  __syncthreads();
  incl += warp_ > 0 ? s_tmp[32 + warp_ - 1] : 0;
  const int grand_total = s_tmp[32 + 31];
  int run = incl - mine;
  const int max_blocks = max_EM / block_size;
  for (int e = e0; e < e1; ++e) {
    offset[e] = run;
    const int nb = (count[e] + block_size - 1) / block_size;
    for (int b = 0; b < nb; ++b) {
      const int blk = run / block_size + b;
      if (blk < max_blocks) expert_ids[blk] = e;
    }
    run += nb * block_size;
  }
  if (tid == kChunk - 1) {
    int EM = grand_total;
    if (EM == 0) EM = block_size;
    if (EM > max_EM) EM = max_EM;
    *out_em = EM;
  }
  __syncthreads();
}

}  // namespace prep
}  // namespace vkernels::kernels::cuda
