// moe_gemv.cu - the layer for a handful of routed slots (one or two decode tokens).
//
// With four to sixteen (token, expert) slots the grouped tcgen05 GEMMs have a few dozen work
// items for 148 SMs (180 and 92 at one token of the gpt-oss shapes) and a pipeline whose fill
// and drain cost as much as its work, around five short helper kernels. Here the same
// arithmetic runs as two flat kernels with one warp per 16 weight rows of one slot, so every SM
// gets an equal share and nothing is sorted, tiled or staged:
//
//   1. gate/up + activation: a warp owns 8 features of one slot = 8 gate rows + 8 up rows; a
//      thread loads 16 bytes (32 codes = one scale group) of two of those rows per step,
//      expands them exactly to bf16 times scale (dequant8, the prefill forms' expansion) and
//      feeds them as the A operand of mma.sync.m16n8k16 (bf16, fp32 accumulate) against the
//      token's row in column 0 of B. K is taken in a permuted order that both operands share,
//      so no value ever moves between lanes. The thread that ends up with a feature's gate sum
//      holds its up sum too: bias, activation, one bf16 store.
//   2. down + ordered combine: a CTA owns 16 output features of one TOKEN, one warp pair per
//      slot (each half of K); the slots' sums meet in shared memory and are added in ascending
//      expert order (the CPU definition's order, reference moe_fused.cpp:539-562) times their
//      routing weights, then stored as bf16.
//
// The legacy tensor-core instruction is used on purpose: the kernels are bound by the weight
// bytes and by the integer work of the expansion, a 16 x 8 tile per warp is all the tensor work
// there is, and it needs no shared-memory or tensor-memory staging at all.
//
// Reference behaviour replaced: the launcher of moe_fused.hip:1448-1663 for M * top_k <= 16.
#include "common.cuh"
#include "moe_fused.hpp"

#include <atomic>
#include <cstdlib>
#include <string>

namespace vkernels::kernels::cuda {

namespace {

constexpr int kTinyMaxSlots = 16;

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// 16 weight rows (this thread: row_lo and row_hi, 8 rows apart in the tile) times one bf16
// vector over K elements [k_begin, k_end), a multiple of 32 each. Lane = 4 g + q: the thread
// takes the 32-element group at 128 c + 32 q of every 128-K step c; column 0 of B is the
// vector (threads with g == 0 carry it, read from shared memory), the other seven columns are
// zero. Returns the two sums of column 0 in the threads with q == 0 (c[0]: row_lo, c[2]: row_hi).
// The loads of the next kDepth steps are issued before the current ones are used: with ten
// warps to an SM it is the bytes in flight per warp that decide how close to the memory rate
// the kernel runs.
constexpr int kDepth = 3;
struct RowsBuf {
  uint4 a[kDepth], b[kDepth];
  uint32_t sa[kDepth], sb[kDepth];
};
__device__ __forceinline__ void rows16_load(RowsBuf& r, const uint8_t* __restrict__ w_lo, const uint8_t* __restrict__ w_hi,
                                            const uint8_t* __restrict__ s_lo, const uint8_t* __restrict__ s_hi, int k0,
                                            int k_end, int q) {
#pragma unroll
  for (int d = 0; d < kDepth; ++d) {
    const int k = k0 + 128 * d + 32 * q;
    r.a[d] = r.b[d] = make_uint4(0u, 0u, 0u, 0u);
    r.sa[d] = r.sb[d] = 0x7Fu;
    if (k < k_end) {
      r.a[d] = __ldcs(reinterpret_cast<const uint4*>(w_lo + (k >> 1)));
      r.b[d] = __ldcs(reinterpret_cast<const uint4*>(w_hi + (k >> 1)));
      r.sa[d] = s_lo[k >> 5];
      r.sb[d] = s_hi[k >> 5];
    }
  }
}
__device__ __forceinline__ void rows16_use(const RowsBuf& r, const uint16_t* vec_smem, int k0, int k_end, int q, bool carries,
                                           float (&c)[4]) {
#pragma unroll
  for (int d = 0; d < kDepth; ++d) {
    const int k = k0 + 128 * d + 32 * q;
    uint4 x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = make_uint4(0u, 0u, 0u, 0u);
    if (carries && k < k_end) {
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = *reinterpret_cast<const uint4*>(vec_smem + k + 8 * i);
    }
    const uint32_t s2a = ue8m0_to_bf16x2(r.sa[d]), s2b = ue8m0_to_bf16x2(r.sb[d]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // eight codes of each row -> two MMAs
      uint32_t va[4], vb[4];
      dequant8(word_of(r.a[d], i), s2a, va);
      dequant8(word_of(r.b[d], i), s2b, vb);
      mma_bf16_16x8x16(c, va[0], vb[0], va[1], vb[1], x[i].x, x[i].y);
      mma_bf16_16x8x16(c, va[2], vb[2], va[3], vb[3], x[i].z, x[i].w);
    }
  }
}
__device__ __forceinline__ void rows16_dot(const uint8_t* __restrict__ w_lo, const uint8_t* __restrict__ w_hi,
                                           const uint8_t* __restrict__ s_lo, const uint8_t* __restrict__ s_hi,
                                           const uint16_t* vec_smem, int k_begin, int k_end, int lane, float (&c)[4]) {
  const int q = lane & 3;
  const bool carries = (lane >> 2) == 0;
  constexpr int kGroup = 128 * kDepth;
  RowsBuf r0, r1;
  int k0 = k_begin;
  if (k0 >= k_end) return;
  rows16_load(r0, w_lo, w_hi, s_lo, s_hi, k0, k_end, q);
  while (true) {
    const int k1 = k0 + kGroup;
    if (k1 < k_end) rows16_load(r1, w_lo, w_hi, s_lo, s_hi, k1, k_end, q);
    rows16_use(r0, vec_smem, k0, k_end, q, carries, c);
    if (k1 >= k_end) break;
    const int k2 = k1 + kGroup;
    if (k2 < k_end) rows16_load(r0, w_lo, w_hi, s_lo, s_hi, k2, k_end, q);
    rows16_use(r1, vec_smem, k1, k_end, q, carries, c);
    if (k2 >= k_end) break;
    k0 = k2;
  }
}

// Expert of routed slot `s` (flat index token * top_k + j), from the alignment: the sorted row
// that holds s belongs to block r / block_size. -1 when the slot is not local (never aligned).
__device__ __forceinline__ int find_slot_expert(const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                                                int EM, int block_size, int s, int tid, int n_threads, int* s_found) {
  if (tid == 0) *s_found = -1;
  __syncthreads();
  for (int r = tid; r < EM; r += n_threads)
    if (sorted_ids[r] == s) *s_found = r;   // at most one row holds the slot
  __syncthreads();
  const int r = *s_found;
  return r < 0 ? -1 : expert_ids[r / block_size];
}

// K is cut into kParts pieces on 128-element boundaries; piece p of [0, K).
__device__ __forceinline__ void k_piece(int K, int parts, int p, int& k_begin, int& k_end) {
  const int len = ((K + parts - 1) / parts + 127) / 128 * 128;
  k_begin = p * len < K ? p * len : K;
  k_end = (p + 1) * len < K ? (p + 1) * len : K;
}

// grid (ispp / 32, N); 128 * kGateupParts threads = 4 feature warps (8 features each) x parts of
// K whose sums meet in shared memory and are added in part order. Measured at one token of the
// gpt-oss shapes: one part (four CTAs of four warps to an SM, all 360 CTAs resident at once) 21 us,
// four parts (one CTA of sixteen warps to an SM by registers, three waves) 26 us - the kernel
// is bound by instruction issue (integer pipe 51 % busy, 1.7 instructions per cycle), not by
// the number of loads in flight.
constexpr int kGateupParts = 1;
__global__ void __launch_bounds__(128 * kGateupParts)
gemv_gateup_kernel(const uint16_t* __restrict__ A, const uint8_t* __restrict__ w13, const uint8_t* __restrict__ w13_scale,
                   const float* __restrict__ b13, const int32_t* __restrict__ sorted_ids,
                   const int32_t* __restrict__ expert_ids, int EM, int block_size, int top_k, int hidden, int ispp,
                   int activation, float limit, float beta, float linear_beta, uint16_t* __restrict__ act,
                   int32_t* __restrict__ slot_expert) {
  __shared__ int s_found;
  __shared__ float part[4][kGateupParts][16];              // [feature warp][part][8 gate sums, 8 up sums]
  extern __shared__ __align__(16) uint16_t vec_smem[];   // the token's row [hidden]
  constexpr int kThreads = 128 * kGateupParts;
  const int s = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int fw = warp / kGateupParts, pt = warp % kGateupParts;
  {
    const uint4* src = reinterpret_cast<const uint4*>(A + (size_t)(s / top_k) * hidden);
    for (int i = tid; i < hidden / 8; i += kThreads) reinterpret_cast<uint4*>(vec_smem)[i] = src[i];
  }
  const int e = find_slot_expert(sorted_ids, expert_ids, EM, block_size, s, tid, kThreads, &s_found);   // (its barriers publish the row)
  if (blockIdx.x == 0 && tid == 0) slot_expert[s] = e;
  if (e < 0) return;
  const int f_warp = blockIdx.x * 32 + fw * 8;   // ispp is a multiple of 8: a warp's features are all in or all out
  if (f_warp < ispp) {
    const int g = lane >> 2;
    const size_t row_g = (size_t)e * 2 * ispp + f_warp + g, row_u = row_g + ispp;
    const int pitch = hidden / 2, spitch = hidden / 32;
    int k_begin, k_end;
    k_piece(hidden, kGateupParts, pt, k_begin, k_end);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    rows16_dot(w13 + row_g * pitch, w13 + row_u * pitch, w13_scale + row_g * spitch, w13_scale + row_u * spitch, vec_smem,
               k_begin, k_end, lane, c);
    if ((lane & 3) == 0) {
      part[fw][pt][g] = c[0];
      part[fw][pt][g + 8] = c[2];
    }
  }
  __syncthreads();
  if (tid < 32) {
    const int w = tid >> 3, g = tid & 7, f = blockIdx.x * 32 + w * 8 + g;
    if (f < ispp) {
      float gs = 0.0f, us = 0.0f;
#pragma unroll
      for (int p = 0; p < kGateupParts; ++p) {
        gs += part[w][p][g];
        us += part[w][p][g + 8];
      }
      if (b13 != nullptr) {
        gs += b13[(size_t)e * 2 * ispp + f];
        us += b13[(size_t)e * 2 * ispp + ispp + f];
      }
      act[(size_t)s * ispp + f] = f32_to_bf16_bits(moe_act_value(activation, gs, us, limit, beta, linear_beta));
    }
  }
}

// grid (hidden / 16, M); 32 * KSPLIT * top_k threads (at most 512): warp KSPLIT * j + h = slot j of
// the token, part h of K (two halves while top_k <= 8, else the whole of it).
template <int KSPLIT>
__global__ void __launch_bounds__(512)
gemv_down_kernel(const uint16_t* __restrict__ act, const uint8_t* __restrict__ w2, const uint8_t* __restrict__ w2_scale,
                 const float* __restrict__ b2, const float* __restrict__ topk_w, const int32_t* __restrict__ slot_expert,
                 int top_k, int hidden, int ispp, uint16_t* __restrict__ y) {
  __shared__ float part[kTinyMaxSlots][KSPLIT][16];
  __shared__ int s_e[kTinyMaxSlots];
  extern __shared__ __align__(16) uint16_t act_smem[];   // the token's activation rows [top_k][ispp]
  const int t = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int j = warp / KSPLIT, half = warp % KSPLIT;
  const int s = t * top_k + j;
  const int e = slot_expert[s];
  if (half == 0 && lane == 0) s_e[j] = e;
  {
    const uint4* src = reinterpret_cast<const uint4*>(act + (size_t)t * top_k * ispp);
    for (int i = tid; i < top_k * ispp / 8; i += blockDim.x) {
      const int jj = i / (ispp / 8);
      reinterpret_cast<uint4*>(act_smem)[i] = slot_expert[t * top_k + jj] >= 0 ? src[i] : make_uint4(0u, 0u, 0u, 0u);   // a skipped slot's row was never written
    }
  }
  __syncthreads();
  const int h0 = blockIdx.x * 16;
  if (e >= 0) {
    const int g = lane >> 2;
    const size_t row_lo = (size_t)e * hidden + h0 + g, row_hi = row_lo + 8;
    const int pitch = ispp / 2, spitch = ispp / 32;
    int k_begin, k_end;
    k_piece(ispp, KSPLIT, half, k_begin, k_end);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    rows16_dot(w2 + row_lo * pitch, w2 + row_hi * pitch, w2_scale + row_lo * spitch, w2_scale + row_hi * spitch,
               act_smem + (size_t)j * ispp, k_begin, k_end, lane, c);
    if ((lane & 3) == 0) {
      part[j][half][g] = c[0];
      part[j][half][g + 8] = c[2];
    }
  }
  __syncthreads();
  if (tid < 16) {
    const int h = h0 + tid;
    float acc = 0.0f;
    int last = -1;   // slots in ascending expert order (a token's experts are distinct)
    for (int n = 0; n < top_k; ++n) {
      int best = -1, best_e = 0x7FFFFFFF;
      for (int jj = 0; jj < top_k; ++jj) {
        const int ee = s_e[jj];
        if (ee > last && ee < best_e) {
          best_e = ee;
          best = jj;
        }
      }
      if (best < 0) break;
      last = best_e;
      float v = 0.0f;
#pragma unroll
      for (int p = 0; p < KSPLIT; ++p) v += part[best][p][tid];
      if (b2 != nullptr) v += b2[(size_t)best_e * hidden + h];
      acc += v * topk_w[t * top_k + best];
    }
    y[(size_t)t * hidden + h] = f32_to_bf16_bits(acc);
  }
}

bool tiny_mode() {
  static const bool on = [] {
    const char* e = std::getenv("VK_MOE_TINY");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return on;
}

}  // namespace

// Whether the flat two-kernel form serves this call (the bf16-output form of the layer only).
bool moe_tiny_eligible(int M, int hidden, int ispp, int top_k) {
  // up to twelve slots: beyond that the expansion, done once per SLOT here and once per EXPERT by the grouped GEMMs,
  // costs more than their pipeline overheads
  return tiny_mode() && M >= 1 && top_k >= 1 && top_k <= kTinyMaxSlots && (long long)M * top_k <= 12 &&
         hidden % 64 == 0 && ispp % 64 == 0 && hidden * 2 <= 48 * 1024 && (long long)top_k * ispp * 2 <= 200 * 1024;
}

// act: at least M * top_k rows of ispp bf16; slot_expert: M * top_k ints of scratch.
void launch_moe_tiny(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                     const uint8_t* w2_scale, const float* topk_w, uint16_t* act, uint16_t* y, int M, int hidden, int ispp,
                     int top_k, const int32_t* sorted_ids, const int32_t* expert_ids, int EM, float swiglu_limit,
                     int activation, float beta, float linear_beta, const float* b13, const float* b2, int block_size,
                     int32_t* slot_expert, cudaStream_t stream) {
  const int N = M * top_k;
  const size_t smem_down = (size_t)top_k * ispp * sizeof(uint16_t);
  expects((size_t)hidden * 2 <= 48 * 1024 && smem_down <= 200 * 1024, "fused_moe_mxfp4: dimensions too large for the flat form");
  if (smem_down > 48 * 1024) {
    static std::atomic<size_t> configured[64];
    int dev = 0;
    VK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || configured[dev].load() < smem_down) {
      VK_CUDA_CHECK(cudaFuncSetAttribute(gemv_down_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down));
      VK_CUDA_CHECK(cudaFuncSetAttribute(gemv_down_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down));
      if (dev >= 0 && dev < 64) configured[dev].store(smem_down);
    }
  }
  gemv_gateup_kernel<<<dim3((unsigned)((ispp + 31) / 32), (unsigned)N), 128 * kGateupParts, (size_t)hidden * sizeof(uint16_t), stream>>>(
      A, w13, w13_scale, b13, sorted_ids, expert_ids, EM, block_size, top_k, hidden, ispp, activation, swiglu_limit, beta,
      linear_beta, act, slot_expert);
  const dim3 grid_down((unsigned)(hidden / 16), (unsigned)M);
  if (top_k <= 8)
    gemv_down_kernel<2><<<grid_down, 64 * top_k, smem_down, stream>>>(act, w2, w2_scale, b2, topk_w, slot_expert, top_k, hidden,
                                                                    ispp, y);
  else
    gemv_down_kernel<1><<<grid_down, 32 * top_k, smem_down, stream>>>(act, w2, w2_scale, b2, topk_w, slot_expert, top_k, hidden,
                                                                    ispp, y);
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
