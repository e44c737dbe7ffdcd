// moe_ep.cu - device helpers of the expert-parallel layer: packing the rows a
// rank sends to each peer, and summing the rows that come back.
//
// Experts are partitioned in contiguous ranges (reference
// src/c/vkernels/dist/dist_moe.cpp:225-240). A token is sent ONCE to every
// rank that owns at least one of its experts, with its k (+ shared) slots
// rewritten to that rank's LOCAL expert ids (-1 for slots owned elsewhere, the
// masking rule of dist_moe.cpp:242-274). The receiving rank therefore sees an
// ordinary [rows, k] routing table and runs the single-GPU alignment and fused
// kernels on it; its fp32 result rows travel back in the same order and the
// home rank adds the at most `world` rows of a token in ascending rank order.
// The reference instead replicates the activations and sums dense per-rank
// outputs (dist_moe.cpp:276-328); the sum over ranks is the same quantity.
#include "common.cuh"
#include "moe_fused.hpp"

namespace vkernels::kernels::cuda {

namespace {

__device__ __forceinline__ int owner_rank(int e, const int32_t* begin, int world) {
  int r = 0;
  while (r + 1 < world && e >= begin[r + 1]) ++r;
  return r;
}

// One warp per token.
//   phase 0: cursor[d] += 1 for every rank d the token must visit
//   phase 1: cursor[d] holds the first free row of rank d's segment; the token
//            takes the next row, row_of[t, d] records it, the row is packed.
__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ topk_ids,
               const float* __restrict__ topk_w, int T, int H, int k, int n_shared, int world,
               int rank, const int32_t* __restrict__ expert_begin, int32_t* __restrict__ cursor,
               int32_t* __restrict__ row_of, uint16_t* __restrict__ send_x,
               int32_t* __restrict__ send_ids, float* __restrict__ send_w, int phase) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int slots = k + n_shared;
  unsigned need = n_shared > 0 ? (1u << rank) : 0u;
  for (int j = 0; j < k; ++j) {
    const int e = topk_ids[(size_t)t * k + j];
    if (e >= 0 && e < expert_begin[world]) need |= 1u << owner_rank(e, expert_begin, world);
  }
  for (int d = 0; d < world; ++d) {
    if (!((need >> d) & 1u)) {
      if (phase == 1 && lane == 0) row_of[(size_t)t * world + d] = -1;
      continue;
    }
    int row = 0;
    if (lane == 0) row = atomicAdd(&cursor[d], 1);
    if (phase == 0) continue;
    row = __shfl_sync(0xFFFFFFFFu, row, 0);
    if (lane == 0) row_of[(size_t)t * world + d] = row;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
    uint4* dst = reinterpret_cast<uint4*>(send_x + (size_t)row * H);
    for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
    const int b = expert_begin[d], e_end = expert_begin[d + 1];
    for (int j = lane; j < slots; j += 32) {
      int id = -1;
      float w = 0.0f;
      if (j < k) {
        const int e = topk_ids[(size_t)t * k + j];
        if (e >= b && e < e_end) {
          id = e - b;
          w = topk_w[(size_t)t * k + j];
        }
      } else if (d == rank) {
        id = (e_end - b) + (j - k);  // shared experts follow the local routed ones
        w = 1.0f;
      }
      send_ids[(size_t)row * slots + j] = id;
      send_w[(size_t)row * slots + j] = w;
    }
  }
}

// out[t, :] = sum over ranks d (ascending) of rows[row_of[t, d], :]
__global__ void __launch_bounds__(256)
ep_combine_kernel(const float* __restrict__ rows, const int32_t* __restrict__ row_of, int T, int H,
                  int world, uint16_t* __restrict__ out_bf16, float* __restrict__ out_f32) {
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int d = 0; d < world; ++d) {
      const int r = row_of[(size_t)t * world + d];
      if (r < 0) continue;
      const float4 v = *reinterpret_cast<const float4*>(rows + (size_t)r * H + c);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (out_f32) *reinterpret_cast<float4*>(out_f32 + (size_t)t * H + c) = acc;
    if (out_bf16) {
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(acc.x) | ((uint32_t)f32_to_bf16_bits(acc.y) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(acc.z) | ((uint32_t)f32_to_bf16_bits(acc.w) << 16);
      *reinterpret_cast<uint2*>(out_bf16 + (size_t)t * H + c) = o;
    }
  }
}

// out[r, k] = dequantised weight (bf16 bits); one thread per 8 elements.
__global__ void __launch_bounds__(256)
dequant_rows_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
                    uint16_t* __restrict__ out, int rows, int K) {
  const size_t words_per_row = K / 8;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * words_per_row) return;
  const size_t r = i / words_per_row, wq = i % words_per_row;
  const uint32_t word = reinterpret_cast<const uint32_t*>(packed + r * (K / 2))[wq];
  const uint32_t s = scale[r * (K / 32) + wq / 4];
  uint32_t o[4];
  dequant8(word, ue8m0_to_bf16x2(s), o);
  uint4* dst = reinterpret_cast<uint4*>(out + r * K + wq * 8);
  *dst = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace

void ep_launch_pack(const uint16_t* x, const int32_t* topk_ids, const float* topk_w, int T, int H,
                    int k, int n_shared, int world, int rank, const int32_t* expert_begin,
                    int32_t* cursor, int32_t* row_of, uint16_t* send_x, int32_t* send_ids,
                    float* send_w, int phase, cudaStream_t stream) {
  expects(T >= 0 && H > 0 && H % 8 == 0 && k > 0, "ep_pack: bad dimensions");
  expects(world >= 1 && world <= 32 && rank >= 0 && rank < world, "ep_pack: bad world/rank");
  expects(phase == 0 || phase == 1, "ep_pack: phase must be 0 or 1");
  if (T == 0) return;
  expects(x && topk_ids && topk_w && expert_begin && cursor, "ep_pack: null buffer");
  expects(phase == 0 || (row_of && send_x && send_ids && send_w), "ep_pack: null output buffer");
  ep_pack_kernel<<<(T + 7) / 8, 256, 0, stream>>>(x, topk_ids, topk_w, T, H, k, n_shared, world,
                                                  rank, expert_begin, cursor, row_of, send_x,
                                                  send_ids, send_w, phase);
  VK_CUDA_CHECK(cudaGetLastError());
}

void ep_launch_combine(const float* rows, const int32_t* row_of, int T, int H, int world,
                       uint16_t* out_bf16, float* out_f32, cudaStream_t stream) {
  expects(T >= 0 && H > 0 && H % 4 == 0 && world >= 1, "ep_combine: bad dimensions");
  if (T == 0) return;
  expects(rows && row_of && (out_bf16 || out_f32), "ep_combine: null buffer");
  ep_combine_kernel<<<T, 256, 0, stream>>>(rows, row_of, T, H, world, out_bf16, out_f32);
  VK_CUDA_CHECK(cudaGetLastError());
}

void launch_dequant_rows(const uint8_t* packed, const uint8_t* scale, uint16_t* out, int rows,
                         int K, cudaStream_t stream) {
  const size_t n = (size_t)rows * (K / 8);
  dequant_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(packed, scale, out, rows, K);
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
