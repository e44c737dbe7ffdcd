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

// Routing records for the peer-memory form of expert parallelism: nothing but the routing
// travels through the collective; the token rows themselves are read (and the results added)
// directly in the home rank's memory by the expert kernels.
// meta row (1 + 2 * slots int32): home token index, local expert id per slot (-1 = not this
// rank's), routing weight bits per slot. One thread per token; cursor as in ep_pack phase 1.
__global__ void __launch_bounds__(256)
ep_pack_meta_kernel(const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w, int T,
                    int k, int n_shared, int world, int rank, const int32_t* __restrict__ expert_begin,
                    int32_t* __restrict__ cursor, int32_t* __restrict__ meta) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int slots = k + n_shared, stride = 1 + 2 * slots;
  unsigned need = n_shared > 0 ? (1u << rank) : 0u;
  for (int j = 0; j < k; ++j) {
    const int e = topk_ids[(size_t)t * k + j];
    if (e >= 0 && e < expert_begin[world]) need |= 1u << owner_rank(e, expert_begin, world);
  }
  for (int d = 0; d < world; ++d) {
    if (!((need >> d) & 1u)) continue;
    const int row = atomicAdd(&cursor[d], 1);
    int32_t* m = meta + (size_t)row * stride;
    m[0] = t;
    const int b = expert_begin[d], e_end = expert_begin[d + 1];
    for (int j = 0; j < slots; ++j) {
      int id = -1;
      float w = 0.0f;
      if (j < k) {
        const int e = topk_ids[(size_t)t * k + j];
        if (e >= b && e < e_end) {
          id = e - b;
          w = topk_w[(size_t)t * k + j];
        }
      } else if (d == rank) {
        id = (e_end - b) + (j - k);
        w = 1.0f;
      }
      m[1 + j] = id;
      m[1 + slots + j] = __float_as_int(w);
    }
  }
}

// Received records -> routing arrays of the local expert call plus, per received row, the
// address of the token's activation row and of its fp32 output row in the home rank's memory.
// Rows arrive grouped by source rank: recv_counts[s] rows from rank s, in rank order.
__global__ void __launch_bounds__(256)
ep_unpack_meta_kernel(const int32_t* __restrict__ meta, int R, int slots,
                      const int32_t* __restrict__ recv_counts, int world,
                      const unsigned long long* __restrict__ x_bases,
                      const unsigned long long* __restrict__ out_bases, int H,
                      int32_t* __restrict__ ids, float* __restrict__ w,
                      unsigned long long* __restrict__ a_rows, unsigned long long* __restrict__ out_rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  int src = 0, first = 0;
  for (; src < world - 1; ++src) {
    const int n = recv_counts[src];
    if (r < first + n) break;
    first += n;
  }
  const int32_t* m = meta + (size_t)r * (1 + 2 * slots);
  const unsigned long long tok = (unsigned long long)m[0];
  a_rows[r] = x_bases[src] + tok * (unsigned long long)H * sizeof(uint16_t);
  out_rows[r] = out_bases[src] + tok * (unsigned long long)H * sizeof(float);
  for (int j = 0; j < slots; ++j) {
    ids[(size_t)r * slots + j] = m[1 + j];
    w[(size_t)r * slots + j] = __int_as_float(m[1 + slots + j]);
  }
}

// Host-free variant of the two kernels above: every rank owns a receive area of `world`
// segments of `cap` records (one per source rank) in memory all ranks can address. A source
// writes its records for rank d straight into its segment of d's area (peer stores) and then
// publishes how many it wrote; no collective call and no host read is needed, and the expert
// call afterwards runs over all world * cap record slots, the unused ones marked as not routed.
__global__ void __launch_bounds__(256)
ep_pack_meta_peer_kernel(const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w, int T,
                         int k, int n_shared, int world, int rank,
                         const int32_t* __restrict__ expert_begin, int32_t* __restrict__ cursor,
                         const unsigned long long* __restrict__ meta_bases, int cap) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int slots = k + n_shared, stride = 1 + 2 * slots;
  unsigned need = n_shared > 0 ? (1u << rank) : 0u;
  for (int j = 0; j < k; ++j) {
    const int e = topk_ids[(size_t)t * k + j];
    if (e >= 0 && e < expert_begin[world]) need |= 1u << owner_rank(e, expert_begin, world);
  }
  for (int d = 0; d < world; ++d) {
    if (!((need >> d) & 1u)) continue;
    const int row = atomicAdd(&cursor[d], 1);
    if (row >= cap) continue;   // cannot happen: a token sends at most one record per rank
    int32_t* m = reinterpret_cast<int32_t*>(meta_bases[d]) + ((size_t)rank * cap + row) * stride;
    m[0] = t;
    const int b = expert_begin[d], e_end = expert_begin[d + 1];
    for (int j = 0; j < slots; ++j) {
      int id = -1;
      float w = 0.0f;
      if (j < k) {
        const int e = topk_ids[(size_t)t * k + j];
        if (e >= b && e < e_end) {
          id = e - b;
          w = topk_w[(size_t)t * k + j];
        }
      } else if (d == rank) {
        id = (e_end - b) + (j - k);
        w = 1.0f;
      }
      m[1 + j] = id;
      m[1 + slots + j] = __float_as_int(w);
    }
  }
}

__global__ void ep_publish_counts_kernel(int32_t* __restrict__ cursor,
                                         const unsigned long long* __restrict__ count_bases, int world,
                                         int rank) {
  const int d = threadIdx.x;
  if (d < world) {
    reinterpret_cast<int32_t*>(count_bases[d])[rank] = cursor[d];
    cursor[d] = 0;   // ready for the next step: the caller zeroes it only once
  }
}

__global__ void __launch_bounds__(256)
ep_unpack_meta_peer_kernel(const int32_t* __restrict__ meta, const int32_t* __restrict__ recv_counts,
                           int world, int cap, int slots, const unsigned long long* __restrict__ x_bases,
                           const unsigned long long* __restrict__ out_bases, int H, int out_rows_per_token,
                           int32_t* __restrict__ ids, float* __restrict__ w,
                           unsigned long long* __restrict__ a_rows, unsigned long long* __restrict__ out_rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= world * cap) return;
  const int src = r / cap, i = r - src * cap;
  const bool valid = i < recv_counts[src];
  const int32_t* m = meta + (size_t)r * (1 + 2 * slots);
  const unsigned long long tok = valid ? (unsigned long long)m[0] : 0ull;
  a_rows[r] = x_bases[src] + tok * (unsigned long long)H * sizeof(uint16_t);
  out_rows[r] = out_bases[src] + tok * (unsigned long long)out_rows_per_token * H * sizeof(float);
  for (int j = 0; j < slots; ++j) {
    ids[(size_t)r * slots + j] = valid ? m[1 + j] : -1;
    w[(size_t)r * slots + j] = valid ? __int_as_float(m[1 + slots + j]) : 0.0f;
  }
}

// Home-rank combine of the slot-store form: part[t, j, :] holds the unweighted result row of
// token t's slot j, stored there by whichever rank owns that expert. y[t, :] = bf16( sum over the
// slots in ascending GLOBAL expert id - the order in which the single-rank CPU definition adds
// (reference moe_fused.cpp:539-562), and with contiguous expert ranges also ascending rank order
// - of w[t, j] * part[t, j, :] ). No atomics anywhere: the result is bit-reproducible. Slots whose
// id is outside [0, n_experts) were never written and are skipped.
__global__ void __launch_bounds__(256)
ep_combine_slots_kernel(const float* __restrict__ part, const int32_t* __restrict__ ids, const float* __restrict__ w,
                        int k, int n_experts, int H, uint16_t* __restrict__ y_bf16, float* __restrict__ out_f32) {
  __shared__ int s_slot[32];
  __shared__ float s_w[32];
  __shared__ int s_n;
  const int t = blockIdx.x;
  if (threadIdx.x < 32) {
    const int j = threadIdx.x;
    int e = -1;
    float wj = 0.0f;
    if (j < k) {
      e = ids[(size_t)t * k + j];
      wj = w[(size_t)t * k + j];
      if (e < 0 || e >= n_experts) e = -1;
    }
    const unsigned valid = __ballot_sync(0xFFFFFFFFu, e >= 0);
    int rank = 0;
    for (int o = 0; o < k; ++o) {
      const int eo = __shfl_sync(0xFFFFFFFFu, e, o);
      if (eo >= 0 && (eo < e || (eo == e && o < j))) ++rank;
    }
    if (e >= 0) {
      s_slot[rank] = j;
      s_w[rank] = wj;
    }
    if (j == 0) s_n = __popc(valid);
  }
  __syncthreads();
  const int n = s_n;
  const float* base = part + (size_t)t * k * H;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < n; ++i) {
      const float4 v = *reinterpret_cast<const float4*>(base + (size_t)s_slot[i] * H + c);
      const float wi = s_w[i];
      acc.x += v.x * wi; acc.y += v.y * wi; acc.z += v.z * wi; acc.w += v.w * wi;
    }
    if (out_f32 != nullptr) *reinterpret_cast<float4*>(out_f32 + (size_t)t * H + c) = acc;
    if (y_bf16 != nullptr) {
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(acc.x) | ((uint32_t)f32_to_bf16_bits(acc.y) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(acc.z) | ((uint32_t)f32_to_bf16_bits(acc.w) << 16);
      *reinterpret_cast<uint2*>(y_bf16 + (size_t)t * H + c) = o;
    }
  }
}

// ---------------------------------------------------------------------------
// Cross-rank barrier on flags in peer-visible memory, with bounded waits
// ---------------------------------------------------------------------------
// Every rank owns a flag array [slots][world] of int32 that all ranks can address. Thread d of
// the single CTA first publishes this rank's arrival - `epoch` stored with system-scope release
// into entry [slot][rank] of rank d's array, after a system-scope fence that orders every
// earlier write of this stream (peer stores included) before it - and then waits, with a
// system-scope acquire load, until entry [slot][d] of its OWN array has reached `epoch`.
// Epochs only grow, so nothing is ever reset. The wait is limited to `limit_clocks` SM clocks:
// a rank that never arrives makes the others record a status (200 + the missing rank) and
// return instead of spinning, and the host reads that status before trusting the step.
__device__ int g_ep_status;

// `epoch_counter` (optional): the epoch is taken from device memory instead of the argument -
// entry [slot] is incremented by every call and its new value used - so a captured graph can
// replay the barrier; every rank must then call the barrier the same number of times.
__global__ void __launch_bounds__(32)
ep_flag_barrier_kernel(const unsigned long long* __restrict__ flag_bases, int world, int rank, int slot,
                       int epoch, long long limit_clocks, int* __restrict__ epoch_counter) {
  const int d = threadIdx.x;
  if (epoch_counter != nullptr) {
    int e = 0;
    if (d == 0) e = atomicAdd(epoch_counter + slot, 1) + 1;
    epoch = __shfl_sync(0xFFFFFFFFu, e, 0);
  }
  if (d >= world) return;
  __threadfence_system();
  int* theirs = reinterpret_cast<int*>(flag_bases[d]) + slot * world + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const int* mine = reinterpret_cast<const int*>(flag_bases[rank]) + slot * world + d;
  const long long t0 = clock64();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v - epoch >= 0) break;
    if (clock64() - t0 > limit_clocks) {
      atomicExch(&g_ep_status, 200 + d);
      break;
    }
    __nanosleep(64);
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

// The same rows through the table expansion of the lone-CTA GEMM form: one thread per 64
// K-elements (two 16-byte chunks, one scale each), table built per CTA exactly as the GEMM does.
__global__ void __launch_bounds__(256)
dequant_rows_lut_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
                        uint16_t* __restrict__ out, int rows, int K) {
  __shared__ uint32_t lut[256 * 32];
  fill_dequant_lut(lut, threadIdx.x, blockDim.x);
  __syncthreads();
  const size_t pieces_per_row = K / 64;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * pieces_per_row) return;
  const size_t r = i / pieces_per_row, pc = i % pieces_per_row;
  const uint4* src = reinterpret_cast<const uint4*>(packed + r * (K / 2) + pc * 32);
  const uint32_t s0 = ue8m0_to_bf16x2(scale[r * (K / 32) + pc * 2]);
  const uint32_t s1 = ue8m0_to_bf16x2(scale[r * (K / 32) + pc * 2 + 1]);
  uint32_t v[32];
  const uint32_t lut_lane = static_cast<uint32_t>(__cvta_generic_to_shared(lut)) + (threadIdx.x & 31u) * 4u;
  dequant64_lut(src[0], src[1], s0, s1, lut_lane, v);
  uint4* dst = reinterpret_cast<uint4*>(out + r * K + pc * 64);
#pragma unroll
  for (int j = 0; j < 8; ++j) dst[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
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

void ep_launch_pack_meta(const int32_t* topk_ids, const float* topk_w, int T, int k, int n_shared,
                         int world, int rank, const int32_t* expert_begin, int32_t* cursor,
                         int32_t* meta, cudaStream_t stream) {
  expects(T >= 0 && k > 0 && n_shared >= 0, "ep_pack_meta: bad dimensions");
  expects(world >= 1 && world <= 32 && rank >= 0 && rank < world, "ep_pack_meta: bad world/rank");
  if (T == 0) return;
  expects(topk_ids && topk_w && expert_begin && cursor && meta, "ep_pack_meta: null buffer");
  ep_pack_meta_kernel<<<(T + 255) / 256, 256, 0, stream>>>(topk_ids, topk_w, T, k, n_shared, world, rank,
                                                           expert_begin, cursor, meta);
  VK_CUDA_CHECK(cudaGetLastError());
}

void ep_launch_unpack_meta(const int32_t* meta, int R, int slots, const int32_t* recv_counts, int world,
                           const unsigned long long* x_bases, const unsigned long long* out_bases,
                           int H, int32_t* ids, float* w, unsigned long long* a_rows,
                           unsigned long long* out_rows, cudaStream_t stream) {
  expects(R >= 0 && slots > 0 && world >= 1 && world <= 32 && H > 0 && H % 8 == 0,
          "ep_unpack_meta: bad dimensions");
  if (R == 0) return;
  expects(meta && recv_counts && x_bases && out_bases && ids && w && a_rows && out_rows,
          "ep_unpack_meta: null buffer");
  ep_unpack_meta_kernel<<<(R + 255) / 256, 256, 0, stream>>>(meta, R, slots, recv_counts, world, x_bases,
                                                             out_bases, H, ids, w, a_rows, out_rows);
  VK_CUDA_CHECK(cudaGetLastError());
}

void ep_launch_pack_meta_peer(const int32_t* topk_ids, const float* topk_w, int T, int k, int n_shared,
                              int world, int rank, const int32_t* expert_begin, int32_t* cursor,
                              const unsigned long long* meta_bases, const unsigned long long* count_bases,
                              int cap, cudaStream_t stream) {
  expects(T >= 0 && k > 0 && n_shared >= 0 && cap >= T, "ep_pack_meta_peer: bad dimensions");
  expects(world >= 1 && world <= 32 && rank >= 0 && rank < world, "ep_pack_meta_peer: bad world/rank");
  expects(expert_begin && cursor && meta_bases && count_bases, "ep_pack_meta_peer: null buffer");
  if (T > 0) {
    expects(topk_ids && topk_w, "ep_pack_meta_peer: null buffer");
    ep_pack_meta_peer_kernel<<<(T + 255) / 256, 256, 0, stream>>>(topk_ids, topk_w, T, k, n_shared, world,
                                                                  rank, expert_begin, cursor, meta_bases, cap);
  }
  ep_publish_counts_kernel<<<1, 32, 0, stream>>>(cursor, count_bases, world, rank);
  VK_CUDA_CHECK(cudaGetLastError());
}

void ep_launch_unpack_meta_peer(const int32_t* meta, const int32_t* recv_counts, int world, int cap,
                                int slots, const unsigned long long* x_bases,
                                const unsigned long long* out_bases, int H, int out_rows_per_token, int32_t* ids,
                                float* w, unsigned long long* a_rows, unsigned long long* out_rows,
                                cudaStream_t stream) {
  expects(out_rows_per_token >= 1, "ep_unpack_meta_peer: out_rows_per_token must be positive");
  expects(cap > 0 && slots > 0 && world >= 1 && world <= 32 && H > 0 && H % 8 == 0,
          "ep_unpack_meta_peer: bad dimensions");
  expects(meta && recv_counts && x_bases && out_bases && ids && w && a_rows && out_rows,
          "ep_unpack_meta_peer: null buffer");
  const int n = world * cap;
  ep_unpack_meta_peer_kernel<<<(n + 255) / 256, 256, 0, stream>>>(meta, recv_counts, world, cap, slots,
                                                                  x_bases, out_bases, H, out_rows_per_token, ids,
                                                                  w, a_rows, out_rows);
  VK_CUDA_CHECK(cudaGetLastError());
}

void ep_launch_flag_barrier(const unsigned long long* flag_bases, int world, int rank, int slot, int epoch,
                            long long limit_clocks, int* epoch_counter, cudaStream_t stream) {
  expects(world >= 1 && world <= 32 && rank >= 0 && rank < world, "ep_flag_barrier: bad world/rank");
  expects(slot >= 0 && slot < 8 && flag_bases != nullptr, "ep_flag_barrier: bad slot or null flag table");
  expects(limit_clocks > 0 && limit_clocks <= 8000000000ll, "ep_flag_barrier: limit must be in (0, 8e9] clocks");
  ep_flag_barrier_kernel<<<1, 32, 0, stream>>>(flag_bases, world, rank, slot, epoch, limit_clocks, epoch_counter);
  VK_CUDA_CHECK(cudaGetLastError());
}

// 0, or 200 + the rank whose arrival a flag barrier gave up waiting for. Synchronises the device.
int ep_last_status() {
  int v = 0;
  VK_CUDA_CHECK(cudaDeviceSynchronize());
  VK_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_ep_status, sizeof(int)));
  return v;
}
void ep_reset_status() {
  const int zero = 0;
  VK_CUDA_CHECK(cudaDeviceSynchronize());
  VK_CUDA_CHECK(cudaMemcpyToSymbol(g_ep_status, &zero, sizeof(int)));
}

void ep_launch_combine_slots(const float* part, const int32_t* ids, const float* w, int T, int k, int n_experts, int H,
                             uint16_t* y_bf16, float* out_f32, cudaStream_t stream) {
  expects(T >= 0 && k >= 1 && k <= 32 && H > 0 && H % 4 == 0 && n_experts > 0, "ep_combine_slots: bad dimensions");
  if (T == 0) return;
  expects(part && ids && w && (y_bf16 || out_f32), "ep_combine_slots: null buffer");
  ep_combine_slots_kernel<<<T, 256, 0, stream>>>(part, ids, w, k, n_experts, H, y_bf16, out_f32);
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

// path 0: the byte-permute decoder (CTA-pair GEMM form); path 1: the table decoder (lone-CTA form).
void launch_dequant_rows(const uint8_t* packed, const uint8_t* scale, uint16_t* out, int rows,
                         int K, int path, cudaStream_t stream) {
  expects(path == 0 || path == 1, "mxfp4_dequant_rows: path must be 0 (permute) or 1 (table)");
  if (path == 0) {
    const size_t n = (size_t)rows * (K / 8);
    dequant_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(packed, scale, out, rows, K);
  } else {
    expects(K % 64 == 0, "mxfp4_dequant_rows: the table path takes K in multiples of 64");
    expects((reinterpret_cast<uintptr_t>(packed) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0,
            "mxfp4_dequant_rows: the table path needs 16-byte aligned buffers");
    const size_t n = (size_t)rows * (K / 64);
    dequant_rows_lut_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(packed, scale, out, rows, K);
  }
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
