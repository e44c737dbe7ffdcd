// moe_route.cu - router of the fused MoE layer: fp32 logits GEMM and top-k.
//
// The reference has no router inside moe_fused; the semantics here follow its
// GPU routing ops: softmax top-k with renormalised weights
// (src/python/vkernels/torch_ops/tokenspeed_amd/routing.py:58-145) and
// sigmoid + bias selection with unbiased weights
// (src/python/vkernels/torch_ops/glm_router.py:43-88,184-201). Ties go to the
// lowest expert index and ids come out in descending order of selection value.
// Group limiting (n_group > 1) is outside what the reference implements; the
// rule used is the DeepSeek-V3 one: a group's score is the sum of its two
// largest biased scores and only experts of the topk_group best groups stay
// eligible.
#include <algorithm>
#include <atomic>
#include "common.cuh"
#include "moe_fused.hpp"
#include "moe_prep.cuh"

namespace vkernels::kernels::cuda {

namespace {

// ----------------------------- logits ---------------------------------------
// logits[T, E] = x[T, H] (bf16) * wr[E, H]^T (fp32), fp32 accumulate.
// 64 x 64 output tile per CTA, 256 threads, 4 x 4 outputs per thread,
// K staged through shared memory 32 at a time.
constexpr int RT = 64, RE = 64, RK = 32;

__global__ void __launch_bounds__(256)
router_logits_kernel(const uint16_t* __restrict__ x, const float* __restrict__ wr,
                     float* __restrict__ logits, int T, int H, int E) {
  __shared__ float xs[RK][RT + 4];
  __shared__ float ws[RK][RE + 4];
  const int tid = threadIdx.x;
  const int t0 = blockIdx.x * RT, e0 = blockIdx.y * RE;
  const int tx = tid & 15, ty = tid >> 4;  // tx -> experts, ty -> tokens
  float acc[4][4] = {};
  for (int k0 = 0; k0 < H; k0 += RK) {
    // 64 rows x 32 k: thread loads row = tid / 4, 8 consecutive k
    {
      const int r = tid >> 2, kk = (tid & 3) * 8;
      const int t = t0 + r, e = e0 + r;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = k0 + kk + j;
        xs[kk + j][r] = (t < T && k < H) ? bf16_bits_to_f32(x[(size_t)t * H + k]) : 0.0f;
        ws[kk + j][r] = (e < E && k < H) ? wr[(size_t)e * H + k] : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < RK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + tx * 4 + j;
      if (e < E) logits[(size_t)t * E + e] = acc[i][j];
    }
  }
}

// ----------------------------- tensor-core router GEMM ----------------------
// Large batches. The fp32 router weight is split on the fly into three bf16 terms
// (w = hi + mid + lo exactly: 3 x 8 mantissa bits), the activations are bf16 already, so
// every product is exact in fp32. Partial sums over 64 K-elements are formed by
// mma.sync.m16n8k16 (smallest terms first) and added to the running fp32 totals in
// registers, which keeps the result within fp32 reassociation noise of a sequential fp32 dot.
// CTA: 64 tokens x ME experts (128 or 64), 8 warps as 4 (tokens) x 2 (experts); warp tile
// 16 x ME / 2. The narrower tile doubles the CTA count (and lets two CTAs share an SM) when the
// batch alone does not fill the machine.
constexpr int MT = 64, MK = 64, MPAD = 8;   // +8 bf16 per row: conflict-free ldmatrix
constexpr int MROW = MK + MPAD;

template <int ME>
struct RouterSmem {
  uint16_t x[2][MT][MROW];
  uint16_t w[2][3][ME][MROW];
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// w -> (hi, mid, lo) bf16 bit patterns with hi + mid + lo == w (round to nearest at each step)
__device__ __forceinline__ void split3(float w, uint16_t& hi, uint16_t& mid, uint16_t& lo) {
  hi = f32_to_bf16_bits(w);
  const float r1 = w - bf16_bits_to_f32(hi);
  mid = f32_to_bf16_bits(r1);
  const float r2 = r1 - bf16_bits_to_f32(mid);
  lo = f32_to_bf16_bits(r2);
}

template <int ME>
__global__ void __launch_bounds__(256)
router_logits_mma_kernel(const uint16_t* __restrict__ x, const float* __restrict__ wr,
                         float* __restrict__ logits, int T, int H, int E) {
  constexpr int NT = ME / 16;        // 8-expert MMA tiles per warp
  constexpr int WV = ME / 16;        // float4 loads of the weight tile per thread and chunk
  extern __shared__ __align__(16) uint8_t router_smem_raw[];
  RouterSmem<ME>& sm = *reinterpret_cast<RouterSmem<ME>*>(router_smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = blockIdx.x * MT, e0 = blockIdx.y * ME;
  const int wt = warp & 3, we = warp >> 2;   // warp tile: tokens wt*16.., experts we*(ME/2)..

  // global -> register staging of one K chunk: x 64 x 64 bf16 (2 x 16 B per thread),
  // w ME x 64 fp32 (ME / 16 x 16 B per thread)
  uint4 xr[2];
  float4 wv[WV];
  auto load_chunk = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * 256;           // 0..511: row = idx / 8, 8 bf16 at (idx % 8) * 8
      const int r = idx >> 3, c = (idx & 7) * 8;
      const int t = t0 + r, k = k0 + c;
      xr[i] = (t < T && k < H) ? *reinterpret_cast<const uint4*>(x + (size_t)t * H + k)
                               : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < WV; ++i) {
      const int idx = tid + i * 256;           // row = idx / 16, 4 fp32 at (idx % 16) * 4
      const int r = idx >> 4, c = (idx & 15) * 4;
      const int e = e0 + r, k = k0 + c;
      wv[i] = (e < E && k < H) ? *reinterpret_cast<const float4*>(wr + (size_t)e * H + k)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto store_chunk = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * 256;
      *reinterpret_cast<uint4*>(&sm.x[buf][idx >> 3][(idx & 7) * 8]) = xr[i];
    }
#pragma unroll
    for (int i = 0; i < WV; ++i) {
      const int idx = tid + i * 256;
      const int r = idx >> 4, c = (idx & 15) * 4;
      const float f[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
      uint16_t h[4], m[4], l[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) split3(f[j], h[j], m[j], l[j]);
      *reinterpret_cast<uint2*>(&sm.w[buf][0][r][c]) =
          make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
      *reinterpret_cast<uint2*>(&sm.w[buf][1][r][c]) =
          make_uint2((uint32_t)m[0] | ((uint32_t)m[1] << 16), (uint32_t)m[2] | ((uint32_t)m[3] << 16));
      *reinterpret_cast<uint2*>(&sm.w[buf][2][r][c]) =
          make_uint2((uint32_t)l[0] | ((uint32_t)l[1] << 16), (uint32_t)l[2] | ((uint32_t)l[3] << 16));
    }
  };

  float total[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) total[n][j] = 0.0f;

  // gridDim.z > 1 splits the reduction into slices so that a batch too small to fill the machine
  // still does: two slices are added into zeroed logits with atomics (a sum of two partials does
  // not depend on their order, so the result stays reproducible); more slices write one plane
  // [T, E] each (`logits` then has gridDim.z planes) and a second kernel adds the planes in order.
  const int all_chunks = (H + MK - 1) / MK;
  const int ch_begin = (int)blockIdx.z * all_chunks / (int)gridDim.z;
  const int n_chunks = ((int)blockIdx.z + 1) * all_chunks / (int)gridDim.z;
  load_chunk(ch_begin * MK);
  store_chunk(ch_begin & 1);
  __syncthreads();
  for (int ch = ch_begin; ch < n_chunks; ++ch) {
    const int buf = ch & 1;
    if (ch + 1 < n_chunks) load_chunk((ch + 1) * MK);
    float part[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[n][j] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < MK / 16; ++ks) {
      uint32_t a[4];
      // lanes 0-15: rows 0-15 at k, lanes 16-31: rows 0-15 at k + 8
      ldmatrix_x4(a, &sm.x[buf][wt * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int term = 2; term >= 0; --term) {   // lo, mid, hi
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {    // two 8-expert tiles per ldmatrix.x4
          uint32_t b[4];
          // matrices: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
          const int row = we * (ME / 2) + np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int col = ks * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(b, &sm.w[buf][term][row][col]);
          mma_bf16_16816(part[np * 2], a, b[0], b[1]);
          mma_bf16_16816(part[np * 2 + 1], a, b[2], b[3]);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) total[n][j] += part[n][j];
    if (ch + 1 < n_chunks) store_chunk(buf ^ 1);
    __syncthreads();
  }
  // c fragment: rows lane / 4 and + 8, columns (lane % 4) * 2 and + 1
  const int r0 = t0 + wt * 16 + (lane >> 2);
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int e = e0 + we * (ME / 2) + n * 8 + (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int t = r0 + half * 8;
      if (t >= T) continue;
      if (gridDim.z != 2) {
        float* plane = logits + (size_t)blockIdx.z * T * E;
        if (e < E) plane[(size_t)t * E + e] = total[n][half * 2];
        if (e + 1 < E) plane[(size_t)t * E + e + 1] = total[n][half * 2 + 1];
      } else {
        if (e < E) atomicAdd(logits + (size_t)t * E + e, total[n][half * 2]);
        if (e + 1 < E) atomicAdd(logits + (size_t)t * E + e + 1, total[n][half * 2 + 1]);
      }
    }
  }
}

// logits[i] = planes[0][i] + planes[1][i] + ... in plane order (fixed: reproducible)
__global__ void __launch_bounds__(256)
sum_planes_kernel(const float* __restrict__ planes, int n_planes, size_t n, float* __restrict__ logits) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 acc = *reinterpret_cast<const float4*>(planes + i);
  for (int z = 1; z < n_planes; ++z) {
    const float4 v = *reinterpret_cast<const float4*>(planes + (size_t)z * n + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  *reinterpret_cast<float4*>(logits + i) = acc;
}

// Small batches: one warp per (token, expert) dot product, 128-bit loads, so a decode
// step fills the machine instead of running on a couple of CTAs.
__global__ void __launch_bounds__(256)
router_logits_warp_kernel(const uint16_t* __restrict__ x, const float* __restrict__ wr,
                          float* __restrict__ logits, int T, int H, int E) {
  const int lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (long long)T * E) return;
  const int t = (int)(pair / E), e = (int)(pair % E);
  const uint2* xr = reinterpret_cast<const uint2*>(x + (size_t)t * H);     // 4 bf16
  const float4* w = reinterpret_cast<const float4*>(wr + (size_t)e * H);   // 4 fp32
  float acc = 0.0f;
  for (int i = lane; i < H / 4; i += 32) {
    const uint2 xv = xr[i];
    const float4 wv = w[i];
    acc = fmaf(bf16_bits_to_f32(xv.x & 0xFFFFu), wv.x, acc);
    acc = fmaf(bf16_bits_to_f32(xv.x >> 16), wv.y, acc);
    acc = fmaf(bf16_bits_to_f32(xv.y & 0xFFFFu), wv.z, acc);
    acc = fmaf(bf16_bits_to_f32(xv.y >> 16), wv.w, acc);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, d);
  if (lane == 0) logits[(size_t)t * E + e] = acc;
}

// Decode batches (a few thousand dot products at most): one CTA per (expert, token) dot, every
// thread a handful of 16-byte loads in flight, so even a single token's 32 dots spread over 32
// SMs and finish in one memory round trip instead of a warp's 90 dependent ones.
__global__ void __launch_bounds__(256)
router_logits_cta_kernel(const uint16_t* __restrict__ x, const float* __restrict__ wr,
                         float* __restrict__ logits, int H, int E) {
  __shared__ float part[8];
  const int e = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
  const uint2* xr = reinterpret_cast<const uint2*>(x + (size_t)t * H);     // 4 bf16
  const float4* w = reinterpret_cast<const float4*>(wr + (size_t)e * H);   // 4 fp32
  float acc = 0.0f;
  for (int i = tid; i < H / 4; i += 256) {
    const uint2 xv = xr[i];
    const float4 wv = w[i];
    acc = fmaf(bf16_bits_to_f32(xv.x & 0xFFFFu), wv.x, acc);
    acc = fmaf(bf16_bits_to_f32(xv.x >> 16), wv.y, acc);
    acc = fmaf(bf16_bits_to_f32(xv.y & 0xFFFFu), wv.z, acc);
    acc = fmaf(bf16_bits_to_f32(xv.y >> 16), wv.w, acc);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, d);
  if ((tid & 31) == 0) part[tid >> 5] = acc;
  __syncthreads();
  if (tid == 0) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += part[i];   // fixed order: reproducible
    logits[(size_t)t * E + e] = s;
  }
}

using namespace prep;

template <int SLOTS>
__global__ void __launch_bounds__(128)
route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E,
                  int k, int sigmoid, int n_group, int topk_group, int renorm, float scaling,
                  int n_shared, int32_t* __restrict__ ids, float* __restrict__ w) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int kk = k + n_shared;
  route_token<SLOTS>(logits + (size_t)t * E, bias, E, k, sigmoid, n_group, topk_group, renorm, scaling, n_shared, lane,
                     ids + (size_t)t * kk, w + (size_t)t * kk);
}

// Small batches - at most 1024 routed slots, the decode regime: routing AND alignment in one CTA.
// The warps route the tokens in turn (the ids stay in shared memory), then the CTA runs the
// one-chunk stable counting sort of the alignment on them. A decode step is a chain of kernels of
// a few microseconds each; this removes one launch and one global round trip from it. Outputs
// are those of route_topk followed by moe_align_block_size (no expert map: the ids are the
// layer's own expert indices, shared experts included).
template <int SLOTS>
__global__ void __launch_bounds__(kChunk)
route_align_small_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k,
                         int sigmoid, int n_group, int topk_group, int renorm, float scaling, int n_shared,
                         int block_size, int max_EM, int32_t* __restrict__ ids, float* __restrict__ w,
                         int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids,
                         int32_t* __restrict__ out_em) {
  extern __shared__ int smem[];
  const int local_n = E + n_shared;
  int* warp_hist = smem;                               // [(kWarps + 1) * local_n]
  int* offset = warp_hist + (kWarps + 1) * local_n;    // [local_n]
  int* s_tmp = offset + local_n;                       // [kChunk]
  int32_t* s_ids = s_tmp + kChunk;                     // [kChunk]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kk = k + n_shared, N = T * kk;
  for (int i = tid; i < max_EM; i += kChunk) sorted_ids[i] = N;
  for (int i = tid; i < max_EM / block_size; i += kChunk) expert_ids[i] = -1;
  for (int t = warp; t < T; t += kWarps)
    route_token<SLOTS>(logits + (size_t)t * E, bias, E, k, sigmoid, n_group, topk_group, renorm, scaling, n_shared,
                       lane, s_ids + t * kk, w + (size_t)t * kk);
  __syncthreads();
  int le = -1;
  if (tid < N) {
    le = s_ids[tid];
    ids[tid] = le;
    if (le < 0 || le >= local_n) le = -1;
  }
  const int rank = chunk_rank(le, local_n, warp_hist);
  scan_experts(warp_hist + kWarps * local_n, offset, local_n, block_size, max_EM, expert_ids, out_em, s_tmp);
  if (le >= 0) {
    const int pos = offset[le] + rank;
    if (pos < max_EM) sorted_ids[pos] = tid;
  }
}

}  // namespace

void router_logits(const uint16_t* x, const float* wr, float* logits, int T, int H, int E,
                   void* stream) {
  expects(T >= 0 && H > 0 && E > 0, "router_logits: bad dimensions");
  if (T == 0) return;
  expects(x && wr && logits, "router_logits: null buffer");
  const bool aligned16 = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(wr) & 15u) == 0;
  if ((long long)T * E <= 8192 && T <= 65535 && H % 8 == 0 && aligned16) {
    router_logits_cta_kernel<<<dim3((unsigned)E, (unsigned)T), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, wr, logits, H, E);
  } else if (T <= 512 && H % 8 == 0 && aligned16) {   // 8- and 16-byte loads of whole rows
    const long long pairs = (long long)T * E;
    router_logits_warp_kernel<<<(unsigned)((pairs + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, wr, logits, T, H, E);
  } else if (H % 8 == 0 && aligned16) {
    // the attribute belongs to the device's context: once per device
    static std::atomic<bool> configured_dev[64];
    int dev = 0;
    VK_CUDA_CHECK(cudaGetDevice(&dev));
    const bool known = dev >= 0 && dev < 64;
    if (!known || !configured_dev[dev].load()) {
      VK_CUDA_CHECK(cudaFuncSetAttribute(router_logits_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(RouterSmem<128>)));
      VK_CUDA_CHECK(cudaFuncSetAttribute(router_logits_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(RouterSmem<64>)));
      if (known) configured_dev[dev].store(true);
    }
    const int t_tiles = (T + MT - 1) / MT;
    if (t_tiles * ((E + 127) / 128) >= 2 * sm_count()) {
      dim3 grid(t_tiles, (E + 127) / 128);
      router_logits_mma_kernel<128><<<grid, 256, sizeof(RouterSmem<128>), static_cast<cudaStream_t>(stream)>>>(
          x, wr, logits, T, H, E);
    } else {
      dim3 grid(t_tiles, (E + 63) / 64);
      const int ctas = (int)(grid.x * grid.y), chunks = (H + MK - 1) / MK;
      cudaStream_t st = static_cast<cudaStream_t>(stream);
      // not enough CTAs for the machine: split K - in up to eight slices of at least four chunks
      int z = 1;
      if (ctas < sm_count() && H >= 4 * MK) z = std::min(std::min(8, chunks / 4), (sm_count() + ctas - 1) / ctas);
      const size_t n = (size_t)T * E;
      if (z > 2 && n % 4 == 0) {
        // one plane per slice in the stream's scratch (behind its first 4 KB), added in order afterwards
        float* planes = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace_get(4096 + (size_t)z * n * sizeof(float), st)) + 4096);
        grid.z = (unsigned)z;
        router_logits_mma_kernel<64><<<grid, 256, sizeof(RouterSmem<64>), st>>>(x, wr, planes, T, H, E);
        sum_planes_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(planes, z, n, logits);
      } else {
        if (z >= 2) {
          grid.z = 2;
          VK_CUDA_CHECK(cudaMemsetAsync(logits, 0, n * sizeof(float), st));
        }
        router_logits_mma_kernel<64><<<grid, 256, sizeof(RouterSmem<64>), st>>>(x, wr, logits, T, H, E);
      }
    }
  } else {
    dim3 grid((T + RT - 1) / RT, (E + RE - 1) / RE);
    router_logits_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, wr, logits, T, H, E);
  }
  VK_CUDA_CHECK(cudaGetLastError());
}

void route_align_small(const float* logits, const float* bias, int T, int E, int k, int sigmoid, int n_group,
                       int topk_group, int renorm, float scaling, int n_shared, int block_size, int max_EM,
                       int32_t* ids, float* w, int32_t* sorted_ids, int32_t* expert_ids, int32_t* out_em,
                       void* stream) {
  expects(T > 0 && E > 0 && k > 0 && k <= E, "route_align_small: need T > 0 and 0 < k <= E");
  expects(E <= 32 * kMaxSlots, "route_align_small: at most 1024 experts");
  expects(n_shared >= 0 && k + n_shared <= 32, "route_align_small: k + n_shared must be at most 32");
  expects((long long)T * (k + n_shared) <= kChunk, "route_align_small: at most 1024 routed slots");
  expects(n_group >= 1 && n_group <= 32 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group,
          "route_align_small: bad group configuration");
  expects(n_group == 1 || sigmoid, "route_align_small: group limiting needs the sigmoid router");
  expects(n_group == 1 || (E / n_group) * topk_group >= k, "route_align_small: kept groups hold fewer than k experts");
  expects(block_size > 0 && max_EM > 0 && max_EM % block_size == 0,
          "route_align_small: max_EM must be a positive multiple of block_size");
  expects(logits && ids && w && sorted_ids && expert_ids && out_em, "route_align_small: null buffer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int local_n = E + n_shared;
  const size_t smem = ((size_t)(kWarps + 1) * local_n + local_n + 2 * kChunk) * sizeof(int);
  expects(smem <= 200 * 1024, "route_align_small: too many experts");
  const int slots = (E + 31) / 32;
#define VK_ROUTE_ALIGN(S)                                                                                     \
  do {                                                                                                        \
    if (smem > 48 * 1024)                                                                                     \
      VK_CUDA_CHECK(cudaFuncSetAttribute(route_align_small_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem));                                                         \
    route_align_small_kernel<S><<<1, kChunk, smem, s>>>(logits, bias, T, E, k, sigmoid, n_group, topk_group,  \
                                                        renorm, scaling, n_shared, block_size, max_EM, ids, w, \
                                                        sorted_ids, expert_ids, out_em);                      \
  } while (0)
  if (slots <= 1) VK_ROUTE_ALIGN(1);
  else if (slots <= 2) VK_ROUTE_ALIGN(2);
  else if (slots <= 4) VK_ROUTE_ALIGN(4);
  else if (slots <= 8) VK_ROUTE_ALIGN(8);
  else if (slots <= 16) VK_ROUTE_ALIGN(16);
  else VK_ROUTE_ALIGN(32);
#undef VK_ROUTE_ALIGN
  VK_CUDA_CHECK(cudaGetLastError());
}

void route_topk(const float* logits, const float* bias, int T, int E, int k, int sigmoid,
                int n_group, int topk_group, int renorm, float scaling, int n_shared,
                int32_t* ids, float* w, void* stream) {
  expects(T >= 0 && E > 0 && k > 0 && k <= E, "route_topk: need 0 < k <= E");
  expects(E <= 32 * kMaxSlots, "route_topk: at most 1024 experts");
  expects(n_shared >= 0 && k + n_shared <= 32, "route_topk: k + n_shared must be at most 32");
  expects(n_group >= 1 && n_group <= 32 && E % n_group == 0 && topk_group >= 1 &&
              topk_group <= n_group,
          "route_topk: bad group configuration");
  expects(n_group == 1 || sigmoid, "route_topk: group limiting needs the sigmoid router");
  expects(n_group == 1 || (E / n_group) * topk_group >= k,
          "route_topk: kept groups hold fewer than k experts");
  if (T == 0) return;
  expects(logits && ids && w, "route_topk: null buffer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int warps = 4;
  dim3 grid((T + warps - 1) / warps);
  const int slots = (E + 31) / 32;
#define VK_ROUTE(S)                                                                          \
  route_topk_kernel<S><<<grid, warps * 32, 0, s>>>(logits, bias, T, E, k, sigmoid, n_group,   \
                                                   topk_group, renorm, scaling, n_shared, ids, w)
  if (slots <= 1) VK_ROUTE(1);
  else if (slots <= 2) VK_ROUTE(2);
  else if (slots <= 4) VK_ROUTE(4);
  else if (slots <= 8) VK_ROUTE(8);
  else if (slots <= 16) VK_ROUTE(16);
  else VK_ROUTE(32);
#undef VK_ROUTE
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
