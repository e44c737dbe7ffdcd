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
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <string>
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

// ---------------------------------------------------------------------------
// Router logits on tcgen05 (prefill-size batches).
//
// D[128 tokens, E experts] = x[128, K] . (hi + mid + lo)[E, K]^T with the fp32 router weight
// split once per call into three bf16 terms (exact: hi + mid + lo == w). One CTA per 128-token
// tile and K slice: a TMA producer warp streams the token tile and the three weight-term tiles
// of each 64-K chunk through a shared-memory ring (128-byte swizzle), one thread issues twelve
// kind::f16 MMAs per chunk (A and B both from shared memory), four warps read the accumulators
// back and store the rows.
//
// The tensor core adds a product to its fp32 accumulator by truncating the addend to the
// accumulator's last bit (measured: adding 0.75 ulp sixty-four times changes nothing), so every
// MMA into a large accumulator costs up to one ulp of it. Hence TWO accumulators: the hi term
// into one (one truncation per 16 K), the mid and lo terms - 2^-8 and 2^-16 of the size, so
// their truncations are that much smaller in absolute terms - into the other; the epilogue
// adds the two in fp32. That leaves K / 16 truncations of at most one ulp with the sign of
// the addend, a random walk about as long as the rounding noise of a sequential fp32 sum over
// K terms - the yardstick the routing parity tests hold the logits to.
// ---------------------------------------------------------------------------
namespace tc {
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait (about two seconds of SM clock); false when it ran out or another role gave up.
__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > 4000000000ll) {
        *abort_flag = code;
        return false;
      }
    }
  }
}
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {   // K-major tile of 128-byte rows, 8-row groups 1024 B apart
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
constexpr int kMaxStages = 3;
struct Bars {
  uint64_t full[kMaxStages], empty[kMaxStages], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};
}  // namespace tc

// fp32 router weight [E, H] -> three bf16 planes [3][E][H] with hi + mid + lo == w
__global__ void __launch_bounds__(256)
split_router_weight_kernel(const float* __restrict__ wr, size_t n, uint16_t* __restrict__ planes) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint16_t h, m, l;
  split3(wr[i], h, m, l);
  planes[i] = h;
  planes[n + i] = m;
  planes[2 * n + i] = l;
}

// grid (ceil(T / 128), n_slices); 192 threads: warp 0 TMA producer, warp 1 MMA issuer (and tensor-
// memory owner), warps 2-5 epilogue. E a multiple of 16, at most 256; H a multiple of 64.
// out: [n_slices][T][E] planes (one slice: the logits themselves).
__global__ void __launch_bounds__(192, 1)
router_logits_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                        float* __restrict__ out, int T, int H, int E, int stages, int* status) {
  extern __shared__ uint8_t tc_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = 128 * 128, b_bytes = E * 128;          // one 64-K chunk: token tile, one weight-term tile
  const int stage_bytes = a_bytes + 3 * b_bytes;
  tc::Bars* bars = reinterpret_cast<tc::Bars*>(smem + stages * stage_bytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &bars->abort_flag;
  const int tmem_cols = 2 * E <= 256 ? 256 : 512;            // two accumulators of E columns
  if (tid == 0) {
    for (int i = 0; i < tc::kMaxStages; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc::smem_u32(&bars->full[i])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc::smem_u32(&bars->empty[i])));
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc::smem_u32(&bars->acc_full)));
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(&bars->tmem_base)),
                 "r"((uint32_t)tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = bars->tmem_base;

  const int t0 = blockIdx.x * 128;
  const int all_chunks = H / 64;
  const int ch_begin = (int)blockIdx.y * all_chunks / (int)gridDim.y;
  const int ch_end = ((int)blockIdx.y + 1) * all_chunks / (int)gridDim.y;

  if (warp == 0) {
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 0;
      for (int ch = ch_begin; ch < ch_end; ++ch) {
        if (!tc::wait(tc::smem_u32(&bars->empty[slot]), phase ^ 1u, abort_flag, 31)) break;
        const uint32_t bar = tc::smem_u32(&bars->full[slot]);
        const uint32_t dst = tc::smem_u32(smem + slot * stage_bytes);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)stage_bytes) : "memory");
        tc::tma_2d(dst, &map_x, ch * 64, t0, bar);                       // rows past T read as zeros (and still count)
        for (int term = 0; term < 3; ++term) tc::tma_2d(dst + a_bytes + term * b_bytes, &map_w, ch * 64, term * E, bar);
        if (++slot == stages) {
          slot = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // bf16 x bf16 -> fp32, both K-major, M = 128, N = E
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(E >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t d_hi = tmem, d_lo = tmem + (uint32_t)E;
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ch = ch_begin; ch < ch_end; ++ch) {
        if (!tc::wait(tc::smem_u32(&bars->full[slot]), phase, abort_flag, 32)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t base = tc::smem_u32(smem + slot * stage_bytes);
        const uint64_t a = tc::desc_sw128(base);
        const uint64_t b_hi = tc::desc_sw128(base + a_bytes), b_mid = tc::desc_sw128(base + a_bytes + b_bytes),
                       b_lo = tc::desc_sw128(base + a_bytes + 2 * b_bytes);
        const uint32_t first = ch != ch_begin ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          tc::mma_ss(d_hi, a + kk * 2, b_hi + kk * 2, idesc, first | (uint32_t)(kk != 0));
          tc::mma_ss(d_lo, a + kk * 2, b_mid + kk * 2, idesc, first | (uint32_t)(kk != 0));
          tc::mma_ss(d_lo, a + kk * 2, b_lo + kk * 2, idesc, 1u);
        }
        tc::commit(tc::smem_u32(&bars->empty[slot]));
        if (++slot == stages) {
          slot = 0;
          phase ^= 1u;
        }
      }
      if (ok) tc::commit(tc::smem_u32(&bars->acc_full));
    }
  } else {
    // epilogue: warp w reads the lane quarter w % 4; thread = token row
    const int q = warp & 3;
    const bool ok = tc::wait(tc::smem_u32(&bars->acc_full), 0, abort_flag, 33);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int t = t0 + q * 32 + lane;
    float* row = out + ((size_t)blockIdx.y * T + (size_t)(t < T ? t : 0)) * E;
    if (ok && ch_end > ch_begin) {
      const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
      for (int c = 0; c < E; c += 32) {
        uint32_t hi[32], lo[32];
        tc::ld32(t_lane + c, hi);
        tc::ld32(t_lane + E + c, lo);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (t < T) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 v;
            v.x = __uint_as_float(hi[j]) + __uint_as_float(lo[j]);
            v.y = __uint_as_float(hi[j + 1]) + __uint_as_float(lo[j + 1]);
            v.z = __uint_as_float(hi[j + 2]) + __uint_as_float(lo[j + 2]);
            v.w = __uint_as_float(hi[j + 3]) + __uint_as_float(lo[j + 3]);
            if (c + j < E) *reinterpret_cast<float4*>(row + c + j) = v;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)tmem_cols) : "memory");
  }
  if (tid == 0 && bars->abort_flag != 0 && status != nullptr) atomicExch(status, 100 + bars->abort_flag);
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

// moe_gemm_sm100.cu
CUtensorMap sm100_make_map_bf16(const void* ptr, uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_outer);
int* sm100_status_address();

namespace {
// VK_MOE_ROUTER=mma keeps prefill-size batches on the mma.sync kernel.
bool router_tc_mode() {
  static const bool on = [] {
    const char* e = std::getenv("VK_MOE_ROUTER");
    return e == nullptr || std::string(e) != "mma";
  }();
  return on;
}

void launch_router_tc(const uint16_t* x, const float* wr, float* logits, int T, int H, int E, cudaStream_t st) {
  const int tiles = (T + 127) / 128, chunks = H / 64;
  int z = std::max(1, std::min(std::min(8, chunks / 4), sm_count() / tiles));
  const size_t n = (size_t)T * E, n_w = (size_t)E * H;
  const size_t w_bytes = (3 * n_w * sizeof(uint16_t) + 1023) & ~size_t(1023);
  uint8_t* ws = static_cast<uint8_t*>(workspace_get(4096 + w_bytes + (z > 1 ? (size_t)z * n * sizeof(float) : 0), st)) + 4096;
  uint16_t* w_planes = reinterpret_cast<uint16_t*>(ws);
  float* planes = z > 1 ? reinterpret_cast<float*>(ws + w_bytes) : logits;
  split_router_weight_kernel<<<(unsigned)((n_w + 255) / 256), 256, 0, st>>>(wr, n_w, w_planes);
  const int stage_bytes = 128 * 128 + 3 * E * 128;
  const int stages = std::min(tc::kMaxStages, (227 * 1024 - 2048) / stage_bytes);
  expects(stages >= 2, "router_logits: expert count too large for the tensor-core kernel");
  const int smem = stages * stage_bytes + (int)sizeof(tc::Bars) + 1024;
  static std::atomic<int> configured[64];
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || configured[dev].load() < smem) {
    VK_CUDA_CHECK(cudaFuncSetAttribute(router_logits_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64) configured[dev].store(smem);
  }
  const CUtensorMap map_x = sm100_make_map_bf16(x, (uint64_t)H, (uint64_t)T, (uint64_t)H * 2, 128);
  const CUtensorMap map_w = sm100_make_map_bf16(w_planes, (uint64_t)H, (uint64_t)3 * E, (uint64_t)H * 2, (uint32_t)E);
  router_logits_tc_kernel<<<dim3((unsigned)tiles, (unsigned)z), 192, smem, st>>>(map_x, map_w, planes, T, H, E, stages,
                                                                              sm100_status_address());
  if (z > 1) sum_planes_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(planes, z, n, logits);
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
  } else if (router_tc_mode() && H % 64 == 0 && E % 16 == 0 && E <= 256 && aligned16) {
    launch_router_tc(x, wr, logits, T, H, E, static_cast<cudaStream_t>(stream));
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
