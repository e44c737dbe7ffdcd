// moe_simt.cu - CUDA-core cross-check implementation of the two grouped GEMMs.
//
// One CTA computes a 16-row block of the sorted layout against 64 output
// features, dequantising the weights into shared memory 64 K-elements at a
// time. Each output adds in the CPU definition's order (a sequential 64-long
// fp32 dot per K block, then one add into the running sum; reference
// moe_fused.cpp:315-325): the products of two bf16 values are exact in fp32,
// so the fused multiply-adds used here give the same bits as separate multiply
// and add. The accumulators therefore match the CPU oracle bit for bit; only
// the activation (device expf) and the atomic combine order differ.
//
// This path is selected explicitly (MoeImpl::kSimt); it is far from the
// roofline and exists to check the tensor-core kernels at sizes the CPU cannot
// reach.
#include "common.cuh"
#include "moe_fused.hpp"

namespace vkernels::kernels::cuda {

namespace {

constexpr int BM = 16, BN = 64, BK = 64;

struct SimtArgs {
  const uint16_t* src;      // A [M, K] (gate/up) or act [EM, K] (down)
  const uint8_t* w;         // [E, n_rows, K/2]
  const uint8_t* w_scale;   // [E, n_rows, K/32]
  const float* bias;        // [E, n_rows] or null
  const float* topk_w;      // down: routing weights
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  uint16_t* act;            // gate/up output [EM, ispp]
  float* out;               // down output [M, hidden]
  int K, n_feat, N, top_k, block_size, w_sorted;
  float limit, beta, linear_beta;
  int activation;
};

// Dequantise rows [n0, n0+64) x K-range [k0, k0+64) of one expert's matrix into
// ws[n][k] (fp32 values of the bf16 weights).
__device__ __forceinline__ void load_w_tile(const uint8_t* w, const uint8_t* sc, int K, int n0,
                                            int k0, float (*ws)[BK + 1]) {
  // 64 rows x 32 packed bytes = 512 words; 256 threads x 2
  for (int i = threadIdx.x; i < BN * (BK / 8); i += 256) {
    const int n = i >> 3, wq = i & 7;  // word wq covers k = 8*wq .. 8*wq+7
    const uint8_t* row = w + (size_t)(n0 + n) * (K / 2) + (k0 >> 1);
    const uint32_t word = reinterpret_cast<const uint32_t*>(row)[wq];
    const uint32_t s = sc[(size_t)(n0 + n) * (K / 32) + ((k0 + 8 * wq) >> 5)];
    uint32_t o[4];
    dequant8(word, ue8m0_to_bf16x2(s), o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ws[n][8 * wq + 2 * j] = bf16_bits_to_f32(o[j] & 0xFFFFu);
      ws[n][8 * wq + 2 * j + 1] = bf16_bits_to_f32(o[j] >> 16);
    }
  }
}

template <bool GATEUP>
__global__ void __launch_bounds__(256) moe_simt_kernel(SimtArgs p) {
  __shared__ float as[BM][BK + 1];
  __shared__ float wg[BN][BK + 1];
  __shared__ float wu[GATEUP ? BN : 1][BK + 1];
  const int rb = blockIdx.x, nb = blockIdx.y;
  const int e = p.expert_ids[(rb * BM) / p.block_size];
  if (e < 0) return;
  const int tid = threadIdx.x, m = tid >> 4, c = (tid & 15) * 4;
  const int row = rb * BM + m;
  const int flat = p.sorted_ids[row];
  const bool real = flat >= 0 && flat < p.N;
  const int n_rows = GATEUP ? 2 * p.n_feat : p.n_feat;
  const uint8_t* w = p.w + (size_t)e * n_rows * (p.K / 2);
  const uint8_t* sc = p.w_scale + (size_t)e * n_rows * (p.K / 32);
  float acc_g[4] = {}, acc_u[4] = {};
  for (int k0 = 0; k0 < p.K; k0 += BK) {
    {  // 16 rows x 64 k, 4 k per thread
      const int r = tid >> 4, kk = (tid & 15) * 4;
      const int f = p.sorted_ids[rb * BM + r];
      const bool ok = f >= 0 && f < p.N;
      const size_t srow = GATEUP ? (size_t)(f / p.top_k) : (size_t)(rb * BM + r);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        as[r][kk + j] = ok ? bf16_bits_to_f32(p.src[srow * p.K + k0 + kk + j]) : 0.0f;
    }
    load_w_tile(w, sc, p.K, nb * BN, k0, wg);
    if (GATEUP) load_w_tile(w, sc, p.K, p.n_feat + nb * BN, k0, wu);
    __syncthreads();
    float dg[4] = {}, du[4] = {};
    for (int k = 0; k < BK; ++k) {
      const float a = as[m][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        dg[j] = fmaf(a, wg[c + j][k], dg[j]);
        if (GATEUP) du[j] = fmaf(a, wu[c + j][k], du[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc_g[j] += dg[j];
      if (GATEUP) acc_u[j] += du[j];
    }
    __syncthreads();
  }
  if (!real) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = nb * BN + c + j;
    if (GATEUP) {
      float g = acc_g[j], u = acc_u[j];
      if (p.bias) {
        g += p.bias[(size_t)e * 2 * p.n_feat + n];
        u += p.bias[(size_t)e * 2 * p.n_feat + p.n_feat + n];
      }
      p.act[(size_t)row * p.n_feat + n] =
          f32_to_bf16_bits(moe_act_value(p.activation, g, u, p.limit, p.beta, p.linear_beta));
    } else {
      float v = acc_g[j];
      if (p.bias) v += p.bias[(size_t)e * p.n_feat + n];
      v *= p.topk_w[p.w_sorted ? row : flat];
      atomicAdd(p.out + (size_t)(flat / p.top_k) * p.n_feat + n, v);
    }
  }
}

}  // namespace

void launch_moe_simt(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                     const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w, int w_sorted,
                     uint16_t* act_scratch, float* out, int M, int hidden, int ispp, int top_k,
                     const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                     float swiglu_limit, int activation, float beta, float linear_beta,
                     const float* b13, const float* b2, int block_size, cudaStream_t stream) {
  SimtArgs g{};
  g.src = A; g.w = w13; g.w_scale = w13_scale; g.bias = b13; g.topk_w = topk_w;
  g.sorted_ids = sorted_ids; g.expert_ids = expert_ids; g.act = act_scratch; g.out = out;
  g.K = hidden; g.n_feat = ispp; g.N = M * top_k; g.top_k = top_k; g.block_size = block_size;
  g.w_sorted = w_sorted; g.limit = swiglu_limit; g.beta = beta; g.linear_beta = linear_beta;
  g.activation = activation;
  moe_simt_kernel<true><<<dim3(EM / BM, ispp / BN), 256, 0, stream>>>(g);
  SimtArgs d = g;
  d.src = act_scratch; d.w = w2; d.w_scale = w2_scale; d.bias = b2; d.K = ispp; d.n_feat = hidden;
  moe_simt_kernel<false><<<dim3(EM / BM, hidden / BN), 256, 0, stream>>>(d);
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
