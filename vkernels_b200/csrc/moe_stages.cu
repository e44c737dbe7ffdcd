// moe_stages.cu - the fused MXFP4 MoE layer split into its four stages, for tensor parallelism.
//
// With the weights sharded along the reduction dimension (w13 along hidden, w2 along ispp) every
// rank computes partial sums that must be added over the ranks BEFORE the non-linear epilogue
// and BEFORE the routing-weighted combine. The reference exposes the layer in four pieces for
// that purpose (src/c/vkernels/kernels/moe_fused.hpp:265-286); these are their counterparts:
//
//   moe_gateup_preact -> [all-reduce gate_up] -> moe_act_epilogue
//     -> moe_down_preact -> [all-reduce partial] -> moe_combine
//
// The two GEMM stages run on the tcgen05 kernel with its plain-result epilogue
// (launch_moe_stage_gemm); the two element-wise stages are the small kernels below. Token blocks
// are 16 rows, as in the reference's stage functions.
#include "common.cuh"
#include "moe_fused.hpp"

namespace vkernels::kernels::cuda {

void launch_moe_stage_gemm(int which, const uint16_t* rows_in, const uint8_t* w, const uint8_t* w_scale,
                           const int32_t* sorted_ids, const int32_t* expert_ids, float* raw, int M,
                           int k_full, int n_out, int top_k, int EM, int k_base, int k_shard,
                           cudaStream_t stream);

namespace {

constexpr int kBlock = 16;   // token rows per expert block

// act[r, i] = bf16(f(gate_up[r, i] + b13[e, i], gate_up[r, ispp + i] + b13[e, ispp + i])) for real rows
// (reference moe_fused.cpp:370-422): one rounding, padding rows and rows of unused blocks untouched.
__global__ void __launch_bounds__(256)
act_epilogue_kernel(const float* __restrict__ gate_up, const float* __restrict__ b13, uint16_t* __restrict__ act,
                    const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids, int N, int ispp,
                    float limit, int activation, float beta, float linear_beta) {
  const int r = blockIdx.x;
  const int e = expert_ids[r / kBlock];
  if (e < 0) return;
  const int flat = sorted_ids[r];
  if (flat < 0 || flat >= N) return;
  const float* g = gate_up + (size_t)r * 2 * ispp;
  const float* bg = b13 ? b13 + (size_t)e * 2 * ispp : nullptr;
  for (int i = threadIdx.x; i < ispp; i += blockDim.x) {
    const float gv = g[i] + (bg ? bg[i] : 0.0f);
    const float uv = g[ispp + i] + (bg ? bg[ispp + i] : 0.0f);
    act[(size_t)r * ispp + i] = f32_to_bf16_bits(moe_act_value(activation, gv, uv, limit, beta, linear_beta));
  }
}

// out[token, h] += (partial[r, h] + b2[e, h]) * topk_w_sorted[r] for real rows (reference
// moe_fused.cpp:523-564). A token's rows are added with atomics, so their order is not the
// reference's sorted order: fp32 reassociation only.
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ partial, const float* __restrict__ b2, const float* __restrict__ w_sorted,
               const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids, float* __restrict__ out,
               int N, int top_k, int hidden) {
  const int r = blockIdx.x;
  const int e = expert_ids[r / kBlock];
  if (e < 0) return;
  const int flat = sorted_ids[r];
  if (flat < 0 || flat >= N) return;
  const float wgt = w_sorted[r];
  const float* src = partial + (size_t)r * hidden;
  const float* bias = b2 ? b2 + (size_t)e * hidden : nullptr;
  float* dst = out + (size_t)(flat / top_k) * hidden;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x)
    atomicAdd(dst + h, (src[h] + (bias ? bias[h] : 0.0f)) * wgt);
}

}  // namespace

void moe_gateup_preact(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const int32_t* sorted_ids,
                       const int32_t* expert_ids, float* gate_up, int M, int hidden, int ispp, int top_k, int EM,
                       int k_base, int hidden_k, void* stream) {
  launch_moe_stage_gemm(0, A, w13, w13_scale, sorted_ids, expert_ids, gate_up, M, hidden, ispp, top_k, EM, k_base,
                        hidden_k, static_cast<cudaStream_t>(stream));
}

void moe_act_epilogue(const float* gate_up, const float* b13, uint16_t* act, const int32_t* sorted_ids,
                      const int32_t* expert_ids, int M, int top_k, int EM, int ispp, float swiglu_limit,
                      int activation, float beta, float linear_beta, void* stream) {
  expects(M >= 0 && EM >= 0 && top_k > 0 && EM % kBlock == 0 && ispp > 0, "moe_act_epilogue: bad dimensions");
  expects(activation == kSwiGLU || activation == kSiTU, "moe_act_epilogue: unknown activation");
  if (M == 0 || EM == 0) return;
  expects(gate_up && act && sorted_ids && expert_ids, "moe_act_epilogue: buffers must not be null");
  act_epilogue_kernel<<<EM, 256, 0, static_cast<cudaStream_t>(stream)>>>(gate_up, b13, act, sorted_ids, expert_ids,
                                                                         M * top_k, ispp, swiglu_limit, activation,
                                                                         beta, linear_beta);
  VK_CUDA_CHECK(cudaGetLastError());
}

void moe_down_preact(const uint16_t* act, const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                     const int32_t* expert_ids, float* partial, int M, int ispp, int hidden, int top_k, int EM,
                     int k_base, int ispp_k, void* stream) {
  launch_moe_stage_gemm(1, act, w2, w2_scale, sorted_ids, expert_ids, partial, M, ispp, hidden, top_k, EM, k_base,
                        ispp_k, static_cast<cudaStream_t>(stream));
}

void moe_combine(const float* partial, const float* b2, const float* topk_w_sorted, const int32_t* sorted_ids,
                 const int32_t* expert_ids, float* out, int M, int hidden, int top_k, int EM, void* stream) {
  expects(M >= 0 && EM >= 0 && top_k > 0 && EM % kBlock == 0 && hidden > 0, "moe_combine: bad dimensions");
  if (M == 0 || EM == 0) return;
  expects(partial && topk_w_sorted && sorted_ids && expert_ids && out, "moe_combine: buffers must not be null");
  combine_kernel<<<EM, 256, 0, static_cast<cudaStream_t>(stream)>>>(partial, b2, topk_w_sorted, sorted_ids,
                                                                    expert_ids, out, M * top_k, top_k, hidden);
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
