// ref_shim.cpp - plain-C entry points over the UNMODIFIED reference sources.
//
// TEST INFRASTRUCTURE ONLY. This file contains no algorithm: it forwards to the
// reference's own functions, which the Makefile beside it compiles from where
// they lie (src/c/vkernels/kernels/moe_fused.cpp, dist/dist_moe.cpp,
// comm/{channel,allreduce}.cpp) into _ref/libvkref.so. The tests use that
// library to pin moe_oracle.c; bench.py may time it as the CPU baseline.
//
// vkr_fused_moe_mxfp4_mt is the one function that adds behaviour: it runs the
// reference's stage functions on 16-row slices from several threads. Every
// 16-row block of the reference is independent of the others
// (moe_fused.cpp:273-364, 456-517) so the bits are those of the single call;
// the combine stage (moe_fused.cpp:523-564) stays one sequential call because
// its accumulation order is row order.
#include <cstdint>
#include <cstring>
#include <exception>
#include <thread>
#include <vector>

#include "vkernels/dist/dist_moe.hpp"
#include "vkernels/kernels/moe_fused.hpp"

namespace vk = vkernels::kernels;
namespace vd = vkernels::dist;

extern "C" {

void vkr_dequant_weight_tile(const uint8_t* packed, const uint8_t* scale, uint16_t* out, int N,
                             int K, int group_size, int stride_packed, int stride_scale_n,
                             int stride_scale_k) {
  vk::dequant_weight_tile(packed, scale, out, N, K, group_size, stride_packed, stride_scale_n,
                          stride_scale_k);
}

void vkr_dequant_weight_tile_ref(const uint8_t* packed, const uint8_t* scale, uint16_t* out,
                                 int N, int K, int group_size, int stride_packed,
                                 int stride_scale_n, int stride_scale_k) {
  vk::dequant_weight_tile_ref(packed, scale, out, N, K, group_size, stride_packed,
                              stride_scale_n, stride_scale_k);
}

int vkr_moe_align_block_size(const int32_t* topk_ids, int M, int top_k, int block_size,
                             int num_experts, int32_t* sorted_ids, int32_t* expert_ids) {
  return vk::moe_align_block_size(topk_ids, M, top_k, block_size, num_experts, sorted_ids,
                                  expert_ids);
}

void vkr_moe_gateup(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                    const int32_t* sorted_ids, const int32_t* expert_ids, float* gate_up, int M,
                    int a_stride, int k_base, int hidden_k, int ispp, int top_k, int EM,
                    int group_size) {
  vk::moe_gateup_cpu(A, w13, w13_scale, sorted_ids, expert_ids, gate_up, M, a_stride, k_base,
                     hidden_k, ispp, top_k, EM, group_size);
}

void vkr_moe_act_epilogue(const float* gate_up, const float* b13, uint16_t* act,
                          const int32_t* sorted_ids, const int32_t* expert_ids, int M, int top_k,
                          int EM, int ispp, float swiglu_limit, int activation, float beta,
                          float linear_beta) {
  vk::moe_act_epilogue_cpu(gate_up, b13, act, sorted_ids, expert_ids, M, top_k, EM, ispp,
                           swiglu_limit, activation, beta, linear_beta);
}

void vkr_moe_down(const uint16_t* act, const uint8_t* w2, const uint8_t* w2_scale,
                  const int32_t* sorted_ids, const int32_t* expert_ids, float* partial, int M,
                  int a_stride, int k_base, int ispp_k, int hidden, int top_k, int EM,
                  int group_size) {
  vk::moe_down_cpu(act, w2, w2_scale, sorted_ids, expert_ids, partial, M, a_stride, k_base,
                   ispp_k, hidden, top_k, EM, group_size);
}

void vkr_moe_combine(const float* partial, const float* b2, const float* topk_w_sorted,
                     const int32_t* sorted_ids, const int32_t* expert_ids, float* out, int M,
                     int hidden, int top_k, int EM) {
  vk::moe_combine_cpu(partial, b2, topk_w_sorted, sorted_ids, expert_ids, out, M, hidden, top_k,
                      EM);
}

int vkr_fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                        const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                        const float* topk_w_sorted, const int32_t* expert_ids,
                        uint16_t* act_scratch, float* out, int M, int hidden, int ispp, int top_k,
                        int EM, int group_size, float swiglu_limit, int activation, float beta,
                        float linear_beta, const float* b13, const float* b2) {
  try {
    vk::fused_moe_mxfp4_cpu(A, w13, w13_scale, w2, w2_scale, sorted_ids, topk_w_sorted,
                            expert_ids, act_scratch, out, M, hidden, ispp, top_k, EM, group_size,
                            swiglu_limit, activation, beta, linear_beta, b13, b2);
  } catch (const std::exception&) {
    return -1;
  }
  return 0;
}

int vkr_fused_moe_mxfp4_mt(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                           const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                           const float* topk_w_sorted, const int32_t* expert_ids,
                           uint16_t* act_scratch, float* out, int M, int hidden, int ispp,
                           int top_k, int EM, int group_size, float swiglu_limit, int activation,
                           float beta, float linear_beta, const float* b13, const float* b2,
                           int n_threads) {
  try {
    constexpr int kRows = 16;
    const int n_blocks = EM / kRows;
    if (n_threads < 1) n_threads = 1;
    std::vector<float> partial(static_cast<std::size_t>(EM) * hidden);
    auto worker = [&](int tid) {
      std::vector<float> gate_up(static_cast<std::size_t>(kRows) * 2 * ispp);
      for (int mb = tid; mb < n_blocks; mb += n_threads) {
        const int32_t* sid = sorted_ids + static_cast<std::size_t>(mb) * kRows;
        const int32_t* eid = expert_ids + mb;
        uint16_t* act = act_scratch + static_cast<std::size_t>(mb) * kRows * ispp;
        float* part = partial.data() + static_cast<std::size_t>(mb) * kRows * hidden;
        vk::moe_gateup_cpu(A, w13, w13_scale, sid, eid, gate_up.data(), M, hidden, 0, hidden,
                           ispp, top_k, kRows, group_size);
        vk::moe_act_epilogue_cpu(gate_up.data(), b13, act, sid, eid, M, top_k, kRows, ispp,
                                 swiglu_limit, activation, beta, linear_beta);
        vk::moe_down_cpu(act, w2, w2_scale, sid, eid, part, M, ispp, 0, ispp, hidden, top_k,
                         kRows, group_size);
      }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < n_threads; ++t) pool.emplace_back(worker, t);
    worker(0);
    for (auto& th : pool) th.join();
    vk::moe_combine_cpu(partial.data(), b2, topk_w_sorted, sorted_ids, expert_ids, out, M,
                        hidden, top_k, EM);
  } catch (const std::exception&) {
    return -1;
  }
  return 0;
}

int vkr_moe_ep_plan(int num_experts, int ep, int rank, int* expert_begin, int* expert_end) {
  try {
    const vd::MoeEPPlan p = vd::moe_ep_plan(num_experts, ep, rank);
    *expert_begin = p.expert_begin;
    *expert_end = p.expert_end;
  } catch (const std::exception&) {
    return -1;
  }
  return 0;
}

int vkr_moe_ep_dispatch(const int32_t* topk_ids, int M, int top_k, int num_experts,
                        int block_size, int ep, int rank, int32_t* sorted_ids,
                        int32_t* expert_ids) {
  try {
    const vd::MoeEPPlan p = vd::moe_ep_plan(num_experts, ep, rank);
    std::vector<int32_t> s, e;
    const int EM = vd::moe_ep_dispatch(topk_ids, M, top_k, num_experts, block_size, p, s, e);
    std::memcpy(sorted_ids, s.data(), s.size() * sizeof(int32_t));
    std::memcpy(expert_ids, e.data(), e.size() * sizeof(int32_t));
    return EM;
  } catch (const std::exception&) {
    return -1;
  }
}

// outs: [ep, M, hidden] fp32, one partial output per rank; the layer output is
// their element-wise sum (dist_moe.hpp:177-191).
int vkr_fused_moe_mxfp4_ep(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                           const uint8_t* w2, const uint8_t* w2_scale, const int32_t* topk_ids,
                           const float* topk_w, const float* b13, const float* b2, int M,
                           int hidden, int ispp, int top_k, int num_experts, int group_size,
                           float swiglu_limit, int activation, float beta, float linear_beta,
                           int block_size, int ep, float* outs) {
  try {
    auto r = vd::fused_moe_mxfp4_ep(A, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, b13, b2,
                                    M, hidden, ispp, top_k, num_experts, group_size,
                                    swiglu_limit, activation, beta, linear_beta, block_size, ep);
    for (int i = 0; i < ep; ++i)
      std::memcpy(outs + static_cast<std::size_t>(i) * M * hidden, r[i].data(),
                  static_cast<std::size_t>(M) * hidden * sizeof(float));
  } catch (const std::exception&) {
    return -1;
  }
  return 0;
}

void vkr_round_bf16(const float* src, uint16_t* dst, int n) { vd::round_bf16(src, dst, n); }

}  // extern "C"
