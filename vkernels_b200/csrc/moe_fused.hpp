// moe_fused.hpp - C++ launcher interface of the B200 fused MXFP4 MoE layer.
//
// The two launchers keep the argument lists of the reference's device entry
// points (src/c/vkernels/kernels/moe_fused.hpp:322-344 `fused_moe_mxfp4`,
// :382-390 `moe_align_block_size_hip`) so a caller of those compiles against
// this header by switching the namespace. Everything else here is additive.
//
// All pointers are device pointers unless a name ends in `_host`. Launchers
// enqueue on `stream` and return; they never synchronise.
#pragma once

#include <cstddef>
#include <cstdint>

namespace vkernels::kernels {

// Epilogue tag (reference moe_fused.hpp:47-50).
enum MoEActivation : int { kSwiGLU = 0, kSiTU = 1 };

namespace cuda {

// Which device implementation runs the two grouped GEMMs.
//   kTcgen05 : persistent tcgen05/TMEM kernels (default)
//   kSimt    : one-thread-per-output CUDA-core kernels that add in the CPU
//              oracle's order; a slow cross-check, selected only explicitly
//              (env VK_MOE_IMPL=simt or set_moe_impl), never as a fallback.
enum class MoeImpl : int { kTcgen05 = 0, kSimt = 1 };
void set_moe_impl(MoeImpl impl);
MoeImpl get_moe_impl();

// Fused layer: act = epilogue(gather(A) @ w13^T + b13); out += w * (act @ w2^T + b2).
//   A [M, hidden] bf16; w13 [E, 2*ispp, hidden/2] packed E2M1 (gate rows then up
//   rows); w13_scale [E, 2*ispp, hidden/32] ue8m0; w2 [E, hidden, ispp/2];
//   w2_scale [E, hidden, ispp/32]; topk_w [M*top_k] raw routing weights read at
//   the flat index; act_scratch [EM, ispp] bf16 (padding rows never written);
//   out [M, hidden] fp32, accumulated into (the caller zeroes it);
//   sorted_ids [EM] / expert_ids [EM/block_size] from the alignment below.
// block_size is the alignment granularity of expert_ids (16, 64 or 128).
// kmajor is accepted for signature compatibility and must be false.
// Throws std::invalid_argument on a contract violation, std::runtime_error on
// a CUDA failure.
void fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                     const uint8_t* w2, const uint8_t* w2_scale, const int32_t* topk_ids,
                     const float* topk_w, uint16_t* act_scratch, float* out, int M, int hidden,
                     int ispp, int top_k, const int32_t* sorted_ids, const int32_t* expert_ids,
                     int EM, float swiglu_limit, int activation = kSwiGLU, float beta = 4.0f,
                     float linear_beta = 25.0f, const float* b13 = nullptr,
                     const float* b2 = nullptr, int block_size = 16, bool kmajor = false,
                     void* stream = nullptr);

// Same layer, routing weights already gathered into sorted-row order
// (`topk_w_sorted [EM]`, the CPU entry point's convention, reference
// moe_fused.hpp:83-101).
void fused_moe_mxfp4_sorted_w(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                              const uint8_t* w2, const uint8_t* w2_scale,
                              const float* topk_w_sorted, uint16_t* act_scratch, float* out,
                              int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                              const int32_t* expert_ids, int EM, float swiglu_limit,
                              int activation, float beta, float linear_beta, const float* b13,
                              const float* b2, int block_size, void* stream);

// The layer with a bf16 result and an ORDERED combine: the down GEMM leaves plain fp32 partial
// rows in the library scratch and a second kernel adds each token's rows in ascending expert
// order - the order of the CPU definition (reference moe_fused.cpp:539-562; the atomic-free
// inverse-permutation gather the reference describes for its W4A4 path, moe_aux.hpp:150-155) -
// and writes y [M, hidden] bf16, overwriting it. Deterministic from run to run; no fp32 output to
// zero beforehand or convert afterwards, which is what a decode step saves. The scratch grows by
// EM * hidden fp32 (workspace_bytes_required_bf16).
void fused_moe_mxfp4_bf16(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                          const uint8_t* w2_scale, const float* topk_w, uint16_t* act_scratch, uint16_t* y_bf16,
                          int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                          const int32_t* expert_ids, int EM, float swiglu_limit, int activation, float beta,
                          float linear_beta, const float* b13, const float* b2, int block_size, void* stream);
size_t workspace_bytes_required_bf16(int max_EM, int hidden, int ispp, int n_local_experts, int N);

// Prepacked weights for decode-size batches. The checkpoint layout costs a decode step integer
// work per weight (nibble -> operand byte) that bounds it below the memory rate; a one-time
// rewrite at model load removes it: every magnitude code c >= 2 becomes c + 2, which makes the
// tensor core's own e2m1 reading of the nibble exactly twice this layer's table value
// ({0, .25, 1, 1.5, 2, 3} -> {0, .5, 2, 3, 4, 6}; the epilogue halves the sums), groups with
// scale byte 0xFF (zero in this layer) become zero codes with scale 1, and the scales are
// regrouped per (expert, 128-row work item, 256-K stage). Same size as the checkpoint form
// (+ 128 rows of padding). The layer's codes 6 and 7 (inf / NaN) cannot be expressed: `nonfinite`
// (device int) receives the number of 32-element groups holding one, and a caller that reads a
// non-zero count must keep that weight set on the checkpoint-layout entry points.
//   which = 0: w13 [E, 2*ispp, hidden/2] + scales [E, 2*ispp, hidden/32]
//   which = 1: w2  [E, hidden, ispp/2]   + scales [E, hidden, ispp/32]
// w_out must be 32-byte aligned; sizes from prepack_sizes.
void prepack_sizes(int which, int E, int hidden, int ispp, size_t* w_bytes, size_t* sf_bytes);
void prepack_weights(int which, const uint8_t* w, const uint8_t* scale, int E, int hidden, int ispp, uint8_t* w_out,
                     uint8_t* sf_out, int* nonfinite, void* stream);
// fused_moe_mxfp4_bf16 on prepacked weights. Serves batches whose token tiles stay within 64 rows
// (M <= 256 always does); larger batches are refused - they belong to the checkpoint-layout
// entry points, whose prefill forms amortise the expansion over hundreds of tokens.
void fused_moe_mxfp4_bf16_prepacked(const uint16_t* A, const uint8_t* w13_codes, const uint8_t* w13_sf,
                                    const uint8_t* w2_codes, const uint8_t* w2_sf, const float* topk_w,
                                    uint16_t* act_scratch, uint16_t* y_bf16, int M, int hidden, int ispp, int top_k,
                                    const int32_t* sorted_ids, const int32_t* expert_ids, int EM, float swiglu_limit,
                                    int activation, float beta, float linear_beta, const float* b13, const float* b2,
                                    int block_size, void* stream);

// Row addresses instead of base pointers: token m's activation row is read at a_rows[m] and
// its result is added at out_rows[m] (hidden bf16 / fp32 values each, 16-byte aligned). The rows
// may live in another GPU's memory mapped into this process (peer loads and reductions over
// NVLink): under expert parallelism this is the dispatch and the combine. tcgen05 path only.
struct RowPtrs {
  const uint16_t* const* a_rows;
  float* const* out_rows;
  // false: every result row is added, times its routing weight, into out_rows[m] (system-scope
  // reductions). true: out_rows[m] is the address of a [top_k, hidden] fp32 block and slot j's
  // row (act @ w2^T + b2, unweighted) is STORED at its row j - plain 16-byte stores, no atomics;
  // the owner of the block adds the slots in a fixed order afterwards (ep_combine_slots).
  bool store_slots = false;
};
void fused_moe_mxfp4_rows(const uint16_t* const* a_rows, const uint8_t* w13, const uint8_t* w13_scale,
                          const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                          uint16_t* act_scratch, float* const* out_rows, int M, int hidden, int ispp,
                          int top_k, const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                          float swiglu_limit, int activation, float beta, float linear_beta,
                          const float* b13, const float* b2, int block_size, void* stream, bool store_slots = false);

// The layer in four stages for tensor parallelism (reference moe_fused.hpp:265-286, same
// argument lists plus the stream): w13 / w2 are this rank's K-shards ([E, 2*ispp, hidden_k/2] and
// [E, hidden, ispp_k/2], scales accordingly), k_base is the first column of A / act the shard
// covers, biases are applied after the caller's all-reduce. Token blocks are 16 rows.
//   gate_up [EM, 2*ispp] fp32 <- moe_gateup_preact   (caller all-reduces)
//   act     [EM, ispp]   bf16 <- moe_act_epilogue    (padding rows not written)
//   partial [EM, hidden] fp32 <- moe_down_preact     (caller all-reduces)
//   out     [M, hidden]  fp32 <- moe_combine         (accumulates; zero it first)
void moe_gateup_preact(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const int32_t* sorted_ids,
                       const int32_t* expert_ids, float* gate_up, int M, int hidden, int ispp, int top_k, int EM,
                       int k_base, int hidden_k, void* stream = nullptr);
void moe_act_epilogue(const float* gate_up, const float* b13, uint16_t* act, const int32_t* sorted_ids,
                      const int32_t* expert_ids, int M, int top_k, int EM, int ispp, float swiglu_limit,
                      int activation, float beta, float linear_beta, void* stream = nullptr);
void moe_down_preact(const uint16_t* act, const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                     const int32_t* expert_ids, float* partial, int M, int ispp, int hidden, int top_k, int EM,
                     int k_base, int ispp_k, void* stream = nullptr);
void moe_combine(const float* partial, const float* b2, const float* topk_w_sorted, const int32_t* sorted_ids,
                 const int32_t* expert_ids, float* out, int M, int hidden, int top_k, int EM, void* stream = nullptr);

// Device alignment, any N = M*top_k (the reference stops at 1024). Output is
// bit-identical to the host `moe_align_block_size`: experts ascending, flat
// index ascending inside an expert, each expert padded to block_size with N,
// expert_ids -1 beyond the last real block; all max_EM entries are written;
// *out_em receives the real EM (block_size when nothing routes).
void moe_align_block_size(const int32_t* topk_ids, const int32_t* expert_map, int M, int top_k,
                          int block_size, int num_experts, int local_n, int max_EM,
                          int32_t* sorted_ids, int32_t* expert_ids, int32_t* out_em,
                          void* stream = nullptr);

// The same alignment for callers that cannot allocate device memory inside a
// call (memory pool frozen after warm-up, no tolerance for cudaMalloc's device
// synchronisation): its scratch is a fixed ~514 KB array inside the library
// image, so nothing is allocated, at the price of limits - at most 262144
// routed slots (M*top_k) and 512 local experts; larger problems are rejected.
// Calls on one device share that array: do not let two of them overlap on the
// GPU. The first call on a device resolves the array's address and should come
// before any stream capture.
void moe_align_block_size_noalloc(const int32_t* topk_ids, const int32_t* expert_map, int M,
                                  int top_k, int block_size, int num_experts, int local_n,
                                  int max_EM, int32_t* sorted_ids, int32_t* expert_ids,
                                  int32_t* out_em, void* stream = nullptr);

// logits[t, e] = sum_k fp32(x[t, k]) * wr[e, k]   (x bf16 [T, H], wr fp32 [E, H]).
void router_logits(const uint16_t* x, const float* wr, float* logits, int T, int H, int E,
                   void* stream);

// Softmax top-k (reference torch_ops/tokenspeed_amd/routing.py:58-145) or, with
// sigmoid != 0, sigmoid + bias with optional group limiting
// (torch_ops/glm_router.py:184-201 plus group selection by the sum of the two
// largest biased scores). ids/w are [T, k + n_shared]; the n_shared trailing
// slots carry expert ids E, E+1, .. with weight 1 (glm_router.py:253-262).
void route_topk(const float* logits, const float* bias, int T, int E, int k, int sigmoid,
                int n_group, int topk_group, int renorm, float scaling, int n_shared,
                int32_t* ids, float* w, void* stream);

// route_topk followed by moe_align_block_size (no expert map; num_experts = local_n = E +
// n_shared) as ONE single-CTA kernel, for batches of at most 1024 routed slots (T * (k +
// n_shared)): the decode regime, where every launch removed from the step counts.
void route_align_small(const float* logits, const float* bias, int T, int E, int k, int sigmoid, int n_group,
                       int topk_group, int renorm, float scaling, int n_shared, int block_size, int max_EM,
                       int32_t* ids, float* w, int32_t* sorted_ids, int32_t* expert_ids, int32_t* out_em,
                       void* stream);

// Library-owned device scratch (tile lists, the gathered activation rows of the gate/up GEMM,
// alignment histograms): one block per (device, stream), so layer calls on different streams do
// not share scratch; calls on ONE stream are ordered by the stream and reuse its block. A block
// is allocated by the first call on its stream or by reserve_workspace; a call that needs more
// allocates a larger block and keeps the old one until release_workspaces (enqueued work or a
// captured graph may still use it). No launcher synchronises or frees. During stream capture an
// allocation is impossible and the call fails with std::invalid_argument: reserve first.
size_t workspace_bytes_required(int max_EM, int hidden, int ispp, int n_local_experts,
                                int N);
void reserve_workspace(size_t bytes, void* stream = nullptr);
void release_workspaces();
size_t workspace_live_bytes();

}  // namespace cuda
}  // namespace vkernels::kernels
