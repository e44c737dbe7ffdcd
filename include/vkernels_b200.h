/* vkernels_b200.h - C ABI of libvkernels_b200.so: the fused MXFP4
 * mixture-of-experts layer for NVIDIA B200 (sm_100a).
 *
 * The first group of entry points keeps the names, argument lists and error
 * behaviour of the reference library's entry points for this path, so a loader
 * written against the reference binds them unchanged; each comment names the
 * reference declaration it replaces (paths relative to the reference tree).
 * The vk_cuda_* group is additive.
 *
 * Conventions (reference src/c/vkernels/capi/capi.hpp:41-68): int-returning
 * functions return VK_OK or a VK_ERROR_* code and leave a message readable
 * through vk_last_error() on the calling thread; nothing throws across this
 * boundary. Device entry points take DEVICE pointers, enqueue on `stream`
 * (NULL = default stream) and return without synchronising. */
#ifndef VKERNELS_B200_H_
#define VKERNELS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes - capi.hpp:41-47. */
enum {
  VK_OK = 0,
  VK_ERROR_INVALID_ARGUMENT = 1,
  VK_ERROR_OUT_OF_RANGE = 2,
  VK_ERROR_UNSUPPORTED = 3,
  VK_ERROR_INTERNAL = 4
};

/* capi.hpp:53-68. */
const char* vk_version(void);
int vk_has_cuda(void);
const char* vk_last_error(void);
int vk_last_error_code(void);
void vk_set_last_error(int code, const char* message);

/* ---- device entry points (DEVICE pointers) ------------------------------ */

/* Replaces vk_hip_fused_moe_mxfp4 - src/c/vkernels/capi/hip_capi.hpp:99-108
 * (C++ launcher src/c/vkernels/kernels/moe_fused.hpp:322-344).
 *   A [M,hidden] bf16; w13 [E,2*ispp,hidden/2] packed E2M1, gate rows then up
 *   rows; w13_scale [E,2*ispp,hidden/32] ue8m0; w2 [E,hidden,ispp/2];
 *   w2_scale [E,hidden,ispp/32]; topk_ids unused by the kernels (kept for the
 *   signature); topk_w [M*top_k] read at the flat index; act_scratch
 *   [EM,ispp] bf16, padding rows never written; out [M,hidden] fp32,
 *   ACCUMULATED INTO - zero it first; sorted_ids [EM], expert_ids
 *   [EM/block_size] as produced by the alignment; activation 0 = SwiGLU
 *   (clamped at swiglu_limit when > 0), 1 = SiTU(beta, linear_beta);
 *   b13 [E,2*ispp] / b2 [E,hidden] fp32 or NULL; block_size = alignment
 *   granularity (any multiple of 16; 16 packs best on this implementation).
 * void like the reference: a contract violation leaves a message in
 * vk_last_error() and launches nothing. */
void vk_hip_fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                            const uint8_t* w2, const uint8_t* w2_scale, const int32_t* topk_ids,
                            const float* topk_w, uint16_t* act_scratch, float* out, int M,
                            int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                            const int32_t* expert_ids, int EM, float swiglu_limit, int activation,
                            float beta, float linear_beta, const float* b13, const float* b2,
                            int block_size, void* stream);

/* Replaces vk_hip_moe_align_block_size - hip_capi.hpp:148-153 (kernel
 * src/c/vkernels/kernels/moe_fused.hip:1983-2099). Same outputs, bit for bit,
 * as the host alignment (src/c/vkernels/kernels/moe_fused.cpp:609-661) for any
 * N = M*top_k: the reference's N <= 1024 limit (VK_ERROR_UNSUPPORTED) is gone.
 * expert_map [num_experts] global->local (-1 = skip) or NULL. All max_EM
 * entries of sorted_ids and max_EM/block_size of expert_ids are written;
 * *out_EM (device) receives the padded row count, block_size when nothing
 * routes. */
int vk_hip_moe_align_block_size(const int32_t* topk_ids, const int32_t* expert_map, int32_t M,
                                int32_t top_k, int32_t block_size, int32_t num_experts,
                                int32_t local_n, int32_t max_EM, int32_t* sorted_ids,
                                int32_t* expert_ids, int32_t* out_EM, void* stream);

/* ---- host entry points (HOST pointers) ----------------------------------- */

/* Replaces vk_fused_moe_mxfp4 - capi.hpp:515-524 (capi_moe.cpp:81-108), whose
 * body is the CPU oracle. Here every buffer is copied to the GPU, the CUDA
 * kernels run and act_scratch/out are copied back; the call synchronises.
 * topk_w_sorted [EM] is in sorted-row order; expert_ids is per 16 rows;
 * group_size must be 32. */
int32_t vk_fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                           const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                           const float* topk_w_sorted, const int32_t* expert_ids,
                           uint16_t* act_scratch, float* out, int M, int hidden, int ispp,
                           int top_k, int EM, int group_size, float swiglu_limit, int activation,
                           float beta, float linear_beta, const float* b13, const float* b2);

/* Replaces vk_moe_align_block_size - capi.hpp:530-533 (capi_moe.cpp:119-140):
 * host buffers, GPU execution, host contract (*out_EM = 0 when nothing
 * routes; only the first *out_EM entries are written). */
int32_t vk_moe_align_block_size(const int32_t* topk_ids, int32_t M, int32_t top_k,
                                int32_t block_size, int32_t num_experts, int32_t* sorted_ids,
                                int32_t* expert_ids, int32_t* out_EM);

/* capi.hpp:537-539 (capi_moe.cpp:110-117). */
size_t vk_moe_align_block_size_max_em(int32_t M, int32_t top_k, int32_t block_size,
                                      int32_t num_experts);

/* ---- additive entry points (DEVICE pointers) ------------------------------ */

/* No counterpart in the reference. The alignment of vk_hip_moe_align_block_size
 * for callers that cannot allocate device memory during a call: a server whose
 * memory pool owns all free memory after warm-up, or a step that cannot afford
 * the device-wide stall of cudaMalloc. The other entry point may grow the
 * library's scratch block for large batches; this one keeps its chunk
 * histograms in a fixed array compiled into the library (about 514 KB of
 * device memory per GPU that loads the library, held until exit) and never
 * allocates. Same arguments, same outputs bit for bit. Limits: M*top_k <=
 * 262144 and local_n <= 512, otherwise VK_ERROR_INVALID_ARGUMENT with a
 * message naming the limit. All calls on a device share the array: calls that
 * may overlap on the GPU (different streams without ordering) race - serialise
 * them. The first call on each device looks up the array's address; make it
 * before starting a stream capture. */
int vk_cuda_moe_align_block_size_noalloc(const int32_t* topk_ids, const int32_t* expert_map,
                                         int32_t M, int32_t top_k, int32_t block_size,
                                         int32_t num_experts, int32_t local_n, int32_t max_EM,
                                         int32_t* sorted_ids, int32_t* expert_ids, int32_t* out_EM,
                                         void* stream);

/* The layer with routing weights already in sorted-row order (the CPU entry
 * point's convention, moe_fused.hpp:83-101) - no reference counterpart on the
 * device side. */
int vk_cuda_fused_moe_mxfp4_sorted_w(const uint16_t* A, const uint8_t* w13,
                                     const uint8_t* w13_scale, const uint8_t* w2,
                                     const uint8_t* w2_scale, const float* topk_w_sorted,
                                     uint16_t* act_scratch, float* out, int M, int hidden,
                                     int ispp, int top_k, const int32_t* sorted_ids,
                                     const int32_t* expert_ids, int EM, float swiglu_limit,
                                     int activation, float beta, float linear_beta,
                                     const float* b13, const float* b2, int block_size,
                                     void* stream);

/* The layer with a bf16 result and an ordered, atomic-free combine (no device-side counterpart
 * in the reference for this path; the idea is its W4A4 scatter-reduce's inverse-permutation
 * gather, src/c/vkernels/kernels/moe_aux.hpp:150-155). Arguments as vk_hip_fused_moe_mxfp4 with
 * y [M, hidden] bf16 in place of the fp32 `out`: y is OVERWRITTEN with bf16(sum over the token's
 * experts in ascending expert order of (act @ w2^T + b2) * w), the order in which the CPU oracle
 * adds (moe_fused.cpp:539-562). Bit-reproducible from run to run; nothing to zero before or
 * convert after the call. At most 32 slots per token. The library scratch of the stream must
 * hold vk_cuda_moe_workspace_bytes_bf16(...) bytes (EM * hidden fp32 more than the plain form). */
int vk_cuda_fused_moe_mxfp4_bf16(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                                 const uint8_t* w2_scale, const float* topk_w, uint16_t* act_scratch, uint16_t* y,
                                 int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                                 const int32_t* expert_ids, int EM, float swiglu_limit, int activation, float beta,
                                 float linear_beta, const float* b13, const float* b2, int block_size, void* stream);
size_t vk_cuda_moe_workspace_bytes_bf16(int max_EM, int hidden, int ispp, int n_local_experts, int N);

/* Prepacked weights for decode-size batches (additive; the reference passes the checkpoint
 * layout through untouched, src/python/vkernels/vllm_experts.py:531-582, and so do all entry
 * points above). A one-time rewrite at model load: magnitude codes c >= 2 become c + 2, so that
 * the tensor core's own e2m1 reading of a nibble is exactly twice the layer's table value
 * (src/c/vkernels/kernels/moe_fused.cpp dequant table {0,.25,1,1.5,2,3}; the kernel halves the
 * sums), groups with scale byte 0xFF become zero codes, and the scales are regrouped per
 * (expert, 128-row work item, 256-K stage). The kernels then expand nothing.
 *   which = 0: w13 [E, 2*ispp, hidden/2] + scales [E, 2*ispp, hidden/32]
 *   which = 1: w2  [E, hidden, ispp/2]   + scales [E, hidden, ispp/32]
 * vk_cuda_moe_prepack_sizes gives the two output sizes (the code buffer is the checkpoint size
 * plus 128 rows and 64 bytes of padding); w_out must be 32-byte aligned. *nonfinite (device int)
 * receives the number of 32-element groups holding code 6 or 7 (inf / NaN in this layer, not
 * expressible in e2m1): a caller that reads a non-zero count must not use the prepacked form. */
int vk_cuda_moe_prepack_sizes(int which, int E, int hidden, int ispp, size_t* w_bytes, size_t* sf_bytes);
int vk_cuda_moe_prepack_weights(int which, const uint8_t* w, const uint8_t* scale, int E, int hidden, int ispp,
                                uint8_t* w_out, uint8_t* sf_out, int* nonfinite, void* stream);
/* vk_cuda_fused_moe_mxfp4_bf16 on prepacked weights (codes + regrouped scales of both sets).
 * Serves batches whose token tiles stay within 64 rows (M <= 256 always does); larger batches
 * return VK_ERROR_INVALID_ARGUMENT and belong to the checkpoint-layout entry points. */
int vk_cuda_fused_moe_mxfp4_bf16_prepacked(const uint16_t* A, const uint8_t* w13_codes, const uint8_t* w13_sf,
                                           const uint8_t* w2_codes, const uint8_t* w2_sf, const float* topk_w,
                                           uint16_t* act_scratch, uint16_t* y, int M, int hidden, int ispp, int top_k,
                                           const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                                           float swiglu_limit, int activation, float beta, float linear_beta,
                                           const float* b13, const float* b2, int block_size, void* stream);

/* Router. The reference has no router in this path; semantics follow its GPU
 * routing ops (src/python/vkernels/torch_ops/tokenspeed_amd/routing.py:58-145,
 * torch_ops/glm_router.py:43-88,184-262).
 * logits[T,E] = bf16 x[T,H] . fp32 wr[E,H]^T, fp32 accumulation.
 * Batches above 512 tokens use the stream's library scratch (the bf16 terms of the router weight
 * and, when the reduction is cut into slices, one [T,E] plane per slice): at most
 * 5 KB + 6*E*H + 32*T*E bytes - less than the layer call of the same batch needs, so a stream
 * reserved for the layer is reserved for its router. */
int vk_cuda_moe_router_logits(const uint16_t* x, const float* wr, float* logits, int T, int H,
                              int E, void* stream);
/* sigmoid = 0: softmax scores, selection on score (+ bias), weights = scores,
 * renorm divides by the selected sum (0 -> 1). sigmoid = 1: selection on
 * sigmoid + bias, weights = unbiased sigmoid, renorm divides by sum + 1e-20;
 * n_group > 1 keeps the topk_group groups with the largest sum of their two
 * best biased scores. Ties go to the lowest index; ids are in descending
 * selection order. ids/w are [T, k + n_shared]; trailing shared slots carry
 * ids E, E+1, ... and weight 1. */
int vk_cuda_moe_route_topk(const float* logits, const float* bias, int T, int E, int k,
                           int sigmoid, int n_group, int topk_group, int renorm, float scaling,
                           int n_shared, int32_t* ids, float* w, void* stream);

/* vk_cuda_moe_route_topk followed by vk_hip_moe_align_block_size (no expert map, num_experts =
 * local_n = E + n_shared) as one single-CTA kernel, for at most 1024 routed slots (T * (k +
 * n_shared)) - the decode regime, where each launch removed from the step counts. Same outputs
 * as the two calls, bit for bit. The reference's precedent for fusing the router into the layer's
 * front end: src/python/vkernels/torch_ops/glm_router_dense.py:112-150, glm_router.py:205-262. */
int vk_cuda_moe_route_align_small(const float* logits, const float* bias, int T, int E, int k, int sigmoid,
                                  int n_group, int topk_group, int renorm, float scaling, int n_shared,
                                  int block_size, int max_EM, int32_t* ids, float* w, int32_t* sorted_ids,
                                  int32_t* expert_ids, int32_t* out_em, void* stream);

/* 0 = tcgen05 tensor-core kernels (default), 1 = CUDA-core cross-check kernels
 * that add in the CPU oracle's order. Also settable with VK_MOE_IMPL=simt. */
int vk_cuda_moe_set_impl(int impl);
int vk_cuda_moe_get_impl(void);

/* Library scratch (alignment histograms, tile lists, gathered activation rows): one block per
 * (device, stream). Layer and alignment calls on different streams therefore never share
 * scratch and may run concurrently; calls on one stream are ordered by the stream. The
 * launchers keep the reference's ownership rule (src/c/vkernels/kernels/moe_fused.hpp:296-307:
 * no synchronisation, no free) with one exception: the FIRST call on a stream, or a call larger
 * than everything before it on that stream, allocates the stream's block with cudaMalloc (the
 * outgrown block stays alive for enqueued work and captured graphs until
 * vk_cuda_moe_release_workspaces). vk_cuda_moe_reserve_workspace_on(bytes, stream) does that
 * allocation ahead of time; with the block reserved the launchers allocate nothing. While
 * `stream` is being captured an allocation is impossible: the call launches nothing and reports
 * VK_ERROR_INVALID_ARGUMENT ("reserve ... before the capture").
 * vk_cuda_moe_reserve_workspace(bytes) reserves for the default stream (NULL).
 * vk_cuda_moe_release_workspaces frees all blocks of the current device: only when none of the
 * library's work is pending and no captured graph using them will be replayed. */
size_t vk_cuda_moe_workspace_bytes(int max_EM, int hidden, int ispp, int n_local_experts, int N);
int vk_cuda_moe_reserve_workspace(size_t bytes);
int vk_cuda_moe_reserve_workspace_on(size_t bytes, void* stream);
int vk_cuda_moe_release_workspaces(void);
size_t vk_cuda_moe_workspace_live_bytes(void);

/* Every wait inside the tensor-core kernels is bounded (about two seconds of SM clock); a wait
 * that runs out makes its CTA free its tensor memory and return, and records 100 + the wait's
 * code in a status word of the device. vk_cuda_moe_kernel_status synchronises the device and
 * returns VK_ERROR_INTERNAL if the word is set (never expected); the word stays set until
 * vk_cuda_moe_reset_kernel_status clears it (also synchronises). */
int vk_cuda_moe_kernel_status(void);
int vk_cuda_moe_reset_kernel_status(void);
/* Test hook for that path: one warp waits with the kernels' own bounded wait on a barrier
 * nobody arrives on and gives up after limit_clocks (1 .. 2e9) SM clocks, which sets the status
 * word like a GEMM kernel would. It returns by itself; nothing hangs and no real launch is
 * starved. */
int vk_cuda_moe_test_wait_timeout(long long limit_clocks, void* stream);

/* Device time of the two GEMM kernels, measured with events on the launch
 * stream around up to max_calls layer calls; _end synchronises and returns the
 * summed milliseconds (the reference's VK_MOE_KTIME=1 prints the same split,
 * src/c/vkernels/kernels/moe_fused.hip:1482-1493, but serialises the stages). */
int vk_cuda_moe_timing_begin(int max_calls);
int vk_cuda_moe_timing_end(float* gateup_ms, float* down_ms, int* calls);

/* out[rows,K] bf16 = dequantised packed[rows,K/2] x scale[rows,K/32] (reference definition
 * moe_fused.cpp:141-174), through the device functions the GEMM kernels decode with:
 * path 0 = the byte-permute decoder of the CTA-pair (prefill) form, path 1 = the shared-memory
 * table decoder of the lone-CTA (decode) form (K % 64 == 0, 16-byte aligned buffers).
 * vk_cuda_mxfp4_dequant_rows is path 0. */
int vk_cuda_mxfp4_dequant_rows(const uint8_t* packed, const uint8_t* scale, uint16_t* out,
                               int rows, int K, void* stream);
int vk_cuda_mxfp4_dequant_rows_path(const uint8_t* packed, const uint8_t* scale, uint16_t* out,
                                    int rows, int K, int path, void* stream);

/* Expert parallelism (partition rule: src/c/vkernels/dist/dist_moe.cpp:225-274).
 * expert_begin [world+1]: first expert of each rank, last entry = E.
 * phase 0: cursor[d] += number of tokens that must visit rank d (cursor zeroed
 *          by the caller).
 * phase 1: cursor[d] = first row of rank d's segment of the send buffers; each
 *          visiting token takes the next row: send_x[row,:] = x[t,:],
 *          send_ids/send_w [row, k + n_shared] = LOCAL expert id / weight of
 *          the slots rank d owns (-1 / 0 elsewhere; shared slots only for
 *          d == rank), row_of[t, d] = row or -1. */
int vk_cuda_moe_ep_pack(const uint16_t* x, const int32_t* topk_ids, const float* topk_w, int T,
                        int H, int k, int n_shared, int world, int rank,
                        const int32_t* expert_begin, int32_t* cursor, int32_t* row_of,
                        uint16_t* send_x, int32_t* send_ids, float* send_w, int phase,
                        void* stream);
/* out[t,:] = sum over ranks d ascending of recv_rows[row_of[t,d], :]; either
 * output may be NULL. */
int vk_cuda_moe_ep_combine(const float* recv_rows, const int32_t* row_of, int T, int H, int world,
                           uint16_t* out_bf16, float* out_f32, void* stream);

/* The layer in four stages for tensor parallelism: counterparts of the reference's
 * hip::moe_gateup_preact / moe_act_epilogue / moe_down_preact / moe_combine
 * (src/c/vkernels/kernels/moe_fused.hpp:265-286), same argument lists plus the stream, status
 * code returned. w13 / w2 are the rank's K-shards ([E, 2*ispp, hidden_k/2], [E, hidden,
 * ispp_k/2], scales accordingly; hidden_k, ispp_k, k_base multiples of 64), k_base is the first
 * column of A / act the shard covers; the caller all-reduces gate_up and partial over the ranks
 * between the stages and passes the biases only to the element-wise stages. Blocks of 16 rows.
 *   gate_up [EM, 2*ispp] fp32 (overwritten for rows of used blocks), act [EM, ispp] bf16
 *   (padding rows not written), partial [EM, hidden] fp32, out [M, hidden] fp32 (accumulated). */
int vk_cuda_moe_gateup_preact(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                              const int32_t* sorted_ids, const int32_t* expert_ids, float* gate_up, int M,
                              int hidden, int ispp, int top_k, int EM, int k_base, int hidden_k, void* stream);
int vk_cuda_moe_act_epilogue(const float* gate_up, const float* b13, uint16_t* act, const int32_t* sorted_ids,
                             const int32_t* expert_ids, int M, int top_k, int EM, int ispp, float swiglu_limit,
                             int activation, float beta, float linear_beta, void* stream);
int vk_cuda_moe_down_preact(const uint16_t* act, const uint8_t* w2, const uint8_t* w2_scale,
                            const int32_t* sorted_ids, const int32_t* expert_ids, float* partial, int M, int ispp,
                            int hidden, int top_k, int EM, int k_base, int ispp_k, void* stream);
int vk_cuda_moe_combine(const float* partial, const float* b2, const float* topk_w_sorted,
                        const int32_t* sorted_ids, const int32_t* expert_ids, float* out, int M, int hidden,
                        int top_k, int EM, void* stream);

/* Peer-memory form of expert parallelism (no reference counterpart: the reference moves token
 * rows and partial results through its collective, dist_moe.cpp:276-328). Only routing records
 * travel through the collective; the expert kernels read each token row and add each result in
 * the home rank's memory, mapped into this process (peer loads and red.global.add over NVLink).
 *
 * vk_cuda_moe_ep_pack_meta: like phase 1 of vk_cuda_moe_ep_pack, but writes only
 *   meta [rows, 1 + 2*(k + n_shared)] int32 = {home token index, local expert id per slot
 *   (-1 = another rank's), routing weight bits per slot}.
 * vk_cuda_moe_ep_unpack_meta: received records (grouped by source rank, recv_counts[s] rows from
 *   rank s) -> ids / w [R, slots] for the local expert call, and per row the address of the
 *   token's activation row (x_bases[s] + token*H*2) and fp32 output row (out_bases[s] + token*H*4).
 * vk_cuda_fused_moe_mxfp4_rows: vk_hip_fused_moe_mxfp4 with row address arrays in place of A and
 *   out (a_rows[m], out_rows[m]: device arrays of M addresses, rows 16-byte aligned). */
int vk_cuda_moe_ep_pack_meta(const int32_t* topk_ids, const float* topk_w, int T, int k, int n_shared,
                             int world, int rank, const int32_t* expert_begin, int32_t* cursor,
                             int32_t* meta, void* stream);
int vk_cuda_moe_ep_unpack_meta(const int32_t* meta, int R, int slots, const int32_t* recv_counts,
                               int world, const uint64_t* x_bases, const uint64_t* out_bases, int H,
                               int32_t* ids, float* w, uint64_t* a_rows, uint64_t* out_rows,
                               void* stream);
/* Host-free record exchange: meta_bases[d] / count_bases[d] are the addresses, in this process,
 * of rank d's receive area (world segments of cap records, one per source rank) and of its
 * count array (world int32). pack: writes this rank's records for d into segment `rank` of d's
 * area and then its count into count_bases[d][rank] (cursor [world] zeroed by the caller).
 * unpack: over all world*cap record slots of the local area; slots past recv_counts[s] become
 * "not routed" rows (ids -1, w 0); out_rows[r] = out_bases[s] + token * out_rows_per_token * H * 4
 * (1 for the reduction form, slots for the slot-store form below). pack also resets its cursor to
 * zero after publishing the counts. A cross-rank barrier belongs between the two. */
int vk_cuda_moe_ep_pack_meta_peer(const int32_t* topk_ids, const float* topk_w, int T, int k,
                                  int n_shared, int world, int rank, const int32_t* expert_begin,
                                  int32_t* cursor, const uint64_t* meta_bases,
                                  const uint64_t* count_bases, int cap, void* stream);
int vk_cuda_moe_ep_unpack_meta_peer(const int32_t* meta, const int32_t* recv_counts, int world, int cap,
                                    int slots, const uint64_t* x_bases, const uint64_t* out_bases,
                                    int H, int out_rows_per_token, int32_t* ids, float* w, uint64_t* a_rows,
                                    uint64_t* out_rows, void* stream);
/* Slot-store form of the combine: vk_cuda_fused_moe_mxfp4_rows_store is
 * vk_cuda_fused_moe_mxfp4_rows with out_blocks[m] = address of a [top_k, hidden] fp32 block of
 * token m (in its home rank's memory); the row of slot j - act @ w2^T + b2, NOT weighted - is
 * written to row j with plain 16-byte stores instead of being added with reductions. After a
 * cross-rank barrier the home rank runs vk_cuda_moe_ep_combine_slots: y[t,:] = bf16(sum over the
 * slots j in ascending global expert id ids[t,j] of w[t,j] * part[t,j,:]); slots with an id
 * outside [0, n_experts) are skipped; either output may be NULL. No atomics: the result is
 * bit-reproducible and adds in the single-rank oracle's order (moe_fused.cpp:539-562). */
int vk_cuda_fused_moe_mxfp4_rows_store(const uint64_t* a_rows, const uint8_t* w13, const uint8_t* w13_scale,
                                       const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                                       uint16_t* act_scratch, const uint64_t* out_blocks, int M, int hidden,
                                       int ispp, int top_k, const int32_t* sorted_ids,
                                       const int32_t* expert_ids, int EM, float swiglu_limit, int activation,
                                       float beta, float linear_beta, const float* b13, const float* b2,
                                       int block_size, void* stream);
int vk_cuda_moe_ep_combine_slots(const float* part, const int32_t* ids, const float* w, int T, int k, int n_experts,
                                 int H, uint16_t* y_bf16, float* out_f32, void* stream);

/* Cross-rank barrier of the peer-memory form, run as a kernel on `stream`: flag_bases[d] is the
 * address, in this process, of rank d's flag array ([8 slots][world] int32, zero at start, in
 * memory every rank can address). The kernel publishes `epoch` into entry [slot][rank] of every
 * rank's array (system-scope release, after a system-scope fence over this stream's earlier
 * writes) and waits until every entry [slot][*] of its own array has reached `epoch` (acquire).
 * Epochs must grow from call to call on a slot. The wait gives up after limit_clocks SM clocks
 * (at most 8e9): the kernel then records 200 + the missing rank in a status word that
 * vk_cuda_moe_kernel_status reports, and returns - a rank that left does not hang the others.
 * epoch_counter (device, [8] int32, zero at start, or NULL): when given, `epoch` is ignored and the
 * kernel increments entry [slot] and uses its new value - the form a captured CUDA graph can
 * replay; every rank must then run the barrier the same number of times. */
int vk_cuda_moe_ep_flag_barrier(const uint64_t* flag_bases, int world, int rank, int slot, int epoch,
                                long long limit_clocks, int32_t* epoch_counter, void* stream);
int vk_cuda_fused_moe_mxfp4_rows(const uint64_t* a_rows, const uint8_t* w13, const uint8_t* w13_scale,
                                 const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                                 uint16_t* act_scratch, const uint64_t* out_rows, int M, int hidden,
                                 int ispp, int top_k, const int32_t* sorted_ids,
                                 const int32_t* expert_ids, int EM, float swiglu_limit, int activation,
                                 float beta, float linear_beta, const float* b13, const float* b2,
                                 int block_size, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VKERNELS_B200_H_ */
