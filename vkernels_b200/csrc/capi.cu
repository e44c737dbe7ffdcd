// capi.cu - extern "C" surface of libvkernels_b200.so (declared in
// include/vkernels_b200.h). No C++ type and no exception crosses this
// boundary: failures become a status code plus a thread-local message, the
// convention of the reference's C ABI (src/c/vkernels/capi/capi.hpp:41-68,
// capi_internal.hpp:37-67).
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "moe_fused.hpp"

namespace vkc = vkernels::kernels::cuda;

namespace vkernels::kernels::cuda {
int sm100_last_status();
void timing_begin(int max_calls);
void timing_end(float* gateup_ms, float* down_ms, int* calls);
void launch_dequant_rows(const uint8_t* packed, const uint8_t* scale, uint16_t* out, int rows,
                         int K, int path, cudaStream_t stream);
void sm100_reset_status();
int ep_last_status();
void ep_reset_status();
void ep_launch_flag_barrier(const unsigned long long* flag_bases, int world, int rank, int slot, int epoch,
                            long long limit_clocks, int* epoch_counter, cudaStream_t stream);
void launch_wait_timeout_probe(long long limit_clocks, cudaStream_t stream);
void ep_launch_pack(const uint16_t* x, const int32_t* topk_ids, const float* topk_w, int T, int H,
                    int k, int n_shared, int world, int rank, const int32_t* expert_begin,
                    int32_t* cursor, int32_t* row_of, uint16_t* send_x, int32_t* send_ids,
                    float* send_w, int phase, cudaStream_t stream);
void ep_launch_combine(const float* recv_rows, const int32_t* row_of, int T, int H, int world,
                       uint16_t* out_bf16, float* out_f32, cudaStream_t stream);
void ep_launch_pack_meta(const int32_t* topk_ids, const float* topk_w, int T, int k, int n_shared,
                         int world, int rank, const int32_t* expert_begin, int32_t* cursor,
                         int32_t* meta, cudaStream_t stream);
void ep_launch_unpack_meta(const int32_t* meta, int R, int slots, const int32_t* recv_counts, int world,
                           const unsigned long long* x_bases, const unsigned long long* out_bases,
                           int H, int32_t* ids, float* w, unsigned long long* a_rows,
                           unsigned long long* out_rows, cudaStream_t stream);
void ep_launch_pack_meta_peer(const int32_t* topk_ids, const float* topk_w, int T, int k, int n_shared,
                              int world, int rank, const int32_t* expert_begin, int32_t* cursor,
                              const unsigned long long* meta_bases, const unsigned long long* count_bases,
                              int cap, cudaStream_t stream);
void ep_launch_unpack_meta_peer(const int32_t* meta, const int32_t* recv_counts, int world, int cap,
                                int slots, const unsigned long long* x_bases,
                                const unsigned long long* out_bases, int H, int out_rows_per_token, int32_t* ids,
                                float* w, unsigned long long* a_rows, unsigned long long* out_rows,
                                cudaStream_t stream);
void ep_launch_combine_slots(const float* part, const int32_t* ids, const float* w, int T, int k, int n_experts, int H,
                             uint16_t* y_bf16, float* out_f32, cudaStream_t stream);
}  // namespace vkernels::kernels::cuda

enum { VK_OK = 0, VK_ERROR_INVALID_ARGUMENT = 1, VK_ERROR_OUT_OF_RANGE = 2,
       VK_ERROR_UNSUPPORTED = 3, VK_ERROR_INTERNAL = 4 };

namespace {
thread_local int g_code = VK_OK;
thread_local std::string g_msg;
void set_error(int code, const char* msg) {
  g_code = code;
  g_msg = msg ? msg : "";
}
}  // namespace

#define VK_TRY try {
#define VK_CATCH(ret_ok, on_error)                                            \
    ret_ok;                                                                   \
  } catch (const std::invalid_argument& e) {                                  \
    set_error(VK_ERROR_INVALID_ARGUMENT, e.what()); on_error(VK_ERROR_INVALID_ARGUMENT); \
  } catch (const std::out_of_range& e) {                                      \
    set_error(VK_ERROR_OUT_OF_RANGE, e.what()); on_error(VK_ERROR_OUT_OF_RANGE); \
  } catch (const std::length_error& e) {                                      \
    set_error(VK_ERROR_INVALID_ARGUMENT, e.what()); on_error(VK_ERROR_INVALID_ARGUMENT); \
  } catch (const std::bad_alloc&) {                                           \
    set_error(VK_ERROR_INTERNAL, "out of memory"); on_error(VK_ERROR_INTERNAL); \
  } catch (const std::exception& e) {                                         \
    set_error(VK_ERROR_INTERNAL, e.what()); on_error(VK_ERROR_INTERNAL);      \
  } catch (...) {                                                             \
    set_error(VK_ERROR_INTERNAL, "unknown C++ exception"); on_error(VK_ERROR_INTERNAL); \
  }
#define VK_RETURN_CODE(c) return (c)
#define VK_RETURN_VOID(c) return

namespace {
// RAII device buffer for the host-pointer entry points.
struct DevBuf {
  void* p = nullptr;
  explicit DevBuf(size_t bytes) {
    if (bytes > 0) VK_CUDA_CHECK(cudaMalloc(&p, bytes));
  }
  DevBuf(const void* host, size_t bytes) : DevBuf(bytes) {
    if (bytes > 0 && host) VK_CUDA_CHECK(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice));
  }
  ~DevBuf() { if (p) cudaFree(p); }
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  template <class T> T* as() const { return static_cast<T*>(p); }
};
}  // namespace

extern "C" {

const char* vk_version(void) { return "0.1.0-b200"; }
int vk_has_cuda(void) { return 1; }
const char* vk_last_error(void) { return g_msg.c_str(); }
int vk_last_error_code(void) { return g_code; }
void vk_set_last_error(int code, const char* message) { set_error(code, message); }

/* ---------------- device entry points (device pointers) ---------------- */

void vk_hip_fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                            const uint8_t* w2, const uint8_t* w2_scale, const int32_t* topk_ids,
                            const float* topk_w, uint16_t* act_scratch, float* out, int M,
                            int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                            const int32_t* expert_ids, int EM, float swiglu_limit, int activation,
                            float beta, float linear_beta, const float* b13, const float* b2,
                            int block_size, void* stream) {
  VK_TRY
  vkc::fused_moe_mxfp4(A, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, act_scratch, out, M,
                       hidden, ispp, top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation,
                       beta, linear_beta, b13, b2, block_size, false, stream);
  VK_CATCH(return, VK_RETURN_VOID)
}

int vk_hip_moe_align_block_size(const int32_t* topk_ids, const int32_t* expert_map, int32_t M,
                                int32_t top_k, int32_t block_size, int32_t num_experts,
                                int32_t local_n, int32_t max_EM, int32_t* sorted_ids,
                                int32_t* expert_ids, int32_t* out_EM, void* stream) {
  VK_TRY
  vkc::moe_align_block_size(topk_ids, expert_map, M, top_k, block_size, num_experts, local_n,
                            max_EM, sorted_ids, expert_ids, out_EM, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_align_block_size_noalloc(const int32_t* topk_ids, const int32_t* expert_map,
                                         int32_t M, int32_t top_k, int32_t block_size,
                                         int32_t num_experts, int32_t local_n, int32_t max_EM,
                                         int32_t* sorted_ids, int32_t* expert_ids, int32_t* out_EM,
                                         void* stream) {
  VK_TRY
  vkc::moe_align_block_size_noalloc(topk_ids, expert_map, M, top_k, block_size, num_experts,
                                    local_n, max_EM, sorted_ids, expert_ids, out_EM, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_fused_moe_mxfp4_sorted_w(const uint16_t* A, const uint8_t* w13,
                                     const uint8_t* w13_scale, const uint8_t* w2,
                                     const uint8_t* w2_scale, const float* topk_w_sorted,
                                     uint16_t* act_scratch, float* out, int M, int hidden,
                                     int ispp, int top_k, const int32_t* sorted_ids,
                                     const int32_t* expert_ids, int EM, float swiglu_limit,
                                     int activation, float beta, float linear_beta,
                                     const float* b13, const float* b2, int block_size,
                                     void* stream) {
  VK_TRY
  vkc::fused_moe_mxfp4_sorted_w(A, w13, w13_scale, w2, w2_scale, topk_w_sorted, act_scratch, out,
                                M, hidden, ispp, top_k, sorted_ids, expert_ids, EM, swiglu_limit,
                                activation, beta, linear_beta, b13, b2, block_size, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_fused_moe_mxfp4_bf16(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                                 const uint8_t* w2_scale, const float* topk_w, uint16_t* act_scratch, uint16_t* y,
                                 int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                                 const int32_t* expert_ids, int EM, float swiglu_limit, int activation, float beta,
                                 float linear_beta, const float* b13, const float* b2, int block_size, void* stream) {
  VK_TRY
  vkc::fused_moe_mxfp4_bf16(A, w13, w13_scale, w2, w2_scale, topk_w, act_scratch, y, M, hidden, ispp, top_k,
                            sorted_ids, expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13, b2,
                            block_size, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
size_t vk_cuda_moe_workspace_bytes_bf16(int max_EM, int hidden, int ispp, int n_local_experts, int N) {
  return vkc::workspace_bytes_required_bf16(max_EM, hidden, ispp, n_local_experts, N);
}

int vk_cuda_moe_prepack_sizes(int which, int E, int hidden, int ispp, size_t* w_bytes, size_t* sf_bytes) {
  VK_TRY
  vkc::prepack_sizes(which, E, hidden, ispp, w_bytes, sf_bytes);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
int vk_cuda_moe_prepack_weights(int which, const uint8_t* w, const uint8_t* scale, int E, int hidden, int ispp,
                                uint8_t* w_out, uint8_t* sf_out, int* nonfinite, void* stream) {
  VK_TRY
  vkc::prepack_weights(which, w, scale, E, hidden, ispp, w_out, sf_out, nonfinite, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
int vk_cuda_fused_moe_mxfp4_bf16_prepacked(const uint16_t* A, const uint8_t* w13_codes, const uint8_t* w13_sf,
                                           const uint8_t* w2_codes, const uint8_t* w2_sf, const float* topk_w,
                                           uint16_t* act_scratch, uint16_t* y, int M, int hidden, int ispp, int top_k,
                                           const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                                           float swiglu_limit, int activation, float beta, float linear_beta,
                                           const float* b13, const float* b2, int block_size, void* stream) {
  VK_TRY
  vkc::fused_moe_mxfp4_bf16_prepacked(A, w13_codes, w13_sf, w2_codes, w2_sf, topk_w, act_scratch, y, M, hidden, ispp,
                                      top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation, beta, linear_beta,
                                      b13, b2, block_size, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_router_logits(const uint16_t* x, const float* wr, float* logits, int T, int H,
                              int E, void* stream) {
  VK_TRY
  vkc::router_logits(x, wr, logits, T, H, E, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_route_topk(const float* logits, const float* bias, int T, int E, int k,
                           int sigmoid, int n_group, int topk_group, int renorm, float scaling,
                           int n_shared, int32_t* ids, float* w, void* stream) {
  VK_TRY
  vkc::route_topk(logits, bias, T, E, k, sigmoid, n_group, topk_group, renorm, scaling, n_shared,
                  ids, w, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_route_align_small(const float* logits, const float* bias, int T, int E, int k, int sigmoid,
                                  int n_group, int topk_group, int renorm, float scaling, int n_shared,
                                  int block_size, int max_EM, int32_t* ids, float* w, int32_t* sorted_ids,
                                  int32_t* expert_ids, int32_t* out_em, void* stream) {
  VK_TRY
  vkc::route_align_small(logits, bias, T, E, k, sigmoid, n_group, topk_group, renorm, scaling, n_shared, block_size,
                         max_EM, ids, w, sorted_ids, expert_ids, out_em, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_set_impl(int impl) {
  if (impl != 0 && impl != 1) {
    set_error(VK_ERROR_INVALID_ARGUMENT, "vk_cuda_moe_set_impl: 0 = tcgen05, 1 = simt");
    return VK_ERROR_INVALID_ARGUMENT;
  }
  vkc::set_moe_impl(static_cast<vkc::MoeImpl>(impl));
  return VK_OK;
}
int vk_cuda_moe_get_impl(void) { return static_cast<int>(vkc::get_moe_impl()); }

size_t vk_cuda_moe_workspace_bytes(int max_EM, int hidden, int ispp, int n_local_experts, int N) {
  return vkc::workspace_bytes_required(max_EM, hidden, ispp, n_local_experts, N);
}
int vk_cuda_moe_reserve_workspace(size_t bytes) {
  VK_TRY
  vkc::reserve_workspace(bytes, nullptr);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
int vk_cuda_moe_reserve_workspace_on(size_t bytes, void* stream) {
  VK_TRY
  vkc::reserve_workspace(bytes, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
int vk_cuda_moe_release_workspaces(void) {
  VK_TRY
  vkc::release_workspaces();
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
size_t vk_cuda_moe_workspace_live_bytes(void) {
  try {
    return vkc::workspace_live_bytes();
  } catch (const std::exception& e) {
    set_error(VK_ERROR_INTERNAL, e.what());
    return 0;
  }
}

/* 0 = every tensor-core launch so far completed its waits; otherwise the code
 * of the wait that ran out. Synchronises the device. */
int vk_cuda_moe_kernel_status(void) {
  VK_TRY
  const int s = vkc::sm100_last_status();
  if (s != 0) {
    const std::string m = "a tcgen05 MoE kernel gave up on a bounded wait (code " + std::to_string(s) + ")";
    set_error(VK_ERROR_INTERNAL, m.c_str());
    return VK_ERROR_INTERNAL;
  }
  const int e = vkc::ep_last_status();
  if (e != 0) {
    const std::string m = "a cross-rank flag barrier gave up on a bounded wait for rank " + std::to_string(e - 200);
    set_error(VK_ERROR_INTERNAL, m.c_str());
    return VK_ERROR_INTERNAL;
  }
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* Clears the status word of the current device. Synchronises the device. */
int vk_cuda_moe_reset_kernel_status(void) {
  VK_TRY
  vkc::sm100_reset_status();
  vkc::ep_reset_status();
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* Test hook: one warp waits, with the kernels' own bounded wait, on a barrier nobody arrives on
 * and gives up after limit_clocks SM clocks, which sets the status word. Nothing hangs. */
int vk_cuda_moe_test_wait_timeout(long long limit_clocks, void* stream) {
  VK_TRY
  vkc::launch_wait_timeout_probe(limit_clocks, static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* Per-kernel device times of the tensor-core path: events are recorded around the
 * gate/up and the down kernels of up to max_calls layer calls (no
 * synchronisation while recording); vk_cuda_moe_timing_end synchronises and
 * returns the summed milliseconds and the number of calls seen. */
int vk_cuda_moe_timing_begin(int max_calls) {
  VK_TRY
  vkc::expects(max_calls > 0, "timing_begin: max_calls must be positive");
  vkc::timing_begin(max_calls);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
int vk_cuda_moe_timing_end(float* gateup_ms, float* down_ms, int* calls) {
  VK_TRY
  vkc::timing_end(gateup_ms, down_ms, calls);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* Test hooks: out[rows, K] bf16 = dequantised packed[rows, K/2] with scale[rows, K/32], through
 * the device functions the GEMM kernels decode with. vk_cuda_mxfp4_dequant_rows runs the
 * byte-permute decoder of the CTA-pair form; the _path variant selects the decoder:
 * 0 = byte permutes, 1 = the shared-memory table of the lone-CTA form (K % 64 == 0). */
int vk_cuda_mxfp4_dequant_rows_path(const uint8_t* packed, const uint8_t* scale, uint16_t* out,
                                    int rows, int K, int path, void* stream) {
  VK_TRY
  vkc::expects(rows >= 0 && K > 0 && K % 32 == 0, "mxfp4_dequant_rows: K must be a multiple of 32");
  if (rows > 0) {
    vkc::expects(packed && scale && out, "mxfp4_dequant_rows: null buffer");
    vkc::launch_dequant_rows(packed, scale, out, rows, K, path, static_cast<cudaStream_t>(stream));
  }
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}
int vk_cuda_mxfp4_dequant_rows(const uint8_t* packed, const uint8_t* scale, uint16_t* out,
                               int rows, int K, void* stream) {
  return vk_cuda_mxfp4_dequant_rows_path(packed, scale, out, rows, K, 0, stream);
}

/* ---------------- expert-parallel helpers (device pointers) ------------- */

int vk_cuda_moe_ep_pack(const uint16_t* x, const int32_t* topk_ids, const float* topk_w, int T,
                        int H, int k, int n_shared, int world, int rank,
                        const int32_t* expert_begin, int32_t* cursor, int32_t* row_of,
                        uint16_t* send_x, int32_t* send_ids, float* send_w, int phase,
                        void* stream) {
  VK_TRY
  vkc::ep_launch_pack(x, topk_ids, topk_w, T, H, k, n_shared, world, rank, expert_begin, cursor,
                      row_of, send_x, send_ids, send_w, phase, static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_combine(const float* recv_rows, const int32_t* row_of, int T, int H, int world,
                           uint16_t* out_bf16, float* out_f32, void* stream) {
  VK_TRY
  vkc::ep_launch_combine(recv_rows, row_of, T, H, world, out_bf16, out_f32,
                         static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_pack_meta(const int32_t* topk_ids, const float* topk_w, int T, int k, int n_shared,
                             int world, int rank, const int32_t* expert_begin, int32_t* cursor,
                             int32_t* meta, void* stream) {
  VK_TRY
  vkc::ep_launch_pack_meta(topk_ids, topk_w, T, k, n_shared, world, rank, expert_begin, cursor, meta,
                           static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_unpack_meta(const int32_t* meta, int R, int slots, const int32_t* recv_counts,
                               int world, const uint64_t* x_bases, const uint64_t* out_bases, int H,
                               int32_t* ids, float* w, uint64_t* a_rows, uint64_t* out_rows,
                               void* stream) {
  VK_TRY
  vkc::ep_launch_unpack_meta(meta, R, slots, recv_counts, world,
                             reinterpret_cast<const unsigned long long*>(x_bases),
                             reinterpret_cast<const unsigned long long*>(out_bases), H, ids, w,
                             reinterpret_cast<unsigned long long*>(a_rows),
                             reinterpret_cast<unsigned long long*>(out_rows),
                             static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_pack_meta_peer(const int32_t* topk_ids, const float* topk_w, int T, int k,
                                  int n_shared, int world, int rank, const int32_t* expert_begin,
                                  int32_t* cursor, const uint64_t* meta_bases,
                                  const uint64_t* count_bases, int cap, void* stream) {
  VK_TRY
  vkc::ep_launch_pack_meta_peer(topk_ids, topk_w, T, k, n_shared, world, rank, expert_begin, cursor,
                                reinterpret_cast<const unsigned long long*>(meta_bases),
                                reinterpret_cast<const unsigned long long*>(count_bases), cap,
                                static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_unpack_meta_peer(const int32_t* meta, const int32_t* recv_counts, int world, int cap,
                                    int slots, const uint64_t* x_bases, const uint64_t* out_bases,
                                    int H, int out_rows_per_token, int32_t* ids, float* w, uint64_t* a_rows,
                                    uint64_t* out_rows, void* stream) {
  VK_TRY
  vkc::ep_launch_unpack_meta_peer(meta, recv_counts, world, cap, slots,
                                  reinterpret_cast<const unsigned long long*>(x_bases),
                                  reinterpret_cast<const unsigned long long*>(out_bases), H, out_rows_per_token, ids, w,
                                  reinterpret_cast<unsigned long long*>(a_rows),
                                  reinterpret_cast<unsigned long long*>(out_rows),
                                  static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_flag_barrier(const uint64_t* flag_bases, int world, int rank, int slot, int epoch,
                                long long limit_clocks, int32_t* epoch_counter, void* stream) {
  VK_TRY
  vkc::ep_launch_flag_barrier(reinterpret_cast<const unsigned long long*>(flag_bases), world, rank, slot, epoch,
                              limit_clocks, epoch_counter, static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_fused_moe_mxfp4_rows(const uint64_t* a_rows, const uint8_t* w13, const uint8_t* w13_scale,
                                 const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                                 uint16_t* act_scratch, const uint64_t* out_rows, int M, int hidden,
                                 int ispp, int top_k, const int32_t* sorted_ids,
                                 const int32_t* expert_ids, int EM, float swiglu_limit, int activation,
                                 float beta, float linear_beta, const float* b13, const float* b2,
                                 int block_size, void* stream) {
  VK_TRY
  vkc::fused_moe_mxfp4_rows(reinterpret_cast<const uint16_t* const*>(a_rows), w13, w13_scale, w2, w2_scale,
                            topk_w, act_scratch, reinterpret_cast<float* const*>(out_rows), M, hidden,
                            ispp, top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation, beta,
                            linear_beta, b13, b2, block_size, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_fused_moe_mxfp4_rows_store(const uint64_t* a_rows, const uint8_t* w13, const uint8_t* w13_scale,
                                       const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                                       uint16_t* act_scratch, const uint64_t* out_blocks, int M, int hidden,
                                       int ispp, int top_k, const int32_t* sorted_ids,
                                       const int32_t* expert_ids, int EM, float swiglu_limit, int activation,
                                       float beta, float linear_beta, const float* b13, const float* b2,
                                       int block_size, void* stream) {
  VK_TRY
  vkc::fused_moe_mxfp4_rows(reinterpret_cast<const uint16_t* const*>(a_rows), w13, w13_scale, w2, w2_scale,
                            topk_w, act_scratch, reinterpret_cast<float* const*>(out_blocks), M, hidden,
                            ispp, top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation, beta,
                            linear_beta, b13, b2, block_size, stream, true);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_ep_combine_slots(const float* part, const int32_t* ids, const float* w, int T, int k, int n_experts,
                                 int H, uint16_t* y_bf16, float* out_f32, void* stream) {
  VK_TRY
  vkc::ep_launch_combine_slots(part, ids, w, T, k, n_experts, H, y_bf16, out_f32, static_cast<cudaStream_t>(stream));
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* ---------------- tensor-parallel stage split (device pointers) --------- */

int vk_cuda_moe_gateup_preact(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                              const int32_t* sorted_ids, const int32_t* expert_ids, float* gate_up, int M,
                              int hidden, int ispp, int top_k, int EM, int k_base, int hidden_k, void* stream) {
  VK_TRY
  vkc::moe_gateup_preact(A, w13, w13_scale, sorted_ids, expert_ids, gate_up, M, hidden, ispp, top_k, EM, k_base,
                         hidden_k, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_act_epilogue(const float* gate_up, const float* b13, uint16_t* act, const int32_t* sorted_ids,
                             const int32_t* expert_ids, int M, int top_k, int EM, int ispp, float swiglu_limit,
                             int activation, float beta, float linear_beta, void* stream) {
  VK_TRY
  vkc::moe_act_epilogue(gate_up, b13, act, sorted_ids, expert_ids, M, top_k, EM, ispp, swiglu_limit, activation,
                        beta, linear_beta, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_down_preact(const uint16_t* act, const uint8_t* w2, const uint8_t* w2_scale,
                            const int32_t* sorted_ids, const int32_t* expert_ids, float* partial, int M, int ispp,
                            int hidden, int top_k, int EM, int k_base, int ispp_k, void* stream) {
  VK_TRY
  vkc::moe_down_preact(act, w2, w2_scale, sorted_ids, expert_ids, partial, M, ispp, hidden, top_k, EM, k_base,
                       ispp_k, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

int vk_cuda_moe_combine(const float* partial, const float* b2, const float* topk_w_sorted,
                        const int32_t* sorted_ids, const int32_t* expert_ids, float* out, int M, int hidden,
                        int top_k, int EM, void* stream) {
  VK_TRY
  vkc::moe_combine(partial, b2, topk_w_sorted, sorted_ids, expert_ids, out, M, hidden, top_k, EM, stream);
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* ---------------- host entry points (HOST pointers) --------------------- */

size_t vk_moe_align_block_size_max_em(int32_t M, int32_t top_k, int32_t block_size,
                                      int32_t num_experts) {
  if (block_size <= 0) return 0;
  const int32_t N = M * top_k;
  const int32_t max_em = ((N + block_size - 1) / block_size + num_experts) * block_size;
  return max_em > 0 ? static_cast<size_t>(max_em) : 0;
}

int32_t vk_moe_align_block_size(const int32_t* topk_ids, int32_t M, int32_t top_k,
                                int32_t block_size, int32_t num_experts, int32_t* sorted_ids,
                                int32_t* expert_ids, int32_t* out_EM) {
  VK_TRY
  vkc::expects(block_size > 0, "block_size must be positive");
  vkc::expects(num_experts >= 0, "num_experts must be non-negative");
  vkc::expects(M >= 0 && top_k >= 0, "M and top_k must be non-negative");
  vkc::expects(out_EM != nullptr, "out_EM must not be null");
  vkc::expects(M == 0 || (topk_ids && sorted_ids && expert_ids),
               "topk_ids/sorted_ids/expert_ids must not be null");
  const size_t cap = vk_moe_align_block_size_max_em(M, top_k, block_size, num_experts);
  if (cap == 0 || M == 0) {  // nothing routes: the host contract reports EM = 0
    *out_EM = 0;
    return VK_OK;
  }
  const size_t n = static_cast<size_t>(M) * top_k;
  DevBuf d_ids(topk_ids, n * 4), d_sorted(cap * 4), d_eids(cap / block_size * 4), d_em(4);
  vkc::moe_align_block_size(d_ids.as<int32_t>(), nullptr, M, top_k, block_size, num_experts,
                            num_experts, static_cast<int>(cap), d_sorted.as<int32_t>(),
                            d_eids.as<int32_t>(), d_em.as<int32_t>(), nullptr);
  int32_t em = 0, first = -1;
  VK_CUDA_CHECK(cudaMemcpy(&em, d_em.p, 4, cudaMemcpyDeviceToHost));
  VK_CUDA_CHECK(cudaMemcpy(&first, d_eids.p, 4, cudaMemcpyDeviceToHost));
  if (first < 0) em = 0;  // the device contract reports one padding block instead
  VK_CUDA_CHECK(cudaMemcpy(sorted_ids, d_sorted.p, static_cast<size_t>(em) * 4,
                           cudaMemcpyDeviceToHost));
  VK_CUDA_CHECK(cudaMemcpy(expert_ids, d_eids.p, static_cast<size_t>(em / block_size) * 4,
                           cudaMemcpyDeviceToHost));
  *out_EM = em;
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

/* Host-pointer form of the layer (reference capi.hpp:515-524): every buffer is
 * copied to the device, the CUDA kernels run, act_scratch and out come back.
 * The number of experts is not an argument; the weight copies cover expert ids
 * 0 .. max(expert_ids). `out` is accumulated into, as in the reference. */
int32_t vk_fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                           const uint8_t* w2, const uint8_t* w2_scale, const int32_t* sorted_ids,
                           const float* topk_w_sorted, const int32_t* expert_ids,
                           uint16_t* act_scratch, float* out, int M, int hidden, int ispp,
                           int top_k, int EM, int group_size, float swiglu_limit, int activation,
                           float beta, float linear_beta, const float* b13, const float* b2) {
  VK_TRY
  vkc::expects(group_size == 32, "fused_moe_mxfp4: group_size must be 32");
  vkc::expects(M >= 0 && EM >= 0 && EM % 16 == 0, "fused_moe_mxfp4: EM must be a multiple of 16");
  if (M > 0 && EM > 0) {
    vkc::expects(A && w13 && w13_scale && w2 && w2_scale && sorted_ids && topk_w_sorted &&
                     expert_ids && act_scratch && out,
                 "fused_moe_mxfp4: buffers must not be null");
    vkc::expects(hidden > 0 && hidden % 64 == 0 && ispp > 0 && ispp % 64 == 0,
                 "fused_moe_mxfp4: hidden and ispp must be multiples of 64");
    int n_exp = 0;
    for (int b = 0; b < EM / 16; ++b) n_exp = expert_ids[b] + 1 > n_exp ? expert_ids[b] + 1 : n_exp;
    if (n_exp > 0) {
      const size_t ih = static_cast<size_t>(ispp) * hidden;
      DevBuf dA(A, static_cast<size_t>(M) * hidden * 2), dw13(w13, n_exp * ih),
          dw13s(w13_scale, n_exp * ih / 16), dw2(w2, n_exp * ih / 2), dw2s(w2_scale, n_exp * ih / 32),
          dsid(sorted_ids, static_cast<size_t>(EM) * 4), dws(topk_w_sorted, static_cast<size_t>(EM) * 4),
          deid(expert_ids, static_cast<size_t>(EM / 16) * 4),
          dact(act_scratch, static_cast<size_t>(EM) * ispp * 2),
          dout(out, static_cast<size_t>(M) * hidden * 4),
          db13(b13, b13 ? static_cast<size_t>(n_exp) * 2 * ispp * 4 : 0),
          db2(b2, b2 ? static_cast<size_t>(n_exp) * hidden * 4 : 0);
      vkc::fused_moe_mxfp4_sorted_w(dA.as<uint16_t>(), dw13.as<uint8_t>(), dw13s.as<uint8_t>(),
                                    dw2.as<uint8_t>(), dw2s.as<uint8_t>(), dws.as<float>(),
                                    dact.as<uint16_t>(), dout.as<float>(), M, hidden, ispp, top_k,
                                    dsid.as<int32_t>(), deid.as<int32_t>(), EM, swiglu_limit,
                                    activation, beta, linear_beta, db13.as<float>(),
                                    db2.as<float>(), 16, nullptr);
      VK_CUDA_CHECK(cudaDeviceSynchronize());
      VK_CUDA_CHECK(cudaMemcpy(act_scratch, dact.p, static_cast<size_t>(EM) * ispp * 2,
                               cudaMemcpyDeviceToHost));
      VK_CUDA_CHECK(cudaMemcpy(out, dout.p, static_cast<size_t>(M) * hidden * 4,
                               cudaMemcpyDeviceToHost));
    }
  }
  VK_CATCH(return VK_OK, VK_RETURN_CODE)
}

}  // extern "C"
