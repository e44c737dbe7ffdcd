// moe_fused.cu - host launchers: argument contract, workspace, dispatch.
#include "moe_fused.hpp"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace vkernels::kernels::cuda {

// defined in moe_simt.cu / moe_gemm_sm100.cu
void launch_moe_simt(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                     const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w, int w_sorted,
                     uint16_t* act_scratch, float* out, int M, int hidden, int ispp, int top_k,
                     const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                     float swiglu_limit, int activation, float beta, float linear_beta,
                     const float* b13, const float* b2, int block_size, cudaStream_t stream);
void launch_moe_sm100(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                      const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                      int w_sorted, uint16_t* act_scratch, float* out, int M, int hidden, int ispp,
                      int top_k, const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                      float swiglu_limit, int activation, float beta, float linear_beta,
                      const float* b13, const float* b2, int block_size, cudaStream_t stream,
                      const RowPtrs* rows, uint16_t* y_bf16, bool w4);
size_t sm100_workspace_bytes(int EM, int hidden, int ispp);
size_t sm100_workspace_bytes_ordered(int EM, int hidden, int ispp, int N);

// ---------------------------------------------------------------------------
// implementation switch
// ---------------------------------------------------------------------------
namespace {
std::atomic<int> g_impl{-1};
int impl_from_env() {
  const char* s = std::getenv("VK_MOE_IMPL");
  if (s != nullptr && std::strcmp(s, "simt") == 0) return (int)MoeImpl::kSimt;
  return (int)MoeImpl::kTcgen05;
}
}  // namespace

void set_moe_impl(MoeImpl impl) { g_impl.store((int)impl); }
MoeImpl get_moe_impl() {
  int v = g_impl.load();
  if (v < 0) {
    v = impl_from_env();
    g_impl.store(v);
  }
  return (MoeImpl)v;
}

// ---------------------------------------------------------------------------
// workspace: one block per (device, stream); see common.cuh for the rules
// ---------------------------------------------------------------------------
namespace {
constexpr int kMaxDevices = 64;
struct WsBlock {
  int dev;
  cudaStream_t stream;
  void* ptr;
  size_t bytes;
};
std::vector<WsBlock> g_ws_live;      // at most one per (device, stream)
std::vector<WsBlock> g_ws_retired;   // outgrown blocks, kept for work that may still use them
std::mutex g_ws_mutex;
std::atomic<int> g_sm_count[kMaxDevices];
}  // namespace

int sm_count() {
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  const bool known = dev >= 0 && dev < kMaxDevices;
  int v = known ? g_sm_count[dev].load() : 0;
  if (v == 0) {
    VK_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
    if (known) g_sm_count[dev].store(v);
  }
  return v;
}

void* workspace_get(size_t bytes, cudaStream_t stream) {
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  WsBlock* mine = nullptr;
  for (auto& b : g_ws_live)
    if (b.dev == dev && b.stream == stream) mine = &b;
  if (mine != nullptr && mine->bytes >= bytes) return mine->ptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  VK_CUDA_CHECK(cudaStreamIsCapturing(stream, &cap));
  expects(cap == cudaStreamCaptureStatusNone,
          "fused_moe_mxfp4: the workspace of this stream is too small and the stream is being "
          "captured; call vk_cuda_moe_reserve_workspace_on(bytes, stream) before the capture");
  const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  void* p = nullptr;
  VK_CUDA_CHECK(cudaMalloc(&p, want));
  if (mine != nullptr) {
    g_ws_retired.push_back(*mine);
    mine->ptr = p;
    mine->bytes = want;
  } else {
    g_ws_live.push_back(WsBlock{dev, stream, p, want});
  }
  return p;
}

void reserve_workspace(size_t bytes, void* stream) { (void)workspace_get(bytes, static_cast<cudaStream_t>(stream)); }

// Frees every block of the current device, live and retired. The caller guarantees that no work
// using them is pending and that no captured graph that points at them will be replayed.
void release_workspaces() {
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  for (auto* v : {&g_ws_live, &g_ws_retired}) {
    for (size_t i = 0; i < v->size();) {
      if ((*v)[i].dev == dev) {
        VK_CUDA_CHECK(cudaFree((*v)[i].ptr));
        v->erase(v->begin() + (long)i);
      } else {
        ++i;
      }
    }
  }
}

size_t workspace_live_bytes() {
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  size_t n = 0;
  for (auto* v : {&g_ws_live, &g_ws_retired})
    for (auto& b : *v)
      if (b.dev == dev) n += b.bytes;
  return n;
}

size_t workspace_bytes_required(int max_EM, int hidden, int ispp, int n_local_experts, int N) {
  const size_t align_bytes =
      ((size_t)((N + 1023) / 1024) + 1) * (size_t)(n_local_experts > 0 ? n_local_experts : 1) * 4;
  const size_t gemm_bytes = sm100_workspace_bytes(max_EM, hidden, ispp);
  return (align_bytes > gemm_bytes ? align_bytes : gemm_bytes) + 4096;
}

// ---------------------------------------------------------------------------
// fused layer
// ---------------------------------------------------------------------------
namespace {
void run_fused(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
               const uint8_t* w2_scale, const float* topk_w, int w_sorted, uint16_t* act_scratch,
               float* out, int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
               const int32_t* expert_ids, int EM, float swiglu_limit, int activation, float beta,
               float linear_beta, const float* b13, const float* b2, int block_size, bool kmajor,
               void* stream, const RowPtrs* rows = nullptr, uint16_t* y_bf16 = nullptr, bool w4 = false) {
  expects(!kmajor, "fused_moe_mxfp4: the K-major weight layout is not supported");
  expects(M >= 0 && EM >= 0 && top_k > 0, "fused_moe_mxfp4: bad M / EM / top_k");
  expects(hidden > 0 && hidden % 64 == 0, "fused_moe_mxfp4: hidden must be a multiple of 64");
  expects(ispp > 0 && ispp % 64 == 0, "fused_moe_mxfp4: ispp must be a multiple of 64");
  expects(block_size >= 16 && block_size % 16 == 0,
          "fused_moe_mxfp4: block_size must be a multiple of 16");
  expects(EM % block_size == 0, "fused_moe_mxfp4: EM must be a multiple of block_size");
  expects(activation == kSwiGLU || activation == kSiTU, "fused_moe_mxfp4: unknown activation");
  expects((long long)M * top_k < (1ll << 30), "fused_moe_mxfp4: M*top_k too large");
  if (M == 0 || EM == 0) return;
  expects(w13 && w13_scale && w2 && w2_scale && topk_w && act_scratch && sorted_ids && expert_ids,
          "fused_moe_mxfp4: buffers must not be null");
  if (rows != nullptr) {
    expects(rows->a_rows && rows->out_rows, "fused_moe_mxfp4_rows: row address arrays must not be null");
    expects(get_moe_impl() == MoeImpl::kTcgen05, "fused_moe_mxfp4_rows: only the tcgen05 path takes row addresses");
  } else {
    expects(A && (out || y_bf16), "fused_moe_mxfp4: buffers must not be null");
  }
  if (y_bf16 != nullptr) {
    expects(get_moe_impl() == MoeImpl::kTcgen05, "fused_moe_mxfp4_bf16: only the tcgen05 path has the ordered combine");
    expects(top_k <= 32 && hidden % 4 == 0, "fused_moe_mxfp4_bf16: at most 32 slots per token");
    expects((reinterpret_cast<uintptr_t>(y_bf16) & 7u) == 0, "fused_moe_mxfp4_bf16: y must be 8-byte aligned");
  }
  expects(!w4 || get_moe_impl() == MoeImpl::kTcgen05, "fused_moe_mxfp4_bf16_prepacked: only the tcgen05 path reads prepacked weights");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (get_moe_impl() == MoeImpl::kSimt)
    launch_moe_simt(A, w13, w13_scale, w2, w2_scale, topk_w, w_sorted, act_scratch, out, M, hidden,
                    ispp, top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation, beta,
                    linear_beta, b13, b2, block_size, s);
  else
    launch_moe_sm100(A, w13, w13_scale, w2, w2_scale, topk_w, w_sorted, act_scratch, out, M,
                     hidden, ispp, top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation,
                     beta, linear_beta, b13, b2, block_size, s, rows, y_bf16, w4);
}
}  // namespace

void fused_moe_mxfp4_rows(const uint16_t* const* a_rows, const uint8_t* w13, const uint8_t* w13_scale,
                          const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                          uint16_t* act_scratch, float* const* out_rows, int M, int hidden, int ispp,
                          int top_k, const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                          float swiglu_limit, int activation, float beta, float linear_beta,
                          const float* b13, const float* b2, int block_size, void* stream, bool store_slots) {
  const RowPtrs rows{a_rows, out_rows, store_slots};
  run_fused(nullptr, w13, w13_scale, w2, w2_scale, topk_w, 0, act_scratch, nullptr, M, hidden, ispp,
            top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13, b2,
            block_size, false, stream, &rows);
}

void fused_moe_mxfp4(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                     const uint8_t* w2, const uint8_t* w2_scale, const int32_t* /*topk_ids*/,
                     const float* topk_w, uint16_t* act_scratch, float* out, int M, int hidden,
                     int ispp, int top_k, const int32_t* sorted_ids, const int32_t* expert_ids,
                     int EM, float swiglu_limit, int activation, float beta, float linear_beta,
                     const float* b13, const float* b2, int block_size, bool kmajor,
                     void* stream) {
  run_fused(A, w13, w13_scale, w2, w2_scale, topk_w, 0, act_scratch, out, M, hidden, ispp, top_k,
            sorted_ids, expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13, b2,
            block_size, kmajor, stream);
}

void fused_moe_mxfp4_bf16(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                          const uint8_t* w2_scale, const float* topk_w, uint16_t* act_scratch, uint16_t* y_bf16,
                          int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                          const int32_t* expert_ids, int EM, float swiglu_limit, int activation, float beta,
                          float linear_beta, const float* b13, const float* b2, int block_size, void* stream) {
  expects(y_bf16 != nullptr || M == 0, "fused_moe_mxfp4_bf16: y must not be null");
  run_fused(A, w13, w13_scale, w2, w2_scale, topk_w, 0, act_scratch, nullptr, M, hidden, ispp, top_k, sorted_ids,
            expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13, b2, block_size, false, stream, nullptr,
            y_bf16);
}

void fused_moe_mxfp4_bf16_prepacked(const uint16_t* A, const uint8_t* w13_codes, const uint8_t* w13_sf,
                                    const uint8_t* w2_codes, const uint8_t* w2_sf, const float* topk_w,
                                    uint16_t* act_scratch, uint16_t* y_bf16, int M, int hidden, int ispp, int top_k,
                                    const int32_t* sorted_ids, const int32_t* expert_ids, int EM, float swiglu_limit,
                                    int activation, float beta, float linear_beta, const float* b13, const float* b2,
                                    int block_size, void* stream) {
  expects(y_bf16 != nullptr || M == 0, "fused_moe_mxfp4_bf16_prepacked: y must not be null");
  run_fused(A, w13_codes, w13_sf, w2_codes, w2_sf, topk_w, 0, act_scratch, nullptr, M, hidden, ispp, top_k, sorted_ids,
            expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13, b2, block_size, false, stream, nullptr,
            y_bf16, true);
}

size_t workspace_bytes_required_bf16(int max_EM, int hidden, int ispp, int n_local_experts, int N) {
  const size_t plain = workspace_bytes_required(max_EM, hidden, ispp, n_local_experts, N);
  const size_t ordered = sm100_workspace_bytes_ordered(max_EM, hidden, ispp, N) + 4096;
  return plain > ordered ? plain : ordered;
}

void fused_moe_mxfp4_sorted_w(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                              const uint8_t* w2, const uint8_t* w2_scale,
                              const float* topk_w_sorted, uint16_t* act_scratch, float* out,
                              int M, int hidden, int ispp, int top_k, const int32_t* sorted_ids,
                              const int32_t* expert_ids, int EM, float swiglu_limit,
                              int activation, float beta, float linear_beta, const float* b13,
                              const float* b2, int block_size, void* stream) {
  run_fused(A, w13, w13_scale, w2, w2_scale, topk_w_sorted, 1, act_scratch, out, M, hidden, ispp,
            top_k, sorted_ids, expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13,
            b2, block_size, false, stream);
}

}  // namespace vkernels::kernels::cuda
