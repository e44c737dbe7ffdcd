// moe_align.cu - device alignment of the routing table for any N = M*top_k.
//
// Output contract (reference moe_fused.cpp:609-661 for the order and padding,
// moe_fused.hip:1983-2099 for expert_map / local_n / max_EM / out_em): flat
// indices grouped by LOCAL expert in ascending order, ascending flat index
// inside an expert (a stable counting sort), each expert padded to block_size
// with the sentinel N, expert_ids = local expert per block and -1 beyond the
// last real block, every one of the max_EM entries written, *out_em = padded
// row count (block_size when nothing routes).
//
// Small N runs in one CTA (histogram, scan and scatter in shared memory).
// Large N runs three kernels over 1024-entry chunks: per-chunk histograms,
// a scan over (expert, chunk), and an ordered scatter; the chunk histograms
// live in the library workspace.
#include <atomic>

#include "common.cuh"
#include "moe_fused.hpp"
#include "moe_prep.cuh"

namespace vkernels::kernels::cuda {

namespace {

using namespace prep;

// ------------------------------ one CTA, N <= kChunk -------------------------
__global__ void __launch_bounds__(kChunk)
align_small_kernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map,
                   int N, int block_size, int num_experts, int local_n, int max_EM,
                   int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids,
                   int32_t* __restrict__ out_em) {
  extern __shared__ int smem[];
  int* warp_hist = smem;                               // [(kWarps+1) * local_n]
  int* offset = warp_hist + (kWarps + 1) * local_n;    // [local_n]
  int* s_tmp = offset + local_n;                       // [kChunk]
  const int tid = threadIdx.x;
  for (int i = tid; i < max_EM; i += kChunk) sorted_ids[i] = N;
  for (int i = tid; i < max_EM / block_size; i += kChunk) expert_ids[i] = -1;
  const int le = local_expert(topk_ids, expert_map, tid, N, num_experts, local_n);
  const int rank = chunk_rank(le, local_n, warp_hist);
  scan_experts(warp_hist + kWarps * local_n, offset, local_n, block_size, max_EM, expert_ids,
               out_em, s_tmp);
  if (le >= 0) {
    const int pos = offset[le] + rank;
    if (pos < max_EM) sorted_ids[pos] = tid;
  }
}

// ------------------------------ large N: three kernels -----------------------
// 1) per-chunk histogram -> hist[chunk][e]; also fills the sentinels.
__global__ void __launch_bounds__(kChunk)
align_hist_kernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map,
                  int N, int block_size, int num_experts, int local_n, int max_EM,
                  int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids,
                  int* __restrict__ hist) {
  extern __shared__ int smem[];
  int* warp_hist = smem;
  const int tid = threadIdx.x, chunk = blockIdx.x;
  for (int i = chunk * kChunk + tid; i < max_EM; i += gridDim.x * kChunk) sorted_ids[i] = N;
  for (int i = chunk * kChunk + tid; i < max_EM / block_size; i += gridDim.x * kChunk)
    expert_ids[i] = -1;
  const int le = local_expert(topk_ids, expert_map, chunk * kChunk + tid, N, num_experts, local_n);
  (void)chunk_rank(le, local_n, warp_hist);
  for (int e = tid; e < local_n; e += kChunk)
    hist[(size_t)chunk * local_n + e] = warp_hist[kWarps * local_n + e];
}

// 2) one CTA: hist[chunk][e] -> exclusive over chunks (in place), totals ->
//    expert offsets, expert_ids, out_em.
__global__ void __launch_bounds__(kChunk)
align_scan_kernel(int* __restrict__ hist, int n_chunks, int local_n, int block_size, int max_EM,
                  int32_t* __restrict__ expert_ids, int32_t* __restrict__ out_em,
                  int* __restrict__ offset /* [local_n] in workspace */) {
  extern __shared__ int smem[];
  int* count = smem;              // [local_n]
  int* s_tmp = count + local_n;   // [kChunk]
  const int tid = threadIdx.x;
  for (int e = tid; e < local_n; e += kChunk) {
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
      int v = hist[(size_t)c * local_n + e];
      hist[(size_t)c * local_n + e] = run;
      run += v;
    }
    count[e] = run;
  }
  __syncthreads();
  scan_experts(count, offset, local_n, block_size, max_EM, expert_ids, out_em, s_tmp);
}

// 3) ordered scatter: row = expert offset + entries in earlier chunks + rank in chunk.
__global__ void __launch_bounds__(kChunk)
align_scatter_kernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map,
                     int N, int num_experts, int local_n, int max_EM,
                     const int* __restrict__ hist, const int* __restrict__ offset,
                     int32_t* __restrict__ sorted_ids) {
  extern __shared__ int smem[];
  int* warp_hist = smem;
  const int tid = threadIdx.x, chunk = blockIdx.x;
  const int i = chunk * kChunk + tid;
  const int le = local_expert(topk_ids, expert_map, i, N, num_experts, local_n);
  const int rank = chunk_rank(le, local_n, warp_hist);
  if (le >= 0) {
    const int pos = offset[le] + hist[(size_t)chunk * local_n + le] + rank;
    if (pos < max_EM) sorted_ids[pos] = i;
  }
}

}  // namespace

void moe_align_block_size(const int32_t* topk_ids, const int32_t* expert_map, int M, int top_k,
                          int block_size, int num_experts, int local_n, int max_EM,
                          int32_t* sorted_ids, int32_t* expert_ids, int32_t* out_em,
                          void* stream) {
  expects(block_size > 0, "moe_align_block_size: block_size must be positive");
  expects(M >= 0 && top_k >= 0 && num_experts >= 0 && local_n >= 0,
          "moe_align_block_size: negative dimension");
  expects(max_EM > 0 && max_EM % block_size == 0,
          "moe_align_block_size: max_EM must be a positive multiple of block_size");
  expects(local_n <= num_experts, "moe_align_block_size: local_n exceeds num_experts");
  expects(out_em != nullptr && sorted_ids != nullptr && expert_ids != nullptr,
          "moe_align_block_size: output buffers must not be null");
  expects(M == 0 || topk_ids != nullptr, "moe_align_block_size: topk_ids must not be null");
  expects((long long)M * top_k < (1ll << 30), "moe_align_block_size: M*top_k too large");
  const int N = M * top_k;
  const int ln = local_n > 0 ? local_n : 1;  // shared-memory sizing only
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t hist_smem = (size_t)(kWarps + 1) * ln * sizeof(int);
  expects(hist_smem + (size_t)(ln + kChunk) * sizeof(int) <= 200 * 1024,
          "moe_align_block_size: too many local experts");
  if (N <= kChunk) {
    const size_t smem = hist_smem + (size_t)(ln + kChunk) * sizeof(int);
    if (smem > 48 * 1024)
      VK_CUDA_CHECK(cudaFuncSetAttribute(align_small_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    align_small_kernel<<<1, kChunk, smem, s>>>(topk_ids, expert_map, N, block_size, num_experts,
                                               local_n, max_EM, sorted_ids, expert_ids, out_em);
  } else {
    const int n_chunks = (N + kChunk - 1) / kChunk;
    // The histograms use this stream's workspace block behind its first 4 KB (the tile count of
    // the GEMM kernels); they are dead before the same stream builds the tile list.
    int* ws = reinterpret_cast<int*>(
        static_cast<uint8_t*>(workspace_get(4096 + ((size_t)n_chunks * ln + ln) * sizeof(int), s)) + 4096);
    int* hist = ws;
    int* offset = ws + (size_t)n_chunks * ln;
    if (hist_smem > 48 * 1024) {
      VK_CUDA_CHECK(cudaFuncSetAttribute(align_hist_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)hist_smem));
      VK_CUDA_CHECK(cudaFuncSetAttribute(align_scatter_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)hist_smem));
    }
    align_hist_kernel<<<n_chunks, kChunk, hist_smem, s>>>(topk_ids, expert_map, N, block_size,
                                                          num_experts, local_n, max_EM, sorted_ids,
                                                          expert_ids, hist);
    const size_t scan_smem = (size_t)(ln + kChunk) * sizeof(int);
    align_scan_kernel<<<1, kChunk, scan_smem, s>>>(hist, n_chunks, local_n, block_size, max_EM,
                                                   expert_ids, out_em, offset);
    align_scatter_kernel<<<n_chunks, kChunk, hist_smem, s>>>(topk_ids, expert_map, N, num_experts,
                                                             local_n, max_EM, hist, offset,
                                                             sorted_ids);
  }
  VK_CUDA_CHECK(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Alignment for callers that must not allocate
// ---------------------------------------------------------------------------
// Some callers of this library cannot tolerate a device allocation inside a
// call: an inference server that has handed all free memory to its own pool
// after warm-up (a later cudaMalloc can simply fail), a latency-critical step
// where cudaMalloc's implicit device-wide synchronisation would stall every
// stream, or code already inside a region where allocation is forbidden. The
// chunked alignment above takes its chunk histograms from the library
// workspace, which may have to grow. This variant keeps them in a fixed array
// that is part of the library image instead: every GPU that loads the library
// holds these ~514 KB until the process exits, and nothing is ever allocated.
//
// Limits (rejected with std::invalid_argument beyond them):
//   M * top_k <= kNoAllocMaxChunks * 1024 = 262144 routed slots
//   local_n   <= kNoAllocMaxLocal      = 512 local experts
//
// The array is shared by every call on a device and keeps the previous call's
// contents. The kernels overwrite each entry they later read (every chunk
// writes its full histogram row, the scan writes every offset), so nothing
// needs clearing between calls; two calls whose kernels overlap on the GPU
// (different streams, no ordering) would race on it - order them.
//
// The first call on each device looks the array's device address up (host code
// only sees a stand-in symbol, not an address); that first call should be made
// before any stream capture begins.
constexpr int kNoAllocMaxChunks = 256;
constexpr int kNoAllocMaxLocal = 512;
static __device__ __align__(256) int g_noalloc_align_scratch[kNoAllocMaxChunks * kNoAllocMaxLocal +
                                                             kNoAllocMaxLocal];

void moe_align_block_size_noalloc(const int32_t* topk_ids, const int32_t* expert_map, int M,
                                  int top_k, int block_size, int num_experts, int local_n,
                                  int max_EM, int32_t* sorted_ids, int32_t* expert_ids,
                                  int32_t* out_em, void* stream) {
  expects(block_size > 0, "moe_align_block_size_noalloc: block_size must be positive");
  expects(M >= 0 && top_k >= 0 && num_experts >= 0 && local_n >= 0,
          "moe_align_block_size_noalloc: negative dimension");
  expects(max_EM > 0 && max_EM % block_size == 0,
          "moe_align_block_size_noalloc: max_EM must be a positive multiple of block_size");
  expects(local_n <= num_experts, "moe_align_block_size_noalloc: local_n exceeds num_experts");
  expects(out_em != nullptr && sorted_ids != nullptr && expert_ids != nullptr,
          "moe_align_block_size_noalloc: output buffers must not be null");
  expects(M == 0 || topk_ids != nullptr, "moe_align_block_size_noalloc: topk_ids must not be null");
  expects((long long)M * top_k <= (long long)kNoAllocMaxChunks * kChunk,
          "moe_align_block_size_noalloc: M*top_k exceeds the fixed scratch (at most 262144 routed "
          "slots); use vk_hip_moe_align_block_size");
  expects(local_n <= kNoAllocMaxLocal,
          "moe_align_block_size_noalloc: local_n exceeds the fixed scratch (at most 512 local "
          "experts); use vk_hip_moe_align_block_size");
  const int N = M * top_k;
  const int ln = local_n > 0 ? local_n : 1;
  const int n_chunks = N > 0 ? (N + kChunk - 1) / kChunk : 1;

  // Device address of the array, looked up once per device with that device current.
  static std::atomic<int*> scratch_of_device[64];
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  expects(dev >= 0 && dev < 64, "moe_align_block_size_noalloc: device index out of range");
  int* hist = scratch_of_device[dev].load();
  if (hist == nullptr) {
    VK_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&hist), g_noalloc_align_scratch));
    scratch_of_device[dev].store(hist);   // two threads racing here store the same address
  }
  int* offset = hist + (size_t)n_chunks * ln;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t hist_smem = (size_t)(kWarps + 1) * ln * sizeof(int);
  if (hist_smem > 48 * 1024) {
    VK_CUDA_CHECK(cudaFuncSetAttribute(align_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)hist_smem));
    VK_CUDA_CHECK(cudaFuncSetAttribute(align_scatter_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_smem));
  }
  align_hist_kernel<<<n_chunks, kChunk, hist_smem, s>>>(topk_ids, expert_map, N, block_size,
                                                        num_experts, local_n, max_EM, sorted_ids,
                                                        expert_ids, hist);
  const size_t scan_smem = (size_t)(ln + kChunk) * sizeof(int);
  align_scan_kernel<<<1, kChunk, scan_smem, s>>>(hist, n_chunks, local_n, block_size, max_EM,
                                                 expert_ids, out_em, offset);
  align_scatter_kernel<<<n_chunks, kChunk, hist_smem, s>>>(topk_ids, expert_map, N, num_experts,
                                                           local_n, max_EM, hist, offset, sorted_ids);
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
