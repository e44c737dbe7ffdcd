// moe_gemm_sm100.cu - the two grouped GEMMs of the fused MXFP4 MoE layer on
// tcgen05 tensor cores (sm_100a only).
//
// Orientation: the WEIGHTS are the M operand. One work item is 128 weight rows
// (gate/up GEMM: 64 gate rows + the 64 matching up rows; down GEMM: 128 rows)
// against up to 256 tokens of ONE expert (320 for a CTA pair, see below). A thread of a dequant warp owns one
// weight row = one TMEM lane: it reads the row's packed nibbles (K-contiguous,
// exactly the memory layout of the weights), expands them to bf16 with the
// exact table (common.cuh) and stores them with tcgen05.st as the A operand in
// tensor memory; the scale of a 32-element group is a per-thread scalar. The
// tokens are the N operand (any multiple of 16 up to 256), staged in shared
// memory by TMA with the 128-byte swizzle, so a ragged expert costs at most 15
// padded columns and a decode batch with a handful of tokens per expert still
// fills all 128 tensor-core rows. Accumulators D[weight row, token] stay in
// tensor memory (fp32) until the epilogue:
//   gate/up : bias, activation, ONE rounding to bf16, act[row, feature] store
//   down    : bias, routing weight, red.global.add.f32 into out[token, h]
//             (the weighted un-permute/combine, fused)
//
// Warp roles (640 threads, one persistent CTA per SM):
//   warp 0      TMA producer: packed weights (2 boxes of 64 rows x 128 B per
//               256-K stage) and scale bytes (bulk copy per item)
//   warp 1      tcgen05.mma issuer + tensor-memory allocation
//   warp 2      TMA producer: token tiles
//   warps 4-19  sixteen workers in sets of four (one warp per tensor-memory lane quarter):
//               dequant sets (shared memory -> registers -> tensor memory, a stage each in
//               turn) and epilogue sets (tensor memory -> registers -> global, a 32-token round
//               each in turn) - two + two for a CTA pair, three + one for a lone CTA
//
// Two forms, chosen by the largest token tile of the launch:
//   lone CTA (tiles up to 128 tokens, the decode regime): the stage length grows as the tile
//     shrinks (256 K-elements up to 64 tokens, 128 up to 128), because the issuer's per-stage
//     handshake costs a few hundred cycles whatever the stage holds;
//   CTA pair (larger tiles, the prefill regime): a cluster of two CTAs works on one item of
//     256 weight rows x up to 320 tokens with cta_group::2 MMAs. Each CTA dequantises its own
//     128 rows and stages HALF of the token rows, which halves the token bytes an SM pulls
//     from L2 per flop. Tensor memory: columns 0..255 main accumulator, 256..319 a second
//     accumulator for tokens 256..319 (fed by a second MMA per K block), 320..511 three A
//     slots of 128 K-elements. One ring serves A slots and token slots: the token bytes are
//     expected on the barrier the dequant warps arrive on.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises a flag all
// roles observe, the CTA frees its tensor memory and returns, and the launcher
// reports the failure through the device-side status word.
//
// Reference behaviour replaced: gateup_swiglu_kernel* and down_combine_kernel*
// (src/c/vkernels/kernels/moe_fused.hip:681-1436) and their launcher
// (moe_fused.hip:1448-1663).
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

#include <cuda_fp8.h>

#include "common.cuh"
#include "moe_fused.hpp"

namespace vkernels::kernels::cuda {

namespace {

// ---------------------------------------------------------------------------
// geometry
// ---------------------------------------------------------------------------
constexpr int kMaxTok = 256;        // tokens (MMA N) per work item of a lone CTA
// A CTA pair takes up to 320 tokens per item: a 256-column accumulator plus a 64-column one
// fed by a second MMA per K block. An expert whose token count is a little over 256 (the common
// case when tokens spread evenly) then costs one pass over its weights instead of two.
constexpr int kPairMainTok = 256;
constexpr int kPairMaxTok = 320;
constexpr int kRows = 128;          // weight rows (MMA M) per work item
constexpr int kWStageK = 256;       // K elements per packed-weight stage (128 B per row)
constexpr int kMaxWStages = 8;    // packed-weight ring depth is chosen per launch (3..8)
constexpr int kMaxAStages = 8;
constexpr int kMaxBStages = 8;
constexpr int kWStageBytes = kRows * 128;          // 16 KB
// 16 worker warps after the four control warps, split by form: a CTA pair (prefill) runs two
// dequant sets and two epilogue sets (the accumulator drains twice as fast, which is what its
// MMA issuer waits for); a lone CTA (decode) runs three dequant sets and one epilogue set (its
// epilogue is a few rounds, its bound is the expansion).
// (the prepacked-fp4 form expands nothing: one set of four warps only copies scale factors)
constexpr int dequant_sets(int ctas, bool = false, bool w4 = false) { return w4 ? 1 : (ctas == 2 ? 2 : 3); }   // dequant warps per TMEM lane quarter
constexpr int epi_sets(int ctas) { return ctas == 2 ? 2 : 1; }       // epilogue warps per lane quarter
constexpr int block_threads(int ctas, bool mx, bool w4 = false) { return (4 + 4 * (dequant_sets(ctas, mx, w4) + epi_sets(ctas))) * 32; }
// Prepacked-fp4 form: a weight stage in shared memory is 128 rows x 256 K as the copy engine
// unpacks them (16 nibbles in the low 8 bytes of every 16: 256 bytes a row, 128-K halves one
// after the other); the stage's scale factors [128 rows][8 groups] are read from global memory.
constexpr int kW4TileBytes = kRows * 128;                  // one 128-K half of a stage: 16 KB
constexpr int kW4SfBytes = kRows * 8;                      // 1 KB
constexpr int kW4StageBytes = 2 * kW4TileBytes;            // 32 KB
constexpr int kTmemCols = 512;
constexpr int kEpiPitch = 72;                     // bf16 per staged token row: 64 features + 16 bytes against bank conflicts
constexpr int kEpiStageBytes = 2 * 2 * 32 * kEpiPitch * 2;   // gate/up epilogue staging (two rounds per set, up to two sets)
constexpr int kEpiStageDownBytes = 4 * 32 * 32 * 4;   // down epilogue: one 32 x 32 fp32 block per warp
// what a launch really stages: a lone CTA runs one epilogue set, half of the above
constexpr int epi_stage_bytes(bool gateup, int ctas) { return (gateup ? kEpiStageBytes : kEpiStageDownBytes) / (ctas == 2 ? 1 : 2); }
// Lone-CTA form: byte -> bf16 pair lookup table in shared memory, one copy per bank (lane l reads
// word 32 * byte + l), so a warp's 32 lookups of different bytes are one conflict-free access.
constexpr int kLutBytes = 256 * 32 * 4;
constexpr long long kWaitLimitClocks = 4000000000ll;   // about two seconds of SM clock

// Device status word of the tensor-core kernels: 0, or 100 + the code of the wait that ran out.
// It lives in the library image (one per GPU that loads the library), so no launch needs a
// buffer for it and nothing but an expired wait writes it.
__device__ int g_kernel_status;

struct TokTile {
  int expert;
  int row0;
  int n_rows;  // multiple of 16, <= kMaxTok (kPairMaxTok for CTA pairs)
  int pad;
};

struct GemmParams {
  const float* tok_scale;     // fp8 form: power-of-two scale of every sorted token row [EM]
  const uint8_t* w_scale;     // [E, n_wrows, K/32]
  const float* bias;          // gate/up: [E, 2*n_feat]; down: [E, n_feat]; or null
  const float* topk_w;        // down only
  const int32_t* sorted_ids;  // [EM]
  uint16_t* act;              // gate/up output [EM, n_feat]
  float* out;                 // down output [M, n_feat]
  float* const* out_rows;     // optional: address of each token's output row (may be another GPU's memory)
  int store_rows;             // with out_rows: out_rows[m] is a [top_k, n_feat] block; slot j's row (act @ w2^T + b2,
                              // unweighted) is STORED at row j instead of being added, weighted, into one row
  float* raw;                 // optional: plain fp32 result rows [EM, raw_ld] instead of the fused epilogue
  int raw_ld;                 //   (the tensor-parallel stage split: the caller reduces across ranks first)
  int k_base;                 // first column of the token rows this launch reduces over (K-sharded weights)
  int piece_rows;             // fp8 form: rows between the two e4m3 pieces of the token operand
  const TokTile* tiles;
  const int* n_tiles;
  int K;                      // reduction length (hidden for gate/up, ispp for down)
  int n_feat;                 // gate/up: ispp; down: hidden
  int n_ftiles;
  int N;                      // M * top_k (sentinel of padded rows)
  int top_k;
  int w_sorted;
  int b_stages;
  int b_stage_bytes;          // max_tok * 128
  int w_stages;
  int max_tok;                // largest token tile of this launch (multiple of 16, <= 256)
  int scale_bufs;
  int scale_buf_bytes;
  int activation;
  float limit, beta, linear_beta;
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// The suspend-time hint keeps a waiting warp parked in hardware instead of spinning through
// the poll loop: a dozen waiting warps per CTA otherwise take issue slots and integer-pipe
// cycles from the dequant warps.
constexpr uint32_t kSuspendHintNs = 20000u;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the CTA is aborting (this wait or another
// role's ran out of iterations).
// `sleep_ns` > 0 is for waits that are long and off the critical path (an epilogue warp waiting
// for a whole item's MMAs, a producer waiting for a free slot of a deep ring): the warp sleeps
// between polls instead of spending issue slots that the dequant warps of the same scheduler need.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int code, unsigned sleep_ns = 0,
                                          long long limit_clocks = kWaitLimitClocks) {
  // try_wait suspends the thread for a hardware-chosen slice, so the limit is kept in clock
  // cycles rather than in poll iterations.
  long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (sleep_ns != 0) __nanosleep(sleep_ns);
    if ((it & 63u) == 63u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > limit_clocks) {
        *abort_flag = code;
        return false;
      }
    }
  }
}
// Whole-warp wait in which each ACTIVE lane polls its own barrier in the same
// instruction; returns once every active lane has seen its phase complete.
__device__ __forceinline__ bool mbar_wait_lanes(uint32_t bar, uint32_t parity, bool active,
                                                volatile int* abort_flag, int code) {
  bool done = !active;
  long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (!done) done = mbar_try_wait(bar, parity);
    if (__all_sync(0xFFFFFFFFu, done)) return true;
    if ((it & 63u) == 63u) {
      int stop = *abort_flag;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (!stop && now - t0 > kWaitLimitClocks) {
        *abort_flag = code;
        stop = 1;
      }
      if (__any_sync(0xFFFFFFFFu, stop != 0)) return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}
// Prefetch of a contiguous range into L2 (no shared-memory destination, no barrier).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]; kind::f16 with bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
      "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tc_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b),
               "r"(c), "r"(d)
               : "memory");
}
// D[tmem] (+)= (A[tmem] x 2^sfa) * (B[smem] x 2^sfb): e5m2 x e4m3 with one ue8m0 scale factor per
// 32 K-elements and row, both scale-factor operands in tensor memory; K = 32 per instruction.
__device__ __forceinline__ void tc_mma_mx(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], [%1], %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// The same with A read from shared memory through a descriptor (e2m1 weights as the copy engine unpacked them).
__device__ __forceinline__ void tc_mma_mx_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 32 columns: thread t gets, per group of 8 columns i, rows t / 4 (registers 4i, 4i+1)
// and t / 4 + 8 (registers 4i+2, 4i+3) at columns 8i + 2 * (t % 4) and the next one.
__device__ __forceinline__ void tc_ld_16x256b_x4(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// One lane of a fully converged warp, chosen by the hardware: code guarded by
// it is known to the compiler to run in a single thread, which lets it keep
// the MMA operands in uniform registers instead of serialising over lanes.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xFFFFFFFF;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// SwiGLU with the hardware exp / reciprocal approximations (relative error
// ~1e-6, far inside the layer's tolerance; the CUDA-core cross-check path keeps
// the accurate functions). Straight-line code - no data-dependent branch - so
// the 16 elements a thread finishes per round overlap their latencies. inf and
// NaN come out as in the CPU definition: NaN stays NaN (comparisons with NaN
// are false), +inf gives inf * u, and -inf, where the definition evaluates
// -inf / inf = NaN, is patched by the final select.
__device__ __forceinline__ float fmin_nan(float a, float b) {   // NaN if either operand is NaN
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float swiglu_fast(float g, float u, float limit) {
  if (limit > 0.0f) {   // uniform across the launch; a NaN operand stays NaN
    g = fmin_nan(g, limit);
    u = fmax_nan(fmin_nan(u, limit), -limit);
  }
  // exp(-g) overflows fp32 beyond 88; the quotient is below 1e-36 in magnitude either way.
  const float ng = fminf(-g, 87.0f);
  const float r = __fdividef(g, 1.0f + __expf(ng));
  return ((g == -INFINITY) ? __int_as_float(0x7FC00000) : r) * u;
}
// ---- CTA-pair (cta_group::2) helpers ---------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// out[0..3] += (a, b, c, d): one 16-byte reduction (address 16-byte aligned).
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
// The same reduction at system scope, for output rows that may live in another GPU's memory:
// several GPUs add into one row, and only system-scope atomics from different GPUs on one
// address are ordered with respect to each other by the memory model.
__device__ __forceinline__ void red_add_v4_sys(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
// Named barrier that also ORs a predicate over its participants.
__device__ __forceinline__ bool named_bar_or(int id, int n, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.b32 q, %1, 0;\n"
      "barrier.cta.red.or.pred p, %2, %3, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(id), "r"(n)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster.
// CTA-scope release (the default): the arrival only hands over tensor-memory contents, which
// the tcgen05 fences order; a cluster-scope release costs over a thousand cycles per arrival.
__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar, uint32_t cta) {
  asm volatile(
      "{\n"
      ".reg .b32 ra;\n"
      "mapa.shared::cluster.u32 ra, %0, %1;\n"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n"
      "}\n" ::"r"(bar),
      "r"(cta)
      : "memory");
}
// Token-tile load of a CTA pair: the data lands in THIS CTA's shared memory, the
// transaction bytes are credited to the barrier at the same offset in the pair's
// leader (even) CTA, whose MMA thread consumes both halves. No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar & 0xFEFFFFFFu)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
          "r"(bar),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int n) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are
// 128 bytes (64 bf16) with the 128-byte swizzle: groups of 8 rows are 1024
// bytes apart (stride byte offset), version 1, layout type 2.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version
  d |= (uint64_t)2 << 61;                        // 128-byte swizzle
  return d;
}
// Instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M = 128.
// Block-scaled instruction descriptor: A e5m2 (format 1, bits 7-9), B e4m3 (format 0), both
// K-major, N >> 3 at bit 17, ue8m0 scale factors (bit 23), M >> 4 at bit 24; the byte of the
// scale-factor column that holds this K block goes to bits 29-30 (A) and 4-5 (B) per instruction.
// (a_format 5 = e2m1, the prepacked-fp4 form)
__device__ __forceinline__ uint32_t make_idesc_mx(int n, uint32_t a_format = 1u) {
  return (a_format << 7) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ uint32_t make_idesc(int n, int m = 128) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// shared-memory carve-up
// ---------------------------------------------------------------------------
// Accumulator columns: a lone CTA sizes them by the stage length (long stages serve small token
// tiles), a pair always holds up to kPairMaxTok tokens.
constexpr int acc_cols(int ks, int ctas) { return ctas == 2 ? kPairMaxTok : (ks == 64 ? 256 : (ks == 128 ? 128 : 64)); }

struct Barriers {
  uint64_t w_full[kMaxWStages], w_empty[kMaxWStages];
  uint64_t a_full[kMaxAStages];    // dequant warps -> MMA issuer (4 arrivals, one per TMEM lane quarter)
  uint64_t stage_done[kMaxAStages];  // MMA completion of a stage: frees its A slot AND its token slot
  uint64_t b_full[kMaxBStages];
  uint64_t sc_full[2], sc_empty[2];
  uint64_t acc_full[2], acc_empty[2];   // the fp8 form alternates between two accumulators
  uint32_t tmem_base;
  int abort_flag;
  // per token column of the current item: gate/up 1 for a real row, 0 for padding;
  // down: address of the token's output row, 0 for padding
  unsigned long long tile_ref[kPairMaxTok];
  float tile_w[kPairMaxTok];
  float tile_s[kPairMaxTok];   // fp8 form: the token's power-of-two scale
};

// Ring position: slot index and phase parity, advanced without division.
struct Ring {
  int slot = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int depth) {
    if (++slot == depth) {
      slot = 0;
      phase ^= 1u;
    }
  }
};

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
// KS = K elements per pipeline stage (one A slot in tensor memory, one token
// slot in shared memory, one handshake of the MMA issuer). The issuer's
// per-stage latency (barrier polls + commit) is a few hundred cycles whatever
// the stage holds, so small token tiles, whose MMAs are short, take long
// stages: KS = 64 for tiles up to 256 tokens, 128 up to 128, 256 up to 64.
//
// MX (lone CTA, 256-K stages, tiles up to 64 tokens - the decode regime): the fp8 form. The
// weights are expanded to ONE byte each instead of two: every value of the layer's table
// {0, .25, 1, 1.5, 2, 3, inf, NaN} is exact in e5m2, and the ue8m0 scale of a 32-element group
// is not multiplied in at all - it goes to tensor memory as the per-row scale factor of a
// block-scaled MMA (kind::mxf8f6f4, one scale per 32 K-elements: exactly the MXFP4 grouping).
// That halves the expansion's instructions and its tensor-memory stores, which is what a decode
// batch is bound by. The token operand must then be fp8 too: a pre-pass splits every bf16
// activation x into two e4m3 pieces with x = s * (p1 + p2), s a power of two per token row
// (8 significant bits = 4 + 4; exact unless an element is more than 2^9 below the row's
// largest). An MMA with a handful of token columns costs as much as one with 128 (its cost is
// per instruction), so the two pieces are stacked along N - rows 0..n-1 of the staged tile are
// p1, rows n..2n-1 are p2 - and ONE MMA per K block yields both partial products in adjacent
// column ranges of the accumulator; the epilogue adds them and multiplies by s (unit token
// scale factors inside the MMA).
// MX = 0: bf16 forms; 32: the fp8 form, token tiles of up to 32 rows (an expert with more rows
// becomes several items). Its tensor memory: a 64-column accumulator (two pieces x 32 tokens),
// 4 columns of unit token scale factors, six A slots of 64 + 8 columns. Three dequant teams with
// six slots means every team owns two slots and alternates between them: the slot a team needs
// next was last used by its own stage before last, whose MMAs were issued a whole team period
// ago - a team never waits for a slot.
//
// W4 (with MX = 32): the prepacked-fp4 form. The weights were rewritten once, when the layer was
// built, into codes whose e2m1 reading by the tensor core is twice the layer's table value
// (0, .25, 1, 1.5, 2, 3 -> 0, .5, 2, 3, 4, 6; the epilogue halves the sums), so nothing is
// expanded at all: the copy engine unpacks the nibbles into the padded shared-memory form the
// MMA reads A from (one 5-D box per stage puts the rows into accumulator order), and the dequant
// warps shrink to one set that copies each stage's scale factors (prepacked as [stage][128
// rows][8]) from global memory into tensor memory. What a small-N MMA costs is its issuing
// thread (about a hundred cycles an instruction), so two warps issue, every other stage each,
// into two accumulators that the epilogue adds.
template <bool GATEUP, int KS, int CTAS, int MX = 0, bool W4 = false>
__global__ void __launch_bounds__(block_threads(CTAS, MX != 0, W4), 1)
moe_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_w,
                      const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_b64, const GemmParams p) {
  static_assert(MX == 0 || (MX == 32 && CTAS == 1 && KS == 256), "the fp8 form is a lone CTA with 256-K stages");
  static_assert(!W4 || MX == 32, "the prepacked-fp4 form is a variant of the fp8 form");
  constexpr int kThreads = block_threads(CTAS, MX != 0, W4);
  constexpr int kWBytes = W4 ? kW4StageBytes : kWStageBytes;         // one slot of the weight ring
  // accumulator columns; the fp8 form keeps the two token pieces side by side
  constexpr int kAccCols = MX ? 2 * MX : acc_cols(KS, CTAS);
  constexpr int kAccBufs = 1;
  // Prepacked-fp4 form: the issuing thread, not the tensor core, is what a small-N MMA costs
  // (about a hundred cycles an instruction whatever N is), so TWO warps issue, each every
  // other stage into its own accumulator; the epilogue adds the two.
  constexpr int kIssuers = W4 ? 2 : 1;
  constexpr int kSfbCol = kAccBufs * kAccCols * kIssuers;             // fp8 form: 4 columns of unit token scale factors
  constexpr int kSlot0 = MX ? kSfbCol + 8 : kAccCols;                 // first A slot
  constexpr int kACols = W4 ? 8 : (MX ? KS / 4 + 8 : KS / 2);         // columns of one A slot (fp8: 64 of values + 8 of scale factors; fp4: the scale factors only)
  constexpr int kSfCol = W4 ? 0 : KS / 4;                             // scale-factor columns inside an fp8 / fp4 slot
  constexpr int kAStages = W4 ? kMaxAStages : (kTmemCols - kSlot0) / kACols;   // lone CTA: 8, 6, 3 (fp8: 6); pair: 6, 3
  constexpr int kSubPerW = kWStageK / KS;                             // stages per packed-weight stage
  constexpr int kPieces = KS / 64;                                    // 64-K pieces of a stage
  static_assert(kAStages <= kMaxAStages, "A ring too deep for the barrier arrays");
  static_assert(CTAS == 1 || KS <= 128, "the CTA-pair form takes 64-K or 128-K stages");
  // CTAS == 2: two CTAs of a cluster work on one item - 256 weight rows (128 per CTA, each CTA
  // dequantises its own) against ONE token tile of up to 256 tokens, of which each CTA stages only
  // half. The leader (even) CTA issues cta_group::2 MMAs that read both halves; every CTA keeps
  // its 128 accumulator rows in its own tensor memory. This halves the token bytes a CTA pulls
  // from L2 per flop and doubles the depth of the token ring that fits in shared memory.
  // A pair keeps ONE ring: token slot i lives and dies with A slot i, and the token bytes are
  // expected on the same barrier the dequant warps arrive on, so the MMA issuer polls a single
  // barrier per stage.
  constexpr bool kMerged = CTAS == 2;
  constexpr int kMxSplit = 1;   // fp8 form: dequant warps per lane quarter sharing one stage
  constexpr int kDequantSets = dequant_sets(CTAS, MX != 0, W4), kEpiSets = epi_sets(CTAS);
  constexpr int kEpiWarp0 = 4 + 4 * kDequantSets;   // first epilogue warp
  static_assert((kEpiWarp0 + 4 * kEpiSets) * 32 == kThreads, "the role split must use every warp");
  const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* w_smem = smem;                                      // w_stages x 16 KB
  uint8_t* b_smem = w_smem + p.w_stages * kWBytes;             // b_stages x b_stage_bytes
  uint8_t* sc_smem = b_smem + p.b_stages * p.b_stage_bytes;    // scale_bufs x scale_buf_bytes
  Barriers* bars = reinterpret_cast<Barriers*>(sc_smem + p.scale_bufs * p.scale_buf_bytes);
  // gate/up epilogue staging: 2 x (32 tokens x 64 features) bf16, 16-byte aligned
  uint16_t* epi_stage = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(bars) + ((sizeof(Barriers) + 127) & ~size_t(127)));
  constexpr bool kUseLut = CTAS == 1 && !MX;
  uint32_t* lut = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(epi_stage) +
                                              epi_stage_bytes(GATEUP, CTAS));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &bars->abort_flag;

  if (kUseLut) fill_dequant_lut(lut, tid, kThreads);
  if (tid == 0) {
    for (int i = 0; i < kMaxWStages; ++i) {
      mbar_init(smem_u32(&bars->w_full[i]), 1);
      // fp8 form: only the owning team reads a stage; fp4 form: the stage's MMAs release it
      mbar_init(smem_u32(&bars->w_empty[i]), W4 ? 1 : (MX ? 4 * kMxSplit : 4 * kDequantSets));
    }
    for (int i = 0; i < kMaxAStages; ++i) {
      mbar_init(smem_u32(&bars->a_full[i]), kMerged ? 4 * CTAS + 1 : (MX ? 4 * kMxSplit : 4));
      mbar_init(smem_u32(&bars->stage_done[i]), 1);
    }
    for (int i = 0; i < kMaxBStages; ++i) mbar_init(smem_u32(&bars->b_full[i]), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->sc_full[i]), 1);
      mbar_init(smem_u32(&bars->sc_empty[i]), 4 * kDequantSets);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->acc_full[i]), (W4 && p.K > KS) ? 2 : 1);   // one commit per issuing warp that has a stage
      mbar_init(smem_u32(&bars->acc_empty[i]), 4 * kEpiSets * CTAS);
    }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&bars->tmem_base)),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&bars->tmem_base)),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int n_tok_tiles = *p.n_tiles;
  const int unit = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // CTA (pair) index
  const int n_units = CTAS == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int n_fgroups = (p.n_ftiles + CTAS - 1) / CTAS;   // feature tiles per token tile, in units of CTAS
  const int n_items = n_tok_tiles * n_fgroups;
  // feature tile of this CTA inside an item; with an odd tile count the last pair's second CTA idles
  auto item_f = [&](int item) { return (item % n_fgroups) * CTAS + (int)cta_rank; };
  const int n_kw = (p.K + kWStageK - 1) / kWStageK;   // packed-weight stages per item
  const int n_stages = (p.K + KS - 1) / KS;           // pipeline stages per item (last may be short)
  const int pitch = p.K / 32;                         // scale bytes per weight row
  const int n_wrows = GATEUP ? 2 * p.n_feat : p.n_feat;
  // one 64-K slice of a token stage (this CTA's rows; a pair's MMA N is the tile rounded up to 32)
  const int slice_bytes = CTAS == 2 ? (((p.max_tok + 31) >> 5) << 4) * 128 : p.max_tok * 128;

  if (warp == 0) {
    // ------------------- TMA producer: packed weights + scales ---------------
    // Runs ahead by the depth of its own ring, independent of the token stages,
    // so the weight stream (the HBM-bound part) is never held back by them.
    if (W4) {
      // Prepacked-fp4 form: ONE copy per stage - a 5-D box (K inside a 128-K half, 8 rows, 2 row
      // groups, 8 groups of 16 accumulator rows, 2 halves) lands the item's 128 rows x 256 K in
      // accumulator row order. Issuing a copy costs the issuing thread a hundred cycles or
      // more, which is why a stage is not split into several.
      if (lane == 0) {
        Ring w;
        bool ok = true;
        for (int item = unit; item < n_items && ok; item += n_units) {
          const TokTile tt = p.tiles[item / n_fgroups];
          const int f = item_f(item);
          const int g0 = GATEUP ? (tt.expert * n_wrows + f * 64) >> 3 : (tt.expert * n_wrows + f * 128) >> 4;
          for (int kw = 0; kw < n_kw; ++kw) {
            if (!mbar_wait(smem_u32(&bars->w_empty[w.slot]), w.phase ^ 1u, abort_flag, 2)) {
              ok = false;
              break;
            }
            const uint32_t bar = smem_u32(&bars->w_full[w.slot]);
            const uint32_t dst = smem_u32(w_smem + w.slot * kWBytes);
            if (p.K - kw * kWStageK > 128) {
              mbar_expect_tx(bar, kW4TileBytes);   // the copy counts packed bytes: half of what it writes
              tma_load_5d(dst, &tmap_w, 0, 0, 0, g0, 2 * kw, bar);
            } else {   // K ends inside the stage's first half: the 4-D map of single halves (in the tmap_b64 slot)
              mbar_expect_tx(bar, kW4TileBytes / 2);
              tma_load_4d(dst, &tmap_b64, kw * kWStageK, 0, 0, g0, bar);
            }
            w.advance(p.w_stages);
          }
        }
      }
    } else if (lane == 0) {
      Ring w;
      uint32_t sc_it = 0;
      bool ok = true;
      for (int item = unit; item < n_items && ok; item += n_units) {
        const TokTile tt = p.tiles[item / n_fgroups];
        const int f = item_f(item);
        int row_a, row_b, rows_valid;   // two boxes of 64 weight rows
        if (GATEUP) {
          row_a = tt.expert * n_wrows + f * 64;
          row_b = row_a + p.n_feat;
          rows_valid = 128;
        } else {
          row_a = tt.expert * n_wrows + f * 128;
          row_b = row_a + 64;
          rows_valid = min(128, p.n_feat - f * 128);
        }
        if (f >= p.n_ftiles) rows_valid = 0;   // idle half of the last pair: nothing to load
        {
          const int sb = sc_it % p.scale_bufs;
          const uint32_t par = ((sc_it / p.scale_bufs) & 1u) ^ 1u;
          if (!mbar_wait(smem_u32(&bars->sc_empty[sb]), par, abort_flag, 1, 128)) break;
          const uint32_t bar = smem_u32(&bars->sc_full[sb]);
          const uint32_t dst = smem_u32(sc_smem + sb * p.scale_buf_bytes);
          const uint32_t half = 64u * pitch;
          if (rows_valid == 0) {
            mbar_arrive(bar);
          } else {
            mbar_expect_tx(bar, rows_valid == 128 ? 2 * half : half);
            bulk_load_1d(dst, p.w_scale + (size_t)row_a * pitch, half, bar);
            if (rows_valid == 128)
              bulk_load_1d(dst + half, p.w_scale + (size_t)row_b * pitch, half, bar);
          }
          ++sc_it;
        }
        for (int kw = 0; kw < n_kw; ++kw) {
          if (!mbar_wait(smem_u32(&bars->w_empty[w.slot]), w.phase ^ 1u, abort_flag, 2, 128)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&bars->w_full[w.slot]);
          const uint32_t dst = smem_u32(w_smem + w.slot * kWStageBytes);
          if (rows_valid == 0) {
            mbar_arrive(bar);
          } else {
            mbar_expect_tx(bar, rows_valid == 128 ? kWStageBytes : kWStageBytes / 2);
            tma_load_2d(dst, &tmap_w, kw * (kWStageK / 2), row_a, bar);
            if (rows_valid == 128)
              tma_load_2d(dst + kWStageBytes / 2, &tmap_w, kw * (kWStageK / 2), row_b, bar);
          }
          w.advance(p.w_stages);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------- TMA producer: token tiles ---------------------------
    // Token slot of stage s is free once the MMAs of stage s - b_stages are done;
    // that event is stage_done of the A slot that stage used (b_stages <= kAStages,
    // so the barrier cannot have moved on to a later phase yet).
    if (kMerged) {
      if (lane == 0) {
        Ring a;
        bool ok = true;
        for (int item = unit; item < n_items && ok; item += n_units) {
          const TokTile tt = p.tiles[item / n_fgroups];
          // The tile, rounded up to 32 rows, is split into a main part (<= 256 rows, first MMA)
          // and an extension (<= 64 rows, second MMA); this CTA stages half of each. Rows past
          // the tile are someone else's (or zero fill past the tensor): their columns are never
          // read back.
          const int n32 = (tt.n_rows + 31) & ~31;
          const int h0 = min(n32, kPairMainTok) >> 1, h1 = (n32 >> 1) - h0;
          const int row_main = tt.row0 + (int)cta_rank * h0;
          const int row_ext = tt.row0 + 2 * h0 + (int)cta_rank * h1;
          for (int st = 0; st < n_stages; ++st) {
            if (!mbar_wait(smem_u32(&bars->stage_done[a.slot]), a.phase ^ 1u, abort_flag, 3, 64)) {
              ok = false;
              break;
            }
            const uint32_t bar = smem_u32(&bars->a_full[a.slot]);
            const uint32_t dst = smem_u32(b_smem + a.slot * p.b_stage_bytes);
            const int n_slices = min(kPieces, (p.K - st * KS) / 64);
            if (leader) mbar_expect_tx(bar, 2 * (h0 + h1) * 128 * n_slices);
            for (int sl = 0; sl < n_slices; ++sl) {
              const uint32_t d = dst + sl * slice_bytes;
              const int k0 = p.k_base + st * KS + sl * 64;
              int r = 0;
              for (; r + 64 <= h0; r += 64) tma_load_2d_pair(d + r * 128, &tmap_b64, k0, row_main + r, bar);
              for (; r < h0; r += 16) tma_load_2d_pair(d + r * 128, &tmap_b, k0, row_main + r, bar);
              for (r = 0; r < h1; r += 16) tma_load_2d_pair(d + (h0 + r) * 128, &tmap_b, k0, row_ext + r, bar);
            }
            a.advance(kAStages);
          }
        }
      }
    } else if (MX) {
      // fp8 tokens, staged as [128-K half][piece 1 rows, piece 2 rows][128 bytes]. A stage is
      // 4 to 8 small boxes (two pieces x two K halves x 16-row groups); one thread issuing them
      // one after the other is slower than the stage's MMAs, so the lanes of the warp issue
      // one box each. A half that sticks out past K is zero-filled by the copy and its bytes
      // still count.
      Ring b, lag;           // lag trails b by b_stages stages, on the A ring
      int issued = 0;        // stages issued so far (all items)
      bool ok = true;
      for (int item = unit; item < n_items && ok; item += n_units) {
        const TokTile tt = p.tiles[item / n_fgroups];
        const int n_r16 = tt.n_rows >> 4;
        for (int st = 0; st < n_stages; ++st, ++issued) {
          if (issued >= p.b_stages) {
            int w = 1;
            if (lane == 0) w = mbar_wait(smem_u32(&bars->stage_done[lag.slot]), lag.phase, abort_flag, 3, 64) ? 1 : 0;
            if (__shfl_sync(0xFFFFFFFFu, w, 0) == 0) {
              ok = false;
              break;
            }
            lag.advance(kAStages);
          }
          const uint32_t bar = smem_u32(&bars->b_full[b.slot]);
          const uint32_t dst = smem_u32(b_smem + b.slot * p.b_stage_bytes);
          const int k0 = st * KS;
          const int n_half = min(2, (p.K - k0 + 127) / 128);
          if (lane == 0) mbar_expect_tx(bar, tt.n_rows * 128 * n_half * 2);
          __syncwarp();
          const int per_piece = n_half * n_r16;
          if (lane < 2 * per_piece) {
            const int pc = lane / per_piece, rem = lane - pc * per_piece;
            const int kh = rem / n_r16, rc = rem - kh * n_r16;
            tma_load_2d(dst + kh * 2 * slice_bytes + (pc * tt.n_rows + rc * 16) * 128, &tmap_b, k0 + kh * 128,
                        pc * p.piece_rows + tt.row0 + rc * 16, bar);
          }
          b.advance(p.b_stages);
        }
      }
    } else if (lane == 0) {
      Ring b, lag;           // lag trails b by b_stages stages, on the A ring
      int issued = 0;        // stages issued so far (all items)
      bool ok = true;
      for (int item = unit; item < n_items && ok; item += n_units) {
        const TokTile tt = p.tiles[item / n_fgroups];
        for (int st = 0; st < n_stages; ++st, ++issued) {
          if (issued >= p.b_stages) {
            if (!mbar_wait(smem_u32(&bars->stage_done[lag.slot]), lag.phase, abort_flag, 3, 64)) {
              ok = false;
              break;
            }
            lag.advance(kAStages);
          }
          const uint32_t bar = smem_u32(&bars->b_full[b.slot]);
          const uint32_t dst = smem_u32(b_smem + b.slot * p.b_stage_bytes);
          const int k0 = st * KS;
          const int n_slices = min(kPieces, (p.K - k0) / 64);
          mbar_expect_tx(bar, tt.n_rows * 128 * n_slices);
          for (int sl = 0; sl < n_slices; ++sl) {
            int r = 0;
            for (; r + 64 <= tt.n_rows; r += 64)
              tma_load_2d(dst + sl * slice_bytes + r * 128, &tmap_b64, p.k_base + k0 + sl * 64, tt.row0 + r, bar);
            for (; r < tt.n_rows; r += 16)
              tma_load_2d(dst + sl * slice_bytes + r * 128, &tmap_b, p.k_base + k0 + sl * 64, tt.row0 + r, bar);
          }
          b.advance(p.b_stages);
        }
      }
    }
  } else if (warp == 1 || (W4 && warp == 3)) {
    // ------------------------------ MMA issuer -----------------------------
    const int iss = W4 && warp == 3 ? 1 : 0;   // prepacked-fp4 form: second issuing warp, odd stages
    // The whole warp stays converged: lanes 0 and 1 poll the A-ready and the
    // tokens-ready barrier of the stage in the SAME instruction (one poll latency
    // instead of two), lane 0 issues the MMAs and one commit per stage.
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t tmem_u = __shfl_sync(0xFFFFFFFFu, tmem_base, 0);
    if (kMerged) {
      // One thread's dependent instructions are the clock of this loop, so everything a stage
      // needs (barrier addresses, tensor-memory column, token descriptor) is carried along and
      // bumped per stage instead of being recomputed from the slot index.
      const uint32_t ready0 = smem_u32(&bars->a_full[0]), done0 = smem_u32(&bars->stage_done[0]);
      const uint32_t acc_full_bar = smem_u32(&bars->acc_full[0]);
      const uint32_t a0 = tmem_u + kAccCols;
      const uint64_t desc_first = make_b_desc(smem_u32(b_smem));
      const uint32_t desc_step = (uint32_t)p.b_stage_bytes >> 4, slice16 = (uint32_t)slice_bytes >> 4;
      uint32_t ready = ready0, done = done0, a_addr = a0, phase = 0;
      uint64_t desc = desc_first;
      int slot = 0;
      for (int item = unit; item < n_items && ok && leader; item += n_units) {
        const int n_rows_u = __shfl_sync(0xFFFFFFFFu, p.tiles[item / n_fgroups].n_rows, 0);
        const int n32 = (n_rows_u + 31) & ~31;
        const int n_main = min(n32, kPairMainTok), n_ext = n32 - n_main;
        const uint32_t idesc = make_idesc(n_main, 256), idesc_ext = make_idesc(n_ext, 256);
        const uint32_t ext16 = (uint32_t)(n_main >> 1) * 8u;   // descriptor offset of the extension rows
        if (!mbar_wait(smem_u32(&bars->acc_empty[0]), acc_phase ^ 1u, abort_flag, 4)) break;
        tc_fence_after();
        for (int st = 0; st < n_stages; ++st) {
          if (!mbar_wait(ready, phase, abort_flag, 5)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (elect_one()) {
            const int n_slices = min(kPieces, (p.K - st * KS) / 64);
#pragma unroll
            for (int sl = 0; sl < kPieces; ++sl) {
              if (sl < n_slices) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                  const uint32_t acc = (sl | kk) != 0 ? 1u : (st != 0 ? 1u : 0u);
                  tc_mma_ts_pair(tmem_u, a_addr + sl * 32 + kk * 8, desc + sl * slice16 + kk * 2, idesc, acc);
                  if (n_ext != 0)
                    tc_mma_ts_pair(tmem_u + kPairMainTok, a_addr + sl * 32 + kk * 8,
                                   desc + ext16 + sl * slice16 + kk * 2, idesc_ext, acc);
                }
              }
            }
            tc_commit_pair(done);   // completion is announced in both CTAs of the pair
            if (st == n_stages - 1) tc_commit_pair(acc_full_bar);
          }
          ready += 8;
          done += 8;
          a_addr += kACols;
          desc += desc_step;
          if (++slot == kAStages) {
            slot = 0;
            phase ^= 1u;
            ready = ready0;
            done = done0;
            a_addr = a0;
            desc = desc_first;
          }
        }
        acc_phase ^= 1u;
      }
    }
    Ring a, b, wr;   // wr: the weight ring, read by the MMAs of the prepacked-fp4 form only
    int acc_it = 0;
    for (int item = unit; item < n_items && ok && !kMerged; item += n_units, ++acc_it) {
      const int n_rows_u = __shfl_sync(0xFFFFFFFFu, p.tiles[item / n_fgroups].n_rows, 0);
      const uint32_t idesc = MX ? make_idesc_mx(2 * n_rows_u, W4 ? 5u : 1u) : make_idesc(n_rows_u);
      const int ab = acc_it % kAccBufs;
      const uint32_t d_addr = tmem_u + ab * kAccCols + iss * kAccCols;
      if (!mbar_wait(smem_u32(&bars->acc_empty[ab]), (((uint32_t)(acc_it / kAccBufs)) & 1u) ^ 1u, abort_flag, 4)) break;
      tc_fence_after();
      for (int st = 0; st < n_stages; ++st) {
        if (kIssuers == 2 && (st & 1) != iss) {   // the other warp's stage
          a.advance(kAStages);
          b.advance(p.b_stages);
          wr.advance(p.w_stages);
          continue;
        }
        const uint32_t first = st >= kIssuers ? 1u : 0u;   // 0 in this warp's first stage of the item
        const uint32_t bar = lane == 0 ? smem_u32(&bars->a_full[a.slot])
                                       : (lane == 1 ? smem_u32(&bars->b_full[b.slot]) : smem_u32(&bars->w_full[wr.slot]));
        const uint32_t par = lane == 0 ? a.phase : (lane == 1 ? b.phase : wr.phase);
        if (!mbar_wait_lanes(bar, par, lane < (W4 ? 3 : 2), abort_flag, 5)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_addr = tmem_u + kSlot0 + a.slot * kACols;
          const uint64_t desc0 = make_b_desc(smem_u32(b_smem + b.slot * p.b_stage_bytes));
          const uint32_t slice16 = (uint32_t)slice_bytes >> 4;
          if (MX) {
            // K blocks of 32: the block's 8 columns of e5m2 weights, its scale-factor byte (four
            // blocks share a group of four columns), and the block's 32 bytes of each token piece
            const int n_kb = min(8, (p.K - st * KS) / 32);
#pragma unroll
            for (int kb = 0; kb < 8; ++kb) {
              if (kb < n_kb) {
                const uint64_t bdesc = desc0 + (kb >> 2) * 2 * slice16 + (kb & 3) * 2;
                const uint32_t id = idesc | ((uint32_t)(kb & 3) << 29), sfa = a_addr + kSfCol + (kb >> 2) * 4;
                if (W4) {
                  // the block's 32 container bytes of every weight row in the stage's shared-memory tile
                  const uint64_t adesc = make_b_desc(smem_u32(w_smem + wr.slot * kWBytes)) +
                                         (uint64_t)((kb >> 2) * (kW4TileBytes >> 4) + (kb & 3) * 2);
                  tc_mma_mx_ss(d_addr, adesc, bdesc, id, sfa, tmem_u + kSfbCol, (first | kb) != 0 ? 1u : 0u);
                } else {
                  tc_mma_mx(d_addr, a_addr + kb * 8, bdesc, id, sfa, tmem_u + kSfbCol, (first | kb) != 0 ? 1u : 0u);
                }
              }
            }
          } else {
            const int n_slices = min(kPieces, (p.K - st * KS) / 64);
#pragma unroll
            for (int sl = 0; sl < kPieces; ++sl) {
              if (sl < n_slices) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                  tc_mma_ts(d_addr, a_addr + sl * 32 + kk * 8, desc0 + sl * slice16 + kk * 2, idesc,
                            (st | sl | kk) != 0 ? 1u : 0u);
              }
            }
          }
          tc_commit(smem_u32(&bars->stage_done[a.slot]));
          if (W4) tc_commit(smem_u32(&bars->w_empty[wr.slot]));   // the MMAs were the stage's last readers
          if (st + kIssuers >= n_stages) tc_commit(smem_u32(&bars->acc_full[ab]));   // this warp's last stage of the item
        }
        __syncwarp();
        a.advance(kAStages);
        b.advance(p.b_stages);
        if (W4) wr.advance(p.w_stages);
      }
    }
  } else if (warp >= 4 && warp < kEpiWarp0) {
    // ------------------------------ dequant --------------------------------
    // Warp (q, h): TMEM lane quarter q; set h takes every kDequantSets-th stage of the
    // running stage sequence. A stage is decoded 64 K-elements (32 columns) at a time:
    // two 16-byte chunks of the thread's row -> 32 registers -> one tcgen05.st.
    // With 64-K stages the store of a stage stays in flight while the warp's next
    // stage is decoded; longer stages overlap their own pieces instead.
    const int q = warp & 3, h = (warp - 4) >> 2;
    const int row = q * 32 + lane;                 // TMEM lane of this thread
    // gate/up items interleave the two halves in groups of 16 lanes: lanes 0-7 of a group hold
    // the gate rows of eight features, lanes 8-15 the matching up rows, so a 16x256b read of
    // the accumulator hands one thread the gate and the up value of the same (feature, token).
    const int srow = GATEUP ? (((row >> 3) & 1) * 64 + (row >> 4) * 8 + (row & 7)) : row;   // row inside the staged tile
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + kSlot0;
    if (MX && h == 0) {
      // unit scale factors of the token operand (the tokens carry their scale to the epilogue):
      // written once; the first stage's hand-over to the MMA issuer orders them before any MMA
      const uint32_t one = 0x7F7F7F7Fu;
      tc_st4(tmem_base + ((uint32_t)(q * 32) << 16) + kSfbCol, one, one, one, one);
    }
    const uint32_t lut_lane = smem_u32(lut) + (uint32_t)lane * 4u;
    Ring w, a;
    uint32_t sc_it = 0;
    int turn = 0;   // which dequant set takes the coming stage, running over all items
    int pending = -1;   // A slot whose stores are not yet handed to the MMA issuer
    bool ok = true;
    auto retire = [&]() {
      if (pending >= 0) {
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTAS == 2 && !leader) mbar_arrive_cta(smem_u32(&bars->a_full[pending]), 0);
          else mbar_arrive(smem_u32(&bars->a_full[pending]));
        }
        pending = -1;
      }
    };
    if (W4) {
      // Prepacked-fp4 form: nothing to expand. Per stage the four warps put the scale factors
      // (sanitised and laid out [stage][accumulator row][8 groups] by the prepack) into the
      // stage's scale-factor columns: column 4 h + i, byte b = tensor-memory row 32 i + lane,
      // group 4 h + b; every lane quarter keeps a full copy. They are read straight from global
      // memory into registers one stage ahead of their use, and one lane pulls them into L2
      // kW4Ahead stages ahead of that (a kilobyte a stage), so the register loads hit L2: a
      // load that went to HBM would take longer than a stage lasts and pace the whole pipeline.
      // (Pulling the WEIGHT stages into L2 ahead of the ring was measured too: a tensor-map
      // prefetch per stage changes nothing, one 128-byte bulk prefetch per row and stage from
      // these 128 threads doubles the kernel's time.)
      Ring sa;
      auto item_sf = [&](int item) {
        const TokTile tt = p.tiles[item / n_fgroups];
        return p.w_scale + ((size_t)tt.expert * p.n_ftiles + item_f(item)) * n_kw * kW4SfBytes;
      };
      // cursor of the L2 prefetch (first warp, lane 0) and of the register prefetch (everyone)
      int pf_item = unit, pf_kw = 0;
      const uint8_t* pf_sf = nullptr;
      constexpr int kW4Ahead = 6;
      auto prefetch_stage = [&]() {
        if (pf_item >= n_items) return;
        if (pf_kw == 0) pf_sf = item_sf(pf_item);
        bulk_prefetch_l2(pf_sf + (size_t)pf_kw * kW4SfBytes, kW4SfBytes);
        if (++pf_kw == n_kw) {
          pf_kw = 0;
          pf_item += n_units;
        }
      };
      const bool pf_lane = warp == 4 && lane == 0;
      if (pf_lane)
        for (int i = 0; i < kW4Ahead; ++i) prefetch_stage();
      int nx_item = unit, nx_kw = 0;
      const uint8_t* nx_sf = nx_item < n_items ? item_sf(nx_item) : nullptr;
      uint2 nxt[4];
      auto load_next = [&]() {
        if (nx_item >= n_items) return;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          nxt[i] = __ldg(reinterpret_cast<const uint2*>(nx_sf + (size_t)nx_kw * kW4SfBytes + (32 * i + lane) * 8));
        if (++nx_kw == n_kw) {
          nx_kw = 0;
          nx_item += n_units;
          if (nx_item < n_items) nx_sf = item_sf(nx_item);
        }
      };
      load_next();
      for (int item = unit; item < n_items && ok; item += n_units) {
        for (int kw = 0; kw < n_kw; ++kw) {
          uint32_t sf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            sf[i] = nxt[i].x;
            sf[4 + i] = nxt[i].y;
          }
          load_next();
          if (pf_lane) prefetch_stage();
          if (!mbar_wait(smem_u32(&bars->stage_done[sa.slot]), sa.phase ^ 1u, abort_flag, 9)) {
            ok = false;
            break;
          }
          tc_fence_after();
          tc_st8(t_row + sa.slot * kACols, sf);
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars->a_full[sa.slot]));
          sa.advance(kAStages);
        }
      }
    } else if (MX) {
      // fp8 form. A team (one warp per tensor-memory lane quarter) takes every kTeams-th stage of
      // this CTA's running stage sequence (items follow each other without a gap in it); a warp
      // expands its 32 rows of the stage in two halves of 128 K, each with the scale factors of
      // its four 32-element groups. A team never touches another team's stages: its ring
      // positions advance by kTeams and a packed-weight slot is released by its team alone.
      // (kMxSplit = 2 would let two warps of a quarter share a stage, one half each: measured, no
      // faster - the expansion is bound by the integer pipe of the scheduler both warps sit on.)
      constexpr int kSplit = kMxSplit;               // warps per lane quarter that share a stage (1 or 2)
      constexpr int kTeams = kDequantSets / kSplit;
      const int team = h / kSplit, half0 = h % kSplit;
      // staged-tile rows whose scale factors this thread copies (tensor-memory rows 32 i + lane)
      int sf_row[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int L = 32 * i + lane;
        sf_row[i] = GATEUP ? (((L >> 3) & 1) * 64 + (L >> 4) * 8 + (L & 7)) : L;
      }
      static_assert(kAStages >= kTeams, "one A slot per team at least");
      int w_slot = team % p.w_stages, a_slot = team;
      uint32_t w_phase = (uint32_t)(team / p.w_stages) & 1u, a_phase = 0;
      int g_base = 0;                        // running index of the item's first stage
      for (int item = unit; item < n_items && ok; item += n_units, g_base += n_kw) {
        const int f = item_f(item);
        const int rows_valid = f >= p.n_ftiles ? 0 : (GATEUP ? 128 : min(128, p.n_feat - f * 128));
        const int sbuf = sc_it % p.scale_bufs;
        if (!mbar_wait(smem_u32(&bars->sc_full[sbuf]), (sc_it / p.scale_bufs) & 1u, abort_flag, 7)) break;
        const uint8_t* sc_tile = sc_smem + sbuf * p.scale_buf_bytes;
        const uint8_t* sf_src[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) sf_src[i] = sf_row[i] < rows_valid ? sc_tile + sf_row[i] * pitch : nullptr;
        for (int kw = (team + kTeams - g_base % kTeams) % kTeams; kw < n_kw; kw += kTeams) {
          if (!mbar_wait(smem_u32(&bars->w_full[w_slot]), w_phase, abort_flag, 8) ||
              !mbar_wait(smem_u32(&bars->stage_done[a_slot]), a_phase ^ 1u, abort_flag, 9)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint8_t* my_row = w_smem + w_slot * kWStageBytes + (srow >> 6) * (kWStageBytes / 2) + (srow & 63) * 128;
          const int n_pieces = min(kPieces, (p.K - kw * kWStageK) / 64);   // 64-K pieces in this stage (4, or fewer at the end of K)
          const uint32_t slot_col = t_row + a_slot * kACols;
#pragma unroll
          for (int half = half0; half < 2; half += kSplit) {
            if (2 * half >= n_pieces) break;
            // Scale factors of my four 32-element groups: column 4 * half + i, byte b = scale of
            // tensor-memory row 32 i + lane for group 4 * half + b; every lane quarter keeps a
            // full copy. A scale byte of 0xFF means zero in this layer but NaN to the tensor
            // core: such a group is rewritten as scale 1 with zeroed values (NaN where the value
            // was inf or NaN, as inf * 0 is).
            uint32_t sf[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              sf[i] = 0x7F7F7F7Fu;
              if (sf_src[i] != nullptr) {
                const uint16_t* sp = reinterpret_cast<const uint16_t*>(sf_src[i] + kw * 8 + half * 4);
                sf[i] = (uint32_t)sp[0] | ((uint32_t)sp[1] << 16);
              }
            }
            const uint32_t mx4 = __vmaxu4(__vmaxu4(sf[0], sf[1]), __vmaxu4(sf[2], sf[3]));
            uint32_t ff = 0u;   // 0x80 in the byte of each of MY row's groups whose scale is 0xFF
            if ((((mx4 & 0x7F7F7F7Fu) + 0x01010101u) & mx4 & 0x80808080u) != 0u) {
              const uint32_t own = q == 0 ? sf[0] : q == 1 ? sf[1] : q == 2 ? sf[2] : sf[3];
              ff = ((own & 0x7F7F7F7Fu) + 0x01010101u) & own & 0x80808080u;
#pragma unroll
              for (int i = 0; i < 4; ++i) sf[i] ^= ((sf[i] & 0x7F7F7F7Fu) + 0x01010101u) & sf[i] & 0x80808080u;   // 0xFF -> 0x7F
            }
#pragma unroll
            for (int pp = 0; pp < 2; ++pp) {
              const int pc = 2 * half + pp;
              if (pc < n_pieces) {
                uint32_t v[16];
                if (srow < rows_valid) {
                  const uint4 p0 = *reinterpret_cast<const uint4*>(my_row + (((2 * pc) ^ (srow & 7)) << 4));
                  const uint4 p1 = *reinterpret_cast<const uint4*>(my_row + (((2 * pc + 1) ^ (srow & 7)) << 4));
                  expand8_e5m2(p0.x, v + 0);
                  expand8_e5m2(p0.y, v + 2);
                  expand8_e5m2(p0.z, v + 4);
                  expand8_e5m2(p0.w, v + 6);
                  expand8_e5m2(p1.x, v + 8);
                  expand8_e5m2(p1.y, v + 10);
                  expand8_e5m2(p1.z, v + 12);
                  expand8_e5m2(p1.w, v + 14);
                  if (ff != 0u) {
#pragma unroll
                    for (int g = 0; g < 2; ++g) {   // groups 2 pp + g of my four
                      if ((ff >> (8 * (2 * pp + g) + 7)) & 1u) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                          const uint32_t x = v[8 * g + i];
                          v[8 * g + i] = ((((x & 0x7C7C7C7Cu) + 0x04040404u) & 0x80808080u) >> 7) * 0x7Eu;
                        }
                      }
                    }
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 16; ++i) v[i] = 0u;
                }
                tc_st16(slot_col + pc * 16, v);
              }
            }
            tc_st4(slot_col + kSfCol + 4 * half, sf[0], sf[1], sf[2], sf[3]);
          }
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(smem_u32(&bars->a_full[a_slot]));
            mbar_arrive(smem_u32(&bars->w_empty[w_slot]));
          }
          w_slot += kTeams;
          while (w_slot >= p.w_stages) { w_slot -= p.w_stages; w_phase ^= 1u; }
          a_slot += kTeams;
          if (a_slot >= kAStages) { a_slot -= kAStages; a_phase ^= 1u; }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->sc_empty[sbuf]));
        ++sc_it;
      }
    }
    for (int item = unit; item < n_items && ok && !MX; item += n_units) {
      const int f = item_f(item);
      const int rows_valid = f >= p.n_ftiles ? 0 : (GATEUP ? 128 : min(128, p.n_feat - f * 128));
      const int sbuf = sc_it % p.scale_bufs;
      if (!mbar_wait(smem_u32(&bars->sc_full[sbuf]), (sc_it / p.scale_bufs) & 1u, abort_flag, 7)) {
        ok = false;
        break;
      }
      const uint8_t* my_scales = sc_smem + sbuf * p.scale_buf_bytes + srow * pitch;
      for (int kw = 0; kw < n_kw && ok; ++kw) {
        if (!mbar_wait(smem_u32(&bars->w_full[w.slot]), w.phase, abort_flag, 8)) {
          ok = false;
          break;
        }
        const uint8_t* my_row = w_smem + w.slot * kWStageBytes + (srow >> 6) * (kWStageBytes / 2) +
                                (srow & 63) * 128;
        const int k_left = p.K - kw * kWStageK;                       // K elements from this W stage on
        const int n_sub = min(kSubPerW, (k_left + KS - 1) / KS);      // pipeline stages in this W stage
        for (int j = 0; j < n_sub; ++j, turn = (turn + 1 == kDequantSets ? 0 : turn + 1), a.advance(kAStages)) {
          if (turn != h) continue;
          if (!mbar_wait(smem_u32(&bars->stage_done[a.slot]), a.phase ^ 1u, abort_flag, 9)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int n_pieces = min(kPieces, (k_left - j * KS) / 64);
#pragma unroll
          for (int pc = 0; pc < kPieces; ++pc) {
            if (pc < n_pieces) {
              uint32_t v[32];
              if (srow < rows_valid) {
                const int c0 = (j * kPieces + pc) * 2;   // two 16-byte chunks = two scale groups
                const uint4 p0 = *reinterpret_cast<const uint4*>(my_row + (((c0) ^ (srow & 7)) << 4));
                const uint4 p1 = *reinterpret_cast<const uint4*>(my_row + (((c0 + 1) ^ (srow & 7)) << 4));
                const uint32_t s0 = ue8m0_to_bf16x2(my_scales[kw * 8 + c0]);
                const uint32_t s1 = ue8m0_to_bf16x2(my_scales[kw * 8 + c0 + 1]);
                if (kUseLut) {
                  dequant64_lut(p0, p1, s0, s1, lut_lane, v);
                } else {
                  dequant8(p0.x, s0, v + 0);
                  dequant8(p0.y, s0, v + 4);
                  dequant8(p0.z, s0, v + 8);
                  dequant8(p0.w, s0, v + 12);
                  dequant8(p1.x, s1, v + 16);
                  dequant8(p1.y, s1, v + 20);
                  dequant8(p1.z, s1, v + 24);
                  dequant8(p1.w, s1, v + 28);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0u;
              }
              if (KS == 64) retire();   // previous stage of this warp: its store had a stage time to land
              tc_st32(t_row + a.slot * kACols + pc * 32, v);
            }
          }
          pending = a.slot;
          if (KS != 64) retire();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->w_empty[w.slot]));
        w.advance(p.w_stages);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->sc_empty[sbuf]));
      ++sc_it;
    }
    retire();
  } else if (warp >= kEpiWarp0) {
    // ------------------------------ epilogue -------------------------------
    // Two sets of four warps (one per lane quarter): the gate/up rounds of 32 tokens alternate
    // between them, and so do the rounds of the down epilogue, which halves the time the MMA
    // issuer waits for the accumulator.
    const int q = warp & 3;
    const int es = (warp - kEpiWarp0) >> 2;          // epilogue set
    const int etid = tid - kEpiWarp0 * 32;           // 0 .. 128 * kEpiSets - 1
    const int ltid = etid & 127;                     // thread inside the set = TMEM lane
    int acc_it = 0;
    int round = 0;   // gate/up staging buffer parity of this set, running over all items
    for (int item = unit; item < n_items; item += n_units, ++acc_it) {
      const int ab = acc_it % kAccBufs;
      const uint32_t acc_phase = ((uint32_t)(acc_it / kAccBufs)) & 1u;
      const TokTile tt = p.tiles[item / n_fgroups];
      const int f = item_f(item);
      // per-token info of this item (previous item's readers are past the barrier below)
      named_bar_sync(1, 128 * kEpiSets);
      for (int j = etid; j < tt.n_rows; j += 128 * kEpiSets) {
        const int flat = p.sorted_ids[tt.row0 + j];
        const bool real = flat >= 0 && flat < p.N;
        if (GATEUP) {
          bars->tile_ref[j] = real ? 1ull : 0ull;
        } else {
          const int token = real ? flat / p.top_k : 0;
          float* orow = p.out_rows ? p.out_rows[token] : p.out + (size_t)token * p.n_feat;
          if (p.store_rows && real) orow += (size_t)(flat - token * p.top_k) * p.n_feat;
          bars->tile_ref[j] = real ? reinterpret_cast<unsigned long long>(orow) : 0ull;
        }
        if (!GATEUP) bars->tile_w[j] = (real && p.topk_w != nullptr) ? p.topk_w[p.w_sorted ? tt.row0 + j : flat] : 0.0f;
        // (prepacked fp4: the codes read as twice the table value)
        if (MX) bars->tile_s[j] = real ? p.tok_scale[tt.row0 + j] * (W4 ? 0.5f : 1.0f) : 0.0f;
      }
      // The wait's outcome is shared by all epilogue warps before anyone acts on it: a warp that
      // gave up must not leave the others standing at a later named barrier.
      const bool gave_up = !mbar_wait(smem_u32(&bars->acc_full[ab]), acc_phase, abort_flag, 10, 256);
      if (named_bar_or(1, 128 * kEpiSets, gave_up)) break;
      tc_fence_after();
      const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16) + ab * kAccCols;
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTAS == 2 && !leader) mbar_arrive_cta(smem_u32(&bars->acc_empty[ab]), 0);
          else mbar_arrive(smem_u32(&bars->acc_empty[ab]));
        }
      };
      if (f >= p.n_ftiles || es * 32 >= tt.n_rows || (!GATEUP && (p.n_feat & 3) != 0 && es != 0)) {
        release_acc();   // idle half of the last pair, or a set with no round in this item
        continue;
      }
      if (GATEUP) {
        // Per 32 token columns the warp reads its two 16-lane groups in the 16x256b shape:
        // a thread then holds gate and up of (feature lane / 4 [+ 8], tokens 8i + 2 * (lane % 4)
        // and the next one), so the activation needs no exchange between lanes.
        const bool situ = p.activation == 1;   // uniform across the launch
        const int fl = q * 16 + (lane >> 2);   // feature inside the item's 64, first lane group
        const int tk = (lane & 3) * 2;
        float bg[2] = {0.f, 0.f}, bu[2] = {0.f, 0.f};
        if (p.bias) {
          const float* bp = p.bias + (size_t)tt.expert * 2 * p.n_feat + f * 64 + fl;
          bg[0] = bp[0]; bg[1] = bp[8]; bu[0] = bp[p.n_feat]; bu[1] = bp[p.n_feat + 8];
        }
        uint16_t* const my_stage = epi_stage + es * (2 * 32 * kEpiPitch);
        for (int c0 = es * 32; c0 < tt.n_rows; c0 += 32 * kEpiSets, ++round) {
          uint32_t va[16], vb[16];
          tc_ld_16x256b_x4(t_lane + c0, va);
          tc_ld_16x256b_x4(t_lane + (16u << 16) + c0, vb);
          if (MX) {   // the second piece's partial products sit n_rows columns further on
            // (fp4 form: and the second issuing warp's accumulator kAccCols further on, if K gave it a stage)
#pragma unroll
            for (int extra = 1; extra < 2 * kIssuers; ++extra) {
              if (extra >= 2 && p.K <= KS) break;
              const uint32_t off = (uint32_t)((extra & 1) * tt.n_rows + (extra >> 1) * kAccCols);
              uint32_t wa[16], wb[16];
              tc_ld_16x256b_x4(t_lane + off + c0, wa);
              tc_ld_16x256b_x4(t_lane + (16u << 16) + off + c0, wb);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                va[i] = __float_as_uint(__uint_as_float(va[i]) + __uint_as_float(wa[i]));
                vb[i] = __float_as_uint(__uint_as_float(vb[i]) + __uint_as_float(wb[i]));
              }
            }
          }
          tc_wait_ld();
          if (c0 + 32 * kEpiSets >= tt.n_rows) release_acc();   // this warp's last read of the accumulator
          if (p.raw != nullptr) {   // stage split: pre-activation sums, gate columns then up columns
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int t = c0 + 8 * i + tk + e;
                if (t < tt.n_rows) {
                  float* d = p.raw + (size_t)(tt.row0 + t) * p.raw_ld + f * 64 + fl;
                  d[0] = __uint_as_float(va[4 * i + e]);
                  d[p.n_feat] = __uint_as_float(va[4 * i + 2 + e]);
                  d[8] = __uint_as_float(vb[4 * i + e]);
                  d[p.n_feat + 8] = __uint_as_float(vb[4 * i + 2 + e]);
                }
              }
            }
            continue;
          }
          // which of the round's 32 tokens are real rows: one shared-memory read per lane and
          // a ballot, so the stores below depend on no load
          const int my_t = c0 + lane;
          const unsigned real = __ballot_sync(0xFFFFFFFFu, my_t < tt.n_rows && bars->tile_ref[my_t] != 0ull);
          // activation -> bf16 into the staging tile [token][feature] of this round ...
          uint16_t* stg = my_stage + (round & 1) * (32 * kEpiPitch) + tk * kEpiPitch + fl;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              // fp8 form: the sums are in units of the token's scale (a power of two: exact)
              const float ts = MX ? bars->tile_s[c0 + 8 * i + tk + e] : 1.0f;
              const float g0 = __uint_as_float(va[4 * i + e]) * ts + bg[0], u0 = __uint_as_float(va[4 * i + 2 + e]) * ts + bu[0];
              const float g1 = __uint_as_float(vb[4 * i + e]) * ts + bg[1], u1 = __uint_as_float(vb[4 * i + 2 + e]) * ts + bu[1];
              uint16_t* d = stg + (8 * i + e) * kEpiPitch;
              if (!situ) {
                d[0] = f32_to_bf16_bits(swiglu_fast(g0, u0, p.limit));
                d[8] = f32_to_bf16_bits(swiglu_fast(g1, u1, p.limit));
              } else {
                d[0] = f32_to_bf16_bits(moe_act_value(1, g0, u0, p.limit, p.beta, p.linear_beta));
                d[8] = f32_to_bf16_bits(moe_act_value(1, g1, u1, p.limit, p.beta, p.linear_beta));
              }
            }
          }
          // ... then rows leave as 16-byte pieces: 8 consecutive threads write one 128-byte act row.
          // One barrier per round: a buffer is rewritten two rounds later, after the barrier of
          // the round in between, which every reader of this round has passed by then.
          named_bar_sync(2 + es, 128);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int piece = ltid + i * 128;           // 256 pieces of 16 bytes
            const int tok = piece >> 3, ch = piece & 7;
            if ((real >> tok) & 1u) {
              const uint4 val = *reinterpret_cast<const uint4*>(my_stage + (round & 1) * (32 * kEpiPitch) + tok * kEpiPitch + ch * 8);
              *reinterpret_cast<uint4*>(p.act + (size_t)(tt.row0 + c0 + tok) * p.n_feat + f * 64 + ch * 8) = val;
            }
          }
        }
      } else {
        const int rows_valid = min(128, p.n_feat - f * 128);
        if ((p.n_feat & 3) == 0) {
          // 16-byte reductions: the warp turns its 32 rows x 32 tokens block around through
          // shared memory, so a lane holds four consecutive output features of one token and
          // adds them with one red.v4 (a quarter of the reduction instructions, which are what
          // this epilogue is bound by). Lane l: features 4 * (l % 8).., tokens l / 8 + 4 * i.
          // The two warp sets take the 32-token rounds in turn; a warp's block is 16 tokens wide,
          // so a round goes through it in two halves.
          float* stage = reinterpret_cast<float*>(epi_stage) + (es * 4 + q) * (16 * 32);
          const int hq = (lane & 7) * 4;                 // feature quad inside the warp's 32 rows
          const int h0 = f * 128 + q * 32 + hq;
          const bool quad_ok = q * 32 + hq < rows_valid;
          float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.bias && quad_ok) b4 = *reinterpret_cast<const float4*>(p.bias + (size_t)tt.expert * p.n_feat + h0);
          for (int c0 = es * 32; c0 < tt.n_rows; c0 += 32 * kEpiSets) {
            uint32_t v[32];
            tc_ld32(t_lane + c0, v);
            if (MX) {   // the second piece's partial products sit n_rows columns further on
#pragma unroll
              for (int extra = 1; extra < 2 * kIssuers; ++extra) {
                if (extra >= 2 && p.K <= KS) break;
                uint32_t v2[32];
                tc_ld32(t_lane + (uint32_t)((extra & 1) * tt.n_rows + (extra >> 1) * kAccCols) + c0, v2);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(v2[i]));
              }
            }
            tc_wait_ld();
            if (c0 + 32 * kEpiSets >= tt.n_rows) release_acc();   // this warp's last read of the accumulator
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              __syncwarp();   // the previous block has been read
#pragma unroll
              for (int j = 0; j < 16; ++j) stage[j * 32 + lane] = __uint_as_float(v[half * 16 + j]);
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int tl = (lane >> 3) + 4 * i;
                const int t = c0 + half * 16 + tl;
                if (p.raw != nullptr) {   // plain partial rows, no bias, no routing weight
                  if (t < tt.n_rows && quad_ok) {
                    float4 a = *reinterpret_cast<const float4*>(stage + tl * 32 + hq);
                    if (MX) {
                      const float ts = bars->tile_s[t];
                      a.x *= ts; a.y *= ts; a.z *= ts; a.w *= ts;
                    }
                    *reinterpret_cast<float4*>(p.raw + (size_t)(tt.row0 + t) * p.raw_ld + h0) = a;
                  }
                  continue;
                }
                float* orow = t < tt.n_rows ? reinterpret_cast<float*>(bars->tile_ref[t]) : nullptr;
                if (orow != nullptr && quad_ok) {
                  const float wgt = bars->tile_w[t];
                  float4 a = *reinterpret_cast<const float4*>(stage + tl * 32 + hq);
                  if (MX) {
                    const float ts = bars->tile_s[t];
                    a.x *= ts; a.y *= ts; a.z *= ts; a.w *= ts;
                  }
                  if (p.store_rows)   // plain 16-byte store of the slot's row; the home rank adds its slots in order
                    *reinterpret_cast<float4*>(orow + h0) = make_float4(a.x + b4.x, a.y + b4.y, a.z + b4.z, a.w + b4.w);
                  else if (p.out_rows != nullptr)
                    red_add_v4_sys(orow + h0, (a.x + b4.x) * wgt, (a.y + b4.y) * wgt,
                                   (a.z + b4.z) * wgt, (a.w + b4.w) * wgt);
                  else
                    red_add_v4(orow + h0, (a.x + b4.x) * wgt, (a.y + b4.y) * wgt,
                               (a.z + b4.z) * wgt, (a.w + b4.w) * wgt);
                }
              }
            }
          }
        } else {
          const int hcol = f * 128 + etid;
          const bool row_ok = etid < rows_valid;
          const float b = (p.bias && row_ok) ? p.bias[(size_t)tt.expert * p.n_feat + hcol] : 0.0f;
          for (int c0 = 0; c0 < tt.n_rows; c0 += 32) {
            uint32_t v[32];
            tc_ld32(t_lane + c0, v);
            if (MX) {
#pragma unroll
              for (int extra = 1; extra < 2 * kIssuers; ++extra) {
                if (extra >= 2 && p.K <= KS) break;
                uint32_t v2[32];
                tc_ld32(t_lane + (uint32_t)((extra & 1) * tt.n_rows + (extra >> 1) * kAccCols) + c0, v2);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(v2[i]));
              }
            }
            tc_wait_ld();
            if (c0 + 32 >= tt.n_rows) release_acc();
#pragma unroll 4
            for (int j = 0; j < 32; ++j) {
              const int t = c0 + j;
              float* orow = t < tt.n_rows ? reinterpret_cast<float*>(bars->tile_ref[t]) : nullptr;
              if (orow != nullptr && row_ok)
                atomicAdd(orow + hcol, (__uint_as_float(v[j]) * (MX ? bars->tile_s[t] : 1.0f) + b) * bars->tile_w[t]);
            }
          }
        }
      }
    }
  }

  // ------------------------------ teardown ---------------------------------
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();   // the peer no longer touches this CTA's barriers or tensor memory
  if (warp == 1) {
    tc_fence_after();
    if (CTAS == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((uint32_t)kTmemCols)
                   : "memory");
  }
  if (tid == 0 && bars->abort_flag != 0) atomicExch(&g_kernel_status, 100 + bars->abort_flag);
}

// One warp waits, with the kernels' own bounded wait, on a barrier nobody arrives on, and
// reports the expiry through the status word like a GEMM kernel would: the way to exercise the
// give-up path without starving a real launch.
__global__ void wait_timeout_probe_kernel(long long limit_clocks) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, 99, 0, limit_clocks);
    if (!ok) atomicExch(&g_kernel_status, 100 + abort_flag);
  }
}

// ---------------------------------------------------------------------------
// pre-pass kernels
// ---------------------------------------------------------------------------

// Token tiles from expert_ids: a run of consecutive blocks with the same
// non-negative expert becomes ceil(rows / max_tok) tiles of (almost) equal
// size, each a multiple of 16 rows.
template <int NT>
__device__ __forceinline__ void build_tiles_block(const int32_t* __restrict__ expert_ids, int n_blocks, int block_size,
                                                  int max_tok, TokTile* __restrict__ tiles, int* __restrict__ n_tiles,
                                                  int max_tiles, int* scan /* [NT] shared */, int* base /* shared */) {
  const int tid = threadIdx.x;
  if (tid == 0) *base = 0;
  __syncthreads();
  for (int b0 = 0; b0 < n_blocks; b0 += NT) {
    const int b = b0 + tid;
    int e = -1, run_blocks = 0;
    if (b < n_blocks) {
      e = expert_ids[b];
      const bool start = e >= 0 && (b == 0 || expert_ids[b - 1] != e);
      if (start) {
        run_blocks = 1;
        while (b + run_blocks < n_blocks && expert_ids[b + run_blocks] == e) ++run_blocks;
      }
    }
    const int rows = run_blocks * block_size;
    const int nt = (rows + max_tok - 1) / max_tok;
    scan[tid] = nt;
    __syncthreads();
    for (int d = 1; d < NT; d <<= 1) {
      const int v = tid >= d ? scan[tid - d] : 0;
      __syncthreads();
      scan[tid] += v;
      __syncthreads();
    }
    if (nt > 0) {
      int at = *base + scan[tid] - nt;
      // equal split, rounded up to 16 rows
      const int per = (((rows + nt - 1) / nt) + 15) & ~15;
      int r = 0;
      for (int i = 0; i < nt; ++i, ++at) {
        const int n = min(per, rows - r);
        if (at < max_tiles && n > 0) tiles[at] = TokTile{e, b * block_size + r, n, 0};
        r += n;
      }
    }
    __syncthreads();
    if (tid == 0) *base += scan[NT - 1];
    __syncthreads();
  }
  if (tid == 0) *n_tiles = min(*base, max_tiles);
}

__global__ void __launch_bounds__(1024)
build_tiles_kernel(const int32_t* __restrict__ expert_ids, int n_blocks, int block_size, int max_tok,
                   TokTile* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles) {
  __shared__ int scan[1024];
  __shared__ int base;
  build_tiles_block<1024>(expert_ids, n_blocks, block_size, max_tok, tiles, n_tiles, max_tiles, scan, &base);
}

// A_sorted[r, :] = A[sorted_ids[r] / top_k, :] (or the row at A_rows[sorted_ids[r] / top_k]) for
// real rows, zeros otherwise: four rows per CTA, 256 threads each. The CTA after the last row
// CTA builds the token-tile list instead (tiles != nullptr), so that the list costs no launch
// of its own and is ready when the rows are.
__global__ void __launch_bounds__(1024)
gather_rows_kernel(const uint16_t* __restrict__ A, const uint16_t* const* __restrict__ A_rows,
                   const int32_t* __restrict__ sorted_ids,
                   const int32_t* __restrict__ expert_ids, int block_size, int EM, int N, int top_k,
                   int H, uint16_t* __restrict__ dst, int32_t* __restrict__ inv, int max_tok,
                   TokTile* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles) {
  if ((int)blockIdx.x * 4 >= EM) {   // the extra CTA
    __shared__ int scan[1024];
    __shared__ int base;
    if (tiles != nullptr)
      build_tiles_block<1024>(expert_ids, EM / block_size, block_size, max_tok, tiles, n_tiles, max_tiles, scan, &base);
    return;
  }
  const int vec_per_row = H / 8;  // 16-byte vectors
  const int r = blockIdx.x * 4 + (threadIdx.x >> 8), t = threadIdx.x & 255;
  if (r >= EM) return;
  if (expert_ids[r / block_size] < 0) return;  // never read by any tile
  const int flat = sorted_ids[r];
  const bool real = flat >= 0 && flat < N;
  const int token = real ? flat / top_k : 0;
  if (real && inv != nullptr && t == 0) inv[flat] = r;
  // a row address from A_rows may lie in another GPU's memory (peer load over NVLink)
  const uint4* src = reinterpret_cast<const uint4*>(
      A_rows != nullptr ? (real ? A_rows[token] : nullptr) : A + (size_t)token * H);
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)r * H);
  for (int i = t; i < vec_per_row; i += 256)
    d[i] = real ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

// Token rows of the fp8 form. Row r of the sorted order (gate/up: the activation row of token
// sorted_ids[r] / top_k, or the row at src_rows[token]; down: row r of `src` itself) becomes two
// e4m3 pieces and a scale: x = s * (p1 + p2), s = 2^(floor(log2 max|x|) - 7), p1 = e4m3(x / s)
// rounded to nearest, p2 = e4m3(x / s - p1). |x / s| < 256, so p1 keeps the top four significant
// bits and p2 the next four: exact for a bf16 value unless it lies more than 2^9 below the row's
// largest (then p2 loses its lowest bits: an error below 2^-17 of the row's largest value).
// inf and NaN become NaN in p1. Padding rows of used blocks are zero; unused blocks are skipped.
// One warp per row, two passes over the row (largest magnitude, then the pieces). The gather
// variant also does two small jobs of the layer's front end so that they cost no launch of their
// own: the CTA after the last row CTA builds the token-tile list (tiles != nullptr), and every
// real row records where its routed slot went (inv[flat] = r, when inv != nullptr).
template <bool GATHER>
__global__ void __launch_bounds__(128)
split_rows_kernel(const uint16_t* __restrict__ src, const uint16_t* const* __restrict__ src_rows,
                  const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                  int block_size, int EM, int N, int top_k, int K, uint8_t* __restrict__ p1,
                  uint8_t* __restrict__ p2, float* __restrict__ tok_scale, int32_t* __restrict__ inv,
                  int max_tok, TokTile* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles) {
  if (GATHER && blockIdx.x * 4 >= EM) {   // the extra CTA
    __shared__ int scan[128];
    __shared__ int base;
    if (tiles != nullptr)
      build_tiles_block<128>(expert_ids, EM / block_size, block_size, max_tok, tiles, n_tiles, max_tiles, scan, &base);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= EM) return;
  if (expert_ids[r / block_size] < 0) return;   // never read by any tile
  const int flat = sorted_ids[r];
  const bool real = flat >= 0 && flat < N;
  if (GATHER && real && inv != nullptr && lane == 0) inv[flat] = r;
  const int n_vec = K / 8;
  uint2* d1 = reinterpret_cast<uint2*>(p1 + (size_t)r * K);
  uint2* d2 = reinterpret_cast<uint2*>(p2 + (size_t)r * K);
  if (!real) {
    for (int i = lane; i < n_vec; i += 32) d1[i] = d2[i] = make_uint2(0u, 0u);
    if (lane == 0) tok_scale[r] = 1.0f;
    return;
  }
  const uint4* row;
  if (GATHER) {
    const int token = flat / top_k;
    row = reinterpret_cast<const uint4*>(src_rows != nullptr ? src_rows[token] : src + (size_t)token * K);
  } else {
    row = reinterpret_cast<const uint4*>(src + (size_t)r * K);
  }
  // pass 1: largest finite magnitude (bf16 bit patterns order like their magnitudes)
  uint32_t mx = 0u;
  for (int i = lane; i < n_vec; i += 32) {
    const uint4 v = row[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = w[j] & 0x7FFFu, hi = (w[j] >> 16) & 0x7FFFu;
      if (lo < 0x7F80u) mx = max(mx, lo);
      if (hi < 0x7F80u) mx = max(mx, hi);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, d));
  int e = (int)(mx >> 7) - 127;            // exponent of the largest magnitude
  if (mx == 0u) e = 7;                      // all-zero row: scale 1
  e = max(e, -119);                         // keep 2^(e - 7) a normal fp32
  const float inv_s = __uint_as_float((uint32_t)(127 + 7 - e) << 23);
  if (lane == 0) tok_scale[r] = __uint_as_float((uint32_t)(127 + e - 7) << 23);
  // pass 2: the two pieces
  for (int i = lane; i < n_vec; i += 32) {
    const uint4 v = row[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o1[2], o2[2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = make_float2(bf16_bits_to_f32(w[j] & 0xFFFFu) * inv_s, bf16_bits_to_f32(w[j] >> 16) * inv_s);
      if (!isfinite(f.x)) f.x = __int_as_float(0x7FC00000);
      if (!isfinite(f.y)) f.y = __int_as_float(0x7FC00000);
      const uint32_t a = (uint32_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
      const __half2_raw hb = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)a, __NV_E4M3);
      const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hb));
      const uint32_t b = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f.x - back.x, f.y - back.y), __NV_SATFINITE, __NV_E4M3);
      if (j & 1) {
        o1[j >> 1] |= a << 16;
        o2[j >> 1] |= b << 16;
      } else {
        o1[j >> 1] = a;
        o2[j >> 1] = b;
      }
    }
    d1[i] = make_uint2(o1[0], o1[1]);
    d2[i] = make_uint2(o2[0], o2[1]);
  }
}

// Ordered combine: y[t, :] = bf16( sum over the token's routed slots, in ascending sorted-row
// order - for one token that is ascending expert order, the order in which the CPU definition
// adds (reference moe_fused.cpp:539-562) - of (partial[r, :] + b2[e, :]) * w ). No atomics: the
// result does not depend on which CTA finished first, and the fp32 accumulator never travels
// through memory. inv[flat] = sorted row of routed slot `flat`; an entry is trusted only if
// sorted_ids[inv[flat]] == flat (slots that were not routed leave stale entries behind).
constexpr int kMaxCombineSlots = 32;
__global__ void __launch_bounds__(256)
combine_rows_kernel(const float* __restrict__ partial, const float* __restrict__ b2, const float* __restrict__ topk_w,
                    int w_sorted, const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                    const int32_t* __restrict__ inv, int block_size, int EM, int top_k, int H,
                    uint16_t* __restrict__ y_bf16, float* __restrict__ out_f32) {
  __shared__ int s_row[kMaxCombineSlots];
  __shared__ int s_exp[kMaxCombineSlots];
  __shared__ float s_w[kMaxCombineSlots];
  __shared__ int s_n;
  const int t = blockIdx.x;
  if (threadIdx.x < 32) {
    // lane j looks slot j up (three dependent loads, all slots at once); a valid slot's place in
    // the order is the number of valid slots on smaller rows
    const int j = threadIdx.x;
    int r = -1, e = -1;
    float w = 0.0f;
    if (j < top_k) {
      const int flat = t * top_k + j;
      const int cand = inv[flat];
      if (cand >= 0 && cand < EM && sorted_ids[cand] == flat) {
        e = expert_ids[cand / block_size];
        if (e >= 0) {
          r = cand;
          w = topk_w[w_sorted ? cand : flat];
        }
      }
    }
    const unsigned valid = __ballot_sync(0xFFFFFFFFu, r >= 0);
    int rank = 0;
    for (int o = 0; o < top_k; ++o) {
      const int ro = __shfl_sync(0xFFFFFFFFu, r, o);
      if (ro >= 0 && ro < r) ++rank;
    }
    if (r >= 0) {
      s_row[rank] = r;
      s_exp[rank] = e;
      s_w[rank] = w;
    }
    if (j == 0) s_n = __popc(valid);
  }
  __syncthreads();
  const int n = s_n;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < n; ++i) {
      float4 v = *reinterpret_cast<const float4*>(partial + (size_t)s_row[i] * H + c);
      if (b2 != nullptr) {
        const float4 b = *reinterpret_cast<const float4*>(b2 + (size_t)s_exp[i] * H + c);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      }
      const float w = s_w[i];
      acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
    }
    if (out_f32 != nullptr) *reinterpret_cast<float4*>(out_f32 + (size_t)t * H + c) = acc;
    if (y_bf16 != nullptr) {
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(acc.x) | ((uint32_t)f32_to_bf16_bits(acc.y) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(acc.z) | ((uint32_t)f32_to_bf16_bits(acc.w) << 16);
      *reinterpret_cast<uint2*>(y_bf16 + (size_t)t * H + c) = o;
    }
  }
}

// ---------------------------------------------------------------------------
// prepack: checkpoint-layout MXFP4 -> the form the prepacked-fp4 GEMM reads
// ---------------------------------------------------------------------------
// Codes. The layer's table {0, .25, 1, 1.5, 2, 3} (magnitude codes 0..5) times two is
// {0, .5, 2, 3, 4, 6}: e2m1 codes 0, 1, 4, 5, 6, 7 - every code from 2 on moves up by two. Codes
// 6 and 7 (inf, NaN in this layer) have no e2m1 counterpart: they are counted, and a caller
// that finds a non-zero count keeps such weights on the checkpoint-layout path. A group whose
// scale byte is 0xFF (zero weights in this layer, NaN to the tensor core) becomes zero codes.
// One thread per 32-element group (16 bytes).
__global__ void prepack_codes_kernel(const uint4* __restrict__ w, const uint8_t* __restrict__ scale, long long n_groups,
                                     uint4* __restrict__ out, int* __restrict__ nonfinite) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  uint4 v = w[g];
  uint32_t x[4] = {v.x, v.y, v.z, v.w}, bad = 0u;
  const bool zero = scale[g] == 0xFFu;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t b1 = x[i] >> 1, b2 = x[i] >> 2;
    bad |= b1 & b2 & 0x11111111u;
    x[i] = zero ? 0u : x[i] + (((b1 | b2) & 0x11111111u) << 1);
  }
  if (bad != 0u && !zero) atomicAdd(nonfinite, 1);
  out[g] = make_uint4(x[0], x[1], x[2], x[3]);
}

// Scale factors, regrouped per (expert, 128-row work item, 256-K stage) as [128 accumulator
// rows][8 groups] so that a stage's kilobyte is one contiguous copy; rows and groups past the
// end read as 1.0 (0x7F), and so does the 0xFF of a zeroed group. One thread per byte.
__global__ void prepack_scales_kernel(const uint8_t* __restrict__ scale, int gateup, int n_feat, int K, int n_ftiles,
                                      int n_kw, long long total, uint8_t* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int b = (int)(i & 7), L = (int)((i >> 3) & 127);
  long long r = i >> 10;
  const int kw = (int)(r % n_kw);  r /= n_kw;
  const int f = (int)(r % n_ftiles);
  const long long e = r / n_ftiles;
  const int kb = kw * 8 + b, pitch = K / 32;
  long long row = -1;
  if (gateup) {
    const int sr = ((L >> 3) & 1) * 64 + (L >> 4) * 8 + (L & 7);   // accumulator row -> staged row (gate rows, then up rows)
    row = e * 2 * n_feat + (sr < 64 ? f * 64 + sr : n_feat + f * 64 + sr - 64);
  } else if (f * 128 + L < n_feat) {
    row = e * n_feat + f * 128 + L;
  }
  uint8_t v = 0x7Fu;
  if (row >= 0 && kb < pitch) {
    v = scale[row * pitch + kb];
    if (v == 0xFFu) v = 0x7Fu;
  }
  out[i] = v;
}

// ---------------------------------------------------------------------------
// host side: tensor maps, workspace layout, launch
// ---------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    VK_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
    if (p == nullptr || qres != cudaDriverEntryPointSuccess)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from the driver");
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t inner, outer, pitch;
  uint32_t box_inner, box_outer;
  int dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && pitch == o.pitch &&
           box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype;
  }
};

// Row-major 2-D tensor [outer, inner] with a byte pitch; box = [box_outer, box_inner];
// 128-byte swizzle. Encoded maps are cached: encoding costs a few microseconds
// and a decode step has only ~10 us in total.
CUtensorMap make_map(const void* ptr, CUtensorMapDataType dt, int elem_bytes, uint64_t inner,
                     uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  static std::mutex mu;
  static std::vector<std::pair<MapKey, CUtensorMap>> cache;
  const MapKey key{ptr, inner, outer, pitch_bytes, box_inner, box_outer, (int)dt};
  std::lock_guard<std::mutex> lock(mu);
  for (auto& kv : cache)
    if (kv.first == key) return kv.second;
  CUtensorMap m;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  expects(box_inner * elem_bytes == 128, "tensor map: the box must be 128 bytes wide");
  const CUresult r = get_encode_fn()(&m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  if (cache.size() >= 64) cache.erase(cache.begin());
  cache.emplace_back(key, m);
  return m;
}

// Prepacked fp4 weights [rows, K / 2] as the copy engine's packed-4-bit type that pads every 16
// nibbles to 16 bytes in shared memory. Four dimensions so that ONE box lands the 128 rows of a
// work item in accumulator row order 16 g + 8 u + j:
//   gate/up: j = feature inside a group of 8, u = gate / up half (n_feat rows apart), g = group;
//   down:    plain row order (u = 8 rows apart, g = 16 rows apart).
// and a fifth dimension counts the 128-K halves of a row, so that one box = one 256-K stage.
// The type wants an inner box of exactly 128 elements and 32-byte strides (K a multiple of 64);
// a row's last stage may read on into the next row: those columns meet zero-filled token columns.
// `half`: the 4-D map whose box is ONE 128-K half (for a last stage that K ends in early).
CUtensorMap make_map_w4(const void* ptr, int K, bool gateup, int n_feat, bool half = false) {
  static std::mutex mu;
  static std::vector<std::pair<MapKey, CUtensorMap>> cache;
  const MapKey key{ptr, (uint64_t)K, (uint64_t)n_feat, (uint64_t)K / 2, half ? 64u : 128u, gateup ? 1u : 2u,
                   (int)CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B};
  std::lock_guard<std::mutex> lock(mu);
  for (auto& kv : cache)
    if (kv.first == key) return kv.second;
  expects((reinterpret_cast<uintptr_t>(ptr) & 31u) == 0 && K % 64 == 0, "prepacked weights: 32-byte alignment, K a multiple of 64");
  CUtensorMap m;
  const uint64_t pitch = (uint64_t)K / 2;
  const cuuint64_t n_halves = (cuuint64_t)((K + kWStageK - 1) / kWStageK) * 2;   // whole stages: the tail reads on into the next row
  const cuuint64_t dims[5] = {half ? n_halves * 128 : 128, 8, 2, (cuuint64_t)1 << 27, n_halves};
  const cuuint64_t strides[4] = {pitch, gateup ? (cuuint64_t)n_feat * pitch : 8 * pitch, gateup ? 8 * pitch : 16 * pitch, 64};
  const cuuint32_t box[5] = {128, 8, 2, 8, 2};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, half ? 4 : 5, const_cast<void*>(ptr), dims, strides, box,
                                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("cuTensorMapEncodeTiled (packed 4-bit) failed with code " + std::to_string((int)r));
  if (cache.size() >= 64) cache.erase(cache.begin());
  cache.emplace_back(key, m);
  return m;
}

int max_tok_tiles(int EM) { return EM / 16 + 1; }

// gathered: [EM, hidden] bf16 rows, or - fp8 form - the two e4m3 pieces [2][EM, hidden] of the
// same size; act8: the pieces of the activation rows [2][EM, ispp]; scales: one fp32 per row each.
// ordered = the bf16-output form: + the inverse permutation [N] and the fp32 partial rows
// [EM, hidden] of the down GEMM.
struct WsLayout {
  size_t tiles_off, count_off, gathered_off, act8_off, scale_x_off, scale_a_off, inv_off, partial_off, total;
};
WsLayout ws_layout(int EM, int hidden, int ispp, bool ordered = false, int N = 0) {
  WsLayout l{};
  size_t off = 0;
  l.count_off = off;  off += 256;
  l.tiles_off = off;  off += (size_t)max_tok_tiles(EM) * sizeof(TokTile);
  off = (off + 1023) & ~size_t(1023);
  l.gathered_off = off;  off += (size_t)EM * hidden * sizeof(uint16_t);
  l.act8_off = off;  off += (size_t)EM * ispp * sizeof(uint16_t);
  l.scale_x_off = off;  off += (size_t)EM * sizeof(float);
  l.scale_a_off = off;  off += (size_t)EM * sizeof(float);
  off = (off + 1023) & ~size_t(1023);
  if (ordered) {
    l.inv_off = off;  off += (size_t)N * sizeof(int32_t);
    off = (off + 1023) & ~size_t(1023);
    l.partial_off = off;  off += (size_t)EM * hidden * sizeof(float);
  }
  l.total = off;
  return l;
}


// Small token tiles (up to 64 rows) run the fp8 form; VK_MOE_SMALL=bf16 keeps them on the
// bf16 table form (which also propagates an infinite activation as inf rather than NaN).
bool small_fp8_mode() {
  static const bool on = [] {
    const char* e = std::getenv("VK_MOE_SMALL");
    return e == nullptr || std::string(e) != "bf16";
  }();
  return on;
}

// Large token tiles run on CTA pairs; VK_MOE_PAIR=0 keeps every launch on single CTAs.
bool pair_mode() {
  static const bool on = [] {
    const char* e = std::getenv("VK_MOE_PAIR");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return on;
}

// Whether the CTA-pair form fits shared memory: one token slot per A slot, one scale buffer,
// at least two packed-weight stages.
bool pair_fits(const GemmParams& p, bool gateup) {
  const int scale_tile = (128 * (p.K / 32) + 127) & ~127;
  const int fixed = 1024 + (((int)sizeof(Barriers) + 127) & ~127) + (gateup ? kEpiStageBytes : kEpiStageDownBytes) + 128;
  const int tokens = 6 * (((p.max_tok + 31) >> 5) << 4) * 128;   // 6 x 64-K or 3 x 128-K slots
  return 227 * 1024 - fixed - scale_tile - tokens >= 2 * kWStageBytes;
}

template <bool GATEUP, int KS, int CTAS, int MX = 0, bool W4 = false>
void launch_gemm_ks(const CUtensorMap& tw, const CUtensorMap& tb, const CUtensorMap& tb64, GemmParams p,
                    cudaStream_t stream) {
  // Shared memory: token stages (this CTA's rows x KS), scales (double-buffered when they fit),
  // barriers, epilogue staging; what is left becomes the packed-weight ring (3..8 stages of
  // 16 KB): the deeper it is, the more weight bytes are in flight, which is what a decode-size
  // batch is bound by.
  constexpr int kAccCols = acc_cols(KS, CTAS);
  constexpr int kAStages = W4 ? kMaxAStages : (MX ? (kTmemCols - 2 * MX - 8) / (KS / 4 + 8) : (kTmemCols - kAccCols) / (KS / 2));
  constexpr int kThreads = block_threads(CTAS, MX != 0, W4);
  constexpr int kWBytes = W4 ? kW4StageBytes : kWStageBytes;
  const int max_smem = 227 * 1024;
  // (the prepacked-fp4 form reads its scale factors straight from global memory: no tile of them)
  const int scale_tile = W4 ? 0 : (128 * (p.K / 32) + 127) & ~127;
  const int fixed = 1024 + (((int)sizeof(Barriers) + 127) & ~127) + epi_stage_bytes(GATEUP, CTAS) + 128 +
                    (CTAS == 1 && !MX ? kLutBytes : 0);
  // a pair's MMA N is the tile rounded up to 32 rows, half of them staged by each CTA
  p.b_stage_bytes = (CTAS == 2 ? (((p.max_tok + 31) >> 5) << 4) : p.max_tok) * 128 * (KS / 64);
  // token ring: 4 slots for a lone CTA; a pair has one token slot per A slot
  // (the fp8 form: token tiles are small - 8 KB a stage at 16 rows - but come a stage at a time
  // from L2 with its full latency, so their ring is as deep as the A ring allows)
  // (prepacked fp4: five token slots and four weight slots measured best at 32-row tiles - the
  // token ring, fed from L2 a stage at a time, is the one that must not run dry)
  int b_stages = CTAS == 2 ? kAStages : (MX ? (p.max_tok <= 16 ? 6 : (W4 ? 5 : 4)) : (kAStages < 4 ? kAStages : 4)), scale_bufs = 2;
  auto w_room = [&]() {
    return (max_smem - fixed - scale_bufs * scale_tile - b_stages * p.b_stage_bytes) / kWBytes;
  };
  if (w_room() < 4) scale_bufs = 1;
  while (CTAS == 1 && w_room() < (W4 ? 4 : 3) && b_stages > 2) --b_stages;
  expects(w_room() >= 2, "fused_moe_mxfp4: reduction dimension too large for shared memory");
  p.w_stages = w_room() > kMaxWStages ? kMaxWStages : w_room();
  if (CTAS == 1 && p.w_stages == kMaxWStages) {   // spare room: deepen the token ring
    const int keep_w = kMaxWStages;
    while (b_stages < kAStages && b_stages < kMaxBStages &&
           (max_smem - fixed - scale_bufs * scale_tile - (b_stages + 1) * p.b_stage_bytes) / kWBytes >= keep_w)
      ++b_stages;
    p.w_stages = w_room() > kMaxWStages ? kMaxWStages : w_room();
  }
  p.b_stages = b_stages;
  p.scale_bufs = scale_bufs;
  p.scale_buf_bytes = scale_tile;
  const int smem = fixed + scale_bufs * scale_tile + b_stages * p.b_stage_bytes + p.w_stages * kWBytes;
  // the attribute belongs to the device's context: once per device and instantiation
  static std::atomic<bool> configured[64];
  int dev = 0;
  VK_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev].load()) {
    VK_CUDA_CHECK(cudaFuncSetAttribute(moe_gemm_sm100_kernel<GATEUP, KS, CTAS, MX, W4>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    if (dev >= 0 && dev < 64) configured[dev].store(true);
  }
  if (CTAS == 1) {
    moe_gemm_sm100_kernel<GATEUP, KS, CTAS, MX, W4><<<sm_count(), kThreads, smem, stream>>>(tw, tb, tb64, p);
  } else {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(sm_count() & ~1));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VK_CUDA_CHECK(cudaLaunchKernelEx(&cfg, moe_gemm_sm100_kernel<GATEUP, KS, CTAS, MX, W4>, tw, tb, tb64, p));
  }
}

// Stage length and CTA grouping by the largest token tile of the launch (see the kernel's comment).
template <bool GATEUP>
void launch_gemm(const CUtensorMap& tw, const CUtensorMap& tb, const CUtensorMap& tb64, GemmParams p,
                 bool use_pair, cudaStream_t stream, bool mx = false, bool w4 = false) {
  if (w4) {
    expects(p.max_tok <= 32 && mx, "prepacked fp4 weights serve token tiles of up to 32 rows");
    launch_gemm_ks<GATEUP, 256, 1, 32, true>(tw, tb, tb64, p, stream);
  } else if (p.max_tok <= 32 && mx) launch_gemm_ks<GATEUP, 256, 1, 32>(tw, tb, tb64, p, stream);
  else if (p.max_tok <= 64) launch_gemm_ks<GATEUP, 256, 1>(tw, tb, tb64, p, stream);
  else if (p.max_tok <= 128) launch_gemm_ks<GATEUP, 128, 1>(tw, tb, tb64, p, stream);
  else if (use_pair) launch_gemm_ks<GATEUP, 128, 2>(tw, tb, tb64, p, stream);
  else launch_gemm_ks<GATEUP, 64, 1>(tw, tb, tb64, p, stream);
}

}  // namespace

size_t sm100_workspace_bytes(int EM, int hidden, int ispp) { return ws_layout(EM, hidden, ispp).total; }
size_t sm100_workspace_bytes_ordered(int EM, int hidden, int ispp, int N) { return ws_layout(EM, hidden, ispp, true, N).total; }

// Sizes of the prepacked form of one weight set. which = 0: w13 [E, 2 * ispp, hidden / 2];
// 1: w2 [E, hidden, ispp / 2]. The code buffer carries 128 rows + 64 bytes of zero padding: a
// work item's box always spans 128 rows and a row's last 128-K box may reach past the row.
void prepack_sizes(int which, int E, int hidden, int ispp, size_t* w_bytes, size_t* sf_bytes) {
  expects(which == 0 || which == 1, "prepack: which must be 0 (w13) or 1 (w2)");
  expects(E > 0 && hidden > 0 && ispp > 0 && hidden % 64 == 0 && ispp % 64 == 0, "prepack: hidden and ispp must be multiples of 64");
  const long long rows = which == 0 ? 2ll * ispp : hidden;
  const int K = which == 0 ? hidden : ispp;
  const int n_ftiles = which == 0 ? ispp / 64 : (hidden + 127) / 128;
  const int n_kw = (K + kWStageK - 1) / kWStageK;
  if (w_bytes) *w_bytes = (size_t)(E * rows + 128) * (K / 2) + 256;
  if (sf_bytes) *sf_bytes = (size_t)E * n_ftiles * n_kw * kW4SfBytes;
}

void prepack_weights(int which, const uint8_t* w, const uint8_t* scale, int E, int hidden, int ispp, uint8_t* w_out,
                     uint8_t* sf_out, int* nonfinite, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  size_t w_bytes = 0, sf_bytes = 0;
  prepack_sizes(which, E, hidden, ispp, &w_bytes, &sf_bytes);
  expects(w && scale && w_out && sf_out && nonfinite, "prepack: buffers must not be null");
  auto aligned = [](const void* p, unsigned a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
  expects(aligned(w, 16) && aligned(w_out, 32) && aligned(sf_out, 16), "prepack: w 16-byte, w_out 32-byte, sf_out 16-byte aligned");
  const long long rows = which == 0 ? 2ll * ispp : hidden;
  const int K = which == 0 ? hidden : ispp;
  const int n_feat = which == 0 ? ispp : hidden;
  const int n_ftiles = which == 0 ? ispp / 64 : (hidden + 127) / 128;
  const int n_kw = (K + kWStageK - 1) / kWStageK;
  const long long n_groups = (long long)E * rows * (K / 32);
  VK_CUDA_CHECK(cudaMemsetAsync(nonfinite, 0, sizeof(int), stream));
  VK_CUDA_CHECK(cudaMemsetAsync(w_out + (size_t)n_groups * 16, 0, w_bytes - (size_t)n_groups * 16, stream));
  prepack_codes_kernel<<<(unsigned)((n_groups + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const uint4*>(w), scale, n_groups, reinterpret_cast<uint4*>(w_out), nonfinite);
  const long long total = (long long)sf_bytes;
  prepack_scales_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(scale, which == 0 ? 1 : 0, n_feat, K, n_ftiles,
                                                                           n_kw, total, sf_out);
  VK_CUDA_CHECK(cudaGetLastError());
}
// ---------------------------------------------------------------------------
// optional per-kernel timing: CUDA events recorded around the two GEMM kernels
// on the launch stream (no synchronisation while recording), summed on demand.
// The counterpart of the reference's VK_MOE_KTIME switch
// (src/c/vkernels/kernels/moe_fused.hip:1482-1493), without serialising stages.
// ---------------------------------------------------------------------------
namespace {
struct KernelTimer {
  bool on = false;
  std::vector<cudaEvent_t> ev;  // 3 per call: before gate/up, between, after down
  size_t used = 0;
} g_timer;
std::mutex g_timer_mu;
}  // namespace

void timing_begin(int max_calls) {
  std::lock_guard<std::mutex> lock(g_timer_mu);
  while (g_timer.ev.size() < (size_t)max_calls * 3) {
    cudaEvent_t e;
    VK_CUDA_CHECK(cudaEventCreate(&e));
    g_timer.ev.push_back(e);
  }
  g_timer.used = 0;
  g_timer.on = true;
}

void timing_end(float* gateup_ms, float* down_ms, int* calls) {
  std::lock_guard<std::mutex> lock(g_timer_mu);
  g_timer.on = false;
  float g = 0.f, d = 0.f;
  const size_t n = g_timer.used / 3;
  if (n > 0) VK_CUDA_CHECK(cudaEventSynchronize(g_timer.ev[n * 3 - 1]));
  for (size_t i = 0; i < n; ++i) {
    float a = 0.f, b = 0.f;
    VK_CUDA_CHECK(cudaEventElapsedTime(&a, g_timer.ev[3 * i], g_timer.ev[3 * i + 1]));
    VK_CUDA_CHECK(cudaEventElapsedTime(&b, g_timer.ev[3 * i + 1], g_timer.ev[3 * i + 2]));
    g += a;
    d += b;
  }
  if (gateup_ms) *gateup_ms = g;
  if (down_ms) *down_ms = d;
  if (calls) *calls = (int)n;
}

namespace {
// Records event `which` (0, 1, 2) of the current call when timing is on.
void timer_mark(int which, cudaStream_t stream) {
  if (!g_timer.on) return;
  std::lock_guard<std::mutex> lock(g_timer_mu);
  if (!g_timer.on) return;
  // used counts recorded events; a call's three events are consecutive
  if (g_timer.used % 3 != (size_t)which || g_timer.used >= g_timer.ev.size()) return;
  cudaEventRecord(g_timer.ev[g_timer.used], stream);
  g_timer.used += 1;
}
}  // namespace


// For the other tcgen05 kernel of the library (the router GEMM, moe_route.cu): a bf16 tensor map
// [outer, inner] with a byte pitch and a 128-byte-wide box, and the device address of the
// status word, so that its bounded waits report through the same word.
CUtensorMap sm100_make_map_bf16(const void* ptr, uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_outer) {
  return make_map(ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, inner, outer, pitch_bytes, 64, box_outer);
}
int* sm100_status_address() {
  int* p = nullptr;
  VK_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_kernel_status));
  return p;
}

// Status of the tcgen05 launches on the current device since the last reset: 0, or
// 100 + the code of the wait that ran out. Synchronises the device.
int sm100_last_status() {
  int v = 0;
  VK_CUDA_CHECK(cudaDeviceSynchronize());
  VK_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof(int)));
  return v;
}

// Clears the status word of the current device (after the failure has been dealt with).
void sm100_reset_status() {
  const int zero = 0;
  VK_CUDA_CHECK(cudaDeviceSynchronize());
  VK_CUDA_CHECK(cudaMemcpyToSymbol(g_kernel_status, &zero, sizeof(int)));
}

// Launches the one-warp probe whose bounded wait is certain to run out after `limit_clocks`.
void launch_wait_timeout_probe(long long limit_clocks, cudaStream_t stream) {
  expects(limit_clocks > 0 && limit_clocks <= 2000000000ll, "wait probe: limit must be in (0, 2e9] clocks");
  wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(limit_clocks);
  VK_CUDA_CHECK(cudaGetLastError());
}


namespace {
// Largest token tile of a launch and whether the CTA-pair form runs it.
struct TileChoice {
  int max_tok;
  bool use_pair;
};
TileChoice choose_tiles(int M, int top_k, int EM, int block_size, int k_gateup, int k_down) {
  // A token meets an expert at most once, so no expert holds more than M rows (+ padding).
  int max_tok = ((M + block_size - 1) / block_size) * block_size;
  max_tok = ((max_tok + 15) / 16) * 16;
  // When an expert sees a few dozen tokens at most, tiles are capped at 64 rows so that the launch
  // takes the long-stage form built for small tiles (an expert with more rows is split into
  // several items); measured crossover against the CTA-pair form: about 48 tokens per expert.
  // The expert count is not an argument of the layer: callers size EM as N + E * (block - 1),
  // which gives a lower bound of E (an exact EM only makes the estimate more conservative).
  {
    const long long n_slots = (long long)M * top_k;
    const long long e_est = std::max<long long>(1, ((long long)EM - n_slots) / (block_size - 1));
    if ((M <= 256 || n_slots <= 48 * e_est) && max_tok > 64) max_tok = 64;
  }
  // Tiles over 128 tokens go to CTA pairs when both GEMMs fit shared memory in that form.
  bool use_pair = false;
  if (max_tok > 128 && pair_mode()) {
    GemmParams probe{};
    probe.max_tok = max_tok > kPairMaxTok ? kPairMaxTok : ((max_tok + 31) & ~31);
    probe.K = k_gateup;
    use_pair = pair_fits(probe, true);
    probe.K = k_down;
    use_pair = use_pair && pair_fits(probe, false);
    if (use_pair) max_tok = probe.max_tok;   // a CTA pair stages half of the rows each
  }
  if (!use_pair && max_tok > kMaxTok) max_tok = kMaxTok;
  return TileChoice{max_tok, use_pair};
}
}  // namespace

// moe_gemv.cu
bool moe_tiny_eligible(int M, int hidden, int ispp, int top_k);
void launch_moe_tiny(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                     const uint8_t* w2_scale, const float* topk_w, uint16_t* act, uint16_t* y, int M, int hidden, int ispp,
                     int top_k, const int32_t* sorted_ids, const int32_t* expert_ids, int EM, float swiglu_limit,
                     int activation, float beta, float linear_beta, const float* b13, const float* b2, int block_size,
                     int32_t* slot_expert, cudaStream_t stream);

void launch_moe_sm100(const uint16_t* A, const uint8_t* w13, const uint8_t* w13_scale,
                      const uint8_t* w2, const uint8_t* w2_scale, const float* topk_w,
                      int w_sorted, uint16_t* act_scratch, float* out, int M, int hidden, int ispp,
                      int top_k, const int32_t* sorted_ids, const int32_t* expert_ids, int EM,
                      float swiglu_limit, int activation, float beta, float linear_beta,
                      const float* b13, const float* b2, int block_size, cudaStream_t stream,
                      const RowPtrs* rows, uint16_t* y_bf16, bool w4) {
  const bool store_rows = rows != nullptr && rows->store_slots;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const uint16_t* const* a_rows = rows ? rows->a_rows : nullptr;
  float* const* out_rows = rows ? rows->out_rows : nullptr;
  expects(aligned16(A) && aligned16(w13) && aligned16(w13_scale) && aligned16(w2) &&
              aligned16(w2_scale) && aligned16(act_scratch),
          "fused_moe_mxfp4: A, weights, scales and act_scratch must be 16-byte aligned");
  // y_bf16 != nullptr: the down GEMM leaves plain partial rows and an ordered combine writes the
  // bf16 result (no atomics, no fp32 output buffer to zero and convert)
  const bool ordered = y_bf16 != nullptr;
  const WsLayout l = ws_layout(EM, hidden, ispp, ordered, M * top_k);
  uint8_t* ws = static_cast<uint8_t*>(workspace_get(l.total, stream));
  TokTile* tiles = reinterpret_cast<TokTile*>(ws + l.tiles_off);
  int* n_tiles = reinterpret_cast<int*>(ws + l.count_off);
  uint16_t* gathered = reinterpret_cast<uint16_t*>(ws + l.gathered_off);
  int32_t* inv = ordered ? reinterpret_cast<int32_t*>(ws + l.inv_off) : nullptr;
  float* partial = ordered ? reinterpret_cast<float*>(ws + l.partial_off) : nullptr;

  // One or two decode tokens: two flat kernels instead of the grouped GEMMs and their helpers.
  if (ordered && rows == nullptr && !w4 && w_sorted == 0 && moe_tiny_eligible(M, hidden, ispp, top_k)) {
    timer_mark(0, stream);
    launch_moe_tiny(A, w13, w13_scale, w2, w2_scale, topk_w, act_scratch, y_bf16, M, hidden, ispp, top_k, sorted_ids,
                    expert_ids, EM, swiglu_limit, activation, beta, linear_beta, b13, b2, block_size,
                    reinterpret_cast<int32_t*>(ws + l.count_off + 64), stream);
    timer_mark(1, stream);
    timer_mark(2, stream);
    return;
  }

  // The number of experts is not an argument of the layer; the tensor maps
  // cover the rows of every expert id that fits an int32 row index.
  const uint64_t w13_rows_cap = (uint64_t)1 << 31;
  const TileChoice choice = choose_tiles(M, top_k, EM, block_size, hidden, ispp);
  const bool mx = choice.max_tok <= 64 && (small_fp8_mode() || w4);
  const int max_tok = mx ? std::min(choice.max_tok, 32) : choice.max_tok;   // the fp8 form takes tiles of up to 32 rows
  expects(!w4 || mx, "fused_moe_mxfp4: prepacked weights serve decode-size batches only (token tiles of up to 64 rows); "
                     "larger batches take the checkpoint-layout weights");
  const bool use_pair = choice.use_pair;
  // a small problem's tile list is built by an extra CTA of the row pre-pass (one launch less)
  // (and a large one's by an extra CTA of the row gather)
  const bool tiles_in_split = mx && EM / block_size <= 1024;
  if (mx && !tiles_in_split)
    build_tiles_kernel<<<1, 1024, 0, stream>>>(expert_ids, EM / block_size, block_size, max_tok, tiles,
                                               n_tiles, max_tok_tiles(EM));
  uint8_t* x8 = reinterpret_cast<uint8_t*>(gathered);            // fp8 form: pieces of the token rows
  uint8_t* a8 = ws + l.act8_off;                                 //           pieces of the activation rows
  float* scale_x = reinterpret_cast<float*>(ws + l.scale_x_off);
  float* scale_a = reinterpret_cast<float*>(ws + l.scale_a_off);
  if (mx)
    split_rows_kernel<true><<<(EM + 3) / 4 + 1, 128, 0, stream>>>(
        A, a_rows, sorted_ids, expert_ids, block_size, EM, M * top_k, top_k, hidden, x8, x8 + (size_t)EM * hidden,
        scale_x, inv, max_tok, tiles_in_split ? tiles : nullptr, n_tiles, max_tok_tiles(EM));
  else
    gather_rows_kernel<<<(EM + 3) / 4 + 1, 1024, 0, stream>>>(A, a_rows, sorted_ids, expert_ids, block_size, EM, M * top_k,
                                                             top_k, hidden, gathered, inv, max_tok, tiles, n_tiles,
                                                             max_tok_tiles(EM));

  GemmParams g{};
  g.sorted_ids = sorted_ids; g.tiles = tiles; g.n_tiles = n_tiles;
  g.N = M * top_k; g.top_k = top_k; g.w_sorted = w_sorted; g.activation = activation;
  g.limit = swiglu_limit; g.beta = beta; g.linear_beta = linear_beta; g.max_tok = max_tok;
  g.piece_rows = EM;
  // token operand: bf16 rows [EM, K], or the fp8 pieces as one byte matrix [2 * EM, K]
  auto token_maps = [&](const void* rows, int K, CUtensorMap& tb, CUtensorMap& tb64) {
    if (mx) {
      tb = make_map(rows, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, 2 * (uint64_t)EM, (uint64_t)K, 128, 16);
      tb64 = make_map(rows, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, 2 * (uint64_t)EM, (uint64_t)K, 128, 64);
    } else {
      tb = make_map(rows, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, EM, (uint64_t)K * 2, 64, 16);
      tb64 = make_map(rows, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, EM, (uint64_t)K * 2, 64, 64);
    }
  };

  {  // gate/up
    GemmParams p = g;
    p.w_scale = w13_scale; p.bias = b13; p.act = act_scratch; p.tok_scale = scale_x;
    p.K = hidden; p.n_feat = ispp; p.n_ftiles = ispp / 64;
    const CUtensorMap tw = w4 ? make_map_w4(w13, hidden, true, ispp)
                              : make_map(w13, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, hidden / 2, w13_rows_cap, hidden / 2, 128, 64);
    CUtensorMap tb, tb64;
    token_maps(mx ? static_cast<const void*>(x8) : static_cast<const void*>(gathered), hidden, tb, tb64);
    if (w4) tb64 = make_map_w4(w13, hidden, true, ispp, true);
    timer_mark(0, stream);
    launch_gemm<true>(tw, tb, tb64, p, use_pair, stream, mx, w4);
    timer_mark(1, stream);
  }
  if (mx)
    split_rows_kernel<false><<<(EM + 3) / 4, 128, 0, stream>>>(act_scratch, nullptr, sorted_ids, expert_ids, block_size,
                                                               EM, M * top_k, top_k, ispp, a8, a8 + (size_t)EM * ispp,
                                                               scale_a, nullptr, 0, nullptr, nullptr, 0);
  {  // down + combine
    GemmParams p = g;
    p.w_scale = w2_scale; p.bias = b2; p.topk_w = topk_w; p.out = out; p.out_rows = out_rows; p.tok_scale = scale_a;
    p.store_rows = store_rows ? 1 : 0;
    p.K = ispp; p.n_feat = hidden; p.n_ftiles = (hidden + 127) / 128;
    if (ordered) {
      p.raw = partial;
      p.raw_ld = hidden;
    }
    const CUtensorMap tw = w4 ? make_map_w4(w2, ispp, false, hidden)
                              : make_map(w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ispp / 2, w13_rows_cap, ispp / 2, 128, 64);
    CUtensorMap tb, tb64;
    token_maps(mx ? static_cast<const void*>(a8) : static_cast<const void*>(act_scratch), ispp, tb, tb64);
    if (w4) tb64 = make_map_w4(w2, ispp, false, hidden, true);
    launch_gemm<false>(tw, tb, tb64, p, use_pair, stream, mx, w4);
    timer_mark(2, stream);
  }
  if (ordered)
    combine_rows_kernel<<<M, 256, 0, stream>>>(partial, b2, topk_w, w_sorted, sorted_ids, expert_ids, inv, block_size, EM,
                                               top_k, hidden, y_bf16, out);
  VK_CUDA_CHECK(cudaGetLastError());
}

// One GEMM of the tensor-parallel stage split (reference moe_fused.hpp:265-286): this rank's
// weights are a K-shard ([E, rows, k_shard/2] packed, [E, rows, k_shard/32] scales), the token
// rows are full width and are read from column k_base on; the result is the plain fp32 partial
// sum (no bias, activation or routing weight), which the caller all-reduces over the ranks.
//   which = 0: gate_up[EM, 2*n_out] = gather(A[M, k_full]) @ w13_shard^T     (n_out = ispp)
//   which = 1: partial[EM, n_out]   = act[EM, k_full]      @ w2_shard^T      (n_out = hidden)
// Rows of blocks with expert_ids < 0 are left untouched, padding rows of real blocks become 0.
void launch_moe_stage_gemm(int which, const uint16_t* rows_in, const uint8_t* w, const uint8_t* w_scale,
                           const int32_t* sorted_ids, const int32_t* expert_ids, float* raw, int M,
                           int k_full, int n_out, int top_k, int EM, int k_base, int k_shard,
                           cudaStream_t stream) {
  constexpr int block_size = 16;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  expects(which == 0 || which == 1, "moe stage: unknown stage");
  expects(M >= 0 && EM >= 0 && top_k > 0 && EM % block_size == 0, "moe stage: bad M / EM / top_k");
  expects(k_full > 0 && k_full % 64 == 0 && n_out > 0 && n_out % 64 == 0, "moe stage: dimensions must be multiples of 64");
  expects(k_shard > 0 && k_shard % 64 == 0 && k_base >= 0 && k_base % 64 == 0 && k_base + k_shard <= k_full,
          "moe stage: the K shard must be a multiple of 64 inside the full reduction length");
  if (M == 0 || EM == 0) return;
  expects(rows_in && w && w_scale && sorted_ids && expert_ids && raw, "moe stage: buffers must not be null");
  expects(aligned16(rows_in) && aligned16(w) && aligned16(w_scale) && aligned16(raw),
          "moe stage: buffers must be 16-byte aligned");
  const WsLayout l = ws_layout(EM, which == 0 ? k_full : 64, 0);
  uint8_t* ws = static_cast<uint8_t*>(workspace_get(l.total, stream));
  TokTile* tiles = reinterpret_cast<TokTile*>(ws + l.tiles_off);
  int* n_tiles = reinterpret_cast<int*>(ws + l.count_off);
  uint16_t* gathered = reinterpret_cast<uint16_t*>(ws + l.gathered_off);
  const TileChoice choice = choose_tiles(M, top_k, EM, block_size, k_shard, k_shard);
  build_tiles_kernel<<<1, 1024, 0, stream>>>(expert_ids, EM / block_size, block_size, choice.max_tok, tiles,
                                             n_tiles, max_tok_tiles(EM));
  const uint16_t* token_rows = rows_in;
  if (which == 0) {
    gather_rows_kernel<<<(EM + 3) / 4, 1024, 0, stream>>>(rows_in, nullptr, sorted_ids, expert_ids, block_size, EM,
                                                          M * top_k, top_k, k_full, gathered, nullptr, 0, nullptr, nullptr, 0);
    token_rows = gathered;
  }
  GemmParams p{};
  p.sorted_ids = sorted_ids; p.tiles = tiles; p.n_tiles = n_tiles;
  p.N = M * top_k; p.top_k = top_k; p.max_tok = choice.max_tok;
  p.w_scale = w_scale; p.K = k_shard; p.k_base = k_base; p.raw = raw;
  p.n_feat = n_out;
  const uint64_t rows_cap = (uint64_t)1 << 31;
  const CUtensorMap tw = make_map(w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k_shard / 2, rows_cap, k_shard / 2, 128, 64);
  const CUtensorMap tb = make_map(token_rows, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_full, EM,
                                  (uint64_t)k_full * 2, 64, 16);
  const CUtensorMap tb64 = make_map(token_rows, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_full, EM,
                                    (uint64_t)k_full * 2, 64, 64);
  if (which == 0) {
    p.n_ftiles = n_out / 64;
    p.raw_ld = 2 * n_out;
    launch_gemm<true>(tw, tb, tb64, p, choice.use_pair, stream);
  } else {
    p.n_ftiles = (n_out + 127) / 128;
    p.raw_ld = n_out;
    launch_gemm<false>(tw, tb, tb64, p, choice.use_pair, stream);
  }
  VK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace vkernels::kernels::cuda
