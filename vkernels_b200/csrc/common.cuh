// common.cuh - shared device/host helpers of the fused MXFP4 MoE kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

namespace vkernels::kernels::cuda {

// ---------------------------------------------------------------------------
// host-side error plumbing
// ---------------------------------------------------------------------------

inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
#define VK_CUDA_CHECK(expr) ::vkernels::kernels::cuda::cuda_check((expr), #expr)

inline void expects(bool ok, const char* msg) {
  if (!ok) throw std::invalid_argument(msg);
}

// Library-owned device scratch (tile lists, gathered activation rows, alignment histograms): one
// block per (device, stream), so calls on different streams never share scratch. A block is
// allocated on the first call of its stream, or ahead of time by reserve_workspace; when a later
// call needs more, a larger block is allocated and the old one is kept until
// release_workspaces() - work already enqueued, or a captured graph, may still point at it.
// No call synchronises the device or frees memory. While `stream` is being captured nothing can
// be allocated: the call throws std::invalid_argument (reserve before capturing).
void* workspace_get(size_t bytes, cudaStream_t stream);

// Number of SMs of the current device.
int sm_count();

// ---------------------------------------------------------------------------
// MXFP4 decode (bit-exact against the layer's CPU definition)
// ---------------------------------------------------------------------------
//
// Nibble magnitudes are {0, 0.25, 1, 1.5, 2, 3, inf, NaN} - NOT the OCP E2M1
// table - and bit 3 is the sign (reference moe_fused.cpp:24-39). A ue8m0 scale
// byte s means 2^(s-127), with s = 0 the subnormal 2^-127 and s = 0xFF zero
// (reference moe_fused.cpp:50-64). The dequantised weight is
// bf16(fp32(nibble) * fp32(scale)); every finite product is exactly
// representable in bf16, so one bf16 multiply of the table value by the scale
// gives the same bits (overflow goes to inf and inf * 0 to NaN on both paths).

// bf16 bit pattern of a ue8m0 scale, replicated in both halves.
__device__ __forceinline__ uint32_t ue8m0_to_bf16x2(uint32_t s) {
  uint32_t b = (s == 0xFFu) ? 0u : (s == 0u ? 0x0040u : (s << 7));
  return b * 0x00010001u;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&a);
  __nv_bfloat162 y = *reinterpret_cast<__nv_bfloat162*>(&b);
  __nv_bfloat162 r = __hmul2(x, y);
  return *reinterpret_cast<uint32_t*>(&r);
}

// Eight packed nibbles (k0 in bits 3:0 ... k7 in bits 31:28) times one scale
// -> four bf16x2 words, word j = (k_2j in the low half, k_2j+1 in the high).
//
// The high and low bytes of the eight table magnitudes fit two 8-byte pools,
// so a byte permute with the 3-bit magnitudes as selectors looks four nibbles
// up at once; a permute in sign-replication mode spreads the four sign bits to
// byte MSBs; two more permutes interleave low and high bytes into bf16 pairs.
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t scale2, uint32_t out[4]) {
  constexpr uint32_t HI0 = 0x3F3F3E00u, HI1 = 0x7F7F4040u;  // high bytes, magnitudes 0-3 / 4-7
  constexpr uint32_t LO0 = 0xC0808000u, LO1 = 0xC0804000u;  // low bytes
  const uint32_t m = w & 0x77777777u;
  const uint32_t mh = m >> 16;
  const uint32_t t = w << 4;
  uint32_t hiA = prmt(HI0, HI1, m), hiB = prmt(HI0, HI1, mh);
  const uint32_t loA = prmt(LO0, LO1, m), loB = prmt(LO0, LO1, mh);
  const uint32_t sgA = prmt(w, t, 0x9D8Cu), sgB = prmt(w, t, 0xBFAEu);
  hiA |= sgA & 0x80808080u;
  hiB |= sgB & 0x80808080u;
  out[0] = mul_bf16x2(prmt(loA, hiA, 0x5140u), scale2);
  out[1] = mul_bf16x2(prmt(loA, hiA, 0x7362u), scale2);
  out[2] = mul_bf16x2(prmt(loB, hiB, 0x5140u), scale2);
  out[3] = mul_bf16x2(prmt(loB, hiB, 0x7362u), scale2);
}

// Expansion through a shared-memory table (256 entries of one bf16 pair, replicated once per
// bank: lane l reads word 32 * byte + l, 32 KB in all): per byte of packed weights one
// integer-pipe instruction to isolate it, one multiply-add for the address, one load and one
// bf16x2 multiply - a quarter of the integer-pipe work of the permute-based dequant8. Same
// bits: table value (exact) times scale in one bf16 multiply.
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// 64 nibbles (two 16-byte chunks, one scale each) in three passes over the same 32 registers:
// all table addresses, all loads, all multiplies - every pass is 32 independent instructions,
// so a lone warp keeps its pipes busy instead of walking one dependent chain at a time.
__device__ __forceinline__ void dequant64_lut(const uint4& p0, const uint4& p1, uint32_t s0, uint32_t s1,
                                              uint32_t lut_lane, uint32_t (&v)[32]) {
  const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[4 * i + 0] = lut_lane + (w[i] & 0xFFu) * 128u;
    v[4 * i + 1] = lut_lane + prmt(w[i], 0u, 0x4441u) * 128u;
    v[4 * i + 2] = lut_lane + prmt(w[i], 0u, 0x4442u) * 128u;
    v[4 * i + 3] = lut_lane + (w[i] >> 24) * 128u;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = lds_u32(v[i]);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = mul_bf16x2(v[i], s0);
#pragma unroll
  for (int i = 16; i < 32; ++i) v[i] = mul_bf16x2(v[i], s1);
}
// bf16 bit pattern of one nibble code (sign in bit 3) under the layer's table
__device__ __forceinline__ uint32_t e2m1_bf16_bits(uint32_t code) {
  const uint32_t m = code & 7u;
  const uint32_t mag = m == 0 ? 0x0000u : m == 1 ? 0x3E80u : m == 2 ? 0x3F80u : m == 3 ? 0x3FC0u
                     : m == 4 ? 0x4000u : m == 5 ? 0x4040u : m == 6 ? 0x7F80u : 0x7FC0u;
  return mag | ((code & 8u) << 12);
}

// Fills the replicated table used by dequant64_lut (all threads of the CTA take part).
__device__ __forceinline__ void fill_dequant_lut(uint32_t* lut, int tid, int n_threads) {
  for (int i = tid; i < 256 * 32; i += n_threads) {
    const uint32_t byte = (uint32_t)i >> 5;
    lut[i] = e2m1_bf16_bits(byte & 15u) | (e2m1_bf16_bits(byte >> 4) << 16);
  }
}

// Eight packed nibbles -> eight e5m2 bytes in K order (out[0] = k0..k3, out[1] = k4..k7). Every
// value of the layer's table is exact in e5m2, inf and NaN included: magnitudes
// {00, 34, 3C, 3E, 40, 42, 7C, 7E}, sign in bit 7. A byte permute with the 3-bit magnitudes as
// selectors looks four nibbles up at once; a second permute in sign-replication mode brings the
// four sign bits to the byte tops.
__device__ __forceinline__ void expand8_e5m2(uint32_t w, uint32_t out[2]) {
  constexpr uint32_t P0 = 0x3E3C3400u, P1 = 0x7E7C4240u;
  const uint32_t m = w & 0x77777777u;
  const uint32_t t = w << 4;
  const uint32_t a0 = prmt(P0, P1, m), a1 = prmt(P0, P1, m >> 16);
  const uint32_t s0 = prmt(w, t, 0x9D8Cu), s1 = prmt(w, t, 0xBFAEu);
  out[0] = a0 | (s0 & 0x80808080u);
  out[1] = a1 | (s1 & 0x80808080u);
}
// value of an e5m2 byte
__device__ __forceinline__ float e5m2_to_f32(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)(b << 8))); }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }

// fp32 -> bf16 bits, round to nearest even (the layer rounds its activations
// exactly once with this rule, reference moe_fused.cpp:41-45,413-417).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Gate/up epilogue of one element (reference moe_fused.cpp:206-226).
__device__ __forceinline__ float moe_act_value(int activation, float g, float u, float limit,
                                               float beta, float linear_beta) {
  if (activation == 1) {
    float sig = 1.0f / (1.0f + expf(-g));
    float go = beta * tanhf(g / beta) * sig;
    float uo = (linear_beta > 0.0f) ? linear_beta * tanhf(u / linear_beta) : u;
    return go * uo;
  }
  if (limit > 0.0f) {
    // comparisons, not fminf/fmaxf: a NaN operand must stay NaN
    g = (g > limit) ? limit : g;
    u = (u > limit) ? limit : u;
    u = (u < -limit) ? -limit : u;
  }
  return (g / (1.0f + expf(-g))) * u;
}

}  // namespace vkernels::kernels::cuda
