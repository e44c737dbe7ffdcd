// common.cuh - shared device/host helpers of the fused MXFP4 MoE kernels.
#pragma once

#include <cuda_bf16.h>
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

// Grow-only device scratch owned by the library, one per device.
struct Workspace {
  void* ptr = nullptr;
  size_t bytes = 0;
};
// Returns a pointer to at least `bytes` of device memory on the current
// device. Grows (cudaMalloc, after a device-wide synchronise and cudaFree of
// the old block) when the request exceeds what is held.
void* workspace_get(size_t bytes);

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
