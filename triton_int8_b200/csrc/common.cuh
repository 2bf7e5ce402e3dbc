// Shared helpers for libi8linear (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/i8linear.h"

namespace i8l {

// Records printf-style text for i8l_last_error() (thread local) and returns `code`.
int fail(int code, const char* fmt, ...);

// I8L_OK when the current device is compute capability 10.x.
int check_arch();

// Shared launch settings of the tensor-core kernels (defined next to the GEMM launcher): the poll limit of
// the bounded device-side waits (lowered only by the test hook) and the number of CTAs a persistent kernel
// launched by this host thread may use (i8l_set_cta_limit, else the SM count).
uint32_t gemm_wait_limit();
int gemm_cta_budget();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define I8L_CUDA_OK(expr)                                                                  \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return i8l::fail(I8L_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));      \
  } while (0)

// ---------------------------------------------------------------- scale / rounding arithmetic
// All operations are spelled with explicit round-to-nearest intrinsics so that the compiler can
// neither contract x*s+0.5 into an FMA nor replace a division by a reciprocal: the int8 values
// and the stored scales must equal the reference's bit for bit.

template <int MODE>
__device__ __forceinline__ void make_scale(float amax, float& s, float& stored) {
  if (MODE == I8L_QMODE_TRITON || MODE == I8L_QMODE_TRITON_BF16S) {
    amax = amax > 1e-4f ? amax : 1e-4f;
    s = __fdiv_rn(127.0f, amax);
    stored = __fdiv_rn(1.0f, s);
    if (MODE == I8L_QMODE_TRITON_BF16S) stored = __bfloat162float(__float2bfloat16_rn(stored));
  } else if (MODE == I8L_QMODE_RNE) {
    amax = fmaxf(amax, 1e-4f);
    s = __fmul_rn(__frcp_rn(amax), 127.0f);
    stored = __frcp_rn(s);
  } else if (MODE == I8L_QMODE_FUSED) {
    s = __fdiv_rn(127.0f, __fadd_rn(amax, 1e-5f));
    stored = s;
  } else {  // I8L_QMODE_ROWRCP
    amax = fmaxf(amax, 1e-4f);
    s = __fmul_rn(__frcp_rn(amax), 127.0f);
    stored = __fdiv_rn(amax, 127.0f);
  }
}

// One value: y = x*s, then floor(y + 0.5) clamped to [-128, 127] (a single saturating
// round-toward-minus-infinity conversion), or rint(y) clamped to [-127, 127] for the RNE mode.
template <int MODE>
__device__ __forceinline__ int quant1(float v, float s) {
  const float y = __fmul_rn(v, s);
  int q;
  if (MODE == I8L_QMODE_RNE) {
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(y));
    q = max(q, -127);
  } else {
    asm("cvt.rmi.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(__fadd_rn(y, 0.5f)));  // never saturates for FUSED: |x*s| < 127
  }
  return q;
}

// Four quantised values (sign-extended in 32-bit registers) -> four bytes, lowest address first.
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  // cvt.pack puts its first operand in bits 8-15, the second in bits 0-7, and the low half of the
  // third operand in bits 16-31
  uint32_t hi, r;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));            // c | d<<8
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));   // a | b<<8 | c<<16 | d<<24
  return r;
}

// Packed fp32 pairs (one issue slot for two IEEE operations).  a - b is fma(b, -1, a): one rounding,
// the same result as a subtraction.
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.f, -1.f), a); }

// Two values at once: the multiply and the +0.5 stay separate roundings, as in quant1.
template <int MODE>
__device__ __forceinline__ void quant2(float2 v, float2 s2, int& q0, int& q1) {
  float2 y = __fmul2_rn(v, s2);
  if (MODE == I8L_QMODE_RNE) {
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(y.x));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(y.y));
    q0 = max(q0, -127);
    q1 = max(q1, -127);
  } else {
    y = __fadd2_rn(y, make_float2(0.5f, 0.5f));
    asm("cvt.rmi.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(y.x));
    asm("cvt.rmi.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(y.y));
  }
}

// Eight bf16 (a 16-byte piece) -> eight int8 in two words.
template <int MODE>
__device__ __forceinline__ uint2 quant_piece(const uint4& u, float s) {
  const float2 s2 = make_float2(s, s);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  int q[8];
#pragma unroll
  for (int k = 0; k < 4; ++k)
    quant2<MODE>(make_float2(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xffff0000u)), s2, q[2 * k], q[2 * k + 1]);
  return make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

__device__ __forceinline__ void unpack8(const uint4& u, float* v) {
  v[0] = bf16_bits_to_float(u.x & 0xffffu); v[1] = __uint_as_float(u.x & 0xffff0000u);
  v[2] = bf16_bits_to_float(u.y & 0xffffu); v[3] = __uint_as_float(u.y & 0xffff0000u);
  v[4] = bf16_bits_to_float(u.z & 0xffffu); v[5] = __uint_as_float(u.z & 0xffff0000u);
  v[6] = bf16_bits_to_float(u.w & 0xffffu); v[7] = __uint_as_float(u.w & 0xffff0000u);
}

__device__ __forceinline__ float round_to_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// 128-point Walsh-Hadamard transform of a row segment held as 8 consecutive values in each of 16
// consecutive lanes (lane & 15 selects the 8-wide chunk).  Butterfly spans double from 1 to 64,
// the order the CPU oracle uses; fp32 adds commute, so the result is bit-equal to it.
__device__ __forceinline__ void fwht128_lanes16(float* v, int lane) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((j & h) == 0) {
        float a = v[j], b = v[j | h];
        v[j] = __fadd_rn(a, b);
        v[j | h] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 16; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = upper ? __fsub_rn(p, v[j]) : __fadd_rn(v[j], p);
    }
  }
}

}  // namespace i8l
