// bf16 -> int8 absmax quantizers (HBM-bound): 128x128-tile kernel with optional transposed
// output and fused 128-point Hadamard rotation, whole-row kernel, column-absmax kernel.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace i8l {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_arch() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(I8L_ERR_CUDA, "cudaGetDevice failed");
  static std::atomic<int> cached_major[64];  // 0 = unknown
  int major = (dev >= 0 && dev < 64) ? cached_major[dev].load(std::memory_order_relaxed) : 0;
  if (major == 0) {
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return fail(I8L_ERR_CUDA, "cudaDeviceGetAttribute failed");
    if (dev >= 0 && dev < 64) cached_major[dev].store(major, std::memory_order_relaxed);
  }
  if (major != 10)
    return fail(I8L_ERR_ARCH, "device %d has compute capability %d.x; this library is sm_100a only", dev, major);
  return I8L_OK;
}

// ------------------------------------------------------------------------------------------------
// Tile kernel.  One CTA of 256 threads owns one 128x128 tile of x.
// Thread mapping: warp w owns tile rows 16w..16w+15; pass it in {0,1}; lane = (half<<4)|cc;
// the thread holds rows 16w + 8it + 4half + i (i<4), columns 8cc..8cc+7: every global load is a
// 16-byte vector and 16 lanes cover one 256-byte row segment.
// ------------------------------------------------------------------------------------------------
constexpr int GRAN_COLFULL = 3;  // internal: per-column scale from a precomputed column absmax
constexpr int GRAN_COLMAX_PASS = 4;  // internal: only accumulate the column absmax of the rotated tile

// |x| maximum of the 8 bf16 values of a 16-byte vector, as two packed maxima (exact: bf16 compare).
__device__ __forceinline__ __nv_bfloat162 absmax8(const uint4& u, __nv_bfloat162 m) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) m = __hmax2(m, __habs2(h[k]));
  return m;
}
__device__ __forceinline__ float hmax_of(__nv_bfloat162 m) { return fmaxf(__low2float(m), __high2float(m)); }

template <int GRAN, int MODE, bool HAD, bool OUT_N, bool OUT_T>
__global__ void __launch_bounds__(256, 4)
quant_tile_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                  int8_t* __restrict__ q, float* __restrict__ scale, int8_t* __restrict__ qt,
                  float* __restrict__ scale_t, const float* __restrict__ colmax) {
  __shared__ float s_red[8];
  __shared__ float s_colred[(GRAN == I8L_GRAN_GROUP128 && OUT_T) ? 8 * 128 : 1];
  __shared__ float s_cols[(GRAN != I8L_GRAN_TILE128 && OUT_T) ? 128 : 1];
  __shared__ uint32_t s_t[OUT_T ? 128 * 32 : 1];

  const int tid = threadIdx.x, w = tid >> 5, l = tid & 31, cc = l & 15, half = l >> 4;
  const int64_t r_base = (int64_t)blockIdx.y * 128, c_base = (int64_t)blockIdx.x * 128;
  const int64_t boff = (int64_t)blockIdx.z * rows * cols;
  const __nv_bfloat16* xb = x + boff;

  // The tile stays in registers as packed bf16 (32 registers per thread, 4 CTAs per SM); with the
  // Hadamard rotation the rotated values, already rounded to bf16, replace the raw ones.
  uint4 raw[2][4];
#pragma unroll
  for (int it = 0; it < 2; ++it)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 16 * w + 8 * it + 4 * half + i;
      raw[it][i] = __ldg(reinterpret_cast<const uint4*>(xb + (r_base + r) * cols + c_base + 8 * cc));
      if (HAD) {
        float v[8];
        unpack8(raw[it][i], v);
        fwht128_lanes16(v, l);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw[it][i]);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
      }
    }

  // ---- scales
  const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
  float s_tile = 0.f;          // TILE128
  float s_row[2][4];           // GROUP128 natural
  float s_col[8];              // column scales (GROUP128 transposed / COLFULL)
  if (GRAN == I8L_GRAN_TILE128) {
    __nv_bfloat162 m2 = zero2;
#pragma unroll
    for (int it = 0; it < 2; ++it)
#pragma unroll
      for (int i = 0; i < 4; ++i) m2 = absmax8(raw[it][i], m2);
    float m = hmax_of(m2);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (l == 0) s_red[w] = m;
    __syncthreads();
    m = s_red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
    float stored;
    make_scale<MODE>(m, s_tile, stored);
    if (tid == 0) {
      const int64_t nrb = rows / 128, ncb = cols / 128;
      if (OUT_N) scale[((int64_t)blockIdx.z * nrb + blockIdx.y) * ncb + blockIdx.x] = stored;
      if (OUT_T) scale_t[((int64_t)blockIdx.z * ncb + blockIdx.x) * nrb + blockIdx.y] = stored;
    }
  } else if (GRAN == I8L_GRAN_GROUP128 && OUT_N) {
#pragma unroll
    for (int it = 0; it < 2; ++it)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float m = hmax_of(absmax8(raw[it][i], zero2));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float stored;
        make_scale<MODE>(m, s_row[it][i], stored);
        if (cc == 0) {
          const int r = 16 * w + 8 * it + 4 * half + i;
          scale[((int64_t)blockIdx.z * rows + r_base + r) * (cols / 128) + blockIdx.x] = stored;
        }
      }
  } else {  // column scales
    if (GRAN == I8L_GRAN_GROUP128) {
      __nv_bfloat162 cm[4] = {zero2, zero2, zero2, zero2};   // per-column maxima of this thread's 8 rows
#pragma unroll
      for (int it = 0; it < 2; ++it)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[it][i]);
#pragma unroll
          for (int k = 0; k < 4; ++k) cm[k] = __hmax2(cm[k], __habs2(h[k]));
        }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float m = (j & 1) ? __high2float(cm[j >> 1]) : __low2float(cm[j >> 1]);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
        if (half == 0) s_colred[w * 128 + 8 * cc + j] = m;
      }
      __syncthreads();
    }
    if (tid < 128) {
      float m;
      if (GRAN == I8L_GRAN_GROUP128) {
        m = s_colred[tid];
#pragma unroll
        for (int k = 1; k < 8; ++k) m = fmaxf(m, s_colred[k * 128 + tid]);
      } else {
        m = colmax[c_base + tid];
      }
      float s, stored;
      make_scale<MODE>(m, s, stored);
      s_cols[tid] = s;
      if (GRAN == I8L_GRAN_GROUP128)
        scale_t[((int64_t)blockIdx.z * cols + c_base + tid) * (rows / 128) + blockIdx.y] = stored;
      else if (blockIdx.y == 0)
        scale_t[c_base + tid] = stored;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) s_col[j] = s_cols[8 * cc + j];
  }

  // ---- quantise, write
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    int b[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v[8];
      unpack8(raw[it][i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float s;
        if (GRAN == I8L_GRAN_TILE128) s = s_tile;
        else if (GRAN == I8L_GRAN_GROUP128 && OUT_N) s = s_row[it][i];
        else s = s_col[j];
        b[i][j] = quant1<MODE>(v[j], s);
      }
    }
    if (OUT_N) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 16 * w + 8 * it + 4 * half + i;
        uint2 o;
        o.x = pack4(b[i][0], b[i][1], b[i][2], b[i][3]);
        o.y = pack4(b[i][4], b[i][5], b[i][6], b[i][7]);
        *reinterpret_cast<uint2*>(q + boff + (r_base + r) * cols + c_base + 8 * cc) = o;
      }
    }
    if (OUT_T) {
      // word (4 consecutive rows of one column) goes to transposed row c = 8cc+j, word index
      // widx = 4w + 2it + half, XOR-swizzled with 2*(c>>3) so that the 32 lanes hit 32 banks.
      const int widx = 4 * w + 2 * it + half;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = 8 * cc + j;
        s_t[c * 32 + (widx ^ (2 * cc))] = pack4(b[0][j], b[1][j], b[2][j], b[3][j]);
      }
    }
  }
  if (OUT_T) {
    __syncthreads();
    int8_t* qtb = qt + boff;
#pragma unroll 4
    for (int t = 0; t < 16; ++t) {
      const int c = 16 * w + t;
      const uint32_t word = s_t[c * 32 + (l ^ (2 * (c >> 3)))];
      *reinterpret_cast<uint32_t*>(qtb + (c_base + c) * rows + r_base + 4 * l) = word;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// One scale per 128 rows x 256 columns (the activation grouping of the reference's TileLang forward).
// One CTA of 256 threads per group: warp w holds rows 16w..16w+15, one 16-byte piece per lane and row
// (32 lanes cover the 512-byte row segment), 64 registers of packed bf16 per thread.
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(256, 3)
quant_tile256_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols, int8_t* __restrict__ q,
                     float* __restrict__ scale) {
  __shared__ float s_red[8];
  const int tid = threadIdx.x, w = tid >> 5, l = tid & 31;
  const int64_t r_base = (int64_t)blockIdx.y * 128, c_base = (int64_t)blockIdx.x * 256;
  const int64_t boff = (int64_t)blockIdx.z * rows * cols;
  uint4 raw[16];
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    raw[i] = __ldg(reinterpret_cast<const uint4*>(x + boff + (r_base + 16 * w + i) * cols + c_base + 8 * l));
    m2 = absmax8(raw[i], m2);
  }
  float m = hmax_of(m2);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (l == 0) s_red[w] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
  float s, stored;
  make_scale<MODE>(m, s, stored);
  if (tid == 0) scale[((int64_t)blockIdx.z * (rows / 128) + blockIdx.y) * (cols / 256) + blockIdx.x] = stored;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    *reinterpret_cast<uint2*>(q + boff + (r_base + 16 * w + i) * cols + c_base + 8 * l) = quant_piece<MODE>(raw[i], s);
}

// ------------------------------------------------------------------------------------------------
// Natural operand with the 128-point rotation along the columns (its contraction axis).  Four lanes
// share a row: lane j of the quad holds the 16-byte pieces 4c+j (c = 0..3) of the row's 128 values,
// so each load instruction of a quad covers 64 contiguous bytes and only two of the seven butterfly
// stages cross lanes (spans 8 and 16); spans 1-4 and 32-64 run in registers.
// ------------------------------------------------------------------------------------------------
template <int GRAN, int MODE>
__global__ void __launch_bounds__(256, 4)
quant_tile_hadcols_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                          int8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float s_red[8];
  const int tid = threadIdx.x, w = tid >> 5, l = tid & 31, j4 = l & 3, rq = l >> 2;
  const int64_t r_base = (int64_t)blockIdx.y * 128, c_base = (int64_t)blockIdx.x * 128;
  const int64_t boff = (int64_t)blockIdx.z * rows * cols;
  float s_tile = 0.f, s_row[2];
  uint4 packed[2][4];  // rotated values, rounded to bf16
  float tmax = 0.f;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int r = 16 * w + 8 * it + rq;
    const __nv_bfloat16* xr = x + boff + (r_base + r) * cols + c_base;
    float2 pv[4][4];  // piece c, pair k = elements 2k, 2k+1 of the piece
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(xr + 8 * (4 * c + j4))), v);
      // span 1: inside each pair
#pragma unroll
      for (int k = 0; k < 4; ++k) pv[c][k] = make_float2(__fadd_rn(v[2 * k], v[2 * k + 1]), __fsub_rn(v[2 * k], v[2 * k + 1]));
      // spans 2, 4: between the pairs of a piece, two butterflies per packed operation
#pragma unroll
      for (int h = 1; h < 4; h <<= 1)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if ((k & h) == 0) {
            const float2 a = pv[c][k], b = pv[c][k | h];
            pv[c][k] = add2(a, b);
            pv[c][k | h] = sub2(a, b);
          }
    }
    // spans 8, 16: across the quad (element index = 32c + 8j + t): partner - own or own + partner
#pragma unroll
    for (int m = 1; m < 4; m <<= 1) {
      const float sg = (j4 & m) ? -1.f : 1.f;
      const float2 sg2 = make_float2(sg, sg);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 o = make_float2(__shfl_xor_sync(0xffffffffu, pv[c][k].x, m), __shfl_xor_sync(0xffffffffu, pv[c][k].y, m));
          pv[c][k] = __ffma2_rn(pv[c][k], sg2, o);   // exact products by +-1: own + partner, or partner - own
        }
    }
    // spans 32, 64: across the four pieces of the lane
#pragma unroll
    for (int h = 1; h < 4; h <<= 1)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if ((c & h) == 0)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 a = pv[c][k], b = pv[c | h][k];
            pv[c][k] = add2(a, b);
            pv[c | h][k] = sub2(a, b);
          }
    __nv_bfloat162 hm = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed[it][c]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        h2[k] = __floats2bfloat162_rn(pv[c][k].x, pv[c][k].y);
        hm = __hmax2(hm, __habs2(h2[k]));
      }
    }
    float m = fmaxf(__low2float(hm), __high2float(hm));
    if (GRAN == I8L_GRAN_GROUP128) {
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      float stored;
      make_scale<MODE>(m, s_row[it], stored);
      if (j4 == 0) scale[((int64_t)blockIdx.z * rows + r_base + r) * (cols / 128) + blockIdx.x] = stored;
    }
    tmax = fmaxf(tmax, m);
  }
  if (GRAN == I8L_GRAN_TILE128) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    if (l == 0) s_red[w] = tmax;
    __syncthreads();
    tmax = s_red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) tmax = fmaxf(tmax, s_red[k]);
    float stored;
    make_scale<MODE>(tmax, s_tile, stored);
    if (tid == 0) scale[((int64_t)blockIdx.z * (rows / 128) + blockIdx.y) * (cols / 128) + blockIdx.x] = stored;
  }
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int r = 16 * w + 8 * it + rq;
    const float s = GRAN == I8L_GRAN_TILE128 ? s_tile : s_row[it];
    int8_t* qr = q + boff + (r_base + r) * cols + c_base;
#pragma unroll
    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint2*>(qr + 8 * (4 * c + j4)) = quant_piece<MODE>(packed[it][c], s);
  }
}

// ------------------------------------------------------------------------------------------------
// Transposed operand with the rotation along ITS contraction axis, i.e. along the rows of x: the dW
// operands dY^T and X^T of a rotated linear layer (contraction over the tokens).  One CTA per 128x128
// tile: the tile is staged in shared memory as fp32, thread (c, h) then owns rows 64h..64h+63 of
// column c, runs six butterfly stages in registers and the last one with its partner lane, rounds to
// bf16, and writes 64 consecutive bytes of output row c.
// ------------------------------------------------------------------------------------------------
template <int GRAN, int MODE>
__global__ void __launch_bounds__(256)
quant_tile_hadrows_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                          int8_t* __restrict__ qt, float* __restrict__ scale_t, float* __restrict__ colmax) {
  extern __shared__ float s_tile[];  // [128][132]: rows 16-byte aligned for vector stores
  __shared__ float s_red[8];
  constexpr int LD = 132;
  const int tid = threadIdx.x, w = tid >> 5, l = tid & 31, cc = l & 15, half = l >> 4;
  const int64_t r_base = (int64_t)blockIdx.y * 128, c_base = (int64_t)blockIdx.x * 128;
  const int64_t boff = (int64_t)blockIdx.z * rows * cols;
  const __nv_bfloat16* xb = x + boff;
#pragma unroll
  for (int it = 0; it < 2; ++it)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 16 * w + 8 * it + 4 * half + i;
      float v[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(xb + (r_base + r) * cols + c_base + 8 * cc)), v);
      *reinterpret_cast<float4*>(s_tile + r * LD + 8 * cc) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(s_tile + r * LD + 8 * cc + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  __syncthreads();
  const int c = tid >> 1, h = tid & 1;
  float2 pv[32];  // pair k = rows 64h + 2k, 64h + 2k + 1 of column c
#pragma unroll
  for (int k = 0; k < 32; ++k) {  // span 1 on the way in
    const float a = s_tile[(64 * h + 2 * k) * LD + c], b = s_tile[(64 * h + 2 * k + 1) * LD + c];
    pv[k] = make_float2(__fadd_rn(a, b), __fsub_rn(a, b));
  }
#pragma unroll
  for (int span = 1; span < 32; span <<= 1) {  // spans 2..32 of the elements: two butterflies per packed operation
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      if ((k & span) == 0) {
        const float2 a = pv[k], b = pv[k | span];
        pv[k] = add2(a, b);
        pv[k | span] = sub2(a, b);
      }
    }
  }
  // span 64: the partner lane holds the other half of the column; then round to bf16 as the
  // reference's rotation does
  uint32_t hv[32];
  __nv_bfloat162 hm = __floats2bfloat162_rn(0.f, 0.f);
  const float sg = h ? -1.f : 1.f;
  const float2 sg2 = make_float2(sg, sg);
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    const float2 o = make_float2(__shfl_xor_sync(0xffffffffu, pv[k].x, 1), __shfl_xor_sync(0xffffffffu, pv[k].y, 1));
    const float2 r = __ffma2_rn(pv[k], sg2, o);  // own + partner, or partner - own
    const __nv_bfloat162 b2 = __floats2bfloat162_rn(r.x, r.y);
    hm = __hmax2(hm, __habs2(b2));
    hv[k] = *reinterpret_cast<const uint32_t*>(&b2);
  }
  float m = fmaxf(__low2float(hm), __high2float(hm));
  float s, stored;
  if (GRAN == I8L_GRAN_TILE128) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (l == 0) s_red[w] = m;
    __syncthreads();
    m = s_red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
    make_scale<MODE>(m, s, stored);
    if (tid == 0) scale_t[((int64_t)blockIdx.z * (cols / 128) + blockIdx.x) * (rows / 128) + blockIdx.y] = stored;
  } else if (GRAN == GRAN_COLMAX_PASS) {  // first pass of the whole-column scale: absmax of the rotated column
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    if (h == 0) atomicMax(reinterpret_cast<int*>(colmax + c_base + c), __float_as_int(m));
    return;
  } else if (GRAN == GRAN_COLFULL) {      // second pass: one scale per output row over all of its elements
    make_scale<MODE>(colmax[c_base + c], s, stored);
    if (h == 0 && blockIdx.y == 0) scale_t[c_base + c] = stored;
  } else {  // one scale per output row (column of x) and 128 contraction elements
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    make_scale<MODE>(m, s, stored);
    if (h == 0) scale_t[((int64_t)blockIdx.z * cols + c_base + c) * (rows / 128) + blockIdx.y] = stored;
  }
  int8_t* out = qt + boff + (c_base + c) * rows + r_base + 64 * h;
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    const uint2 lo = quant_piece<MODE>(make_uint4(hv[k], hv[k + 1], hv[k + 2], hv[k + 3]), s);
    const uint2 hi = quant_piece<MODE>(make_uint4(hv[k + 4], hv[k + 5], hv[k + 6], hv[k + 7]), s);
    *reinterpret_cast<uint4*>(out + 2 * k) = make_uint4(lo.x, lo.y, hi.x, hi.y);
  }
}

// ------------------------------------------------------------------------------------------------
// Both rotated operands of a 128x128 tile from ONE read of x: q (rotation along the columns, as
// quant_tile_hadcols_kernel) and qt (the transpose, rotation along the rows, as quant_tile_hadrows_kernel),
// each with its own per-tile scale.  Results are bit-identical to those two kernels.
//   Phase A: hadcols thread mapping; every 16-byte piece is also parked in shared memory as raw bf16.
//   Phase B: thread (c, h) owns column c and the 64 rows whose bit 1 equals h (rows 4m+2h, 4m+2h+1), so
//   that the butterfly of span 2 is the one that crosses the lane pair and the two lanes read different
//   shared-memory banks; spans run in the order 1, 2, 4, ... 64 like everywhere else.  The quantized byte
//   pairs are exchanged once more so that each lane stores 64 contiguous bytes of output row c.
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(256, 3)
quant_tile_had_dual_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                           int8_t* __restrict__ q, float* __restrict__ scale, int8_t* __restrict__ qt,
                           float* __restrict__ scale_t) {
  constexpr int LDB = 272;  // bytes per shared row: 256 + 16 (keeps 16-byte alignment, spreads the banks)
  __shared__ __align__(16) uint8_t s_raw[128 * LDB];
  __shared__ float s_red[8], s_red_t[8];
  const int tid = threadIdx.x, w = tid >> 5, l = tid & 31, j4 = l & 3, rq = l >> 2;
  const int64_t r_base = (int64_t)blockIdx.y * 128, c_base = (int64_t)blockIdx.x * 128;
  const int64_t boff = (int64_t)blockIdx.z * rows * cols;
  // ---------------------------------------------------------------- phase A: rotation along the columns
  float s_tile = 0.f;
  uint4 packed[2][4];
  float tmax = 0.f;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int r = 16 * w + 8 * it + rq;
    const __nv_bfloat16* xr = x + boff + (r_base + r) * cols + c_base;
    float2 pv[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(xr + 8 * (4 * c + j4)));
      *reinterpret_cast<uint4*>(s_raw + r * LDB + 16 * (4 * c + j4)) = u;
      float v[8];
      unpack8(u, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) pv[c][k] = make_float2(__fadd_rn(v[2 * k], v[2 * k + 1]), __fsub_rn(v[2 * k], v[2 * k + 1]));
#pragma unroll
      for (int h = 1; h < 4; h <<= 1)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if ((k & h) == 0) {
            const float2 a = pv[c][k], b = pv[c][k | h];
            pv[c][k] = add2(a, b);
            pv[c][k | h] = sub2(a, b);
          }
    }
#pragma unroll
    for (int m = 1; m < 4; m <<= 1) {
      const float sg = (j4 & m) ? -1.f : 1.f;
      const float2 sg2 = make_float2(sg, sg);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 o = make_float2(__shfl_xor_sync(0xffffffffu, pv[c][k].x, m), __shfl_xor_sync(0xffffffffu, pv[c][k].y, m));
          pv[c][k] = __ffma2_rn(pv[c][k], sg2, o);
        }
    }
#pragma unroll
    for (int h = 1; h < 4; h <<= 1)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if ((c & h) == 0)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 a = pv[c][k], b = pv[c | h][k];
            pv[c][k] = add2(a, b);
            pv[c | h][k] = sub2(a, b);
          }
    __nv_bfloat162 hm = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed[it][c]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        h2[k] = __floats2bfloat162_rn(pv[c][k].x, pv[c][k].y);
        hm = __hmax2(hm, __habs2(h2[k]));
      }
    }
    tmax = fmaxf(tmax, fmaxf(__low2float(hm), __high2float(hm)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
  if (l == 0) s_red[w] = tmax;
  __syncthreads();   // also: the raw tile is complete in shared memory
  tmax = s_red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) tmax = fmaxf(tmax, s_red[k]);
  {
    float stored;
    make_scale<MODE>(tmax, s_tile, stored);
    if (tid == 0) scale[((int64_t)blockIdx.z * (rows / 128) + blockIdx.y) * (cols / 128) + blockIdx.x] = stored;
  }
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int r = 16 * w + 8 * it + rq;
    int8_t* qr = q + boff + (r_base + r) * cols + c_base;
#pragma unroll
    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint2*>(qr + 8 * (4 * c + j4)) = quant_piece<MODE>(packed[it][c], s_tile);
  }
  // ---------------------------------------------------------------- phase B: rotation along the rows
  const int c = tid >> 1, h = tid & 1;
  float2 pv[32];   // pv[m] = rows 4m+2h, 4m+2h+1 of column c
#pragma unroll
  for (int m = 0; m < 32; ++m) {   // span 1 on the way in
    const uint8_t* p0 = s_raw + (4 * m + 2 * h) * LDB + 2 * c;
    const float a = bf16_bits_to_float(*reinterpret_cast<const uint16_t*>(p0));
    const float b = bf16_bits_to_float(*reinterpret_cast<const uint16_t*>(p0 + LDB));
    pv[m] = make_float2(__fadd_rn(a, b), __fsub_rn(a, b));
  }
  {   // span 2: the partner lane holds the rows with the other value of bit 1
    const float sg = h ? -1.f : 1.f;
    const float2 sg2 = make_float2(sg, sg);
#pragma unroll
    for (int m = 0; m < 32; ++m) {
      const float2 o = make_float2(__shfl_xor_sync(0xffffffffu, pv[m].x, 1), __shfl_xor_sync(0xffffffffu, pv[m].y, 1));
      pv[m] = __ffma2_rn(pv[m], sg2, o);   // own + partner, or partner - own
    }
  }
#pragma unroll
  for (int span = 1; span < 32; span <<= 1) {   // spans 4..64 of the rows = 1..16 of m
#pragma unroll
    for (int m = 0; m < 32; ++m) {
      if ((m & span) == 0) {
        const float2 a = pv[m], b = pv[m | span];
        pv[m] = add2(a, b);
        pv[m | span] = sub2(a, b);
      }
    }
  }
  uint32_t hv[32];
  __nv_bfloat162 hm = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
  for (int m = 0; m < 32; ++m) {
    const __nv_bfloat162 b2 = __floats2bfloat162_rn(pv[m].x, pv[m].y);
    hm = __hmax2(hm, __habs2(b2));
    hv[m] = *reinterpret_cast<const uint32_t*>(&b2);
  }
  float mt = fmaxf(__low2float(hm), __high2float(hm));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
  if (l == 0) s_red_t[w] = mt;
  __syncthreads();
  mt = s_red_t[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) mt = fmaxf(mt, s_red_t[k]);
  float st, stored_t;
  make_scale<MODE>(mt, st, stored_t);
  if (tid == 0) scale_t[((int64_t)blockIdx.z * (cols / 128) + blockIdx.x) * (rows / 128) + blockIdx.y] = stored_t;
  // quantize: byte pair m = (row 4m+2h, row 4m+2h+1) -> 16 bits; two pairs per 32-bit word
  uint32_t pw[16];   // pw[i] = pair 2i | pair 2i+1 << 16
  const float2 st2 = make_float2(st, st);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    int q0, q1, q2, q3;
    quant2<MODE>(make_float2(__uint_as_float(hv[2 * i] << 16), __uint_as_float(hv[2 * i] & 0xffff0000u)), st2, q0, q1);
    quant2<MODE>(make_float2(__uint_as_float(hv[2 * i + 1] << 16), __uint_as_float(hv[2 * i + 1] & 0xffff0000u)), st2, q2, q3);
    pw[i] = pack4(q0, q1, q2, q3);
  }
  // lane h keeps the pairs of m in [16h, 16h+16) and receives the partner's pairs of the same m: output
  // bytes 4m..4m+3 = (pair of lane 0, pair of lane 1)
  uint32_t outw[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t send = h ? pw[i] : pw[8 + i];          // what the partner needs from this lane
    const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 1);
    const uint32_t mine = h ? pw[8 + i] : pw[i];          // pairs 2i', 2i'+1 of the m range this lane writes
    const uint32_t lo = h ? got : mine, hi = h ? mine : got;   // lane 0's pairs go to bytes 0-1, lane 1's to bytes 2-3
    outw[2 * i] = __byte_perm(lo, hi, 0x5410);            // m = 2i':   lo.pair0 | hi.pair0 << 16
    outw[2 * i + 1] = __byte_perm(lo, hi, 0x7632);        // m = 2i'+1: lo.pair1 | hi.pair1 << 16
  }
  int8_t* out = qt + boff + (c_base + c) * rows + r_base + 64 * h;
#pragma unroll
  for (int i = 0; i < 16; i += 4)
    *reinterpret_cast<uint4*>(out + 4 * i) = make_uint4(outw[i], outw[i + 1], outw[i + 2], outw[i + 3]);
}

// Column absmax of x [rows, cols] into colmax[cols] (pre-zeroed); |x| >= 0 so the float bit
// patterns order like integers and atomicMax on int is exact.
__global__ void __launch_bounds__(256)
col_absmax_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols, float* __restrict__ colmax) {
  __shared__ float s_colred[8 * 128];
  const int tid = threadIdx.x, w = tid >> 5, l = tid & 31, cc = l & 15, half = l >> 4;
  const int64_t r_base = (int64_t)blockIdx.y * 128, c_base = (int64_t)blockIdx.x * 128;
  float m[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) m[j] = 0.f;
#pragma unroll
  for (int it = 0; it < 2; ++it)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 16 * w + 8 * it + 4 * half + i;
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(x + (r_base + r) * cols + c_base + 8 * cc));
      float v[8];
      unpack8(u, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) m[j] = fmaxf(m[j], fabsf(v[j]));
    }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    m[j] = fmaxf(m[j], __shfl_xor_sync(0xffffffffu, m[j], 16));
    if (half == 0) s_colred[w * 128 + 8 * cc + j] = m[j];
  }
  __syncthreads();
  if (tid < 128) {
    float mm = s_colred[tid];
#pragma unroll
    for (int k = 1; k < 8; ++k) mm = fmaxf(mm, s_colred[k * 128 + tid]);
    atomicMax(reinterpret_cast<int*>(colmax + c_base + tid), __float_as_int(mm));
  }
}

// ------------------------------------------------------------------------------------------------
// Row kernel: one CTA per row, two sweeps over the row (the second one hits L1/L2).
// HAD128: the 16 lanes that hold one 128-wide group rotate it with shuffles in both sweeps.
// ------------------------------------------------------------------------------------------------
template <int MODE, bool HAD128>
__global__ void __launch_bounds__(256)
quant_row_kernel(const __nv_bfloat16* __restrict__ x, int64_t cols, int8_t* __restrict__ q,
                 float* __restrict__ scale) {
  __shared__ float s_red[8];
  const int tid = threadIdx.x, l = tid & 31;
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
  const int nchunks = (int)(cols / 8);

  float m = 0.f;
  for (int base = 0; base < nchunks; base += 256) {
    const int ch = base + tid;
    float v[8];
    if (ch < nchunks) unpack8(__ldg(xr + ch), v);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    if (HAD128) {
      fwht128_lanes16(v, l);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = round_to_bf16(v[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(v[j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (l == 0) s_red[tid >> 5] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
  float s, stored;
  make_scale<MODE>(m, s, stored);
  if (tid == 0) scale[row] = stored;

  uint2* qr = reinterpret_cast<uint2*>(q + row * cols);
  for (int base = 0; base < nchunks; base += 256) {
    const int ch = base + tid;
    float v[8];
    if (ch < nchunks) unpack8(__ldg(xr + ch), v);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    if (HAD128) {
      fwht128_lanes16(v, l);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = round_to_bf16(v[j]);
    }
    if (ch < nchunks) {
      uint2 o;
      o.x = pack4(quant1<MODE>(v[0], s), quant1<MODE>(v[1], s), quant1<MODE>(v[2], s), quant1<MODE>(v[3], s));
      o.y = pack4(quant1<MODE>(v[4], s), quant1<MODE>(v[5], s), quant1<MODE>(v[6], s), quant1<MODE>(v[7], s));
      qr[ch] = o;
    }
  }
}

// Row kernel with the 128-point rotation for rows of at most 8192 elements: the rotated values (already
// rounded to bf16) stay in registers between the absmax sweep and the quantizing sweep, so the row is read
// and rotated once instead of twice.  Same arithmetic as quant_row_kernel<MODE, true>, bit for bit.
template <int MODE>
__global__ void __launch_bounds__(256)
quant_row_had128_cached_kernel(const __nv_bfloat16* __restrict__ x, int64_t cols, int8_t* __restrict__ q,
                               float* __restrict__ scale) {
  __shared__ float s_red[8];
  const int tid = threadIdx.x, l = tid & 31;
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
  const int nchunks = (int)(cols / 8);
  uint4 cache[4];
  __nv_bfloat162 hm = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int ch = it * 256 + tid;
    float v[8];
    if (ch < nchunks) unpack8(__ldg(xr + ch), v);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    fwht128_lanes16(v, l);   // whole warps take part: a 128-wide group never straddles the end of the row
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&cache[it]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
      hm = __hmax2(hm, __habs2(h[k]));
    }
  }
  float m = fmaxf(__low2float(hm), __high2float(hm));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (l == 0) s_red[tid >> 5] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
  float s, stored;
  make_scale<MODE>(m, s, stored);
  if (tid == 0) scale[row] = stored;
  uint2* qr = reinterpret_cast<uint2*>(q + row * cols);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int ch = it * 256 + tid;
    if (ch < nchunks) qr[ch] = quant_piece<MODE>(cache[it], s);
  }
}

// Whole-row Hadamard (power-of-two cols <= 32768): the row lives in shared memory as fp32.
// Spans 1..64 run in registers/shuffles exactly as above, spans >= 128 as shared-memory passes.
template <int MODE>
__global__ void __launch_bounds__(256)
quant_row_hadfull_kernel(const __nv_bfloat16* __restrict__ x, int64_t cols, int8_t* __restrict__ q,
                         float* __restrict__ scale) {
  extern __shared__ float s_row[];
  __shared__ float s_red[8];
  const int tid = threadIdx.x, l = tid & 31;
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
  const int n = (int)cols, nchunks = n / 8;

  for (int base = 0; base < nchunks; base += 256) {
    const int ch = base + tid;
    float v[8];
    if (ch < nchunks) unpack8(__ldg(xr + ch), v);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    fwht128_lanes16(v, l);
    if (ch < nchunks) {
      *reinterpret_cast<float4*>(s_row + 8 * ch) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(s_row + 8 * ch + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  __syncthreads();
  for (int h = 128; h < n; h <<= 1) {
    for (int p = tid; p < n / 2; p += 256) {
      const int i = ((p & ~(h - 1)) << 1) | (p & (h - 1));
      const float a = s_row[i], b = s_row[i + h];
      s_row[i] = __fadd_rn(a, b);
      s_row[i + h] = __fsub_rn(a, b);
    }
    __syncthreads();
  }
  float m = 0.f;
  for (int i = tid; i < n; i += 256) {
    const float r = round_to_bf16(s_row[i]);
    s_row[i] = r;
    m = fmaxf(m, fabsf(r));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (l == 0) s_red[tid >> 5] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, s_red[k]);
  float s, stored;
  make_scale<MODE>(m, s, stored);
  if (tid == 0) scale[row] = stored;
  uint32_t* qr = reinterpret_cast<uint32_t*>(q + row * cols);
  for (int i = tid; i < n / 4; i += 256) {
    const float4 f = *reinterpret_cast<const float4*>(s_row + 4 * i);
    qr[i] = pack4(quant1<MODE>(f.x, s), quant1<MODE>(f.y, s), quant1<MODE>(f.z, s), quant1<MODE>(f.w, s));
  }
}

// ------------------------------------------------------------------------------------------------ host
constexpr int MAX_DEVICES = 64;
static int device_ordinal() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev < 0 || dev >= MAX_DEVICES) ? 0 : dev;
}
// Raises a kernel's dynamic shared-memory limit once per device (function attributes are per device;
// the call is idempotent, so two threads racing here only repeat it).
template <typename Kernel>
static cudaError_t ensure_smem(Kernel kernel, std::atomic<bool>* done_per_device, size_t bytes) {
  std::atomic<bool>& done = done_per_device[device_ordinal()];
  if (done.load(std::memory_order_acquire)) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) done.store(true, std::memory_order_release);
  return e;
}

static int check_dims(int64_t batch, int64_t rows, int64_t cols) {
  if (batch <= 0 || rows <= 0 || cols <= 0 || rows % 128 || cols % 128)
    return fail(I8L_ERR_SHAPE, "batch=%lld rows=%lld cols=%lld: all must be positive and rows, cols multiples of 128",
                (long long)batch, (long long)rows, (long long)cols);
  if (batch > 65535 || rows / 128 > 65535 || rows * cols >= (1ll << 40))
    return fail(I8L_ERR_SHAPE, "shape too large for the launch grid");
  return I8L_OK;
}

template <int GRAN, int MODE, bool HAD, bool OUT_N, bool OUT_T>
static void launch_tile(const void* x, int64_t batch, int64_t rows, int64_t cols, int8_t* q, float* scale,
                        int8_t* qt, float* scale_t, const float* colmax, cudaStream_t st) {
  dim3 grid((unsigned)(cols / 128), (unsigned)(rows / 128), (unsigned)batch);
  quant_tile_kernel<GRAN, MODE, HAD, OUT_N, OUT_T><<<grid, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), rows, cols, q, scale, qt, scale_t, colmax);
}

template <int GRAN, int MODE>
static int dispatch_tile(const void* x, int64_t batch, int64_t rows, int64_t cols, bool had, int8_t* q,
                         float* scale, int8_t* qt, float* scale_t, const float* colmax, cudaStream_t st) {
  const bool n = q != nullptr, t = qt != nullptr;
  if (had && n && t && GRAN == I8L_GRAN_TILE128) {  // both rotated operands from one read of the tile
    dim3 grid((unsigned)(cols / 128), (unsigned)(rows / 128), (unsigned)batch);
    quant_tile_had_dual_kernel<MODE><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, q, scale, qt, scale_t);
  } else if (had) {  // the two orientations rotate along different axes: one launch each
    if (n) {
      dim3 grid((unsigned)(cols / 128), (unsigned)(rows / 128), (unsigned)batch);
      quant_tile_hadcols_kernel<GRAN, MODE><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, q, scale);
    }
    if (t) {
      constexpr size_t smem = 128 * 132 * sizeof(float);
      static std::atomic<bool> attr_done[MAX_DEVICES];
      I8L_CUDA_OK(ensure_smem(quant_tile_hadrows_kernel<GRAN, MODE>, attr_done, smem));
      dim3 grid((unsigned)(cols / 128), (unsigned)(rows / 128), (unsigned)batch);
      quant_tile_hadrows_kernel<GRAN, MODE><<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, qt, scale_t, nullptr);
    }
  } else if (GRAN == I8L_GRAN_TILE128) {
    if (n && t) launch_tile<GRAN, MODE, false, true, true>(x, batch, rows, cols, q, scale, qt, scale_t, colmax, st);
    else if (n) launch_tile<GRAN, MODE, false, true, false>(x, batch, rows, cols, q, scale, qt, scale_t, colmax, st);
    else launch_tile<GRAN, MODE, false, false, true>(x, batch, rows, cols, q, scale, qt, scale_t, colmax, st);
  } else {  // grouped scales differ between the two orientations: one launch each
    if (n) launch_tile<GRAN, MODE, false, true, false>(x, batch, rows, cols, q, scale, nullptr, nullptr, colmax, st);
    if (t) launch_tile<GRAN, MODE, false, false, true>(x, batch, rows, cols, nullptr, nullptr, qt, scale_t, colmax, st);
  }
  I8L_CUDA_OK(cudaGetLastError());
  return I8L_OK;
}

}  // namespace i8l

using namespace i8l;

extern "C" const char* i8l_last_error(void) { return g_err; }
extern "C" int i8l_version(void) { return 100; }

extern "C" int i8l_quant_tile(const void* x, int64_t batch, int64_t rows, int64_t cols, int gran, int qmode,
                              int hadamard, int8_t* q, float* scale, int8_t* qt, float* scale_t, void* stream) {
  if (int e = check_dims(batch, rows, cols)) return e;
  if (!x || (!q && !qt) || (q && !scale) || (qt && !scale_t)) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(x) || !aligned16(q) || !aligned16(qt)) return fail(I8L_ERR_ALIGN, "x, q, qt must be 16-byte aligned");
  if (hadamard != I8L_HAD_NONE && hadamard != I8L_HAD_128)
    return fail(I8L_ERR_ARG, "i8l_quant_tile: hadamard must be NONE or 128");
  if (int e = check_arch()) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool had = hadamard == I8L_HAD_128;
  if (gran == I8L_GRAN_TILE128X256) {
    if (cols % 256 || had || qt || !q) return fail(I8L_ERR_ARG, "i8l_quant_tile: 128x256 groups need cols %% 256 == 0, no rotation, q only");
    const dim3 grid((unsigned)(cols / 256), (unsigned)(rows / 128), (unsigned)batch);
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
    if (qmode == I8L_QMODE_TRITON) quant_tile256_kernel<I8L_QMODE_TRITON><<<grid, 256, 0, st>>>(xp, rows, cols, q, scale);
    else if (qmode == I8L_QMODE_TRITON_BF16S) quant_tile256_kernel<I8L_QMODE_TRITON_BF16S><<<grid, 256, 0, st>>>(xp, rows, cols, q, scale);
    else return fail(I8L_ERR_ARG, "i8l_quant_tile: 128x256 groups support qmode TRITON and TRITON_BF16S");
    I8L_CUDA_OK(cudaGetLastError());
    return I8L_OK;
  }
#define I8L_TILE_CASE(G, Mo) \
  if (gran == G && qmode == Mo) return dispatch_tile<G, Mo>(x, batch, rows, cols, had, q, scale, qt, scale_t, nullptr, st);
  I8L_TILE_CASE(I8L_GRAN_TILE128, I8L_QMODE_TRITON)
  I8L_TILE_CASE(I8L_GRAN_TILE128, I8L_QMODE_RNE)
  I8L_TILE_CASE(I8L_GRAN_TILE128, I8L_QMODE_FUSED)
  I8L_TILE_CASE(I8L_GRAN_GROUP128, I8L_QMODE_TRITON)
  I8L_TILE_CASE(I8L_GRAN_GROUP128, I8L_QMODE_RNE)
  I8L_TILE_CASE(I8L_GRAN_GROUP128, I8L_QMODE_FUSED)
#undef I8L_TILE_CASE
  return fail(I8L_ERR_ARG, "i8l_quant_tile: unsupported gran=%d qmode=%d", gran, qmode);
}

extern "C" int i8l_quant_row(const void* x, int64_t rows, int64_t cols, int qmode, int hadamard, int8_t* q,
                             float* scale, void* stream) {
  if (rows <= 0 || cols <= 0 || cols % 128 || rows > 0x7fffffffll || cols > (1 << 20))
    return fail(I8L_ERR_SHAPE, "rows=%lld cols=%lld: need rows>0, cols a positive multiple of 128",
                (long long)rows, (long long)cols);
  if (!x || !q || !scale) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(x) || !aligned16(q)) return fail(I8L_ERR_ALIGN, "x, q must be 16-byte aligned");
  if (int e = check_arch()) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  if (hadamard == I8L_HAD_FULL) {
    if ((cols & (cols - 1)) || cols > 32768)
      return fail(I8L_ERR_SHAPE, "full Hadamard needs cols a power of two <= 32768, got %lld", (long long)cols);
    const size_t smem = (size_t)cols * sizeof(float);
#define I8L_HF_CASE(Mo)                                                                                        \
  if (qmode == Mo) {                                                                                           \
    I8L_CUDA_OK(cudaFuncSetAttribute(quant_row_hadfull_kernel<Mo>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                     (int)smem));                                                              \
    quant_row_hadfull_kernel<Mo><<<(unsigned)rows, 256, smem, st>>>(xp, cols, q, scale);                       \
    I8L_CUDA_OK(cudaGetLastError());                                                                           \
    return I8L_OK;                                                                                             \
  }
    I8L_HF_CASE(I8L_QMODE_TRITON)
    I8L_HF_CASE(I8L_QMODE_RNE)
    I8L_HF_CASE(I8L_QMODE_ROWRCP)
#undef I8L_HF_CASE
    return fail(I8L_ERR_ARG, "i8l_quant_row: unsupported qmode=%d", qmode);
  }
  if (hadamard != I8L_HAD_NONE && hadamard != I8L_HAD_128) return fail(I8L_ERR_ARG, "bad hadamard=%d", hadamard);
#define I8L_ROW_CASE(Mo)                                                                              \
  if (qmode == Mo) {                                                                                  \
    if (hadamard && cols <= 8192) quant_row_had128_cached_kernel<Mo><<<(unsigned)rows, 256, 0, st>>>(xp, cols, q, scale); \
    else if (hadamard) quant_row_kernel<Mo, true><<<(unsigned)rows, 256, 0, st>>>(xp, cols, q, scale);     \
    else quant_row_kernel<Mo, false><<<(unsigned)rows, 256, 0, st>>>(xp, cols, q, scale);             \
    I8L_CUDA_OK(cudaGetLastError());                                                                  \
    return I8L_OK;                                                                                    \
  }
  I8L_ROW_CASE(I8L_QMODE_TRITON)
  I8L_ROW_CASE(I8L_QMODE_RNE)
  I8L_ROW_CASE(I8L_QMODE_ROWRCP)
  I8L_ROW_CASE(I8L_QMODE_TRITON_BF16S)
#undef I8L_ROW_CASE
  return fail(I8L_ERR_ARG, "i8l_quant_row: unsupported qmode=%d", qmode);
}

extern "C" int i8l_quant_col_t(const void* x, int64_t rows, int64_t cols, int qmode, int8_t* qt, float* scale_t,
                               float* colmax_scratch, void* stream) {
  if (int e = check_dims(1, rows, cols)) return e;
  if (!x || !qt || !scale_t || !colmax_scratch) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(x) || !aligned16(qt)) return fail(I8L_ERR_ALIGN, "x, qt must be 16-byte aligned");
  if (int e = check_arch()) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  I8L_CUDA_OK(cudaMemsetAsync(colmax_scratch, 0, (size_t)cols * sizeof(float), st));
  dim3 grid((unsigned)(cols / 128), (unsigned)(rows / 128), 1);
  col_absmax_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, colmax_scratch);
  I8L_CUDA_OK(cudaGetLastError());
#define I8L_COL_CASE(Mo)                                                                                     \
  if (qmode == Mo) {                                                                                         \
    launch_tile<GRAN_COLFULL, Mo, false, false, true>(x, 1, rows, cols, nullptr, nullptr, qt, scale_t,       \
                                                      colmax_scratch, st);                                   \
    I8L_CUDA_OK(cudaGetLastError());                                                                         \
    return I8L_OK;                                                                                           \
  }
  I8L_COL_CASE(I8L_QMODE_TRITON)
  I8L_COL_CASE(I8L_QMODE_RNE)
  I8L_COL_CASE(I8L_QMODE_ROWRCP)
#undef I8L_COL_CASE
  return fail(I8L_ERR_ARG, "i8l_quant_col_t: unsupported qmode=%d", qmode);
}

template <int MODE>
static int launch_col_t_rot(const void* x, int64_t rows, int64_t cols, int8_t* qt, float* scale_t, float* colmax,
                            cudaStream_t st) {
  constexpr size_t smem = 128 * 132 * sizeof(float);
  static std::atomic<bool> attr_done_pass[MAX_DEVICES], attr_done_full[MAX_DEVICES];
  I8L_CUDA_OK(ensure_smem(quant_tile_hadrows_kernel<GRAN_COLMAX_PASS, MODE>, attr_done_pass, smem));
  I8L_CUDA_OK(ensure_smem(quant_tile_hadrows_kernel<GRAN_COLFULL, MODE>, attr_done_full, smem));
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  dim3 grid((unsigned)(cols / 128), (unsigned)(rows / 128), 1);
  quant_tile_hadrows_kernel<GRAN_COLMAX_PASS, MODE><<<grid, 256, smem, st>>>(xp, rows, cols, nullptr, nullptr, colmax);
  quant_tile_hadrows_kernel<GRAN_COLFULL, MODE><<<grid, 256, smem, st>>>(xp, rows, cols, qt, scale_t, colmax);
  I8L_CUDA_OK(cudaGetLastError());
  return I8L_OK;
}

extern "C" int i8l_quant_col_t_rot(const void* x, int64_t rows, int64_t cols, int qmode, int8_t* qt, float* scale_t,
                                   float* colmax_scratch, void* stream) {
  if (int e = check_dims(1, rows, cols)) return e;
  if (!x || !qt || !scale_t || !colmax_scratch) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(x) || !aligned16(qt)) return fail(I8L_ERR_ALIGN, "x, qt must be 16-byte aligned");
  if (int e = check_arch()) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  I8L_CUDA_OK(cudaMemsetAsync(colmax_scratch, 0, (size_t)cols * sizeof(float), st));
  if (qmode == I8L_QMODE_TRITON) return launch_col_t_rot<I8L_QMODE_TRITON>(x, rows, cols, qt, scale_t, colmax_scratch, st);
  if (qmode == I8L_QMODE_RNE) return launch_col_t_rot<I8L_QMODE_RNE>(x, rows, cols, qt, scale_t, colmax_scratch, st);
  if (qmode == I8L_QMODE_ROWRCP) return launch_col_t_rot<I8L_QMODE_ROWRCP>(x, rows, cols, qt, scale_t, colmax_scratch, st);
  return fail(I8L_ERR_ARG, "i8l_quant_col_t_rot: unsupported qmode=%d", qmode);
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of i8l_quant_col_t: the column-absmax scratch lives in a file-scope device
// array instead of caller memory.  In host code `g_colmax_static` is only a stand-in symbol, not a
// device address; the real address is looked up once per device with cudaGetSymbolAddress (with
// that device current) and cached.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_colmax_static[I8L_STATIC_SCRATCH_MAX_COLS];
static std::atomic<float*> g_colmax_static_addr[MAX_DEVICES];  // per device ordinal, nullptr = not looked up yet

extern "C" int i8l_quant_col_t_static(const void* x, int64_t rows, int64_t cols, int qmode, int8_t* qt,
                                      float* scale_t, void* stream) {
  if (cols > I8L_STATIC_SCRATCH_MAX_COLS)
    return fail(I8L_ERR_SHAPE, "i8l_quant_col_t_static: cols=%lld exceeds the built-in scratch of %d columns; "
                "use i8l_quant_col_t with caller-provided scratch", (long long)cols, I8L_STATIC_SCRATCH_MAX_COLS);
  // the same argument and device checks as i8l_quant_col_t, before the symbol query
  if (int e = check_dims(1, rows, cols)) return e;
  if (!x || !qt || !scale_t) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(x) || !aligned16(qt)) return fail(I8L_ERR_ALIGN, "x, qt must be 16-byte aligned");
  if (int e = check_arch()) return e;
  int dev = 0;
  I8L_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return fail(I8L_ERR_ARG, "device ordinal %d out of range", dev);
  float* ptr = g_colmax_static_addr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    I8L_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colmax_static));
    g_colmax_static_addr[dev].store(ptr, std::memory_order_release);
  }
  return i8l_quant_col_t(x, rows, cols, qmode, qt, scale_t, ptr, stream);
}
