// Single-kernel fused INT8 GEMM: bf16 operands in, bf16 (or fp32) result out, nothing quantized ever
// reaches global memory.  This is the structure of the reference's fused variant
// (triton/fused_triton_fwd32.py:23-69, triton/fused_triton_bwd33.py:24-61): every CTA re-derives the
// scale of each operand tile it consumes and quantizes it on the fly, per 128-wide K step.
//
// One persistent CTA per SM, 640 threads, tile 128 x 128, K step 128:
//   warp 0       TMA producer: the bf16 A tile (128 x 128) and B tile (128 x 128) of every K step into a two-slot
//                staging ring in shared memory (unswizzled 256-byte rows), so the loads run ahead of the math.
//   warp 1       tcgen05.mma kind::i8 issuer (M = 128, N = 128, K = 32, four per stage), accumulators alternate
//                between two 128-column tensor-memory buffers per K step, tcgen05.commit frees the stage.
//   warps 4-19   sixteen worker warps that each do both remaining jobs, one K step apart.  Transform: read a
//                share of the staged tiles (16-byte vectors, 16 lanes per row) into registers and give the
//                staging slot back at once; absmax per A tile and per B row (forward) or per B tile
//                (backward), scale = 127 / (amax + 1e-5), q = floor(x * scale + 0.5), int8 written into the
//                K-major 128B-swizzled shared-memory stage the tensor core reads, fence.proxy.async and an
//                arrival on the stage's "full" barrier; the step's factors go to a small ring in shared
//                memory.  Drain: the int32 partial product of the PREVIOUS step (its MMAs ran meanwhile) leaves
//                tensor memory, acc += P / (s_a * s_b[n]) (a multiplication by the rounded reciprocal unless
//                the reference operation order is asked for); after the last step the final cast and store.
// The integers and scales are those of quantizing each operand once (i8l_quant_tile with I8L_QMODE_FUSED)
// and running i8l_gemm_block with I8L_GEMM_DIVIDE; this kernel repeats the quantization N/128 (A) and M/128
// (B) times like the reference does, so it is the slower of the two on large shapes and exists for callers
// that want the reference's single-launch, no-intermediate form.
//
// Every mbarrier wait is bounded; the worker warps meet at a named barrier each step, so after a timeout
// they keep stepping through their loops without loading, waiting or arriving, and the kernel terminates.
#include <atomic>

#include "common.cuh"
#include "ptx.cuh"

namespace i8l {
namespace fusedk {

constexpr int TM = 128, TN = 128, TK = 128;
constexpr int NS = 2;                       // int8 stages: 16 KB A + 16 KB B each
constexpr int NB = 2;                       // bf16 staging slots: 32 KB A + 32 KB B each
constexpr int STAGE_A = TM * TK, STAGE_B = TN * TK;
constexpr int BF_A = TM * TK * 2, BF_B = TN * TK * 2;
constexpr int RING = 8;                     // scale ring entries (a step's scales live until its drain)
constexpr int THREADS = 640;
constexpr int WORKERS = 512;              // warps 4-19: each quantizes a share of every step and drains a share of the accumulator
constexpr int SMEM_DYN = NS * (STAGE_A + STAGE_B) + NB * (BF_A + BF_B) + 1024;
constexpr int TMEM_COLS = 256;
constexpr int BAR_XF = 9;                   // named barrier of the transform warps
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
constexpr uint32_t MAGIC_I = 0x4B400000u;
constexpr float MAGIC_F = 12582912.f;

struct Params {
  void* c;
  int32_t* status;
  int64_t K;
  int m_blocks, mpb, n_tiles, N, KB;
  int b_batched, per_row_b, exact, out_f32;
  uint32_t max_polls;
};

struct __align__(8) Ctl {
  uint64_t full[NS], empty[NS], bfull[NB], bempty[NB], tfull[2], tempty[2], done;
  uint32_t tmem_base;
  int abort_flag;
  float red_a[2][16], red_b[2][16]; // per-warp absmax partials, double buffered over the K steps
  float sa[RING];                   // A tile multiplier of the step (reference order only)
  float colv[RING][TN];             // per output column: 1 / (s_a * s_b[n]), or s_b[n] for the reference order
};

__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint2 v) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
fused_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Ctl ctl;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = smem_base, smem_b = smem_base + NS * STAGE_A;
  const uint32_t smem_bfa = smem_base + NS * (STAGE_A + STAGE_B), smem_bfb = smem_bfa + NB * BF_A;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&ctl.full[s]), WORKERS);
      mbar_init(smem_u32(&ctl.empty[s]), 1);
    }
    for (int s = 0; s < NB; ++s) {
      mbar_init(smem_u32(&ctl.bfull[s]), 1);
      mbar_init(smem_u32(&ctl.bempty[s]), WORKERS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl.tfull[b]), 1);
      mbar_init(smem_u32(&ctl.tempty[b]), WORKERS);
    }
    mbar_init(smem_u32(&ctl.done), 1);
    ctl.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;
  const int total_tiles = p.m_blocks * p.n_tiles;
  const int KB = p.KB;

  if (warp < 4) {
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer (bf16 staging)
      int s = 0;
      uint32_t ph = 0, issued = 0, issued_ph = 0;   // bit s: a load into slot s is (or was) in flight, with parity
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m_blk = t % p.m_blocks, n_tile = t / p.m_blocks;
        const int a_row = m_blk * TM;
        const int b_row = (p.b_batched ? (m_blk / p.mpb) * p.N : 0) + n_tile * TN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!(ok = mbar_wait(smem_u32(&ctl.bempty[s]), ph ^ 1u, abort_flag, p.max_polls))) break;
          if (lane == 0) {
            const uint32_t bar = smem_u32(&ctl.bfull[s]);
            mbar_expect_tx(bar, BF_A + BF_B);
            tma_load_2d(smem_bfa + s * BF_A, &map_a, bar, kb * TK, a_row);
            tma_load_2d(smem_bfb + s * BF_B, &map_b, bar, kb * TK, b_row);
          }
          issued |= 1u << s;
          issued_ph = (issued_ph & ~(1u << s)) | (ph << s);
          if (++s == NB) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {   // let copies already in flight land before the CTA's shared memory is released
        for (int k = 0; k < NB; ++k)
          if (issued & (1u << k)) {
            int dummy = 0;
            mbar_wait(smem_u32(&ctl.bfull[k]), (issued_ph >> k) & 1u, &dummy, 1u << 15);
          }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      int s = 0, ab = 0;
      uint32_t ph = 0, aph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb) {
          if (!(ok = mbar_wait(smem_u32(&ctl.full[s]), ph, abort_flag, p.max_polls))) break;
          if (!(ok = mbar_wait(smem_u32(&ctl.tempty[ab]), aph ^ 1u, abort_flag, p.max_polls))) break;
          tc_fence_after();
          if (lane == 0) {
            const uint64_t da = smem_desc(smem_a + s * STAGE_A), db = smem_desc(smem_b + s * STAGE_B);
            const uint32_t d = tmem_base + ab * TN;
#pragma unroll
            for (int k4 = 0; k4 < TK / 32; ++k4) tc_mma_i8(d, da + 2 * k4, db + 2 * k4, IDESC, k4 > 0 ? 1u : 0u);
            tc_commit(smem_u32(&ctl.empty[s]));
            tc_commit(smem_u32(&ctl.tfull[ab]));
          }
          __syncwarp();
          ab ^= 1;
          if (ab == 0) aph ^= 1u;
          if (++s == NS) { s = 0; ph ^= 1u; }
        }
      }
      if (lane == 0) tc_commit(smem_u32(&ctl.done));   // all MMAs issued here have retired before tensor memory is freed
      __syncwarp();
      int dummy = 0;
      mbar_wait(smem_u32(&ctl.done), 0, &dummy);
    }
  } else {
    // -------------------------------------------------------------------- 16 worker warps (512 threads)
    // Every worker does both jobs, one K step apart: quantize its share of step j's tiles into the tensor
    // core's stage, then drain its share of step j-1's accumulator (whose MMAs ran while step j was being
    // quantized).  Transform share: warp xw holds rows 8xw..8xw+7 of both tiles, 16 lanes per 256-byte row.
    // Accumulator share: warp % 4 selects the 32 tensor-memory lanes (rows), (warp - 4) / 4 the 32 columns.
    // No early exit: the warps meet at a named barrier every step, so after a timeout they run through the
    // remaining steps without loading, waiting or arriving.
    const int xw = warp - 4, cc = lane & 15, half = lane >> 4, xtid = xw * 32 + lane;
    const int q = warp & 3, cg = xw >> 2;
    const int tix = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    int s = 0, sb = 0;
    uint32_t ph = 0, bph = 0, step = 0;
    bool ok = true;
    float2 acc[16];

    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int m_blk = t % p.m_blocks, n_tile = t / p.m_blocks;
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = make_float2(0.f, 0.f);
      for (int kb = 0; kb <= KB; ++kb) {
       if (kb < KB) {
        // ---- transform step `step`
        uint4 ra[4], rb[4];
        float rowmax[4];
        ok = ok && mbar_wait(smem_u32(&ctl.bfull[sb]), bph, abort_flag, p.max_polls);   // the step's bf16 tiles have landed
        if (ok) {
          const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
          __nv_bfloat162 ma = zero2, mbt = zero2;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = 8 * xw + 4 * half + i;
            ra[i] = *reinterpret_cast<const uint4*>(smem_raw + (smem_bfa - smem_u32(smem_raw)) + sb * BF_A + r * 256 + 16 * cc);
            rb[i] = *reinterpret_cast<const uint4*>(smem_raw + (smem_bfb - smem_u32(smem_raw)) + sb * BF_B + r * 256 + 16 * cc);
          }
          mbar_arrive(smem_u32(&ctl.bempty[sb]));   // the tiles are in registers: the slot can be refilled
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra[i]);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb[i]);
            __nv_bfloat162 mrow = zero2;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              ma = __hmax2(ma, __habs2(ha[k]));
              mrow = __hmax2(mrow, __habs2(hb[k]));
            }
            mbt = __hmax2(mbt, mrow);
            float m = fmaxf(__low2float(mrow), __high2float(mrow));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));   // the row's 16 lanes
            rowmax[i] = m;
          }
          float am = fmaxf(__low2float(ma), __high2float(ma)), bm = fmaxf(__low2float(mbt), __high2float(mbt));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
          }
          if (lane == 0) {
            ctl.red_a[step & 1][xw] = am;
            ctl.red_b[step & 1][xw] = bm;
          }
        }
        named_sync(BAR_XF, WORKERS);
        if (ok) {
          float am = ctl.red_a[step & 1][0], bm = ctl.red_b[step & 1][0];
#pragma unroll
          for (int k = 1; k < 16; ++k) {
            am = fmaxf(am, ctl.red_a[step & 1][k]);
            bm = fmaxf(bm, ctl.red_b[step & 1][k]);
          }
          float s_a, s_bt, unused;
          make_scale<I8L_QMODE_FUSED>(am, s_a, unused);
          make_scale<I8L_QMODE_FUSED>(bm, s_bt, unused);
          ok = mbar_wait(smem_u32(&ctl.empty[s]), ph ^ 1u, abort_flag, p.max_polls);   // the int8 stage is free again
          if (ok) {
            const int e = step & (RING - 1);
            const uint32_t sa_addr = smem_a + s * STAGE_A, sb_addr = smem_b + s * STAGE_B;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = 8 * xw + 4 * half + i;
              float s_b = s_bt;
              if (p.per_row_b) make_scale<I8L_QMODE_FUSED>(rowmax[i], s_b, unused);
              // K-major, 128-byte rows, 8-row groups of 1024 bytes, 16-byte chunks XOR-swizzled with the row
              const uint32_t off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((((cc >> 1) ^ (r & 7))) << 4) + (cc & 1) * 8);
              st_shared_v2(sa_addr + off, quant_piece<I8L_QMODE_FUSED>(ra[i], s_a));
              st_shared_v2(sb_addr + off, quant_piece<I8L_QMODE_FUSED>(rb[i], s_b));
              if (p.per_row_b && cc == 0)
                ctl.colv[e][r] = p.exact ? s_b : __frcp_rn(__fmul_rn(s_a, s_b));
            }
            if (!p.per_row_b && xtid < TN) ctl.colv[e][xtid] = p.exact ? s_bt : __frcp_rn(__fmul_rn(s_a, s_bt));
            if (xtid == 0) ctl.sa[e] = s_a;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads what was just stored
            mbar_arrive(smem_u32(&ctl.full[s]));
          }
        }
        if (++s == NS) { s = 0; ph ^= 1u; }
        if (++sb == NB) { sb = 0; bph ^= 1u; }
        ++step;
       } else {
        named_sync(BAR_XF, WORKERS);   // the last step's factors (written after its barrier) are visible to every drainer
       }
       // ---- drain the previous step (its MMAs ran while the step above was being quantized): acc += P / (s_a * s_b[n]).
       // Its factors were written after the barrier of that step and are read after the barrier of this one; a
       // ring entry is rewritten eight steps later.
       if (kb > 0) {
        const uint32_t dstep = step - (kb < KB ? 2u : 1u);
        const int e = dstep & (RING - 1), ab = dstep & 1;
        ok = ok && mbar_wait(smem_u32(&ctl.tfull[ab]), (dstep >> 1) & 1u, abort_flag, p.max_polls);
        if (ok) {
          tc_fence_after();
          const uint32_t taddr = tmem_base + lane_addr + ab * TN + cg * 32;
          const float* colv = ctl.colv[e] + cg * 32;
          const float sa = ctl.sa[e];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[8];
            tc_ld8(taddr + c * 8, r);
            tc_ld_wait();
            if (c == 3) {   // all of this thread's loads of the buffer have completed
              tc_fence_before();
              mbar_arrive(smem_u32(&ctl.tempty[ab]));
            }
            if (p.exact) {   // acc += float(P) / (s_a * s_b[n]), unfused: triton/fused_triton_fwd32.py:65
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float t0 = __fdiv_rn(__int2float_rn((int)r[2 * j]), __fmul_rn(sa, colv[c * 8 + 2 * j]));
                const float t1 = __fdiv_rn(__int2float_rn((int)r[2 * j + 1]), __fmul_rn(sa, colv[c * 8 + 2 * j + 1]));
                acc[c * 4 + j] = make_float2(__fadd_rn(acc[c * 4 + j].x, t0), __fadd_rn(acc[c * 4 + j].y, t1));
              }
            } else {
              const float2* f2 = reinterpret_cast<const float2*>(colv + c * 8);
              if (c & 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  acc[c * 4 + j] = __ffma2_rn(make_float2(__int2float_rn((int)r[2 * j]), __int2float_rn((int)r[2 * j + 1])), f2[j], acc[c * 4 + j]);
              } else {   // the same float(P) through an integer add and a packed subtract: balances the two pipes
                const float2 nm = make_float2(-MAGIC_F, -MAGIC_F);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 v = __fadd2_rn(make_float2(__uint_as_float(MAGIC_I + r[2 * j]), __uint_as_float(MAGIC_I + r[2 * j + 1])), nm);
                  acc[c * 4 + j] = __ffma2_rn(v, f2[j], acc[c * 4 + j]);
                }
              }
            }
          }
        }
       }
      }
      if (ok) {
        const int64_t row = (int64_t)m_blk * TM + tix;
        const int col0 = n_tile * TN + cg * 32;
        if (p.out_f32) {
          float* o = static_cast<float*>(p.c) + row * p.N + col0;
#pragma unroll
          for (int j = 0; j < 16; j += 2)
            *reinterpret_cast<float4*>(o + 2 * j) = make_float4(acc[j].x, acc[j].y, acc[j + 1].x, acc[j + 1].y);
        } else {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.c) + row * p.N + col0;
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(acc[j + k].x, acc[j + k].y);
              w[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && ctl.abort_flag && p.status) atomicExch(p.status, I8L_ERR_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace fusedk
}  // namespace i8l

using namespace i8l;

extern "C" int i8l_fused_gemm(const void* a_bf, const void* b_bf, void* c, int64_t batch, int64_t M, int64_t N, int64_t K,
                              int b_batched, int flags, int32_t* status, void* stream) {
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128)
    return fail(I8L_ERR_SHAPE, "batch=%lld M=%lld N=%lld K=%lld: all positive, M, N, K multiples of 128",
                (long long)batch, (long long)M, (long long)N, (long long)K);
  if (batch * M >= (1ll << 31) || batch * N >= (1ll << 31) || (batch * M / 128) * (N / 128) >= (1ll << 31))
    return fail(I8L_ERR_SHAPE, "problem too large for 32-bit tile coordinates");
  if (!a_bf || !b_bf || !c) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(a_bf) || !aligned16(b_bf) || !aligned16(c)) return fail(I8L_ERR_ALIGN, "a, b, c must be 16-byte aligned");
  if (flags & ~(I8L_GEMM_EXACT_ORDER | I8L_GEMM_OUT_F32)) return fail(I8L_ERR_ARG, "i8l_fused_gemm: flags may hold EXACT_ORDER and OUT_F32");
  if (int e = check_arch()) return e;
  fusedk::Params p{};
  CUtensorMap map_a, map_b;
  if (int e = make_tile_map_bf16(&map_a, a_bf, batch * M, K)) return e;
  if (int e = make_tile_map_bf16(&map_b, b_bf, b_batched ? batch * N : N, K)) return e;
  p.c = c;
  p.status = status;
  p.K = K;
  p.m_blocks = (int)(batch * M / 128);
  p.mpb = (int)(M / 128);
  p.n_tiles = (int)(N / 128);
  p.N = (int)N;
  p.KB = (int)(K / 128);
  p.b_batched = b_batched ? 1 : 0;
  p.per_row_b = b_batched ? 0 : 1;   // forward: B scale per (row, K step); backward: per tile
  p.exact = (flags & I8L_GEMM_EXACT_ORDER) ? 1 : 0;
  p.out_f32 = (flags & I8L_GEMM_OUT_F32) ? 1 : 0;
  p.max_polls = gemm_wait_limit();
  static std::atomic<bool> attr_done[64];
  int dev = 0;
  I8L_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_done[dev].load(std::memory_order_acquire)) {
    I8L_CUDA_OK(cudaFuncSetAttribute(fusedk::fused_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fusedk::SMEM_DYN));
    attr_done[dev].store(true, std::memory_order_release);
  }
  const int64_t tiles = (int64_t)p.m_blocks * p.n_tiles;
  const int ctas = gemm_cta_budget();
  const int grid = (int)(tiles < ctas ? tiles : ctas);
  fusedk::fused_gemm_kernel<<<grid, fusedk::THREADS, fusedk::SMEM_DYN, static_cast<cudaStream_t>(stream)>>>(map_a, map_b, p);
  I8L_CUDA_OK(cudaGetLastError());
  return I8L_OK;
}
