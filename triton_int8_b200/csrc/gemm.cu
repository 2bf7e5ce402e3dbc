// INT8 GEMMs on the 5th-generation tensor cores: tcgen05.mma kind::i8 with int32 accumulators in
// tensor memory, operands staged by TMA into a 128B-swizzled shared-memory ring.
//
// One persistent CTA per SM, 640 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      tensor-memory allocator + MMA issuer (one elected lane)
//   warp 2      factor warp (fast block-scaled kind): prepares, one tile ahead, the signed per-K-block
//               factors and the column scales the epilogue needs; idle in the other kinds
//   warp 3      idle (completes the first warpgroup so register budgets can be rebalanced)
//   warps 4-19  epilogue: warp%4 selects the 32 accumulator lanes (rows) a warp may read, the
//               group of four warps selects 64 of the 256 columns of the 128x256 tile.  Sixteen
//               warps (four per scheduler) because the per-K-block drain is bound by instruction
//               latency, not by a pipe: more resident warps hide it.
// Tensor memory holds two 128x256 int32 accumulators (all 512 columns).  In block-scaled mode the
// MMA warp alternates between them every 128-wide K block while the epilogue drains the other one
// into fp32 registers (acc += float(P) * scale; in the fast kind float(P) is formed by an integer add of
// a magic number whose multiple is kept bounded by alternating signs and removed at the tile end); in
// row x column mode a buffer holds a whole tile and the epilogue of tile i overlaps the main loop of tile i+1.
//
// Every wait on an mbarrier is bounded (a poll count worth about two seconds); on expiry the CTA raises
// a shared abort flag and reports through the status word.  The producer and the MMA issuer then leave
// their loops; the epilogue warps run through their remaining tiles without waiting, computing or
// storing; copies in flight are awaited, so the kernel always terminates and frees its tensor memory.
//
// Scatter mode (i8l_gemm_block_scatter): the epilogue writes each 128-row block into a slot of a
// buffer owned by another GPU (plain stores to peer-mapped memory), for a reduce-scatter without a
// separate collective kernel.
#include <cuda.h>

#include <atomic>
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace i8l {

constexpr int BM = 128, BN = 256, BK = 128;
#ifndef I8L_STAGES
#define I8L_STAGES 4
#endif
constexpr int A_STAGE = BM * BK;  // bytes
// One CTA per tile: 128x256 tile, 4 stages of 16 KB (A) + 32 KB (B).
// CTA pair per tile (cta_group::2): 256x256 tile, each CTA stages its own 128 rows of A and 128 of the
// 256 rows of B (16 KB + 16 KB), 6 stages: half the B traffic through each SM's shared memory.
template <bool TWO> struct Cfg {
  static constexpr int STAGES = TWO ? 6 : I8L_STAGES;
  static constexpr int B_STAGE = TWO ? BM * BK : BN * BK;
  static constexpr uint32_t STAGE_TX = TWO ? 2u * (A_STAGE + BM * BK) : (uint32_t)(A_STAGE + BN * BK);
};
constexpr int MAX_STAGES = 6;
constexpr int EPI_WARPS = 16;                 // four groups of four warps, 64 accumulator columns per group
constexpr int EPI_COLS = BN / (EPI_WARPS / 4);
constexpr int THREADS = 128 + 32 * EPI_WARPS;
constexpr int FAC_MAX = 512;                  // K blocks whose factors are staged in shared memory at a time
constexpr int TMEM_COLS = 512;
constexpr int SMEM_DYN = 4 * (A_STAGE + BN * BK) + 1024;  // == 6 * (16 KB + 16 KB) + 1024

struct GemmParams {
  const float* a_scale;
  const float* b_scale;
  const __nv_bfloat16* bias;
  void* c;
  int32_t* status;
  int m_blocks;  // batch*M/128
  int mpb;       // M/128 (m-blocks per batch)
  int n_tiles;   // ceil(N/256)
  int M, N, KB;  // KB = K/128
  int a_kind, b_kind, b_batched;
  int exact, divide, out_f32, dump;  // dump: 0 none, 1 whole-K int32, 2 per-K-block int32
  int a_kshift;       // an A tile scale serves 2^a_kshift consecutive K blocks (1 for 128x256 groups)
  int product_first;  // exact order only: float(P) * (a_s*b_s) instead of (float(P)*a_s)*b_s
  int raster;
  int c_align32;  // the output pointer is 32-byte aligned: 256-bit stores
  // scatter mode (rs_rows > 0): rows [o*rs_rows, (o+1)*rs_rows) of the product go to c_slots[o], a
  // [world, rs_rows, N] bf16 buffer of rank o (peer memory), at slot rs_rank
  void* c_slots[I8L_MAX_RANKS];
  int rs_rows, rs_rank;
  int m_rot;  // 128-row blocks by which the tile order is rotated (0 unless scattering)
  float post_scale;
  uint32_t max_polls;  // limit of every mbarrier wait, in polls (WAIT_MAX_POLLS unless a test lowers it)
  int withhold;        // test hook: the producer leaves out the last operand load of its first tile
};

// Instruction descriptor: D=s32, A=B=s8, both K-major, M=128, N=256, dense, no saturation.
constexpr uint32_t IDESC_I8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                              ((uint32_t)(BM >> 4) << 24);
// Same with M=256 for the CTA-pair instruction (128 rows per CTA).
constexpr uint32_t IDESC_I8_PAIR = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)((2 * BM) >> 4) << 24);

struct TileCoord {
  int m_blk, n_tile;
};
__device__ __forceinline__ TileCoord tile_coord(int t, int m_units, const GemmParams& p) {
  const int per_group = p.raster * p.n_tiles;
  const int g = t / per_group, local = t - g * per_group;
  const int first = g * p.raster;
  const int gsize = min(p.raster, m_units - first);
  TileCoord tc;
  tc.m_blk = first + local % gsize;
  tc.n_tile = local / gsize;
  return tc;
}

struct __align__(8) SharedCtl {   // tempty must directly follow tfull (the fast epilogue addresses both from one base)
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], tfull[2], tempty[2], done;
  uint64_t fready[2], ffree[2];  // fast block kind: factor buffers written (factor warp) / consumed (every epilogue thread)
  uint32_t tmem_base;
  int abort_flag;
  float bscale[EPI_WARPS / 4][EPI_COLS];     // per-tile column scales of each epilogue group (CHANNEL)
  float bstep[EPI_WARPS / 4][2][EPI_COLS];   // per-K-block column scales (GROUP), double buffered
  // K_BLOCK_FAST, written by the factor warp one unit (tile, or 512-K-block chunk of a tile) ahead, two buffers:
  float fac[2][EPI_WARPS / 4][FAC_MAX];      // signed per-K-block scalar factors
  float fbscale[2][EPI_WARPS / 4][EPI_COLS]; // per-channel column scales (times post_scale)
  float fbias[2][EPI_WARPS / 4][2];          // running sum of the signed factors of the tile (value, error term)
  // scatter mode of the fast block kind: four output rows x 128 bytes per epilogue warp, staged so that one
  // store instruction writes whole 128-byte row segments into the peer's memory
  uint4 xpose[EPI_WARPS][4][8];
};

// Epilogue kinds.  Everything but K_ROWCOL drains the accumulator every 128-wide K block.
constexpr int K_ROWCOL = 0;      // one drain per tile, (float(acc)*a_s[m])*b_s[n]
constexpr int K_BLOCK_GEN = 1;   // block-scaled, any scale layout, reference operation order, dumps
constexpr int K_BLOCK_FAST = 2;  // block-scaled, one scalar factor per (tile, K block) and 64-column group
constexpr int K_BLOCK_ROWFAC = 4;  // block-scaled, per-(row, K block) A scale x per-tile or per-channel B scale
constexpr int K_BLOCK_COLFAC = 3;  // block-scaled, per-tile A scale x per-(column, K block) B scale (fused forward)
constexpr uint32_t MAGIC_I = 0x4B400000u;   // the bits of 1.5 * 2^23
constexpr float MAGIC_F = 12582912.f;       // 1.5 * 2^23

// Sixteen int32 partial products (|P| < 2^22) -> fp32, exactly.  The conversion instruction runs at half
// rate on one pipe; MAGIC_I + P read as a float is 1.5*2^23 + P, and subtracting 1.5*2^23 (a packed add on
// the other pipe) gives the same float(P).  Alternating the two forms between chunks balances the pipes
// (measured 6 % faster than either alone).
__device__ __forceinline__ void to_float16(bool via_add, const uint32_t* r, float* v) {
  if (via_add) {
    const float2 nm = make_float2(-MAGIC_F, -MAGIC_F);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 t = __fadd2_rn(make_float2(__uint_as_float(MAGIC_I + r[2 * j]), __uint_as_float(MAGIC_I + r[2 * j + 1])), nm);
      v[2 * j] = t.x;
      v[2 * j + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __int2float_rn((int)r[j]);
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void st_global_256(void* ptr, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// Final rescale, bias, cast and store of one thread's EPI_COLS consecutive columns.  Every lane of
// a warp writes a different row, so each store instruction touches 32 lines: 32-byte stores (whole
// sectors, half as many instructions) are used when the output pointer allows them.
// POST = false: the caller has already folded post_scale into the scales it passes.
template <bool POST = true>
__device__ __forceinline__ void store_cols(const GemmParams& p, const float* acc, const float* bscale_or_null,
                                           int64_t row, int col0, void* cbase) {
#pragma unroll
  for (int j0 = 0; j0 < EPI_COLS; j0 += 16) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = acc[j0 + j];
      if (bscale_or_null) v[j] *= bscale_or_null[j0 + j];
      if (POST && p.post_scale != 1.f) v[j] = __fmul_rn(v[j], p.post_scale);
    }
    if (p.bias) {  // a uniform branch: no predicated-off loads and adds when there is no bias
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __fadd_rn(v[j], __bfloat162float(p.bias[col0 + j0 + j]));
    }
    if (p.out_f32) {
      float* o = static_cast<float*>(cbase) + row * p.N + col0 + j0;
      if (p.c_align32) {
        st_global_256(o, reinterpret_cast<const uint32_t*>(v));
        st_global_256(o + 8, reinterpret_cast<const uint32_t*>(v + 8));
      } else {
#pragma unroll
        for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(cbase) + row * p.N + col0 + j0;
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
      if (p.c_align32) {
        st_global_256(o, w);
      } else {
        *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(o + 8) = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }
}

template <int KIND, bool TWO>
__global__ void __launch_bounds__(THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
  constexpr bool BLOCK = KIND != K_ROWCOL;
  constexpr int STAGES = Cfg<TWO>::STAGES, B_STAGE = Cfg<TWO>::B_STAGE;
  constexpr uint32_t STAGE_TX = Cfg<TWO>::STAGE_TX;
  extern __shared__ uint8_t smem_raw[];
  __shared__ SharedCtl ctl;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = smem_base, smem_b = smem_base + STAGES * A_STAGE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl.abort_flag;
  // CTA pair: rank 0 (the leader) owns the operand-ready and accumulator-free barriers and issues the MMAs
  const uint32_t rank = TWO ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  // tile-processing unit (CTA or pair) and their count: read from the special registers at each use
  // instead of being kept live (the epilogue runs at its register budget)
#define I8L_UNIT (TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x)
#define I8L_N_UNITS (TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl.full[s]), 1);
      mbar_init(smem_u32(&ctl.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl.tfull[b]), 1);
      // arrivals that free an accumulator buffer: one per epilogue warp (of both CTAs of a pair); the fast
      // block kernel lets every epilogue thread arrive for itself (no warp sync, no branch in its loop)
      mbar_init(smem_u32(&ctl.tempty[b]), KIND == K_BLOCK_FAST ? EPI_WARPS * 32 : (TWO ? 2 : 1) * EPI_WARPS);
    }
    mbar_init(smem_u32(&ctl.done), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl.fready[b]), 1);
      mbar_init(smem_u32(&ctl.ffree[b]), EPI_WARPS * 32);
    }
    ctl.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (TWO) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;
  // tiles of this unit: m_blocks counts 128-row blocks; a pair takes two consecutive ones
  const int total_tiles = (TWO ? p.m_blocks / 2 : p.m_blocks) * p.n_tiles;
  auto unit_tile = [&](int t) {  // 128-row block of THIS CTA and 256-column tile
    if constexpr (TWO) {
      TileCoord tc = tile_coord(t, p.m_blocks / 2, p);
      tc.m_blk = 2 * tc.m_blk + (int)cluster_ctarank();
      return tc;
    } else {
      TileCoord tc = tile_coord(t, p.m_blocks, p);
      tc.m_blk += p.m_rot;  // scatter mode: every rank starts at a different owner's rows (no incast)
      if (tc.m_blk >= p.m_blocks) tc.m_blk -= p.m_blocks;
      return tc;
    }
  };
  const int KB = p.KB;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      int s = 0;
      uint32_t ph = 0;
      uint32_t issued = 0, issued_ph = 0;  // bit s: a load into stage s is (or was) in flight, with parity
      bool ok = true;
      for (int t = I8L_UNIT; t < total_tiles && ok; t += I8L_N_UNITS) {
        const TileCoord tc = unit_tile(t);
        const int a_row = tc.m_blk * BM;
        const int b_row = (p.b_batched ? (tc.m_blk / p.mpb) * p.N : 0) + tc.n_tile * BN + (TWO ? (int)rank * BM : 0);
        for (int kb = 0; kb < KB; ++kb) {
          if (!(ok = mbar_wait<!BLOCK>(smem_u32(&ctl.empty[s]), ph ^ 1u, abort_flag, p.max_polls))) break;
          if (p.withhold && t == I8L_UNIT && kb == KB - 1) {
            // test hook: this stage is never filled, so the waits that depend on it run into their limit
            if (++s == STAGES) { s = 0; ph ^= 1u; }
            continue;
          }
          if (lane == 0) {
            const uint32_t bar = smem_u32(&ctl.full[s]);
            if (TWO) {  // both CTAs' copies complete on the leader's barrier, which expects the bytes of both
              if (leader) mbar_expect_tx(bar, STAGE_TX);
              const uint32_t lbar = map_to_cta(bar, 0);
              tma_load_2d_pair(smem_a + s * A_STAGE, &map_a, lbar, kb * BK, a_row);
              tma_load_2d_pair(smem_b + s * B_STAGE, &map_b, lbar, kb * BK, b_row);
            } else {
              mbar_expect_tx(bar, STAGE_TX);
              tma_load_2d(smem_a + s * A_STAGE, &map_a, bar, kb * BK, a_row);
              tma_load_2d(smem_b + s * B_STAGE, &map_b, bar, kb * BK, b_row);
            }
          }
          issued |= 1u << s;
          issued_ph = (issued_ph & ~(1u << s)) | (ph << s);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok && leader) {
        // let copies already in flight land before the CTA's shared memory is released
        for (int k = 0; k < STAGES; ++k)
          if (issued & (1u << k)) {
            int dummy = 0;
            mbar_wait(smem_u32(&ctl.full[k]), (issued_ph >> k) & 1u, &dummy, 1u << 15);
          }
      }
    } else if (warp == 1 && leader) {
      // ------------------------------------------------------------------ MMA issuer
      int s = 0, ab = 0;
      uint32_t ph = 0, aph = 0;
      bool ok = true;
      for (int t = I8L_UNIT; t < total_tiles && ok; t += I8L_N_UNITS) {
        for (int kb = 0; kb < KB; ++kb) {
          const bool drain_start = BLOCK || kb == 0, drain_end = BLOCK || kb == KB - 1;
          // block-scaled kinds wait for the accumulator buffer last (the epilogue's release is what holds
          // the next MMA up); the whole-K kinds measured 0.7 % faster the other way round
          if (!BLOCK && drain_start) {
            if (!(ok = mbar_wait<!BLOCK>(smem_u32(&ctl.tempty[ab]), aph ^ 1u, abort_flag, p.max_polls))) break;
          }
          if (!(ok = mbar_wait<!BLOCK>(smem_u32(&ctl.full[s]), ph, abort_flag, p.max_polls))) break;
          if (BLOCK) {
            if (!(ok = mbar_wait<!BLOCK>(smem_u32(&ctl.tempty[ab]), aph ^ 1u, abort_flag, p.max_polls))) break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint64_t da = smem_desc(smem_a + s * A_STAGE), db = smem_desc(smem_b + s * B_STAGE);
            const uint32_t d = tmem_base + ab * BN;
#pragma unroll
            for (int k4 = 0; k4 < BK / 32; ++k4) {
              if (TWO) tc_mma_i8_pair(d, da + 2 * k4, db + 2 * k4, IDESC_I8_PAIR, (k4 > 0 || !drain_start) ? 1u : 0u);
              else tc_mma_i8(d, da + 2 * k4, db + 2 * k4, IDESC_I8, (k4 > 0 || !drain_start) ? 1u : 0u);
            }
            if (TWO) {  // both CTAs' producers and epilogues wait on their own copies of these barriers
              tc_commit_pair(smem_u32(&ctl.empty[s]));
              if (drain_end) tc_commit_pair(smem_u32(&ctl.tfull[ab]));
            } else {
              tc_commit(smem_u32(&ctl.empty[s]));
              if (drain_end) tc_commit(smem_u32(&ctl.tfull[ab]));
            }
          }
          __syncwarp();
          if (drain_end) {
            ab ^= 1;
            if (ab == 0) aph ^= 1u;
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      // all MMAs issued by this thread must have retired before tensor memory is freed
      if (lane == 0) {
        if (TWO) tc_commit_pair_local(smem_u32(&ctl.done));
        else tc_commit(smem_u32(&ctl.done));
      }
      __syncwarp();
      int dummy = 0;
      mbar_wait(smem_u32(&ctl.done), 0, &dummy);
    } else if (KIND == K_BLOCK_FAST && warp == 2) {
      // ------------------------------------------------------------------ factor warp (fast block kind)
      // Prepares, one unit ahead of the epilogue, what the epilogue needs besides the accumulators: the
      // signed factor of every K block and the column scales.  Block d contributes g_d * (MAGIC_F + s_d P_d)
      // with g_d = s_d f_d (see the epilogue), so the accumulators carry MAGIC_F * sum(g) on top of sum(f P).
      // Choosing s_d against the sign of the running sum keeps |sum(g)| <= max f whatever the scales are, which
      // bounds the rounding error the bias can cause; the epilogue takes the sum out after the last K block.
      // Hand-over through two mbarrier pairs (buffer written / buffer consumed), waits bounded like all others.
      const bool chan = p.b_kind == I8L_BSCALE_CHANNEL;
      float run = 0.f, low = 0.f;   // lanes 0-3: the running sum of column group `lane` as an unevaluated pair
      uint32_t u = 0;
      for (int t = I8L_UNIT; t < total_tiles; t += I8L_N_UNITS) {
        const TileCoord tc = unit_tile(t);
        for (int k0 = 0; k0 < KB; k0 += FAC_MAX, ++u) {
          const int dn = KB - k0 < FAC_MAX ? KB - k0 : FAC_MAX;
          const int buf = u & 1;
          if (u >= 2 && !mbar_wait(smem_u32(&ctl.ffree[buf]), ((u >> 1) - 1) & 1u, abort_flag, p.max_polls)) {
            t = total_tiles;   // gave up (or another warp did): leave both loops
            break;
          }
          for (int g = 0; g < EPI_WARPS / 4; ++g) {
            const int col0 = tc.n_tile * BN + g * EPI_COLS;
            const bool active = col0 < p.N;
            const int64_t bcol0 = (int64_t)(p.b_batched ? tc.m_blk / p.mpb : 0) * p.N + col0;
            if (chan)   // post_scale rides on the column scale (on the factors otherwise)
              for (int i = lane; i < EPI_COLS; i += 32)
                ctl.fbscale[buf][g][i] = active ? __ldg(p.b_scale + bcol0 + i) * p.post_scale : 0.f;
            const float* as_ptr = p.a_scale + (int64_t)tc.m_blk * (KB >> p.a_kshift);
            const float* bs_ptr = p.b_scale + (bcol0 >> 7) * KB + k0;
            for (int i = lane; i < dn; i += 32)
              ctl.fac[buf][g][i] = __ldg(as_ptr + ((k0 + i) >> p.a_kshift)) * ((!chan && active) ? __ldg(bs_ptr + i) * p.post_scale : 1.f);
          }
          __syncwarp();
          if (lane < EPI_WARPS / 4) {
            if (k0 == 0) run = low = 0.f;
            float* f = ctl.fac[buf][lane];
            for (int i = 0; i < dn; ++i) {
              float g = f[i];
              g = run > 0.f ? -g : g;
              const float sum = __fadd_rn(run, g);
              const float bb = __fsub_rn(sum, run);   // two-sum: the rounding error of run + g, off the critical chain
              low = __fadd_rn(low, __fadd_rn(__fsub_rn(run, __fsub_rn(sum, bb)), __fsub_rn(g, bb)));
              run = sum;
              f[i] = g;
            }
            ctl.fbias[buf][lane][0] = run;
            ctl.fbias[buf][lane][1] = low;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl.fready[buf]));   // release: the warp's writes above are visible to waiters
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (16 warps)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int q = warp & 3, wg = (warp - 4) >> 2;  // lane quarter, 64-column group
    const int tix = q * 32 + lane;                 // row within the tile == thread index within the group
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    int ab = 0;
    uint32_t aph = 0;
    bool ok = true;
    auto release_accumulator = [&]() {  // all of this warp's tensor-memory loads of the buffer have completed
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (TWO) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl.tempty[ab]), 0));  // the leader's barrier
        else mbar_arrive(smem_u32(&ctl.tempty[ab]));
      }
    };
    if constexpr (KIND == K_BLOCK_FAST) {
      // One scalar factor per (tile, K block) and column group: a per-tile A scale times a per-tile or
      // per-channel B scale.  The K-block loop keeps only the accumulators, one chunk of tensor-memory
      // data and a few scalars live: the factors of the tile are staged in shared memory first, and
      // what the final store needs is recomputed from the tile index afterwards.
      const uint32_t tfull0 = smem_u32(&ctl.tfull[0]);
      constexpr uint32_t TEMPTY_OFF = 2 * sizeof(uint64_t);   // tempty[] follows tfull[2] in SharedCtl: one base register serves both
      // Values derived from the thread index pass through an empty asm statement: the compiler then
      // keeps them in registers instead of recomputing them from the special register at every use
      // inside the K-block loop (which cost about 35 ALU instructions per warp and K block).
      uint32_t taddr0 = tmem_base + lane_addr + wg * EPI_COLS, fac_base = smem_u32(&ctl.fac[0][wg][0]);
      asm volatile("" : "+r"(taddr0), "+r"(fac_base));
      const bool chan = p.b_kind == I8L_BSCALE_CHANNEL;
      constexpr int CH = 8;
      uint32_t gstep = 0, unit = 0;
      // The loops below never exit early (one exit and nothing to carry but the accumulators compiles to the
      // leanest code): after a wait timeout a warp runs through the remaining tiles without waiting or storing.
      for (int t = I8L_UNIT; t < total_tiles; t += I8L_N_UNITS) {
        float2 acc[EPI_COLS / 2];
#pragma unroll
        for (int j = 0; j < EPI_COLS / 2; ++j) acc[j] = make_float2(0.f, 0.f);
        const bool active = unit_tile(t).n_tile * BN + wg * EPI_COLS < p.N;
        for (int k0 = 0; k0 < KB; k0 += FAC_MAX) {
          const int dn = KB - k0 < FAC_MAX ? KB - k0 : FAC_MAX;
          if (k0) {   // the previous chunk's factors are no longer needed
            mbar_arrive(smem_u32(&ctl.ffree[unit & 1]));
            ++unit;
          }
          mbar_wait_or_flag(smem_u32(&ctl.fready[unit & 1]), (unit >> 1) & 1u, abort_flag, p.max_polls);   // written by the factor warp
          const uint32_t fac0 = fac_base + (unit & 1) * (uint32_t)sizeof(ctl.fac[0]);
          for (int d = 0; d < dn; ++d) {
            float f;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(fac0 + 4 * d));
            // No early exit and no success flag: a loop with one exit and nothing to carry but the
            // accumulators compiles to the leanest code.  After a timeout the abort flag is set, the status
            // word reports it, and the remaining K blocks run on whatever tensor memory holds.
            mbar_spin_or_flag(tfull0 + 8 * ab, aph, abort_flag, p.max_polls);
            tc_fence_after();
            auto release = [&]() {  // all of this warp's tensor-memory loads of the buffer have completed
              tc_fence_before();
              mbar_arrive(tfull0 + TEMPTY_OFF + 8 * ab);   // every thread arrives for itself: no warp sync, no branch
            };
            if (active) {
              // int32 -> fp32 without the conversion unit: |P| <= 128*127*127 < 2^22, so the integer MAGIC_I + P
              // (or MAGIC_I - P), read as a float, IS the number 1.5*2^23 + P (or - P): one full-rate integer
              // add per element instead of a half-rate conversion.  The factor carries the sign, so the product
              // is f*P plus a multiple of MAGIC_F that the factor warp keeps small and the tile end removes.
              const uint32_t taddr = taddr0 + ab * BN;
              const float2 f2 = make_float2(f, f);
              if (f >= 0.f) {
#pragma unroll
                for (int c = 0; c < EPI_COLS / CH; ++c) {  // 8-column chunks: 16-column ones spill here
                  uint32_t r[CH];
                  tc_ld8(taddr + c * CH, r);
                  tc_ld_wait();
                  if (c == EPI_COLS / CH - 1) release();
#pragma unroll
                  for (int j = 0; j < CH / 2; ++j)
                    acc[c * (CH / 2) + j] = __ffma2_rn(make_float2(__uint_as_float(MAGIC_I + r[2 * j]), __uint_as_float(MAGIC_I + r[2 * j + 1])),
                                                       f2, acc[c * (CH / 2) + j]);
                }
              } else {
#pragma unroll
                for (int c = 0; c < EPI_COLS / CH; ++c) {
                  uint32_t r[CH];
                  tc_ld8(taddr + c * CH, r);
                  tc_ld_wait();
                  if (c == EPI_COLS / CH - 1) release();
#pragma unroll
                  for (int j = 0; j < CH / 2; ++j)
                    acc[c * (CH / 2) + j] = __ffma2_rn(make_float2(__uint_as_float(MAGIC_I - r[2 * j]), __uint_as_float(MAGIC_I - r[2 * j + 1])),
                                                       f2, acc[c * (CH / 2) + j]);
                }
              }
            } else {
              release();
            }
            ++gstep;  // buffer and phase from one running count of K blocks
            ab = gstep & 1;
            aph = (gstep >> 1) & 1u;
          }
        }
        // after a timeout the accumulators are not a product: nothing is stored (decided per warp: the store
        // path below synchronises the warp)
        if (active && __all_sync(0xffffffffu, !*abort_flag)) {
          int t2 = t;
          asm volatile("" : "+r"(t2));  // keeps the tile's coordinates out of the K-block loop's live registers
          const TileCoord tc = unit_tile(t2);
          // take out MAGIC_F * sum(g): the leading part first (close to the accumulator, so the difference is
          // nearly exact), then the small remainder
          const float* fb = ctl.fbias[unit & 1][wg];
          const float b_hi = __fmul_rn(-MAGIC_F, fb[0]);
          const float b_lo = __fmaf_rn(-MAGIC_F, fb[0], -b_hi) + __fmul_rn(-MAGIC_F, fb[1]);
          float out[EPI_COLS];
#pragma unroll
          for (int j = 0; j < EPI_COLS / 2; ++j) {
            out[2 * j] = __fadd_rn(__fadd_rn(acc[j].x, b_hi), b_lo);
            out[2 * j + 1] = __fadd_rn(__fadd_rn(acc[j].y, b_hi), b_lo);
          }
          int64_t row = (int64_t)tc.m_blk * BM + tix;
          void* cbase = p.c;
          if (p.rs_rows) {  // scatter mode: this 128-row block belongs to rank `owner`; write into our slot of its buffer
            const int owner = (tc.m_blk * BM) / p.rs_rows;
            cbase = p.c_slots[owner];
            row += (int64_t)(p.rs_rank - owner) * p.rs_rows;
          }
          const float* bsc = chan ? ctl.fbscale[unit & 1][wg] : nullptr;
          const int col0 = tc.n_tile * BN + wg * EPI_COLS;
          if (p.rs_rows && !p.out_f32 && !p.bias) {
            // Peer stores.  A lane owns one row, so a plain store instruction would send 32 separate 32-byte
            // pieces over NVLink; here the warp passes four rows at a time through shared memory (16-byte
            // slots, XOR-swizzled so that writers and readers are conflict-free) and every store instruction
            // then covers four rows x 128 contiguous bytes.  Same values as store_cols.
            uint32_t w[EPI_COLS / 2];
#pragma unroll
            for (int j = 0; j < EPI_COLS / 2; ++j) {
              float a = out[2 * j], b = out[2 * j + 1];
              if (bsc) { a *= bsc[2 * j]; b *= bsc[2 * j + 1]; }
              w[j] = pack_bf16x2(a, b);
            }
            uint4* xp = &ctl.xpose[warp - 4][0][0];
            const int wr = lane & 3, rr = lane >> 3, rc = lane & 7;
            __nv_bfloat16* obase = static_cast<__nv_bfloat16*>(cbase) + (row - lane) * p.N + col0 + rc * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if ((lane >> 2) == j) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                  xp[wr * 8 + (c ^ (wr << 1))] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
              }
              __syncwarp();
              const uint4 v = xp[rr * 8 + (rc ^ (rr << 1))];
              *reinterpret_cast<uint4*>(obase + (int64_t)(4 * j + rr) * p.N) = v;
              __syncwarp();
            }
          } else {
            store_cols<false>(p, out, bsc, row, col0, cbase);
          }
        }
        mbar_arrive(smem_u32(&ctl.ffree[unit & 1]));   // this tile's factors and column scales are no longer needed
        ++unit;
      }
    } else
    for (int t = I8L_UNIT; t < total_tiles; t += I8L_N_UNITS) {  // no early exit either (named barriers inside)
      const TileCoord tc = unit_tile(t);
      const int batch = tc.m_blk / p.mpb;
      const int64_t row = (int64_t)tc.m_blk * BM + tix;  // row in the folded [batch*M] space
      const int col0 = tc.n_tile * BN + wg * EPI_COLS;
      const bool active = col0 < p.N;
      const int64_t bcol0 = (int64_t)(p.b_batched ? batch : 0) * p.N + col0;  // first b_scale column index
      const bool chan = p.b_kind == I8L_BSCALE_CHANNEL && !p.dump;
      if (chan) {  // K-invariant column scales of this group -> shared memory
        named_sync(1 + wg, 128);
        if (tix < EPI_COLS) ctl.bscale[wg][tix] = active ? __ldg(p.b_scale + bcol0 + tix) : 0.f;
        named_sync(1 + wg, 128);
      }

      if constexpr (KIND == K_BLOCK_ROWFAC) {
        // one factor a_s * b_s per (row or tile, K block) and column group, fetched by each thread
        const float* as_ptr = p.a_scale + (p.a_kind == I8L_ASCALE_TILE ? (int64_t)tc.m_blk : row) * KB;
        const float* bs_ptr = p.b_scale + (bcol0 >> 7) * KB;
        float2 acc[EPI_COLS / 2];
#pragma unroll
        for (int j = 0; j < EPI_COLS / 2; ++j) acc[j] = make_float2(0.f, 0.f);
        float f_next = __ldg(as_ptr) * ((!chan && active) ? __ldg(bs_ptr) : 1.f);
        for (int d = 0; d < KB; ++d) {
          const float f = f_next;
          if (d + 1 < KB) f_next = __ldg(as_ptr + d + 1) * ((!chan && active) ? __ldg(bs_ptr + d + 1) : 1.f);
          ok = ok && mbar_wait<!BLOCK>(smem_u32(&ctl.tfull[ab]), aph, abort_flag, p.max_polls);  // single-exit loop, see K_BLOCK_FAST
          tc_fence_after();
          if (ok && active) {
            const uint32_t taddr = tmem_base + lane_addr + ab * BN + wg * EPI_COLS;
            const float2 f2 = make_float2(f, f);
#pragma unroll
            for (int c = 0; c < EPI_COLS / 16; ++c) {
              uint32_t r[16];
              tc_ld16(taddr + c * 16, r);
              tc_ld_wait();
              if (c == EPI_COLS / 16 - 1) release_accumulator();
              // one conversion and half a packed FMA per accumulator element; each pass is a run of
              // independent instructions
              float v[16];
              to_float16((c & 1) != 0, r, v);   // c is an unrolled loop index: the choice folds at compile time
#pragma unroll
              for (int j = 0; j < 8; ++j)
                acc[c * 8 + j] = __ffma2_rn(make_float2(v[2 * j], v[2 * j + 1]), f2, acc[c * 8 + j]);
            }
          } else {
            release_accumulator();
          }
          ab ^= 1;
          if (ab == 0) aph ^= 1u;
        }
        if (ok && active) {
          float out[EPI_COLS];
#pragma unroll
          for (int j = 0; j < EPI_COLS / 2; ++j) {
            out[2 * j] = acc[j].x;
            out[2 * j + 1] = acc[j].y;
          }
          store_cols(p, out, chan ? ctl.bscale[wg] : nullptr, row, col0, p.c);
        }
      } else if constexpr (KIND == K_BLOCK_COLFAC) {
        constexpr bool COLFAC = true;
        // factor of a K block: a_s * b_s, or its reciprocal when the scales are multipliers (fused
        // variants: acc += P / (s_a * s_b); the reciprocal replaces the reference's division, 1 ulp)
        const float* as_ptr = p.a_scale + (p.a_kind == I8L_ASCALE_TILE ? (int64_t)tc.m_blk : row) * KB;
        const int64_t bcol = bcol0 + (tix & (EPI_COLS - 1));  // COLFAC: the column whose factor this thread publishes
        const float* bs_ptr = COLFAC ? p.b_scale + (p.b_kind == I8L_BSCALE_GROUP ? bcol : bcol >> 7) * KB
                                     : p.b_scale + (bcol0 >> 7) * KB;
        const bool use_b = COLFAC ? active : (!chan && active);
        const bool recip = COLFAC && p.divide;
        auto factor = [&](int d) {
          float f = __ldg(as_ptr + d);
          if (use_b) f *= __ldg(bs_ptr + d);
          if (COLFAC) f = recip ? __frcp_rn(f) : f;
          return f;
        };
        float2 acc[EPI_COLS / 2];
#pragma unroll
        for (int j = 0; j < EPI_COLS / 2; ++j) acc[j] = make_float2(0.f, 0.f);
        float f_next = factor(0);
        for (int d = 0; d < KB; ++d) {
          const float f = f_next;
          if (d + 1 < KB) f_next = factor(d + 1);
          if (COLFAC) {  // thread i < 64 publishes the factor of column i of this group for this K block
            if (tix < EPI_COLS) ctl.bstep[wg][d & 1][tix] = f;
            named_sync(1 + wg, 128);
          }
          ok = ok && mbar_wait<!BLOCK>(smem_u32(&ctl.tfull[ab]), aph, abort_flag, p.max_polls);  // single-exit loop, see K_BLOCK_FAST
          tc_fence_after();
          if (ok && active) {
            const uint32_t taddr = tmem_base + lane_addr + ab * BN + wg * EPI_COLS;
            const float2 f2 = make_float2(f, f);
            const float2* fcol = reinterpret_cast<const float2*>(ctl.bstep[wg][d & 1]);
#pragma unroll
            for (int c = 0; c < EPI_COLS / 16; ++c) {
              uint32_t r[16];
              tc_ld16(taddr + c * 16, r);
              tc_ld_wait();
              if (c == EPI_COLS / 16 - 1) release_accumulator();
              // one conversion and half a packed FMA per accumulator element; each pass is a run of
              // independent instructions
              float v[16];
              to_float16((c & 1) != 0, r, v);   // c is an unrolled loop index: the choice folds at compile time
#pragma unroll
              for (int j = 0; j < 8; ++j)
                acc[c * 8 + j] = __ffma2_rn(make_float2(v[2 * j], v[2 * j + 1]), COLFAC ? fcol[c * 8 + j] : f2, acc[c * 8 + j]);
            }
          } else {
            release_accumulator();
          }
          ab ^= 1;
          if (ab == 0) aph ^= 1u;
        }
        if (ok && active) {
          float out[EPI_COLS];
#pragma unroll
          for (int j = 0; j < EPI_COLS / 2; ++j) {
            out[2 * j] = acc[j].x;
            out[2 * j + 1] = acc[j].y;
          }
          store_cols(p, out, (!COLFAC && chan) ? ctl.bscale[wg] : nullptr, row, col0, p.c);
        }
      } else {
        // ---- generic paths: reference operation order, per-column / per-step scales, dumps, row x column
        float acc[BLOCK ? EPI_COLS : 1];
        if (BLOCK) {
#pragma unroll
          for (int j = 0; j < EPI_COLS; ++j) acc[j] = 0.f;
        }
        const int ndrain = BLOCK ? KB : 1;
        for (int d = 0; d < ndrain; ++d) {
          float sa = 1.f, sb = 1.f;
          if (BLOCK && !p.dump) {
            sa = p.a_kind == I8L_ASCALE_GROUP ? __ldg(p.a_scale + row * KB + d)
                                              : __ldg(p.a_scale + (int64_t)tc.m_blk * (KB >> p.a_kshift) + (d >> p.a_kshift));
            if (p.b_kind == I8L_BSCALE_TILE && active) sb = __ldg(p.b_scale + (bcol0 >> 7) * KB + d);
            if (p.b_kind == I8L_BSCALE_GROUP) {
              if (tix < EPI_COLS) ctl.bstep[wg][d & 1][tix] = active ? __ldg(p.b_scale + (bcol0 + tix) * KB + d) : 0.f;
              named_sync(1 + wg, 128);
            }
          }
          ok = ok && mbar_wait<!BLOCK>(smem_u32(&ctl.tfull[ab]), aph, abort_flag, p.max_polls);
          tc_fence_after();
          const bool live = ok && active;
          const uint32_t taddr = tmem_base + lane_addr + ab * BN + wg * EPI_COLS;
#pragma unroll
          for (int c = 0; c < EPI_COLS / 16; ++c) {
            uint32_t r[16];
            if (live) {
              tc_ld16(taddr + c * 16, r);
              tc_ld_wait();
            }
            if (c == EPI_COLS / 16 - 1) release_accumulator();
            if (!live) continue;
            if (BLOCK) {
              if (p.dump) {
                int32_t* o = static_cast<int32_t*>(p.c) +
                             (((int64_t)batch * KB + d) * p.M + (row - (int64_t)batch * p.M)) * p.N + col0 + c * 16;
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
              } else {
                const float* sbv = p.b_kind == I8L_BSCALE_CHANNEL ? ctl.bscale[wg]
                                   : p.b_kind == I8L_BSCALE_GROUP ? ctl.bstep[wg][d & 1]
                                                                  : nullptr;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float pf = __int2float_rn((int)r[j]);
                  const float sbj = sbv ? sbv[c * 16 + j] : sb;
                  float term;
                  if (p.divide) term = __fdiv_rn(pf, __fmul_rn(sa, sbj));
                  else if (p.product_first) term = __fmul_rn(pf, __fmul_rn(sa, sbj));
                  else term = __fmul_rn(__fmul_rn(pf, sa), sbj);
                  acc[c * 16 + j] = __fadd_rn(acc[c * 16 + j], term);
                }
              }
            } else if (p.dump) {
              int32_t* o = static_cast<int32_t*>(p.c) + row * p.N + col0 + c * 16;
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
              // row x column epilogue straight from the accumulator chunk
              const float sar = __ldg(p.a_scale + row);
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                v[j] = __fmul_rn(__fmul_rn(__int2float_rn((int)r[j]), sar), ctl.bscale[wg][c * 16 + j]);
                if (p.post_scale != 1.f || p.bias) {
                  // the reference stores the GEMM result in the output type before its 1/K pass: a bf16
                  // rounding for bf16 outputs, none for fp32 ones
                  if (!p.out_f32) v[j] = round_to_bf16(v[j]);
                  v[j] = __fmul_rn(v[j], p.post_scale);
                  if (p.bias) v[j] = __fadd_rn(v[j], __bfloat162float(p.bias[col0 + c * 16 + j]));
                }
              }
              if (p.out_f32) {
                float* o = static_cast<float*>(p.c) + row * p.N + col0 + c * 16;
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              } else {
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.c) + row * p.N + col0 + c * 16;
#pragma unroll
                for (int j = 0; j < 16; j += 8)
                  *reinterpret_cast<uint4*>(o + j) = make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                                pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
              }
            }
          }
          ab ^= 1;
          if (ab == 0) aph ^= 1u;
        }
        if constexpr (BLOCK) {
          if (ok && active && !p.dump) store_cols(p, acc, nullptr, row, col0, p.c);
        }
      }
    }
  }

#undef I8L_UNIT
#undef I8L_N_UNITS
  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();  // no remote arrival or tensor-memory write of the pair is still pending
  if (threadIdx.x == 0 && ctl.abort_flag && p.status) atomicExch(p.status, I8L_ERR_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    if (TWO) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// out[r, c] = sum over the `world` slots of slots[w, r, c], added in slot order in fp32 and rounded once:
// the local half of the reduce-scatter whose other half is the scatter-mode GEMM epilogue.
__global__ void __launch_bounds__(256) sum_slots_kernel(const uint4* __restrict__ slots, uint4* __restrict__ out,
                                                        int world, int64_t n16) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int w = 0; w < world; ++w) {
      float v[8];
      unpack8(__ldg(slots + (int64_t)w * n16 + i), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], v[j]);
    }
    out[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                        pack_bf16x2(acc[6], acc[7]));
  }
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    cached.store(fn, std::memory_order_release);
  }
  return fn;
}

// int8 [rows, K] row-major -> boxes of box_rows x 128 bytes, 128B swizzle.  A tensor map depends only
// on (pointer, rows, K, box rows); a training loop calls with the same few operands step after step, so
// the last maps of each host thread are kept (no lock: the cache is thread local) and the driver's
// encode call leaves the launch path.
struct MapKey {
  const void* ptr;
  int64_t rows, K;
  int box_rows;
};
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
  constexpr int SLOTS = 16;
  thread_local MapKey keys[SLOTS] = {};
  thread_local CUtensorMap maps[SLOTS];
  thread_local int next_slot = 0;
  for (int i = 0; i < SLOTS; ++i)
    if (keys[i].ptr == ptr && keys[i].rows == rows && keys[i].K == K && keys[i].box_rows == box_rows) {
      *map = maps[i];
      return I8L_OK;
    }
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(I8L_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(I8L_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  keys[next_slot] = MapKey{ptr, rows, K, box_rows};
  maps[next_slot] = *map;
  next_slot = (next_slot + 1) % SLOTS;
  return I8L_OK;
}

// bf16 [rows, K] row-major -> boxes of 128 rows x 128 elements (256-byte rows in shared memory, no swizzle):
// the staging tiles of the single-kernel fused GEMM.
int make_tile_map_bf16(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(I8L_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(I8L_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed with CUresult %d", (int)r);
  return I8L_OK;
}

constexpr int MAX_DEVICES = 64;
static int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev < 0 || dev >= MAX_DEVICES) ? 0 : dev;
}

static int sm_count() {
  static std::atomic<int> cached[MAX_DEVICES];
  const int dev = current_device();
  int n = cached[dev].load(std::memory_order_relaxed);
  if (!n) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// i8l_set_cta_limit: CTAs a persistent GEMM launched by this host thread may occupy (0 = every SM).
static thread_local int g_cta_limit = 0;

// Test hooks (i8l_test_set_wait_limit): 0 = production values.
static std::atomic<uint32_t> g_test_max_polls{0};
static std::atomic<int> g_test_withhold{0};

uint32_t gemm_wait_limit() {
  const uint32_t lim = g_test_max_polls.load(std::memory_order_relaxed);
  return lim ? lim : WAIT_MAX_POLLS;
}
int gemm_cta_budget() {
  const int sms = sm_count();
  return (g_cta_limit > 0 && g_cta_limit < sms) ? g_cta_limit : sms;
}

template <int KIND, bool TWO>
static int launch_kind(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int64_t tiles, cudaStream_t st) {
  // per-device set-up, done by whichever thread comes first (idempotent, so a race only repeats it)
  static std::atomic<int> max_units[MAX_DEVICES];   // 0 = not set up yet
  const int dev = current_device();
  auto kernel = gemm_i8_kernel<KIND, TWO>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_DYN;
  cfg.stream = st;
  if (TWO) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  int units = max_units[dev].load(std::memory_order_acquire);
  if (!units) {
    I8L_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
    units = sm_count();
    if (TWO) {  // how many CTA pairs can be co-resident (GPCs with an odd SM count leave one SM unpaired)
      cfg.gridDim = dim3(2 * sm_count(), 1, 1);
      int n = 0;
      I8L_CUDA_OK(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
      units = n > 0 ? n : 1;
    }
    max_units[dev].store(units, std::memory_order_release);
  }
  if (g_cta_limit > 0) {   // leave SMs free for a kernel that runs beside this one
    const int lim = TWO ? g_cta_limit / 2 : g_cta_limit;
    units = units < lim ? units : (lim > 0 ? lim : 1);
  }
  const int grid_units = (int)(tiles < units ? tiles : units);
  cfg.gridDim = dim3(TWO ? 2 * grid_units : grid_units, 1, 1);
  I8L_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, p));
  return I8L_OK;
}

static int launch_gemm(bool block, const int8_t* a_q, const int8_t* b_q, GemmParams p, int64_t batch, int64_t M,
                       int64_t N, int64_t K, cudaStream_t st) {
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128)
    return fail(I8L_ERR_SHAPE, "batch=%lld M=%lld N=%lld K=%lld: all positive, M, N, K multiples of 128",
                (long long)batch, (long long)M, (long long)N, (long long)K);
  if (batch * M >= (1ll << 31) || batch * N >= (1ll << 31) || K >= (1ll << 31) ||
      (batch * M / 128) * ((N + BN - 1) / BN) >= (1ll << 31))
    return fail(I8L_ERR_SHAPE, "problem too large for 32-bit tile coordinates");
  if (!a_q || !b_q || !p.c) return fail(I8L_ERR_ARG, "null pointer");
  if (!aligned16(a_q) || !aligned16(b_q) || !aligned16(p.c)) return fail(I8L_ERR_ALIGN, "a_q, b_q, c must be 16-byte aligned");
  if (int e = check_arch()) return e;
  // CTA pairs (cta_group::2) need two 128-row blocks of the same batch per tile.  They pay off for the
  // whole-K accumulation (half the B traffic per SM: +2.5 % sustained at the power cap); the per-K-block
  // hand-off of the block-scaled kinds is slower across two CTAs (990 vs 1510 TOP/s), so those stay 1-CTA.
  const bool two = !block && (M % 256 == 0);
  CUtensorMap ma, mb;
  if (int e = make_map(&ma, a_q, batch * M, K, BM)) return e;
  if (int e = make_map(&mb, b_q, p.b_batched ? batch * N : N, K, two ? BM : BN)) return e;
  p.m_blocks = (int)(batch * M / 128);
  p.mpb = (int)(M / 128);
  p.n_tiles = (int)((N + BN - 1) / BN);
  p.M = (int)M;
  p.N = (int)N;
  p.KB = (int)(K / 128);
  {
    p.max_polls = gemm_wait_limit();
    p.withhold = g_test_withhold.load(std::memory_order_relaxed);
  }
  p.c_align32 = (reinterpret_cast<uintptr_t>(p.c) & 31u) == 0;
  for (int r = 0; r < I8L_MAX_RANKS; ++r)
    if (p.rs_rows && p.c_slots[r] && (reinterpret_cast<uintptr_t>(p.c_slots[r]) & 31u)) p.c_align32 = 0;
  // M-units (128-row blocks, or 256-row pair blocks) per raster group: the group's A panel should stay
  // L2-resident while the N tiles are swept (measured best: 4096 rows at K = 8192, flat for deeper K).
  {
    const int64_t fit = (32ll << 20) / (128 * K);
    const int blocks = (int)(fit < 16 ? 16 : (fit > 32 ? 32 : fit));  // below 16 the B re-reads double (ncu: 17.6 vs 9.4 GB)
    p.raster = two ? blocks / 2 : blocks;
  }
  const int64_t tiles = (int64_t)(two ? p.m_blocks / 2 : p.m_blocks) * p.n_tiles;
  const bool scalar_factor = block && !p.exact && !p.dump && !p.divide && p.b_kind != I8L_BSCALE_GROUP;
  const bool column_factor = block && !p.exact && !p.dump && !scalar_factor && p.a_kind == I8L_ASCALE_TILE &&
                             p.b_kind != I8L_BSCALE_CHANNEL;
  if (!block) return two ? launch_kind<K_ROWCOL, true>(ma, mb, p, tiles, st) : launch_kind<K_ROWCOL, false>(ma, mb, p, tiles, st);
  // the fast kind encodes a sign in its factors: it needs them positive (scales are; post_scale must be too)
  if (scalar_factor && p.a_kind == I8L_ASCALE_TILE && p.post_scale > 0.f) return launch_kind<K_BLOCK_FAST, false>(ma, mb, p, tiles, st);
  if (scalar_factor) return launch_kind<K_BLOCK_ROWFAC, false>(ma, mb, p, tiles, st);
  if (column_factor) return launch_kind<K_BLOCK_COLFAC, false>(ma, mb, p, tiles, st);
  return launch_kind<K_BLOCK_GEN, false>(ma, mb, p, tiles, st);
}

}  // namespace i8l

using namespace i8l;

extern "C" int i8l_gemm_block(const int8_t* a_q, const int8_t* b_q, const float* a_scale, const float* b_scale,
                              int a_scale_kind, int b_scale_kind, int b_batched, const void* bias, float post_scale,
                              void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int flags, int32_t* status,
                              void* stream) {
  if (!a_scale || !b_scale) return fail(I8L_ERR_ARG, "null scale pointer");
  if (a_scale_kind != I8L_ASCALE_TILE && a_scale_kind != I8L_ASCALE_GROUP && a_scale_kind != I8L_ASCALE_TILE256)
    return fail(I8L_ERR_ARG, "bad a_scale_kind");
  if (a_scale_kind == I8L_ASCALE_TILE256 && (K % 256 || b_scale_kind != I8L_BSCALE_CHANNEL || (flags & I8L_GEMM_DIVIDE)))
    return fail(I8L_ERR_ARG, "I8L_ASCALE_TILE256 needs K %% 256 == 0 and per-channel b scales");
  if ((flags & I8L_GEMM_PRODUCT_FIRST) && !(flags & I8L_GEMM_EXACT_ORDER))
    return fail(I8L_ERR_ARG, "I8L_GEMM_PRODUCT_FIRST selects an operation order: it needs I8L_GEMM_EXACT_ORDER");
  if (b_scale_kind < I8L_BSCALE_CHANNEL || b_scale_kind > I8L_BSCALE_GROUP) return fail(I8L_ERR_ARG, "bad b_scale_kind");
  if ((flags & I8L_GEMM_DIVIDE) && b_scale_kind == I8L_BSCALE_CHANNEL)
    return fail(I8L_ERR_ARG, "I8L_GEMM_DIVIDE needs per-K-block b scales");
  GemmParams p{};
  p.a_scale = a_scale; p.b_scale = b_scale; p.bias = static_cast<const __nv_bfloat16*>(bias); p.c = c;
  p.status = status; p.b_kind = b_scale_kind; p.b_batched = b_batched ? 1 : 0;
  // 128x256 groups are per-tile scales indexed with a halved K-block number
  p.a_kind = a_scale_kind == I8L_ASCALE_TILE256 ? I8L_ASCALE_TILE : a_scale_kind;
  p.a_kshift = a_scale_kind == I8L_ASCALE_TILE256 ? 1 : 0;
  p.product_first = (flags & I8L_GEMM_PRODUCT_FIRST) ? 1 : 0;
  p.exact = (flags & I8L_GEMM_EXACT_ORDER) ? 1 : 0;
  p.divide = (flags & I8L_GEMM_DIVIDE) ? 1 : 0;
  p.out_f32 = (flags & I8L_GEMM_OUT_F32) ? 1 : 0;
  p.post_scale = post_scale;
  return launch_gemm(true, a_q, b_q, p, batch, M, N, K, static_cast<cudaStream_t>(stream));
}

extern "C" int i8l_gemm_rowcol(const int8_t* a_q, const int8_t* b_q, const float* a_scale, const float* b_scale,
                               int b_batched, const void* bias, float post_scale, void* c, int64_t batch, int64_t M,
                               int64_t N, int64_t K, int flags, int32_t* status, void* stream) {
  if (!a_scale || !b_scale) return fail(I8L_ERR_ARG, "null scale pointer");
  GemmParams p{};
  p.a_scale = a_scale; p.b_scale = b_scale; p.bias = static_cast<const __nv_bfloat16*>(bias); p.c = c;
  p.status = status; p.b_batched = b_batched ? 1 : 0; p.b_kind = I8L_BSCALE_CHANNEL;
  p.out_f32 = (flags & I8L_GEMM_OUT_F32) ? 1 : 0;
  p.post_scale = post_scale;
  return launch_gemm(false, a_q, b_q, p, batch, M, N, K, static_cast<cudaStream_t>(stream));
}

extern "C" int i8l_gemm_dump_i32(const int8_t* a_q, const int8_t* b_q, int b_batched, int32_t* out, int64_t batch,
                                 int64_t M, int64_t N, int64_t K, int per_block, int32_t* status, void* stream) {
  GemmParams p{};
  p.c = out; p.status = status; p.b_batched = b_batched ? 1 : 0; p.dump = per_block ? 2 : 1; p.post_scale = 1.f;
  return launch_gemm(per_block != 0, a_q, b_q, p, batch, M, N, K, static_cast<cudaStream_t>(stream));
}

extern "C" int i8l_gemm_block_scatter(const int8_t* a_q, const int8_t* b_q, const float* a_scale, const float* b_scale,
                                      int b_scale_kind, float post_scale, void* const* c_slots, int world, int rank,
                                      int64_t M, int64_t N, int64_t K, int32_t* status, void* stream) {
  if (!a_scale || !b_scale || !c_slots) return fail(I8L_ERR_ARG, "null pointer");
  if (b_scale_kind != I8L_BSCALE_CHANNEL && b_scale_kind != I8L_BSCALE_TILE) return fail(I8L_ERR_ARG, "bad b_scale_kind");
  if (world < 1 || world > I8L_MAX_RANKS || rank < 0 || rank >= world)
    return fail(I8L_ERR_ARG, "rank %d of %d: at most %d ranks", rank, world, I8L_MAX_RANKS);
  if (M <= 0 || M % ((int64_t)world * 128))
    return fail(I8L_ERR_SHAPE, "M=%lld must split into %d row blocks that are multiples of 128", (long long)M, world);
  GemmParams p{};
  p.a_scale = a_scale; p.b_scale = b_scale; p.status = status;
  p.a_kind = I8L_ASCALE_TILE; p.b_kind = b_scale_kind; p.post_scale = post_scale;
  for (int r = 0; r < world; ++r) {
    if (!c_slots[r] || !aligned16(c_slots[r])) return fail(I8L_ERR_ALIGN, "c_slots[%d] must be a 16-byte aligned device pointer", r);
    p.c_slots[r] = c_slots[r];
  }
  p.c = c_slots[rank];
  p.rs_rows = (int)(M / world);
  p.rs_rank = rank;
  // All ranks walk the row blocks in the same order; starting rank r at the rows of rank r+1 keeps the
  // ranks on different owners at any time (with eight ranks all writing to the same owner the dX GEMM
  // took 5.3 ms instead of 2.5 ms).
  p.m_rot = (int)(((rank + 1) % world) * (M / world / 128));
  return launch_gemm(true, a_q, b_q, p, 1, M, N, K, static_cast<cudaStream_t>(stream));
}

extern "C" int i8l_sum_slots(const void* slots, void* out, int world, int64_t rows, int64_t cols, void* stream) {
  if (!slots || !out) return fail(I8L_ERR_ARG, "null pointer");
  if (world < 1 || rows <= 0 || cols <= 0 || cols % 8) return fail(I8L_ERR_SHAPE, "world >= 1, rows > 0, cols a positive multiple of 8");
  if (!aligned16(slots) || !aligned16(out)) return fail(I8L_ERR_ALIGN, "slots and out must be 16-byte aligned");
  if (int e = check_arch()) return e;
  const int64_t n16 = rows * cols / 8;
  const int64_t want = (n16 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  const int grid = (int)(want < cap ? want : cap);
  sum_slots_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(slots),
                                                                        static_cast<uint4*>(out), world, n16);
  I8L_CUDA_OK(cudaGetLastError());
  return I8L_OK;
}

extern "C" int i8l_set_cta_limit(int max_ctas) {
  if (max_ctas < 0) return fail(I8L_ERR_ARG, "i8l_set_cta_limit: max_ctas must be >= 0");
  g_cta_limit = max_ctas;
  return I8L_OK;
}

extern "C" int i8l_test_set_wait_limit(uint32_t max_polls, int withhold_one_load) {
  g_test_max_polls.store(max_polls, std::memory_order_relaxed);
  g_test_withhold.store(withhold_one_load ? 1 : 0, std::memory_order_relaxed);
  return I8L_OK;
}
