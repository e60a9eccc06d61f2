// Flash attention backward on tcgen05, recompute-based, deterministic (no atomics):
//   delta = rowsum(dO * O)                                  fa_delta_kernel
//   dQ    : one CTA per (query tile, query head, batch)     fa_bwd_dq_kernel
//             per KV block:  S = Q K^T, dP = dO V^T  (TMEM; Q and dO are read from TMEM too)
//                            -> dS = P*(dP-delta)*scale (packed bf16, written back over dP in TMEM)
//                            dQ += dS K               (TMEM accumulator)
//   dK,dV : one CTA per (KV tile, KV head, batch), looping over the query heads of the GQA group
//           and the query tiles that can see the KV tile   fa_bwd_dkv_kernel
//             S^T = K Q^T, dP^T = V dO^T (TMEM) -> P^T, dS^T (packed bf16 over the same columns)
//             dV += P^T dO, dK += dS^T Q             (TMEM accumulators)
// Operands that are needed "transposed" are not copied: the same 128-byte-swizzled shared-memory
// tile is described K-major for one MMA and MN-major for the other.
// Roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..17 softmax
// (four warpgroups, each owning 32 of the 128 score columns of every block).
// Replaces crates/kernels/wgsl/gqa_bwd_{dscores,dv,dq,dk}.wgsl (which read a saved T x T probs buffer).
#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

struct FaBwdArgs {
  const __nv_bfloat16* q;     // [B*T, ldq]: the dQ kernel parks its tile's rows in TMEM
  const __nv_bfloat16* dout;  // [B*T, lddo]
  int ldq, lddo;
  const float* lse;    // [B, hq, T] natural log
  const float* delta;  // [B, hq, T]
  __nv_bfloat16* dQ;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  int lddq, lddk, lddv;
  int B, T, S, hq, hk;
  float scale, scale_log2;
  int causal;
  int* err;
#ifdef BB_TIMELINE
  int dbg;         // profiling builds: bit 0 = softmax phases skip their math, bit 1 = and their TMEM traffic
  long long* tl;  // clock64 stamps of CTA (0,0,0): dQ kernel at [0, 3*4096), dK/dV kernel after it
#endif
};

// Timeline stamps exist only in builds made with -DBB_TIMELINE (a profiling build); the production
// kernels carry no clock reads.
#ifdef BB_TIMELINE
#define BWD_DBG (args.dbg)
#define BWD_TL_DECL(base) long long* tl = ((blockIdx.x | blockIdx.y | blockIdx.z) == 0 && args.tl) ? args.tl + (base) : nullptr
#define BWD_STAMP(slot) do { if (tl && (slot) < 4096 * 3) tl[(slot)] = clock64(); } while (0)
#else
#define BWD_DBG 0
#define BWD_TL_DECL(base) do { } while (0)
#define BWD_STAMP(slot) do { } while (0)
#endif

static constexpr int SUB = 128 * 128;  // bytes of a [128 rows][64 bf16] swizzled sub-tile

// Hoisted descriptor arithmetic for the single MMA-issuing thread: the upper descriptor word is a
// constant, the lower word is (address >> 4) | (lbo >> 4) << 16, so stepping through a tile is one
// 32-bit add per operand instead of rebuilding the 64-bit descriptor.
static constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t base) {
  return ((base & 0x3FFFF) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t base) {
  return ((base & 0x3FFFF) >> 4) | ((uint32_t)(SUB >> 4) << 16);
}
__device__ __forceinline__ uint64_t desc_of(uint32_t lo) { return ((uint64_t)DESC_HI << 32) | lo; }
// offsets, in 16-byte units, of k-step t inside a tile
__device__ __forceinline__ constexpr uint32_t kstep_kmajor(int t) { return (t / 4) * (SUB >> 4) + (t % 4) * 2; }
__device__ __forceinline__ constexpr uint32_t kstep_mnmajor(int t) { return t * 128; }

// ------------------------------------------------------------------------------------ delta
// delta[b, h, t] = sum_d dO[t, h, d] * O[t, h, d].  hd / 8 lanes per (row, head), 16 bytes per lane and
// tensor: the two rows are read once, fully coalesced (the first form read 4 bytes per lane and
// reached 0.37 of the copy bandwidth).  Taking delta inside the dQ kernel instead (the thread that
// parks a dO row in TMEM also reading the O row) was built and measured slower: 1003 against 984 us
// for the whole backward, the row dot product sits in the kernel's serial prologue.
template <int LANES>   // lanes per (row, head) = hd / 8: 16 (hd 128) or 8 (hd 64)
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ o, int ldo,
                                const __nv_bfloat16* __restrict__ dout, int lddo,
                                float* __restrict__ delta, int B, int T, int hq) {
  const long gt = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long item = gt / LANES;            // (row, head)
  const int sub = (int)(gt % LANES);
  const long total = (long)B * T * hq;
  const bool live = item < total;
  const long row = live ? item / hq : 0;
  const int h = live ? (int)(item % hq) : 0;
  float acc = 0.f;
  if (live) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * ldo + h * (LANES * 8) + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dout + row * lddo + h * (LANES * 8) + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc += __uint_as_float(aw[q] << 16) * __uint_as_float(gw[q] << 16);
      acc += __uint_as_float(aw[q] & 0xFFFF0000u) * __uint_as_float(gw[q] & 0xFFFF0000u);
    }
  }
#pragma unroll
  for (int m = LANES / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (live && sub == 0) {
    const int b = (int)(row / T), t = (int)(row % T);
    delta[((size_t)b * hq + h) * T + t] = acc;
  }
}

// ------------------------------------------------------------------------------------ dQ
// One CTA per (query tile, query head, batch) walks the KV blocks its rows can see.  Every MMA is
// 128 wide (see the note on MMA cost at the dK/dV kernel).
// The tile's Q and dO rows are the A operands of every S and dP MMA of the CTA.  Read from shared
// memory they cost 2 x 32 KB of shared-memory bandwidth per block, and with them a block's MMAs move
// 224 KB through shared memory (operands plus the TMA writes of K and V): more than the 128 B/clock
// an SM delivers in the time the math takes.  A timeline build with the softmax work switched off
// measured 2229 clocks per block against 1716 of math.  So the softmax warps park both tiles in TMEM
// once (packed bf16, HD/2 columns each) and the MMAs read them there.
// TMEM (512 columns): S at 0, dP at 128, dQ at 256, Q at 384, dO at 384 + HD/2.
// Softmax warpgroup g (of four) owns key columns [32g, 32g + 32) of every block; the packed bf16 dS it
// produces replaces the first 16 of its own dP columns, so k-step t of the dQ MMA reads its A operand
// at column 32*(t/2) + 8*(t%2) of the dP buffer.  S has one buffer: the softmax warps pull a block's
// scores into registers at once and release the buffer (s_free), so S of the next block is computed
// while they work.  Per block:
//   phase 1  P = exp2(S*c - lse)  (registers only)   | tensor core: dQ of the block before, dP of this one
//   phase 2  dS = P (dP*scale - delta)                | tensor core: S of the next block
// MMAs execute in issue order, so "dP of the next block" may overwrite the columns dQ just read.
// Roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..17 softmax.
template <int HD>
struct DqCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int TILE = NSUB * SUB;
  static constexpr int KST = 3;                     // K stages: S runs a block ahead of dQ, one in flight
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KST * TILE;  // 2 stages
  static constexpr int OFF_BAR = OFF_V + 2 * TILE;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 256, TM_Q = 384, TM_DO = 384 + HD / 2;
};

// Copy one bf16 row of HD elements from global memory into this thread's TMEM lane (packed pairs).
template <int HD>
__device__ __forceinline__ void row_to_tmem(const __nv_bfloat16* src, bool valid, uint32_t taddr) {
#pragma unroll
  for (int c = 0; c < HD / 64; ++c) {
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 x = valid ? __ldg(reinterpret_cast<const uint4*>(src + c * 64) + i)
                            : make_uint4(0u, 0u, 0u, 0u);
      w[4 * i] = x.x;
      w[4 * i + 1] = x.y;
      w[4 * i + 2] = x.z;
      w[4 * i + 3] = x.w;
    }
    tmem_st32(taddr + c * 32, w);
  }
  tmem_wait_st();
}

// Four softmax warpgroups (16 warps) of 32 score columns each: with two (8 warps, 64 columns per
// thread) no pipe was saturated (ncu: 32 % XU, 35 % ALU, 19 % FMA, 1.8 instructions per clock) and
// only two warps per scheduler were there to hide the TMEM round trips; sixteen warps at half the
// registers give every scheduler four.
// Packing to bf16 by TRUNCATION (one PRMT per pair) instead of round-to-nearest (a conversion on the
// unit the exponentials need, or three integer instructions): the value to be packed is first scaled
// by (1 + 0.0029), which is free because it folds into the exponent offset (P) or into the two
// constants of the FMA (dP*scale - delta*scale).  0.0029 is about 3/8 of a bf16 ulp relative to the
// value, so truncation then lands within +-1/2 ulp of the exact value for most mantissas and the
// mean error over mantissas is ~0 (truncation alone would be biased by -1/2 ulp).
static constexpr float kTruncScale = 1.0029f;
static constexpr float kTruncLog2 = 0.0041778f;   // log2(1.0029)
__device__ __forceinline__ uint32_t pack_bf16x2_trunc(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Experiment switch: one exponential in kPolyEvery evaluated by exp2_poly on the FMA pipe instead of
// the special-function unit.  0 = none, which is what measures fastest: with every fourth on the FMA
// pipe the dQ iteration grew from 2812 to 2951 clocks and the dK/dV iteration from 3234 to 4454.
#ifndef BB_FA_POLY_EVERY
#define BB_FA_POLY_EVERY 0
#endif
static constexpr int kPolyEvery = BB_FA_POLY_EVERY;
static constexpr int NWG = 4;
static constexpr int WCOLS = 128 / NWG;               // score columns per warpgroup and block
static constexpr int BWD_THREADS = 64 + 128 * NWG;    // producer warp, MMA warp, softmax warps

// Named barrier over the 128 threads of softmax warpgroup g (barrier 0 is __syncthreads).
__device__ __forceinline__ void wg_sync(int g) {
  asm volatile("bar.sync %0, 128;" ::"r"(g + 1) : "memory");
}

// TMEM column (relative to the operand's base) of k-step t (16 score columns) of a packed bf16 A
// operand: every warpgroup packs its WCOLS columns into the first WCOLS / 2 columns of its own range
__device__ __forceinline__ constexpr uint32_t packed_kstep_col(int t) {
  return (t / (WCOLS / 16)) * WCOLS + (t % (WCOLS / 16)) * 8;
}

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdArgs args) {
  using Cfg = DqCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  constexpr int KST = Cfg::KST;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* qdo_ready = bars;       // Q and dO rows parked in TMEM (256 arrivals)
  uint64_t* k_full = bars + 1;      // KST stages
  uint64_t* k_empty = bars + 4;     // KST
  uint64_t* v_full = bars + 7;      // 2
  uint64_t* v_empty = bars + 9;     // 2
  uint64_t* s_full = bars + 11;     // S of a block is in TMEM
  uint64_t* s_free = bars + 12;     // ... and has been pulled into registers (128 * NWG arrivals)
  uint64_t* dp_full = bars + 13;    // 1
  uint64_t* ds_ready = bars + 14;   // 1 (128 * NWG arrivals)
  uint64_t* dq_done = bars + 15;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int T = args.T, S = args.S;
  const int q0 = qt * 128;
  const int kvh = h / (args.hq / args.hk);
  const int off = S - T;
  int n_blocks = (S + 127) / 128;
  if (args.causal) {
    const int last = (q0 + 127 + off) / 128 + 1;
    n_blocks = last < n_blocks ? last : n_blocks;
  }

  if (threadIdx.x == 0) {
    mbar_init(qdo_ready, 256);
    for (int i = 0; i < KST; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 128 * NWG);
    mbar_init(dp_full, 1);
    mbar_init(ds_ready, 128 * NWG);
    mbar_init(dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base + Cfg::TM_S, tDP = tmem_base + Cfg::TM_DP, tDQ = tmem_base + Cfg::TM_DQ;
  const uint32_t tQ = tmem_base + Cfg::TM_Q, tDO = tmem_base + Cfg::TM_DO;
  BWD_TL_DECL(0);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = 0; j < n_blocks; ++j) {
        const int ks = j % KST, vs = j & 1;
        if (!mbar_wait(&k_empty[ks], ((j / KST) & 1) ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(&k_full[ks], Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sK + ks * Cfg::TILE + c * SUB, &tmK, &k_full[ks], kvh * HD + c * 64, b * S + j * 128);
        if (!mbar_wait(&v_empty[vs], ((j >> 1) & 1) ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(&v_full[vs], Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sV + vs * Cfg::TILE + c * SUB, &tmV, &v_full[vs], kvh * HD + c * 64, b * S + j * 128);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_s = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_dq = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(qdo_ready, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      tc_fence_after();
      // S of block j (A = the Q rows in TMEM; waits for the K tile)
      auto issue_s = [&](int j) -> bool {
        const int ks = j % KST;
        if (!mbar_wait(&k_full[ks], (j / KST) & 1)) return false;
        tc_fence_after();
        const uint32_t lk = desc_lo_kmajor(smem_u32(sK + ks * Cfg::TILE));
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ts(tS, tQ + t * 8, desc_of(lk + kstep_kmajor(t)), idesc_s, t != 0);
        umma_commit(s_full);
        return true;
      };
      // dP of block j (A = the dO rows in TMEM; waits for the V tile, releases it)
      auto issue_dp = [&](int j) -> bool {
        const int vs = j & 1;
        if (!mbar_wait(&v_full[vs], (j >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t lv = desc_lo_kmajor(smem_u32(sV + vs * Cfg::TILE));
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ts(tDP, tDO + t * 8, desc_of(lv + kstep_kmajor(t)), idesc_s, t != 0);
        umma_commit(dp_full);
        umma_commit(&v_empty[vs]);
        return true;
      };
      if (ok) ok = issue_s(0) && issue_dp(0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) {
          // the scores of block j are in registers: the buffer takes the next block's
          if (!mbar_wait(s_free, j & 1)) {
            set_error(args.err, ERR_WAIT_MMA_TMEM);
            ok = false;
            break;
          }
          tc_fence_after();
          if (!issue_s(j + 1)) {
            set_error(args.err, ERR_WAIT_MMA_FULL);
            ok = false;
            break;
          }
        }
        if (!mbar_wait(ds_ready, j & 1)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        BWD_STAMP(4 * j);
        const int ks = j % KST;
        const uint32_t lkm = desc_lo_mnmajor(smem_u32(sK + ks * Cfg::TILE));
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tDQ, tDP + packed_kstep_col(t), desc_of(lkm + kstep_mnmajor(t)), idesc_dq,
                      (j | t) != 0);
        umma_commit(&k_empty[ks]);
        if (j + 1 < n_blocks && !issue_dp(j + 1)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
        }
        BWD_STAMP(4 * j + 1);
      }
      if (ok) umma_commit(dq_done);
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    const int g = (warp - 2) >> 2;  // owns key columns [WCOLS*g, WCOLS*g + WCOLS) of every block
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    const bool row_ok = q_idx < T;
    const size_t stat = ((size_t)b * args.hq + h) * T + (row_ok ? q_idx : 0);
    const float lse2 = row_ok ? args.lse[stat] * 1.4426950408889634f - kTruncLog2 : INFINITY;
    const float scale_t = args.scale * kTruncScale;
    const float dlt = row_ok ? -args.delta[stat] * scale_t : 0.f;  // -delta * scale
    const uint32_t tD = tDP + g * WCOLS + lane_sel;
    const uint32_t tSg = tS + g * WCOLS + lane_sel;
    static_assert(WCOLS == 32, "one 32-column TMEM access per phase and thread");
    // warpgroup 0 parks the Q rows of the tile in TMEM, warpgroup 1 the dO rows (one row per thread)
    if (g < 2) {
      const size_t grow = (size_t)(b * T + (row_ok ? q_idx : 0));
      const __nv_bfloat16* src = (g == 0 ? args.q + grow * args.ldq : args.dout + grow * args.lddo) + h * HD;
      row_to_tmem<HD>(src, row_ok, (g == 0 ? tQ : tDO) + lane_sel);
      tc_fence_before();
      mbar_arrive(qdo_ready);
    }
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      // ---- phase 1: P (kept packed in registers)
      const bool stamper = g < 2 && (warp & 3) == 2 && lane == 0;
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * j);
      ok = mbar_wait(s_full, j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * j + 1);
      const int kvb = j * 128 + g * WCOLS;
      const bool need_mask = (kvb + WCOLS - 1 > kv_limit_row);
      const int lim = kv_limit_row - kvb;   // columns <= lim are visible
      uint32_t pk[16];
      {
        uint32_t rs[32];
        __syncwarp();
        if (!(BWD_DBG & 2)) {
          tmem_ld32(tSg, rs);
          tmem_wait_ld();
        }
        // the block's scores are in registers: the S buffer may take the next block's
        tc_fence_before();
        mbar_arrive(s_free);
        if (BWD_DBG & 1) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) pk[i >> 1] = (BWD_DBG & 2) ? 0u : rs[i];
        } else
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(rs[i]) * args.scale_log2 - lse2);
          // every fourth exponential runs as a polynomial on the FMA pipe (kPolyEvery)
          const float x1 = __uint_as_float(rs[i + 1]) * args.scale_log2 - lse2;
          float p1 = (kPolyEvery && (i + 1) % (kPolyEvery ? kPolyEvery : 1) == kPolyEvery - 1) ? exp2_poly(x1) : exp2f(x1);
          if (need_mask) {
            if (i > lim) p0 = 0.f;
            if (i + 1 > lim) p1 = 0.f;
          }
          pk[i >> 1] = pack_bf16x2_trunc(p0, p1);
        }
      }
      // ---- phase 2: dS = P * (dP * scale - delta * scale), packed over this warpgroup's dP columns
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * j + 2);
      ok = mbar_wait(dp_full, j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * j + 3);
      {
        uint32_t rp[32];
        __syncwarp();
        if (!(BWD_DBG & 2)) {
          tmem_ld32(tD, rp);
          tmem_wait_ld();
        }
        if (BWD_DBG & 1) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) pk[i >> 1] ^= (BWD_DBG & 2) ? 0u : rp[i];
        } else
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          // the factor is packed by truncation (see kTruncScale) and multiplied in bf16x2: one FMA per
          // element, one PRMT and one packed multiply per pair, nothing on the conversion unit
          const uint32_t t = pack_bf16x2_trunc(fmaf(__uint_as_float(rp[i]), scale_t, dlt),
                                               fmaf(__uint_as_float(rp[i + 1]), scale_t, dlt));
          pk[i >> 1] = mul_bf16x2(pk[i >> 1], t);
        }
      }
      if (!(BWD_DBG & 2)) {
        tmem_st16(tD, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(ds_ready);
    }
    if (ok && n_blocks > 0) {
      ok = mbar_wait(dq_done, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      // the warpgroups share the 32-column chunks of dQ round-robin
      __nv_bfloat16* orow = args.dQ + (size_t)(b * T + q_idx) * args.lddq + h * HD;
#pragma unroll 1
      for (int c = g; c < HD / 32; c += NWG) {
        uint32_t r[32];
        __syncwarp();
        if (n_blocks > 0) {
          tmem_ld32(tDQ + lane_sel + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------ dK, dV
// One CTA per (KV tile, KV head, batch) loops over the query heads of the GQA group and the query
// tiles that can see the KV tile.  Every MMA is 128 wide: on this part a tcgen05.mma with M = 128,
// K = 16 takes about 68 clocks for any N <= 128 (129 at N = 256), so narrower tiles waste the
// tensor pipe in proportion.
// TMEM (512 columns, all used): S^T at 0 and dP^T at 128 (128 fp32 columns each: one column per
// query of the tile), dV at 256, dK at 384.  Softmax warpgroup g (of four) owns query columns
// [32g, 32g+32): it replaces the first 16 of ITS OWN columns by the packed bf16 P^T (then dS^T) values,
// so the warpgroups never touch each other's columns and the A operand of k-step t of the dV / dK
// MMAs sits at column 32*(t/2) + 8*(t%2).
// The work of an iteration is cut in two phases so that the tensor core always has MMAs queued:
//   phase 1  P^T = exp2(S^T*c - lse)           -> tensor core: dV += P^T dO, then S^T of the next tile
//   phase 2  dS^T = P^T (dP^T*scale - delta)   -> tensor core: dK += dS^T Q, then dP^T of the next tile
// MMAs execute in issue order, so "S^T of the next tile" may overwrite the columns dV just read.
template <int HD>
struct DkvCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int TILE = NSUB * SUB;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE;
  static constexpr int OFF_Q = OFF_V + TILE;        // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * TILE;   // 2 stages
  static constexpr int OFF_STAT = OFF_DO + 2 * TILE;  // per warpgroup: lse2[64], delta[64]
  static constexpr int OFF_RAW = OFF_STAT + 1024;     // per warpgroup: 2 stages x 64 raw values
  static constexpr int OFF_BAR = OFF_RAW + 2048;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
  static constexpr uint32_t TM_ST = 0, TM_DPT = 128, TM_DV = 256, TM_DK = 384;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                  const FaBwdArgs args) {
  using Cfg = DkvCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;         // K and V tiles (once)
  uint64_t* qdo_full = bars + 1;    // 2 stages: Q and dO of an iteration
  uint64_t* qdo_empty = bars + 3;   // 2
  uint64_t* st_full = bars + 5;     // S^T of the iteration is in TMEM
  uint64_t* dpt_full = bars + 6;    // dP^T of the iteration is in TMEM
  uint64_t* p_ready = bars + 7;     // P^T written (256 arrivals)
  uint64_t* ds_ready = bars + 8;    // dS^T written (256 arrivals)
  uint64_t* dkv_done = bars + 9;    // all dV/dK MMAs finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int T = args.T, S = args.S;
  const int kv0 = kt * 128;
  const int group = args.hq / args.hk;
  const int off = S - T;
  const int n_qt = (T + 127) / 128;
  // first query tile that can see this KV tile: q_idx + off >= kv0  <=>  q_idx >= kv0 - off
  int qt_first = 0;
  if (args.causal) {
    const int qmin = kv0 - off;
    qt_first = qmin > 0 ? qmin / 128 : 0;
  }
  const int per_head = n_qt - qt_first;
  const int n_iter = per_head > 0 ? per_head * group : 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(dpt_full, 1);
    mbar_init(p_ready, 128 * NWG);
    mbar_init(ds_ready, 128 * NWG);
    mbar_init(dkv_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tST = tmem_base + Cfg::TM_ST, tDPT = tmem_base + Cfg::TM_DPT;
  const uint32_t tDV = tmem_base + Cfg::TM_DV, tDK = tmem_base + Cfg::TM_DK;
  BWD_TL_DECL(3 * 4096);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::TILE);
#pragma unroll
      for (int c = 0; c < NSUB; ++c) {
        tma_load_2d(sK + c * SUB, &tmK, kv_full, kvh * HD + c * 64, b * S + kv0);
        tma_load_2d(sV + c * SUB, &tmV, kv_full, kvh * HD + c * 64, b * S + kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int h = kvh * group + it / per_head;
        const int qt = qt_first + it % per_head;
        const int st = it & 1;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(&qdo_full[st], 2 * Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c) {
          tma_load_2d(sQ + st * Cfg::TILE + c * SUB, &tmQ, &qdo_full[st], h * HD + c * 64,
                      b * T + qt * 128);
          tma_load_2d(sDO + st * Cfg::TILE + c * SUB, &tmDO, &qdo_full[st], h * HD + c * 64,
                      b * T + qt * 128);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_st = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_acc = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      const uint32_t lkk = desc_lo_kmajor(smem_u32(sK)), lvv = desc_lo_kmajor(smem_u32(sV));
      auto issue_st = [&](int st) {      // S^T = K Q^T for the 128 queries of stage st
        const uint32_t lq = desc_lo_kmajor(smem_u32(sQ + st * Cfg::TILE));
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tST, desc_of(lkk + kstep_kmajor(t)), desc_of(lq + kstep_kmajor(t)), idesc_st, t != 0);
        umma_commit(st_full);
      };
      auto issue_dpt = [&](int st) {     // dP^T = V dO^T
        const uint32_t ldo = desc_lo_kmajor(smem_u32(sDO + st * Cfg::TILE));
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tDPT, desc_of(lvv + kstep_kmajor(t)), desc_of(ldo + kstep_kmajor(t)), idesc_st, t != 0);
        umma_commit(dpt_full);
      };
      if (ok) {
        if (!mbar_wait(&qdo_full[0], 0)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
        } else {
          tc_fence_after();
          issue_st(0);
          issue_dpt(0);
        }
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1;
        const uint32_t lqm = desc_lo_mnmajor(smem_u32(sQ + st * Cfg::TILE));
        const uint32_t ldom = desc_lo_mnmajor(smem_u32(sDO + st * Cfg::TILE));
        // ---- after phase 1: dV += P^T dO, then S^T of the next tile
        if (!mbar_wait(p_ready, ph)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        BWD_STAMP(4 * it);
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tDV, tST + packed_kstep_col(t), desc_of(ldom + kstep_mnmajor(t)), idesc_acc,
                      (it | t) != 0);
        if (it + 1 < n_iter) {
          if (!mbar_wait(&qdo_full[st ^ 1], ((it + 1) >> 1) & 1)) {
            set_error(args.err, ERR_WAIT_MMA_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_st(st ^ 1);
        }
        BWD_STAMP(4 * it + 1);
        // ---- after phase 2: dK += dS^T Q, then dP^T of the next tile
        if (!mbar_wait(ds_ready, ph)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        BWD_STAMP(4 * it + 2);
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tDK, tDPT + packed_kstep_col(t), desc_of(lqm + kstep_mnmajor(t)), idesc_acc,
                      (it | t) != 0);
        umma_commit(&qdo_empty[st]);   // both tiles of this stage have been read
        if (it + 1 < n_iter) issue_dpt(st ^ 1);
        BWD_STAMP(4 * it + 3);
      }
      if (ok) umma_commit(dkv_done);
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    const int g = (warp - 2) >> 2;    // owns query columns [WCOLS*g, WCOLS*g + WCOLS) of every tile
    const int sw = warp & 3;
    const int row = sw * 32 + lane;   // kv row inside the tile
    const int kv_idx = kv0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int wt = threadIdx.x - 64 - g * 128;  // 0..127 inside the warpgroup
    float* ls = s_stat + g * (2 * WCOLS);       // lse2 of this warpgroup's query columns
    float* dl = ls + WCOLS;                     // -delta * scale of the same columns
    const uint32_t tS = tST + g * WCOLS + lane_sel, tD = tDPT + g * WCOLS + lane_sel;
    static_assert(WCOLS == 32, "one 32-column TMEM access per phase and thread");
    // Per-query statistics of iteration i: threads 0..31 of the warpgroup fetch lse, threads 32..63
    // delta, one value each, with a 4-byte cp.async into a two-stage raw buffer one iteration ahead
    // (a plain global load issued "early" can be moved next to its use by the compiler, which put
    // a full memory latency at the top of every iteration); the same thread later converts its own
    // value (lse -> log2 units minus the truncation offset, delta -> -delta * scale) into ls / dl.
    float* raw = reinterpret_cast<float*>(smem + Cfg::OFF_RAW) + g * (4 * WCOLS);
    auto fetch_stat = [&](int i) {
      if (wt >= 2 * WCOLS) return;
      const int hh = kvh * group + i / per_head;
      const int qi = (qt_first + i % per_head) * 128 + g * WCOLS + (wt & (WCOLS - 1));
      const size_t stat = ((size_t)b * args.hq + hh) * T + (qi < T ? qi : 0);
      const float* src = (wt < WCOLS ? args.lse : args.delta) + stat;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(raw + (i & 1) * (2 * WCOLS) + wt)),
                   "l"(src)
                   : "memory");
    };
    if (n_iter > 0) fetch_stat(0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    bool ok = true;
    const float scale_t = args.scale * kTruncScale;
    for (int it = 0; it < n_iter; ++it) {
      const int qt = qt_first + it % per_head;
      const int q0 = qt * 128 + g * WCOLS;
      const uint32_t ph = it & 1;
      {
        asm volatile("cp.async.wait_group 0;" ::: "memory");   // this thread's value of iteration it
        wg_sync(g);                                            // previous iteration's reads of ls / dl done
        if (wt < 2 * WCOLS) {
          const float r = raw[(it & 1) * (2 * WCOLS) + wt];
          const bool qok = qt * 128 + g * WCOLS + (wt & (WCOLS - 1)) < T;
          ls[wt] = wt < WCOLS ? (qok ? r * 1.4426950408889634f - kTruncLog2 : INFINITY)
                              : (qok ? -r * scale_t : 0.f);    // wt >= WCOLS lands in dl[]
        }
        if (it + 1 < n_iter) fetch_stat(it + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        wg_sync(g);
      }
      // column (query) c is visible from this kv row iff kv_idx <= q + off  <=>  q >= kv_idx - off
      const int q_min = args.causal ? (kv_idx - off) : -0x40000000;
      const bool need_mask = args.causal && (q0 < q_min);
      const int first_ok = q_min - q0;  // columns i >= first_ok are visible
      // ---- phase 1: P^T
      const bool stamper = g < 2 && (warp & 3) == 2 && lane == 0;
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * it);
      ok = mbar_wait(st_full, ph);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * it + 1);
      uint32_t pk[16];
      {
        uint32_t rs[32];
        __syncwarp();
        if (!(BWD_DBG & 2)) {
          tmem_ld32(tS, rs);
          tmem_wait_ld();
        }
        const float4* ls4 = reinterpret_cast<const float4*>(ls);
        if (BWD_DBG & 1) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) pk[i >> 1] = (BWD_DBG & 2) ? 0u : rs[i];
        } else
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l = ls4[i >> 2];
          float p0 = exp2f(__uint_as_float(rs[i]) * args.scale_log2 - l.x);
          float p1 = exp2f(__uint_as_float(rs[i + 1]) * args.scale_log2 - l.y);
          float p2 = exp2f(__uint_as_float(rs[i + 2]) * args.scale_log2 - l.z);
          const float x3 = __uint_as_float(rs[i + 3]) * args.scale_log2 - l.w;
          float p3 = (kPolyEvery && (i + 3) % (kPolyEvery ? kPolyEvery : 1) == kPolyEvery - 1) ? exp2_poly(x3) : exp2f(x3);
          if (need_mask) {
            if (i < first_ok) p0 = 0.f;
            if (i + 1 < first_ok) p1 = 0.f;
            if (i + 2 < first_ok) p2 = 0.f;
            if (i + 3 < first_ok) p3 = 0.f;
          }
          pk[i >> 1] = pack_bf16x2_trunc(p0, p1);
          pk[(i >> 1) + 1] = pack_bf16x2_trunc(p2, p3);
        }
      }
      // this warpgroup's S^T columns are in registers: the packed P^T may overwrite them
      if (!(BWD_DBG & 2)) {
        tmem_st16(tS, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(p_ready);
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * it + 2);
      // ---- phase 2: dS^T = P^T * (dP^T * scale - delta * scale), P^T as it was rounded for the MMA
      ok = mbar_wait(dpt_full, ph);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (stamper) BWD_STAMP(4096 * (1 + g) + 4 * it + 3);
      {
        uint32_t rp[32];
        __syncwarp();
        if (!(BWD_DBG & 2)) {
          tmem_ld32(tD, rp);
          tmem_wait_ld();
        }
        const float4* dl4 = reinterpret_cast<const float4*>(dl);
        if (BWD_DBG & 1) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) pk[i >> 1] ^= (BWD_DBG & 2) ? 0u : rp[i];
        } else
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 d = dl4[i >> 2];
          const uint32_t t0 = pack_bf16x2_trunc(fmaf(__uint_as_float(rp[i]), scale_t, d.x),
                                                fmaf(__uint_as_float(rp[i + 1]), scale_t, d.y));
          const uint32_t t1 = pack_bf16x2_trunc(fmaf(__uint_as_float(rp[i + 2]), scale_t, d.z),
                                                fmaf(__uint_as_float(rp[i + 3]), scale_t, d.w));
          pk[i >> 1] = mul_bf16x2(pk[i >> 1], t0);
          pk[(i >> 1) + 1] = mul_bf16x2(pk[(i >> 1) + 1], t1);
        }
      }
      if (!(BWD_DBG & 2)) {
        tmem_st16(tD, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(ds_ready);
    }
    if (ok && n_iter > 0) {
      ok = mbar_wait(dkv_done, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      // the lower half of the warpgroups writes dV, the upper half dK; each pair shares the chunks
      const bool row_ok = kv_idx < S;
      const bool is_k = g >= NWG / 2;
      __nv_bfloat16* drow = (is_k ? args.dK + (size_t)(b * S + kv_idx) * args.lddk
                                  : args.dV + (size_t)(b * S + kv_idx) * args.lddv) + kvh * HD;
#pragma unroll 1
      for (int c = g % (NWG / 2); c < HD / 32; c += NWG / 2) {
        uint32_t r[32];
        __syncwarp();
        if (n_iter > 0) {
          tmem_ld32((is_k ? tDK : tDV) + lane_sel + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
          __nv_bfloat16* dst = drow + c * 32;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + q * 8) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
static int launch_fa_bwd(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                         const void* dout, int lddo, const FaBwdArgs& a, cudaStream_t stream) {
  CUtensorMap tmQ, tmK, tmV, tmDO;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = make_tmap_2d(&tmQ, bf, 2, q, (uint64_t)a.hq * HD, (uint64_t)a.B * a.T, (uint64_t)ldq * 2,
                        64, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, bf, 2, k, (uint64_t)a.hk * HD, (uint64_t)a.B * a.S, (uint64_t)ldk * 2, 64,
                    128);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, bf, 2, v, (uint64_t)a.hk * HD, (uint64_t)a.B * a.S, (uint64_t)ldv * 2, 64,
                    128);
  if (rc) return rc;
  rc = make_tmap_2d(&tmDO, bf, 2, dout, (uint64_t)a.hq * HD, (uint64_t)a.B * a.T,
                    (uint64_t)lddo * 2, 64, 128);
  if (rc) return rc;
  static PerDeviceOnce once_dq, once_dkv;
  {
    cudaError_t e = ensure_dyn_smem(once_dq, fa_bwd_dq_kernel<HD>, DqCfg<HD>::SMEM);
    if (e != cudaSuccess) return (int)e;
    e = ensure_dyn_smem(once_dkv, fa_bwd_dkv_kernel<HD>, DkvCfg<HD>::SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 gq((a.T + 127) / 128, a.hq, a.B);
  fa_bwd_dq_kernel<HD><<<gq, BWD_THREADS, DqCfg<HD>::SMEM, stream>>>(tmQ, tmK, tmV, tmDO, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  dim3 gk((a.S + 127) / 128, a.hk, a.B);
  fa_bwd_dkv_kernel<HD><<<gk, BWD_THREADS, DkvCfg<HD>::SMEM, stream>>>(tmQ, tmK, tmV, tmDO, a);
  return (int)cudaGetLastError();
}

}  // namespace bb

#ifdef BB_TIMELINE
static long long* g_bwd_timeline = nullptr;
// Profiling builds only: device buffer of 6*4096 int64 that CTA (0,0,0) of each kernel stamps.
BB_API int bb_flash_bwd_timeline(long long* buf) {
  g_bwd_timeline = buf;
  return 0;
}
#endif

// Backward of bb_flash_fwd.  `out`/`dout`: [B*T, ld]; lse from the forward; delta: scratch
// [B, hq, T] fp32 written here; dq/dk/dv: [B*T or B*S, ld] bf16, fully overwritten.
BB_API int bb_flash_bwd(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                        const void* out, int ldo, const void* dout, int lddo, const float* lse,
                        float* delta, void* dq, int lddq, void* dk, int lddk, void* dv, int lddv,
                        int B, int T, int S, int hq, int hk, int hd, float scale, int causal,
                        void* stream) {
  using namespace bb;
  if (B <= 0 || T <= 0 || S < T || hq % hk) return BB_EARG;
  if ((lddq % 8) || (lddk % 8) || (lddv % 8)) return BB_EARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    // 16-byte loads: the row pitches and the head offset must keep them aligned
    if ((ldo % 8) || (lddo % 8) || (hd != 64 && hd != 128)) return BB_EARG;
    const long threads = (long)B * T * hq * (hd / 8);
    const int blocks = (int)((threads + 255) / 256);
    if (hd == 128)
      fa_delta_kernel<16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)out, ldo, (const __nv_bfloat16*)dout, lddo,
                                                 delta, B, T, hq);
    else
      fa_delta_kernel<8><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)out, ldo, (const __nv_bfloat16*)dout, lddo,
                                                delta, B, T, hq);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  FaBwdArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.dout = static_cast<const __nv_bfloat16*>(dout);
  a.ldq = ldq;
  a.lddo = lddo;
  a.lse = lse;
  a.delta = delta;
  a.dQ = static_cast<__nv_bfloat16*>(dq);
  a.dK = static_cast<__nv_bfloat16*>(dk);
  a.dV = static_cast<__nv_bfloat16*>(dv);
  a.lddq = lddq;
  a.lddk = lddk;
  a.lddv = lddv;
  a.B = B;
  a.T = T;
  a.S = S;
  a.hq = hq;
  a.hk = hk;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.err = device_error_word();
#ifdef BB_TIMELINE
  a.tl = g_bwd_timeline;
  {
    const char* e = std::getenv("BB_FA_DEBUG");   // profiling builds only
    a.dbg = e ? std::atoi(e) : 0;
  }
#endif
  if (hd == 128) return launch_fa_bwd<128>(q, ldq, k, ldk, v, ldv, dout, lddo, a, s);
  if (hd == 64) return launch_fa_bwd<64>(q, ldq, k, ldk, v, ldv, dout, lddo, a, s);
  return BB_EARG;
}
