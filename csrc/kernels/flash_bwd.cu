// Flash attention backward on tcgen05, recompute-based, deterministic (no atomics):
//   delta = rowsum(dO * O)                                  fa_delta_kernel
//   dQ    : one CTA per (query tile, query head, batch)     fa_bwd_dq_kernel
//             per KV block:  S = Q K^T, dP = dO V^T  (TMEM) -> dS = P*(dP-delta)*scale (packed bf16,
//                            written back over S in TMEM)
//                            dQ += dS K               (TMEM accumulator)
//   dK,dV : one CTA per (KV tile, KV head, batch), looping over the query heads of the GQA group
//           and the query tiles that can see the KV tile   fa_bwd_dkv_kernel
//             S^T = K Q^T, dP^T = V dO^T (TMEM) -> P^T, dS^T (packed bf16 over the same columns)
//             dV += P^T dO, dK += dS^T Q             (TMEM accumulators)
// Operands that are needed "transposed" are not copied: the same 128-byte-swizzled shared-memory
// tile is described K-major for one MMA and MN-major for the other.
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9 softmax
// (two warpgroups that alternate 64-wide units so the tensor core never waits for the exponentials).
// Replaces crates/kernels/wgsl/gqa_bwd_{dscores,dv,dq,dk}.wgsl (which read a saved T x T probs buffer).
#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

struct FaBwdArgs {
  // row-major operands as plain pointers (leading dimensions in elements): the tiles that stay
  // resident for a whole CTA are copied global -> registers -> TMEM by the softmax warps
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* dout;
  int ldq, ldk, ldv, lddo;
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
  long long* tl;  // optional clock64 stamps of CTA (0,0,0): [0,4096) MMA, then one 4096 block per warpgroup
};

static constexpr int SUB = 128 * 128;  // bytes of a [128 rows][64 bf16] swizzled sub-tile

// Write 32 consecutive bf16 (columns c0..c0+31 of `row`) of a [128][128] operand tile stored as two
// K-major 128B-swizzled sub-tiles.
__device__ __forceinline__ void store_row_chunk32(uint8_t* tile, int row, int c, const uint32_t (&pk)[16]) {
  uint8_t* prow = tile + (c >> 1) * SUB + row * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int chunk = ((c & 1) * 4 + q) ^ (row & 7);
    *reinterpret_cast<uint4*>(prow + chunk * 16) =
        make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
  }
}

// K-major A/B operand: k-step t covers 16 columns: sub-tile t/4, 32-byte offset (t%4)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int t) {
  return umma_smem_desc(base + (t / 4) * SUB + (t % 4) * 32, 16, 1024);
}
// MN-major B operand over a [rows = K][HD] tile: k-step t covers 16 rows
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int t) {
  return umma_smem_desc(base + t * 2048, SUB, 1024);
}

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
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ o, int ldo,
                                const __nv_bfloat16* __restrict__ dout, int lddo,
                                float* __restrict__ delta, int B, int T, int hq, int hd) {
  const long gw = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = (long)B * T * hq;
  if (gw >= total) return;
  const long row = gw / hq;
  const int h = (int)(gw % hq);
  const __nv_bfloat16* op = o + row * ldo + h * hd;
  const __nv_bfloat16* dp = dout + row * lddo + h * hd;
  float acc = 0.f;
  for (int i = lane * 2; i < hd; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + i));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + i));
    acc += a.x * g.x + a.y * g.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const int b = (int)(row / T), t = (int)(row % T);
    delta[((size_t)b * hq + h) * T + t] = acc;
  }
}

// ------------------------------------------------------------------------------------ dQ
// Work is cut into UNITS of 64 key columns.  Two softmax warpgroups alternate units (warpgroup g
// owns half g of every 128-row K/V tile and TMEM buffer g), so while one warpgroup turns S/dP of
// its unit into dS, the tensor core already runs S/dP of the other unit and the dQ MMA of the unit
// before: tensor-core order is  SdP(0,0) SdP(0,1) dQ(0,0) SdP(1,0) dQ(0,1) SdP(1,1) dQ(1,0) ...
// MMAs execute in issue order, so S of unit (j+1,g) may be issued straight after dQ of unit (j,g)
// although it overwrites the TMEM columns that dQ reads its dS operand from.
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9 softmax.
// TMEM columns: S[g] at g*64, dP[g] at 128 + g*64 (64 fp32 columns each; the packed bf16 dS of a
// unit overwrites the first 32 columns of its S buffer), dQ at 256, and the CTA's Q and dO tiles as
// packed bf16 at 384 and 448 (HD/2 columns each).  Q and dO are the A operands of every S and dP
// MMA of the CTA: held in TMEM they cost no shared-memory bandwidth, which is what bounds an
// M=128, N=64 MMA whose A operand comes from shared memory (4 KB of A against 2 KB of B per k-step).
template <int HD>
struct DqCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int TILE = NSUB * SUB;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + 2 * TILE;
  static constexpr int OFF_BAR = OFF_V + 2 * TILE;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
  static constexpr uint32_t TM_DQ = 256, TM_Q = 384, TM_DO = 448;
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

static constexpr int BWD_THREADS = 320;

#define BWD_STAMP(slot) do { if (tl) tl[(slot)] = clock64(); } while (0)

// Named barrier over the 128 threads of softmax warpgroup g (barrier 0 is __syncthreads).
__device__ __forceinline__ void wg_sync(int g) {
  if (g == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  else asm volatile("bar.sync 2, 128;" ::: "memory");
}

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdArgs args) {
  using Cfg = DqCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* qdo_ready = bars;      // Q and dO rows stored to TMEM (256 arrivals)
  uint64_t* k_full = bars + 1;     // 2 stages
  uint64_t* k_empty = bars + 3;    // 2
  uint64_t* v_full = bars + 5;     // 2
  uint64_t* v_empty = bars + 7;    // 2
  uint64_t* sdp_full = bars + 9;   // 2 (one per TMEM buffer / warpgroup)
  uint64_t* ds_ready = bars + 11;  // 2 (128 arrivals each)
  uint64_t* dq_done = bars + 13;   // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&ds_ready[i], 128);
    }
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
  const uint32_t tDQ = tmem_base + Cfg::TM_DQ;
  const uint32_t tQ = tmem_base + Cfg::TM_Q, tDO = tmem_base + Cfg::TM_DO;
  long long* tl = (blockIdx.x | blockIdx.y | blockIdx.z) == 0 ? args.tl : nullptr;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1) || !mbar_wait(&v_empty[st], ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          ok = false;
          break;
        }
        mbar_expect_tx(&k_full[st], Cfg::TILE);
        mbar_expect_tx(&v_full[st], Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c) {
          tma_load_2d(sK + st * Cfg::TILE + c * SUB, &tmK, &k_full[st], kvh * HD + c * 64,
                      b * S + j * 128);
          tma_load_2d(sV + st * Cfg::TILE + c * SUB, &tmV, &v_full[st], kvh * HD + c * 64,
                      b * S + j * 128);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(1, 1, 1, 0, 0, 128, 64);
      constexpr uint32_t idesc_dq = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(qdo_ready, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      tc_fence_after();
      // S and dP of half g of block j into TMEM buffer g (A = Q / dO rows resident in TMEM)
      auto issue_sdp = [&](int j, int g) {
        const int st = j & 1;
        const uint32_t lk = desc_lo_kmajor(smem_u32(sK + st * Cfg::TILE) + g * 8192);
        const uint32_t lv = desc_lo_kmajor(smem_u32(sV + st * Cfg::TILE) + g * 8192);
        const uint32_t tS = tmem_base + g * 64, tDP = tmem_base + 128 + g * 64;
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ts(tS, tQ + t * 8, desc_of(lk + kstep_kmajor(t)), idesc_s, t != 0);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ts(tDP, tDO + t * 8, desc_of(lv + kstep_kmajor(t)), idesc_s, t != 0);
        umma_commit(&sdp_full[g]);
        if (g == 1) umma_commit(&v_empty[st]);
      };
      if (ok && n_blocks > 0) {
        if (!mbar_wait(&k_full[0], 0) || !mbar_wait(&v_full[0], 0)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
        } else {
          tc_fence_after();
          issue_sdp(0, 0);
          issue_sdp(0, 1);
        }
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t lkm = desc_lo_mnmajor(smem_u32(sK + st * Cfg::TILE));
        for (int g = 0; g < 2 && ok; ++g) {
          if (!mbar_wait(&ds_ready[g], j & 1)) {
            set_error(args.err, ERR_WAIT_MMA_TMEM);
            ok = false;
            break;
          }
          tc_fence_after();
          if (2 * j + g < 1024) BWD_STAMP(4 * j + 2 * g);
          const uint32_t tS = tmem_base + g * 64;
#pragma unroll
          for (int t = 0; t < 4; ++t)
            umma_f16_ts(tDQ, tS + t * 8, desc_of(lkm + g * 512 + kstep_mnmajor(t)), idesc_dq,
                        (j | g | t) != 0);
          if (g == 1) umma_commit(&k_empty[st]);
          if (j + 1 < n_blocks) {
            if (g == 0) {
              const uint32_t ph = ((j + 1) >> 1) & 1;
              if (!mbar_wait(&k_full[st ^ 1], ph) || !mbar_wait(&v_full[st ^ 1], ph)) {
                set_error(args.err, ERR_WAIT_MMA_FULL);
                ok = false;
                break;
              }
              tc_fence_after();
            }
            issue_sdp(j + 1, g);
          }
          if (2 * j + g < 1024) BWD_STAMP(4 * j + 2 * g + 1);
        }
      }
      if (ok) umma_commit(dq_done);
    }
  } else {
    const int g = (warp - 2) >> 2;  // warpgroup = half of every K/V tile = TMEM buffer
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    const bool row_ok = q_idx < T;
    const size_t stat = ((size_t)b * args.hq + h) * T + (row_ok ? q_idx : 0);
    const float lse2 = row_ok ? args.lse[stat] * 1.4426950408889634f : INFINITY;
    const float dlt = row_ok ? -args.delta[stat] * args.scale : 0.f;  // -delta * scale
    const uint32_t tS = tmem_base + g * 64 + lane_sel, tDP = tmem_base + 128 + g * 64 + lane_sel;
    // warpgroup 0 parks the Q tile in TMEM, warpgroup 1 the dO tile (one row per thread)
    {
      const size_t grow = (size_t)(b * T + (row_ok ? q_idx : 0));
      const __nv_bfloat16* src = (g == 0 ? args.q + grow * args.ldq : args.dout + grow * args.lddo) + h * HD;
      row_to_tmem<HD>(src, row_ok, (g == 0 ? tQ : tDO) + lane_sel);
      tc_fence_before();
      mbar_arrive(qdo_ready);
    }
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(&sdp_full[g], j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if ((warp & 3) == 2 && lane == 0 && j < 1024) BWD_STAMP(4096 * (1 + g) + 2 * j);
      const int kv0 = j * 128 + g * 64;
      const bool need_mask = (kv0 + 63 > kv_limit_row);
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        __syncwarp();
        tmem_ld32(tS + c * 32, rs);
        tmem_ld32(tDP + c * 32, rp);
        tmem_wait_ld();
        const int lim = kv_limit_row - (kv0 + c * 32);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(rs[i]) * args.scale_log2 - lse2);
          float p1 = exp2f(__uint_as_float(rs[i + 1]) * args.scale_log2 - lse2);
          if (need_mask) {
            if (i > lim) p0 = 0.f;
            if (i + 1 > lim) p1 = 0.f;
          }
          pk[c * 16 + (i >> 1)] = pack_bf16x2_alu(p0 * fmaf(__uint_as_float(rp[i]), args.scale, dlt),
                                              p1 * fmaf(__uint_as_float(rp[i + 1]), args.scale, dlt));
        }
      }
      // all 64 S columns of this unit are in registers: the packed dS may overwrite them
      tmem_st32(tS, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&ds_ready[g]);
      if ((warp & 3) == 2 && lane == 0 && j < 1024) BWD_STAMP(4096 * (1 + g) + 2 * j + 1);
    }
    if (ok) {
      ok = mbar_wait(dq_done, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      // warpgroup g writes columns [g*HD/2, (g+1)*HD/2) of dQ
      __nv_bfloat16* orow = args.dQ + (size_t)(b * T + q_idx) * args.lddq + h * HD;
#pragma unroll 1
      for (int c = g * (HD / 64); c < (g + 1) * (HD / 64); ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tDQ + lane_sel + c * 32, r);
        tmem_wait_ld();
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
// Same unit pipeline with the roles of rows and columns swapped: a unit is 64 QUERY rows of the
// current (head, query tile) iteration; warpgroup g owns half g of every 128-row Q/dO tile.
// TMEM columns: S^T[g] at g*64, dP^T[g] at 128 + g*64, dV at 256, dK at 384.  P^T (packed bf16)
// overwrites the first 32 columns of its S^T buffer, dS^T those of its dP^T buffer.
template <int HD>
struct DkvCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int TILE = NSUB * SUB;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE;
  static constexpr int OFF_Q = OFF_V + TILE;        // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * TILE;   // 2 stages
  static constexpr int OFF_STAT = OFF_DO + 2 * TILE;  // per warpgroup: lse2[64], delta[64]
  static constexpr int OFF_BAR = OFF_STAT + 1024;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
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
  uint64_t* st_full = bars + 5;     // 2: S^T and dP^T of a unit ready in TMEM buffer g
  uint64_t* pds_ready = bars + 7;   // 2: P^T, dS^T written (128 arrivals each)
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
      mbar_init(&st_full[i], 1);
      mbar_init(&pds_ready[i], 128);
    }
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
  const uint32_t tDV = tmem_base + 256, tDK = tmem_base + 384;
  long long* tl = (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && args.tl ? args.tl + 3 * 4096 : nullptr;

  if (warp == 0) {
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
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_st = umma_idesc(1, 1, 1, 0, 0, 128, 64);
      constexpr uint32_t idesc_acc = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      const uint32_t ak = smem_u32(sK), av = smem_u32(sV);
      const uint32_t lkk = desc_lo_kmajor(ak), lvv = desc_lo_kmajor(av);
      auto issue_st = [&](int it, int g) {
        const int st = it & 1;
        const uint32_t lq = desc_lo_kmajor(smem_u32(sQ + st * Cfg::TILE) + g * 8192);
        const uint32_t ldo = desc_lo_kmajor(smem_u32(sDO + st * Cfg::TILE) + g * 8192);
        const uint32_t tST = tmem_base + g * 64, tDPT = tmem_base + 128 + g * 64;
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tST, desc_of(lkk + kstep_kmajor(t)), desc_of(lq + kstep_kmajor(t)), idesc_st, t != 0);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tDPT, desc_of(lvv + kstep_kmajor(t)), desc_of(ldo + kstep_kmajor(t)), idesc_st, t != 0);
        umma_commit(&st_full[g]);
      };
      if (ok) {
        if (!mbar_wait(&qdo_full[0], 0)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
        } else {
          tc_fence_after();
          issue_st(0, 0);
          issue_st(0, 1);
        }
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t lqm = desc_lo_mnmajor(smem_u32(sQ + st * Cfg::TILE));
        const uint32_t ldom = desc_lo_mnmajor(smem_u32(sDO + st * Cfg::TILE));
        for (int g = 0; g < 2 && ok; ++g) {
          if (!mbar_wait(&pds_ready[g], it & 1)) {
            set_error(args.err, ERR_WAIT_MMA_TMEM);
            ok = false;
            break;
          }
          tc_fence_after();
          if (2 * it + g < 1024) BWD_STAMP(4 * it + 2 * g);
          const uint32_t tST = tmem_base + g * 64, tDPT = tmem_base + 128 + g * 64;
#pragma unroll
          for (int t = 0; t < 4; ++t)
            umma_f16_ts(tDV, tST + t * 8, desc_of(ldom + g * 512 + kstep_mnmajor(t)), idesc_acc,
                        (it | g | t) != 0);
#pragma unroll
          for (int t = 0; t < 4; ++t)
            umma_f16_ts(tDK, tDPT + t * 8, desc_of(lqm + g * 512 + kstep_mnmajor(t)), idesc_acc,
                        (it | g | t) != 0);
          if (g == 1) umma_commit(&qdo_empty[st]);
          if (it + 1 < n_iter) {
            if (g == 0) {
              if (!mbar_wait(&qdo_full[st ^ 1], ((it + 1) >> 1) & 1)) {
                set_error(args.err, ERR_WAIT_MMA_FULL);
                ok = false;
                break;
              }
              tc_fence_after();
            }
            issue_st(it + 1, g);
          }
          if (2 * it + g < 1024) BWD_STAMP(4 * it + 2 * g + 1);
        }
      }
      if (ok) umma_commit(dkv_done);
    }
  } else {
    const int g = (warp - 2) >> 2;
    const int sw = warp & 3;
    const int row = sw * 32 + lane;   // kv row inside the tile
    const int kv_idx = kv0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int wt = threadIdx.x - 64 - g * 128;  // 0..127 inside the warpgroup
    float* ls = s_stat + g * 128;               // lse2 of the unit's 64 query rows
    float* dl = ls + 64;                        // -delta * scale of the same rows
    const uint32_t tST = tmem_base + g * 64 + lane_sel, tDPT = tmem_base + 128 + g * 64 + lane_sel;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int h = kvh * group + it / per_head;
      const int qt = qt_first + it % per_head;
      const int q0 = qt * 128 + g * 64;
      {
        // stage the unit's per-query statistics; named barrier 1+g = this warpgroup's 128 threads
        const int qi = q0 + (wt & 63);
        const bool qok = qi < T;
        const size_t stat = ((size_t)b * args.hq + h) * T + (qok ? qi : 0);
        float val;
        if (wt < 64) val = qok ? args.lse[stat] * 1.4426950408889634f : INFINITY;
        else val = qok ? -args.delta[stat] * args.scale : 0.f;  // -delta * scale: one FMA per element below
        wg_sync(g);    // previous unit's reads done
        ls[wt] = val;  // wt >= 64 lands in dl[]
        wg_sync(g);
      }
      ok = mbar_wait(&st_full[g], it & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if ((warp & 3) == 2 && lane == 0 && it < 1024) BWD_STAMP(4096 * (1 + g) + 2 * it);
      // column (query) c is visible from this kv row iff kv_idx <= q + off  <=>  q >= kv_idx - off
      const int q_min = args.causal ? (kv_idx - off) : -0x40000000;
      const bool need_mask = args.causal && (q0 < q_min);
      uint32_t pk[32], dk_[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        __syncwarp();
        tmem_ld32(tST + c * 32, rs);
        tmem_ld32(tDPT + c * 32, rp);
        tmem_wait_ld();
        const int first_ok = q_min - (q0 + c * 32);  // columns i >= first_ok are visible
        // the per-query statistics are the same for every thread: fetch them four at a time
        const float4* ls4 = reinterpret_cast<const float4*>(ls + c * 32);
        const float4* dl4 = reinterpret_cast<const float4*>(dl + c * 32);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l = ls4[i >> 2], d = dl4[i >> 2];
          float p0 = exp2f(__uint_as_float(rs[i]) * args.scale_log2 - l.x);
          float p1 = exp2f(__uint_as_float(rs[i + 1]) * args.scale_log2 - l.y);
          float p2 = exp2f(__uint_as_float(rs[i + 2]) * args.scale_log2 - l.z);
          float p3 = exp2f(__uint_as_float(rs[i + 3]) * args.scale_log2 - l.w);
          if (need_mask) {
            if (i < first_ok) p0 = 0.f;
            if (i + 1 < first_ok) p1 = 0.f;
            if (i + 2 < first_ok) p2 = 0.f;
            if (i + 3 < first_ok) p3 = 0.f;
          }
          pk[c * 16 + (i >> 1)] = pack_bf16x2_alu(p0, p1);
          pk[c * 16 + (i >> 1) + 1] = pack_bf16x2_alu(p2, p3);
          // dS^T = P^T * (dP^T * scale - delta * scale)
          dk_[c * 16 + (i >> 1)] = pack_bf16x2_alu(p0 * fmaf(__uint_as_float(rp[i]), args.scale, d.x),
                                               p1 * fmaf(__uint_as_float(rp[i + 1]), args.scale, d.y));
          dk_[c * 16 + (i >> 1) + 1] = pack_bf16x2_alu(p2 * fmaf(__uint_as_float(rp[i + 2]), args.scale, d.z),
                                                   p3 * fmaf(__uint_as_float(rp[i + 3]), args.scale, d.w));
        }
      }
      tmem_st32(tST, pk);
      tmem_st32(tDPT, dk_);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&pds_ready[g]);
      if ((warp & 3) == 2 && lane == 0 && it < 1024) BWD_STAMP(4096 * (1 + g) + 2 * it + 1);
    }
    if (ok && n_iter > 0) {
      ok = mbar_wait(dkv_done, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      // warpgroup 0 writes dV, warpgroup 1 writes dK
      const bool row_ok = kv_idx < S;
      const bool is_k = g == 1;
      __nv_bfloat16* drow = (is_k ? args.dK + (size_t)(b * S + kv_idx) * args.lddk
                                  : args.dV + (size_t)(b * S + kv_idx) * args.lddv) + kvh * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
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
                         const void* dout, int lddo, const FaBwdArgs& a_in, cudaStream_t stream) {
  FaBwdArgs a = a_in;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v);
  a.dout = static_cast<const __nv_bfloat16*>(dout);
  a.ldq = ldq;
  a.ldk = ldk;
  a.ldv = ldv;
  a.lddo = lddo;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dout)) & 15)
    return BB_EARG;
  if ((ldq | ldk | ldv | lddo) & 7) return BB_EARG;
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

static long long* g_bwd_timeline = nullptr;

// Profiling aid: when set to a device buffer of 6*4096 int64, CTA (0,0,0) of the dQ kernel (first
// 3*4096 slots) and of the dK/dV kernel (next 3*4096) record clock64 stamps: per unit the MMA
// issuer's [after the dS wait, after issuing], and per warpgroup [S/dP ready, dS handed over].
BB_API int bb_flash_bwd_timeline(long long* buf) {
  g_bwd_timeline = buf;
  return 0;
}

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
  const long total = (long)B * T * hq;
  fa_delta_kernel<<<(int)((total + 7) / 8), 256, 0, s>>>(
      (const __nv_bfloat16*)out, ldo, (const __nv_bfloat16*)dout, lddo, delta, B, T, hq, hd);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  FaBwdArgs a{};
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
  a.tl = g_bwd_timeline;
  if (hd == 128) return launch_fa_bwd<128>(q, ldq, k, ldk, v, ldv, dout, lddo, a, s);
  if (hd == 64) return launch_fa_bwd<64>(q, ldq, k, ldk, v, ldv, dout, lddo, a, s);
  return BB_EARG;
}
