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
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax.
// Replaces crates/kernels/wgsl/gqa_bwd_{dscores,dv,dq,dk}.wgsl (which read a saved T x T probs buffer).
#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

struct FaBwdArgs {
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
template <int HD>
struct DqCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int TILE = NSUB * SUB;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + TILE;
  static constexpr int OFF_K = OFF_DO + TILE;
  static constexpr int OFF_V = OFF_K + 2 * TILE;
  static constexpr int OFF_BAR = OFF_V + 2 * TILE;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdArgs args) {
  using Cfg = DqCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;        // Q and dO
  uint64_t* k_full = bars + 1;    // 2
  uint64_t* k_empty = bars + 3;   // 2
  uint64_t* v_full = bars + 5;    // 2
  uint64_t* v_empty = bars + 7;   // 2
  uint64_t* sdp_full = bars + 9;  // 1
  uint64_t* ds_ready = bars + 10; // 1 (128 arrivals)
  uint64_t* dq_done = bars + 11;  // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);

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
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(ds_ready, 128);
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
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * Cfg::TILE);
#pragma unroll
      for (int c = 0; c < NSUB; ++c) {
        tma_load_2d(sQ + c * SUB, &tmQ, q_full, h * HD + c * 64, b * T + q0);
        tma_load_2d(sDO + c * SUB, &tmDO, q_full, h * HD + c * 64, b * T + q0);
      }
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
      constexpr uint32_t idesc_s = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_dq = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      const uint32_t aq = smem_u32(sQ), ado = smem_u32(sDO);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph) || !mbar_wait(&v_full[st], ph)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t bk = smem_u32(sK + st * Cfg::TILE), bv = smem_u32(sV + st * Cfg::TILE);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tS, desc_kmajor(aq, t), desc_kmajor(bk, t), idesc_s, t != 0);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tDP, desc_kmajor(ado, t), desc_kmajor(bv, t), idesc_s, t != 0);
        umma_commit(sdp_full);
        umma_commit(&v_empty[st]);
        if (!mbar_wait(ds_ready, j & 1)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tDQ, tS + t * 8, desc_mnmajor(bk, t), idesc_dq, (j | t) != 0);
        umma_commit(dq_done);
        umma_commit(&k_empty[st]);
      }
    }
  } else {
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    const bool row_ok = q_idx < T;
    const size_t stat = ((size_t)b * args.hq + h) * T + (row_ok ? q_idx : 0);
    const float lse2 = row_ok ? args.lse[stat] * 1.4426950408889634f : INFINITY;
    const float dlt = row_ok ? args.delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(sdp_full, j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (j > 0) {  // already complete (S_j was issued after dQ_{j-1}); keeps the phase in step
        ok = mbar_wait(dq_done, (j - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const int kv0 = j * 128;
      const bool need_mask = (kv0 + 127 > kv_limit_row);
      // two halves of 64 kv columns; dS (packed bf16) overwrites the S columns already consumed
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t rs0[32], rs1[32], rp0[32], rp1[32];
        __syncwarp();
        tmem_ld32(tS + lane_sel + hf * 64, rs0);
        tmem_ld32(tS + lane_sel + hf * 64 + 32, rs1);
        tmem_ld32(tDP + lane_sel + hf * 64, rp0);
        tmem_ld32(tDP + lane_sel + hf * 64 + 32, rp1);
        tmem_wait_ld();
        const int lim = kv_limit_row - (kv0 + hf * 64);
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(rs0[i]) * args.scale_log2 - lse2);
          float p1 = exp2f(__uint_as_float(rs0[i + 1]) * args.scale_log2 - lse2);
          float p2 = exp2f(__uint_as_float(rs1[i]) * args.scale_log2 - lse2);
          float p3 = exp2f(__uint_as_float(rs1[i + 1]) * args.scale_log2 - lse2);
          if (need_mask) {
            if (i > lim) p0 = 0.f;
            if (i + 1 > lim) p1 = 0.f;
            if (i + 32 > lim) p2 = 0.f;
            if (i + 33 > lim) p3 = 0.f;
          }
          pk[i >> 1] = pack_bf16x2(p0 * (__uint_as_float(rp0[i]) - dlt) * args.scale,
                                   p1 * (__uint_as_float(rp0[i + 1]) - dlt) * args.scale);
          pk[16 + (i >> 1)] = pack_bf16x2(p2 * (__uint_as_float(rp1[i]) - dlt) * args.scale,
                                          p3 * (__uint_as_float(rp1[i + 1]) - dlt) * args.scale);
        }
        tmem_st32(tS + lane_sel + hf * 32, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(ds_ready);
    }
    if (ok) {
      ok = mbar_wait(dq_done, (n_blocks - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      __nv_bfloat16* orow = args.dQ + (size_t)(b * T + q_idx) * args.lddq + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
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
template <int HD>
struct DkvCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int TILE = NSUB * SUB;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE;
  static constexpr int OFF_Q = OFF_V + TILE;
  static constexpr int OFF_DO = OFF_Q + TILE;
  static constexpr int OFF_STAT = OFF_DO + TILE;  // lse2[128], delta[128]
  static constexpr int OFF_BAR = OFF_STAT + 1024;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
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
  float* s_lse2 = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  float* s_delta = s_lse2 + 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;        // K and V tiles (once)
  uint64_t* qdo_full = bars + 1;   // Q and dO of the current iteration
  uint64_t* qdo_empty = bars + 2;
  uint64_t* st_full = bars + 3;    // S^T and dP^T ready in TMEM
  uint64_t* pds_ready = bars + 4;  // P^T, dS^T written (128 arrivals)
  uint64_t* dkv_done = bars + 5;   // dV/dK MMAs of the iteration finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

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
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(st_full, 1);
    mbar_init(pds_ready, 128);
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
  const uint32_t tST = tmem_base, tDPT = tmem_base + 128, tDV = tmem_base + 256,
                 tDK = tmem_base + 384;

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
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(qdo_full, 2 * Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c) {
          tma_load_2d(sQ + c * SUB, &tmQ, qdo_full, h * HD + c * 64, b * T + qt * 128);
          tma_load_2d(sDO + c * SUB, &tmDO, qdo_full, h * HD + c * 64, b * T + qt * 128);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_st = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_acc = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      const uint32_t ak = smem_u32(sK), av = smem_u32(sV), bq = smem_u32(sQ), bdo = smem_u32(sDO);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (!mbar_wait(qdo_full, it & 1)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tST, desc_kmajor(ak, t), desc_kmajor(bq, t), idesc_st, t != 0);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t)
          umma_f16_ss(tDPT, desc_kmajor(av, t), desc_kmajor(bdo, t), idesc_st, t != 0);
        umma_commit(st_full);
        if (!mbar_wait(pds_ready, it & 1)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tDV, tST + t * 8, desc_mnmajor(bdo, t), idesc_acc, (it | t) != 0);
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tDK, tDPT + t * 8, desc_mnmajor(bq, t), idesc_acc, (it | t) != 0);
        umma_commit(dkv_done);
        umma_commit(qdo_empty);
      }
    }
  } else {
    const int sw = warp & 3;
    const int row = sw * 32 + lane;   // kv row inside the tile
    const int kv_idx = kv0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int st_tid = threadIdx.x - 64;  // 0..127
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int h = kvh * group + it / per_head;
      const int qt = qt_first + it % per_head;
      const int q0 = qt * 128;
      // stage per-query statistics of this tile (each softmax thread loads one)
      {
        const int qi = q0 + st_tid;
        const bool qok = qi < T;
        const size_t stat = ((size_t)b * args.hq + h) * T + (qok ? qi : 0);
        // named barrier 1: all 128 softmax threads finished reading the previous statistics
        asm volatile("bar.sync 1, 128;" ::: "memory");
        s_lse2[st_tid] = qok ? args.lse[stat] * 1.4426950408889634f : INFINITY;
        s_delta[st_tid] = qok ? args.delta[stat] : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      ok = mbar_wait(st_full, it & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (it > 0) {  // already complete; keeps the barrier phase in step for the final wait
        ok = mbar_wait(dkv_done, (it - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      // column (query) c is visible from this kv row iff kv_idx <= q + off  <=>  q >= kv_idx - off
      const int q_min = args.causal ? (kv_idx - off) : -0x40000000;
      const bool need_mask = args.causal && (q0 < q_min);
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t rs0[32], rs1[32], rp0[32], rp1[32];
        __syncwarp();
        tmem_ld32(tST + lane_sel + hf * 64, rs0);
        tmem_ld32(tST + lane_sel + hf * 64 + 32, rs1);
        tmem_ld32(tDPT + lane_sel + hf * 64, rp0);
        tmem_ld32(tDPT + lane_sel + hf * 64 + 32, rp1);
        tmem_wait_ld();
        uint32_t pk[32], dk_[32];
        const int first_ok = q_min - (q0 + hf * 64);  // columns i >= first_ok are visible
        const float* ls = s_lse2 + hf * 64;
        const float* dl = s_delta + hf * 64;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(rs0[i]) * args.scale_log2 - ls[i]);
          float p1 = exp2f(__uint_as_float(rs0[i + 1]) * args.scale_log2 - ls[i + 1]);
          float p2 = exp2f(__uint_as_float(rs1[i]) * args.scale_log2 - ls[32 + i]);
          float p3 = exp2f(__uint_as_float(rs1[i + 1]) * args.scale_log2 - ls[33 + i]);
          if (need_mask) {
            if (i < first_ok) p0 = 0.f;
            if (i + 1 < first_ok) p1 = 0.f;
            if (i + 32 < first_ok) p2 = 0.f;
            if (i + 33 < first_ok) p3 = 0.f;
          }
          pk[i >> 1] = pack_bf16x2(p0, p1);
          pk[16 + (i >> 1)] = pack_bf16x2(p2, p3);
          dk_[i >> 1] = pack_bf16x2(p0 * (__uint_as_float(rp0[i]) - dl[i]) * args.scale,
                                    p1 * (__uint_as_float(rp0[i + 1]) - dl[i + 1]) * args.scale);
          dk_[16 + (i >> 1)] = pack_bf16x2(p2 * (__uint_as_float(rp1[i]) - dl[32 + i]) * args.scale,
                                           p3 * (__uint_as_float(rp1[i + 1]) - dl[33 + i]) * args.scale);
        }
        tmem_st32(tST + lane_sel + hf * 32, pk);
        tmem_st32(tDPT + lane_sel + hf * 32, dk_);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(pds_ready);
    }
    if (ok && n_iter > 0) {
      ok = mbar_wait(dkv_done, (n_iter - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      const bool row_ok = kv_idx < S;
      __nv_bfloat16* vrow = args.dV + (size_t)(b * S + kv_idx) * args.lddv + kvh * HD;
      __nv_bfloat16* krow = args.dK + (size_t)(b * S + kv_idx) * args.lddk + kvh * HD;
#pragma unroll 1
      for (int c = 0; c < 2 * (HD / 32); ++c) {
        const bool is_k = c >= HD / 32;
        const int cc = is_k ? c - HD / 32 : c;
        uint32_t r[32];
        __syncwarp();
        if (n_iter > 0) {
          tmem_ld32((is_k ? tDK : tDV) + lane_sel + cc * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
          __nv_bfloat16* dst = (is_k ? krow : vrow) + cc * 32;
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_dq_kernel<HD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DqCfg<HD>::SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(fa_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DkvCfg<HD>::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 gq((a.T + 127) / 128, a.hq, a.B);
  fa_bwd_dq_kernel<HD><<<gq, 192, DqCfg<HD>::SMEM, stream>>>(tmQ, tmK, tmV, tmDO, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  dim3 gk((a.S + 127) / 128, a.hk, a.B);
  fa_bwd_dkv_kernel<HD><<<gk, 192, DkvCfg<HD>::SMEM, stream>>>(tmQ, tmK, tmV, tmDO, a);
  return (int)cudaGetLastError();
}

}  // namespace bb

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
  if (hd == 128) return launch_fa_bwd<128>(q, ldq, k, ldk, v, ldv, dout, lddo, a, s);
  if (hd == 64) return launch_fa_bwd<64>(q, ldq, k, ldk, v, ldv, dout, lddo, a, s);
  return BB_EARG;
}
