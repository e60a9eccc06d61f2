// Causal / full GQA flash attention forward on tcgen05 (no T x T materialisation).
//
// One CTA per (128-row query tile, query head, batch).  Per 128-row KV block j:
//   S_j   = Q K_j^T            tcgen05.mma  (SS, fp32 accumulator in TMEM)
//   P_j   = exp2(S_j*c - m)    128 softmax threads, one query row each: the whole row is pulled
//                              into registers with four back-to-back tcgen05.ld and one wait,
//                              online max with lazy rescale of the O accumulator
//                              (tcgen05.ld/st), and P is written back as packed bf16 OVER the S
//                              columns in TMEM (tcgen05.st) — no shared-memory round trip
//   O    += P_j V_j            tcgen05.mma  (A = P from TMEM, B = V tile read MN-major)
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax
// and epilogue.  A CTA uses 256 TMEM columns and < 100 KB of shared memory, so two CTAs share an
// SM: while one runs its softmax the other keeps the tensor pipe busy.
// Q/K/V are read with 2-D TMA maps over the [tokens, heads*hd] activations (row pitch free), so
// strided views of a fused qkv buffer work without a copy.
//
// Replaces crates/kernels/wgsl/{gqa_scores,attn_softmax,gqa_apply,flash_attn_causal_gqa}.wgsl.
#include <cstdlib>

#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

struct FaFwdArgs {
  __nv_bfloat16* O;
  float* lse;        // [B, hq, T] natural-log LSE (for backward); may be null
  int ldo;           // row pitch of O in elements
  int B, T, S;       // query length T, key length S (S >= T; causal offset = S - T)
  int hq, hk;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int* err;
  long long* timeline;  // optional [n_blocks][8] clock64 stamps of CTA (0,0,0) (profiling aid)
  // Paged, variable-length form (serving prefill): sequences are packed along the rows of Q / O,
  // keys and values are read straight from the paged KV pool through the block table.
  const int* block_tables;   // [n_seq][max_blocks] physical block of every logical block
  const int* seq_row0;       // [n_seq + 1] first packed row of every sequence
  const int* seq_ctx;        // [n_seq] context length (cached prefix + new rows)
  const int* tile_seq;       // [gridDim.x] sequence of every query tile
  const int* tile_qt;        // [gridDim.x] tile index inside its sequence
  int max_blocks, block_rows;  // pool block = block_rows token rows per KV head
};

template <int HD>
struct FaFwdCfg {
  static constexpr int NSUB = HD / 64;             // 64-column swizzled sub-tiles per row
  static constexpr int SUB_BYTES = 128 * 128;      // [128 rows][64 bf16]
  static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE_BYTES;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + TILE_BYTES;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  // at least 80 KB so at most two CTAs are resident per SM (each allocates 256 TMEM columns)
  static constexpr int SMEM = SMEM_MIN < 80 * 1024 ? 80 * 1024 : SMEM_MIN;
  static constexpr int TMEM_COLS = 256;
};

template <int HD>
__global__ void __launch_bounds__(192, 2)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const FaFwdArgs args) {
  using Cfg = FaFwdCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;   // 128 arrivals
  uint64_t* pv_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // stamps exist only in profiling builds (-DBB_TIMELINE); otherwise a compile-time null
#ifdef BB_TIMELINE
  long long* const tl = (args.timeline && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? args.timeline : nullptr;
#else
  long long* const tl = nullptr;
#endif
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
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
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;        // fp32 scores, later packed bf16 P in its first 64 cols
  const uint32_t tmem_O = tmem_base + 128;  // fp32 output accumulator (HD columns)

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < NSUB; ++c)
        tma_load_2d(sQ + c * Cfg::SUB_BYTES, &tmQ, q_full, h * HD + c * 64, b * T + q0);
      for (int j = 0; j < n_blocks; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_empty, ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(k_full, Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sK + c * Cfg::SUB_BYTES, &tmK, k_full, kvh * HD + c * 64, b * S + j * 128);
        if (!mbar_wait(v_empty, ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(v_full, Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sV + c * Cfg::SUB_BYTES, &tmV, v_full, kvh * HD + c * 64, b * S + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK), bv = smem_u32(sV);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_full, ph)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        if (tl) tl[j * 8 + 7] = clock64();
        // S = Q K^T.  Issued after PV_{j-1}, so the tensor pipe's in-order execution guarantees
        // P_{j-1} (which aliases these columns) has been consumed.
#pragma unroll
        for (int t = 0; t < HD / 16; ++t) {
          const uint32_t o = (t / 4) * Cfg::SUB_BYTES + (t % 4) * 32;
          umma_f16_ss(tmem_S, umma_smem_desc(aq + o, 16, 1024), umma_smem_desc(bk + o, 16, 1024),
                      idesc_qk, t != 0);
        }
        umma_commit(s_full);
        umma_commit(k_empty);
        if (!mbar_wait(p_ready, ph) || !mbar_wait(v_full, ph)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        if (tl) tl[j * 8 + 6] = clock64();
        // O += P V: A = packed bf16 P in TMEM (8 columns per 16-wide k-step), B = V MN-major
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tmem_O, tmem_S + t * 8, umma_smem_desc(bv + t * 2048, Cfg::SUB_BYTES, 1024),
                      idesc_pv, (j | t) != 0);
        umma_commit(pv_done);
        umma_commit(v_empty);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    const uint32_t tS = tmem_S + lane_sel;
    const uint32_t tO = tmem_O + lane_sel;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(s_full, j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool rec = tl && threadIdx.x == 64;
      if (rec) tl[j * 8 + 0] = clock64();
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld32(tS, r0);
      tmem_ld32(tS + 32, r1);
      tmem_ld32(tS + 64, r2);
      tmem_ld32(tS + 96, r3);
      tmem_wait_ld();
      if (rec) tl[j * 8 + 1] = clock64();
      const int kv0 = j * 128;
      const bool need_mask = (kv0 + 127 > kv_limit_row);
      const int lim = kv_limit_row - kv0;  // columns <= lim are visible
      float mx = -INFINITY;
      if (!need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          mx = fmaxf(mx, fmaxf(fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])),
                               fmaxf(__uint_as_float(r2[i]), __uint_as_float(r3[i]))));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i <= lim) mx = fmaxf(mx, __uint_as_float(r0[i]));
          if (i + 32 <= lim) mx = fmaxf(mx, __uint_as_float(r1[i]));
          if (i + 64 <= lim) mx = fmaxf(mx, __uint_as_float(r2[i]));
          if (i + 96 <= lim) mx = fmaxf(mx, __uint_as_float(r3[i]));
        }
      }
      mx *= args.scale_log2;
      if (rec) tl[j * 8 + 2] = clock64();
      float m_new = m_ref;
      if (mx > m_ref + 8.f) m_new = mx;  // lazy: keep the old reference while p stays <= 2^8
      const float alpha =
          (m_new == m_ref) ? 1.f : ((m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new));
      if (j > 0) {
        ok = mbar_wait(pv_done, (j - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO + c * 32, r);
          }
        }
      }
      if (rec) tl[j * 8 + 3] = clock64();
      l *= alpha;
      m_ref = m_new;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      const float sc = args.scale_log2;
      uint32_t pk0[32], pk1[32];  // 128 probabilities as 64 packed bf16x2 words
      float ls = 0.f;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float a0 = exp2f(__uint_as_float(r0[i]) * sc - m_use);
        float a1 = exp2f(__uint_as_float(r0[i + 1]) * sc - m_use);
        float b0 = exp2f(__uint_as_float(r1[i]) * sc - m_use);
        float b1 = exp2f(__uint_as_float(r1[i + 1]) * sc - m_use);
        float c0 = exp2f(__uint_as_float(r2[i]) * sc - m_use);
        float c1 = exp2f(__uint_as_float(r2[i + 1]) * sc - m_use);
        float d0 = exp2f(__uint_as_float(r3[i]) * sc - m_use);
        float d1 = exp2f(__uint_as_float(r3[i + 1]) * sc - m_use);
        if (need_mask) {
          if (i > lim) a0 = 0.f;
          if (i + 1 > lim) a1 = 0.f;
          if (i + 32 > lim) b0 = 0.f;
          if (i + 33 > lim) b1 = 0.f;
          if (i + 64 > lim) c0 = 0.f;
          if (i + 65 > lim) c1 = 0.f;
          if (i + 96 > lim) d0 = 0.f;
          if (i + 97 > lim) d1 = 0.f;
        }
        ls += (a0 + a1) + (b0 + b1) + (c0 + c1) + (d0 + d1);
        pk0[i >> 1] = pack_bf16x2(a0, a1);         // kv columns   0..31  -> words  0..15
        pk0[16 + (i >> 1)] = pack_bf16x2(b0, b1);  // kv columns  32..63  -> words 16..31
        pk1[i >> 1] = pack_bf16x2(c0, c1);         // kv columns  64..95  -> words 32..47
        pk1[16 + (i >> 1)] = pack_bf16x2(d0, d1);  // kv columns  96..127 -> words 48..63
      }
      l += ls;
      if (rec) tl[j * 8 + 4] = clock64();
      tmem_st32(tS, pk0);
      tmem_st32(tS + 32, pk1);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_ready);
      if (rec) tl[j * 8 + 5] = clock64();
    }
    if (ok) {
      ok = mbar_wait(pv_done, (n_blocks - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = args.O + (size_t)(b * T + q_idx) * args.ldo + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tO + c * 32, r);
        tmem_wait_ld();
        if (q_idx < T) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
      if (args.lse && q_idx < T)
        args.lse[((size_t)b * args.hq + h) * T + q_idx] =
            (l > 0.f) ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

static constexpr float kFwdTruncLog2 = 0.0041778f;   // log2(1.0029), see the packing note in fa_fwd2_kernel

// Second form of the forward kernel: the KV block is processed as two 64-key UNITS with two score
// buffers in TMEM, so the tensor pipe never sits on the softmax's critical path:
//   issue order   S(0) S(1) | P(0)? PV(0) S(2) | P(1)? PV(1) S(3) | ...
// S(u+1) is computed while the softmax warps work on S(u), PV(u) while they work on S(u+1); the
// softmax warps wait for the tensor pipe only at the start and when the (lazy) running-max update
// forces a rescale of O.  In the first form S(j+1) cannot be issued before P(j) is consumed (they
// share columns), which left the tensor pipe idle two thirds of the time (ncu: 31 % active).
// TMEM: S0 [0,64) S1 [64,128) fp32 scores, P(u) packed bf16 over the first 32 columns of its
// buffer, O [128, 128+HD).  Same shared-memory footprint, still two CTAs per SM.
// PAGED: one CTA per (query tile of a packed sequence, query head); K/V tiles are assembled from
// the pool's blocks (one TMA copy per block and 64-column half) instead of one copy per tile.
template <int HD, bool PAGED>
__global__ void __launch_bounds__(192, 2)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const FaFwdArgs args) {
  using Cfg = FaFwdCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;    // [2], one per score buffer
  uint64_t* p_ready = bars + 7;   // [2], 128 arrivals each
  uint64_t* pv_done = bars + 9;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = PAGED ? args.tile_seq[blockIdx.x] : 0;
  const int qt = PAGED ? args.tile_qt[blockIdx.x] : (int)(gridDim.x - 1 - blockIdx.x);  // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int row_base = PAGED ? args.seq_row0[seq] : b * args.T;   // first packed row of this sequence
  const int T = PAGED ? args.seq_row0[seq + 1] - row_base : args.T;
  const int S = PAGED ? args.seq_ctx[seq] : args.S;
  const int q0 = qt * 128;
  const int kvh = h / (args.hq / args.hk);
  const int off = S - T;
  int n_blocks = (S + 127) / 128;
  if (args.causal) {
    const int last = (q0 + 127 + off) / 128 + 1;
    n_blocks = last < n_blocks ? last : n_blocks;
  }
  const int n_units = 2 * n_blocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(p_ready + i, 128);
      mbar_init(pv_done + i, 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_O = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < NSUB; ++c)
        tma_load_2d(sQ + c * Cfg::SUB_BYTES, &tmQ, q_full, h * HD + c * 64, row_base + q0);
      for (int j = 0; j < n_blocks; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_empty, ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(k_full, Cfg::TILE_BYTES);
        if (PAGED) {
          // pool layout [blocks][kv heads][block_rows][HD]: block i of this tile lands at row i*block_rows
          const int br = args.block_rows, per_tile = 128 / br;
          const int* tab = args.block_tables + (size_t)seq * args.max_blocks + j * per_tile;
          for (int i = 0; i < per_tile; ++i) {
            const bool live = (j * 128 + i * br) < S && (j * per_tile + i) < args.max_blocks;
            const int blk = live ? max(tab[i], 0) : 0;   // dead blocks are masked by the key limit
            for (int c = 0; c < NSUB; ++c)
              tma_load_2d(sK + c * Cfg::SUB_BYTES + i * br * 128, &tmK, k_full, c * 64,
                          (blk * args.hk + kvh) * br);
          }
        } else {
#pragma unroll
          for (int c = 0; c < NSUB; ++c)
            tma_load_2d(sK + c * Cfg::SUB_BYTES, &tmK, k_full, kvh * HD + c * 64, b * S + j * 128);
        }
        if (!mbar_wait(v_empty, ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(v_full, Cfg::TILE_BYTES);
        if (PAGED) {
          const int br = args.block_rows, per_tile = 128 / br;
          const int* tab = args.block_tables + (size_t)seq * args.max_blocks + j * per_tile;
          for (int i = 0; i < per_tile; ++i) {
            const bool live = (j * 128 + i * br) < S && (j * per_tile + i) < args.max_blocks;
            const int blk = live ? max(tab[i], 0) : 0;
            for (int c = 0; c < NSUB; ++c)
              tma_load_2d(sV + c * Cfg::SUB_BYTES + i * br * 128, &tmV, v_full, c * 64,
                          (blk * args.hk + kvh) * br);
          }
        } else {
#pragma unroll
          for (int c = 0; c < NSUB; ++c)
            tma_load_2d(sV + c * Cfg::SUB_BYTES, &tmV, v_full, kvh * HD + c * 64, b * S + j * 128);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 1, 0, 0, 128, 64);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK), bv = smem_u32(sV);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      // S(u) = Q . K[unit u]^T into score buffer u & 1 (64 keys = rows half*64.. of the K tile)
      auto issue_s = [&](int u) -> bool {
        const int j = u >> 1, half = u & 1;
        if (half == 0) {
          if (!mbar_wait(k_full, j & 1)) return false;
          tc_fence_after();
        }
#pragma unroll
        for (int t = 0; t < HD / 16; ++t) {
          const uint32_t o = (t / 4) * Cfg::SUB_BYTES + (t % 4) * 32;
          umma_f16_ss(tmem_base + half * 64, umma_smem_desc(aq + o, 16, 1024),
                      umma_smem_desc(bk + o + half * 8192, 16, 1024), idesc_qk, t != 0);
        }
        umma_commit(s_full + half);
        if (half == 1) umma_commit(k_empty);
        return true;
      };
      if (ok && n_units > 0) ok = issue_s(0);
      if (ok && n_units > 1) ok = issue_s(1);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      for (int u = 0; u < n_units && ok; ++u) {
        const int j = u >> 1, half = u & 1;
        if (!mbar_wait(p_ready + half, j & 1) || (half == 0 && !mbar_wait(v_full, j & 1))) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        // O += P(u) V[unit u]: A = packed bf16 P in TMEM (8 columns per 16-key step), B = V MN-major
#pragma unroll
        for (int t = 0; t < 4; ++t)
          umma_f16_ts(tmem_O, tmem_base + half * 64 + t * 8,
                      umma_smem_desc(bv + (half * 4 + t) * 2048, Cfg::SUB_BYTES, 1024), idesc_pv,
                      (u | t) != 0);
        umma_commit(pv_done + half);
        if (half == 1) umma_commit(v_empty);
        if (u + 2 < n_units && !issue_s(u + 2)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    const uint32_t tO = tmem_O + lane_sel;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int u = 0; u < n_units; ++u) {
      const int half = u & 1;
      const uint32_t tS = tmem_base + half * 64 + lane_sel;
      ok = mbar_wait(s_full + half, (u >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld32(tS, r0);
      tmem_ld32(tS + 32, r1);
      tmem_wait_ld();
      const int kv0 = u * 64;
      const bool need_mask = (kv0 + 63 > kv_limit_row);
      const int lim = kv_limit_row - kv0;  // columns <= lim are visible
      float mx = -INFINITY;
      if (!need_mask) {
        // four independent running maxima: one chain of 32 dependent FMNMX would leave the two warps
        // a scheduler holds here waiting on its latency
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            m4[q] = fmaxf(m4[q], fmaxf(__uint_as_float(r0[i + q]), __uint_as_float(r1[i + q])));
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i <= lim) mx = fmaxf(mx, __uint_as_float(r0[i]));
          if (i + 32 <= lim) mx = fmaxf(mx, __uint_as_float(r1[i]));
        }
      }
      mx *= args.scale_log2;
      float m_new = m_ref;
      if (mx > m_ref + 8.f) m_new = mx;  // lazy: keep the old reference while p stays <= 2^8
      const float alpha =
          (m_new == m_ref) ? 1.f : ((m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new));
      if (u > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O changes scale: every PV issued so far must have landed first
        ok = mbar_wait(pv_done + ((u - 1) & 1), ((u - 1) >> 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tO + c * 32, r);
        }
      }
      l *= alpha;
      m_ref = m_new;
      // P is packed by truncation (one PRMT per pair) after a 1.0029 pre-scale that folds into the
      // exponent offset: truncation of the scaled value is unbiased on average, the row sum runs over
      // the same scaled values (so O / l is unchanged) and the stored log-sum-exp takes the factor out
      const float m_use = ((m_ref == -INFINITY) ? 0.f : m_ref) - kFwdTruncLog2;
      const float sc = args.scale_log2;
      uint32_t pk[32];  // 64 probabilities as 32 packed bf16x2 words
      float ls = 0.f, ls_b = 0.f;    // two running sums (alternating iterations) halve the add chain
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float a0 = exp2f(__uint_as_float(r0[i]) * sc - m_use);
        float a1 = exp2f(__uint_as_float(r0[i + 1]) * sc - m_use);
        float b0 = exp2f(__uint_as_float(r1[i]) * sc - m_use);
        float b1 = exp2f(__uint_as_float(r1[i + 1]) * sc - m_use);
        if (need_mask) {
          if (i > lim) a0 = 0.f;
          if (i + 1 > lim) a1 = 0.f;
          if (i + 32 > lim) b0 = 0.f;
          if (i + 33 > lim) b1 = 0.f;
        }
        if (i & 2) ls_b += (a0 + a1) + (b0 + b1);
        else ls += (a0 + a1) + (b0 + b1);
        // integer-pipe packing: cvt.rn.bf16x2 would share the quarter-rate unit with ex2
        pk[i >> 1] = __byte_perm(__float_as_uint(a0), __float_as_uint(a1), 0x7632);         // keys  0..31 -> words  0..15
        pk[16 + (i >> 1)] = __byte_perm(__float_as_uint(b0), __float_as_uint(b1), 0x7632);  // keys 32..63 -> words 16..31
      }
      l += ls + ls_b;
      tmem_st32(tS, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_ready + half);
    }
    if (ok && n_units > 0) {
      ok = mbar_wait(pv_done + ((n_units - 1) & 1), ((n_units - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = args.O + (size_t)(row_base + q_idx) * args.ldo + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tO + c * 32, r);
        tmem_wait_ld();
        if (q_idx < T) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
      if (!PAGED && args.lse && q_idx < T)
        args.lse[((size_t)b * args.hq + h) * T + q_idx] =
            (l > 0.f) ? (m_ref + log2f(l) - kFwdTruncLog2) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int HD>
static int launch_fa_fwd(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                         const FaFwdArgs& a, cudaStream_t stream) {
  using Cfg = FaFwdCfg<HD>;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, (uint64_t)a.hq * HD,
                        (uint64_t)a.B * a.T, (uint64_t)ldq * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, (uint64_t)a.hk * HD,
                    (uint64_t)a.B * a.S, (uint64_t)ldk * 2, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v, (uint64_t)a.hk * HD,
                    (uint64_t)a.B * a.S, (uint64_t)ldv * 2, 64, 128);
  if (rc) return rc;
  static PerDeviceOnce once1, once2;
  {
    cudaError_t e = ensure_dyn_smem(once1, fa_fwd_kernel<HD>, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    e = ensure_dyn_smem(once2, fa_fwd2_kernel<HD, false>, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((a.T + 127) / 128, a.hq, a.B);
  // the two-unit form is the default (478 -> 309 us at B4 T4096 16q/8kv hd128); BB_FA_FWD=1 selects
  // the first form, which also carries the timeline stamps.  (A third form with one 128-key score
  // tile per block, single-buffered, measured 380 us: with two CTAs per SM the idle tensor time
  // during a CTA's softmax was not filled by its neighbour.  A fourth form, one CTA per SM working
  // on two query tiles that take turns on the tensor pipe, 128-wide score MMAs, one softmax
  // warpgroup of one row per thread per tile, all 512 TMEM columns, was correct and measured 372 us:
  // each tile is one serial chain scores -> 128 exponentials per thread -> PV -> next scores, and two
  // such chains per SM hide less than the four shorter ones of this form.)
  static const int form = [] {
    const char* e = getenv("BB_FA_FWD");
    return (e && e[0] == '1') ? 1 : 2;
  }();
  if (form == 2 && a.timeline == nullptr)
    fa_fwd2_kernel<HD, false><<<grid, 192, Cfg::SMEM, stream>>>(tmQ, tmK, tmV, a);
  else
    fa_fwd_kernel<HD><<<grid, 192, Cfg::SMEM, stream>>>(tmQ, tmK, tmV, a);
  return (int)cudaGetLastError();
}

}  // namespace bb

BB_API int bb_flash_fwd_timeline(const void*, int, const void*, int, const void*, int, void*, int,
                                 float*, int, int, int, int, int, int, float, int, long long*, void*);

// q: [B*T, ldq] (head h at columns h*hd), k/v: [B*S, ldk/ldv]; out: [B*T, ldo]; lse: [B, hq, T].
// Requires ldo % 8 == 0 and 16-byte aligned bases.  hd in {64, 128}.
// Causal attention of packed, variable-length query rows against a PAGED KV pool (serving prefill
// and mixed steps): sequence s owns rows [seq_row0[s], seq_row0[s+1]) of q / out, its context is the
// first seq_ctx[s] token rows named by block_tables[s][:] (the new rows' K/V are already in the pool),
// and query row i of the sequence sees keys [0, seq_ctx[s] - T_s + i].  One launch for all sequences;
// no gather of the cached prefix into a contiguous buffer.  tile_seq / tile_qt list the 128-row query
// tiles (host-built).  Pools: bf16 [pool_blocks][hk][block_rows][hd], block_rows in {16, 32, 64, 128}.
BB_API int bb_flash_fwd_paged(const void* q, int ldq, const void* k_pool, const void* v_pool, void* out,
                              int ldo, const int* block_tables, int max_blocks, int block_rows,
                              int pool_blocks, const int* seq_row0, const int* seq_ctx,
                              const int* tile_seq, const int* tile_qt, int n_tiles, int total_rows, int hq,
                              int hk, int hd, float scale, void* stream) {
  using namespace bb;
  if (n_tiles <= 0) return BB_OK;
  if (hq % hk || total_rows <= 0 || max_blocks <= 0 || pool_blocks <= 0) return BB_EARG;
  if (block_rows != 16 && block_rows != 32 && block_rows != 64 && block_rows != 128) return BB_EARG;
  if (hd != 128 && hd != 64) return BB_EARG;
  FaFwdArgs a{};
  a.O = static_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.hq = hq;
  a.hk = hk;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = 1;
  a.err = device_error_word();
  a.block_tables = block_tables;
  a.seq_row0 = seq_row0;
  a.seq_ctx = seq_ctx;
  a.tile_seq = tile_seq;
  a.tile_qt = tile_qt;
  a.max_blocks = max_blocks;
  a.block_rows = block_rows;
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = make_tmap_2d(&tmQ, bf, 2, q, (uint64_t)hq * hd, (uint64_t)total_rows, (uint64_t)ldq * 2, 64, 128);
  if (rc) return rc;
  const uint64_t pool_rows = (uint64_t)pool_blocks * hk * block_rows;
  rc = make_tmap_2d(&tmK, bf, 2, k_pool, (uint64_t)hd, pool_rows, (uint64_t)hd * 2, 64, block_rows);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, bf, 2, v_pool, (uint64_t)hd, pool_rows, (uint64_t)hd * 2, 64, block_rows);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(n_tiles, hq, 1);
  if (hd == 128) {
    static PerDeviceOnce once;
    cudaError_t e = ensure_dyn_smem(once, fa_fwd2_kernel<128, true>, FaFwdCfg<128>::SMEM);
    if (e != cudaSuccess) return (int)e;
    fa_fwd2_kernel<128, true><<<grid, 192, FaFwdCfg<128>::SMEM, s>>>(tmQ, tmK, tmV, a);
  } else {
    static PerDeviceOnce once;
    cudaError_t e = ensure_dyn_smem(once, fa_fwd2_kernel<64, true>, FaFwdCfg<64>::SMEM);
    if (e != cudaSuccess) return (int)e;
    fa_fwd2_kernel<64, true><<<grid, 192, FaFwdCfg<64>::SMEM, s>>>(tmQ, tmK, tmV, a);
  }
  return (int)cudaGetLastError();
}

BB_API int bb_flash_fwd(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                        void* out, int ldo, float* lse, int B, int T, int S, int hq, int hk, int hd,
                        float scale, int causal, void* stream) {
  return bb_flash_fwd_timeline(q, ldq, k, ldk, v, ldv, out, ldo, lse, B, T, S, hq, hk, hd, scale,
                               causal, nullptr, stream);
}

// Same, with (in builds made with -DBB_TIMELINE only) an optional device buffer of (T/128) x 8 clock64 stamps filled by the CTA of the last
// query tile of head 0 / batch 0: per KV block [0] scores ready, [1] row in registers, [2] max
// done, [3] O rescaled, [4] exponentials done, [5] P stored + signalled, [6] PV issued, [7] QK issued.
BB_API int bb_flash_fwd_timeline(const void* q, int ldq, const void* k, int ldk, const void* v,
                                 int ldv, void* out, int ldo, float* lse, int B, int T, int S,
                                 int hq, int hk, int hd, float scale, int causal,
                                 long long* timeline, void* stream) {
  using namespace bb;
  if (B <= 0 || T <= 0 || S < T || hq % hk) return BB_EARG;
  if ((ldo % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) return BB_EARG;
  FaFwdArgs a{};
  a.O = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.ldo = ldo;
  a.B = B;
  a.T = T;
  a.S = S;
  a.hq = hq;
  a.hk = hk;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.err = device_error_word();
  a.timeline = timeline;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (hd == 128) return launch_fa_fwd<128>(q, ldq, k, ldk, v, ldv, a, s);
  if (hd == 64) return launch_fa_fwd<64>(q, ldq, k, ldk, v, ldv, a, s);
  return BB_EARG;
}
