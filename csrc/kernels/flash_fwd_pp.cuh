// Flash attention forward, third form: TWO query tiles per CTA taking turns on the tensor pipe.
// (Included by flash_fwd.cu, which defines FaFwdArgs / FaFwdCfg and the launcher.)
//
// One CTA per (pair of adjacent 128-row query tiles A and B, query head, batch), one CTA per SM, all
// 512 TMEM columns: S_A at 0, S_B at 128 (fp32 scores of a whole 128-key block, so every QK^T MMA is
// 128 wide: a tcgen05.mma costs the same ~70 clocks at N = 64 and N = 128), O_A at 256, O_B at 384.
// Two softmax warpgroups, one per tile.  Issue order of the MMA thread:
//
//     S_A(0) S_B(0) | PV_A(0) S_A(1) | PV_B(0) S_B(1) | PV_A(1) S_A(2) | ...
//
// While warpgroup A turns S_A(j) into P_A(j) the tensor pipe runs PV_B(j-1) and S_B(j); while
// warpgroup B works on S_B(j) it runs PV_A(j) and S_A(j+1).  Each tile's scores have one buffer
// (P is written back over S as packed bf16 and consumed from there), and MMAs execute in issue
// order, so S_x(j+1) may overwrite the columns PV_x(j) has just read.  K and V have two stages
// each and are shared by the two tiles (half the K/V shared-memory traffic per query row of the
// one-tile forms).  With causal masking tile B sees one block more than tile A.
//
// P is packed by truncation after scaling by 1.0029 (the factor folds into the exponent offset;
// the row sum is taken over the same scaled values and the stored LSE is corrected), which keeps
// the conversion unit free for the exponentials and costs one PRMT per pair.
#pragma once

namespace bb {

template <int HD>
struct FaPpCfg {
  static constexpr int NSUB = HD / 64;
  static constexpr int SUB_BYTES = 128 * 128;
  static constexpr int TILE = NSUB * SUB_BYTES;
  static constexpr int OFF_QA = 0;
  static constexpr int OFF_QB = OFF_QA + TILE;
  static constexpr int OFF_K = OFF_QB + TILE;      // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * TILE;   // 2 stages
  static constexpr int OFF_BAR = OFF_V + 2 * TILE;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;   // one CTA per SM
  static constexpr int THREADS = 64 + 2 * 128;
};

static constexpr float kFwdTruncLog2 = 0.0041778f;   // log2(1.0029)

template <int HD>
__global__ void __launch_bounds__(FaPpCfg<HD>::THREADS, 1)
fa_fwd_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FaFwdArgs args) {
  using Cfg = FaPpCfg<HD>;
  constexpr int NSUB = Cfg::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ[2] = {smem + Cfg::OFF_QA, smem + Cfg::OFF_QB};
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;          // both Q tiles
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2] one per tile
  uint64_t* p_ready = bars + 11;    // [2] 128 arrivals each
  uint64_t* pv_done = bars + 13;    // [2] one per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = gridDim.x - 1 - blockIdx.x;   // heavy (late) pairs first
  const int h = blockIdx.y, b = blockIdx.z;
  const int T = args.T, S = args.S;
  const int kvh = h / (args.hq / args.hk);
  const int off = S - T;
  const int total_blocks = (S + 127) / 128;
  // blocks visible to tile x (0 = A, 1 = B); a tile that starts past T does nothing
  int n_of[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int q0 = (2 * pair + x) * 128;
    int n = total_blocks;
    if (args.causal) {
      const int last = (q0 + 127 + off) / 128 + 1;
      n = last < n ? last : n;
    }
    n_of[x] = q0 < T ? n : 0;
  }
  const int n_max = n_of[0] > n_of[1] ? n_of[0] : n_of[1];

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
      mbar_init(s_full + i, 1);
      mbar_init(p_ready + i, 128);
      mbar_init(pv_done + i, 1);
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_max > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * Cfg::TILE);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sQ[x] + c * Cfg::SUB_BYTES, &tmQ, q_full, h * HD + c * 64, b * T + (2 * pair + x) * 128);
      for (int j = 0; j < n_max; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_empty + st, ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(k_full + st, Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sK + st * Cfg::TILE + c * Cfg::SUB_BYTES, &tmK, k_full + st, kvh * HD + c * 64, b * S + j * 128);
        if (!mbar_wait(v_empty + st, ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          break;
        }
        mbar_expect_tx(v_full + st, Cfg::TILE);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sV + st * Cfg::TILE + c * Cfg::SUB_BYTES, &tmV, v_full + st, kvh * HD + c * 64, b * S + j * 128);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_max > 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) set_error(args.err, ERR_WAIT_MMA_FULL);
      tc_fence_after();
      // which tile touches block j first / last (the K and V stages are acquired by the first and
      // released after the last): A when it sees the block, else B
      auto first_user = [&](int j) { return j < n_of[0] ? 0 : 1; };
      auto last_user = [&](int j) { return j < n_of[1] ? 1 : 0; };
      // S_x(j) = Q_x K_j^T
      auto issue_s = [&](int x, int j) -> bool {
        const int st = j & 1;
        if (x == first_user(j)) {
          if (!mbar_wait(k_full + st, (j >> 1) & 1)) return false;
          tc_fence_after();
        }
        const uint32_t aq = smem_u32(sQ[x]), bk = smem_u32(sK + st * Cfg::TILE);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t) {
          const uint32_t o = (t / 4) * Cfg::SUB_BYTES + (t % 4) * 32;
          umma_f16_ss(tmem_base + x * 128, umma_smem_desc(aq + o, 16, 1024), umma_smem_desc(bk + o, 16, 1024),
                      idesc_qk, t != 0);
        }
        umma_commit(s_full + x);
        if (x == last_user(j)) umma_commit(k_empty + st);
        return true;
      };
      // O_x += P_x(j) V_j: A = packed bf16 P in TMEM (8 columns per 16-key step), B = V MN-major
      auto issue_pv = [&](int x, int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(p_ready + x, j & 1)) return false;
        if (x == first_user(j) && !mbar_wait(v_full + st, (j >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t bv = smem_u32(sV + st * Cfg::TILE);
#pragma unroll
        for (int t = 0; t < 8; ++t)
          umma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + t * 8,
                      umma_smem_desc(bv + t * 2048, Cfg::SUB_BYTES, 1024), idesc_pv, (j | t) != 0);
        umma_commit(pv_done + x);
        if (x == last_user(j)) umma_commit(v_empty + st);
        return true;
      };
      if (ok && n_of[0] > 0) ok = issue_s(0, 0);
      if (ok && n_of[1] > 0) ok = issue_s(1, 0);
      for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!ok || j >= n_of[x]) continue;
          ok = issue_pv(x, j);
          if (ok && j + 1 < n_of[x]) ok = issue_s(x, j + 1);
        }
      }
      if (!ok) set_error(args.err, ERR_WAIT_MMA_TMEM);
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue, one warpgroup per tile
    const int x = (warp - 2) >> 2;
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q0 = (2 * pair + x) * 128;
    const int q_idx = q0 + row;
    const int n_blocks = n_of[x];
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    const uint32_t tS = tmem_base + x * 128 + lane_sel;
    const uint32_t tO = tmem_base + 256 + x * 128 + lane_sel;
    const float sc = args.scale_log2;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(s_full + x, j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t r[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(r + c * 32));
      tmem_wait_ld();
      const int kv0 = j * 128;
      const bool need_mask = (kv0 + 127 > kv_limit_row);
      const int lim = kv_limit_row - kv0;  // columns <= lim are visible
      float mx = -INFINITY;
      if (!need_mask) {
#pragma unroll
        for (int i = 0; i < 128; i += 4)
          mx = fmaxf(mx, fmaxf(fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                               fmaxf(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]))));
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i <= lim) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
      mx *= sc;
      float m_new = m_ref;
      if (mx > m_ref + 8.f) m_new = mx;  // lazy: keep the old reference while p stays <= 2^8
      const float alpha = (m_new == m_ref) ? 1.f : ((m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new));
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O changes scale: the PV of the block before must have landed first
        ok = mbar_wait(pv_done + x, (j - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tO + c * 32, o);
        }
      }
      l *= alpha;
      m_ref = m_new;
      // the exponent offset carries the truncation factor: p' = 1.0029 p, packed by truncation
      const float m_use = ((m_ref == -INFINITY) ? 0.f : m_ref) - kFwdTruncLog2;
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int i = 0; i < 128; i += 2) {
        float a0 = exp2f(__uint_as_float(r[i]) * sc - m_use);
        float a1 = exp2f(__uint_as_float(r[i + 1]) * sc - m_use);
        if (need_mask) {
          if (i > lim) a0 = 0.f;
          if (i + 1 > lim) a1 = 0.f;
        }
        ls0 += a0;
        ls1 += a1;
        r[i >> 1] = __byte_perm(__float_as_uint(a0), __float_as_uint(a1), 0x7632);
      }
      l += ls0 + ls1;
      tmem_st32(tS, *reinterpret_cast<const uint32_t(*)[32]>(r));
      tmem_st32(tS + 32, *reinterpret_cast<const uint32_t(*)[32]>(r + 32));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_ready + x);
    }
    if (ok && n_blocks > 0) {
      ok = mbar_wait(pv_done + x, (n_blocks - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok) {
      if (lane == 0) set_error(args.err, ERR_WAIT_SOFTMAX);
    } else if (q0 < T) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = args.O + (size_t)(b * T + q_idx) * args.ldo + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        __syncwarp();
        if (n_blocks > 0) {
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (q_idx < T) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * inv, __uint_as_float(o[q * 8 + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * inv, __uint_as_float(o[q * 8 + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * inv, __uint_as_float(o[q * 8 + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * inv, __uint_as_float(o[q * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = w;
          }
        }
      }
      // l sums the 1.0029-scaled probabilities: take the factor out of the stored log-sum-exp
      if (args.lse && q_idx < T)
        args.lse[((size_t)b * args.hq + h) * T + q_idx] =
            (l > 0.f) ? (m_ref + log2f(l) - kFwdTruncLog2) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace bb
