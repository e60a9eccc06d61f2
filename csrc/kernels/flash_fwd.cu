// Causal / full GQA flash attention forward on tcgen05 (no T x T materialisation).
//
// One CTA per (128-row query tile, query head, batch).  Per 128-row KV block j:
//   S_j   = Q K_j^T            tcgen05.mma  (SS, fp32 accumulator in TMEM, double buffered)
//   P_j   = exp2(S_j*c - m)    128 softmax threads, one query row each (tcgen05.ld), online max
//                              with lazy rescale of the O accumulator (tcgen05.ld/st) and P written
//                              to shared memory in the 128-byte-swizzled K-major operand layout
//   O    += P_j V_j            tcgen05.mma  (A = P from smem, B = V tile read MN-major)
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax
// and epilogue.  Q/K/V are read with 2-D TMA maps over the [tokens, heads*hd] activations (row
// pitch free), so strided views of a fused qkv buffer work without a copy.
//
// Replaces crates/kernels/wgsl/{gqa_scores,attn_softmax,gqa_apply,flash_attn_causal_gqa}.wgsl.
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
};

template <int HD>
struct FaFwdCfg {
  static constexpr int NSUB = HD / 64;             // 64-column swizzled sub-tiles per row
  static constexpr int SUB_BYTES = 128 * 128;      // [128 rows][64 bf16]
  static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  static constexpr int P_BYTES = 2 * SUB_BYTES;    // [128][128] bf16
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * TILE_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_MIN = OFF_BAR + 256 + 1024;
  // at least 120 KB so only one CTA is resident per SM (each allocates all 512 TMEM columns)
  static constexpr int SMEM = SMEM_MIN < 120 * 1024 ? 120 * 1024 : SMEM_MIN;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
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
  uint8_t* sP = smem + Cfg::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* p_ready = bars + 11;    // 1 (128 arrivals)
  uint64_t* pv_done = bars + 12;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
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
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < NSUB; ++c)
        tma_load_2d(sQ + c * Cfg::SUB_BYTES, &tmQ, q_full, h * HD + c * 64, b * T + q0);
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          ok = false;
          break;
        }
        mbar_expect_tx(&k_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sK + st * Cfg::TILE_BYTES + c * Cfg::SUB_BYTES, &tmK, &k_full[st],
                      kvh * HD + c * 64, b * S + j * 128);
        if (!mbar_wait(&v_empty[st], ph ^ 1)) {
          set_error(args.err, ERR_WAIT_PRODUCER);
          ok = false;
          break;
        }
        mbar_expect_tx(&v_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NSUB; ++c)
          tma_load_2d(sV + st * Cfg::TILE_BYTES + c * Cfg::SUB_BYTES, &tmV, &v_full[st],
                      kvh * HD + c * 64, b * S + j * 128);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 1, 0, 1, 128, HD);
      bool ok = true;
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t) {
          const uint32_t o = (t / 4) * Cfg::SUB_BYTES + (t % 4) * 32;
          umma_f16_ss(tmem_base + (j & 1) * 128, umma_smem_desc(aq + o, 16, 1024),
                      umma_smem_desc(bk + o, 16, 1024), idesc_qk, t != 0);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[st]);
        return true;
      };
      if (!mbar_wait(q_full, 0)) {
        set_error(args.err, ERR_WAIT_MMA_FULL);
        ok = false;
      }
      if (ok && !issue_qk(0)) {
        set_error(args.err, ERR_WAIT_MMA_FULL);
        ok = false;
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks && !issue_qk(j + 1)) {
          set_error(args.err, ERR_WAIT_MMA_FULL);
          ok = false;
          break;
        }
        if (!mbar_wait(p_ready, j & 1) || !mbar_wait(&v_full[j & 1], (j >> 1) & 1)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t ap = smem_u32(sP), bv = smem_u32(sV + (j & 1) * Cfg::TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 8; ++t) {  // 128 kv rows, 16 per MMA
          const uint32_t oa = (t / 4) * Cfg::SUB_BYTES + (t % 4) * 32;
          umma_f16_ss(tmem_O, umma_smem_desc(ap + oa, 16, 1024),
                      umma_smem_desc(bv + t * 2048, Cfg::SUB_BYTES, 1024), idesc_pv,
                      (j | t) != 0);
        }
        umma_commit(pv_done);
        umma_commit(&v_empty[j & 1]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    const int sw = warp & 3;
    const int row = sw * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = (uint32_t)(sw * 32) << 16;
    const int kv_limit_row = args.causal ? min(q_idx + off, S - 1) : S - 1;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tS = tmem_base + lane_sel + (j & 1) * 128;
      const int kv0 = j * 128;
      const bool need_mask = (kv0 + 127 > kv_limit_row);  // per-row decision, loads stay uniform
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tS + c * 32, r);
        tmem_wait_ld();
        const int lim = kv_limit_row - (kv0 + c * 32);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]);
          if (!need_mask || i <= lim) mx = fmaxf(mx, s);
        }
      }
      mx *= args.scale_log2;
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
            tmem_ld32(tmem_O + lane_sel + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tmem_O + lane_sel + c * 32, r);
          }
          tmem_wait_st();
        }
      }
      l *= alpha;
      m_ref = m_new;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tS + c * 32, r);
        tmem_wait_ld();
        const int lim = kv_limit_row - (kv0 + c * 32);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(r[i]) * args.scale_log2 - m_use);
          float p1 = exp2f(__uint_as_float(r[i + 1]) * args.scale_log2 - m_use);
          if (need_mask) {
            if (i > lim) p0 = 0.f;
            if (i + 1 > lim) p1 = 0.f;
          }
          l += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        // 32 columns = 4 x 16-byte chunks of sub-tile c/2; chunk index XOR (row % 8) = 128B swizzle
        uint8_t* prow = sP + (c >> 1) * Cfg::SUB_BYTES + row * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = ((c & 1) * 4 + q) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) =
              make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
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
        tmem_ld32(tmem_O + lane_sel + c * 32, r);
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
    tmem_dealloc(tmem_base, 512);
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<HD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((a.T + 127) / 128, a.hq, a.B);
  fa_fwd_kernel<HD><<<grid, 192, Cfg::SMEM, stream>>>(tmQ, tmK, tmV, a);
  return (int)cudaGetLastError();
}

}  // namespace bb

// q: [B*T, ldq] (head h at columns h*hd), k/v: [B*S, ldk/ldv]; out: [B*T, ldo]; lse: [B, hq, T].
// Requires ldo % 8 == 0 and 16-byte aligned bases.  hd in {64, 128}.
BB_API int bb_flash_fwd(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                        void* out, int ldo, float* lse, int B, int T, int S, int hq, int hk, int hd,
                        float scale, int causal, void* stream) {
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
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (hd == 128) return launch_fa_fwd<128>(q, ldq, k, ldk, v, ldv, a, s);
  if (hd == 64) return launch_fa_fwd<64>(q, ldq, k, ldk, v, ldv, a, s);
  return BB_EARG;
}
