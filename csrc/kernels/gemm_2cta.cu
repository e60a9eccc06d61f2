// Dense bf16 GEMM on CTA PAIRS: one tcgen05.mma.cta_group::2 computes a 256 x 256 output tile over
// two SMs of a 2-CTA cluster.
//
//   C[M,N] (op)= alpha * A[M,K] * B[N,K]^T        (operand layouts as in gemm_tcgen05.cu)
//
// Why pairs: a single CTA computing 128 x 256 has to pull 48 KB (A 16 KB + B 32 KB) through its
// L2 -> shared-memory path per 64-deep k-block, and that path, not the tensor pipe, bounds the
// single-CTA kernel (the k-block's four MMAs take about 520 clocks, the fill about 750).  In a pair
// every CTA loads its own 128 rows of A and only HALF of the B tile (its 128 of the 256 columns);
// the pair's MMA reads both halves.  32 KB per CTA and k-block: the fill drops below the math.
// Every load is a plain per-CTA TMA copy from this GPU's memory into the CTA's own shared memory.
//
// Protocol (leader = cluster rank 0, which issues every MMA):
//   full[s]        in the LEADER's shared memory, 1 arrival: the leader's producer posts the byte count of
//                  both CTAs; the TMA copies of both CTAs complete on it
//   empty[s]       per CTA; the leader's tcgen05.commit arrives on both CTAs' barriers
//   tmem_full[a]   per CTA; committed to both by the leader when a tile's MMAs are done
//   tmem_empty[a]  in the leader's shared memory, 8 arrivals: one per epilogue warp of the pair
// TMEM: 512 columns per CTA = two 256-column accumulators (rows 0..127 of the pair tile in the
// leader, 128..255 in its peer), so a tile's epilogue overlaps the next tile's main loop.
// Every wait is bounded; on expiry the role records a code in the device error word and falls
// through to the common exit (cluster barrier, TMEM release).
//
// Replaces, like gemm_tcgen05.cu, the reference's register-tiled GEMMs
// (crates/kernels/wgsl/matmul_reg3.wgsl, matmul_dx_reg.wgsl, matmul_dw_reg.wgsl).
#include <cuda_runtime.h>

#include <cstdlib>

#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {
namespace pair {

// ---------------------------------------------------------------- cluster / pair PTX
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
               "r"(bytes)
               : "memory");
}
// TMA tile load into this CTA's shared memory whose completion is counted on a barrier that may
// live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// int8 operands, s32 accumulator (K = 32 per instruction: the same 32 bytes per operand row)
__device__ __forceinline__ void umma_i8_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at `cluster_addr` (either CTA of the pair) once every MMA issued so far by
// this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

struct PairArgs {
  const float* scale_m;  // int8: per-row (token) scale
  const float* scale_n;  // int8: per-column (channel) scale
  float alpha;
  int M, N, K;
  int a_mn, b_mn;
  int out_mode;  // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (TMA reduce-add)
  int split_k;
  int* err;
#ifdef BB_TIMELINE
  long long* dbg;  // profiling builds: cycle counters of pair 0 ([0] MMA loop, [1] waiting for data,
                   // [2] waiting for an accumulator, [3]/[4] leader / peer producer waiting for a free slot)
#endif
};

#ifdef BB_TIMELINE
#define PAIR_CLK() clock64()
#define PAIR_ADD(slot, v) do { if (args.dbg && pair_id == 0) atomicAdd((unsigned long long*)&args.dbg[slot], (unsigned long long)(v)); } while (0)
#else
#define PAIR_CLK() 0LL
#define PAIR_ADD(slot, v) do { } while (0)
#endif

static constexpr int BM = 128;        // rows per CTA; the pair tile is 2 * BM rows
static constexpr int BNP = 256;       // columns of the pair tile; each CTA stages BNP / 2 of them
static constexpr int BK = 64;         // bf16 elements per k-block (128 bytes); the int8 form has 128
static constexpr int A_BYTES = BM * 128;
static constexpr int B_BYTES = (BNP / 2) * 128;
static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB
static constexpr int STAGES = 6;
static constexpr int OUT_STAGE_BYTES = 128 * 128;
static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * OUT_STAGE_BYTES + 1024 + 256;

template <bool I8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const PairArgs args) {
  constexpr int S = STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* out_stage = smem + S * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + 2 * OUT_STAGE_BYTES);
  uint64_t* full = bars;               // used in the leader only
  uint64_t* empty = bars + S;          // per CTA
  uint64_t* tmem_full = bars + 2 * S;  // per CTA
  uint64_t* tmem_empty = bars + 2 * S + 2;  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int M = args.M, N = args.N, K = args.K;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (N + BNP - 1) / BNP;
  const int split_k = args.split_k > 1 ? args.split_k : 1;
  const int ntiles = tiles_m * tiles_n * split_k;
  constexpr int BKE = I8 ? 2 * BK : BK;   // elements per 128-byte k-block
  const int nkb_all = (K + BKE - 1) / BKE;
  const int kb_per_split = (nkb_all + split_k - 1) / split_k;
  constexpr int GROUP_M = 8;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);    // the leader's producer arrives with the byte count of both CTAs
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);  // 4 epilogue warps in each CTA
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_info = [&](int t, int& tm, int& tn, int& kb0, int& nkb) {
    kb0 = 0;
    nkb = nkb_all;
    if (split_k > 1) {
      const int per = tiles_m * tiles_n;
      const int ks = t / per;
      t -= ks * per;
      kb0 = ks * kb_per_split;
      nkb = min(kb_per_split, nkb_all - kb0);
    }
    const int per_group = GROUP_M * tiles_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(tiles_m - first_m, GROUP_M);
    tm = first_m + (t % per_group) % gsz;
    tn = (t % per_group) / gsz;
    return nkb > 0;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair_id; t < ntiles && ok; t += n_pairs) {
        int tm, tn, kb0, nkb;
        if (!tile_info(t, tm, tn, kb0, nkb)) continue;
        const int m0 = tm * 2 * BM + (int)rank * BM;       // this CTA's rows of A
        const int n0 = tn * BNP + (int)rank * (BNP / 2);   // this CTA's half of the B columns
        for (int kb = 0; kb < nkb; ++kb) {
          const long long w0 = PAIR_CLK();
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            set_error(args.err, ERR_WAIT_PRODUCER);
            ok = false;
            break;
          }
          PAIR_ADD(3 + (int)rank, PAIR_CLK() - w0);
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // Only the leader arrives on full[s], announcing the bytes of BOTH CTAs; the peer's copies
          // just complete on that barrier (a remote arrive per k-block costs the producer a cluster-
          // scope release, which made it the slowest role).  Bytes that land before the leader's
          // announcement leave the count negative for a moment; the phase cannot complete without
          // the leader's arrival.
          const uint32_t bar = map_to_rank(smem_u32(&full[stage]), 0);
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          const int k0 = (kb0 + kb) * BKE;
          if (!args.a_mn) {
            tma_load_2d_pair(sa, &tmA, bar, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * (BK * 128), &tmA, bar, m0 + c * 64, k0);
          }
          if (!args.b_mn) {
            tma_load_2d_pair(sb, &tmB, bar, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BNP / 128; ++c) tma_load_2d_pair(sb + c * (BK * 128), &tmB, bar, n0 + c * 64, k0);
          }
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      const uint32_t idesc = (I8 ? umma_idesc(2, 1, 1, 0, 0, 2 * BM, BNP) : umma_idesc(1, 1, 1, 0, 0, 2 * BM, BNP)) |
                             (uint32_t)(args.a_mn & 1) << 15 | (uint32_t)(args.b_mn & 1) << 16;
      const uint32_t a_adv = args.a_mn ? 16 * 128 : 32;
      const uint32_t b_adv = args.b_mn ? 16 * 128 : 32;
      const uint32_t a_lbo = args.a_mn ? BK * 128 : 16;
      const uint32_t b_lbo = args.b_mn ? BK * 128 : 16;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      const long long loop0 = PAIR_CLK();
      for (int t = pair_id; t < ntiles && ok; t += n_pairs) {
        int tm, tn, kb0, nkb;
        if (!tile_info(t, tm, tn, kb0, nkb)) continue;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        const long long e0 = PAIR_CLK();
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        PAIR_ADD(2, PAIR_CLK() - e0);
        const uint32_t d_tmem = tmem_base + acc * BNP;
        for (int kb = 0; kb < nkb; ++kb) {
          const long long f0 = PAIR_CLK();
          if (!mbar_wait(&full[stage], phase)) {
            set_error(args.err, ERR_WAIT_MMA_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          PAIR_ADD(1, PAIR_CLK() - f0);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_smem_desc(sa + k * a_adv, a_lbo, 1024);
            const uint64_t db = umma_smem_desc(sb + k * b_adv, b_lbo, 1024);
            if (I8) umma_i8_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0);
            else umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          // the slot is free in BOTH CTAs once these MMAs have read it
          const uint32_t e = smem_u32(&empty[stage]);
          umma_commit_pair(map_to_rank(e, 0));
          umma_commit_pair(map_to_rank(e, 1));
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t f = smem_u32(&tmem_full[acc]);
          umma_commit_pair(map_to_rank(f, 0));
          umma_commit_pair(map_to_rank(f, 1));
        }
      }
      PAIR_ADD(0, PAIR_CLK() - loop0);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int ew = warp & 3;  // TMEM lane quarter this warp may touch
    const uint32_t tmem_empty_leader0 = map_to_rank(smem_u32(&tmem_empty[0]), 0);
    const uint32_t tmem_empty_leader1 = map_to_rank(smem_u32(&tmem_empty[1]), 0);
    const bool f32out = args.out_mode != 0;
    const bool issuer = threadIdx.x == 128;
    const float alpha = args.alpha;
    int it = 0;
    int out_slabs = 0;
    for (int t = pair_id; t < ntiles; t += n_pairs) {
      int tm, tn, kb0, nkb;
      if (!tile_info(t, tm, tn, kb0, nkb)) continue;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      bool ok = mbar_wait(&tmem_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) set_error(args.err, ERR_WAIT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const int n0 = tn * BNP;
      const int y0 = tm * 2 * BM + (int)rank * BM;
      const int r_tile = ew * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(ew * 32) << 16) + acc * BNP;
#pragma unroll 1
      for (int c = 0; c < BNP / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) break;  // uniform across the CTA
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        if (c == BNP / 32 - 1 || col0 + 32 >= N) {  // last TMEM read of this tile: release the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc ? tmem_empty_leader1 : tmem_empty_leader0);
        }
        float v[32];
        if (I8) {
          const int grow = y0 + r_tile;
          const float sm = (args.scale_m && grow < M) ? args.scale_m[grow] * alpha : alpha;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float sn = args.scale_n ? ((col0 + j < N) ? args.scale_n[col0 + j] : 0.f) : 1.f;
            v[j] = (float)(int)r[j] * sm * sn;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
        }
        const int slab = f32out ? c : (c >> 1);
        const bool first_half = f32out || (c & 1) == 0;
        const bool last_half = f32out || (c & 1) == 1 || col0 + 32 >= N;
        uint8_t* buf = out_stage + (out_slabs & 1) * OUT_STAGE_BYTES;
        if (first_half) {
          // the store that last used this buffer (two slabs ago) must have finished reading it
          if (issuer) tma_store_wait_read<1>();
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        uint8_t* prow = buf + r_tile * 128;
        if (f32out) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(prow + ((q ^ (r_tile & 7)) << 4)) =
                make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
            *reinterpret_cast<uint4*>(prow + ((((c & 1) * 4 + q) ^ (r_tile & 7)) << 4)) = o;
          }
        }
        if (last_half) {
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
            const int x0 = n0 + slab * (f32out ? 32 : 64);
            if (args.out_mode == 2) tma_reduce_add_2d(&tmC, buf, x0, y0);
            else tma_store_2d(&tmC, buf, x0, y0);
            tma_store_commit();
          }
          ++out_slabs;
        }
      }
    }
    if (issuer) tma_store_wait<0>();  // smem must outlive the bulk stores that read it
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its peer may still signal it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace pair
}  // namespace bb

#ifdef BB_TIMELINE
static long long* g_pair_dbg = nullptr;
BB_API int bb_gemm_pair_set_debug(long long* buf) {
  g_pair_dbg = buf;
  return 0;
}
#endif

// Number of 2-CTA clusters the current device runs at once, as found by the first launch (0 before).
static std::atomic<int> g_last_pairs_fit{0};
BB_API int bb_gemm_pair_clusters() { return g_last_pairs_fit.load(); }

// Pair-tile bf16 GEMM (see the top of the file).  Same argument meaning as bb_gemm_bf16; serves
// out_mode 0 / 1 / 2 without bias.  Returns BB_ESIZE when the shape or alignment does not suit the
// pair kernel (the caller then uses the single-CTA kernel): C must be 16-byte aligned with a
// 16-byte pitch, and the grid is sized to whole CTA pairs.
template <bool I8>
static int launch_pair(const void* A, const void* B, void* C, const float* scale_m, const float* scale_n, int M,
                       int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode, float alpha,
                       int split_k, int max_ctas, void* stream) {
  using namespace bb;
  using namespace bb::pair;
  if (M <= 0 || N <= 0 || K <= 0 || out_mode < 0 || out_mode > 2) return BB_EARG;
  if (I8 && (a_mn || b_mn || out_mode != 0)) return BB_EARG;
  const bool f32out = out_mode != 0;
  const int ces = f32out ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || ((uint64_t)ldc * ces) % 16) return BB_ESIZE;
  const CUtensorMapDataType dt = I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  constexpr int ES = I8 ? 1 : 2;             // operand element bytes
  constexpr int BKE = I8 ? 2 * BK : BK;      // elements per 128-byte k-block
  CUtensorMap tmA, tmB, tmC;
  int rc = !a_mn ? make_tmap_2d(&tmA, dt, ES, A, K, M, (uint64_t)lda * ES, BKE, BM)
                 : make_tmap_2d(&tmA, dt, ES, A, M, K, (uint64_t)lda * ES, 64, BK);
  if (rc) return rc;
  rc = !b_mn ? make_tmap_2d(&tmB, dt, ES, B, K, N, (uint64_t)ldb * ES, BKE, BNP / 2)
             : make_tmap_2d(&tmB, dt, ES, B, N, K, (uint64_t)ldb * ES, 64, BK);
  if (rc) return rc;
  rc = make_tmap_2d(&tmC, f32out ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ces,
                    C, N, M, (uint64_t)ldc * ces, f32out ? 32 : 64, BM);
  if (rc) return rc;
  static PerDeviceOnce smem_once;
  {
    cudaError_t e = ensure_dyn_smem(smem_once, gemm_pair_kernel<I8>, SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  // how many 2-CTA clusters the device holds at once (an odd SM count per GPC leaves one SM out)
  static std::atomic<int> max_pairs[64];
  int dev = 0;
  cudaGetDevice(&dev);
  int pairs_fit = (dev >= 0 && dev < 64) ? max_pairs[dev].load(std::memory_order_relaxed) : 0;
  if (pairs_fit == 0) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<I8>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2 - 2;
    }
    pairs_fit = n;
    if (dev >= 0 && dev < 64) max_pairs[dev].store(n, std::memory_order_relaxed);
  }
  {
    static const int forced = [] {
      const char* e = getenv("BB_PAIR_CLUSTERS");
      return e ? atoi(e) : 0;
    }();
    if (forced > 0) pairs_fit = forced;
  }
  g_last_pairs_fit.store(pairs_fit);
  PairArgs a{};
  a.scale_m = scale_m;
  a.scale_n = scale_n;
  a.alpha = alpha;
  a.M = M;
  a.N = N;
  a.K = K;
  a.a_mn = a_mn;
  a.b_mn = b_mn;
  a.out_mode = out_mode;
  a.split_k = (out_mode == 2 && split_k > 1) ? split_k : 1;
  a.err = device_error_word();
#ifdef BB_TIMELINE
  a.dbg = g_pair_dbg;
#endif
  const long tiles = (long)((M + 2 * BM - 1) / (2 * BM)) * ((N + BNP - 1) / BNP) * a.split_k;
  long pairs = tiles < pairs_fit ? tiles : pairs_fit;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  if (pairs < 1) pairs = 1;
  gemm_pair_kernel<I8><<<(int)(2 * pairs), 256, SMEM, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, tmC, a);
  return (int)cudaGetLastError();
}

BB_API int bb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                             int ldb, int ldc, int a_mn, int b_mn, int out_mode, float alpha,
                             int split_k, int max_ctas, void* stream) {
  return launch_pair<false>(A, B, C, nullptr, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, alpha,
                            split_k, max_ctas, stream);
}

// W8A8 on CTA pairs: C[M,N] bf16 = (A[M,K] int8 . B[N,K]^T int8) * scale_m[row] * scale_n[col].
// Same restrictions as the bf16 form (BB_ESIZE when C's alignment does not suit the TMA store).
BB_API int bb_gemm_i8_pair(const void* A, const void* B, void* C, const float* scale_m, const float* scale_n,
                           int M, int N, int K, int lda, int ldb, int ldc, int max_ctas, void* stream) {
  if ((lda % 16) || (ldb % 16)) return bb::BB_ESIZE;   // TMA pitch: multiples of 16 bytes
  return launch_pair<true>(A, B, C, scale_m, scale_n, M, N, K, lda, ldb, ldc, 0, 0, 0, 1.f, 1, max_ctas, stream);
}
