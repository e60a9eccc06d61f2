// Persistent warp-specialised GEMM on the 5th-gen tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA into a 128-byte-swizzled shared-memory ring).
//
//   C[M,N] (op)= alpha * A[M,K] * B[N,K]^T (+ bias[N])
//
// A and B can each be K-major ([rows][K], K contiguous — the nn.Linear layout) or MN-major
// ([K][rows], rows contiguous), so forward (x·Wᵀ), dX (dy·W) and dW (dyᵀ·x) all run on the same
// kernel without a transpose pass.  The int8 variant (kind::i8, s32 accumulate) applies per-row
// and per-column scales in the epilogue (W8A8).
//
// Replaces the reference's register-tiled fp32 GEMM family (crates/kernels/wgsl/matmul_reg3.wgsl,
// matmul_dx_reg.wgsl, matmul_dw_reg.wgsl, matmul_i8_dyn.wgsl).
//
// Roles (256 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane),
// warp 2 = TMEM allocator, warps 4..7 = epilogue (TMEM -> registers -> global).
// Two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
#include <cstdlib>

#include "../common/host.hpp"
#include "../common/peer.cuh"
#include "../common/ptx.cuh"

namespace bb {

struct GemmArgs {
  void* C;
  const float* bias;     // [N] or null
  const float* scale_m;  // int8: per-row (token) scale, else null
  const float* scale_n;  // int8: per-column (channel) scale, else null
  float alpha;
  int M, N, K;
  int ldc;
  int a_mn, b_mn;
  int out_mode;  // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate, 3 bf16 store of gelu(x) (tanh)
  int split_k;   // >1 (accumulate mode only): the k-blocks are cut into this many slices, each slice is a
                 // tile of its own and adds its partial product into C
  // Grouped (mixture-of-experts) GEMMs, one launch for all experts:
  //  mode 1 "row-grouped": A rows are expert-sorted and padded so every 128-row tile belongs to one
  //         expert; tile_group[tile_m] names it (-1 = unused tile, skipped); B holds the experts'
  //         matrices stacked along its row (K-major) / k (MN-major) axis, b_group_rows apart.
  //  mode 2 "k-grouped" (weight gradients): group g reduces over rows [group_offsets[g],
  //         group_offsets[g+1]) (multiples of 128) of the MN-major A and B and writes
  //         C + g * c_group_stride.  Empty groups are skipped (use with accumulate or zeroed C).
  int group_mode;
  const int* tile_group;
  int b_group_rows;
  const int* group_offsets;
  int num_groups;
  long c_group_stride;
  int* err;
  long long* timeline;  // optional [tiles][8] clock64 stamps of CTA 0 (profiling aid)
  int tma_store;        // 1: epilogue stages 128-byte-row slabs in smem and writes them with TMA
  // Tensor-parallel fusion (sequence-parallel Megatron layout), rows split evenly over tp ranks:
  //  mode 1 "all-gather -> GEMM": the first tp_copy_ctas CTAs only move data: they pull every
  //         rank's [rows_per_rank, K] shard of A over NVLink (plain peer loads) into the local
  //         [M, K] buffer that tmA maps and publish one flag per 128-row tile; the remaining CTAs
  //         run the GEMM, local rows first, and their TMA producer waits (bounded) on the flag of
  //         the tile row it is about to read.  Each remote row crosses NVLink exactly once.
  //  mode 2 "GEMM -> reduce-scatter": the epilogue TMA-stores every output tile into slot
  //         [tp_rank] of the receive buffer of the rank that owns those rows (tp_cmaps[dest]); the
  //         last CTA to finish exchanges "landed" flags with all peers, so when the kernel ends
  //         every rank holds all tp partials of its rows (summed by the consumer kernel).
  int tp_mode;
  int tp_rank, tp_world;
  int rows_per_rank;
  PeerPtrs tp_src;
  void* tp_full;
  int* tp_row_flags;
  int tp_copy_ctas;
  PeerPtrs tp_sig;
  uint32_t tp_epoch;
  const CUtensorMap* tp_cmaps;
  unsigned int* tp_counter;
  long long tp_wait_limit;
  //  mode 3 "expert dispatch -> grouped GEMM" (row-grouped GEMMs only): the mover CTAs fill the
  //         expert-sorted operand buffer (tp_full, [M, K]) tile by tile with the token rows routed to
  //         this rank's experts, pulled from every rank's symmetric activation buffer (tp_src) by the
  //         dispatch table ep_pair_of_pos (pair = token * ep_k + slot, token = rank * ep_n_per_rank +
  //         local; < 0 = padding row, zero-filled), optionally scaled by the pair's routing weight.
  //         A tile's flag is published when its 128 rows are in place and the GEMM side waits per
  //         tile, so the all-to-all runs under the expert GEMM instead of in front of it.
  const int* ep_pair_of_pos;
  const float* ep_w;
  int ep_n_per_rank, ep_k;
  // "grouped GEMM -> expert combine" (row-grouped, bf16 output): output row `row` belongs to routed
  // pair sc_pair[row] (< 0: padding row, not stored); the epilogue stores it straight into slot
  // (pair % sc_pairs_per_rank) of the [pairs_per_rank, ldc] slot buffer of the rank that owns the
  // token (pair / sc_pairs_per_rank; sc_dst.p[rank], symmetric memory), so the return all-to-all is
  // the GEMM's own stores, tile by tile, and the owner only sums its k slots per token afterwards.
  const int* sc_pair;
  PeerPtrs sc_dst;
  int sc_pairs_per_rank;
};

// Per-tile clock64 stamps exist only in profiling builds (-DBB_TIMELINE): in production the stamp
// pointer is a compile-time null, so the kernels carry no clock reads.
#ifdef BB_TIMELINE
#define GEMM_TL(expr) (expr)
#else
#define GEMM_TL(expr) (static_cast<long long*>(nullptr))
#endif

static constexpr int BM = 128;

// Peer-memory copy of n 16-byte vectors by `nthreads` threads (this one is `tid`): every thread issues
// U loads before its first store, so U x 16 bytes per thread are in flight.  (A load-then-store loop
// keeps ONE load per thread in flight: with a peer round trip of about 2 us, 16 mover CTAs of 256
// threads then pull 32 GB/s over a 770 GB/s link.)
template <int U>
__device__ __forceinline__ void copy_vecs_batched(uint4* __restrict__ dst, const uint4* src, size_t n, int tid,
                                                  int nthreads) {
  for (size_t v0 = tid; v0 < n; v0 += (size_t)nthreads * U) {
    uint4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + (size_t)u * nthreads;
      if (v < n) x[u] = ld_volatile_u4(src + v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + (size_t)u * nthreads;
      if (v < n) dst[v] = x[u];
    }
  }
}
static constexpr int TILE_K_BYTES = 128;  // one swizzle row

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * TILE_K_BYTES;  // 16 KB
  static constexpr int B_BYTES = BN * TILE_K_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int OUT_STAGE_BYTES = 128 * 128;  // one [128 rows][128 B] output slab
  static constexpr int SMEM =
      STAGES * STAGE_BYTES + 2 * OUT_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}

template <int BN, bool I8>
__global__ void __launch_bounds__(256, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const GemmArgs args) {
  using Cfg = GemmCfg<BN>;
  constexpr int S = Cfg::STAGES;
  constexpr int BK = I8 ? 128 : 64;      // elements per k-block (128 bytes)
  constexpr int UK = I8 ? 32 : 16;       // elements per tcgen05.mma
  constexpr int NK = BK / UK;            // 4 MMAs per k-block

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* out_stage = smem + S * Cfg::STAGE_BYTES;  // 2 slabs, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + 2 * Cfg::OUT_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* tmem_full = bars + 2 * S;
  uint64_t* tmem_empty = bars + 2 * S + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int M = args.M, N = args.N, K = args.K;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int split_k = args.split_k > 1 ? args.split_k : 1;
  const int ntiles = tiles_m * tiles_n * (args.group_mode == 2 ? args.num_groups : split_k);
  const int nkb_all = (K + BK - 1) / BK;
  const int kb_per_split = (nkb_all + split_k - 1) / split_k;
  constexpr int GROUP_M = 16;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile index -> coordinates, group, and k-block range; returns false when the tile is skipped.
  // Every role evaluates this identically, so their pipeline counters stay in step.
  auto tile_info = [&](int t, int& tm, int& tn, int& grp, int& kb0, int& nkb) -> bool {
    grp = 0;
    kb0 = 0;
    nkb = nkb_all;
    if (args.group_mode == 2) {
      const int per = tiles_m * tiles_n;
      grp = t / per;
      t -= grp * per;
      const int r0 = args.group_offsets[grp], r1 = args.group_offsets[grp + 1];
      kb0 = r0 / BK;
      nkb = (r1 - r0) / BK;
    } else if (split_k > 1) {  // slice index outermost: neighbouring tiles share the slice's A/B panels in L2
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
    if (args.group_mode == 1) {
      grp = args.tile_group[tm];
      if (grp < 0) return false;
    }
    if (args.tp_mode) {  // start with this rank's own rows (mode 1) / the next rank's rows (mode 2)
      const int per_rank = args.rows_per_rank / BM;
      tm = (tm + (args.tp_rank + (args.tp_mode == 2 ? 1 : 0)) * per_rank) % tiles_m;
    }
    return nkb > 0;
  };
  const bool gated = args.tp_mode == 1 || args.tp_mode == 3;  // A tiles arrive through mover CTAs
  const int n_copy = gated ? args.tp_copy_ctas : 0;
  const int cta0 = (int)blockIdx.x - n_copy;
  const int cta_stride = (int)gridDim.x - n_copy;

  if (cta0 < 0 && args.tp_mode == 3 && args.ep_w == nullptr &&
      (size_t)K * 2 <= (size_t)Cfg::STAGE_BYTES) {
    // ---------------------------------------------------------- expert-dispatch data movers (copy engine)
    // Unscaled rows: one thread per mover CTA drives bulk copies (peer or local row -> a slot of this
    // CTA's unused stage ring -> the expert-sorted operand buffer), R rows per slot, S slots in
    // flight; the other warps zero-fill the padding rows at the tail of the tile.  A tile's routed
    // rows form a prefix of its 128 positions (positions are handed out consecutively per expert
    // and experts are padded to whole tiles); a tile where that does not hold takes the register path.
    __shared__ int s_pair[BM];
    const size_t row_bytes = (size_t)K * 2;
    const int R = (int)(Cfg::STAGE_BYTES / row_bytes);
    constexpr int LA = S - 2;
    long n_ld = 0, n_st = 0;          // slot uses so far (thread 0 only)
    for (int tmr = blockIdx.x; tmr < tiles_m; tmr += n_copy) {
      if (args.tile_group[tmr] < 0) continue;    // unused tile: the GEMM side skips it too
      __syncthreads();                           // s_pair of the previous tile is no longer read
      if (threadIdx.x < BM) s_pair[threadIdx.x] = args.ep_pair_of_pos[tmr * BM + threadIdx.x];
      const int n_valid = __syncthreads_count(threadIdx.x < BM && s_pair[threadIdx.x] >= 0);
      const int prefix_ok = __syncthreads_and(threadIdx.x >= BM || ((s_pair[threadIdx.x] >= 0) == ((int)threadIdx.x < n_valid)));
      uint8_t* tile_dst = reinterpret_cast<uint8_t*>(args.tp_full) + (size_t)tmr * BM * row_bytes;
      if (!prefix_ok) {
        for (int r = warp; r < BM; r += 8) {
          uint4* dst = reinterpret_cast<uint4*>(tile_dst + (size_t)r * row_bytes);
          const int pair = s_pair[r];
          if (pair < 0) {
            for (size_t v = lane; v < row_bytes / 16; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
            continue;
          }
          const int token = pair / args.ep_k;
          const int src_rank = token / args.ep_n_per_rank;
          const int local = token - src_rank * args.ep_n_per_rank;
          copy_vecs_batched<8>(dst, reinterpret_cast<const uint4*>(args.tp_src.p[src_rank]) + (size_t)local * (row_bytes / 16),
                               row_bytes / 16, lane, 32);
        }
      } else if (threadIdx.x == 0) {
        const int G = (n_valid + R - 1) / R;
        bool ok = true;
        for (int g = 0; g < G + LA && ok; ++g) {
          if (g < G) {
            const int slot = (int)(n_ld % S);
            if (n_ld >= S) tma_store_wait_read<1>();
            const int r0 = g * R, r1 = min(r0 + R, n_valid);
            mbar_expect_tx(&full[slot], (uint32_t)((r1 - r0) * row_bytes));
            for (int r = r0; r < r1; ++r) {
              const int pair = s_pair[r];
              const int token = pair / args.ep_k;
              const int src_rank = token / args.ep_n_per_rank;
              const int local = token - src_rank * args.ep_n_per_rank;
              bulk_load(smem + (size_t)slot * Cfg::STAGE_BYTES + (size_t)(r - r0) * row_bytes,
                        reinterpret_cast<const uint8_t*>(args.tp_src.p[src_rank]) + (size_t)local * row_bytes,
                        (uint32_t)row_bytes, &full[slot]);
            }
            ++n_ld;
          }
          const int k = g - LA;
          if (k >= 0 && k < G) {
            const int slot = (int)(n_st % S);
            if (!mbar_wait(&full[slot], (uint32_t)((n_st / S) & 1))) {
              set_error(args.err, ERR_WAIT_PEER);
              ok = false;
              break;
            }
            const int r0 = k * R, r1 = min(r0 + R, n_valid);
            bulk_store(tile_dst + (size_t)r0 * row_bytes, smem + (size_t)slot * Cfg::STAGE_BYTES,
                       (uint32_t)((r1 - r0) * row_bytes));
            tma_store_commit();
            ++n_st;
          }
        }
        tma_store_wait<0>();                     // the tile's routed rows are written
        asm volatile("fence.proxy.async;" ::: "memory");
      } else if (warp >= 1) {
        for (int r = n_valid + (warp - 1); r < BM; r += 7) {
          uint4* dst = reinterpret_cast<uint4*>(tile_dst + (size_t)r * row_bytes);
          for (size_t v = lane; v < row_bytes / 16; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) st_release_gpu_s32(args.tp_row_flags + tmr, (int)args.tp_epoch);
    }
  } else if (cta0 < 0 && args.tp_mode == 3) {
    // ---------------------------------------------------------- expert-dispatch data movers (registers:
    // rows scaled by their routing weight on the way, or rows wider than a ring slot)
    const size_t row_vecs = (size_t)K * 2 / 16;  // 16-byte vectors per row
    for (int tmr = blockIdx.x; tmr < tiles_m; tmr += n_copy) {
      if (args.tile_group[tmr] < 0) continue;    // unused tile: the GEMM side skips it too
      for (int r = warp; r < BM; r += 8) {
        const int pos = tmr * BM + r;
        const int pair = pos < M ? args.ep_pair_of_pos[pos] : -1;
        uint4* dst = reinterpret_cast<uint4*>(args.tp_full) + (size_t)pos * row_vecs;
        if (pos >= M) continue;
        if (pair < 0) {
          for (size_t v = lane; v < row_vecs; v += 32) dst[v] = make_uint4(0u, 0u, 0u, 0u);
          continue;
        }
        const int token = pair / args.ep_k;
        const int src_rank = token / args.ep_n_per_rank;
        const int local = token - src_rank * args.ep_n_per_rank;
        const uint4* src = reinterpret_cast<const uint4*>(args.tp_src.p[src_rank]) + (size_t)local * row_vecs;
        if (args.ep_w) {
          const float g = args.ep_w[pair];
          for (size_t v0 = lane; v0 < row_vecs; v0 += 32 * 8) {
            uint4 x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (v0 + u * 32 < row_vecs) x[u] = ld_volatile_u4(src + v0 + u * 32);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              if (v0 + u * 32 >= row_vecs) continue;
              auto scaled = [g](uint32_t w) {
                return pack_bf16x2(__uint_as_float(w << 16) * g, __uint_as_float(w & 0xFFFF0000u) * g);
              };
              dst[v0 + u * 32] = make_uint4(scaled(x[u].x), scaled(x[u].y), scaled(x[u].z), scaled(x[u].w));
            }
          }
        } else {
          copy_vecs_batched<8>(dst, src, row_vecs, lane, 32);
        }
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) st_release_gpu_s32(args.tp_row_flags + tmr, (int)args.tp_epoch);
    }
  } else if (cta0 < 0) {
    // ---------------------------------------------------------- all-gather data movers
    // One thread per mover CTA drives the copy engine: bulk loads pull a peer's rows into this CTA's
    // (otherwise unused) stage ring, bulk stores put them into the local landing buffer.  S slots
    // of STAGE_BYTES are in flight per CTA without holding a register (a register copy keeps 32 KB per
    // CTA in flight at best).  More, smaller slots (one per spare mbarrier, 10 x 19 KB) measured slower:
    // 783 against 675 us on 16384 x 6144 x 4096 at 2 ranks; the single issuing thread pays per chunk.
    const int per_rank = args.rows_per_rank / BM;
    if (blockIdx.x == 0 && threadIdx.x < args.tp_world) {  // "my shard is complete"
      __threadfence_system();
      st_release_sys_u64(reinterpret_cast<uint64_t*>(args.tp_sig.p[threadIdx.x]) + args.tp_rank,
                         (uint64_t)args.tp_epoch);
    }
    if (threadIdx.x == 0) {
      const size_t row_bytes = (size_t)K * (I8 ? 1 : 2);
      constexpr uint32_t SLOT = Cfg::STAGE_BYTES;
      constexpr int LA = S - 2;          // loads run LA chunks ahead of the stores
      // chunk cursor: (tile slot i of this CTA, byte offset inside the tile)
      struct Cur {
        int i;
        size_t off;
      };
      auto tile_of = [&](int i) { return (i + args.tp_rank * per_rank) % tiles_m; };
      auto tile_bytes = [&](int tmr) { return (size_t)min(BM, M - tmr * BM) * row_bytes; };
      auto advance = [&](Cur& c) {
        c.off += SLOT;
        if (c.off >= tile_bytes(tile_of(c.i))) {
          c.i += n_copy;
          c.off = 0;
        }
      };
      Cur ld{(int)blockIdx.x, 0}, stc{(int)blockIdx.x, 0};
      bool ok = true;
      int waited_rank = -1;
      for (long n = 0; ok; ++n) {
        const bool have_load = ld.i < tiles_m;
        if (!have_load && stc.i >= tiles_m) break;
        if (have_load) {
          const int tmr = tile_of(ld.i);
          const int src_rank = tmr / per_rank;
          if (ld.off == 0 && src_rank != waited_rank) {   // first touch of a peer's shard: it must be complete
            const uint64_t* flag = reinterpret_cast<const uint64_t*>(args.tp_sig.p[args.tp_rank]) + src_rank;
            if (!wait_epoch(flag, args.tp_epoch, 0, args.tp_wait_limit)) {
              set_error(args.err, ERR_WAIT_PEER);
              ok = false;
              break;
            }
            waited_rank = src_rank;
          }
          if (n >= S) tma_store_wait_read<1>();             // the store that last read this slot is done with it
          const size_t tb = tile_bytes(tmr);
          const uint32_t bytes = (uint32_t)min((size_t)SLOT, tb - ld.off);
          const uint8_t* src = reinterpret_cast<const uint8_t*>(args.tp_src.p[src_rank]) +
                               (size_t)(tmr - src_rank * per_rank) * BM * row_bytes + ld.off;
          const int slot = (int)(n % S);
          mbar_expect_tx(&full[slot], bytes);
          bulk_load(smem + (size_t)slot * SLOT, src, bytes, &full[slot]);
          advance(ld);
        }
        const long k = n - LA;
        if (k >= 0 && stc.i < tiles_m) {
          const int slot = (int)(k % S);
          if (!mbar_wait(&full[slot], (uint32_t)((k / S) & 1))) {
            set_error(args.err, ERR_WAIT_PEER);
            ok = false;
            break;
          }
          const int tmr = tile_of(stc.i);
          const size_t tb = tile_bytes(tmr);
          const uint32_t bytes = (uint32_t)min((size_t)SLOT, tb - stc.off);
          uint8_t* dst = reinterpret_cast<uint8_t*>(args.tp_full) + (size_t)tmr * BM * row_bytes + stc.off;
          bulk_store(dst, smem + (size_t)slot * SLOT, bytes);
          tma_store_commit();
          const bool tile_done = stc.off + SLOT >= tb;
          advance(stc);
          if (tile_done) {
            tma_store_wait<0>();                            // the tile's rows are written
            asm volatile("fence.proxy.async;" ::: "memory");
            __threadfence();
            st_release_gpu_s32(args.tp_row_flags + tmr, (int)args.tp_epoch);
          }
        }
      }
      tma_store_wait<0>();
    }
  } else

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int armed_stage = -1;
      uint32_t armed_phase = 0;
      bool ok = true;
      for (int t = cta0; t < ntiles && ok; t += cta_stride) {
        int tm, tn, grp, kb0, nkb;
        if (!tile_info(t, tm, tn, grp, kb0, nkb)) continue;
        const int m0 = tm * BM, n0 = tn * BN;
        const int b_off = args.group_mode == 1 ? grp * args.b_group_rows : 0;
        if (gated) {
          if (!wait_flag_ge(args.tp_row_flags + tm, (int)args.tp_epoch, args.tp_wait_limit)) {
            set_error(args.err, ERR_WAIT_PEER);
            ok = false;
            break;
          }
          // rows were written by ordinary stores of another CTA; TMA reads them via the async proxy
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            set_error(args.err, ERR_WAIT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const int k0 = (kb0 + kb) * BK;
          if (!args.a_mn) {
            tma_load_2d(sa, &tmA, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (BK * 128), &tmA, &full[stage], m0 + c * 64, k0);
          }
          if (!args.b_mn) {
            tma_load_2d(sb, &tmB, &full[stage], k0, b_off + n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (BK * 128), &tmB, &full[stage], n0 + c * 64, b_off + k0);
          }
          armed_stage = stage;
          armed_phase = phase;
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // On the error path give copies still in flight a bounded chance to land before exit.
      if (!ok && armed_stage >= 0) (void)mbar_wait(&full[armed_stage], armed_phase);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_base = I8 ? umma_idesc(2, 1, 1, 0, 0, BM, BN)
                                         : umma_idesc(1, 1, 1, 0, 0, BM, BN);
      const uint32_t idesc =
          idesc_base | (uint32_t)(args.a_mn & 1) << 15 | (uint32_t)(args.b_mn & 1) << 16;
      // K-major: advance 32 B per MMA inside the swizzle row; MN-major: UK k-rows of 128 B.
      const uint32_t a_adv = args.a_mn ? UK * 128 : 32;
      const uint32_t b_adv = args.b_mn ? UK * 128 : 32;
      const uint32_t a_lbo = args.a_mn ? BK * 128 : 16;
      const uint32_t b_lbo = args.b_mn ? BK * 128 : 16;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = cta0; t < ntiles && ok; t += cta_stride) {
        int tm, tn, grp, kb0, nkb;
        if (!tile_info(t, tm, tn, grp, kb0, nkb)) continue;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        long long* const tl = GEMM_TL((args.timeline && blockIdx.x == 0 && it <= 16) ? args.timeline + (it - 1) * 16 : nullptr);
        if (tl) tl[0] = clock64();
        long long waited = 0;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          set_error(args.err, ERR_WAIT_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          const long long w0 = tl ? clock64() : 0;
          if (kb == 0 && tl) tl[1] = w0;
          if (!mbar_wait(&full[stage], phase)) {
            set_error(args.err, ERR_WAIT_MMA_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          if (tl) waited += clock64() - w0;
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < NK; ++k) {
            const uint64_t da = umma_smem_desc(sa + k * a_adv, a_lbo, 1024);
            const uint64_t db = umma_smem_desc(sb + k * b_adv, b_lbo, 1024);
            if (I8)
              umma_i8_ss(d_tmem, da, db, idesc, (kb | k) != 0);
            else
              umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty[stage]);  // frees the smem slot once these MMAs have read it
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
        if (tl) {
          tl[2] = waited;      // cycles spent waiting for TMA data in this tile
          tl[3] = clock64();   // all MMAs of the tile issued
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int ew = warp & 3;  // TMEM lane quarter this warp may touch
    int it = 0;
    int out_slabs = 0;  // staged slabs issued so far (selects the staging buffer)
    for (int t = cta0; t < ntiles; t += cta_stride) {
      int tm, tn, grp, kb0, nkb;
      if (!tile_info(t, tm, tn, grp, kb0, nkb)) continue;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      long long* const tl = GEMM_TL((args.timeline && blockIdx.x == 0 && it <= 16 && threadIdx.x == 128) ? args.timeline + (it - 1) * 16 : nullptr);
      if (tl) tl[4] = clock64();
      bool ok = mbar_wait(&tmem_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) set_error(args.err, ERR_WAIT_EPILOGUE);
        break;
      }
      tc_fence_after();
      if (tl) tl[5] = clock64();
      const size_t c_off = args.group_mode == 2 ? (size_t)grp * args.c_group_stride : 0;
      const int row = tm * BM + ew * 32 + lane;
      const int n0 = tn * BN;
      const bool row_ok = row < M;
      const float sm = (I8 && row_ok && args.scale_m) ? args.scale_m[row] : 1.f;
      const uint32_t t_row = tmem_base + ((uint32_t)(ew * 32) << 16) + acc * BN;
      if (args.tma_store) {
        // ---- staged epilogue: registers -> 128B-swizzled smem slab -> TMA store / reduce-add
        const bool f32out = args.out_mode == 1 || args.out_mode == 2;
        const int r_tile = ew * 32 + lane;  // row inside the tile
        const int y0 = tm * BM + (args.group_mode == 2 ? grp * M : 0);
        const bool issuer = threadIdx.x == 128;
        const float alpha = args.alpha;
        const float* __restrict__ bias = args.bias;
        const float* __restrict__ scale_n = args.scale_n;
        const bool do_gelu = args.out_mode == 3;
        const bool plain_epilogue = bias == nullptr && !do_gelu;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;  // uniform across the CTA
          uint32_t r[32];
          __syncwarp();
          tmem_ld32(t_row + c * 32, r);
          tmem_wait_ld();
          if (c == BN / 32 - 1 || col0 + 32 >= N) {  // last TMEM read of this tile: release it early
            tc_fence_before();
            mbar_arrive(&tmem_empty[acc]);
          }
          float v[32];
          if (!I8 && plain_epilogue) {
            // hot path: nothing but the scale (the general path's per-element tests cost ~30
            // cycles per element and made the epilogue the bottleneck of K ~ 1024 GEMMs)
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = I8 ? (float)(int)r[j] : __uint_as_float(r[j]);
              x *= alpha;
              if (I8) {
                x *= sm;
                if (scale_n) x *= (col0 + j < N) ? scale_n[col0 + j] : 0.f;
              }
              if (bias && col0 + j < N) x += bias[col0 + j];
              if (do_gelu) x = gelu_tanh(x);
              v[j] = x;
            }
          }
          const int slab = f32out ? c : (c >> 1);
          const bool first_half = f32out || (c & 1) == 0;
          const bool last_half = f32out || (c & 1) == 1 || col0 + 32 >= N;
          uint8_t* buf = out_stage + (out_slabs & 1) * Cfg::OUT_STAGE_BYTES;
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
              if (args.tp_mode == 2) {
                const int per_rank = args.rows_per_rank / BM;
                const int dest = tm / per_rank;
                const int yd = (tm - dest * per_rank) * BM + args.tp_rank * args.rows_per_rank;
                tma_store_2d(args.tp_cmaps + dest, buf, x0, yd);
              } else if (args.out_mode == 2) {
                tma_reduce_add_2d(&tmC, buf, x0, y0);
              } else {
                tma_store_2d(&tmC, buf, x0, y0);
              }
              tma_store_commit();
            }
            ++out_slabs;
          }
        }
        if (tl) tl[6] = clock64();
        continue;
      }
      // combine epilogue: this thread's row goes to the token owner's slot buffer (or nowhere)
      __nv_bfloat16* sc_base = nullptr;
      bool sc_skip = false;
      if (args.sc_pair) {
        const int pair = row_ok ? args.sc_pair[row] : -1;
        if (pair < 0) {
          sc_skip = true;
        } else {
          const int dest = pair / args.sc_pairs_per_rank;
          sc_base = reinterpret_cast<__nv_bfloat16*>(args.sc_dst.p[dest]) +
                    (size_t)(pair - dest * args.sc_pairs_per_rank) * args.ldc;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (!row_ok || col0 >= N || sc_skip) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float x = I8 ? (float)(int)r[j] : __uint_as_float(r[j]);
          x *= args.alpha;
          if (I8) {
            x *= sm;
            if (args.scale_n) x *= (col0 + j < N) ? args.scale_n[col0 + j] : 0.f;
          }
          if (args.bias && col0 + j < N) x += args.bias[col0 + j];
          v[j] = x;
        }
        const bool full_chunk = (col0 + 32 <= N);
        if (args.out_mode == 0 || args.out_mode == 3) {
          if (args.out_mode == 3) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
          }
          __nv_bfloat16* crow = sc_base ? sc_base + col0
                                        : reinterpret_cast<__nv_bfloat16*>(args.C) + c_off +
                                              (size_t)row * args.ldc + col0;
          if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
            uint4* dst = reinterpret_cast<uint4*>(crow);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              dst[q] = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < N; ++j) crow[j] = __float2bfloat16(v[j]);
          }
        } else {
          float* crow = reinterpret_cast<float*>(args.C) + c_off + (size_t)row * args.ldc + col0;
          const bool accum = args.out_mode == 2;
          if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
            float4* dst = reinterpret_cast<float4*>(crow);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (accum) {
                const float4 old = dst[q];
                o.x += old.x;
                o.y += old.y;
                o.z += old.z;
                o.w += old.w;
              }
              dst[q] = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < N; ++j) crow[j] = accum ? crow[j] + v[j] : v[j];
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
      if (tl) tl[6] = clock64();
    }
  }

  if (args.tma_store && threadIdx.x == 128) tma_store_wait<0>();  // smem must outlive the reads
  if (args.tp_mode == 2) {
    // all of this CTA's tiles are written; the last CTA of the grid tells every peer and waits
    // until every peer has told us, so the kernel's end means "all partials of my rows landed"
    __shared__ bool s_last;
    if (threadIdx.x == 128) {
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence_system();
      s_last = atomicAdd(args.tp_counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last && threadIdx.x < args.tp_world) {
      st_release_sys_u64(reinterpret_cast<uint64_t*>(args.tp_sig.p[threadIdx.x]) + args.tp_world +
                             args.tp_rank,
                         (uint64_t)args.tp_epoch);
      const uint64_t* flag = reinterpret_cast<const uint64_t*>(args.tp_sig.p[args.tp_rank]) +
                             args.tp_world + threadIdx.x;
      if (!wait_epoch(flag, args.tp_epoch, 0, args.tp_wait_limit)) set_error(args.err, ERR_WAIT_PEER);
      if (threadIdx.x == 0) *args.tp_counter = 0u;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool I8>
static int launch_gemm(const void* A, const void* B, const GemmArgs& args, int lda, int ldb,
                       cudaStream_t stream, int max_ctas, int b_rows_override = 0, int force_grid = 0) {
  using Cfg = GemmCfg<BN>;
  constexpr int ES = I8 ? 1 : 2;
  constexpr int BK = I8 ? 128 : 64;
  const CUtensorMapDataType dt = I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmA, tmB;
  int rc;
  if (!args.a_mn)
    rc = make_tmap_2d(&tmA, dt, ES, A, args.K, args.M, (uint64_t)lda * ES, BK, BM);
  else
    rc = make_tmap_2d(&tmA, dt, ES, A, args.M, args.K, (uint64_t)lda * ES, 64, BK);
  if (rc) return rc;
  // outer extent of B's map: N rows (K-major) or K rows (MN-major); stacked experts override it
  const uint64_t b_outer = b_rows_override > 0 ? (uint64_t)b_rows_override
                                               : (uint64_t)(args.b_mn ? args.K : args.N);
  if (!args.b_mn)
    rc = make_tmap_2d(&tmB, dt, ES, B, args.K, b_outer, (uint64_t)ldb * ES, BK, BN);
  else
    rc = make_tmap_2d(&tmB, dt, ES, B, args.N, b_outer, (uint64_t)ldb * ES, 64, BK);
  if (rc) return rc;

  // Output map for the staged epilogue: [rows][N] with 128-byte-wide boxes.  Needs a 16-byte
  // aligned base and pitch; k-grouped outputs additionally need whole tiles per group.
  CUtensorMap tmC;
  GemmArgs largs = args;
  {
    const bool f32out = args.out_mode == 1 || args.out_mode == 2;
    const int ces = f32out ? 4 : 2;
    const bool aligned = (reinterpret_cast<uintptr_t>(args.C) & 15) == 0 &&
                         ((uint64_t)args.ldc * ces) % 16 == 0;
    const bool group_ok = args.group_mode != 2 || (args.M % BM == 0 &&
                          args.c_group_stride == (long)args.M * args.ldc);
    largs.tma_store = 0;
    if (args.tp_mode == 2) {
      largs.tma_store = 1;
      tmC = tmA;
    } else if (aligned && group_ok) {
      const uint64_t rows = args.group_mode == 2 ? (uint64_t)args.M * args.num_groups : (uint64_t)args.M;
      int rc2 = make_tmap_2d(&tmC, f32out ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                             ces, args.C, args.N, rows, (uint64_t)args.ldc * ces, f32out ? 32 : 64, BM);
      if (rc2 == 0) largs.tma_store = 1;
    }
    if (args.sc_pair) largs.tma_store = 0;  // rows scatter to per-row destinations: direct stores
    if (!largs.tma_store) tmC = tmA;  // unused, but the parameter must be a valid object
    // K slices add into C concurrently: only the TMA reduce-add epilogue does that atomically
    if (!largs.tma_store || args.tp_mode || args.out_mode != 2) largs.split_k = 1;
  }
  static PerDeviceOnce smem_once;
  {
    cudaError_t e = ensure_dyn_smem(smem_once, gemm_kernel<BN, I8>, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  const long tiles = (long)((args.M + BM - 1) / BM) * ((args.N + BN - 1) / BN) *
                     (args.group_mode == 2 ? args.num_groups : (largs.split_k > 1 ? largs.split_k : 1));
  int grid = tiles < sm_count() ? (int)tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (force_grid > 0) grid = force_grid;
  gemm_kernel<BN, I8><<<grid, 256, Cfg::SMEM, stream>>>(tmA, tmB, tmC, largs);
  return (int)cudaGetLastError();
}

}  // namespace bb

#ifdef BB_TIMELINE
static long long* g_gemm_timeline = nullptr;
// Profiling aid: when set, CTA 0 of the next bf16 GEMMs writes per-tile clock64 stamps
// ([0] tile start, [1] first TMA wait, [2] cycles waiting on TMA, [3] MMAs issued, [4] epilogue
// waits, [5] accumulator ready, [6] accumulator released) for its first 16 tiles.
BB_API void bb_gemm_set_timeline(long long* buf) { g_gemm_timeline = buf; }
#else
static long long* const g_gemm_timeline = nullptr;
#endif

// CTA-pair kernel (gemm_2cta.cu)
BB_API int bb_gemm_i8_pair(const void* A, const void* B, void* C, const float* scale_m, const float* scale_n,
                           int M, int N, int K, int lda, int ldb, int ldc, int max_ctas, void* stream);
// BB_GEMM_PAIR=0 keeps every GEMM on the single-CTA kernel
static int pair_enabled() {
  static const int mode = [] {
    const char* e = getenv("BB_GEMM_PAIR");
    return e ? atoi(e) : 1;
  }();
  return mode;
}
BB_API int bb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                             int ldb, int ldc, int a_mn, int b_mn, int out_mode, float alpha,
                             int split_k, int max_ctas, void* stream);

// C ABI ------------------------------------------------------------------------------------------
// bf16 GEMM.  a_mn/b_mn: 0 = operand stored [rows][K] (K contiguous), 1 = stored [K][rows].
// lda/ldb/ldc in elements.  out_mode: 0 bf16, 1 fp32, 2 fp32 accumulate, 3 bf16 gelu.
// bn: tile width (256/128/64/32) or 0 = choose.  max_ctas: 0 = all SMs (leave SMs to a
// concurrent communication kernel by passing fewer).
BB_API int bb_gemm_bf16(const void* A, const void* B, void* C, const float* bias, int M, int N,
                        int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode,
                        float alpha, int bn, int max_ctas, void* stream) {
  using namespace bb;
  if (M <= 0 || N <= 0 || K <= 0) return BB_EARG;
  GemmArgs a{};
  a.C = C;
  a.bias = bias;
  a.alpha = alpha;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.a_mn = a_mn;
  a.b_mn = b_mn;
  a.out_mode = out_mode;
  a.err = device_error_word();
  a.timeline = g_gemm_timeline;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool auto_bn = bn == 0;
  if (bn == 0) {
    const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    const long tiles128 = (long)((M + 127) / 128) * ((N + 127) / 128);
    const int sms = sm_count();
    bn = (tiles256 >= sms) ? 256 : (tiles128 >= sms / 2 ? 128 : 64);
    if (N <= 64) bn = 64;
    if (out_mode == 2 && K >= 4096) bn = 256 <= N ? 256 : (N >= 128 ? 128 : 64);  // split-K fills the SMs instead
  }
  if (out_mode == 2 && K >= 4096 && max_ctas == 0) {
    // Accumulating GEMMs (weight gradients: small M x N, long K) rarely give a whole number of
    // waves.  Cut K into the slice count (<= 8, >= 16 k-blocks each) with the best wave efficiency;
    // every slice adds into C, which this mode does anyway.
    const long tiles = (long)((M + 127) / 128) * ((N + bn - 1) / bn);
    const int sms = sm_count(), nkb = (K + 63) / 64;
    double best = 0.0;
    int pick = 1;
    for (int sk = 1; sk <= 8 && nkb / sk >= 16; ++sk) {
      const long t = tiles * sk;
      const double eff = (double)t / (double)(((t + sms - 1) / sms) * sms) - 0.01 * (sk - 1);
      if (eff > best + 1e-9) {
        best = eff;
        pick = sk;
      }
    }
    a.split_k = pick;
  }
  // Large plain GEMMs go to the CTA-pair kernel (256 x 256 tiles over two SMs, gemm_2cta.cu): it
  // halves the B-operand bytes each SM pulls from L2, which is what bounds this kernel at bn 256.
  const int pair_mode = pair_enabled();
  if (pair_mode && auto_bn && bn == 256 && bias == nullptr && out_mode != 3 && M >= 256 && N >= 256 &&
      a.timeline == nullptr) {
    const int rc = bb_gemm_bf16_pair(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, alpha,
                                     a.split_k, max_ctas, stream);
    if (rc != BB_ESIZE) return rc;
  }
  switch (bn) {
    case 256: return launch_gemm<256, false>(A, B, a, lda, ldb, s, max_ctas);
    case 128: return launch_gemm<128, false>(A, B, a, lda, ldb, s, max_ctas);
    case 64: return launch_gemm<64, false>(A, B, a, lda, ldb, s, max_ctas);
    default: return BB_EARG;
  }
}

// W8A8: C[M,N] bf16 = (A_i8[M,K] · B_i8[N,K]^T) * scale_m[M] * scale_n[N]; both operands K-major.
BB_API int bb_gemm_i8(const void* A, const void* B, void* C, const float* scale_m,
                      const float* scale_n, int M, int N, int K, int lda, int ldb, int ldc, int bn,
                      int max_ctas, void* stream) {
  using namespace bb;
  if (M <= 0 || N <= 0 || K <= 0) return BB_EARG;
  GemmArgs a{};
  a.C = C;
  a.scale_m = scale_m;
  a.scale_n = scale_n;
  a.alpha = 1.f;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.out_mode = 0;
  a.err = device_error_word();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool auto_bn = bn == 0;
  if (bn == 0) {
    const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    const long tiles128 = (long)((M + 127) / 128) * ((N + 127) / 128);
    const int sms = sm_count();
    bn = (tiles256 >= sms) ? 256 : (tiles128 >= sms / 2 ? 128 : 64);
  }
  // prefill-sized problems go to the CTA-pair kernel (each SM stages half of B: the single-CTA
  // int8 kernel is bound by its L2 -> shared-memory fill at a third of the tensor rate)
  if (pair_enabled() && auto_bn && bn == 256 && M >= 256 && N >= 256 && K >= 256) {
    const int rc = bb_gemm_i8_pair(A, B, C, scale_m, scale_n, M, N, K, lda, ldb, ldc, max_ctas, stream);
    if (rc != BB_ESIZE) return rc;
  }
  switch (bn) {
    case 256: return launch_gemm<256, true>(A, B, a, lda, ldb, s, max_ctas);
    case 128: return launch_gemm<128, true>(A, B, a, lda, ldb, s, max_ctas);
    case 64: return launch_gemm<64, true>(A, B, a, lda, ldb, s, max_ctas);
    default: return BB_EARG;
  }
}

// Grouped bf16 GEMM for mixture-of-experts layers (one launch covers every expert).
//  mode 1: C[M,N] = A[M,K] . B_g^T per 128-row tile, g = tile_group[tile] (-1 skips the tile).
//          b_mn = 0: B is [G*b_group_rows, K] (expert g's [N,K] matrix at row g*b_group_rows);
//          b_mn = 1: B is [G*b_group_rows, N] (expert g's [K,N] matrix at row g*b_group_rows).
//  mode 2: for g < num_groups: C_g[M,N] (op)= A[rows_g, M]^T . B[rows_g, N] with
//          rows_g = [group_offsets[g], group_offsets[g+1]); C_g = C + g*c_group_stride.
//          (a_mn = b_mn = 1 implied.)  K = total rows of A/B.
BB_API int bb_gemm_bf16_grouped(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                                int ldb, int ldc, int b_mn, int out_mode, int group_mode,
                                const int* tile_group, int b_group_rows, int b_total_rows,
                                const int* group_offsets, int num_groups, long c_group_stride,
                                int bn, void* stream) {
  using namespace bb;
  if (M <= 0 || N <= 0 || K <= 0) return BB_EARG;
  if (group_mode != 1 && group_mode != 2) return BB_EARG;
  GemmArgs a{};
  a.C = C;
  a.alpha = 1.f;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.a_mn = group_mode == 2 ? 1 : 0;
  a.b_mn = group_mode == 2 ? 1 : b_mn;
  a.out_mode = out_mode;
  a.group_mode = group_mode;
  a.tile_group = tile_group;
  a.b_group_rows = b_group_rows;
  a.group_offsets = group_offsets;
  a.num_groups = num_groups;
  a.c_group_stride = c_group_stride;
  a.err = device_error_word();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 0) bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
  // the B tensor map must span every expert: describe it with its true row count
  GemmArgs amap = a;
  (void)amap;
  const void* Bp = B;
  switch (bn) {
    case 256: return launch_gemm<256, false>(A, Bp, a, lda, ldb, s, 0, b_total_rows);
    case 128: return launch_gemm<128, false>(A, Bp, a, lda, ldb, s, 0, b_total_rows);
    case 64: return launch_gemm<64, false>(A, Bp, a, lda, ldb, s, 0, b_total_rows);
    default: return BB_EARG;
  }
}

// Row-grouped GEMM whose epilogue is the expert-parallel combine's transfer: output row r (an
// expert-sorted position) is stored into slot pair_of_pos[r] % pairs_per_rank of rank
// pair_of_pos[r] / pairs_per_rank's [pairs_per_rank, ldc] bf16 slot buffer (dst_ptrs[rank]; the
// local rank's own pointer for a single GPU); rows with pair_of_pos < 0 are padding and dropped.
// The caller orders the launch against the slot buffers' previous readers and follows it with a
// symmetric barrier before any rank sums its slots.
BB_API int bb_gemm_bf16_grouped_scatter(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                                        int ldc, int b_mn, const int* tile_group, int b_group_rows,
                                        int b_total_rows, const int* pair_of_pos, const uint64_t* dst_ptrs,
                                        int world, int pairs_per_rank, void* stream) {
  using namespace bb;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > MAX_RANKS || pairs_per_rank <= 0 || !pair_of_pos)
    return BB_EARG;
  GemmArgs a{};
  a.C = reinterpret_cast<void*>(dst_ptrs[0]);
  a.alpha = 1.f;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.b_mn = b_mn;
  a.out_mode = 0;
  a.group_mode = 1;
  a.tile_group = tile_group;
  a.b_group_rows = b_group_rows;
  a.err = device_error_word();
  a.sc_pair = pair_of_pos;
  for (int r = 0; r < world; ++r) a.sc_dst.p[r] = reinterpret_cast<void*>(dst_ptrs[r]);
  a.sc_pairs_per_rank = pairs_per_rank;
  const int bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (bn) {
    case 256: return launch_gemm<256, false>(A, B, a, lda, ldb, s, 0, b_total_rows);
    case 128: return launch_gemm<128, false>(A, B, a, lda, ldb, s, 0, b_total_rows);
    default: return launch_gemm<64, false>(A, B, a, lda, ldb, s, 0, b_total_rows);
  }
}

// Expert-parallel dispatch fused into the row-grouped GEMM (tp_mode 3 of the kernel): `xp` [M, K] is
// the local expert-sorted operand buffer that the kernel's mover CTAs fill from `src_ptrs[r]` (every
// rank's [n_per_rank, K] activations, symmetric memory) by `pair_of_pos` (int32 [M], -1 = padding),
// scaled by `w[pair]` when given; the GEMM side consumes each 128-row tile as soon as it is in place.
// `row_flags`: persistent int32 [>= M/128], compared against the increasing `epoch`.  The caller
// orders "every rank's activations are written" before this launch (a symmetric barrier).
BB_API int bb_gemm_bf16_grouped_ep(void* xp, const void* B, void* C, int M, int N, int K, int ldb, int ldc,
                                   int b_mn, const int* tile_group, int b_group_rows, int b_total_rows,
                                   const uint64_t* src_ptrs, int world, int n_per_rank,
                                   const int* pair_of_pos, const float* w, int k, int* row_flags,
                                   unsigned int epoch, int copy_ctas, double wait_seconds, void* stream) {
  using namespace bb;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > MAX_RANKS || M % BM || K % 8) return BB_EARG;
  GemmArgs a{};
  a.C = C;
  a.alpha = 1.f;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.b_mn = b_mn;
  a.out_mode = 0;
  a.group_mode = 1;
  a.tile_group = tile_group;
  a.b_group_rows = b_group_rows;
  a.err = device_error_word();
  a.tp_mode = 3;
  a.tp_world = world;
  for (int r = 0; r < world; ++r) a.tp_src.p[r] = reinterpret_cast<void*>(src_ptrs[r]);
  a.tp_full = xp;
  a.tp_row_flags = row_flags;
  a.tp_epoch = epoch;
  a.tp_wait_limit = (long long)(wait_seconds * 1.9e9);
  a.tp_copy_ctas = copy_ctas > 0 ? copy_ctas : 24;
  if (a.tp_copy_ctas > sm_count() / 2) a.tp_copy_ctas = sm_count() / 2;
  a.ep_pair_of_pos = pair_of_pos;
  a.ep_w = w;
  a.ep_n_per_rank = n_per_rank;
  a.ep_k = k;
  const int bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int force_grid = sm_count();  // movers and consumers must be co-resident
  switch (bn) {
    case 256: return launch_gemm<256, false>(xp, B, a, K, ldb, s, 0, b_total_rows, force_grid);
    case 128: return launch_gemm<128, false>(xp, B, a, K, ldb, s, 0, b_total_rows, force_grid);
    default: return launch_gemm<64, false>(xp, B, a, K, ldb, s, 0, b_total_rows, force_grid);
  }
}

// Tensor-parallel fused GEMMs (bf16, x.W^T layout: A [M,K] K-major, B [N,K] K-major).
//  mode 1 (all-gather -> GEMM): `a_full` is this rank's [M, K] landing buffer; `a_src_ptrs[r]`
//    is rank r's [rows_per_rank, K] shard; `row_flags` int32[M/128] local (persistent, compared
//    against the monotonically increasing `epoch`); C [M, N] local.
//  mode 2 (GEMM -> reduce-scatter): A [M, K] local; `cmaps` = device array of `world` tensor maps
//    made by bb_tp_make_cmaps over every rank's receive buffer [world*rows_per_rank, N];
//    `counter` = one zeroed uint32 of local device memory.
//  `sig_ptrs[r]`: rank r's signal words (uint64[2*world], zeroed once).  M = world*rows_per_rank,
//  rows_per_rank % 128 == 0.
BB_API int bb_gemm_bf16_tp(int mode, const void* A, const void* B, void* C, int M, int N, int K,
                           int lda, int ldb, int ldc, int rank, int world, int rows_per_rank,
                           const uint64_t* a_src_ptrs, int* row_flags, int copy_ctas,
                           const uint64_t* sig_ptrs, unsigned int epoch, const void* cmaps,
                           unsigned int* counter, double wait_seconds, void* stream) {
  using namespace bb;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > MAX_RANKS) return BB_EARG;
  if (rows_per_rank % BM || (long)rows_per_rank * world != M) return BB_EARG;
  if (mode != 1 && mode != 2) return BB_EARG;
  GemmArgs a{};
  a.C = C;
  a.alpha = 1.f;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.out_mode = 0;
  a.err = device_error_word();
  a.tp_mode = mode;
  a.tp_rank = rank;
  a.tp_world = world;
  a.rows_per_rank = rows_per_rank;
  a.tp_epoch = epoch;
  a.tp_wait_limit = (long long)(wait_seconds * 1.9e9);
  for (int r = 0; r < world; ++r) a.tp_sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  if (mode == 1) {
    if (lda != K) return BB_EARG;  // the landing buffer is dense
    for (int r = 0; r < world; ++r) a.tp_src.p[r] = reinterpret_cast<void*>(a_src_ptrs[r]);
    a.tp_full = const_cast<void*>(A);
    a.tp_row_flags = row_flags;
    // copy-engine movers: four per rank (16384 rows x 4096: 2 ranks 4 -> 918 us, 8 -> 675, 12 -> 686;
    // 4 ranks 8 -> 511 us, 16 -> 373, 24 -> 384), at most 32
    a.tp_copy_ctas = copy_ctas > 0 ? copy_ctas : (4 * world < 32 ? 4 * world : 32);
    if (a.tp_copy_ctas > sm_count() / 2) a.tp_copy_ctas = sm_count() / 2;
  } else {
    a.tp_cmaps = static_cast<const CUtensorMap*>(cmaps);
    a.tp_counter = counter;
  }
  const int bn = N >= 256 ? 256 : (N >= 128 ? 128 : 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the persistent grid must be fully co-resident (one CTA per SM): movers and consumers wait
  // on each other only in the mover -> consumer direction, and movers have the lowest block ids
  const int force_grid = sm_count();
  switch (bn) {
    case 256: return launch_gemm<256, false>(A, B, a, lda, ldb, s, 0, 0, force_grid);
    case 128: return launch_gemm<128, false>(A, B, a, lda, ldb, s, 0, 0, force_grid);
    default: return launch_gemm<64, false>(A, B, a, lda, ldb, s, 0, 0, force_grid);
  }
}

// Encode, for every destination rank, a bf16 output map over its receive buffer
// [world*rows_per_rank rows][N] (pitch ldc elements), 128x64 boxes, and copy the `world` maps to
// `dst_dev` (device memory, 64-byte aligned, world*128 bytes).
BB_API int bb_tp_make_cmaps(void* dst_dev, const uint64_t* recv_ptrs, int world, int rows_total,
                            int N, int ldc) {
  using namespace bb;
  if (world < 1 || world > MAX_RANKS) return BB_EARG;
  CUtensorMap maps[MAX_RANKS];
  for (int r = 0; r < world; ++r) {
    int rc = make_tmap_2d(&maps[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          reinterpret_cast<void*>(recv_ptrs[r]), (uint64_t)N, (uint64_t)rows_total,
                          (uint64_t)ldc * 2, 64, BM);
    if (rc) return rc;
  }
  return (int)cudaMemcpy(dst_dev, maps, sizeof(CUtensorMap) * world, cudaMemcpyHostToDevice);
}
