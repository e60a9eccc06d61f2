// Mixture-of-experts row movement (the part of the layer that is not a GEMM):
//   moe_plan      expert counts -> 128-row-padded offsets, per-tile expert table, zeroed fill
//   moe_positions deterministic position of every (token, slot) pair inside its expert's segment
//                 (one block per expert scanning the routing table in token order, so the order of
//                 rows — and therefore the summation order of the weight gradients — is fixed)
//   moe_gather    xp[pos] = x[token]            (optionally scaled by the routing weight: backward)
//   moe_combine   y[token] = sum_s w[token,s] * yp[pos(token,s)]   (gather, no atomics)
//   moe_rowdot    dw[token,s] = <dy[token], yp[pos(token,s)]>       (routing-weight gradient)
// Source rows may live in a peer GPU's memory (expert parallelism): gather/combine then take a
// table of per-rank base pointers and read them with plain peer loads.
// Reference: crates/kernels/wgsl/{router_topk_compact,row_scatter,moe_scatter_scaled_add,
// scale_add,scale_add_dgate}.wgsl, crates/model/src/moe.rs:485-605 (compact path).
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {

static constexpr int MOE_MAX_RANKS = 16;
struct MoePeers {
  const void* p[MOE_MAX_RANKS];
};

// counts[E] -> offsets[E+1] (each segment padded to 128 rows), tile_group[max_tiles] (-1 beyond
// the used tiles), fill[E] = 0.  One block.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                int* __restrict__ tile_group, int max_tiles) {
  __shared__ int s_off[1025];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_off[e];
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E - 1;  // last e with s_off[e] <= row
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid - 1;
      }
      g = lo;
    }
    tile_group[t] = g;
  }
}

// One block per local expert e: walk idx[n_pairs] (pair p = token*k + slot) in order; the j-th pair
// routed to (e_first + e) gets position offsets[e] + j.  pos_of_pair[p] = position (or -1 when the
// pair's expert is not local); pair_of_pos[position] = p (-1 for padding rows, pre-filled).
__global__ void moe_positions_kernel(const int* __restrict__ idx, long n_pairs, int e_first,
                                     const int* __restrict__ offsets, int* __restrict__ pos_of_pair,
                                     int* __restrict__ pair_of_pos) {
  __shared__ int warp_tot[8];
  __shared__ int base;
  const int e = blockIdx.x;
  const int want = e_first + e;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base = offsets[e];
  __syncthreads();
  for (long p0 = 0; p0 < n_pairs; p0 += blockDim.x) {
    const long p = p0 + threadIdx.x;
    const bool hit = p < n_pairs && idx[p] == want;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(m & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int woff = 0, tot = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      if (w < warp) woff += warp_tot[w];
      tot += warp_tot[w];
    }
    if (hit) {
      const int pos = base + woff + before;
      pos_of_pair[p] = pos;
      pair_of_pos[pos] = (int)p;
    }
    __syncthreads();
    if (threadIdx.x == 0) base += tot;
    __syncthreads();
  }
}

// xp[pos, :] = src[token(pos), :] * (w ? w[pair] : 1); padding rows (pair < 0) are zero-filled.
// `src` rows are addressed as (rank = token / n_per_rank, local = token % n_per_rank).
__global__ void moe_gather_kernel(MoePeers src, int n_per_rank, const int* __restrict__ pair_of_pos,
                                  const float* __restrict__ w, int k, __nv_bfloat16* __restrict__ xp,
                                  const int* __restrict__ offsets, int E, int dv, int world BB_ERR_PARAM) {
  const int rows = offsets[E];
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int pos = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; pos < rows; pos += warps) {
    const int pair = pair_of_pos[pos];
    bf16x8* dst = reinterpret_cast<bf16x8*>(xp) + (size_t)pos * dv;
    if (pair < 0) {
      bf16x8 z;
#pragma unroll
      for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int c = lane; c < dv; c += 32) dst[c] = z;
      continue;
    }
    const int token = pair / k;
    // the pair id comes from the routing tables: beyond the tokens of the ranks that were passed it
    // would select a null base pointer (bounds-checking builds record it and leave the row alone)
    if (!BB_INDEX_OK(token, (long long)n_per_rank * world)) continue;
    const int rank = token / n_per_rank, local = token - rank * n_per_rank;
    const bf16x8* s = reinterpret_cast<const bf16x8*>(src.p[rank]) + (size_t)local * dv;
    if (w) {
      const float g = w[pair];
      for (int c = lane; c < dv; c += 32) {
        float f[8];
        unpack8(s[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= g;
        dst[c] = pack8(f);
      }
    } else {
      for (int c = lane; c < dv; c += 32) dst[c] = s[c];
    }
  }
}

// y[token, :] = sum_s (w ? w[token,s] : 1) * yp_rank(s)[pos, :].  pos_of_pair gives, per pair,
// the row inside the buffer of the rank that owns the pair's expert (rank = expert / e_per_rank).
__global__ void moe_combine_kernel(MoePeers yp, const int* __restrict__ idx, MoePeers pos_tabs,
                                   long pair_offset, const float* __restrict__ w, int k,
                                   int e_per_rank, __nv_bfloat16* __restrict__ y, int n_tok, int dv) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < n_tok; t += warps) {
    for (int c = lane; c < dv; c += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int s = 0; s < k; ++s) {
        const int pair = t * k + s;
        const int rank = idx[pair] / e_per_rank;
        // the row's position is known to the rank that owns the expert: read it from that rank's table
        const int pos = reinterpret_cast<const int*>(pos_tabs.p[rank])[pair_offset + pair];
        if (pos < 0) continue;
        float f[8];
        unpack8(reinterpret_cast<const bf16x8*>(yp.p[rank])[(size_t)pos * dv + c], f);
        const float g = w ? w[pair] : 1.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += g * f[j];
      }
      reinterpret_cast<bf16x8*>(y)[(size_t)t * dv + c] = pack8(acc);
    }
  }
}

// dw[pair] = <dy[token, :], yp[pos(pair), :]>
__global__ void moe_rowdot_kernel(const __nv_bfloat16* __restrict__ dy, MoePeers yp,
                                  const int* __restrict__ idx, MoePeers pos_tabs, long pair_offset,
                                  int k, int e_per_rank, float* __restrict__ dw, long n_pairs,
                                  int dv) {
  const long warps = ((long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long pair = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; pair < n_pairs;
       pair += warps) {
    const int rank = idx[pair] / e_per_rank;
    const int pos = reinterpret_cast<const int*>(pos_tabs.p[rank])[pair_offset + pair];
    float acc = 0.f;
    if (pos >= 0) {
      const long t = pair / k;
      const bf16x8* a = reinterpret_cast<const bf16x8*>(dy) + (size_t)t * dv;
      const bf16x8* b = reinterpret_cast<const bf16x8*>(yp.p[rank]) + (size_t)pos * dv;
      for (int c = lane; c < dv; c += 32) {
        float f[8], g[8];
        unpack8(a[c], f);
        unpack8(b[c], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += f[j] * g[j];
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[pair] = acc;
  }
}

}  // namespace bb

using namespace bb;

BB_API int bb_moe_plan(const int* counts, int E, int* offsets, int* tile_group, int max_tiles,
                       void* stream) {
  if (E < 1 || E > 1024) return BB_EARG;
  moe_plan_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(counts, E, offsets, tile_group, max_tiles);
  return (int)cudaGetLastError();
}

BB_API int bb_moe_positions(const int* idx, long n_pairs, int e_first, int e_local,
                            const int* offsets, int* pos_of_pair, int* pair_of_pos, void* stream) {
  if (e_local < 1) return BB_EARG;
  moe_positions_kernel<<<e_local, 256, 0, (cudaStream_t)stream>>>(idx, n_pairs, e_first, offsets,
                                                                  pos_of_pair, pair_of_pos);
  return (int)cudaGetLastError();
}

static int fill_peers(MoePeers& p, const uint64_t* ptrs, int world) {
  if (world < 1 || world > MOE_MAX_RANKS) return BB_EARG;
  for (int r = 0; r < world; ++r) p.p[r] = reinterpret_cast<const void*>(ptrs[r]);
  return BB_OK;
}

// src_ptrs: `world` base pointers of the [n_per_rank, d] bf16 token buffers (world = 1: local).
BB_API int bb_moe_gather(const uint64_t* src_ptrs, int world, int n_per_rank,
                         const int* pair_of_pos, const float* w, int k, void* xp,
                         const int* offsets, int E, int d, int max_rows, void* stream) {
  MoePeers p{};
  if (int rc = fill_peers(p, src_ptrs, world)) return rc;
  if (d % 8) return BB_EARG;
  int blocks = (max_rows + 7) / 8;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  moe_gather_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, n_per_rank, pair_of_pos, w, k,
                                                             (__nv_bfloat16*)xp, offsets, E, d / 8,
                                                             world BB_ERR_ARG);
  return (int)cudaGetLastError();
}

// pos_ptrs[r]: rank r's pos_of_pair table over ALL ranks' pairs; pair_offset = first pair of this
// rank's tokens in that global numbering (0 on a single rank).
BB_API int bb_moe_combine(const uint64_t* yp_ptrs, const uint64_t* pos_ptrs, int world,
                          const int* idx, long pair_offset, const float* w, int k, int e_per_rank,
                          void* y, int n_tok, int d, void* stream) {
  MoePeers p{}, pt{};
  if (int rc = fill_peers(p, yp_ptrs, world)) return rc;
  if (int rc = fill_peers(pt, pos_ptrs, world)) return rc;
  if (d % 8) return BB_EARG;
  int blocks = (n_tok + 7) / 8;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  moe_combine_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, idx, pt, pair_offset, w, k,
                                                              e_per_rank, (__nv_bfloat16*)y, n_tok,
                                                              d / 8);
  return (int)cudaGetLastError();
}

BB_API int bb_moe_rowdot(const void* dy, const uint64_t* yp_ptrs, const uint64_t* pos_ptrs,
                         int world, const int* idx, long pair_offset, int k, int e_per_rank,
                         float* dw, long n_pairs, int d, void* stream) {
  MoePeers p{}, pt{};
  if (int rc = fill_peers(p, yp_ptrs, world)) return rc;
  if (int rc = fill_peers(pt, pos_ptrs, world)) return rc;
  if (d % 8) return BB_EARG;
  long blocks = (n_pairs + 7) / 8;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  moe_rowdot_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, p, idx, pt, pair_offset, k, e_per_rank, dw, n_pairs, d / 8);
  return (int)cudaGetLastError();
}
