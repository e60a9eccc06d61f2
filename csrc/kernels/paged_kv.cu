// Paged KV cache kernels.  Cache layout (K and V separately): [num_blocks][n_kv_heads][block_size]
// [head_dim] bf16, so one (block, head) chunk is contiguous (16 tokens x 128 x 2 B = 4 KB).
//   kv_append    scatter the new tokens' K/V rows into their slots (slot = block*bs + offset)
//   kv_gather    copy a sequence's first S tokens out of its pages into a contiguous [S, hk*hd]
//                buffer (chunked prefill runs the tcgen05 flash kernel over it)
//   paged_decode split-KV decode attention: grid (sequence, kv head, split); one warp per
//                (CTA, 32-key group): lane-per-key dot products against the GQA group's query
//                vectors, online softmax, lane-per-column P.V; partial (m, l, o) merged by
//                paged_decode_merge.  Memory-bound by design: K and V are read exactly once.
// Reference contracts: crates/kernels/wgsl/{paged_kv_append_batched,paged_decode_scores_batched,
// decode_softmax_batched,paged_decode_apply_batched}.wgsl, crates/qwen3/src/serve.rs:1262-1288.
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {

// k, v: [n, ld] rows (head h at column h*hd); slots: int32[n] (= block*bs + offset, <0 skips).
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, int ldk,
                                 const __nv_bfloat16* __restrict__ v, int ldv,
                                 const int* __restrict__ slots, __nv_bfloat16* __restrict__ kc,
                                 __nv_bfloat16* __restrict__ vc, int n, int hk, int hd, int bs) {
  const int hv = hd >> 3;  // 16-byte vectors per head row
  const long total = (long)n * hk * hv;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % hv);
    const int h = (int)((i / hv) % hk);
    const int t = (int)(i / ((long)hv * hk));
    const int slot = slots[t];
    if (slot < 0) continue;
    const int blk = slot / bs, off = slot - blk * bs;
    const size_t dst = (((size_t)blk * hk + h) * bs + off) * hd + c * 8;
    *reinterpret_cast<bf16x8*>(kc + dst) =
        *reinterpret_cast<const bf16x8*>(k + (size_t)t * ldk + h * hd + c * 8);
    *reinterpret_cast<bf16x8*>(vc + dst) =
        *reinterpret_cast<const bf16x8*>(v + (size_t)t * ldv + h * hd + c * 8);
  }
}

// out_k/out_v: [S, hk*hd]; block_table: int32[max_blocks] of one sequence.
__global__ void kv_gather_kernel(const __nv_bfloat16* __restrict__ kc,
                                 const __nv_bfloat16* __restrict__ vc,
                                 const int* __restrict__ block_table, __nv_bfloat16* __restrict__ ok,
                                 __nv_bfloat16* __restrict__ ov, int S, int hk, int hd, int bs) {
  const int hv = hd >> 3;
  const long total = (long)S * hk * hv;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % hv);
    const int h = (int)((i / hv) % hk);
    const int t = (int)(i / ((long)hv * hk));
    const int blk = block_table[t / bs], off = t % bs;
    const size_t src = (((size_t)blk * hk + h) * bs + off) * hd + c * 8;
    const size_t dst = (size_t)t * hk * hd + h * hd + c * 8;
    *reinterpret_cast<bf16x8*>(ok + dst) = *reinterpret_cast<const bf16x8*>(kc + src);
    *reinterpret_cast<bf16x8*>(ov + dst) = *reinterpret_cast<const bf16x8*>(vc + src);
  }
}

// One CTA (4 warps) per (sequence b, kv head, split).  G = query heads per kv head (<= 8).
// q: [B, hq*hd]; block_tables: int32 [B, max_blocks]; seqlens: int32[B] (keys visible to the query).
// part_o: fp32 [B, hq, splits, hd], part_ml: fp32 [B, hq, splits, 2] (running max in log2 domain, sum).
//
// Work layout: the head dimension is split over 8 lanes (HD/8 contiguous dims each), so a warp holds
// four 8-lane groups and each group owns one key per step; the CTA's 4 warps x 4 groups take the 16
// keys of one KV block per step (one block-table lookup per warp and step).  The query slice and the
// output accumulators of all G heads stay in registers; a key's dot products are finished by a
// 3-step butterfly inside its group, which leaves the score in all 8 lanes, so P.V needs no further
// exchange.  Every group keeps its own running (max, sum, output) and the 16 partial states are
// merged once at the end.  An earlier form (one lane per key, query read from shared memory for
// every multiply) spent ~300 us per layer at batch 256 and was the largest item of a decode step.
template <int HD, int G>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                    const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ seqlens, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int hq, int hk, int bs, int splits,
                    float scale_log2) {
  constexpr int DPL = HD / 8;   // dims per lane: 16 (hd 128) or 8 (hd 64)
  constexpr int NV = DPL / 8;   // 16-byte vectors per lane per row
  const int b = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, sub = lane & 7;
  const int S = seqlens[b];
  const int per_split = ((S + splits - 1) / splits + 31) / 32 * 32;
  const int k_begin = sp * per_split;
  const int k_end = min(S, k_begin + per_split);
  __shared__ float s_o[4][G][HD];
  __shared__ float s_m[4][G], s_l[4][G];

  float qr[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const bf16x8* qp = reinterpret_cast<const bf16x8*>(q + (size_t)b * ldq + (kvh * G + g) * HD + sub * DPL);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float f[8];
      unpack8(qp[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) qr[g][v * 8 + j] = f[j] * scale_log2;
    }
  }
  float m[G], l[G], o[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) o[g][j] = 0.f;
  }
  const int* bt = block_tables + (size_t)b * max_blocks;
  // 16 keys per CTA step: warp w takes keys [k0 + 4w, k0 + 4w + 4), group g one of them.  The rows of
  // the NEXT step are fetched before the current ones are used, so two steps of loads are in flight.
  bf16x8 kraw[NV], vraw[NV], knext[NV], vnext[NV];
  auto fetch = [&](int k0, bf16x8 (&kk)[NV], bf16x8 (&vv)[NV]) -> bool {
    const int key = k0 + warp * 4 + grp;
    if (key >= k_end) return false;
    const int blk = bt[key / bs], off = key % bs;
    const size_t row = (((size_t)blk * hk + kvh) * bs + off) * HD + sub * DPL;
    const bf16x8* kr = reinterpret_cast<const bf16x8*>(kc + row);
    const bf16x8* vr = reinterpret_cast<const bf16x8*>(vc + row);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      kk[v] = kr[v];
      vv[v] = vr[v];
    }
    return true;
  };
  bool valid = fetch(k_begin, kraw, vraw);
  for (int k0 = k_begin; k0 < k_end; k0 += 16) {
    const bool valid_next = (k0 + 16 < k_end) ? fetch(k0 + 16, knext, vnext) : false;
    if (valid) {
      float kf[DPL], vf[DPL];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float t[8];
        unpack8(kraw[v], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) kf[v * 8 + j] = t[j];
        unpack8(vraw[v], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) vf[v * 8 + j] = t[j];
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sc = 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) sc += kf[j] * qr[g][j];
        // the 8 lanes of a group are all valid or all invalid, so they shuffle among themselves
        const unsigned int gm = 0xffu << (grp * 8);
        sc += __shfl_xor_sync(gm, sc, 1);
        sc += __shfl_xor_sync(gm, sc, 2);
        sc += __shfl_xor_sync(gm, sc, 4);
        if (sc > m[g]) {   // new running maximum: rescale what this group accumulated so far
          const float alpha = exp2f(m[g] - sc);   // exp2(-inf) = 0 on the first key
          l[g] *= alpha;
#pragma unroll
          for (int j = 0; j < DPL; ++j) o[g][j] *= alpha;
          m[g] = sc;
        }
        const float pg = exp2f(sc - m[g]);
        l[g] += pg;
#pragma unroll
        for (int j = 0; j < DPL; ++j) o[g][j] += pg * vf[j];
      }
    }
    valid = valid_next;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      kraw[v] = knext[v];
      vraw[v] = vnext[v];
    }
  }
  // merge the 4 groups of the warp (lanes sub, sub+8, sub+16, sub+24 hold the same dims)
#pragma unroll
  for (int step = 8; step <= 16; step <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[g], step);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[g], step);
      const float mm = fmaxf(m[g], m2);
      const float a1 = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mm);
      const float a2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mm);
#pragma unroll
      for (int j = 0; j < DPL; ++j) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[g][j], step);
        o[g][j] = o[g][j] * a1 + o2 * a2;
      }
      l[g] = l[g] * a1 + l2 * a2;
      m[g] = mm;
    }
  }
  // merge the 4 warps of the CTA
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (sub == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
#pragma unroll
      for (int j = 0; j < DPL; ++j) s_o[warp][g][sub * DPL + j] = o[g][j];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    const int g = i / HD, c = i % HD;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, oo = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float a = (s_m[w][g] == -INFINITY) ? 0.f : exp2f(s_m[w][g] - mm);
      ll += s_l[w][g] * a;
      oo += s_o[w][g][c] * a;
    }
    const size_t idx = ((size_t)b * hq + kvh * G + g) * splits + sp;
    part_o[idx * HD + c] = oo;
    if (c == 0) {
      part_ml[idx * 2] = mm;
      part_ml[idx * 2 + 1] = ll;
    }
  }
}

// out[b, h, :] = sum_sp o_sp * 2^(m_sp - M) / sum_sp l_sp * 2^(m_sp - M)
__global__ void paged_decode_merge_kernel(const float* __restrict__ part_o,
                                          const float* __restrict__ part_ml,
                                          __nv_bfloat16* __restrict__ out, int ldo, int hq, int hd,
                                          int splits) {
  const int b = blockIdx.x, h = blockIdx.y;
  const size_t base = ((size_t)b * hq + h) * splits;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    ll += (ms == -INFINITY) ? 0.f : part_ml[(base + s) * 2 + 1] * exp2f(ms - mm);
  }
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
  for (int c = threadIdx.x; c < hd; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) acc += part_o[(base + s) * hd + c] * exp2f(ms - mm);
    }
    out[(size_t)b * ldo + h * hd + c] = __float2bfloat16(acc * inv);
  }
}

}  // namespace bb

using namespace bb;

BB_API int bb_kv_append(const void* k, int ldk, const void* v, int ldv, const int* slots, void* kc,
                        void* vc, int n, int hk, int hd, int bs, void* stream) {
  if (n <= 0) return BB_OK;
  if (hd % 8 || ldk % 8 || ldv % 8) return BB_EARG;
  const long total = (long)n * hk * (hd / 8);
  long blocks = (total + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  kv_append_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, slots, (__nv_bfloat16*)kc,
      (__nv_bfloat16*)vc, n, hk, hd, bs);
  return (int)cudaGetLastError();
}

BB_API int bb_kv_gather(const void* kc, const void* vc, const int* block_table, void* ok, void* ov,
                        int S, int hk, int hd, int bs, void* stream) {
  if (S <= 0) return BB_OK;
  if (hd % 8) return BB_EARG;
  const long total = (long)S * hk * (hd / 8);
  long blocks = (total + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  kv_gather_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, (__nv_bfloat16*)ok,
      (__nv_bfloat16*)ov, S, hk, hd, bs);
  return (int)cudaGetLastError();
}

// part_o: fp32 [B*hq*splits*hd], part_ml: fp32 [B*hq*splits*2] scratch provided by the caller.
BB_API int bb_paged_decode(const void* q, int ldq, const void* kc, const void* vc,
                           const int* block_tables, int max_blocks, const int* seqlens, void* out,
                           int ldo, float* part_o, float* part_ml, int B, int hq, int hk, int hd,
                           int bs, int splits, float scale, void* stream) {
  if (B <= 0) return BB_OK;
  if (hq % hk || splits < 1) return BB_EARG;
  const int G = hq / hk;
  dim3 grid(B, hk, splits);
  const float sl2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
#define BB_LAUNCH_PD(HD_, G_)                                                                     \
  paged_decode_kernel<HD_, G_><<<grid, 128, 0, s>>>(                                              \
      (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,           \
      block_tables, max_blocks, seqlens, part_o, part_ml, hq, hk, bs, splits, sl2)
  if (hd == 128) {
    switch (G) {
      case 1: BB_LAUNCH_PD(128, 1); break;
      case 2: BB_LAUNCH_PD(128, 2); break;
      case 4: BB_LAUNCH_PD(128, 4); break;
      case 8: BB_LAUNCH_PD(128, 8); break;
      default: return BB_EARG;
    }
  } else if (hd == 64) {
    switch (G) {
      case 1: BB_LAUNCH_PD(64, 1); break;
      case 2: BB_LAUNCH_PD(64, 2); break;
      case 3: BB_LAUNCH_PD(64, 3); break;
      case 4: BB_LAUNCH_PD(64, 4); break;
      default: return BB_EARG;
    }
  } else {
    return BB_EARG;
  }
#undef BB_LAUNCH_PD
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  paged_decode_merge_kernel<<<dim3(B, hq), 128, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, ldo,
                                                        hq, hd, splits);
  return (int)cudaGetLastError();
}
