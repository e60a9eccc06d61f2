// Paged KV cache kernels.  Cache layout (K and V separately): [num_blocks][n_kv_heads][block_size]
// [head_dim] bf16, so one (block, head) chunk is contiguous (16 tokens x 128 x 2 B = 4 KB).
//   kv_append    scatter the new tokens' K/V rows into their slots (slot = block*bs + offset)
//   kv_gather    copy a sequence's first S tokens out of its pages into a contiguous [S, hk*hd]
//                buffer (chunked prefill runs the tcgen05 flash kernel over it)
//   paged_decode split-KV decode attention: grid (sequence, kv head, split); one warp per
//                (CTA, 32-key group): lane-per-key dot products against the GQA group's query
//                vectors, online softmax, lane-per-column P.V; partial (m, l, o) merged by
//                paged_decode_merge.  Memory-bound by design: K and V are read exactly once.
// int8 cache (kv_append_i8 / kv_gather_i8 / paged_decode with I8): the pools hold int8 rows of the
// same layout plus one fp32 scale per (block, head, slot); a row's scale is
// min(absmax(row), clip[head]) / 127 (crates/kernels/wgsl/paged_kv_append_i8_clipped_batched.wgsl).
// Decode multiplies the integer dot product by the key's scale and the probability by the value's.
// Reference contracts: crates/kernels/wgsl/{paged_kv_append_batched,paged_decode_scores_batched,
// decode_softmax_batched,paged_decode_apply_batched}.wgsl, crates/qwen3/src/serve.rs:1262-1288.
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"
#include <type_traits>

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

// One warp per (token, kv head, K|V): absmax over the row, scale = min(absmax, clip) / 127, int8 row
// and its scale written to the slot.  clip: fp32 [2][hk] (K then V) or null for no ceiling.
__global__ void kv_append_i8_kernel(const __nv_bfloat16* __restrict__ k, int ldk,
                                    const __nv_bfloat16* __restrict__ v, int ldv,
                                    const int* __restrict__ slots, int8_t* __restrict__ kc,
                                    int8_t* __restrict__ vc, float* __restrict__ ks,
                                    float* __restrict__ vs, const float* __restrict__ clip, int n,
                                    int hk, int hd, int bs) {
  const int lane = threadIdx.x & 31;
  const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long w = warp; w < (long)n * hk * 2; w += nwarps) {
    const int which = (int)(w & 1);
    const int h = (int)((w >> 1) % hk);
    const int t = (int)((w >> 1) / hk);
    const int slot = slots[t];
    if (slot < 0) continue;
    const __nv_bfloat16* src = which ? v + (size_t)t * ldv + h * hd : k + (size_t)t * ldk + h * hd;
    float x[4];  // hd <= 128: up to 4 elements per lane
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
      x[j] = c < hd ? __bfloat162float(src[c]) : 0.f;
      amax = fmaxf(amax, fabsf(x[j]));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (clip) amax = fminf(amax, clip[which * hk + h]);
    const float sc = amax / 127.f;
    const float inv = sc > 0.f ? 1.f / sc : 0.f;
    const int blk = slot / bs, off = slot - blk * bs;
    const size_t row = ((size_t)blk * hk + h) * bs + off;
    int8_t* dst = (which ? vc : kc) + row * hd;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
      if (c < hd) dst[c] = (int8_t)max(-127, min(127, __float2int_rn(x[j] * inv)));
    }
    if (lane == 0) (which ? vs : ks)[row] = sc;
  }
}

// Dequantising gather: out_k/out_v [S, hk*hd] bf16 from the int8 pools of one sequence.
__global__ void kv_gather_i8_kernel(const int8_t* __restrict__ kc, const int8_t* __restrict__ vc,
                                    const float* __restrict__ ks, const float* __restrict__ vs,
                                    const int* __restrict__ block_table,
                                    __nv_bfloat16* __restrict__ ok, __nv_bfloat16* __restrict__ ov,
                                    int S, int hk, int hd, int bs) {
  const int hv = hd >> 3;  // 8 elements (8 bytes in, 16 bytes out) per thread
  const long total = (long)S * hk * hv;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % hv);
    const int h = (int)((i / hv) % hk);
    const int t = (int)(i / ((long)hv * hk));
    const int blk = block_table[t / bs], off = t % bs;
    const size_t row = ((size_t)blk * hk + h) * bs + off;
    const size_t dst = (size_t)t * hk * hd + h * hd + c * 8;
    const float sk = ks[row], sv = vs[row];
    const char4* pk = reinterpret_cast<const char4*>(kc + row * hd + c * 8);
    const char4* pv = reinterpret_cast<const char4*>(vc + row * hd + c * 8);
    const char4 k0 = pk[0], k1 = pk[1], v0 = pv[0], v1 = pv[1];
    const float fk[8] = {k0.x * sk, k0.y * sk, k0.z * sk, k0.w * sk, k1.x * sk, k1.y * sk, k1.z * sk, k1.w * sk};
    const float fv[8] = {v0.x * sv, v0.y * sv, v0.z * sv, v0.w * sv, v1.x * sv, v1.y * sv, v1.z * sv, v1.w * sv};
    *reinterpret_cast<bf16x8*>(ok + dst) = pack8(fk);
    *reinterpret_cast<bf16x8*>(ov + dst) = pack8(fv);
  }
}

template <int N>
struct alignas(N) i8vec {
  uint32_t w[N / 4];
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)),
               "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)),
               "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One CTA (4 warps) per (sequence b, kv head, split).  G = query heads per kv head (<= 8).
// q: [B, hq*hd]; block_tables: int32 [B, max_blocks]; seqlens: int32[B] (keys visible to the query).
// part_o: fp32 [B, hq, splits, hd], part_ml: fp32 [B, hq, splits, 2] (running max in log2 domain, sum).
//
// Data movement: the CTA walks its keys 16 at a time.  The 16 K rows and 16 V rows of a step are
// copied global -> shared with cp.async (16 bytes per request, no registers held), NST steps deep,
// so each CTA keeps (NST-1) x 16 x 2 rows in flight; with three CTAs per SM that is enough
// outstanding bytes to cover HBM latency.  (Register prefetch of one step ahead left ~16 KB per SM
// in flight and reached about a third of the copy bandwidth.)
//
// Work layout: the head dimension is split over 8 lanes (HD/8 contiguous dims each), so a warp holds
// four 8-lane groups and each group owns one key per step; the CTA's 4 warps x 4 groups take the 16
// keys of a step.  The query slice and the output accumulators of all G heads stay in registers; a
// key's dot products are finished by a 3-step butterfly inside its group, which leaves the score in
// all 8 lanes, so P.V needs no further exchange.  Every group keeps its own running (max, sum,
// output) and the 16 partial states are merged once at the end.
//
// I8: kc/vc point at int8 pools and ks/vs at their per-row scales; a lane's slice of a row is DPL
// bytes, the dot product runs on the integer values and the key's scale multiplies the score, the
// value's scale multiplies the probability.
template <int HD, int G, bool I8>
__global__ void __launch_bounds__(128, 3)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                    const void* __restrict__ kc_, const void* __restrict__ vc_,
                    const float* __restrict__ ks, const float* __restrict__ vs,
                    const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ seqlens, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int hq, int hk, int bs, int splits,
                    float scale_log2, int gsplit) {
  // gsplit > 1: a kv head's query heads are divided over gsplit CTAs of G heads each (8 heads per
  // kv head would need 256 registers for q and o alone); the siblings re-read K/V through L2.
  constexpr int DPL = HD / 8;            // dims per lane: 16 (hd 128) or 8 (hd 64)
  constexpr int ES = I8 ? 1 : 2;         // bytes per stored element
  constexpr int ROWB = HD * ES;          // bytes per K or V row
  constexpr int CPR = ROWB / 16;         // 16-byte requests per row
  constexpr int NST = 4;                 // pipeline depth (steps of 16 keys)
  constexpr int STAGE = 16 * ROWB;       // bytes per stage per tensor
  constexpr int PIPE_BYTES = 2 * NST * STAGE;
  constexpr int MERGE_BYTES = 4 * G * HD * 4;
  constexpr int SMEM_BYTES = PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES;
  __shared__ __align__(16) unsigned char s_raw[SMEM_BYTES];   // pipeline stages, then the merge buffer
  __shared__ float s_sc[NST][2][16];                          // I8: row scales (K, V) per stage
  __shared__ float s_m[4][G], s_l[4][G];
  unsigned char* s_k = s_raw;
  unsigned char* s_v = s_raw + NST * STAGE;
  const unsigned char* kc = static_cast<const unsigned char*>(kc_);
  const unsigned char* vc = static_cast<const unsigned char*>(vc_);

  const int b = blockIdx.x, kvh = blockIdx.y / gsplit, sp = blockIdx.z;
  const int head0 = (kvh * gsplit + blockIdx.y % gsplit) * G;   // first query head of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, sub = lane & 7;
  const int S = seqlens[b];
  const int per_split = ((S + splits - 1) / splits + 31) / 32 * 32;
  const int k_begin = sp * per_split;
  const int k_end = min(S, k_begin + per_split);
  const int nsteps = k_end > k_begin ? (k_end - k_begin + 15) >> 4 : 0;
  const int* bt = block_tables + (size_t)b * max_blocks;

  // copy the rows of step i into its stage (rows past k_end are left as they are and never used)
  auto issue = [&](int i) {
    const int st = i % NST;
    const int k0 = k_begin + i * 16;
#pragma unroll
    for (int c = threadIdx.x; c < 16 * CPR; c += 128) {
      const int kl = c / CPR, part = c % CPR;
      const int key = k0 + kl;
      if (key < k_end) {
        const int blk = bt[key / bs], off = key % bs;
        const size_t r = ((size_t)blk * hk + kvh) * bs + off;
        cp_async16(s_k + st * STAGE + kl * ROWB + part * 16, kc + r * ROWB + part * 16);
        cp_async16(s_v + st * STAGE + kl * ROWB + part * 16, vc + r * ROWB + part * 16);
      }
    }
    if constexpr (I8) {
      if (threadIdx.x < 32) {
        const int kl = threadIdx.x & 15, which = threadIdx.x >> 4;
        const int key = k0 + kl;
        if (key < k_end) {
          const int blk = bt[key / bs], off = key % bs;
          const size_t r = ((size_t)blk * hk + kvh) * bs + off;
          cp_async4(&s_sc[st][which][kl], (which ? vs : ks) + r);
        }
      }
    }
  };
#pragma unroll
  for (int i = 0; i < NST - 1; ++i) {
    if (i < nsteps) issue(i);
    cp_async_commit();
  }

  // bf16: the query slice as floats (pre-scaled).  I8: the query slice as two int8 terms per element,
  // q ~ qs * (hi + lo / 128) with qs = absmax / 127 per head, so that a key's dot product runs on
  // dp4a over the stored bytes (no int8 -> float conversion of K at all); 14 bits relative to the
  // head's largest component keep more of q than its bf16 storage does for all but tiny components.
  float qr[I8 ? 1 : G][I8 ? 1 : DPL];
  int qhi[I8 ? G : 1][I8 ? DPL / 4 : 1], qlo[I8 ? G : 1][I8 ? DPL / 4 : 1];
  float qs[I8 ? G : 1];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const bf16x8* qp = reinterpret_cast<const bf16x8*>(q + (size_t)b * ldq + (head0 + g) * HD + sub * DPL);
    float qf[DPL];
#pragma unroll
    for (int v = 0; v < DPL / 8; ++v) {
      float f[8];
      unpack8(qp[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) qf[v * 8 + j] = f[j];
    }
    if constexpr (I8) {
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < DPL; ++j) amax = fmaxf(amax, fabsf(qf[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      const float inv = amax > 0.f ? 127.f / amax : 0.f;
      qs[g] = amax * (1.f / 127.f) * scale_log2;
#pragma unroll
      for (int v = 0; v < DPL / 4; ++v) {
        uint32_t hi = 0, lo = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float x = qf[v * 4 + j] * inv;
          const int h = __float2int_rn(x);                       // |h| <= 127
          const int r = __float2int_rn((x - (float)h) * 128.f);  // |r| <= 64
          hi |= (uint32_t)(h & 0xff) << (8 * j);
          lo |= (uint32_t)(r & 0xff) << (8 * j);
        }
        qhi[g][v] = (int)hi;
        qlo[g][v] = (int)lo;
      }
    } else {
#pragma unroll
      for (int j = 0; j < DPL; ++j) qr[g][j] = qf[j] * scale_log2;
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

  const int kl = warp * 4 + grp;   // this group's key within a step
  for (int i = 0; i < nsteps; ++i) {
    cp_async_wait<NST - 2>();      // step i has landed (for this thread's requests)
    __syncthreads();               // ... for everyone's; and everyone is done with step i-1's stage
    if (i + NST - 1 < nsteps) issue(i + NST - 1);
    cp_async_commit();
    const int st = i % NST;
    if (k_begin + i * 16 + kl < k_end) {
      float xf[DPL];
      float sc[G];
      const unsigned char* krow = s_k + st * STAGE + kl * ROWB + sub * DPL * ES;
      // the 8 lanes of a group are all valid or all invalid, so they shuffle among themselves
      const unsigned int gm = 0xffu << (grp * 8);
      if constexpr (I8) {
        const i8vec<DPL> raw = *reinterpret_cast<const i8vec<DPL>*>(krow);
        const float kscale = s_sc[st][0][kl];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          int ah = 0, al = 0;
#pragma unroll
          for (int v = 0; v < DPL / 4; ++v) {
            ah = __dp4a((int)raw.w[v], qhi[g][v], ah);
            al = __dp4a((int)raw.w[v], qlo[g][v], al);
          }
          // |ah| <= 128*127*127 and |al| <= 128*127*64 per head: 128*ah + al fits an int
          int a = ah * 128 + al;
          a += __shfl_xor_sync(gm, a, 1);
          a += __shfl_xor_sync(gm, a, 2);
          a += __shfl_xor_sync(gm, a, 4);
          sc[g] = (float)a * (qs[g] * (1.f / 128.f)) * kscale;
        }
      } else {
#pragma unroll
        for (int v = 0; v < DPL / 8; ++v) {
          float t[8];
          unpack8(reinterpret_cast<const bf16x8*>(krow)[v], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) xf[v * 8 + j] = t[j];
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float a = 0.f;
#pragma unroll
          for (int j = 0; j < DPL; ++j) a += xf[j] * qr[g][j];
          a += __shfl_xor_sync(gm, a, 1);
          a += __shfl_xor_sync(gm, a, 2);
          a += __shfl_xor_sync(gm, a, 4);
          sc[g] = a;
        }
      }
      const unsigned char* vrow = s_v + st * STAGE + kl * ROWB + sub * DPL * ES;
      if constexpr (I8) {
        const i8vec<DPL> raw = *reinterpret_cast<const i8vec<DPL>*>(vrow);
#pragma unroll
        for (int v = 0; v < DPL / 4; ++v)
#pragma unroll
          for (int j = 0; j < 4; ++j) xf[v * 4 + j] = (float)(int8_t)(raw.w[v] >> (8 * j));
      } else {
#pragma unroll
        for (int v = 0; v < DPL / 8; ++v) {
          float t[8];
          unpack8(reinterpret_cast<const bf16x8*>(vrow)[v], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) xf[v * 8 + j] = t[j];
        }
      }
      const float vscale = I8 ? s_sc[st][1][kl] : 1.f;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (sc[g] > m[g]) {   // new running maximum: rescale what this group accumulated so far
          const float alpha = exp2f(m[g] - sc[g]);   // exp2(-inf) = 0 on the first key
          l[g] *= alpha;
#pragma unroll
          for (int j = 0; j < DPL; ++j) o[g][j] *= alpha;
          m[g] = sc[g];
        }
        const float pg = exp2f(sc[g] - m[g]);
        l[g] += pg;
        const float pv = I8 ? pg * vscale : pg;
#pragma unroll
        for (int j = 0; j < DPL; ++j) o[g][j] += pv * xf[j];
      }
    }
  }
  cp_async_wait<0>();
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
  // merge the 4 warps of the CTA through shared memory (the pipeline stages are free now)
  __syncthreads();
  float* s_o = reinterpret_cast<float*>(s_raw);   // [4][G][HD]
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (sub == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
#pragma unroll
      for (int j = 0; j < DPL; ++j) s_o[(warp * G + g) * HD + sub * DPL + j] = o[g][j];
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
      oo += s_o[(w * G + g) * HD + c] * a;
    }
    const size_t idx = ((size_t)b * hq + head0 + g) * splits + sp;
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

static int launch_paged_decode(bool i8, const void* q, int ldq, const void* kc, const void* vc,
                               const float* ks, const float* vs, const int* block_tables,
                               int max_blocks, const int* seqlens, void* out, int ldo, float* part_o,
                               float* part_ml, int B, int hq, int hk, int hd, int bs, int splits,
                               float scale, void* stream) {
  if (B <= 0) return BB_OK;
  if (hq % hk || splits < 1) return BB_EARG;
  const int G = hq / hk;
  const int gsplit = G == 8 ? 2 : 1;
  dim3 grid(B, hk * gsplit, splits);
  const float sl2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
#define BB_LAUNCH_PD(HD_, G_)                                                                     \
  do {                                                                                            \
    if (i8)                                                                                       \
      paged_decode_kernel<HD_, G_, true><<<grid, 128, 0, s>>>(                                    \
          (const __nv_bfloat16*)q, ldq, kc, vc, ks, vs, block_tables, max_blocks, seqlens,        \
          part_o, part_ml, hq, hk, bs, splits, sl2, gsplit);                                      \
    else                                                                                          \
      paged_decode_kernel<HD_, G_, false><<<grid, 128, 0, s>>>(                                   \
          (const __nv_bfloat16*)q, ldq, kc, vc, nullptr, nullptr, block_tables, max_blocks,       \
          seqlens, part_o, part_ml, hq, hk, bs, splits, sl2, gsplit);                             \
  } while (0)
  if (hd == 128) {
    switch (G) {
      case 1: BB_LAUNCH_PD(128, 1); break;
      case 2: BB_LAUNCH_PD(128, 2); break;
      case 4: BB_LAUNCH_PD(128, 4); break;
      case 8: BB_LAUNCH_PD(128, 4); break;   // two CTAs of 4 heads per kv head
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

// part_o: fp32 [B*hq*splits*hd], part_ml: fp32 [B*hq*splits*2] scratch provided by the caller.
BB_API int bb_paged_decode(const void* q, int ldq, const void* kc, const void* vc,
                           const int* block_tables, int max_blocks, const int* seqlens, void* out,
                           int ldo, float* part_o, float* part_ml, int B, int hq, int hk, int hd,
                           int bs, int splits, float scale, void* stream) {
  return launch_paged_decode(false, q, ldq, kc, vc, nullptr, nullptr, block_tables, max_blocks,
                             seqlens, out, ldo, part_o, part_ml, B, hq, hk, hd, bs, splits, scale,
                             stream);
}

// int8 pools kc/vc with per-row scales ks/vs: fp32 [num_blocks, hk, bs].
BB_API int bb_paged_decode_i8(const void* q, int ldq, const void* kc, const void* vc,
                              const float* ks, const float* vs, const int* block_tables,
                              int max_blocks, const int* seqlens, void* out, int ldo,
                              float* part_o, float* part_ml, int B, int hq, int hk, int hd, int bs,
                              int splits, float scale, void* stream) {
  return launch_paged_decode(true, q, ldq, kc, vc, ks, vs, block_tables, max_blocks, seqlens, out,
                             ldo, part_o, part_ml, B, hq, hk, hd, bs, splits, scale, stream);
}

// clip: fp32 [2, hk] ceilings on the row absmax (K heads then V heads), or null.
BB_API int bb_kv_append_i8(const void* k, int ldk, const void* v, int ldv, const int* slots,
                           void* kc, void* vc, float* ks, float* vs, const float* clip, int n,
                           int hk, int hd, int bs, void* stream) {
  if (n <= 0) return BB_OK;
  if (hd > 128 || hd % 8) return BB_EARG;
  const long warps = (long)n * hk * 2;
  long blocks = (warps + 7) / 8;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  kv_append_i8_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, slots, (int8_t*)kc, (int8_t*)vc,
      ks, vs, clip, n, hk, hd, bs);
  return (int)cudaGetLastError();
}

BB_API int bb_kv_gather_i8(const void* kc, const void* vc, const float* ks, const float* vs,
                           const int* block_table, void* ok, void* ov, int S, int hk, int hd,
                           int bs, void* stream) {
  if (S <= 0) return BB_OK;
  if (hd % 8) return BB_EARG;
  const long total = (long)S * hk * (hd / 8);
  long blocks = (total + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  kv_gather_i8_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const int8_t*)kc, (const int8_t*)vc, ks, vs, block_table, (__nv_bfloat16*)ok,
      (__nv_bfloat16*)ov, S, hk, hd, bs);
  return (int)cudaGetLastError();
}
