// 3D Gaussian splat rasteriser as compute kernels, headless (renders into a device buffer):
//   project  -> per-Gaussian screen position, conic, opacity, depth, pixel radius, tile rectangle
//   scan     -> exclusive prefix sum of tiles touched (generic u32 scan, reused by the sort)
//   emit     -> (tile << 32 | depth bits, Gaussian index) pairs
//   sort     -> stable LSD radix sort of the pairs, 8 bits per pass
//   ranges   -> [start, end) of every tile in the sorted list
//   rasterise-> one CTA per 16x16 tile, front-to-back alpha compositing with early termination
//   backward -> back-to-front replay per tile: dL/d(colour, opacity, conic, screen xy), atomics
// Math contract: crates/splat/src/reference.rs (CPU oracle); the reference builds the same stages
// from atomic-free WGSL kernels (crates/splat/src/{renderer,sort}.rs).
#include "../common/host.hpp"

#include <cstdint>

namespace bb {

static constexpr int TILE = 16;

struct SplatCam {
  float v[12];
  float fx, fy, cx, cy;
  int w, h;
  float eps2d, znear, zfar;
  int antialiased;
};

// ------------------------------------------------------------------------------------ project
__global__ void splat_project_kernel(const float* __restrict__ means, const float* __restrict__ quats,
                                     const float* __restrict__ scales, const float* __restrict__ opac, int n,
                                     SplatCam c, float2* __restrict__ xy, float4* __restrict__ conic_op,
                                     float* __restrict__ depth, float2* __restrict__ rad,
                                     int4* __restrict__ rect, unsigned int* __restrict__ touched) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  touched[i] = 0u;
  const float* m = means + 3 * (size_t)i;
  const float x = c.v[0] * m[0] + c.v[1] * m[1] + c.v[2] * m[2] + c.v[3];
  const float y = c.v[4] * m[0] + c.v[5] * m[1] + c.v[6] * m[2] + c.v[7];
  const float z = c.v[8] * m[0] + c.v[9] * m[1] + c.v[10] * m[2] + c.v[11];
  if (z < c.znear || z > c.zfar) return;
  const float* q = quats + 4 * (size_t)i;
  const float qn = sqrtf(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]) + 1e-8f;
  const float qw = q[0] / qn, qx = q[1] / qn, qy = q[2] / qn, qz = q[3] / qn;
  const float R[3][3] = {
      {1.f - 2.f * (qy * qy + qz * qz), 2.f * (qx * qy - qw * qz), 2.f * (qx * qz + qw * qy)},
      {2.f * (qx * qy + qw * qz), 1.f - 2.f * (qx * qx + qz * qz), 2.f * (qy * qz - qw * qx)},
      {2.f * (qx * qz - qw * qy), 2.f * (qy * qz + qw * qx), 1.f - 2.f * (qx * qx + qy * qy)}};
  const float* sc = scales + 3 * (size_t)i;
  const float s2[3] = {sc[0] * sc[0], sc[1] * sc[1], sc[2] * sc[2]};
  float sig[3][3], a3[3][3], cc[3][3];
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < 3; ++b) sig[a][b] = s2[0] * R[a][0] * R[b][0] + s2[1] * R[a][1] * R[b][1] + s2[2] * R[a][2] * R[b][2];
  const float W[3][3] = {{c.v[0], c.v[1], c.v[2]}, {c.v[4], c.v[5], c.v[6]}, {c.v[8], c.v[9], c.v[10]}};
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < 3; ++b) a3[a][b] = W[a][0] * sig[0][b] + W[a][1] * sig[1][b] + W[a][2] * sig[2][b];
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < 3; ++b) cc[a][b] = a3[a][0] * W[b][0] + a3[a][1] * W[b][1] + a3[a][2] * W[b][2];
  const float rz = 1.f / z;
  const float w = (float)c.w, h = (float)c.h;
  const float tfx = 0.5f * w / c.fx, tfy = 0.5f * h / c.fy;
  const float lxp = (w - c.cx) / c.fx + 0.3f * tfx, lxn = c.cx / c.fx + 0.3f * tfx;
  const float lyp = (h - c.cy) / c.fy + 0.3f * tfy, lyn = c.cy / c.fy + 0.3f * tfy;
  const float txc = z * fminf(fmaxf(x * rz, -lxn), lxp);
  const float tyc = z * fminf(fmaxf(y * rz, -lyn), lyp);
  const float j00 = c.fx * rz, j02 = -c.fx * txc * rz * rz, j11 = c.fy * rz, j12 = -c.fy * tyc * rz * rz;
  float sa = j00 * j00 * cc[0][0] + 2.f * j00 * j02 * cc[0][2] + j02 * j02 * cc[2][2];
  const float sb = j00 * (cc[0][1] * j11 + cc[0][2] * j12) + j02 * (cc[2][1] * j11 + cc[2][2] * j12);
  float scv = j11 * j11 * cc[1][1] + 2.f * j11 * j12 * cc[1][2] + j12 * j12 * cc[2][2];
  const float det0 = sa * scv - sb * sb;
  sa += c.eps2d;
  scv += c.eps2d;
  const float det = sa * scv - sb * sb;
  if (det <= 0.f) return;
  float op = opac[i];
  if (c.antialiased) op *= sqrtf(fmaxf(det0 / det, 0.005f * 0.005f));
  if (op < 1.f / 255.f) return;
  const float extend = fminf(sqrtf(fmaxf(2.f * logf(op * 255.f), 0.f)), 3.33f);
  const float rx = ceilf(extend * sqrtf(sa)), ry = ceilf(extend * sqrtf(scv));
  if (rx <= 0.f || ry <= 0.f) return;
  const float px = c.fx * x * rz + c.cx, py = c.fy * y * rz + c.cy;
  if (px + rx <= 0.f || px - rx >= w || py + ry <= 0.f || py - ry >= h) return;
  xy[i] = make_float2(px, py);
  conic_op[i] = make_float4(scv / det, -sb / det, sa / det, op);
  depth[i] = z;
  rad[i] = make_float2(rx, ry);
  const int tx = (c.w + TILE - 1) / TILE, ty = (c.h + TILE - 1) / TILE;
  int4 r;
  r.x = min(tx, max(0, (int)floorf((px - rx) / TILE)));
  r.y = min(ty, max(0, (int)floorf((py - ry) / TILE)));
  r.z = min(tx, max(0, (int)floorf((px + rx) / TILE) + 1));
  r.w = min(ty, max(0, (int)floorf((py + ry) / TILE) + 1));
  rect[i] = r;   // conservative: the exact per-pixel radius test happens in the rasteriser
  touched[i] = (unsigned int)((r.z - r.x) * (r.w - r.y));
}

// ------------------------------------------------------------------------------------ scan (u32, exclusive)
// Level kernel: each block scans 1024 elements, writes the exclusive scan and its block total.
__global__ void scan_block_kernel(const unsigned int* __restrict__ in, unsigned int* __restrict__ out,
                                  unsigned int* __restrict__ block_sums, long n) {
  __shared__ unsigned int warp_tot[32];
  const long i = (long)blockIdx.x * 1024 + threadIdx.x;
  const unsigned int v = i < n ? in[i] : 0u;
  unsigned int incl = v;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    unsigned int w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  const unsigned int base = wid ? warp_tot[wid - 1] : 0u;
  if (i < n) out[i] = base + incl - v;
  if (threadIdx.x == 1023 && block_sums) block_sums[blockIdx.x] = base + incl;
}
__global__ void scan_add_kernel(unsigned int* __restrict__ out, const unsigned int* __restrict__ block_offs, long n) {
  const long i = (long)blockIdx.x * 1024 + threadIdx.x;
  if (i < n) out[i] += block_offs[blockIdx.x];
}

// scratch must hold at least n/1024 + n/1024^2 + 3 elements
static int scan_u32(const unsigned int* in, unsigned int* out, long n, unsigned int* scratch, cudaStream_t s) {
  if (n <= 0) return 0;
  const long blocks = (n + 1023) / 1024;
  if (blocks == 1) {
    scan_block_kernel<<<1, 1024, 0, s>>>(in, out, nullptr, n);
    return (int)cudaGetLastError();
  }
  unsigned int* sums = scratch;
  scan_block_kernel<<<(int)blocks, 1024, 0, s>>>(in, out, sums, n);
  int rc = scan_u32(sums, sums, blocks, scratch + blocks, s);   // in place is fine: one read per element
  if (rc) return rc;
  scan_add_kernel<<<(int)blocks, 1024, 0, s>>>(out, sums, n);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------ emit
__global__ void splat_emit_kernel(const int4* __restrict__ rect, const float* __restrict__ depth,
                                  const unsigned int* __restrict__ touched, const unsigned int* __restrict__ offs,
                                  int n, int tiles_x, unsigned long long* __restrict__ keys,
                                  unsigned int* __restrict__ vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n || touched[i] == 0u) return;
  const int4 r = rect[i];
  const unsigned int d = __float_as_uint(depth[i]);   // depth > 0: the bit pattern orders like the value
  unsigned int o = offs[i];
  for (int ty = r.y; ty < r.w; ++ty)
    for (int tx = r.x; tx < r.z; ++tx) {
      keys[o] = ((unsigned long long)(ty * tiles_x + tx) << 32) | d;
      vals[o] = (unsigned int)i;
      ++o;
    }
}

// ------------------------------------------------------------------------------------ radix sort (LSD, 8 bits, stable)
static constexpr int SORT_BLOCK = 256;
static constexpr int SORT_ITEMS = 8;                  // keys per thread
static constexpr int SORT_CHUNK = SORT_BLOCK * SORT_ITEMS;

__global__ void radix_hist_kernel(const unsigned long long* __restrict__ keys, long n, int shift,
                                  unsigned int* __restrict__ hist, int nblocks) {
  __shared__ unsigned int h[256];
  h[threadIdx.x] = 0u;
  __syncthreads();
  const long base = (long)blockIdx.x * SORT_CHUNK;
  for (int k = 0; k < SORT_ITEMS; ++k) {
    const long i = base + k * SORT_BLOCK + threadIdx.x;
    if (i < n) atomicAdd(&h[(keys[i] >> shift) & 255u], 1u);
  }
  __syncthreads();
  hist[(size_t)threadIdx.x * nblocks + blockIdx.x] = h[threadIdx.x];   // digit-major: one scan gives global offsets
}

// Stable scatter: the block walks its chunk in rounds of 256 keys (one per thread, in order); inside a
// round a key's rank among equal digits is its warp-local rank (match_any) plus the counts of the
// earlier warps, and the per-digit running offset advances after each round.
__global__ void radix_scatter_kernel(const unsigned long long* __restrict__ keys_in,
                                     const unsigned int* __restrict__ vals_in, long n, int shift,
                                     const unsigned int* __restrict__ offs, int nblocks,
                                     unsigned long long* __restrict__ keys_out, unsigned int* __restrict__ vals_out) {
  __shared__ unsigned int run[256];               // next output slot of each digit for this block
  __shared__ unsigned int wcount[8][256];         // per-warp digit counts of the current round
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  run[threadIdx.x] = offs[(size_t)threadIdx.x * nblocks + blockIdx.x];
  const long base = (long)blockIdx.x * SORT_CHUNK;
  for (int k = 0; k < SORT_ITEMS; ++k) {
    for (int j = threadIdx.x; j < 8 * 256; j += SORT_BLOCK) (&wcount[0][0])[j] = 0u;
    __syncthreads();
    const long i = base + k * SORT_BLOCK + threadIdx.x;
    const bool live = i < n;
    unsigned long long key = 0ull;
    unsigned int digit = 0u, rank = 0u;
    if (live) {
      key = keys_in[i];
      digit = (unsigned int)(key >> shift) & 255u;
    }
    const unsigned int active = __ballot_sync(0xffffffffu, live);
    if (live) {
      const unsigned int peers = __match_any_sync(active, digit);
      rank = __popc(peers & ((1u << lane) - 1u));
      if (rank == 0) wcount[wid][digit] = __popc(peers);
    }
    __syncthreads();
    if (live) {
      unsigned int before = 0u;
      for (int w = 0; w < wid; ++w) before += wcount[w][digit];
      const unsigned int dst = run[digit] + before + rank;
      keys_out[dst] = key;
      vals_out[dst] = vals_in[i];
    }
    __syncthreads();
    {
      unsigned int tot = 0u;
#pragma unroll
      for (int w = 0; w < 8; ++w) tot += wcount[w][threadIdx.x];
      run[threadIdx.x] += tot;
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------ tile ranges
__global__ void splat_ranges_kernel(const unsigned long long* __restrict__ keys, long n, int2* __restrict__ ranges) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned int t = (unsigned int)(keys[i] >> 32);
  if (i == 0 || (unsigned int)(keys[i - 1] >> 32) != t) ranges[t].x = (int)i;
  if (i == n - 1 || (unsigned int)(keys[i + 1] >> 32) != t) ranges[t].y = (int)(i + 1);
}

// ------------------------------------------------------------------------------------ rasterise
__global__ void __launch_bounds__(TILE * TILE)
splat_raster_kernel(const int2* __restrict__ ranges, const unsigned int* __restrict__ order,
                    const float2* __restrict__ xy, const float4* __restrict__ conic_op,
                    const float* __restrict__ depth, const float2* __restrict__ rad, const float* __restrict__ colors,
                    int w, int h, int tiles_x, float bg0, float bg1, float bg2, int depth_mode,
                    float* __restrict__ img, float* __restrict__ final_t, int* __restrict__ n_contrib) {
  __shared__ float2 s_xy[256];
  __shared__ float4 s_co[256];
  __shared__ float4 s_cd[256];   // colour rgb + depth
  __shared__ float2 s_rad[256];  // pixel radius (rx, ry) of the bounding rectangle
  const int tile = blockIdx.y * tiles_x + blockIdx.x;
  const int px = blockIdx.x * TILE + threadIdx.x, py = blockIdx.y * TILE + threadIdx.y;
  const int tid = threadIdx.y * TILE + threadIdx.x;
  const bool inside = px < w && py < h;
  const float fx = px + 0.5f, fy = py + 0.5f;
  const int2 rg = ranges[tile];
  float T = 1.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, dep = 0.f;
  bool done = !inside;
  int contrib = 0, last = 0;
  for (int b0 = rg.x; b0 < rg.y; b0 += 256) {
    if (__syncthreads_and(done)) break;
    const int j = b0 + tid;
    if (j < rg.y) {
      const unsigned int g = order[j];
      s_xy[tid] = xy[g];
      s_co[tid] = conic_op[g];
      s_cd[tid] = make_float4(colors[3 * (size_t)g], colors[3 * (size_t)g + 1], colors[3 * (size_t)g + 2], depth[g]);
      s_rad[tid] = rad[g];
    }
    __syncthreads();
    const int cnt = min(256, rg.y - b0);
    for (int k = 0; k < cnt && !done; ++k) {
      ++contrib;
      const float2 p = s_xy[k];
      const float4 co = s_co[k];
      const float dx = p.x - fx, dy = p.y - fy;
      const float2 rr = s_rad[k];
      if (fabsf(dx) > rr.x || fabsf(dy) > rr.y) continue;
      const float sigma = 0.5f * (co.x * dx * dx + co.z * dy * dy) + co.y * dx * dy;
      if (sigma < 0.f) continue;
      const float alpha = fminf(co.w * __expf(-sigma), 0.99f);
      if (alpha < 1.f / 255.f) continue;
      const float nt = T * (1.f - alpha);
      if (nt <= 1e-4f) {
        done = true;
        break;
      }
      const float wgt = alpha * T;
      const float4 cd = s_cd[k];
      c0 += cd.x * wgt;
      c1 += cd.y * wgt;
      c2 += cd.z * wgt;
      dep += cd.w * wgt;
      T = nt;
      last = contrib;
    }
    __syncthreads();
  }
  if (inside) {
    float* q = img + ((size_t)py * w + px) * 4;
    const float a = 1.f - T;
    if (!depth_mode) {
      q[0] = c0 + T * bg0;
      q[1] = c1 + T * bg1;
      q[2] = c2 + T * bg2;
    } else {
      const float d = a > 1e-6f ? dep / a : 0.f;
      q[0] = q[1] = q[2] = d;
    }
    q[3] = a;
    if (final_t) final_t[(size_t)py * w + px] = T;
    if (n_contrib) n_contrib[(size_t)py * w + px] = last;
  }
}

// Backward of the colour mode: replays each pixel's contributors back to front.
//   C = sum_k c_k a_k T_k + T_final bg,  A = 1 - T_final
// given dL/dC (3) and dL/dA per pixel, accumulates dL/d colour, opacity, conic (3), screen xy.
__global__ void __launch_bounds__(TILE * TILE)
splat_raster_bwd_kernel(const int2* __restrict__ ranges, const unsigned int* __restrict__ order,
                        const float2* __restrict__ xy, const float4* __restrict__ conic_op,
                        const float2* __restrict__ rad, const float* __restrict__ colors, int w, int h, int tiles_x,
                        float bg0, float bg1, float bg2,
                        const float* __restrict__ final_t, const int* __restrict__ n_contrib,
                        const float* __restrict__ dimg, float* __restrict__ d_colors, float* __restrict__ d_opac,
                        float* __restrict__ d_conic, float* __restrict__ d_xy) {
  __shared__ float2 s_xy[256];
  __shared__ float4 s_co[256];
  __shared__ float4 s_c[256];
  __shared__ float2 s_rad[256];
  __shared__ unsigned int s_id[256];
  const int tile = blockIdx.y * tiles_x + blockIdx.x;
  const int px = blockIdx.x * TILE + threadIdx.x, py = blockIdx.y * TILE + threadIdx.y;
  const int tid = threadIdx.y * TILE + threadIdx.x;
  const bool inside = px < w && py < h;
  const float fx = px + 0.5f, fy = py + 0.5f;
  const int2 rg = ranges[tile];
  const int total = rg.y - rg.x;
  const float Tf = inside ? final_t[(size_t)py * w + px] : 0.f;
  const int last = inside ? n_contrib[(size_t)py * w + px] : 0;
  float g0 = 0.f, g1 = 0.f, g2 = 0.f, ga = 0.f;
  if (inside) {
    const float* d = dimg + ((size_t)py * w + px) * 4;
    g0 = d[0];
    g1 = d[1];
    g2 = d[2];
    ga = d[3];
  }
  // dL/dT_final: colour through the background term, alpha = 1 - T_final
  const float dT_final = g0 * bg0 + g1 * bg1 + g2 * bg2 - ga;
  float T = Tf;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;   // colour accumulated BEHIND the current Gaussian
  const int rounds = (total + 255) / 256;
  for (int r = rounds - 1; r >= 0; --r) {
    const int b0 = rg.x + r * 256;
    const int j = b0 + tid;
    __syncthreads();
    if (j < rg.y) {
      const unsigned int g = order[j];
      s_id[tid] = g;
      s_xy[tid] = xy[g];
      s_co[tid] = conic_op[g];
      s_c[tid] = make_float4(colors[3 * (size_t)g], colors[3 * (size_t)g + 1], colors[3 * (size_t)g + 2], 0.f);
      s_rad[tid] = rad[g];
    }
    __syncthreads();
    const int cnt = min(256, rg.y - b0);
    for (int k = cnt - 1; k >= 0; --k) {
      const int ordinal = r * 256 + k + 1;     // 1-based position in the tile's list
      if (!inside || ordinal > last) continue;
      const float2 p = s_xy[k];
      const float4 co = s_co[k];
      const float dx = p.x - fx, dy = p.y - fy;
      const float2 rr = s_rad[k];
      if (fabsf(dx) > rr.x || fabsf(dy) > rr.y) continue;
      const float sigma = 0.5f * (co.x * dx * dx + co.z * dy * dy) + co.y * dx * dy;
      if (sigma < 0.f) continue;
      const float G = __expf(-sigma);
      const float araw = co.w * G;
      const float alpha = fminf(araw, 0.99f);
      if (alpha < 1.f / 255.f) continue;
      T = T / (1.f - alpha);                   // transmittance in front of this Gaussian
      const float4 c = s_c[k];
      const float wgt = alpha * T;
      const unsigned int g = s_id[k];
      atomicAdd(d_colors + 3 * (size_t)g, g0 * wgt);
      atomicAdd(d_colors + 3 * (size_t)g + 1, g1 * wgt);
      atomicAdd(d_colors + 3 * (size_t)g + 2, g2 * wgt);
      // dL/dalpha = T (c - behind/(1-alpha)) . g  - T_final/(1-alpha) * dT_final-term
      float dalpha = ((c.x * T - acc0 / (1.f - alpha)) * g0 + (c.y * T - acc1 / (1.f - alpha)) * g1 +
                      (c.z * T - acc2 / (1.f - alpha)) * g2);
      dalpha += -Tf / (1.f - alpha) * dT_final;
      acc0 += c.x * wgt;
      acc1 += c.y * wgt;
      acc2 += c.z * wgt;
      if (araw >= 0.99f) continue;             // clamped: no gradient through alpha
      const float dG = co.w * dalpha;
      atomicAdd(d_opac + g, G * dalpha);
      const float dsig = -G * dG;
      atomicAdd(d_conic + 3 * (size_t)g, 0.5f * dx * dx * dsig);
      atomicAdd(d_conic + 3 * (size_t)g + 1, dx * dy * dsig);
      atomicAdd(d_conic + 3 * (size_t)g + 2, 0.5f * dy * dy * dsig);
      atomicAdd(d_xy + 2 * (size_t)g, (co.x * dx + co.y * dy) * dsig);
      atomicAdd(d_xy + 2 * (size_t)g + 1, (co.z * dy + co.y * dx) * dsig);
    }
  }
}

}  // namespace bb

using namespace bb;

static SplatCam make_cam(const float* cam16, int w, int h, const float* opts6, int flags) {
  SplatCam c;
  for (int i = 0; i < 12; ++i) c.v[i] = cam16[i];
  c.fx = cam16[12];
  c.fy = cam16[13];
  c.cx = cam16[14];
  c.cy = cam16[15];
  c.w = w;
  c.h = h;
  c.eps2d = opts6[3];
  c.znear = opts6[4];
  c.zfar = opts6[5];
  c.antialiased = (flags >> 1) & 1;
  return c;
}

// Stage 1: project + count + scan.  cam16/opts6 are HOST arrays.  offs[n] (exclusive scan of touched);
// the caller reads offs[n-1] + touched[n-1] for the pair count.
BB_API int bb_splat_project(const float* means, const float* quats, const float* scales, const float* opac, int n,
                            const float* cam16, int w, int h, const float* opts6, int flags, void* xy,
                            void* conic_op, float* depth, void* rad, void* rect, unsigned int* touched, unsigned int* offs,
                            unsigned int* scratch, void* stream) {
  if (n <= 0) return BB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const SplatCam c = make_cam(cam16, w, h, opts6, flags);
  splat_project_kernel<<<(n + 255) / 256, 256, 0, s>>>(means, quats, scales, opac, n, c, (float2*)xy,
                                                      (float4*)conic_op, depth, (float2*)rad, (int4*)rect, touched);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return scan_u32(touched, offs, n, scratch, s);
}

// Generic exclusive scan of u32 (scratch: n/1024 + n/1024^2 + 3 elements).
BB_API int bb_scan_u32(const unsigned int* in, unsigned int* out, long n, unsigned int* scratch, void* stream) {
  return scan_u32(in, out, n, scratch, static_cast<cudaStream_t>(stream));
}

// Stable LSD radix sort of (u64 key, u32 value) pairs on bits [0, key_bits).  keys/vals are sorted in
// place using the *_tmp buffers; hist: 256 * ceil(n/2048) u32; scratch as for the scan of that size.
BB_API int bb_radix_sort_pairs(unsigned long long* keys, unsigned int* vals, unsigned long long* keys_tmp,
                               unsigned int* vals_tmp, long n, int key_bits, unsigned int* hist,
                               unsigned int* scratch, void* stream) {
  if (n <= 0) return BB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nblocks = (int)((n + SORT_CHUNK - 1) / SORT_CHUNK);
  int passes = (key_bits + 7) / 8;
  if (passes & 1) ++passes;   // an even number of passes leaves the result in keys/vals
  unsigned long long *ki = keys, *ko = keys_tmp;
  unsigned int *vi = vals, *vo = vals_tmp;
  for (int p = 0; p < passes; ++p) {
    radix_hist_kernel<<<nblocks, SORT_BLOCK, 0, s>>>(ki, n, p * 8, hist, nblocks);
    int rc = scan_u32(hist, hist, 256L * nblocks, scratch, s);
    if (rc) return rc;
    radix_scatter_kernel<<<nblocks, SORT_BLOCK, 0, s>>>(ki, vi, n, p * 8, hist, nblocks, ko, vo);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    unsigned long long* tk = ki;
    ki = ko;
    ko = tk;
    unsigned int* tv = vi;
    vi = vo;
    vo = tv;
  }
  return BB_OK;
}

// Stage 2: emit the (tile, depth) pairs.
BB_API int bb_splat_emit(const void* rect, const float* depth, const unsigned int* touched,
                         const unsigned int* offs, int n, int tiles_x, unsigned long long* keys,
                         unsigned int* vals, void* stream) {
  if (n <= 0) return BB_OK;
  splat_emit_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const int4*)rect, depth, touched, offs, n, tiles_x, keys, vals);
  return (int)cudaGetLastError();
}

// Stage 3: tile ranges (ranges must be zeroed: tiles without pairs keep [0, 0)) and rasterisation.
BB_API int bb_splat_raster(const unsigned long long* keys, const unsigned int* order, long n_pairs, void* ranges,
                           const void* xy, const void* conic_op, const float* depth, const void* rad,
                           const float* colors, int w, int h, const float* opts6, int flags, float* img,
                           float* final_t, int* n_contrib, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tx = (w + TILE - 1) / TILE, ty = (h + TILE - 1) / TILE;
  if (n_pairs > 0) {
    splat_ranges_kernel<<<(int)((n_pairs + 255) / 256), 256, 0, s>>>(keys, n_pairs, (int2*)ranges);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  splat_raster_kernel<<<dim3(tx, ty), dim3(TILE, TILE), 0, s>>>(
      (const int2*)ranges, order, (const float2*)xy, (const float4*)conic_op, depth, (const float2*)rad, colors, w, h,
      tx, opts6[0], opts6[1], opts6[2], flags & 1, img, final_t, n_contrib);
  return (int)cudaGetLastError();
}

BB_API int bb_splat_raster_bwd(const void* ranges, const unsigned int* order, const void* xy, const void* conic_op,
                               const void* rad, const float* colors, int w, int h, const float* opts6, const float* final_t,
                               const int* n_contrib, const float* dimg, float* d_colors, float* d_opac,
                               float* d_conic, float* d_xy, void* stream) {
  const int tx = (w + TILE - 1) / TILE, ty = (h + TILE - 1) / TILE;
  splat_raster_bwd_kernel<<<dim3(tx, ty), dim3(TILE, TILE), 0, static_cast<cudaStream_t>(stream)>>>(
      (const int2*)ranges, order, (const float2*)xy, (const float4*)conic_op, (const float2*)rad, colors, w, h, tx,
      opts6[0], opts6[1], opts6[2], final_t, n_contrib, dimg, d_colors, d_opac, d_conic, d_xy);
  return (int)cudaGetLastError();
}
