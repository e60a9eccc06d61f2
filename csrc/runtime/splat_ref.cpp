// CPU oracle of the 3D Gaussian splat rasteriser: projection of anisotropic Gaussians through a
// pinhole camera (EWA), depth sort, front-to-back alpha compositing per pixel.  This is the
// reference the CUDA kernels in csrc/kernels/splat.cu are checked against and the timed CPU
// baseline of the renderer.  It restates the math of the reference's CPU oracle
// (crates/splat/src/reference.rs: project_one / render) as plain C++ with std::thread rows.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

struct Proj {
  float x, y, conic[3], opacity, depth, rx, ry;
  int idx;
};

struct Cam {
  float v[12];  // world -> camera, row-major 3x4
  float fx, fy, cx, cy;
  int w, h;
};

struct Opts {
  float bg[3];
  int depth_mode, antialiased;
  float eps2d, znear, zfar;
};

bool project_one(const float* mean, const float* quat, const float* scale, float opacity, const Cam& c,
                 const Opts& o, Proj* out) {
  const float* v = c.v;
  const float x = v[0] * mean[0] + v[1] * mean[1] + v[2] * mean[2] + v[3];
  const float y = v[4] * mean[0] + v[5] * mean[1] + v[6] * mean[2] + v[7];
  const float z = v[8] * mean[0] + v[9] * mean[1] + v[10] * mean[2] + v[11];
  if (z < o.znear || z > o.zfar) return false;
  const float qn = std::sqrt(quat[0] * quat[0] + quat[1] * quat[1] + quat[2] * quat[2] + quat[3] * quat[3]) + 1e-8f;
  const float qw = quat[0] / qn, qx = quat[1] / qn, qy = quat[2] / qn, qz = quat[3] / qn;
  const float R[3][3] = {
      {1.f - 2.f * (qy * qy + qz * qz), 2.f * (qx * qy - qw * qz), 2.f * (qx * qz + qw * qy)},
      {2.f * (qx * qy + qw * qz), 1.f - 2.f * (qx * qx + qz * qz), 2.f * (qy * qz - qw * qx)},
      {2.f * (qx * qz - qw * qy), 2.f * (qy * qz + qw * qx), 1.f - 2.f * (qx * qx + qy * qy)}};
  const float s2[3] = {scale[0] * scale[0], scale[1] * scale[1], scale[2] * scale[2]};
  float sig[3][3], a3[3][3], cc[3][3];
  for (int a = 0; a < 3; ++a)
    for (int b = 0; b < 3; ++b) {
      float s = 0.f;
      for (int k = 0; k < 3; ++k) s += s2[k] * R[a][k] * R[b][k];
      sig[a][b] = s;
    }
  const float W[3][3] = {{v[0], v[1], v[2]}, {v[4], v[5], v[6]}, {v[8], v[9], v[10]}};
  for (int i = 0; i < 3; ++i)
    for (int j = 0; j < 3; ++j) {
      float s = 0.f;
      for (int k = 0; k < 3; ++k) s += W[i][k] * sig[k][j];
      a3[i][j] = s;
    }
  for (int i = 0; i < 3; ++i)
    for (int j = 0; j < 3; ++j) {
      float s = 0.f;
      for (int k = 0; k < 3; ++k) s += a3[i][k] * W[j][k];
      cc[i][j] = s;
    }
  const float rz = 1.f / z;
  const float w = (float)c.w, h = (float)c.h;
  const float tfx = 0.5f * w / c.fx, tfy = 0.5f * h / c.fy;
  const float lxp = (w - c.cx) / c.fx + 0.3f * tfx, lxn = c.cx / c.fx + 0.3f * tfx;
  const float lyp = (h - c.cy) / c.fy + 0.3f * tfy, lyn = c.cy / c.fy + 0.3f * tfy;
  const float txc = z * std::min(std::max(x * rz, -lxn), lxp);
  const float tyc = z * std::min(std::max(y * rz, -lyn), lyp);
  const float j00 = c.fx * rz, j02 = -c.fx * txc * rz * rz, j11 = c.fy * rz, j12 = -c.fy * tyc * rz * rz;
  float sa = j00 * j00 * cc[0][0] + 2.f * j00 * j02 * cc[0][2] + j02 * j02 * cc[2][2];
  const float sb = j00 * (cc[0][1] * j11 + cc[0][2] * j12) + j02 * (cc[2][1] * j11 + cc[2][2] * j12);
  float sc = j11 * j11 * cc[1][1] + 2.f * j11 * j12 * cc[1][2] + j12 * j12 * cc[2][2];
  const float det0 = sa * sc - sb * sb;
  sa += o.eps2d;
  sc += o.eps2d;
  const float det = sa * sc - sb * sb;
  if (det <= 0.f) return false;
  float op = opacity;
  if (o.antialiased) op *= std::sqrt(std::max(det0 / det, 0.005f * 0.005f));
  if (op < 1.f / 255.f) return false;
  const float extend = std::min(std::sqrt(std::max(2.f * std::log(op * 255.f), 0.f)), 3.33f);
  const float rx = std::ceil(extend * std::sqrt(sa)), ry = std::ceil(extend * std::sqrt(sc));
  if (rx <= 0.f || ry <= 0.f) return false;
  const float px = c.fx * x * rz + c.cx, py = c.fy * y * rz + c.cy;
  if (px + rx <= 0.f || px - rx >= w || py + ry <= 0.f || py - ry >= h) return false;
  out->x = px;
  out->y = py;
  out->conic[0] = sc / det;
  out->conic[1] = -sb / det;
  out->conic[2] = sa / det;
  out->opacity = op;
  out->depth = z;
  out->rx = rx;
  out->ry = ry;
  return true;
}

}  // namespace

// cam: 12 view-matrix floats, fx, fy, cx, cy (16 floats); dims: width, height; opts: bg[3], eps2d,
// near, far (6 floats); flags: bit 0 depth mode, bit 1 antialiased.  img: [h][w][4] fp32.
BBH_API int bbh_splat_render(const float* means, const float* quats, const float* scales, const float* opac,
                             const float* colors, int64_t n, const float* cam, int width, int height,
                             const float* opts, int flags, float* img, int threads) {
  Cam c;
  std::memcpy(c.v, cam, 12 * sizeof(float));
  c.fx = cam[12];
  c.fy = cam[13];
  c.cx = cam[14];
  c.cy = cam[15];
  c.w = width;
  c.h = height;
  Opts o;
  o.bg[0] = opts[0];
  o.bg[1] = opts[1];
  o.bg[2] = opts[2];
  o.eps2d = opts[3];
  o.znear = opts[4];
  o.zfar = opts[5];
  o.depth_mode = flags & 1;
  o.antialiased = (flags >> 1) & 1;
  std::vector<Proj> pr;
  pr.reserve((size_t)n);
  for (int64_t i = 0; i < n; ++i) {
    Proj p;
    if (project_one(means + 3 * i, quats + 4 * i, scales + 3 * i, opac[i], c, o, &p)) {
      p.idx = (int)i;
      pr.push_back(p);
    }
  }
  std::stable_sort(pr.begin(), pr.end(), [](const Proj& a, const Proj& b) { return a.depth < b.depth; });
  if (threads < 1) threads = 1;
  auto rows = [&](int y0, int y1) {
    for (int py = y0; py < y1; ++py)
      for (int px = 0; px < width; ++px) {
        const float fx = px + 0.5f, fy = py + 0.5f;
        float t = 1.f, col[3] = {0.f, 0.f, 0.f}, dep = 0.f;
        for (const Proj& p : pr) {
          const float dx = p.x - fx, dy = p.y - fy;
          if (std::fabs(dx) > p.rx || std::fabs(dy) > p.ry) continue;
          const float sigma = 0.5f * (p.conic[0] * dx * dx + p.conic[2] * dy * dy) + p.conic[1] * dx * dy;
          if (sigma < 0.f) continue;
          const float alpha = std::min(p.opacity * std::exp(-sigma), 0.99f);
          if (alpha < 1.f / 255.f) continue;
          const float nt = t * (1.f - alpha);
          if (nt <= 1e-4f) break;
          const float wgt = alpha * t;
          for (int k = 0; k < 3; ++k) col[k] += colors[3 * (size_t)p.idx + k] * wgt;
          dep += p.depth * wgt;
          t = nt;
        }
        const float a = 1.f - t;
        float* q = img + ((size_t)py * width + px) * 4;
        if (!o.depth_mode) {
          for (int k = 0; k < 3; ++k) q[k] = col[k] + t * o.bg[k];
        } else {
          const float d = a > 1e-6f ? dep / a : 0.f;
          q[0] = q[1] = q[2] = d;
        }
        q[3] = a;
      }
  };
  std::vector<std::thread> pool;
  const int chunk = (height + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const int y0 = t * chunk, y1 = std::min(height, y0 + chunk);
    if (y0 >= y1) break;
    pool.emplace_back(rows, y0, y1);
  }
  for (auto& th : pool) th.join();
  return (int)pr.size();
}
